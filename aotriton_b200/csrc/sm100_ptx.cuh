// Thin inline-PTX layer for the Blackwell (sm_100a) execution model: mbarriers with
// bounded waits, TMA tile loads (each CTA fetches its own tiles), tensor memory (TMEM) management,
// tcgen05 MMA issue/commit, TMEM loads/stores, and the shared-memory / instruction
// descriptors those need.  Nothing here allocates or synchronises on its own.
#pragma once
#include <cstdio>

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "common.cuh"
#include "launch.h"

namespace ab200 {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier ---------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One try: returns true when the phase with this parity has completed.  The instruction may
// park the thread for a system-dependent time while the phase is still pending and wakes it when
// the phase completes (measured: 87 cycles from the arrive to the waiter's next instruction).  The
// form without a suspend-time hint is used: with a hint the compiler emits a polling loop with a
// sleep of its own, which costs more instructions per wait.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Every wait in the kernels is bounded: after kWaitLimitCycles SM cycles (about a second)
// without success the waiter records where it gave up (in *status, a global word the host can
// read), raises the CTA-wide abort flag and returns false.  All roles test the abort flag while
// they poll, so a stuck pipeline drains within about one limit and the CTA exits normally; CTAs
// that start after a failure was recorded return at once (the kernels test *status first).
constexpr long long kWaitLimitCycles = 2000000000ll;
constexpr int kSpinsPerCheck = 64;

// The CTA's abort word is followed by the wait limit of this launch in units of 1024 cycles
// (0 = kWaitLimitCycles); the thread that initialises the barriers writes both.
__device__ __forceinline__ void init_abort_and_limit(volatile uint32_t* abort_flag, uint32_t limit_kcycles) {
  abort_flag[0] = 0u;
  abort_flag[1] = limit_kcycles;
}
__device__ __forceinline__ long long wait_limit_cycles(volatile uint32_t* abort_flag) {
  const uint32_t k = abort_flag[1];
  return k != 0u ? (long long)k * 1024ll : kWaitLimitCycles;
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          unsigned int* status, uint32_t where) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    // The polling loop proper is two instructions; the abort flag and the clock are looked at once
    // in kSpinsPerCheck polls.  (Waiting warps share their scheduler's issue slots with the warps
    // that do the work: with the checks in every iteration, polling made up a third of all
    // instructions the kernels executed.)
#pragma unroll 1
    for (int spin = 0; spin < kSpinsPerCheck; ++spin)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) {
#ifdef AB200_DEBUG_WAITS
      if ((threadIdx.x & 31) == 0) printf("blk %d,%d,%d warp %d saw abort at %x\n", blockIdx.x, blockIdx.y, blockIdx.z, threadIdx.x >> 5, where);
#endif
      return false;
    }
    // (the launch's limit is read here, once in kSpinsPerCheck polls, not ahead of the loop: every
    // blocking wait of the pipeline passes through this function and must start polling at once)
    if (clock64() - t0 > wait_limit_cycles(abort_flag)) break;
  }
#ifdef AB200_DEBUG_WAITS
  if ((threadIdx.x & 31) == 0) printf("blk %d,%d,%d warp %d TIMEOUT at %x\n", blockIdx.x, blockIdx.y, blockIdx.z, threadIdx.x >> 5, where);
#endif
  *abort_flag = 1u;
  if (status) atomicCAS(status, 0u, where);
  return false;
}

// The same for roles that run well ahead of their consumers (a stager, a scheduler): between polls
// the thread sleeps, so that it does not take issue slots from the warps on the critical path.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                  unsigned int* status, uint32_t where) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int spin = 0; spin < kSpinsPerCheck; ++spin) {
      if (mbar_try_wait(bar, parity)) return true;
      __nanosleep(200);
    }
    if (*abort_flag) return false;
    if (clock64() - t0 > wait_limit_cycles(abort_flag)) break;
  }
  *abort_flag = 1u;
  if (status) atomicCAS(status, 0u, where);
  return false;
}

// Bounded wait without side effects, for draining copies on the failure path.
__device__ __forceinline__ void mbar_wait_quiet(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
  const long long t0 = clock64();
  const long long limit = wait_limit_cycles(abort_flag);
  while (!mbar_try_wait(bar, parity))
    if (clock64() - t0 > limit) return;
}

// Packed pairs of fp32 operations (one instruction for two lanes of work on sm_100).
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 sub2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "sub.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

// 16-byte load from shared memory by its shared-space address (a load through a generic pointer
// costs the address-space check and extra address arithmetic in the inner loops).
__device__ __forceinline__ float4 lds128(uint32_t saddr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(saddr));
  return v;
}

// max of three (one instruction on sm_100).
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// 2^x on the special-function unit (flushes denormals; -inf -> 0).
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x for a pair of finite arguments on the FMA pipe (no special-function unit): x = n + f with
// n = round(x), f in [-0.5, 0.5]; 2^f by a degree-3 polynomial (relative error 7.5e-5, far below
// the 16-bit rounding the result goes through), 2^n by adding n to the exponent field.  Arguments
// below -126 give about 1e-38 instead of 0, so this is only used where every argument belongs to an
// unmasked score (a masked score needs an exact 0).
__device__ __forceinline__ float2 exp2_fma_pair(float2 x) {
  const float2 magic = make_float2(12582912.f, 12582912.f);     // 1.5 * 2^23: the sum holds round(x) in its low bits
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 t = add2(x, magic);
  const float2 f = sub2(x, sub2(t, magic));
  float2 p = fma2(f, make_float2(5.517166712e-02f, 5.517166712e-02f), make_float2(2.426111220e-01f, 2.426111220e-01f));
  p = fma2(p, f, make_float2(6.932609858e-01f, 6.932609858e-01f));
  p = fma2(p, f, make_float2(9.999280736e-01f, 9.999280736e-01f));
  float2 r;
  r.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
  return r;
}

// ---- proxies / fences -------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Warp-collective: zero rows [valid_rows, 128) of a [128 rows x 64*halves columns] 16-bit tile in
// the TMA tile layout (row r of 64-column half hf at hf*16384 + r*128; the 128-byte swizzle only
// permutes 16-byte chunks inside a row), then make the writes visible to the tensor core.  Used on
// the last, partial block of a sequence: the bulk copy is bounded by the tensor, not by the
// sequence, so the rows beyond the sequence's end hold a neighbour's tokens or padding, and a zero
// probability times a non-finite value there would poison the product (the reference zero-fills
// such rows with masked loads, modules/flash/kernel/masked_load_store.py:214-307).
// (Not inlined on purpose: it runs at most once per sequence end, and its loops inside the MMA
// issuer's loop cost that warp registers and instruction-cache room on every block.)
static __device__ __noinline__ void zero_tail_rows(uint8_t* tile, int valid_rows, int halves, int lane) {
  const uint4 z = make_uint4(0u, 0u, 0u, 0u);
  for (int hf = 0; hf < halves; ++hf)
    for (int o = valid_rows * 128 + lane * 16; o < 16384; o += 512)
      *reinterpret_cast<uint4*>(tile + hf * 16384 + o) = z;
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- TMA (tile mode, this CTA only) ------------------------------------------------
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 4-D tile load: coordinates innermost first.  c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
      "r"(c3)
      : "memory");
}

// The same tile towards L2 only (no shared-memory destination, no barrier): a later tma_load_4d of it
// then finds it there.
__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap* m, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

// ---- TMEM -------------------------------------------------------------------------
// Warp-collective.  ncols: power of two in [32, 512].  The base address lands in *smem_slot.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---- tcgen05.mma ------------------------------------------------------------------
// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by ONE thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]; A holds 16-bit elements packed two per 32-bit column.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` once every tcgen05 operation this thread issued so far has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Shared-memory matrix descriptor (sm_100 format): 128-byte swizzle, 8-row groups 1024 bytes
// apart (SBO); `lbo_bytes` is the distance between 64-element atoms along the M/N dimension
// for MN-major operands and ignored for K-major ones.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);           // start address, bits [0,14)
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;      // leading byte offset, bits [16,30)
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;      // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                                  // descriptor version 1 (Blackwell)
  d |= (uint64_t)2 << 61;                                  // layout type 2 = SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16 with fp32 accumulation.
// ab_format: 0 = fp16, 1 = bf16.  *_mn_major: 1 when the operand is stored M/N-contiguous.
__host__ __device__ constexpr uint32_t instr_desc_f16(uint32_t ab_format, uint32_t m, uint32_t n,
                                                      uint32_t a_mn_major, uint32_t b_mn_major) {
  return (1u << 4)                 // accumulator format f32
         | (ab_format << 7)        // A format
         | (ab_format << 10)       // B format
         | (a_mn_major << 15) | (b_mn_major << 16)
         | ((n >> 3) << 17)        // N / 8
         | ((m >> 4) << 24);       // M / 16
}

// ---- TMEM <-> registers (32 lanes x 32-bit, N consecutive columns per thread) -------
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32f(uint32_t taddr, float* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]),
        "=f"(r[8]), "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]),
        "=f"(r[16]), "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]),
        "=f"(r[24]), "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld8f(uint32_t taddr, float* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16f(uint32_t taddr, float* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]),
        "=f"(r[8]), "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),
      "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Move registers between warpgroups (all four warps of a warpgroup must execute the same one).
template <uint32_t N>
__device__ __forceinline__ void reg_alloc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <uint32_t N>
__device__ __forceinline__ void reg_dealloc() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

}  // namespace ptx

// ---- element-type helpers shared by the tcgen05 kernels ------------------------------
template <typename T> struct Fmt;
template <> struct Fmt<__half> { static constexpr uint32_t code = 0; };
template <> struct Fmt<__nv_bfloat16> { static constexpr uint32_t code = 1; };

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

inline bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

// A view the TMA tile maps can describe: 16-byte aligned base and outer strides, unit inner stride.
inline bool tma_friendly(const View4& v) {
  if (v.ptr == nullptr || !aligned16(v.ptr)) return false;
  for (int i = 0; i < 3; ++i)
    if (v.n[i] > 1 && (v.s[i] % 8 != 0 || v.s[i] <= 0)) return false;
  for (int i = 0; i < 4; ++i)
    if (v.n[i] <= 0 || v.n[i] > 0x7fffffffLL) return false;
  return v.s[3] == 1;
}

// Rows written with 16-byte vector stores.
inline bool vector_store_friendly(const View4& v) {
  return v.ptr != nullptr && aligned16(v.ptr) && v.s[0] % 8 == 0 && v.s[1] % 8 == 0 && v.s[2] % 8 == 0 && v.s[3] == 1;
}

// ---- host side: TMA descriptor encoding goes through the host-call table (launch.h), which looks
// the driver's encoder up at run time, so that the library does not link libcuda.
// ---- write-out of a [128 rows x D] 16-bit tile through shared memory -----------------------
// A thread that owns one row of a tile (a TMEM lane) would store 16 bytes per instruction at a
// row stride: 32 separate memory lines per warp instruction, which costs thousands of cycles per
// tile.  Instead each warp transposes its 32 rows through a staging tile and writes row segments.
// Staging layout: row r starts at r * row_bytes; 16-byte chunk c of the row sits at position
// (c & ~7) | ((c ^ r) & 7), which makes both the row-per-thread writes and the chunk-per-thread
// reads free of bank conflicts.
__device__ __forceinline__ uint32_t stage_chunk_offset(int r, int c, int row_bytes) {
  return (uint32_t)(r * row_bytes + (((c & ~7) | ((c ^ r) & 7)) << 4));
}
// 32 consecutive values (columns d0..d0+31, d0 a multiple of 32) of row r
template <typename T>
__device__ __forceinline__ void stage_put32(uint8_t* stage, int r, int d0, const float* v, float scale, int row_bytes) {
#pragma unroll
  for (int v8 = 0; v8 < 4; ++v8) {
    uint4 w;
    w.x = pack2<T>(v[v8 * 8 + 0] * scale, v[v8 * 8 + 1] * scale);
    w.y = pack2<T>(v[v8 * 8 + 2] * scale, v[v8 * 8 + 3] * scale);
    w.z = pack2<T>(v[v8 * 8 + 4] * scale, v[v8 * 8 + 5] * scale);
    w.w = pack2<T>(v[v8 * 8 + 6] * scale, v[v8 * 8 + 7] * scale);
    *reinterpret_cast<uint4*>(stage + stage_chunk_offset(r, (d0 >> 3) + v8, row_bytes)) = w;
  }
}
// Write-out by the warp that staged them: rows row0..row0+31 of the staging tile, 16-byte chunks
// c0..c0+nchunks-1 of each row (nchunks = 4: eight rows of 64 bytes per instruction; nchunks =
// 16: two full rows per instruction).  Only a __syncwarp() separates staging from write-out.
// `tile` points at row 0 of the tile in global memory (rows `row_stride` elements apart, 16-byte
// aligned); rows below `nrows` and columns below `dmax` (a multiple of 8) are written.
template <typename T, int NCHUNKS>
__device__ __forceinline__ void warp_copy_out(const uint8_t* stage, T* tile, int64_t row_stride, int nrows, int dmax,
                                              int row0, int c0, int lane, int row_bytes) {
  constexpr int kRowsPerInstr = 32 / NCHUNKS;
  const int c = c0 + (lane & (NCHUNKS - 1));
  const int rl = lane / NCHUNKS;
  if (c * 8 >= dmax) return;
#pragma unroll
  for (int k = 0; k < 32 / kRowsPerInstr; ++k) {
    const int r = row0 + k * kRowsPerInstr + rl;
    if (r < nrows)
      *reinterpret_cast<uint4*>(tile + (int64_t)r * row_stride + c * 8) =
          *reinterpret_cast<const uint4*>(stage + stage_chunk_offset(r, c, row_bytes));
  }
}

// Tile map over a (B, H, S, D) view of 16-bit elements: box = 64 columns x `box_rows` rows,
// 128-byte swizzle, zero fill outside the extents.  Dimensions are given innermost first.
inline bool make_tile_map_16bit(CUtensorMap* out, const View4& v, int64_t d_extent, int64_t s_extent, int box_rows) {
  cuuint64_t dims[4] = {(cuuint64_t)d_extent, (cuuint64_t)s_extent, (cuuint64_t)v.n[1], (cuuint64_t)v.n[0]};
  cuuint64_t strides[3] = {(cuuint64_t)v.s[2] * 2, (cuuint64_t)v.s[1] * 2, (cuuint64_t)v.s[0] * 2};
  // A unit extent may carry any stride; give it a legal one.
  for (int i = 0; i < 3; ++i)
    if (dims[i + 1] == 1 && (strides[i] == 0 || strides[i] % 16 != 0)) strides[i] = 16;
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const int r = host().encode_tiled(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, v.ptr, dims, strides, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == 0;
}

}  // namespace ab200
