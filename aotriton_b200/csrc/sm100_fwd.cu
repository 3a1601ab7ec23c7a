// Forward attention on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
// One CTA owns TWO tiles of 128 query rows (256 consecutive rows) of one (sequence, q-head) and
// walks the key/value blocks (128 keys each) their window can reach; each K/V block is loaded
// once and used by both tiles.  Twelve warps:
//
//   warp 0       TMA producer   both Q tiles once, then K and V blocks through two 2-stage rings
//                               (cp.async.bulk.tensor, 128-byte swizzle, this CTA only)
//   warp 1       MMA issuer     walks its loop warp-uniformly; one elected lane issues, per
//                               tile,  S = Q K^T  (operands in shared memory) and  O += P V  (P read straight from tensor
//                               memory, V from shared memory, N-major); completion is signalled
//                               with tcgen05.commit.  P arrives in two halves of 64 keys, so
//                               the first half of P V runs under the second half's exponentials
//   warps 4-7    softmax, tile 0        thread r owns query row r of its tile: tcgen05.ld of the S
//   warps 8-11   softmax, tile 1        row, scale, bias, mask, running max / sum in the exp2
//                               domain, dropout, P written back over S as packed 16-bit, lazy
//                               rescale of O, final normalisation, O (transposed per warp
//                               through the idle Q buffer, whole rows per store) and LSE stores
//
// While one tile's softmax warps work on block j, the tensor core runs the other tile's PV and
// QK^T: the two tiles ping-pong.  The producer and issuer warps give most of their registers
// to the softmax warps (setmaxnreg).
//
// Tensor memory (512 columns): S0 [0,128)  S1 [128,256)  O0 [256,256+HD)  O1 [384,384+HD).
// P of a tile aliases the first 64 columns of its S.
//
// Arithmetic contract (ROCm/aotriton modules/flash/kernel/fwd_kernel_inner.py:126-277,
// fwd_kernel.py:573-620): logits scaled by sm_scale*log2(e), bias*log2(e) added, masked
// scores -inf, row sum taken BEFORE dropout, P cast to the value dtype before P V,
// O = acc / l / (1-p), LSE = (m + log2 l) * ln2, rows that see no key give O = 0, LSE = +inf.
// The running maximum is only advanced when it grows by more than 8 (a factor 256 in P);
// the result is the same function of the inputs, with fewer passes over O.
//
// Every wait is bounded (sm100_ptx.cuh); on a time-out the CTA drains and exits, and the
// word behind `status` records which wait gave up.
#include <atomic>
#include "launch.h"
#include "sm100_ptx.cuh"

namespace ab200 {

__device__ unsigned int g_sm100_fwd_status = 0;

// Optional pipeline trace (compile with -DAB200_TRACE): SM cycle stamps of one softmax thread
// of the first CTA, eight per key block, read back with ab200_debug_read_fwd_trace().
#ifndef AB200_TRACE_TID
#define AB200_TRACE_TID 128
#endif
#ifdef AB200_TRACE
__device__ long long g_fwd_trace[8 * 256];
#define AB200_FSTAMP(iter, slot)                                                                                     \
  do {                                                                                                               \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == AB200_TRACE_TID && (iter) < 256)     \
      g_fwd_trace[(iter) * 8 + (slot)] = clock64();                                                                  \
  } while (0)
#else
#define AB200_FSTAMP(iter, slot) do {} while (0)
#endif

namespace {

using namespace ptx;

constexpr int kBM = 128, kBN = 128;
constexpr int kFwdThreads = 384;
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;

// Head dims up to 128: two query tiles per CTA and two-stage K and V rings.  Head dims up to 256:
// a tile is 64 KB, so one query tile per CTA (S in 128 and O in 256 tensor-memory columns) and one
// stage each for K and V; the K copy of block j+1 then runs under the softmax and P V of block j,
// the V copy under Q K^T and the softmax of block j+1.
template <int HD>
struct FwdSmem {
  static constexpr int kTiles = HD > 128 ? 1 : 2;
  static constexpr int kStages = HD > 128 ? 1 : 2;
  static constexpr int kCtaRows = kTiles * kBM;
  static constexpr int kHalves = HD / 64;
  static constexpr int kTileBytes = kHalves * 128 * 128;     // 128 rows x HD x 2 bytes
  static constexpr int kQ = 0;                               // kTiles tiles
  static constexpr int kK = kQ + kTiles * kTileBytes;
  static constexpr int kV = kK + kStages * kTileBytes;
  static constexpr int kBars = kV + kStages * kTileBytes;
  // barrier slots (8 bytes each)
  static constexpr int bQFull = 0 /*2*/, bKFull = 2, bKEmpty = 4, bVFull = 6, bVEmpty = 8, bSFull = 10 /*2*/,
                       bPFull = 12 /*2*/, bPvDone = 14 /*2*/, bPHalf = 16 /*2*/, bCount = 18;
  static constexpr int kTmemSlot = kBars + bCount * 8;
  static constexpr int kAbort = kTmemSlot + 4;               // abort word, then the launch's wait limit
  static constexpr int kTotal = kAbort + 8;
  static constexpr int kDynamic = kTotal + 1024;             // slack for manual 1024-byte alignment
};

// Rows [m0, m0+rows) of the output that have no key at all: O = 0, LSE = +inf.
template <typename T>
__device__ void write_dead_rows(const Params& p, const Seq& sq, int h, int m0, int rows) {
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    int m = m0 + r;
    if (m >= sq.sq) continue;
    T* op = reinterpret_cast<T*>(p.out.ptr) + (int64_t)sq.bidx * p.out.s[0] + (int64_t)h * p.out.s[1] +
            (sq.q0 + m) * p.out.s[2];
    for (int d = 0; d < p.dvo; ++d) op[d] = from_f32<T>(0.f);
    if (p.lse) p.lse[lse_offset(p, sq, h) + m] = INFINITY;
  }
}

// EXACT: a dense problem whose sequence lengths are multiples of 128 and whose head dimensions equal
// HD.  Every tile is then full, so the instantiation carries no tail handling and fixed GEMM shapes:
// the MMA issuer's loop is latency-critical, and even untaken branches and a call site in it cost
// several per cent of the kernel's time (measured: 3 to 10 % over the three tcgen05 kernels).
template <typename T, int HD, bool EXACT>
__global__ void __launch_bounds__(kFwdThreads, 1)
sm100_fwd_kernel(const __grid_constant__ Params p, const __grid_constant__ CUtensorMap tm_q,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                 unsigned int* status) {
  using L = FwdSmem<HD>;
  constexpr int kStages = L::kStages, kCtaRows = L::kCtaRows;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlot);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::kAbort);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Order of the CTAs (the hardware starts them by linear block index): (batch, head) pairs are taken
  // in groups of kHeadGroup; inside a group the row-tile index runs slowest, from the tile with the
  // most key blocks of a causal problem to the one with the fewest.  The heavy tiles of a group so
  // start together and the grid ends on light ones, while the CTAs in flight share the K/V of one
  // group of heads, which stays resident in L2.
#ifndef AB200_FWD_HEAD_GROUP
#define AB200_FWD_HEAD_GROUP 32
#endif
  int z = blockIdx.z, h = blockIdx.y, m0 = (int)(gridDim.x - 1 - blockIdx.x) * kCtaRows;
  if constexpr (AB200_FWD_HEAD_GROUP > 0) {
    constexpr int kHeadGroup = AB200_FWD_HEAD_GROUP > 0 ? AB200_FWD_HEAD_GROUP : 1;
    const int nx = (int)gridDim.x, nh = (int)gridDim.y, nhz = nh * (int)gridDim.z;
    const int lin = (int)blockIdx.x + nx * ((int)blockIdx.y + nh * (int)blockIdx.z);
    const int grp = lin / (kHeadGroup * nx), r = lin - grp * (kHeadGroup * nx);
    const int gsize = min(kHeadGroup, nhz - grp * kHeadGroup);
    const int xi = r / gsize, hz = grp * kHeadGroup + (r - xi * gsize);
    z = hz / nh;
    h = hz - z * nh;
    m0 = (nx - 1 - xi) * kCtaRows;
  }
  // An earlier CTA timed out: the whole CTA leaves (one read, one CTA-wide decision).
  if (__syncthreads_or(threadIdx.x == 0 && *reinterpret_cast<volatile unsigned int*>(status) != 0u)) return;
  // One thread of the grid reports the seed and offset actually used, before any early exit.
  if (p.dropout_on && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) {
    uint64_t seed = p.seed_ptr ? *p.seed_ptr : 0ull;
    uint64_t base = p.off2 + (p.off1_ptr ? *p.off1_ptr : 0ull);
    if (p.seed_out) *p.seed_out = seed;
    if (p.off_out) *p.off_out = base;
  }
  const Seq sq = resolve_seq(p, z);
  if (m0 >= sq.sq) return;
  const int hk = h / p.group;
  const int ntile = (L::kTiles == 2 && m0 + kBM < sq.sq) ? 2 : 1;   // the second tile may lie beyond the sequence

  // Block range: the union over the CTA's rows; a tile simply sees fully masked blocks outside its own.
  int n_lo, n_hi;
  key_range(p, sq, m0, min(m0 + kCtaRows, sq.sq) - 1, n_lo, n_hi);
  if (n_hi < n_lo) {            // CTA-uniform: nothing to attend to
    write_dead_rows<T>(p, sq, h, m0, kCtaRows);
    return;
  }
  const int jb_lo = n_lo / kBN;
  const int nblk = n_hi / kBN - jb_lo + 1;

  // ---- set-up -----------------------------------------------------------------------
  if (threadIdx.x == 0) {
    init_abort_and_limit(abort_flag, p.wait_limit_kcycles);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars[L::bQFull + s], 1);
      mbar_init(&bars[L::bKFull + s], 1);
      mbar_init(&bars[L::bKEmpty + s], 1);
      mbar_init(&bars[L::bVFull + s], 1);
      mbar_init(&bars[L::bVEmpty + s], 1);
      mbar_init(&bars[L::bSFull + s], 1);
      mbar_init(&bars[L::bPFull + s], 4);      // one arrival per softmax warp of the tile
      mbar_init(&bars[L::bPvDone + s], 1);
      mbar_init(&bars[L::bPHalf + s], 4);      // first 64 keys of P written
    }
    fence_barrier_init();
    // This thread is also the TMA producer: both Q tiles and the first blocks of K and V (the ring
    // stages are all free) are requested right away, before the CTA-wide synchronisation and the
    // tensor-memory allocation, which then overlap with the copies' latency.
    for (int t = 0; t < ntile; ++t) {
      const int qrow = (int)(sq.q0 + m0 + t * kBM);
      mbar_expect_tx(&bars[L::bQFull + t], L::kTileBytes);
      for (int hf = 0; hf < L::kHalves; ++hf)
        tma_load_4d(smem + L::kQ + t * L::kTileBytes + hf * 16384, &tm_q, &bars[L::bQFull + t], hf * 64, qrow, h, sq.bidx);
    }
    for (int j = 0; j < min(kStages, nblk); ++j) {
      const int krow = (int)(sq.k0 + (int64_t)(jb_lo + j) * kBN);
      mbar_expect_tx(&bars[L::bKFull + j], L::kTileBytes);
      for (int hf = 0; hf < L::kHalves; ++hf)
        tma_load_4d(smem + L::kK + j * L::kTileBytes + hf * 16384, &tm_k, &bars[L::bKFull + j], hf * 64, krow, hk, sq.bidx);
      if (p.drop_copy == 1 && j == 0) continue;   // test hook: this block's V never arrives
      mbar_expect_tx(&bars[L::bVFull + j], L::kTileBytes);
      for (int hf = 0; hf < L::kHalves; ++hf)
        tma_load_4d(smem + L::kV + j * L::kTileBytes + hf * 16384, &tm_v, &bars[L::bVFull + j], hf * 64, krow, hk, sq.bidx);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4) {
    reg_dealloc<56>();
    if (warp == 0) {
      // =============================== TMA producer ===================================
      if (lane == 0) {
        // (the Q tiles and the first kStages blocks were requested during set-up)
        int issued = 2 * min(kStages, nblk);
        for (int j = min(kStages, nblk); j < nblk; ++j) {
          const int s = j % kStages;
          const uint32_t ph = (uint32_t)(j / kStages) & 1u;
          const int krow = (int)(sq.k0 + (int64_t)(jb_lo + j) * kBN);
          if (!mbar_wait(&bars[L::bKEmpty + s], ph ^ 1u, abort_flag, status, 0x100 + j)) break;
          mbar_expect_tx(&bars[L::bKFull + s], L::kTileBytes);
          for (int hf = 0; hf < L::kHalves; ++hf)
            tma_load_4d(smem + L::kK + s * L::kTileBytes + hf * 16384, &tm_k, &bars[L::bKFull + s], hf * 64, krow, hk,
                        sq.bidx);
          if (!mbar_wait(&bars[L::bVEmpty + s], ph ^ 1u, abort_flag, status, 0x200 + j)) { issued = j * 2 + 1; break; }
          mbar_expect_tx(&bars[L::bVFull + s], L::kTileBytes);
          for (int hf = 0; hf < L::kHalves; ++hf)
            tma_load_4d(smem + L::kV + s * L::kTileBytes + hf * 16384, &tm_v, &bars[L::bVFull + s], hf * 64, krow, hk,
                        sq.bidx);
          issued = j * 2 + 2;
        }
        if (*abort_flag) {
          // Let copies that are still in flight land before the CTA gives its shared memory back.
          for (int t = 0; t < ntile; ++t) mbar_wait_quiet(&bars[L::bQFull + t], 0, abort_flag);
          for (int i = max(0, issued - 2 * kStages); i < issued; ++i) {
            int j = i >> 1, s = j % kStages;
            uint32_t ph = (uint32_t)(j / kStages) & 1u;
            if (p.drop_copy == 1 && i == 1) continue;   // (never issued)
            mbar_wait_quiet((i & 1) ? &bars[L::bVFull + s] : &bars[L::bKFull + s], ph, abort_flag);
          }
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // ================================ MMA issuer ====================================
      // The whole warp walks the loop and waits; one elected lane issues.  With warp-uniform
      // control flow the descriptors stay in uniform registers and a GEMM costs few issue slots.
      // The contraction of Q K^T runs over the head dimension rounded up to 16 and P V produces the
      // value head dimension rounded up to 16 (the copies zero-fill up to the 64-column box), so a
      // padded head dimension costs its own size, not the kernel's.
      constexpr uint32_t kIdescQK = instr_desc_f16(Fmt<T>::code, 128, 128, 0, 0);
      // (EXACT: both equal the kernel's head dimension, known at compile time)
      const uint32_t kIdescPV = instr_desc_f16(Fmt<T>::code, 128, EXACT ? (uint32_t)HD : (uint32_t)((p.dvo + 15) & ~15), 0, 1);
      const int ksteps = EXACT ? HD / 16 : (p.dqk + 15) >> 4;
      // Descriptors are built once; a k-step, a tile or a ring stage only moves the 14-bit
      // start-address field (units of 16 bytes), which cannot carry out of the field.
      const uint64_t q_desc = smem_desc_sw128(smem_u32(smem + L::kQ), 16, 1024);
      const uint64_t k_desc = smem_desc_sw128(smem_u32(smem + L::kK), 16, 1024);
      const uint64_t v_desc = smem_desc_sw128(smem_u32(smem + L::kV), 16384, 1024);
      constexpr uint32_t kStageStep = L::kTileBytes >> 4;
      auto wait = [&](int bar, uint32_t parity, uint32_t where) {
        return __all_sync(0xffffffffu, mbar_wait(&bars[bar], parity, abort_flag, status, where)) != 0;
      };
      // S_t = Q_t K_j^T; `release_k`: this is the last reader of the K stage
      auto issue_qk = [&](int t, int j, bool release_k) {
        const uint64_t qd = q_desc + (uint64_t)((uint32_t)t * kStageStep);
        const uint64_t kd = k_desc + (uint64_t)((uint32_t)(j % kStages) * kStageStep);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            constexpr uint32_t kHalfStep = 16384u >> 4, kInner = 32u >> 4;
            const uint32_t off = (uint32_t)(kk >> 2) * kHalfStep + (uint32_t)(kk & 3) * kInner;
            if (kk < ksteps) mma_ss(tmem_base + (uint32_t)t * 128u, qd + off, kd + off, kIdescQK, kk > 0 ? 1u : 0u);
          }
          mma_commit(&bars[L::bSFull + t]);
          if (release_k) mma_commit(&bars[L::bKEmpty + (j % kStages)]);
        }
        __syncwarp();
      };
      // index of the sequence's last key block if it is a partial one (the only block whose V tile
      // holds rows beyond the sequence), else -1
      const int tail_j = (sq.sk % kBN != 0) ? (sq.sk - 1) / kBN - jb_lo : -1;
      bool ok = true;
      for (int t = 0; ok && t < ntile; ++t) ok = wait(L::bQFull + t, 0, 0x300 + t);
      if (ok) ok = wait(L::bKFull + 0, 0, 0x400);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < ntile; ++t) issue_qk(t, 0, t == ntile - 1);
      }
      for (int j = 0; ok && j < nblk; ++j) {
        const int s = j % kStages;
        const uint32_t par = (uint32_t)j & 1u;
        if (!wait(L::bVFull + s, (uint32_t)(j / kStages) & 1u, 0x600 + j)) break;
        // Last, partial block of the sequence: the rows of V beyond its end must not reach P V.
        if constexpr (!EXACT) {
          if (j == tail_j)
            zero_tail_rows(smem + L::kV + s * L::kTileBytes, sq.sk - (jb_lo + j) * kBN, L::kHalves, lane);
        }
        if (j + 1 < nblk) {
          if (!wait(L::bKFull + ((j + 1) % kStages), (uint32_t)((j + 1) / kStages) & 1u, 0x400 + j + 1)) break;
        }
        const uint64_t vd = v_desc + (uint64_t)((uint32_t)s * kStageStep);
        const uint32_t first = (j > 0) ? 1u : 0u;
        for (int t = 0; ok && t < ntile; ++t) {
          // P arrives in two halves of 64 keys: the first half of P V runs while the softmax warps
          // are still working on the second.
          const uint32_t pcol = tmem_base + (uint32_t)t * 128u;
          const uint32_t ocol = tmem_base + 256u + (uint32_t)t * 128u;
          if (!wait(L::bPHalf + t, par, 0x580 + 2 * j + t)) { ok = false; break; }
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < kBN / 32; ++kk) {
              // 16 keys per step: 8 packed columns of P, 2048 bytes of V (two 8-key groups)
              mma_ts(ocol, pcol + (uint32_t)kk * 8u, vd + (uint32_t)kk * (2048u >> 4), kIdescPV, kk > 0 ? 1u : first);
            }
          }
          __syncwarp();
          if (!wait(L::bPFull + t, par, 0x500 + 2 * j + t)) { ok = false; break; }
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int kk = kBN / 32; kk < kBN / 16; ++kk)
              mma_ts(ocol, pcol + (uint32_t)kk * 8u, vd + (uint32_t)kk * (2048u >> 4), kIdescPV, 1u);
            mma_commit(&bars[L::bPvDone + t]);
            if (t == ntile - 1) mma_commit(&bars[L::bVEmpty + s]);
          }
          __syncwarp();
          // the tile's S buffer is free again: PV_t(j), just issued, runs first
          if (j + 1 < nblk) issue_qk(t, j + 1, t == ntile - 1);
        }
      }
    }
  } else {
    // ================================== softmax =====================================
    reg_alloc<216>();
    const int t = (warp - 4) >> 2;              // tile of this warpgroup
    if (t < ntile) {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int m = m0 + t * kBM + r;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_addr + (uint32_t)t * 128u;
    const uint32_t o_addr = tmem_base + lane_addr + 256u + (uint32_t)t * 128u;
    int row_lo = 0, row_hi = sq.sk - 1;
    if (p.causal) {
      int64_t lo = (int64_t)m - sq.wl, hi = (int64_t)m + sq.wr;
      if (lo > row_lo) row_lo = (int)(lo > 0x7fffffffLL ? 0x7fffffffLL : lo);
      if (hi < row_hi) row_hi = (int)(hi < -1 ? -1 : hi);
    }
    if (m >= sq.sq) { row_lo = 1; row_hi = 0; }
    // the tightest bounds over the warp's rows: a block needs masking iff it is not inside them
    const int warp_lo = __reduce_max_sync(0xffffffffu, row_lo), warp_hi = __reduce_min_sync(0xffffffffu, row_hi);
    DropoutCtx dctx;
    if (p.dropout_on) dctx = dropout_ctx(p, z, h);
    // (the ten round keys of Philox depend on the seed only: kept in registers, they save every counter
    // two additions per round, 13 to 18 % of a dropout forward)
    PhiloxKeys pkeys;
    if (p.dropout_on) pkeys = philox_keys(dctx.seed);
    const T* bias_row = nullptr;
    if (p.has_bias)
      bias_row = reinterpret_cast<const T*>(p.bias.ptr) + (int64_t)sq.bidx * p.bias.s[0] + (int64_t)h * p.bias.s[1] +
                 (int64_t)min(m, sq.sq - 1) * p.bias.s[2];

    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk; ++j) {
      const int n0 = (jb_lo + j) * kBN;
      const uint32_t par = (uint32_t)j & 1u;
      if (p.has_bias && p.bias_vec) {
        // the thread's 256 bytes of bias for this block: on their way to L2 while the tensor pipe computes S
        const char* bp = reinterpret_cast<const char*>(bias_row + n0);
        asm volatile("prefetch.global.L2 [%0];" ::"l"(bp));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(bp + 128));
      }
      if (!mbar_wait(&bars[L::bSFull + t], par, abort_flag, status, 0x700 + 2 * j + t)) { ok = false; break; }
      AB200_FSTAMP(j, 0);
      tc_fence_after();
      float sc[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32f(s_addr + c * 32, &sc[c * 32]);
      tmem_wait_ld();
      AB200_FSTAMP(j, 1);
      // Scores -> exponent arguments.  The common case (no bias, positive scale, ordinary
      // magnitudes) keeps the raw scores and folds scale and maximum into one FMA per element
      // later.  Otherwise the scaled scores are formed first, so that equal raw scores give
      // exactly equal arguments however large they are.
      // (warp-uniform without a vote per block: compared with the warp's extreme bounds)
      const bool any_mask = !(n0 >= warp_lo && n0 + kBN - 1 <= warp_hi);
      bool simple = !p.has_bias && p.qk_scale > 0.f;
      float mx;
      if (simple) {
        if (any_mask) {
#pragma unroll
          for (int c = 0; c < 128; ++c) {
            const int n = n0 + c;
            sc[c] = (n >= row_lo && n <= row_hi) ? sc[c] : -INFINITY;
          }
        }
        float m8[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) m8[c] = fmaxf(sc[2 * c], sc[2 * c + 1]);
#pragma unroll
        for (int c = 16; c < 128; c += 2) m8[(c >> 1) & 7] = fmax3(m8[(c >> 1) & 7], sc[c], sc[c + 1]);
        mx = fmaxf(fmax3(m8[0], m8[1], m8[2]), fmaxf(fmax3(m8[3], m8[4], m8[5]), fmaxf(m8[6], m8[7])));
        mx *= p.qk_scale;
        const bool huge = fabsf(mx) > 1.0e6f && mx != -INFINITY;
        if (__any_sync(0xffffffffu, huge)) simple = false;
      }
      if (!simple) {
#pragma unroll
        for (int c = 0; c < 128; ++c) sc[c] *= p.qk_scale;
        if (p.has_bias) {
          const int nmax = sq.sk - n0;
          if (p.bias_vec && nmax >= kBN) {
            // the thread's 128 bias values are 256 contiguous bytes: sixteen 16-byte loads, four in flight
            const uint4* bp = reinterpret_cast<const uint4*>(bias_row + n0);
#pragma unroll
            for (int g = 0; g < 16; g += 4) {
              uint4 w[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) w[u] = __ldg(bp + g + u);
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const T* e = reinterpret_cast<const T*>(&w[u]);
#pragma unroll
                for (int i = 0; i < 8; ++i) sc[(g + u) * 8 + i] = fmaf(to_f32<T>(e[i]), kLog2e, sc[(g + u) * 8 + i]);
              }
            }
          } else {
#pragma unroll
            for (int c = 0; c < 128; ++c)
              if (c < nmax) sc[c] = fmaf(to_f32<T>(bias_row[(int64_t)(n0 + c) * p.bias.s[3]]), kLog2e, sc[c]);
          }
        }
        if (any_mask) {
#pragma unroll
          for (int c = 0; c < 128; ++c) {
            const int n = n0 + c;
            sc[c] = (n >= row_lo && n <= row_hi) ? sc[c] : -INFINITY;
          }
        }
        float m8[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) m8[c] = fmaxf(sc[2 * c], sc[2 * c + 1]);
#pragma unroll
        for (int c = 16; c < 128; c += 2) m8[(c >> 1) & 7] = fmax3(m8[(c >> 1) & 7], sc[c], sc[c + 1]);
        mx = fmaxf(fmax3(m8[0], m8[1], m8[2]), fmaxf(fmax3(m8[3], m8[4], m8[5]), fmaxf(m8[6], m8[7])));
      }
      AB200_FSTAMP(j, 2);
      // Advance the reference maximum only when it moved by more than the threshold.
      const bool grow = mx > m_used + kRescaleThreshold;     // false when mx == -inf
      float alpha = 1.f;
      if (grow) {
        alpha = ex2(m_used - mx);                            // m_used == -inf -> 0
        m_used = mx;
      }
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // O must be complete up to block j-1 before it is rescaled.
        // (S of block j was issued behind P V of block j-1, so this wait returns at once.)
        if (!mbar_wait(&bars[L::bPvDone + t], (uint32_t)(j - 1) & 1u, abort_flag, status, 0x800 + 2 * j + t)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          if (c * 32 >= p.dvo) break;          // columns the P V product never writes
          uint32_t o[32];
          tmem_ld32(o_addr + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(o_addr + c * 32, o);
        }
        tmem_wait_st();
      }
      AB200_FSTAMP(j, 3);
      l *= alpha;
      const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
      float2 s4[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) s4[c] = make_float2(0.f, 0.f);
      // Exponentials, dropout and the packed P in two halves of 64 keys; the first half is handed
      // to the MMA issuer while the second is being computed.
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int cb = half * 64;
        if (simple) {
          const float2 sc2 = make_float2(p.qk_scale, p.qk_scale), nm2 = make_float2(-m_safe, -m_safe);
#ifndef AB200_FWD_POLY
#define AB200_FWD_POLY 0
#endif
#if AB200_FWD_POLY > 0
          if (!any_mask) {
            // Every score of this block is unmasked for every row of the warp: one pair in
            // AB200_FWD_POLY takes its exponentials on the FMA pipe, which otherwise idles while the
            // special-function unit (16 results per clock and SM) paces the loop.
#pragma unroll
            for (int c = cb; c < cb + 64; c += 2) {
              const float2 a = fma2(make_float2(sc[c], sc[c + 1]), sc2, nm2);
              if (((c >> 1) % AB200_FWD_POLY) == AB200_FWD_POLY - 1) {
                const float2 e = exp2_fma_pair(a);
                sc[c] = e.x;
                sc[c + 1] = e.y;
              } else {
                sc[c] = ex2(a.x);
                sc[c + 1] = ex2(a.y);
              }
              s4[(c >> 1) & 3] = add2(s4[(c >> 1) & 3], make_float2(sc[c], sc[c + 1]));
            }
          } else
#endif
#pragma unroll
          for (int c = cb; c < cb + 64; c += 2) {
            const float2 a = fma2(make_float2(sc[c], sc[c + 1]), sc2, nm2);
            sc[c] = ex2(a.x);
            sc[c + 1] = ex2(a.y);
            s4[(c >> 1) & 3] = add2(s4[(c >> 1) & 3], make_float2(sc[c], sc[c + 1]));
          }
        } else {
          const float2 nm2 = make_float2(-m_safe, -m_safe);
#pragma unroll
          for (int c = cb; c < cb + 64; c += 2) {
            const float2 a = add2(make_float2(sc[c], sc[c + 1]), nm2);
            sc[c] = ex2(a.x);
            sc[c + 1] = ex2(a.y);
            s4[(c >> 1) & 3] = add2(s4[(c >> 1) & 3], make_float2(sc[c], sc[c + 1]));
          }
        }
        // (the row sum uses the values before dropout: it was accumulated above)
        if (p.dropout_on) {
          const int mm = min(m, p.max_sq - 1);
#pragma unroll
          for (int c4 = half * 16; c4 < half * 16 + 16; ++c4) dropout_zero4_keys(dctx, pkeys, mm, (n0 >> 2) + c4, &sc[c4 * 4]);
        }
        // P over the first 64 columns of this S buffer, two 16-bit values per column.
        {
          uint32_t pk[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) pk[i] = pack2<T>(sc[half * 64 + 2 * i], sc[half * 64 + 2 * i + 1]);
          tmem_st32(s_addr + half * 32, pk);
        }
        if (half == 0) {
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars[L::bPHalf + t]);
          AB200_FSTAMP(j, 4);
        }
      }
      const float sum = ((s4[0].x + s4[0].y) + (s4[1].x + s4[1].y)) + ((s4[2].x + s4[2].y) + (s4[3].x + s4[3].y));
      l += sum;
      AB200_FSTAMP(j, 5);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[L::bPFull + t]);
      AB200_FSTAMP(j, 6);
    }
    // ---- epilogue ---------------------------------------------------------------------
    // P V of every block but the last is complete (S of the last block was issued behind it),
    // so only the last phase of this barrier can still be pending.
    if (ok) ok = mbar_wait(&bars[L::bPvDone + t], (uint32_t)(nblk - 1) & 1u, abort_flag, status, 0x900 + t);
    if (ok) {
      tc_fence_after();
      const float inv = (l > 0.f) ? p.dropout_scale / l : 0.f;
      // Each warp transposes its 32 rows through the tile's (now idle) Q buffer, so that the global
      // stores are whole rows instead of 16 bytes per row.
      uint8_t* stage = smem + L::kQ + t * L::kTileBytes;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        if (c * 32 >= p.dvo) break;
        float o[32];
        tmem_ld32f(o_addr + c * 32, o);
        tmem_wait_ld();
        stage_put32<T>(stage, r, c * 32, o, inv, HD * 2);
      }
      __syncwarp();
      warp_copy_out<T, HD / 8>(stage, reinterpret_cast<T*>(p.out.ptr) + (int64_t)sq.bidx * p.out.s[0] +
                                          (int64_t)h * p.out.s[1] + (sq.q0 + m0 + t * kBM) * p.out.s[2],
                               p.out.s[2], min(kBM, sq.sq - (m0 + t * kBM)), p.dvo, quarter * 32, 0, lane, HD * 2);
      if (p.lse != nullptr && m < sq.sq)
        p.lse[lse_offset(p, sq, h) + m] = (l > 0.f) ? (m_used + log2f(l)) * kLn2 : INFINITY;
    }
    }   // t < ntile
  }

  // ---- tear-down ------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

inline bool exact_tiles(const Params& p, int hd) {
  return p.varlen_mode == 0 && p.max_sq % 128 == 0 && p.max_sk % 128 == 0 && p.dqk == hd && p.dvo == hd;
}

template <typename T, int HD, bool EXACT>
cudaError_t launch_fwd_TE(const Params& p, cudaStream_t st) {
  using L = FwdSmem<HD>;
  CUtensorMap tq, tk, tv;
  if (!make_tile_map_16bit(&tq, p.q, p.dqk, p.q.n[2], kBM) || !make_tile_map_16bit(&tk, p.k, p.dqk, p.k.n[2], kBN) ||
      !make_tile_map_16bit(&tv, p.v, p.dvo, p.v.n[2], kBN))
    return cudaErrorInvalidValue;
  // The shared-memory attribute belongs to the (function, device) pair and the status word's
  // address to the device: both are looked up once per device (the current one, which the entry
  // points make the stream's device) and remembered.
  static std::atomic<unsigned int*> status_of[64];
  static std::atomic<bool> attr_set[64];
  int dev = 0;
  cudaError_t e = host().get_device(&dev);
  if (e != cudaSuccess) return e;
  const bool cached = dev >= 0 && dev < 64 && !host_pretends();
  if (!cached || !attr_set[dev].load(std::memory_order_acquire)) {
    e = host().func_set_smem(reinterpret_cast<const void*>(sm100_fwd_kernel<T, HD, EXACT>), L::kDynamic);
    if (e != cudaSuccess) return e;
    if (cached) attr_set[dev].store(true, std::memory_order_release);
  }
  unsigned int* status = cached ? status_of[dev].load(std::memory_order_acquire) : nullptr;
  if (status == nullptr) {
    e = host().symbol_address(reinterpret_cast<void**>(&status), reinterpret_cast<const void*>(&g_sm100_fwd_status));
    if (e != cudaSuccess) return e;
    if (cached) status_of[dev].store(status, std::memory_order_release);
  }
  dim3 grid((p.max_sq + L::kCtaRows - 1) / L::kCtaRows, p.hq, p.batch);
  e = launch_kernel(sm100_fwd_kernel<T, HD, EXACT>, grid, dim3(kFwdThreads), L::kDynamic, st, p, tq, tk, tv, status);
  if (e == cudaSuccess) count_launch();
  return e;
}

template <typename T, int HD>
cudaError_t launch_fwd_T(const Params& p, cudaStream_t st) {
  return exact_tiles(p, HD) ? launch_fwd_TE<T, HD, true>(p, st) : launch_fwd_TE<T, HD, false>(p, st);
}

}  // namespace

bool sm100_fwd_supported(int dtype, const Params& p) {
  if (dtype != 2 && dtype != 3) return false;                    // fp16 / bf16 only
  if (p.dqk > 256 || p.dvo > 256 || p.dqk % 8 != 0 || p.dvo % 8 != 0) return false;
  if (p.max_sq <= 0 || p.max_sk <= 0 || p.batch <= 0) return false;
  if (!tma_friendly(p.q) || !tma_friendly(p.k) || !tma_friendly(p.v)) return false;
  // O is written with 16-byte vector stores
  if (!aligned16(p.out.ptr) || p.out.s[0] % 8 != 0 || p.out.s[1] % 8 != 0 || p.out.s[2] % 8 != 0) return false;
  if (p.q.n[3] != p.dqk || p.k.n[3] != p.dqk || p.v.n[3] != p.dvo) return false;
  return host().have_encoder();
}

cudaError_t launch_sm100_fwd(int dtype, const Params& p, cudaStream_t st) {
  const int dmax = p.dqk > p.dvo ? p.dqk : p.dvo;
  if (dtype == 2)
    return dmax <= 64 ? launch_fwd_T<__half, 64>(p, st)
                      : (dmax <= 128 ? launch_fwd_T<__half, 128>(p, st) : launch_fwd_T<__half, 256>(p, st));
  return dmax <= 64 ? launch_fwd_T<__nv_bfloat16, 64>(p, st)
                    : (dmax <= 128 ? launch_fwd_T<__nv_bfloat16, 128>(p, st) : launch_fwd_T<__nv_bfloat16, 256>(p, st));
}

#ifdef AB200_TRACE
extern "C" __attribute__((visibility("default"))) int ab200_debug_read_fwd_trace(long long* out, int n) {
  return (int)cudaMemcpyFromSymbol(out, g_fwd_trace, sizeof(long long) * (size_t)(n < 2048 ? n : 2048));
}
#endif

unsigned int sm100_fwd_status(bool reset) {
  unsigned int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_sm100_fwd_status, sizeof(v)) != cudaSuccess) { (void)cudaGetLastError(); return 0xffffffffu; }
  if (reset && v != 0) {
    unsigned int zero = 0;
    if (cudaMemcpyToSymbol(g_sm100_fwd_status, &zero, sizeof(zero)) != cudaSuccess) (void)cudaGetLastError();
  }
  return v;
}

}  // namespace ab200
