// Backward attention on tcgen05 (sm_100a): the dK/dV kernel and the dQ(+dBias) kernel.
// (delta = rowsum(O * dO) is produced beforehand by the streaming preprocess kernel.)
//
// Both kernels recompute the probabilities from Q, K and the forward's logsumexp and share
// one scheme.  A unit of work is 128 rows of the output (keys for dK/dV, queries for dQ) against
// all reachable 128-wide blocks of the other sequence dimension.  The dQ kernel runs one CTA per
// unit; the dK/dV kernel is persistent (one CTA per SM draws units from a ticket counter and keeps
// its pipeline up across them).  Twenty warps:
//
//   warp 0      TMA producer   resident operand pair per unit, the streamed operands through
//                              rings (cp.async.bulk.tensor, 128-byte swizzle): Q and dO together
//                              in two stages (dK/dV); K in three stages, V in two (dQ)
//   warp 1      MMA issuer     walks its loop warp-uniformly, one elected lane issues all
//                              tcgen05.mma and tcgen05.commit
//   warp 2      (dK/dV only)   stages -logsumexp*log2(e) and -delta of the streamed query
//                              block in shared memory
//   warp 3      (dK/dV only)   draws the CTA's next unit from the ticket counter
//   warps 4-19  compute        thread = one output row of the 128x128 score tile (TMEM lane),
//                              the four warpgroups split its columns 32 apiece
//
//   dK/dV, per query block i:   S^T = K Q_i^T      dP^T = V dO_i^T        (operands in smem)
//                               P^T, dS^T computed in registers, written back over S^T / dP^T
//                               as packed 16-bit
//                               dV += P^T dO_i     dK += dS^T Q_i         (A from TMEM)
//   dQ, per key block i:        S = Q K_i^T        dP = dO V_i^T
//                               dQ += dS K_i       dB = dS
//                               (dP runs two blocks ahead in two buffers, S one and a half)
//
// Tensor memory, dK/dV: [0,128) S^T, [128,256) dP^T then P^T and dS^T, [256,384) dV, [384,512) dK.
// Tensor memory, dQ:    [0,128) S, [128,256) and [256,384) two dP / dS buffers, [384,512) dQ.
// A warpgroup writes its packed 16-bit results into the first half of ITS OWN column range
// (columns it has already read), so the warpgroups never overwrite each other's input;
// the MMA issuer addresses the four pieces separately.
//
// Arithmetic contract (ROCm/aotriton modules/flash/kernel/bwd_inner_dk_dv.py:117-256,
// bwd_inner_dq.py:117-205, bwd_kernel_dk_dv.py:387-391, bwd_kernel_dq.py:374-376):
//   P = exp2(qk_scale * QK^T + bias*log2e - LSE*log2e), 0 where masked;
//   dP = dO V^T, with dropout: keep ? dP/(1-p) : 0;   dS = P * (dP - delta) with the un-dropped P;
//   dV += cast(keep ? P/(1-p) : 0)^T dO;  dK += cast(dS)^T Q;  dQ += cast(dS) K;  dB = cast(dS);
//   dK and dQ are multiplied by sm_scale at the end.
//
// The dK/dV kernel has a second form (FUSED) that also produces dQ, so that the backward runs the
// five GEMMs it is counted with instead of seven: per query block it forms the partial
// dQ^T = K^T dS^T (head dim x queries, keys contracted), which the compute warps -- idle at that
// point, waiting for the next S^T -- add to a zero-initialised fp32 accumulator with
// red.global.add (lane = head-dim index: 128 contiguous bytes per instruction); a conversion kernel (general_kernels.cu)
// then scales and casts the accumulator into dQ.  This is the reference's DQ_ACC / bwd_postprocess
// path (include/aotriton/flash.h:40,170, modules/flash/kernel/bwd_postprocess.py:14-84); the sum
// order of the atomics is not fixed, so it is used only when attn_options::deterministic is false.
// In that form dS^T also goes to shared memory (the tile the write-out staging uses between items)
// as the N-major B operand of dQ^T, and the dQ^T partial of iteration i takes the S^T columns once
// the compute warps have copied S^T_{i+1} out: it runs under their first exponentials of iteration
// i+1 and is added out between the remaining ones; S^T_{i+2} follows it into the columns.
//   order on the tensor pipe:  dV_i | dQ^T_i  dK_i  dP^T_{i+1} | S^T_{i+2}
//
// Every wait is bounded (sm100_ptx.cuh).
#include <atomic>
#include "launch.h"
#include "sm100_ptx.cuh"

namespace ab200 {

__device__ unsigned int g_sm100_bwd_status = 0;

// Ticket counters of the persistent dK/dV kernel.  Each launch takes the next one of the pool and
// zeroes it in stream order, so launches on different streams do not share a counter unless more
// than kTicketPool of them are in flight at once.
constexpr unsigned int kTicketPool = 256;
__device__ unsigned int g_dkdv_ticket[kTicketPool];

// Optional pipeline trace (compile with -DAB200_TRACE): SM cycle stamps of the hand-offs of the
// first CTA of the dK/dV kernel, six per iteration, read back with ab200_debug_read_trace().
#ifndef AB200_TRACE_TID
#define AB200_TRACE_TID 128   // thread whose compute-side stamps are recorded
#endif
#ifdef AB200_TRACE
__device__ long long g_bwd_trace[16 * 256];
#define AB200_STAMP(iter, slot)                                                                         \
  do {                                                                                                  \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (iter) < 256) g_bwd_trace[(iter) * 16 + (slot)] = clock64(); \
  } while (0)
#else
#define AB200_STAMP(iter, slot) do {} while (0)
#endif
#if defined(AB200_TRACE) && defined(AB200_TRACE_DQ)   // stamps of the dQ kernel's last-launched first CTA instead
#define AB200_STAMPQ(iter, slot)                                                                        \
  do {                                                                                                  \
    if (blockIdx.x == gridDim.x - 1 && blockIdx.y == 0 && blockIdx.z == 0 && (iter) < 256) g_bwd_trace[(iter) * 16 + (slot)] = clock64(); \
  } while (0)
#else
#define AB200_STAMPQ(iter, slot) do {} while (0)
#endif

namespace {

using namespace ptx;

constexpr int kBlk = 128;
constexpr int kBwdThreads = 640;
constexpr int kFusedThreads = kBwdThreads;
constexpr int kComputeWarps = 16;      // warps 4..19; each arrives on the hand-off barriers once (lane 0)
constexpr int kWgCols = 32;            // score columns per compute warpgroup
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColDP = 128, kColAcc0 = 256, kColAcc1 = 384;

template <int HD>
struct BwdSmem {
  static constexpr int kHalves = HD / 64;
  static constexpr int kTile = kHalves * 16384;          // 128 rows x HD x 2 bytes
  static constexpr int kResA = 0, kResB = kTile;         // resident pair
  static constexpr int kRingA = 2 * kTile, kRingB = 4 * kTile;   // two stages each
  static constexpr int kStage = 6 * kTile;               // write-out staging: 128 rows x HD, 16-bit
  static constexpr int kAux = kStage + kTile;            // 2 stages x (128 lse2 + 128 delta) floats
  static constexpr int kAuxFlag = kAux + 2 * 256 * 4;    // per stage: 1 when some |lse2| is huge
  static constexpr int kSched = kAuxFlag + 16;             // two slots: next work item of this CTA
  static constexpr int kBars = kSched + 16;
  static constexpr int bResFull = 0, bRingFull = 1, bRingEmpty = 3, bSFull = 5 /* two */, bAuxEmpty = 7,
                       bDpFull = 10 /* two: one per dP buffer in the dQ kernel */, bDsFull = 12, bAccDone = 13, bSRead = 14,
                       bResEmpty = 15, bPFull = 16, bSchedFull = 17, bSchedEmpty = 19, bDqFull = 21, bDqRead = 22,
                       bStageFree = 23, bCount = 24;
  static constexpr int kTmemSlot = kBars + bCount * 8;
  static constexpr int kAbort = kTmemSlot + 4;           // abort word, then the launch's wait limit
  static constexpr int kUsed = kAbort + 8;
  // The tiles need 1024-byte alignment, which is established at run time; the kernel checks that
  // the padding it needed still fits (without static shared memory the base is aligned already).
  static constexpr int kDynamic = kUsed + 512;
};

// Descriptors are built once per tile base; a k-step or a ring stage only moves the 14-bit
// start-address field (units of 16 bytes).
// K-major view of a [128 x HD] tile: k-step kk covers head-dim columns 16kk..16kk+15.
__device__ __forceinline__ uint64_t kmajor_base(uint32_t tile_addr) { return smem_desc_sw128(tile_addr, 16, 1024); }
__device__ __forceinline__ constexpr uint32_t kmajor_step(int kk) {
  return (uint32_t)(kk >> 2) * (16384u >> 4) + (uint32_t)(kk & 3) * (32u >> 4);
}
// MN-major view of the same tile: k-step kk covers rows 16kk..16kk+15, N runs over the head dim.
__device__ __forceinline__ uint64_t mnmajor_base(uint32_t tile_addr) { return smem_desc_sw128(tile_addr, 16384, 1024); }
__device__ __forceinline__ constexpr uint32_t mnmajor_step(int kk) { return (uint32_t)kk * (2048u >> 4); }
// Column of the packed 16-bit A operand for k-step kk (16 source columns = 8 packed columns):
// each warpgroup packed its 32 source columns into the first 16 columns of its own range.
__device__ __forceinline__ uint32_t split_a_col(int kk) { return (uint32_t)(kWgCols * (kk >> 1) + (kk & 1) * 8); }

template <typename T>
__device__ __forceinline__ void store_row_chunk32(T* dst, const float* v, float scale, int d0, int dmax) {
#pragma unroll
  for (int v8 = 0; v8 < 4; ++v8) {
    const int d = d0 + v8 * 8;
    if (d < dmax) {
      uint4 w;
      w.x = pack2<T>(v[v8 * 8 + 0] * scale, v[v8 * 8 + 1] * scale);
      w.y = pack2<T>(v[v8 * 8 + 2] * scale, v[v8 * 8 + 3] * scale);
      w.z = pack2<T>(v[v8 * 8 + 4] * scale, v[v8 * 8 + 5] * scale);
      w.w = pack2<T>(v[v8 * 8 + 6] * scale, v[v8 * 8 + 7] * scale);
      *reinterpret_cast<uint4*>(dst + d) = w;
    }
  }
}

// Bias of a key-per-thread kernel.  A warp owns 32 keys (one per lane) x 32 query rows of the score
// tile, i.e. a 32 x 32 tile of the bias matrix whose rows (queries) are 64 contiguous bytes.  A
// thread needs a COLUMN of it; reading that directly takes 32 two-byte loads per thread at a row
// stride.  Instead the warp reads the tile with four 16-byte loads per thread (load t: lane 8q+e
// reads keys 8q..8q+7 of query row 8t+e) and transposes it in registers: within each group of
// eight lanes an 8 x 8 transpose of 16-bit values, three exchange steps (lane bit <-> position bit).
// Adds bias * log2(e) to pr[c] (c = query row in the tile).  `tile` points at (first query row,
// first key of the warp); rows are `row_stride` elements apart and 16-byte aligned.
template <typename T>
__device__ __forceinline__ void add_bias_column32(float* pr, const T* tile, int64_t row_stride, int lane) {
  const int q = lane >> 3, e = lane & 7;
  uint4 raw[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) raw[t] = __ldg(reinterpret_cast<const uint4*>(tile + (int64_t)(8 * t + e) * row_stride + 8 * q));
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    uint32_t w[4] = {raw[t].x, raw[t].y, raw[t].z, raw[t].w};
    // lane bit 0 <-> low/high half
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t o = __shfl_xor_sync(0xffffffffu, w[k], 1);
      w[k] = (lane & 1) ? __byte_perm(w[k], o, 0x3276) : __byte_perm(w[k], o, 0x5410);
    }
    // lane bit 1 <-> register index bit 0, lane bit 2 <-> register index bit 1
#pragma unroll
    for (int k = 0; k < 4; k += 2) {
      const bool up = (lane & 2) != 0;
      const uint32_t got = __shfl_xor_sync(0xffffffffu, up ? w[k] : w[k + 1], 2);
      if (up) w[k] = got; else w[k + 1] = got;
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const bool up = (lane & 4) != 0;
      const uint32_t got = __shfl_xor_sync(0xffffffffu, up ? w[k] : w[k + 2], 4);
      if (up) w[k] = got; else w[k + 2] = got;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const T* h = reinterpret_cast<const T*>(&w[k]);
      pr[8 * t + 2 * k] = fmaf(to_f32<T>(h[0]), kLog2e, pr[8 * t + 2 * k]);
      pr[8 * t + 2 * k + 1] = fmaf(to_f32<T>(h[1]), kLog2e, pr[8 * t + 2 * k + 1]);
    }
  }
}

template <typename T>
__device__ void zero_rows(const View4& v, int b, int h, int64_t tok0, int row0, int nrows, int d) {
  for (int r = threadIdx.x; r < kBlk; r += blockDim.x) {
    if (row0 + r >= nrows) continue;
    T* ptr = reinterpret_cast<T*>(v.ptr) + (int64_t)b * v.s[0] + (int64_t)h * v.s[1] + (tok0 + row0 + r) * v.s[2];
    for (int c = 0; c < d; ++c) ptr[c] = from_f32<T>(0.f);
  }
}

template <int HD>
__device__ __forceinline__ void init_barriers(uint64_t* bars, volatile uint32_t* abort_flag, uint32_t limit_kcycles) {
  using L = BwdSmem<HD>;
  init_abort_and_limit(abort_flag, limit_kcycles);
  mbar_init(&bars[L::bResFull], 1);
  for (int s = 0; s < 2; ++s) {
    mbar_init(&bars[L::bRingFull + s], 1);
    mbar_init(&bars[L::bRingEmpty + s], 1);
    mbar_init(&bars[L::bSFull + s], 2);          // the S GEMM's commit and the aux warp's arrival
    mbar_init(&bars[L::bAuxEmpty + s], kComputeWarps);
    mbar_init(&bars[L::bSchedFull + s], 1);
    mbar_init(&bars[L::bSchedEmpty + s], kComputeWarps + 3);   // compute warps, producer, MMA issuer, aux warp
  }
  mbar_init(&bars[L::bDqFull], 1);
  mbar_init(&bars[L::bDqRead], kComputeWarps);
  mbar_init(&bars[L::bStageFree], kComputeWarps);
  mbar_init(&bars[L::bDpFull], 1);
  mbar_init(&bars[L::bDpFull + 1], 1);
  mbar_init(&bars[L::bDsFull], kComputeWarps);
  mbar_init(&bars[L::bPFull], kComputeWarps);
  mbar_init(&bars[L::bAccDone], 1);
  mbar_init(&bars[L::bSRead], kComputeWarps);
  mbar_init(&bars[L::bResEmpty], 1);
  fence_barrier_init();
}

// =========================================================================================
// dK / dV.  Persistent: one CTA per SM walks work items (128 keys of one sequence and kv head),
// heaviest first; the pipeline (rings, barriers, tensor memory) stays up across items, so the
// next item's K/V and first Q/dO blocks are fetched and its first two GEMMs issued while the
// current item is still finishing.  All roles enumerate the same items and keep the same running
// counters: G counts query-block iterations since the kernel started (ring stage G&1, hand-off
// parity G&1), `live` counts items that had work (parity of the once-per-item barriers).
struct DkdvItem {
  int z, hk, n0;
  Seq sq;
  int mb_lo, nmb, niter;   // niter == 0: keys no query attends to (gradients are zero)
  bool valid;              // false: key block beyond this sequence
};

__device__ __forceinline__ DkdvItem dkdv_item(const Params& p, int w) {
  DkdvItem it;
  const int per = p.batch * p.hk;
  const int nkb = (p.max_sk + kBlk - 1) / kBlk;
  const int grp = w / (nkb * 8), r = w - grp * (nkb * 8);
  const int kb = r >> 3, rem = grp * 8 + (r & 7);
  it.z = min(rem, per - 1) / p.hk;
  it.hk = min(rem, per - 1) - it.z * p.hk;
  it.n0 = kb * kBlk;
  it.sq = resolve_seq(p, it.z);
  it.valid = rem < per && it.n0 < it.sq.sk;
  it.mb_lo = it.nmb = it.niter = 0;
  if (it.valid) {
    int m_lo, m_hi;
    query_range(p, it.sq, it.n0, min(it.n0 + kBlk, it.sq.sk) - 1, m_lo, m_hi);
    if (m_hi >= m_lo) {
      it.mb_lo = m_lo / kBlk;
      it.nmb = m_hi / kBlk - it.mb_lo + 1;
      it.niter = it.nmb * p.group;
    }
  }
  return it;
}

// EXACT: a dense problem whose sequence lengths are multiples of 128 and whose head dimensions equal
// HD: every tile is full, so the instantiation carries no tail handling and fixed GEMM shapes (the
// MMA issuer's loop is latency-critical: even untaken branches and call sites in it cost several
// per cent of the kernel's time).
template <typename T, int HD, bool FUSED, bool EXACT>
__global__ void __launch_bounds__(FUSED ? kFusedThreads : kBwdThreads, 1)
sm100_bwd_dkdv_kernel(const __grid_constant__ Params p, const __grid_constant__ CUtensorMap tm_q,
                      const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const __grid_constant__ CUtensorMap tm_do, unsigned int* status, int nitems,
                      unsigned int* ticket, float* dq_acc) {
  using L = BwdSmem<HD>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlot);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::kAbort);
  float* aux = reinterpret_cast<float*>(smem + L::kAux);
  const uint32_t aux_s = smem_u32(smem + L::kAux);
  volatile uint32_t* aux_flag = reinterpret_cast<volatile uint32_t*>(smem + L::kAuxFlag);
  volatile int* sched = reinterpret_cast<volatile int*>(smem + L::kSched);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // An earlier CTA timed out: the whole CTA leaves (one read, one CTA-wide decision).
  if (__syncthreads_or(threadIdx.x == 0 && *reinterpret_cast<volatile unsigned int*>(status) != 0u)) return;
  if ((int)(smem - smem_raw) + L::kUsed > L::kDynamic) {      // the alignment padding did not fit
    if (threadIdx.x == 0) atomicCAS(status, 0u, 0x1F00u);
    return;
  }

  // Work items are handed out dynamically: the first one is the CTA's index, every further one
  // comes from a global ticket counter (warp 3 draws it one item ahead and publishes it in a
  // two-slot ring that every other role reads).  `m` counts the items a role has drawn.
  auto next_item = [&](uint32_t m, bool whole_warp) -> int {
    const uint32_t k = m & 1u;
    if (!mbar_wait(&bars[L::bSchedFull + k], (m >> 1) & 1u, abort_flag, status, 0x1B00)) return 0x7fffffff;
    const int w = sched[k];
    if (whole_warp) {
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[L::bSchedEmpty + k]);
    } else {
      mbar_arrive(&bars[L::bSchedEmpty + k]);
    }
    return w;
  };

  if (threadIdx.x == 0) {
    init_barriers<HD>(bars, abort_flag, p.wait_limit_kcycles);
    prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v); prefetch_tmap(&tm_do);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (warp == 0) {
    // ================================ TMA producer ===================================
    if (lane == 0) {
      uint32_t G = 0, live = 0, drawn = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < nitems; w = next_item(drawn++, false)) {
        const DkdvItem it = dkdv_item(p, w);
        if (!it.valid || it.niter == 0) continue;
        // K and V of the previous item are free once its last S and dP GEMMs have run.
        if (!mbar_wait(&bars[L::bResEmpty], (live & 1u) ^ 1u, abort_flag, status, 0x1000)) break;
        const int krow = (int)(it.sq.k0 + it.n0);
        mbar_expect_tx(&bars[L::bResFull], 2 * L::kTile);
        for (int hf = 0; hf < L::kHalves; ++hf) {
          tma_load_4d(smem + L::kResA + hf * 16384, &tm_k, &bars[L::bResFull], hf * 64, krow, it.hk, it.sq.bidx);
          tma_load_4d(smem + L::kResB + hf * 16384, &tm_v, &bars[L::bResFull], hf * 64, krow, it.hk, it.sq.bidx);
        }
        for (int i = 0, hg = 0, mb = 0; i < it.niter; ++i, ++G) {     // hg, mb: i / nmb, i % nmb
          const int s = (int)(G & 1u);
          const int h = it.hk * p.group + hg;
          const int mrow = (int)(it.sq.q0 + (int64_t)(it.mb_lo + mb) * kBlk);
          if (++mb == it.nmb) { mb = 0; ++hg; }
          if (!mbar_wait(&bars[L::bRingEmpty + s], ((G >> 1) & 1u) ^ 1u, abort_flag, status, 0x1100)) { ok = false; break; }
          if (p.drop_copy == 2 && G == 0) continue;   // test hook: this Q/dO block never arrives
          mbar_expect_tx(&bars[L::bRingFull + s], 2 * L::kTile);
          for (int hf = 0; hf < L::kHalves; ++hf) {
            tma_load_4d(smem + L::kRingA + s * L::kTile + hf * 16384, &tm_q, &bars[L::bRingFull + s], hf * 64, mrow, h,
                        it.sq.bidx);
            tma_load_4d(smem + L::kRingB + s * L::kTile + hf * 16384, &tm_do, &bars[L::bRingFull + s], hf * 64, mrow, h,
                        it.sq.bidx);
          }
        }
        ++live;
      }
      if (*abort_flag) {
        // Let copies that are still in flight land before the CTA gives its shared memory back.
        if (live > 0) mbar_wait_quiet(&bars[L::bResFull], (live - 1) & 1u, abort_flag);
        for (uint32_t g = (G >= 2 ? G - 2 : 0); g < G; ++g) {
          if (p.drop_copy == 2 && g == 0) continue;   // (never issued)
          mbar_wait_quiet(&bars[L::bRingFull + (g & 1u)], (g >> 1) & 1u, abort_flag);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================================= MMA issuer ====================================
    // The whole warp walks the loop and waits; one elected lane issues.  With warp-uniform control
    // flow the descriptors stay in uniform registers and a GEMM costs few issue slots.
    // Contractions over a head dimension run over it rounded up to 16, products into a head
    // dimension produce it rounded up to 16 (the copies zero-fill up to the 64-column box).
    constexpr uint32_t kIdescSS = instr_desc_f16(Fmt<T>::code, 128, 128, 0, 0);
    // (EXACT: all equal the kernel's head dimension, known at compile time)
    const uint32_t kIdescDV = instr_desc_f16(Fmt<T>::code, 128, EXACT ? (uint32_t)HD : (uint32_t)((p.dvo + 15) & ~15), 0, 1);
    const uint32_t kIdescDK = instr_desc_f16(Fmt<T>::code, 128, EXACT ? (uint32_t)HD : (uint32_t)((p.dqk + 15) & ~15), 0, 1);
    const int ksteps_qk = EXACT ? HD / 16 : (p.dqk + 15) >> 4, ksteps_vo = EXACT ? HD / 16 : (p.dvo + 15) >> 4;
    constexpr uint32_t kStageStep = L::kTile >> 4;
    const uint64_t k_km = kmajor_base(smem_u32(smem + L::kResA)), v_km = kmajor_base(smem_u32(smem + L::kResB));
    const uint64_t q_km = kmajor_base(smem_u32(smem + L::kRingA)), do_km = kmajor_base(smem_u32(smem + L::kRingB));
    const uint64_t q_mn = mnmajor_base(smem_u32(smem + L::kRingA)), do_mn = mnmajor_base(smem_u32(smem + L::kRingB));
    // fused form: K as the M-major A operand of dQ^T, the dS^T tile as its N-major B operand
    const uint64_t k_mn = mnmajor_base(smem_u32(smem + L::kResA));
    const uint64_t ds_mn = mnmajor_base(smem_u32(smem + L::kStage));
    constexpr uint32_t kIdescDQT = instr_desc_f16(Fmt<T>::code, 128, 128, 1, 1);
    auto wait = [&](int bar, uint32_t parity, uint32_t where) {
      return __all_sync(0xffffffffu, mbar_wait(&bars[bar], parity, abort_flag, status, where)) != 0;
    };
    auto issue_s = [&](uint32_t g) {      // S^T = K Q_g^T
      const uint64_t qa = q_km + (uint64_t)((g & 1u) * kStageStep);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          if (kk < ksteps_qk)
            mma_ss(tmem_base + kColS, k_km + kmajor_step(kk), qa + kmajor_step(kk), kIdescSS, kk > 0 ? 1u : 0u);
        mma_commit(&bars[L::bSFull + (g & 1u)]);
      }
      __syncwarp();
    };
    // dP^T = V dO_g^T; `release_kv`: these are the last readers of the item's K and V
    auto issue_dp = [&](uint32_t g, bool release_kv) {
      const uint64_t da = do_km + (uint64_t)((g & 1u) * kStageStep);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          if (kk < ksteps_vo)
            mma_ss(tmem_base + kColDP, v_km + kmajor_step(kk), da + kmajor_step(kk), kIdescSS, kk > 0 ? 1u : 0u);
        mma_commit(&bars[L::bDpFull]);
        if (release_kv) mma_commit(&bars[L::bResEmpty]);
      }
      __syncwarp();
    };
    uint32_t G = 0, live = 0, drawn = 0;
    bool ok = true;
    for (int w = blockIdx.x; ok && w < nitems; w = next_item(drawn++, true)) {
      const DkdvItem it = dkdv_item(p, w);
      if (!it.valid || it.niter == 0) continue;
      // first iteration of the item: K/V resident, Q/dO block landed, S buffer read out by the
      // compute warps (the dP buffer is released in issue order by the previous item's dV/dK)
      if (!wait(L::bResFull, live & 1u, 0x1200)) break;
      // Last, partial key block of the sequence: keys beyond its end are rows of S^T / dP^T that are
      // never stored, but in the fused form they are contracted over by dQ^T, where a zero dS^T times
      // a non-finite K row (or dS^T made non-finite by a V row) would poison the sum.
      if constexpr (!EXACT) {
        if (it.sq.sk - it.n0 < kBlk) {
          zero_tail_rows(smem + L::kResA, it.sq.sk - it.n0, L::kHalves, lane);
          zero_tail_rows(smem + L::kResB, it.sq.sk - it.n0, L::kHalves, lane);
        }
      }
      if (G > 0 && !wait(L::bSRead, (G - 1) & 1u, 0x1201)) break;
      if constexpr (FUSED) {      // the previous item's last dQ^T partial has left the S columns
        if (G > 0 && !wait(L::bDqRead, (G - 1) & 1u, 0x1203)) break;
      }
      if (!wait(L::bRingFull + (G & 1u), (G >> 1) & 1u, 0x1202)) break;
      if (lane == 0) AB200_STAMP(G, 15);
      // Last, partial query block of the sequence: rows of Q and dO beyond its end must not reach
      // the dV / dK products (a zero probability times a non-finite value would poison them).
      auto zero_ring_tail = [&](uint32_t g, int mb) {
        if constexpr (!EXACT) {
          const int valid = it.sq.sq - (it.mb_lo + mb) * kBlk;
          if (valid < kBlk) {
            zero_tail_rows(smem + L::kRingA + (g & 1u) * L::kTile, valid, L::kHalves, lane);
            zero_tail_rows(smem + L::kRingB + (g & 1u) * L::kTile, valid, L::kHalves, lane);
          }
        }
      };
      zero_ring_tail(G, 0);
      tc_fence_after();
      issue_s(G);
      issue_dp(G, !FUSED && it.niter == 1);
      if (lane == 0) AB200_STAMP(G, 8);
      // dQ^T_g = K^T dS^T_g into the S columns (free once the compute warps have copied the next S^T
      // out): both operands in shared memory, keys contracted in 8 steps of 16
      auto issue_dqt = [&](uint32_t g) {
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            mma_ss(tmem_base + kColS, k_mn + mnmajor_step(kk), ds_mn + mnmajor_step(kk), kIdescDQT, kk > 0 ? 1u : 0u);
          mma_commit(&bars[L::bDqFull]);
        }
        __syncwarp();
      };
      for (int i = 0, mb_next = 1; i < it.niter; ++i, ++G, ++mb_next) {     // mb_next: (i + 1) % nmb
        const uint32_t s = G & 1u, par = G & 1u;
        if (mb_next == it.nmb) mb_next = 0;
        if constexpr (FUSED) {
          // The S columns hold dQ^T_{g-1} (issued at the end of the previous iteration, when S_g had
          // been copied out); S_{g+1} follows once the compute warps have fetched that partial.
          if (i > 0) {
            if (!wait(L::bDqRead, (G - 1) & 1u, 0x1580)) { ok = false; break; }
            if (lane == 0) AB200_STAMP(G, 14);
          } else if (!wait(L::bSRead, par, 0x1300)) { ok = false; break; }
          if (i + 1 < it.niter) {
            if (!wait(L::bRingFull + ((G + 1) & 1u), ((G + 1) >> 1) & 1u, 0x1400)) { ok = false; break; }
            zero_ring_tail(G + 1, mb_next);
            tc_fence_after();
            issue_s(G + 1);
            if (lane == 0) AB200_STAMP(G, 13);
          }
        } else if (i + 1 < it.niter) {
          // S_g sits in registers of every compute thread: its buffer can take S_{g+1} already.
          if (!wait(L::bSRead, par, 0x1300)) { ok = false; break; }
          if (!wait(L::bRingFull + ((G + 1) & 1u), ((G + 1) >> 1) & 1u, 0x1400)) { ok = false; break; }
          zero_ring_tail(G + 1, mb_next);
          tc_fence_after();
          issue_s(G + 1);
        }
        const uint32_t first = (i > 0) ? 1u : 0u;
        // P^T is handed over ahead of dS^T (it does not need the dS arithmetic): dV runs meanwhile
        if (!wait(L::bPFull, par, 0x1480)) { ok = false; break; }
        tc_fence_after();
        if (elect_one()) {   // dV += P^T dO_g   (P^T: first 16 packed columns of each warpgroup's range of the dP buffer)
          const uint64_t da = do_mn + (uint64_t)(s * kStageStep);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            mma_ts(tmem_base + kColAcc0, tmem_base + kColDP + split_a_col(kk), da + mnmajor_step(kk), kIdescDV,
                   kk > 0 ? 1u : first);
        }
        __syncwarp();
        if (!wait(L::bDsFull, par, 0x1500)) { ok = false; break; }
        if (lane == 0) AB200_STAMP(G, 5);
        tc_fence_after();
        if constexpr (FUSED) {
          // dQ^T_g goes first: the compute warps, now in iteration g+1, need it after their first
          // exponentials; it takes the S columns as soon as they have copied S_{g+1} out.
          if (i + 1 < it.niter) {
            if (!wait(L::bSRead, (G + 1) & 1u, 0x1301)) { ok = false; break; }
            tc_fence_after();
            issue_dqt(G);
            if (lane == 0) AB200_STAMP(G, 9);
          }
        }
        if (elect_one()) {   // dK += dS^T Q_g  (dS^T: the next 16 packed columns)
          const uint64_t qa = q_mn + (uint64_t)(s * kStageStep);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            mma_ts(tmem_base + kColAcc1, tmem_base + kColDP + 16u + split_a_col(kk), qa + mnmajor_step(kk), kIdescDK,
                   kk > 0 ? 1u : first);
          mma_commit(&bars[L::bRingEmpty + s]);
          if (i + 1 == it.niter) mma_commit(&bars[L::bAccDone]);
        }
        __syncwarp();
        if (i + 1 < it.niter) {
          issue_dp(G + 1, !FUSED && i + 2 == it.niter);
        } else if constexpr (FUSED) {
          // the item's last partial: the S columns are free (no S^T of this item follows)
          issue_dqt(G);
          if (elect_one()) mma_commit(&bars[L::bResEmpty]);      // K was still being read by dQ^T
          __syncwarp();
        }
      }
      if (!ok) break;
      ++live;
    }
  } else if (warp == 2) {
    // logsumexp (in log2 units) and delta of the streamed query blocks
    uint32_t G = 0, drawn = 0;
    bool ok = true;
    for (int w = blockIdx.x; ok && w < nitems; w = next_item(drawn++, true)) {
      const DkdvItem it = dkdv_item(p, w);
      if (!it.valid || it.niter == 0) continue;
      for (int i = 0, hg = 0, mb = 0; i < it.niter; ++i, ++G) {     // hg, mb: i / nmb, i % nmb
        const int s = (int)(G & 1u);
        if (!mbar_wait_relaxed(&bars[L::bAuxEmpty + s], ((G >> 1) & 1u) ^ 1u, abort_flag, status, 0x1600)) { ok = false; break; }
        const int h = it.hk * p.group + hg;
        const int mbase = (it.mb_lo + mb) * kBlk;
        if (++mb == it.nmb) { mb = 0; ++hg; }
        const int64_t lrow = lse_offset(p, it.sq, h);
        float* dst = aux + s * 256;
        bool huge = false;
        float l2[4], dl[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {     // all eight loads in flight before the first store
          const int m = mbase + lane * 4 + t;
          const bool in = m < it.sq.sq;
          l2[t] = in ? __ldg(p.lse + lrow + m) : INFINITY;
          dl[t] = in ? __ldg(p.delta + lrow + m) : 0.f;
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          l2[t] *= kLog2e;
          huge = huge || (fabsf(l2[t]) > 1.0e6f && l2[t] != INFINITY);
        }
        // staged NEGATED (-logsumexp*log2e, -delta): the compute warps add them with packed
        // instructions, which take no negate modifier
        *reinterpret_cast<float4*>(dst + lane * 4) = make_float4(-l2[0], -l2[1], -l2[2], -l2[3]);
        *reinterpret_cast<float4*>(dst + 128 + lane * 4) = make_float4(-dl[0], -dl[1], -dl[2], -dl[3]);
        const bool any_huge = __any_sync(0xffffffffu, huge);
        if (lane == 0) aux_flag[s] = any_huge ? 1u : 0u;
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[L::bSFull + s]);
      }
    }
  } else if (warp == 3) {
    // ================================= scheduler =====================================
    if (lane == 0) {
      for (uint32_t m = 0;; ++m) {
        const uint32_t k = m & 1u;
        if (!mbar_wait_relaxed(&bars[L::bSchedEmpty + k], ((m >> 1) & 1u) ^ 1u, abort_flag, status, 0x1C00)) break;
        const unsigned int t = atomicAdd(ticket, 1u);
        const int w = t < 0x40000000u ? (int)(gridDim.x + t) : 0x7fffffff;
        sched[k] = w;
        mbar_arrive(&bars[L::bSchedFull + k]);
        if (w >= nitems) break;
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ================================== compute ======================================
    const int quarter = warp & 3, wg = (warp - 4) >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int cbase = kWgCols * wg;
    uint32_t G = 0, live = 0, drawn = 0;
    bool ok = true;
    // Philox seed and offset are read once; the round keys depend on the seed only
    const uint64_t ph_seed = (p.dropout_on && p.seed_ptr) ? *p.seed_ptr : 0ull;
    const uint64_t ph_off = p.off2 + ((p.dropout_on && p.off1_ptr) ? *p.off1_ptr : 0ull);
    PhiloxKeys pkeys;
    if (p.dropout_on) pkeys = philox_keys(ph_seed);
    for (int w = blockIdx.x; ok && w < nitems; w = next_item(drawn++, true)) {
      const DkdvItem it = dkdv_item(p, w);
      if (!it.valid) continue;
      const Seq& sq = it.sq;
      const int hk = it.hk, z = it.z;
      const int n = it.n0 + r;
      if (it.niter == 0) {          // no query attends to these keys
        if (wg == 0 && n < sq.sk) {
          T* dkp = reinterpret_cast<T*>(p.dk.ptr) + (int64_t)sq.bidx * p.dk.s[0] + (int64_t)hk * p.dk.s[1] +
                   (sq.k0 + n) * p.dk.s[2];
          T* dvp = reinterpret_cast<T*>(p.dv.ptr) + (int64_t)sq.bidx * p.dv.s[0] + (int64_t)hk * p.dv.s[1] +
                   (sq.k0 + n) * p.dv.s[2];
          for (int c = 0; c < p.dqk; ++c) dkp[c] = from_f32<T>(0.f);
          for (int c = 0; c < p.dvo; ++c) dvp[c] = from_f32<T>(0.f);
        }
        __syncwarp();
        continue;
      }
      int col_lo = 0, col_hi = sq.sq - 1;     // valid query rows for this key
      if (p.causal) {
        int64_t lo = (int64_t)n - sq.wr, hi = (int64_t)n + sq.wl;
        if (lo > col_lo) col_lo = (int)(lo > 0x7fffffffLL ? 0x7fffffffLL : lo);
        if (hi < col_hi) col_hi = (int)(hi < -1 ? -1 : hi);
      }
      if (n >= sq.sk) { col_lo = 1; col_hi = 0; }
      // the tightest bounds over the warp's rows: a block needs masking iff it is not inside them
      const int warp_lo = __reduce_max_sync(0xffffffffu, col_lo), warp_hi = __reduce_min_sync(0xffffffffu, col_hi);
      // Fused form: the dQ^T partial of iteration g (head dim x queries, in the S columns) is taken
      // out during iteration g+1.  This thread owns head-dim row d = its TMEM lane and the 32 query
      // columns of its warpgroup; for a fixed query the warp's lanes add to 32 consecutive floats
      // of the accumulator row (one 128-byte red.global.add).  dq_dst / dq_rows describe the
      // partial that is pending.
      float* dq_dst = nullptr;
      int dq_rows = 0;
      auto dq_add8 = [&](const float* v, int c8) {
        if (r < p.dqk) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int c = 8 * c8 + j;
            if (c < dq_rows) atomicAdd(dq_dst + (int64_t)c * p.dqk, v[j]);
          }
        }
      };
      for (int i = 0, hg = 0, mb = 0; i < it.niter; ++i, ++G) {     // hg, mb: i / nmb, i % nmb
        const int s = (int)(G & 1u);
        const uint32_t par = G & 1u;
        const int h = hk * p.group + hg;
        const int mbase = (it.mb_lo + mb) * kBlk + cbase;    // first query row of this thread's columns
        if (++mb == it.nmb) { mb = 0; ++hg; }
        const uint32_t lse2 = aux_s + (uint32_t)(s * 256 + cbase) * 4u;      // shared-space addresses
        const uint32_t dlt = lse2 + 128u * 4u;
        if (threadIdx.x == AB200_TRACE_TID) AB200_STAMP(G, 4);
        // (the warp's 32 x 32 bias tile, one 64-byte row per lane: on its way to L2 meanwhile)
        if (p.has_bias && p.bias_vec)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const T*>(p.bias.ptr) + (int64_t)sq.bidx * p.bias.s[0] +
                                                       (int64_t)h * p.bias.s[1] + (int64_t)min(mbase + lane, sq.sq - 1) * p.bias.s[2] +
                                                       (it.n0 + quarter * 32)));
        // S^T of this block and its logsumexp/delta stage (two arrivals on one barrier)
        if (!mbar_wait(&bars[L::bSFull + s], (G >> 1) & 1u, abort_flag, status, 0x1800)) { ok = false; break; }
        if (threadIdx.x == AB200_TRACE_TID) AB200_STAMP(G, 0);
        tc_fence_after();
        float pr[32];
        tmem_ld32f(tmem_base + lane_addr + kColS + cbase, pr);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[L::bSRead]);
        if (threadIdx.x == AB200_TRACE_TID) AB200_STAMP(G, 6);
        // (warp-uniform without a vote per block: compared with the warp's extreme bounds)
        const bool any_mask = !(mbase >= warp_lo && mbase + kWgCols - 1 <= warp_hi);
        // exponent arguments: scaled score (+ bias) minus the row's logsumexp, all in log2 units.
        // Common case: one packed FMA per two elements.  With bias, or when the logsumexp is so
        // large that product rounding matters (the aux warp flags that), scale first and subtract
        // second, so that the forward's reference point cancels exactly.
        // Fused form: the previous iteration's dQ^T partial was issued when this warp released the S
        // columns just now and completes under the first exponentials; it is then fetched eight
        // query columns at a time and added out between the remaining ones (the exponentials keep
        // the special-function unit busy and leave the load/store unit idle).
        const bool dq_now = FUSED && i > 0;
        auto exp4 = [&](int c4, float2 sc2) {
          const float4 l4 = lds128(lse2 + 16u * c4);
          const float2 a = fma2(make_float2(pr[4 * c4], pr[4 * c4 + 1]), sc2, make_float2(l4.x, l4.y));
          const float2 b = fma2(make_float2(pr[4 * c4 + 2], pr[4 * c4 + 3]), sc2, make_float2(l4.z, l4.w));
          pr[4 * c4 + 0] = ex2(a.x);
          pr[4 * c4 + 1] = ex2(a.y);
          pr[4 * c4 + 2] = ex2(b.x);
          pr[4 * c4 + 3] = ex2(b.y);
        };
        if (!p.has_bias && aux_flag[s] == 0) {
          const float2 sc2 = make_float2(p.qk_scale, p.qk_scale);
          if (dq_now) {
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) exp4(c4, sc2);
            if (!mbar_wait(&bars[L::bDqFull], (G - 1) & 1u, abort_flag, status, 0x1D00)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int c8 = 0; c8 < 4; ++c8) {
              float dqv[8];
              tmem_ld8f(tmem_base + lane_addr + kColS + cbase + 8 * c8, dqv);
              exp4(4 + c8, sc2);
              tmem_wait_ld();
              if (c8 == 3) {      // everything fetched: the S columns can take the next S^T
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars[L::bDqRead]);
              }
              dq_add8(dqv, c8);
            }
            __syncwarp();
          } else {
#pragma unroll
            for (int c4 = 0; c4 < 8; ++c4) exp4(c4, sc2);
          }
        } else {
          if (dq_now) {
            if (!mbar_wait(&bars[L::bDqFull], (G - 1) & 1u, abort_flag, status, 0x1D00)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int c8 = 0; c8 < 4; ++c8) {
              float dqv[8];
              tmem_ld8f(tmem_base + lane_addr + kColS + cbase + 8 * c8, dqv);
              tmem_wait_ld();
              dq_add8(dqv, c8);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[L::bDqRead]);
          }
#pragma unroll
          for (int c = 0; c < 32; ++c) pr[c] *= p.qk_scale;
          if (p.has_bias && p.bias_vec && mbase + 32 <= sq.sq && it.n0 + quarter * 32 + 32 <= sq.sk) {
            // the warp's whole 32 x 32 bias tile is inside the sequence: vector loads and a transpose
            add_bias_column32<T>(pr, reinterpret_cast<const T*>(p.bias.ptr) + (int64_t)sq.bidx * p.bias.s[0] +
                                         (int64_t)h * p.bias.s[1] + (int64_t)mbase * p.bias.s[2] + (it.n0 + quarter * 32),
                                 p.bias.s[2], lane);
          } else if (p.has_bias && n < sq.sk) {
            const T* bcol = reinterpret_cast<const T*>(p.bias.ptr) + (int64_t)sq.bidx * p.bias.s[0] +
                            (int64_t)h * p.bias.s[1] + (int64_t)n * p.bias.s[3];
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const int m = mbase + c;
              if (m < sq.sq) pr[c] = fmaf(to_f32<T>(bcol[(int64_t)m * p.bias.s[2]]), kLog2e, pr[c]);
            }
          }
          __syncwarp();   // lanes beyond the sequence skipped the loads
#pragma unroll
          for (int c4 = 0; c4 < 8; ++c4) {
            const float4 l4 = lds128(lse2 + 16u * c4);
            pr[4 * c4 + 0] = ex2(pr[4 * c4 + 0] + l4.x);
            pr[4 * c4 + 1] = ex2(pr[4 * c4 + 1] + l4.y);
            pr[4 * c4 + 2] = ex2(pr[4 * c4 + 2] + l4.z);
            pr[4 * c4 + 3] = ex2(pr[4 * c4 + 3] + l4.w);
          }
        }
        if (any_mask) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int m = mbase + c;
            pr[c] = (m >= col_lo && m <= col_hi) ? pr[c] : 0.f;
          }
        }
        if (threadIdx.x == AB200_TRACE_TID) AB200_STAMP(G, 7);
        uint32_t keep = 0xffffffffu;
        if (p.dropout_on) {
          // One Philox counter serves four consecutive keys of one query row, and the four lanes of
          // a quad own exactly such keys (same n >> 2): lane q4 of the quad draws the counters of
          // query rows mbase + q4 + 4k (k = 0..7) for all four keys, then the quad exchanges them.
          const DropoutCtx dctx = dropout_ctx_from(p, ph_seed, ph_off, z, h);
          const int q4 = lane & 3;
          uint32_t mine = 0u;            // nibble k: keep bits of keys 4a..4a+3 for query row mbase + q4 + 4k
#pragma unroll
          for (int k = 0; k < 8; ++k)
            mine |= dropout_keep4_keys(dctx, pkeys, min(mbase + q4 + 4 * k, p.max_sq - 1), n >> 2) << (4 * k);
          keep = 0u;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t w = __shfl_sync(0xffffffffu, mine, (lane & ~3) | i);
            keep |= ((w >> q4) & 0x11111111u) << i;      // this lane's key, query rows mbase + i + 4k -> bit 4k + i
          }
        }
        if (threadIdx.x == AB200_TRACE_TID) AB200_STAMP(G, 1);
        if (!mbar_wait(&bars[L::bDpFull], par, abort_flag, status, 0x1900)) { ok = false; break; }
        if (threadIdx.x == AB200_TRACE_TID) AB200_STAMP(G, 2);
        tc_fence_after();
        {
          float dp[32];
          tmem_ld32f(tmem_base + lane_addr + kColDP + cbase, dp);
          tmem_wait_ld();
          if (threadIdx.x == AB200_TRACE_TID) AB200_STAMP(G, 10);
          // This thread has now read its 32 columns of dP: they can take P^T (packed, 16 columns)
          // followed by dS^T (packed, 16 columns).
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            float a = pr[2 * c], b = pr[2 * c + 1];
            if (p.dropout_on) {
              a = ((keep >> (2 * c)) & 1u) ? a * p.dropout_scale : 0.f;
              b = ((keep >> (2 * c + 1)) & 1u) ? b * p.dropout_scale : 0.f;
            }
            pk[c] = pack2<T>(a, b);
          }
          tmem_st16(tmem_base + lane_addr + kColDP + cbase, pk);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars[L::bPFull]);
          if (p.dropout_on) {
#pragma unroll
            for (int c = 0; c < 32; ++c) dp[c] = ((keep >> c) & 1u) ? dp[c] * p.dropout_scale : 0.f;
          }
#pragma unroll
          for (int c4 = 0; c4 < 8; ++c4) {
            const float4 d4 = lds128(dlt + 16u * c4);
            const float2 a = mul2(make_float2(pr[4 * c4], pr[4 * c4 + 1]),
                                  add2(make_float2(dp[4 * c4], dp[4 * c4 + 1]), make_float2(d4.x, d4.y)));
            const float2 b = mul2(make_float2(pr[4 * c4 + 2], pr[4 * c4 + 3]),
                                  add2(make_float2(dp[4 * c4 + 2], dp[4 * c4 + 3]), make_float2(d4.z, d4.w)));
            pk[2 * c4] = pack2<T>(a.x, a.y);
            pk[2 * c4 + 1] = pack2<T>(b.x, b.y);
          }
          tmem_st16(tmem_base + lane_addr + kColDP + cbase + 16, pk);
          if constexpr (FUSED) {
            if (i == 0 && live > 0 &&
                !mbar_wait(&bars[L::bStageFree], (live - 1) & 1u, abort_flag, status, 0x1E00)) { ok = false; break; }
            // dS^T of this key row, query columns cbase..cbase+31, into the shared-memory tile both dK
            // and dQ^T read: 64-column half wg >> 1, row r, four 16-byte chunks at (wg & 1) * 4,
            // swizzled like a TMA tile (chunk ^ (row & 7)); conflict-free across the warp's rows.
            uint8_t* row = smem + L::kStage + (wg >> 1) * 16384 + r * 128;
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<uint4*>(row + (((((wg & 1) << 2) + j) ^ (r & 7)) << 4)) =
                  make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
            fence_proxy_async_smem();
          }
        }
        if (threadIdx.x == AB200_TRACE_TID) AB200_STAMP(G, 11);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars[L::bDsFull]);
          mbar_arrive(&bars[L::bAuxEmpty + s]);
        }
        if (threadIdx.x == AB200_TRACE_TID) AB200_STAMP(G, 3);
        if constexpr (FUSED) {      // this iteration's dQ^T partial is taken out during the next one
          dq_dst = dq_acc + (((int64_t)sq.bidx * p.hq + h) * p.dq.n[2] + sq.q0 + mbase) * p.dqk + r;
          dq_rows = sq.sq - mbase;
        }
      }
      if (!ok) break;
      // ---- this item's dV and dK: wait for the last two GEMMs, read out, store ----
      if (!mbar_wait(&bars[L::bAccDone], live & 1u, abort_flag, status, 0x1A00)) { ok = false; break; }
      if (threadIdx.x == AB200_TRACE_TID) AB200_STAMP(G - 1, 13);
      ++live;
      if constexpr (FUSED) {
        // The item's last partial (it also is the last reader of the dS^T tile, which the write-out
        // below reuses as its staging tile).
        if (!mbar_wait(&bars[L::bDqFull], (G - 1) & 1u, abort_flag, status, 0x1D01)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          float dqv[8];
          tmem_ld8f(tmem_base + lane_addr + kColS + cbase + 8 * c8, dqv);
          tmem_wait_ld();
          dq_add8(dqv, c8);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[L::bDqRead]);
      }
      if (wg < HD / 32) {
        // Each warp transposes its 32 rows x 32 columns through the staging tile, so that the global
        // stores are 64-byte row segments instead of 16 bytes per row.
        uint8_t* stage = smem + L::kStage;
        const int nrows = min(kBlk, sq.sk - it.n0);
        const int d0 = wg * 32;
        float v[32];
        tc_fence_after();
        tmem_ld32f(tmem_base + lane_addr + kColAcc0 + d0, v);
        tmem_wait_ld();
        stage_put32<T>(stage, r, d0, v, 1.0f, HD * 2);
        __syncwarp();
        warp_copy_out<T, 4>(stage, reinterpret_cast<T*>(p.dv.ptr) + (int64_t)sq.bidx * p.dv.s[0] + (int64_t)hk * p.dv.s[1] +
                                       (sq.k0 + it.n0) * p.dv.s[2],
                            p.dv.s[2], nrows, p.dvo, quarter * 32, wg * 4, lane, HD * 2);
        tmem_ld32f(tmem_base + lane_addr + kColAcc1 + d0, v);
        tmem_wait_ld();
        // The accumulators are in registers now: the next item's first dV/dK GEMMs (which start from
        // zero) are only issued after this thread's next hand-off, i.e. after these loads.
        tc_fence_before();
        __syncwarp();
        stage_put32<T>(stage, r, d0, v, p.sm_scale, HD * 2);
        __syncwarp();
        warp_copy_out<T, 4>(stage, reinterpret_cast<T*>(p.dk.ptr) + (int64_t)sq.bidx * p.dk.s[0] + (int64_t)hk * p.dk.s[1] +
                                       (sq.k0 + it.n0) * p.dk.s[2],
                            p.dk.s[2], nrows, p.dqk, quarter * 32, wg * 4, lane, HD * 2);
        __syncwarp();
      }
      // The staging tile is the next item's dS^T tile: no compute warp may write dS^T there while
      // another one is still copying its rows out (waited for before the next item's first dS^T).
      if constexpr (FUSED) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[L::bStageFree]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Shared memory and barriers of the dQ kernel: Q and dO resident, K through a three-stage ring
// (a K block is read twice, by S_i early and by dQ_i late), V through a two-stage ring (read once,
// by dP_i, two iterations ahead of its use).
template <int HD>
struct DqSmem {
  static constexpr int kHalves = HD / 64;
  static constexpr int kTile = kHalves * 16384;          // 128 rows x HD x 2 bytes
  static constexpr int kKStages = 3, kVStages = 2;
  static constexpr int kResA = 0, kResB = kTile;
  static constexpr int kK = 2 * kTile, kV = kK + kKStages * kTile;
  static constexpr int kBars = kV + kVStages * kTile;
  static constexpr int bResFull = 0, bKFull = 1, bKEmpty = 4, bVFull = 7, bVEmpty = 9, bSFull = 11, bSRead = 12,
                       bDpFull = 13, bDsFull = 15, bAccDone = 17, bCount = 18;
  static constexpr int kTmemSlot = kBars + bCount * 8;
  static constexpr int kAbort = kTmemSlot + 4;
  static constexpr int kDynamic = kAbort + 8 + 1024;
};

// =========================================================================================
// dQ (+ dBias).  grid = (cdiv(max_sq, 128), Hq, batch)
template <typename T, int HD, bool EXACT>
__global__ void __launch_bounds__(kBwdThreads, 1)
sm100_bwd_dq_kernel(const __grid_constant__ Params p, const __grid_constant__ CUtensorMap tm_q,
                    const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                    const __grid_constant__ CUtensorMap tm_do, unsigned int* status) {
  using L = DqSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlot);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::kAbort);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Order of the CTAs (the hardware starts them by linear block index): (batch, head) pairs in groups
  // of kHeadGroup, inside a group the query-block index slowest, from the block with the most key
  // blocks of a causal problem to the one with the fewest.  The heavy blocks of a group start
  // together, the grid ends on light ones, and the CTAs in flight share the K/V of one group of
  // heads, which stays resident in L2.
#ifndef AB200_DQ_HEAD_GROUP
#define AB200_DQ_HEAD_GROUP 0    // measured: grouping does not pay here (+3 % on the dense causal benchmark)
#endif
  int z = blockIdx.z, h = blockIdx.y, m0 = (int)(gridDim.x - 1 - blockIdx.x) * kBlk;
  if constexpr (AB200_DQ_HEAD_GROUP > 0) {
    constexpr int kHeadGroup = AB200_DQ_HEAD_GROUP > 0 ? AB200_DQ_HEAD_GROUP : 1;
    const int nx = (int)gridDim.x, nh = (int)gridDim.y, nhz = nh * (int)gridDim.z;
    const int lin = (int)blockIdx.x + nx * ((int)blockIdx.y + nh * (int)blockIdx.z);
    const int grp = lin / (kHeadGroup * nx), rr = lin - grp * (kHeadGroup * nx);
    const int gsize = min(kHeadGroup, nhz - grp * kHeadGroup);
    const int xi = rr / gsize, hz = grp * kHeadGroup + (rr - xi * gsize);
    z = hz / nh;
    h = hz - z * nh;
    m0 = (nx - 1 - xi) * kBlk;
  }
  if (__syncthreads_or(threadIdx.x == 0 && *reinterpret_cast<volatile unsigned int*>(status) != 0u)) return;
  const Seq sq = resolve_seq(p, z);
  if (m0 >= sq.sq) return;
  const int hk = h / p.group;
  int n_lo, n_hi;
  key_range(p, sq, m0, min(m0 + kBlk, sq.sq) - 1, n_lo, n_hi);
  if (n_hi < n_lo) {
    zero_rows<T>(p.dq, sq.bidx, h, sq.q0, m0, sq.sq, p.dqk);
    zero_dbias_outside<T>(p, sq, h, m0, kBlk, 0, 0);
    return;
  }
  const int jb_lo = n_lo / kBlk;
  const int niter = n_hi / kBlk - jb_lo + 1;
  zero_dbias_outside<T>(p, sq, h, m0, kBlk, jb_lo * kBlk, (jb_lo + niter) * kBlk);

  if (threadIdx.x == 0) {
    init_abort_and_limit(abort_flag, p.wait_limit_kcycles);
    mbar_init(&bars[L::bResFull], 1);
    for (int s = 0; s < L::kKStages; ++s) { mbar_init(&bars[L::bKFull + s], 1); mbar_init(&bars[L::bKEmpty + s], 1); }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars[L::bVFull + s], 1);
      mbar_init(&bars[L::bVEmpty + s], 1);
      mbar_init(&bars[L::bDpFull + s], 1);
      mbar_init(&bars[L::bDsFull + s], kComputeWarps);
    }
    mbar_init(&bars[L::bSFull], 1);
    mbar_init(&bars[L::bSRead], kComputeWarps);
    mbar_init(&bars[L::bAccDone], 1);
    fence_barrier_init();
    // This thread is also the TMA producer: Q, dO and the first two K and V blocks (all ring stages
    // are free) are requested right away, before the CTA-wide synchronisation and the tensor-memory
    // allocation, which then overlap with the copies' latency.
    const int qrow = (int)(sq.q0 + m0);
    mbar_expect_tx(&bars[L::bResFull], 2 * L::kTile);
    for (int hf = 0; hf < L::kHalves; ++hf) {
      tma_load_4d(smem + L::kResA + hf * 16384, &tm_q, &bars[L::bResFull], hf * 64, qrow, h, sq.bidx);
      tma_load_4d(smem + L::kResB + hf * 16384, &tm_do, &bars[L::bResFull], hf * 64, qrow, h, sq.bidx);
    }
    for (int i = 0; i < min(2, niter); ++i) {
      const int krow = (int)(sq.k0 + (int64_t)(jb_lo + i) * kBlk);
      mbar_expect_tx(&bars[L::bKFull + i], L::kTile);
      for (int hf = 0; hf < L::kHalves; ++hf)
        tma_load_4d(smem + L::kK + i * L::kTile + hf * 16384, &tm_k, &bars[L::bKFull + i], hf * 64, krow, hk, sq.bidx);
      if (p.drop_copy == 3 && i == 0) continue;   // test hook: this block's V never arrives
      mbar_expect_tx(&bars[L::bVFull + i], L::kTile);
      for (int hf = 0; hf < L::kHalves; ++hf)
        tma_load_4d(smem + L::kV + i * L::kTile + hf * 16384, &tm_v, &bars[L::bVFull + i], hf * 64, krow, hk, sq.bidx);
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

  if (warp == 0) {
    if (lane == 0) {
      // (Q, dO and the first two K and V blocks were requested during set-up)
      int issued_k = min(2, niter), issued_v = min(2, niter);
      for (int i = min(2, niter); i < niter; ++i) {
        const int sv = i & 1, sk = i % L::kKStages;
        const int krow = (int)(sq.k0 + (int64_t)(jb_lo + i) * kBlk);
        if (!mbar_wait(&bars[L::bKEmpty + sk], ((uint32_t)(i / L::kKStages) & 1u) ^ 1u, abort_flag, status, 0x2180 + i)) break;
        mbar_expect_tx(&bars[L::bKFull + sk], L::kTile);
        for (int hf = 0; hf < L::kHalves; ++hf)
          tma_load_4d(smem + L::kK + sk * L::kTile + hf * 16384, &tm_k, &bars[L::bKFull + sk], hf * 64, krow, hk, sq.bidx);
        issued_k = i + 1;
        if (!mbar_wait(&bars[L::bVEmpty + sv], ((uint32_t)(i >> 1) & 1u) ^ 1u, abort_flag, status, 0x2100 + i)) break;
        mbar_expect_tx(&bars[L::bVFull + sv], L::kTile);
        for (int hf = 0; hf < L::kHalves; ++hf)
          tma_load_4d(smem + L::kV + sv * L::kTile + hf * 16384, &tm_v, &bars[L::bVFull + sv], hf * 64, krow, hk, sq.bidx);
        issued_v = i + 1;
      }
      if (*abort_flag) {
        mbar_wait_quiet(&bars[L::bResFull], 0, abort_flag);
        for (int i = max(0, issued_k - L::kKStages); i < issued_k; ++i)
          mbar_wait_quiet(&bars[L::bKFull + i % L::kKStages], (uint32_t)(i / L::kKStages) & 1u, abort_flag);
        for (int i = max(0, issued_v - 2); i < issued_v; ++i) {
          if (p.drop_copy == 3 && i == 0) continue;   // (never issued)
          mbar_wait_quiet(&bars[L::bVFull + (i & 1)], (uint32_t)(i >> 1) & 1u, abort_flag);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // The whole warp walks the loop and waits; one elected lane issues.  Keeping the control
    // flow warp-uniform lets the descriptors live in uniform registers, which makes the issue of
    // a GEMM several times cheaper in issue slots than a single-lane branch.
    constexpr uint32_t kIdescSS = instr_desc_f16(Fmt<T>::code, 128, 128, 0, 0);
    const uint32_t kIdescDQ = instr_desc_f16(Fmt<T>::code, 128, EXACT ? (uint32_t)HD : (uint32_t)((p.dqk + 15) & ~15), 0, 1);
    const int ksteps_qk = EXACT ? HD / 16 : (p.dqk + 15) >> 4, ksteps_vo = EXACT ? HD / 16 : (p.dvo + 15) >> 4;
    constexpr uint32_t kStageStep = L::kTile >> 4;
    const uint64_t q_km = kmajor_base(smem_u32(smem + L::kResA)), do_km = kmajor_base(smem_u32(smem + L::kResB));
    const uint64_t k_km = kmajor_base(smem_u32(smem + L::kK)), v_km = kmajor_base(smem_u32(smem + L::kV));
    const uint64_t k_mn = mnmajor_base(smem_u32(smem + L::kK));
    auto wait = [&](int bar, uint32_t parity, uint32_t where) {
      return __all_sync(0xffffffffu, mbar_wait(&bars[bar], parity, abort_flag, status, where)) != 0;
    };
    // Last, partial key block of the sequence: rows of K and V beyond its end must not reach the
    // dP and dQ products (a zero dS times a non-finite K row, or dO times a non-finite V row).
    auto zero_tail = [&](int base, int i, int stage) {
      if constexpr (!EXACT) {
        const int valid = sq.sk - (jb_lo + i) * kBlk;
        if (valid < kBlk) zero_tail_rows(smem + base + stage * L::kTile, valid, L::kHalves, lane);
      }
    };
    auto issue_s = [&](int i) {      // S = Q K_i^T
      zero_tail(L::kK, i, i % L::kKStages);
      if constexpr (!EXACT) tc_fence_after();
      const uint64_t ka = k_km + (uint64_t)((uint32_t)(i % L::kKStages) * kStageStep);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          if (kk < ksteps_qk)
            mma_ss(tmem_base + kColS, q_km + kmajor_step(kk), ka + kmajor_step(kk), kIdescSS, kk > 0 ? 1u : 0u);
        mma_commit(&bars[L::bSFull]);
      }
      __syncwarp();
    };
    auto issue_dp = [&](int i) {     // dP = dO V_i^T, into dP buffer i & 1; frees V's ring stage
      zero_tail(L::kV, i, i & 1);
      if constexpr (!EXACT) tc_fence_after();
      const uint64_t va = v_km + (uint64_t)((uint32_t)(i & 1) * kStageStep);
      const uint32_t d = tmem_base + kColDP + (uint32_t)(i & 1) * 128u;
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          if (kk < ksteps_vo)
            mma_ss(d, do_km + kmajor_step(kk), va + kmajor_step(kk), kIdescSS, kk > 0 ? 1u : 0u);
        mma_commit(&bars[L::bDpFull + (i & 1)]);
        mma_commit(&bars[L::bVEmpty + (i & 1)]);
      }
      __syncwarp();
    };
    // Order on the tensor pipe: ... dQ_i, S_{i+2}, dP_{i+2}, dQ_{i+1}, ...  S_{i+2} only needs the
    // compute warps to have copied S_{i+1} out (early in their iteration i+1) and K_{i+2}, which the
    // third ring stage has brought in already; dP runs two iterations ahead in its two buffers.  In
    // steady state neither the compute warps nor the pipe wait for the issuing warp.
    bool ok = wait(L::bResFull, 0, 0x2200) && wait(L::bKFull + 0, 0, 0x2201);
    if (ok) {
      tc_fence_after();
      issue_s(0);
      ok = wait(L::bVFull + 0, 0, 0x2202);
    }
    if (ok) {
      tc_fence_after();
      issue_dp(0);
    }
    if (ok && niter > 1) {
      ok = wait(L::bVFull + 1, 0, 0x2203);
      if (ok) {
        tc_fence_after();
        issue_dp(1);
        ok = wait(L::bSRead, 0, 0x2300) && wait(L::bKFull + 1, 0, 0x2400);
      }
      if (ok) {
        tc_fence_after();
        issue_s(1);
      }
    }
    for (int i = 0; ok && i < niter; ++i) {
      const int s = i & 1;
      // (a compute warp may be a whole iteration ahead of another one, since dP_{i+1} is already
      // there: the hand-off barrier alternates with the dP buffer)
      if (!wait(L::bDsFull + s, (uint32_t)(i >> 1) & 1u, 0x2500 + i)) break;
      if (lane == 0) AB200_STAMPQ(i, 5);
      tc_fence_after();
      {   // dQ += dS K_i
        const uint64_t ka = k_mn + (uint64_t)((uint32_t)(i % L::kKStages) * kStageStep);
        const uint32_t first = (i > 0) ? 1u : 0u;
        const uint32_t ds_col = tmem_base + kColDP + (uint32_t)s * 128u;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            mma_ts(tmem_base + kColAcc1, ds_col + split_a_col(kk), ka + mnmajor_step(kk), kIdescDQ,
                   kk > 0 ? 1u : first);
          mma_commit(&bars[L::bKEmpty + i % L::kKStages]);
        }
        __syncwarp();
      }
      if (i + 2 < niter) {
        // S_{i+1} has been copied to registers by every compute thread: its buffer is free.
        if (!wait(L::bSRead, (uint32_t)(i + 1) & 1u, 0x2300 + i + 1)) break;
        if (!wait(L::bKFull + (i + 2) % L::kKStages, (uint32_t)((i + 2) / L::kKStages) & 1u, 0x2400 + i + 2)) break;
        tc_fence_after();
        issue_s(i + 2);
        if (lane == 0) AB200_STAMPQ(i + 2, 8);
        // dP_{i+2} takes the buffer dQ_i has just read (the pipe runs in issue order)
        if (!wait(L::bVFull + s, (uint32_t)((i + 2) >> 1) & 1u, 0x2580 + i)) break;
        tc_fence_after();
        issue_dp(i + 2);
      }
      if (lane == 0) AB200_STAMPQ(i, 9);
    }
    if (elect_one()) mma_commit(&bars[L::bAccDone]);
    __syncwarp();
  } else if (warp >= 4) {
    const int quarter = warp & 3, wg = (warp - 4) >> 2;
    const int r = quarter * 32 + lane;
    const int m = m0 + r;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int cbase = kWgCols * wg;
    int row_lo = 0, row_hi = sq.sk - 1;     // valid keys for this query row
    if (p.causal) {
      int64_t lo = (int64_t)m - sq.wl, hi = (int64_t)m + sq.wr;
      if (lo > row_lo) row_lo = (int)(lo > 0x7fffffffLL ? 0x7fffffffLL : lo);
      if (hi < row_hi) row_hi = (int)(hi < -1 ? -1 : hi);
    }
    if (m >= sq.sq) { row_lo = 1; row_hi = 0; }
    // the tightest bounds over the warp's rows: a block needs masking iff it is not inside them
    const int warp_lo = __reduce_max_sync(0xffffffffu, row_lo), warp_hi = __reduce_min_sync(0xffffffffu, row_hi);
    const int64_t lrow = lse_offset(p, sq, h);
    const float lse2 = (m < sq.sq) ? p.lse[lrow + m] * kLog2e : INFINITY;
    const float dlt = (m < sq.sq) ? p.delta[lrow + m] : 0.f;
    // one packed FMA per two elements unless bias is present or the logsumexp is so large that
    // product rounding matters (then: scale first, subtract second, like the forward)
    const bool simple = !p.has_bias && !__any_sync(0xffffffffu, fabsf(lse2) > 1.0e6f && lse2 != INFINITY);
    DropoutCtx dctx;
    if (p.dropout_on) dctx = dropout_ctx(p, z, h);
    PhiloxKeys pkeys;      // Philox round keys: they depend on the seed only
    if (p.dropout_on) pkeys = philox_keys(dctx.seed);
    const int mm = min(m, sq.sq - 1);
    const T* bias_row = p.has_bias ? reinterpret_cast<const T*>(p.bias.ptr) + (int64_t)sq.bidx * p.bias.s[0] +
                                         (int64_t)h * p.bias.s[1] + (int64_t)mm * p.bias.s[2]
                                   : nullptr;
    T* db_row = p.has_dbias ? reinterpret_cast<T*>(p.dbias.ptr) + (int64_t)sq.bidx * p.dbias.s[0] +
                                  (int64_t)h * p.dbias.s[1] + (int64_t)mm * p.dbias.s[2]
                            : nullptr;
    bool ok = true;
    for (int i = 0; i < niter; ++i) {
      const uint32_t par = (uint32_t)i & 1u;
      const int nbase = (jb_lo + i) * kBlk + cbase;     // first key of this thread's columns
      if (threadIdx.x == AB200_TRACE_TID) AB200_STAMPQ(i, 4);
      // (the thread's 64 bytes of bias for this block: on their way to L2 while the tensor pipe computes S)
      if (p.has_bias && p.bias_vec) asm volatile("prefetch.global.L2 [%0];" ::"l"(bias_row + nbase));
      if (!mbar_wait(&bars[L::bSFull], par, abort_flag, status, 0x2600 + i)) { ok = false; break; }
      if (threadIdx.x == AB200_TRACE_TID) AB200_STAMPQ(i, 0);
      tc_fence_after();
      float pr[32];
      tmem_ld32f(tmem_base + lane_addr + kColS + cbase, pr);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[L::bSRead]);
      if (threadIdx.x == AB200_TRACE_TID) AB200_STAMPQ(i, 6);
      // (warp-uniform without a vote per block: compared with the warp's extreme bounds)
      const bool any_mask = !(nbase >= warp_lo && nbase + kWgCols - 1 <= warp_hi);
      if (simple) {
        const float2 sc2 = make_float2(p.qk_scale, p.qk_scale), nl2 = make_float2(-lse2, -lse2);
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const float2 a = fma2(make_float2(pr[c], pr[c + 1]), sc2, nl2);
          pr[c] = ex2(a.x);
          pr[c + 1] = ex2(a.y);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) pr[c] *= p.qk_scale;
        if (p.has_bias) {
          if (p.bias_vec && nbase + kWgCols <= sq.sk) {
            // the thread's 32 bias values are 64 contiguous bytes: four 16-byte loads
            const uint4* bp = reinterpret_cast<const uint4*>(bias_row + nbase);
            uint4 w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) w[u] = __ldg(bp + u);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const T* e = reinterpret_cast<const T*>(&w[u]);
#pragma unroll
              for (int i = 0; i < 8; ++i) pr[u * 8 + i] = fmaf(to_f32<T>(e[i]), kLog2e, pr[u * 8 + i]);
            }
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const int n = nbase + c;
              if (n < sq.sk) pr[c] = fmaf(to_f32<T>(bias_row[(int64_t)n * p.bias.s[3]]), kLog2e, pr[c]);
            }
          }
        }
#pragma unroll
        for (int c = 0; c < 32; ++c) pr[c] = ex2(pr[c] - lse2);
      }
      if (any_mask) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int n = nbase + c;
          pr[c] = (n >= row_lo && n <= row_hi) ? pr[c] : 0.f;
        }
      }
      uint32_t keep = 0xffffffffu;
      if (p.dropout_on) {
        keep = 0u;
        const int md = min(m, p.max_sq - 1);
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) keep |= dropout_keep4_keys(dctx, pkeys, md, (nbase >> 2) + c4) << (4 * c4);
      }
      const uint32_t dp_col = tmem_base + lane_addr + kColDP + (uint32_t)(i & 1) * 128u + cbase;
      if (threadIdx.x == AB200_TRACE_TID) AB200_STAMPQ(i, 7);
      if (!mbar_wait(&bars[L::bDpFull + (i & 1)], (uint32_t)(i >> 1) & 1u, abort_flag, status, 0x2700 + i)) { ok = false; break; }
      if (threadIdx.x == AB200_TRACE_TID) AB200_STAMPQ(i, 2);
      tc_fence_after();
      {
        float dp[32];
        tmem_ld32f(dp_col, dp);
        tmem_wait_ld();
        if (threadIdx.x == AB200_TRACE_TID) AB200_STAMPQ(i, 10);
        if (p.dropout_on) {
#pragma unroll
          for (int c = 0; c < 32; ++c) dp[c] = ((keep >> c) & 1u) ? dp[c] * p.dropout_scale : 0.f;
        }
        uint32_t pk[16];
        const float2 dl2 = make_float2(dlt, dlt);
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const float2 a = mul2(make_float2(pr[2 * c], pr[2 * c + 1]), sub2(make_float2(dp[2 * c], dp[2 * c + 1]), dl2));
          pk[c] = pack2<T>(a.x, a.y);
        }
        tmem_st16(dp_col, pk);
        if (p.has_dbias && m < sq.sq) {
          // dB = cast(dS): the packed pairs are exactly the values to store
          if (p.dbias.s[3] == 1 && nbase + 32 <= sq.sk && (reinterpret_cast<uintptr_t>(db_row + nbase) & 15u) == 0) {
#pragma unroll
            for (int v4 = 0; v4 < 4; ++v4)
              *reinterpret_cast<uint4*>(db_row + nbase + v4 * 8) =
                  make_uint4(pk[v4 * 4], pk[v4 * 4 + 1], pk[v4 * 4 + 2], pk[v4 * 4 + 3]);
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const int n = nbase + c;
              if (n < sq.sk) {
                const uint16_t bits = (uint16_t)((pk[c >> 1] >> ((c & 1) * 16)) & 0xffffu);
                reinterpret_cast<uint16_t*>(db_row)[(int64_t)n * p.dbias.s[3]] = bits;
              }
            }
          }
        }
      }
      __syncwarp();   // the dB stores diverge; TMEM instructions are warp-collective
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[L::bDsFull + (i & 1)]);
      if (threadIdx.x == AB200_TRACE_TID) AB200_STAMPQ(i, 3);
    }
    if (ok) ok = mbar_wait(&bars[L::bAccDone], 0, abort_flag, status, 0x2800);
    if (ok && wg < HD / 32) {
      // Each warp transposes its 32 rows x 32 columns of dQ through the (now idle) Q tile, so that
      // the global stores are 64-byte row segments instead of 16 bytes per row.
      uint8_t* stage = smem + L::kResA;
      tc_fence_after();
      float v[32];
      const int d0 = wg * 32;
      tmem_ld32f(tmem_base + lane_addr + kColAcc1 + d0, v);
      tmem_wait_ld();
      stage_put32<T>(stage, r, d0, v, p.sm_scale, HD * 2);
      __syncwarp();
      warp_copy_out<T, 4>(stage, reinterpret_cast<T*>(p.dq.ptr) + (int64_t)sq.bidx * p.dq.s[0] + (int64_t)h * p.dq.s[1] +
                                     (sq.q0 + m0) * p.dq.s[2],
                          p.dq.s[2], min(kBlk, sq.sq - m0), p.dqk, quarter * 32, wg * 4, lane, HD * 2);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// which: 1 dK/dV, 2 dQ(+dBias), 3 dK/dV fused with dQ accumulation into `dq_acc` (HD == 128 only)
template <typename T, int HD>
cudaError_t launch_bwd_T(int which, const Params& p, cudaStream_t st, float* dq_acc) {
  using L = BwdSmem<HD>;
  CUtensorMap tq, tk, tv, tdo;
  if (!make_tile_map_16bit(&tq, p.q, p.dqk, p.q.n[2], kBlk) || !make_tile_map_16bit(&tk, p.k, p.dqk, p.k.n[2], kBlk) ||
      !make_tile_map_16bit(&tv, p.v, p.dvo, p.v.n[2], kBlk) ||
      !make_tile_map_16bit(&tdo, p.dout, p.dvo, p.dout.n[2], kBlk))
    return cudaErrorInvalidValue;
  // Per-device facts (addresses of the status word and the ticket pool, SM count, the shared-memory
  // attribute of each kernel) are looked up once for the current device, which the entry points
  // make the stream's device, and remembered.
  struct PerDevice { std::atomic<unsigned int*> status{nullptr}, tickets{nullptr}; std::atomic<int> sms{0}; };
  static PerDevice per_device[64];
  static std::atomic<bool> attr_set[64][5];
  const bool exact = p.varlen_mode == 0 && p.max_sq % 128 == 0 && p.max_sk % 128 == 0 && p.dqk == HD && p.dvo == HD;
  int dev = 0;
  cudaError_t e = host().get_device(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  // (a pretended device, used by host-side tests, gets a scratch record that is never reused)
  PerDevice scratch;
  const bool pretend = host_pretends();
  PerDevice& pd = pretend ? scratch : per_device[dev];
  unsigned int* status = pd.status.load(std::memory_order_acquire);
  if (status == nullptr) {
    if ((e = host().symbol_address(reinterpret_cast<void**>(&status), reinterpret_cast<const void*>(&g_sm100_bwd_status))) != cudaSuccess) return e;
    pd.status.store(status, std::memory_order_release);
  }
  auto set_smem = [&](int slot, const void* fn, int bytes) -> cudaError_t {
    if (!pretend && attr_set[dev][slot].load(std::memory_order_acquire)) return cudaSuccess;
    cudaError_t r = host().func_set_smem(fn, bytes);
    if (r == cudaSuccess && !pretend) attr_set[dev][slot].store(true, std::memory_order_release);
    return r;
  };
  if (which == 1 || which == 3) {
    const bool fused = which == 3;
    if (fused && HD != 128) return cudaErrorInvalidValue;
    auto kern_split = exact ? sm100_bwd_dkdv_kernel<T, HD, false, true> : sm100_bwd_dkdv_kernel<T, HD, false, false>;
    auto kern_fused = sm100_bwd_dkdv_kernel<T, 128, true, false>;
    e = fused ? set_smem(2, reinterpret_cast<const void*>(kern_fused), BwdSmem<128>::kDynamic)
              : set_smem(exact ? 3 : 0, reinterpret_cast<const void*>(kern_split), L::kDynamic);
    if (e != cudaSuccess) return e;
    const int nitems = ((p.max_sk + kBlk - 1) / kBlk) * ((p.hk * p.batch + 7) / 8) * 8;
    int sms = pd.sms.load(std::memory_order_acquire);
    if (sms == 0) {
      if ((e = host().device_attr(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
      pd.sms.store(sms, std::memory_order_release);
    }
    dim3 grid(nitems < sms ? nitems : sms, 1, 1);     // persistent: one CTA per SM
    // ticket counter of this launch: one of a small pool, zeroed in stream order
    static std::atomic<unsigned int> launch_seq{0};
    unsigned int* tickets = pd.tickets.load(std::memory_order_acquire);
    if (tickets == nullptr) {
      if ((e = host().symbol_address(reinterpret_cast<void**>(&tickets), reinterpret_cast<const void*>(&g_dkdv_ticket))) != cudaSuccess) return e;
      pd.tickets.store(tickets, std::memory_order_release);
    }
    unsigned int* ticket = tickets + (launch_seq.fetch_add(1) % kTicketPool);
    if ((e = host().memset_async(ticket, 0, sizeof(unsigned int), st)) != cudaSuccess) return e;
    if (fused)
      e = launch_kernel(kern_fused, grid, dim3(kFusedThreads), BwdSmem<128>::kDynamic, st, p, tq, tk, tv, tdo, status, nitems,
                        ticket, dq_acc);
    else
      e = launch_kernel(kern_split, grid, dim3(kBwdThreads), L::kDynamic, st, p, tq, tk, tv, tdo, status, nitems, ticket,
                        static_cast<float*>(nullptr));
  } else {
    auto kern_dq = exact ? sm100_bwd_dq_kernel<T, HD, true> : sm100_bwd_dq_kernel<T, HD, false>;
    e = set_smem(exact ? 4 : 1, reinterpret_cast<const void*>(kern_dq), DqSmem<HD>::kDynamic);
    if (e != cudaSuccess) return e;
    dim3 grid((p.max_sq + kBlk - 1) / kBlk, p.hq, p.batch);
    e = launch_kernel(kern_dq, grid, dim3(kBwdThreads), DqSmem<HD>::kDynamic, st, p, tq, tk, tv, tdo, status);
  }
  if (e == cudaSuccess) count_launch();
  return e;
}

#include "sm100_bwd_wide.cuh"

cudaError_t launch_bwd(int which, int dtype, const Params& p, cudaStream_t st, float* dq_acc) {
  if (p.dqk > 128 || p.dvo > 128) {      // wide heads: one launch per gradient (sm100_bwd_wide.cuh)
    if (which == 3) return cudaErrorInvalidValue;
    return dtype == 2 ? launch_bwd_wide_T<__half>(which, p, st) : launch_bwd_wide_T<__nv_bfloat16>(which, p, st);
  }
  const bool small = p.dqk <= 64 && p.dvo <= 64 && which != 3;
  if (dtype == 2)
    return small ? launch_bwd_T<__half, 64>(which, p, st, dq_acc) : launch_bwd_T<__half, 128>(which, p, st, dq_acc);
  return small ? launch_bwd_T<__nv_bfloat16, 64>(which, p, st, dq_acc)
               : launch_bwd_T<__nv_bfloat16, 128>(which, p, st, dq_acc);
}

}  // namespace

bool sm100_bwd_supported(int dtype, const Params& p) {
  if (dtype != 2 && dtype != 3) return false;
  if (p.dqk > 256 || p.dvo > 256 || p.dqk % 8 != 0 || p.dvo % 8 != 0) return false;
  if (p.max_sq <= 0 || p.max_sk <= 0 || p.batch <= 0) return false;
  if (!tma_friendly(p.q) || !tma_friendly(p.k) || !tma_friendly(p.v) || !tma_friendly(p.dout)) return false;
  if (p.q.n[3] != p.dqk || p.k.n[3] != p.dqk || p.v.n[3] != p.dvo || p.dout.n[3] != p.dvo) return false;
  // gradients are written with 16-byte vector stores (absent ones are not written at all)
  if (p.dq.ptr && !vector_store_friendly(p.dq)) return false;
  if (p.dk.ptr && !vector_store_friendly(p.dk)) return false;
  if (p.dv.ptr && !vector_store_friendly(p.dv)) return false;
  return host().have_encoder();
}

cudaError_t launch_sm100_bwd_dkdv(int dtype, const Params& p, cudaStream_t st) { return launch_bwd(1, dtype, p, st, nullptr); }
cudaError_t launch_sm100_bwd_dq(int dtype, const Params& p, cudaStream_t st) { return launch_bwd(2, dtype, p, st, nullptr); }

// The fused form needs the accumulator's layout to follow dQ's logical shape, 128-wide tiles, and
// no dBias (which the dQ kernel produces).
bool sm100_bwd_fused_supported(int dtype, const Params& p) {
  if (!sm100_bwd_supported(dtype, p)) return false;
  if (p.has_dbias) return false;
  if (p.dqk > 128 || p.dvo > 128) return false;      // neither have the kernels for wide heads
  if (p.dqk <= 64 && p.dvo <= 64) return false;      // the 64-wide instantiation has no fused form
  return p.dq.ptr != nullptr;
}
cudaError_t launch_sm100_bwd_fused(int dtype, const Params& p, float* dq_acc, cudaStream_t st) {
  return launch_bwd(3, dtype, p, st, dq_acc);
}

#ifdef AB200_TRACE
extern "C" __attribute__((visibility("default"))) int ab200_debug_read_trace(long long* out, int n) {
  return (int)cudaMemcpyFromSymbol(out, g_bwd_trace, sizeof(long long) * (size_t)(n < 4096 ? n : 4096));
}
#endif

unsigned int sm100_bwd_status(bool reset) {
  unsigned int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_sm100_bwd_status, sizeof(v)) != cudaSuccess) { (void)cudaGetLastError(); return 0xffffffffu; }
  if (reset && v != 0) {
    unsigned int zero = 0;
    if (cudaMemcpyToSymbol(g_sm100_bwd_status, &zero, sizeof(zero)) != cudaSuccess) (void)cudaGetLastError();
  }
  return v;
}

}  // namespace ab200
