// Backward attention on tcgen05 for head dimensions above 128 (up to 256).
// Included by sm100_bwd.cu inside its namespaces; it uses that file's descriptor helpers, status
// word and write-out helpers.
//
// With 256-wide heads the scheme of the 128-wide kernels does not fit an SM: four 128 x 256 16-bit
// tiles are 256 KB of shared memory, and two 128 x 256 fp32 accumulators fill tensor memory.  So
// each gradient gets a launch of its own with ONE 256-column accumulator, and the other sequence
// dimension is streamed in blocks of 64 rows.  One kernel serves all three; a CTA owns 128 rows
// (keys for dV and dK, queries for dQ) of one head:
//
//   mode   resident (128 rows)   streamed (64 rows)      per streamed block i
//   dV     K                     Q (early), dO (late)    S' = K Q_i^T;                 dV += P'^T-tile dO_i
//   dK     K, V                  dO (early), Q (late)    S' = K Q_i^T, dP' = V dO_i^T; dK += dS' Q_i
//   dQ     Q, dO                 V (early), K (late)     S' = Q K_i^T, dP' = dO V_i^T; dQ += dS' K_i
//
// "early" tiles feed only the first GEMMs of a block and live in one stage (two for dV, in the place
// of the second resident tile); "late" tiles also feed the accumulating GEMM at the block's end and
// live in two stages, so the dP' / S' GEMMs of block i+1 run while the compute warps work on block i.
// Shared memory: 2 x 64 KB resident, 2 x 32 KB late, 32 KB early.  Tensor memory: [0,64) S', [64,128) and [128,192) two dP' buffers, whose first columns
// then take the packed 16-bit P' / dS' (the A operand of the accumulating GEMM), [256,512) the
// accumulator.  Twelve warps: TMA producer, MMA issuer, logsumexp/delta stager (dV, dK), one idle,
// eight compute warps (thread = one row of the 128 x 64 score tile, two warpgroups split its columns
// 32 apiece).  The arithmetic is that of the 128-wide kernels (see the head of sm100_bwd.cu); dK and dV
// recompute the probabilities separately, which is the price of the one-accumulator form.
// Every wait is bounded.

constexpr int kWideThreads = 384;
constexpr int kWideCompute = 8;        // warps 4..11
constexpr int kNB = 64;                // rows of a streamed block
constexpr uint32_t kWColS = 0, kWColDP = 64, kWColAcc = 256;
constexpr int kWideDV = 0, kWideDK = 1, kWideDQ = 2;

struct WideSmem {
  static constexpr int kBoxes = 4;                       // 64-column boxes per 256-wide tile
  static constexpr int kResBox = 16384, kStrBox = 8192;  // 128 / 64 rows x 64 columns x 2 bytes
  static constexpr int kRes = kBoxes * kResBox, kStr = kBoxes * kStrBox;
  static constexpr int kResA = 0, kResB = kRes;
  static constexpr int kLate = 2 * kRes;                 // two stages
  static constexpr int kEarly = kLate + 2 * kStr;        // one stage
  static constexpr int kAux = kEarly + kStr;             // 2 stages x (64 lse2 + 64 delta) floats
  static constexpr int kAuxFlag = kAux + 2 * 2 * kNB * 4;
  static constexpr int kBars = kAuxFlag + 16;
  static constexpr int bResFull = 0, bLateFull = 1, bLateEmpty = 3, bEarlyFull = 5, bEarlyEmpty = 7, bSFull = 9,
                       bSRead = 10, bDpFull = 11, bDsFull = 13, bAccDone = 15, bAuxFull = 16, bAuxEmpty = 18, bCount = 20;
  static constexpr int kTmemSlot = kBars + bCount * 8;
  static constexpr int kAbort = kTmemSlot + 8;
  static constexpr int kUsed = kAbort + 8;
  static constexpr int kDynamic = kUsed + 512;
};
static_assert(WideSmem::kDynamic <= 232448, "shared memory of the wide backward kernel");
static_assert(WideSmem::kBars % 8 == 0, "barrier alignment");

// zero_tail_rows (sm100_ptx.cuh) for a streamed tile: rows [valid_rows, 64) of its four boxes.
static __device__ __noinline__ void zero_tail_rows_streamed(uint8_t* tile, int valid_rows, int lane) {
  const uint4 z = make_uint4(0u, 0u, 0u, 0u);
  if (valid_rows < 0) valid_rows = 0;
  for (int b = 0; b < WideSmem::kBoxes; ++b)
    for (int o = valid_rows * 128 + lane * 16; o < WideSmem::kStrBox; o += 512)
      *reinterpret_cast<uint4*>(tile + b * WideSmem::kStrBox + o) = z;
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
}

// grid = (cdiv(rows, 128), heads, batch): rows/heads are keys/kv heads (dV, dK) or queries/q heads (dQ)
template <typename T, int MODE>
__global__ void __launch_bounds__(kWideThreads, 1)
sm100_bwd_wide_kernel(const __grid_constant__ Params p, const __grid_constant__ CUtensorMap tm_r1,
                      const __grid_constant__ CUtensorMap tm_r2, const __grid_constant__ CUtensorMap tm_late,
                      const __grid_constant__ CUtensorMap tm_early, unsigned int* status) {
  using L = WideSmem;
  constexpr bool kKeys = MODE != kWideDQ;      // the CTA's rows are keys
  constexpr bool kHasDp = MODE != kWideDV;
  // The early tile has one stage; dV, which keeps only K resident, gives it two in the second
  // resident tile's place.
  constexpr int kEarlyStages = MODE == kWideDV ? 2 : 1;
  constexpr int kEarlyBase = MODE == kWideDV ? WideSmem::kResB : WideSmem::kEarly;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kTmemSlot);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::kAbort);
  float* aux = reinterpret_cast<float*>(smem + L::kAux);
  const uint32_t aux_s = smem_u32(smem + L::kAux);
  volatile uint32_t* aux_flag = reinterpret_cast<volatile uint32_t*>(smem + L::kAuxFlag);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (__syncthreads_or(threadIdx.x == 0 && *reinterpret_cast<volatile unsigned int*>(status) != 0u)) return;
  if ((int)(smem - smem_raw) + L::kUsed > L::kDynamic) {      // the alignment padding did not fit
    if (threadIdx.x == 0) atomicCAS(status, 0u, 0x3F00u);
    return;
  }
  // dV / dK: the first key blocks of a causal problem see the most queries; dQ: the last query blocks
  // see the most keys.  Heavy CTAs start first.
  const int z = blockIdx.z, hrow = blockIdx.y;
  const int r0 = (kKeys ? (int)blockIdx.x : (int)(gridDim.x - 1 - blockIdx.x)) * kBlk;
  const Seq sq = resolve_seq(p, z);
  const int rows_total = kKeys ? sq.sk : sq.sq, cols_total = kKeys ? sq.sq : sq.sk;
  if (r0 >= rows_total) return;
  int c_lo, c_hi;
  if constexpr (kKeys) query_range(p, sq, r0, min(r0 + kBlk, sq.sk) - 1, c_lo, c_hi);
  else key_range(p, sq, r0, min(r0 + kBlk, sq.sq) - 1, c_lo, c_hi);
  const View4& outv = MODE == kWideDV ? p.dv : (MODE == kWideDK ? p.dk : p.dq);
  const int d_out = MODE == kWideDV ? p.dvo : p.dqk;
  const int64_t row_tok0 = kKeys ? sq.k0 : sq.q0, col_tok0 = kKeys ? sq.q0 : sq.k0;
  if (c_hi < c_lo) {      // rows nothing attends to / that attend to nothing: the gradient is zero
    zero_rows<T>(outv, sq.bidx, hrow, row_tok0, r0, rows_total, d_out);
    if constexpr (MODE == kWideDQ) zero_dbias_outside<T>(p, sq, hrow, r0, kBlk, 0, 0);
    return;
  }
  const int cb_lo = c_lo / kNB;
  const int ncb = c_hi / kNB - cb_lo + 1;
  if constexpr (MODE == kWideDQ) zero_dbias_outside<T>(p, sq, hrow, r0, kBlk, cb_lo * kNB, (cb_lo + ncb) * kNB);
  const int niter = kKeys ? ncb * p.group : ncb;      // dV / dK walk the q heads of the kv head's group
  const int hk = kKeys ? hrow : hrow / p.group;

  if (threadIdx.x == 0) {
    init_abort_and_limit(abort_flag, p.wait_limit_kcycles);
    mbar_init(&bars[L::bResFull], 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars[L::bLateFull + s], 1);
      mbar_init(&bars[L::bLateEmpty + s], 1);
      mbar_init(&bars[L::bDpFull + s], 1);
      mbar_init(&bars[L::bDsFull + s], kWideCompute);
      mbar_init(&bars[L::bAuxFull + s], 1);
      mbar_init(&bars[L::bAuxEmpty + s], kWideCompute);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars[L::bEarlyFull + s], 1);
      mbar_init(&bars[L::bEarlyEmpty + s], 1);
    }
    mbar_init(&bars[L::bSFull], 1);
    mbar_init(&bars[L::bSRead], kWideCompute);
    mbar_init(&bars[L::bAccDone], 1);
    fence_barrier_init();
    prefetch_tmap(&tm_r1); prefetch_tmap(&tm_r2); prefetch_tmap(&tm_late); prefetch_tmap(&tm_early);
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
      const int rrow = (int)(row_tok0 + r0);
      mbar_expect_tx(&bars[L::bResFull], (kHasDp ? 2 : 1) * L::kRes);
      for (int b = 0; b < L::kBoxes; ++b) {
        tma_load_4d(smem + L::kResA + b * L::kResBox, &tm_r1, &bars[L::bResFull], b * 64, rrow, hrow, sq.bidx);
        if constexpr (kHasDp)
          tma_load_4d(smem + L::kResB + b * L::kResBox, &tm_r2, &bars[L::bResFull], b * 64, rrow, hrow, sq.bidx);
      }
      // test hook of the bounded waits: the first early tile never arrives
      const bool drop_first = kKeys ? p.drop_copy == 2 : p.drop_copy == 3;
      int issued_l = 0, issued_e = 0;
      for (int i = 0, hg = 0, cb = 0; i < niter; ++i) {      // hg, cb: i / ncb, i % ncb
        const int s = i & 1;
        const int hs = kKeys ? hk * p.group + hg : hk;
        const int srow = (int)(col_tok0 + (int64_t)(cb_lo + cb) * kNB);
        if (++cb == ncb) { cb = 0; ++hg; }
        // the early tile first: it is what the block's first GEMM waits for
        const int es = i % kEarlyStages;
        if (!mbar_wait(&bars[L::bEarlyEmpty + es], ((uint32_t)(i / kEarlyStages) & 1u) ^ 1u, abort_flag, status, 0x3100)) break;
        if (!(drop_first && i == 0)) {
          mbar_expect_tx(&bars[L::bEarlyFull + es], L::kStr);
          for (int b = 0; b < L::kBoxes; ++b)
            tma_load_4d(smem + kEarlyBase + es * L::kStr + b * L::kStrBox, &tm_early, &bars[L::bEarlyFull + es], b * 64, srow,
                        hs, sq.bidx);
          issued_e = i + 1;
        }
        if (!mbar_wait(&bars[L::bLateEmpty + s], ((uint32_t)(i >> 1) & 1u) ^ 1u, abort_flag, status, 0x3000)) break;
        mbar_expect_tx(&bars[L::bLateFull + s], L::kStr);
        for (int b = 0; b < L::kBoxes; ++b)
          tma_load_4d(smem + L::kLate + s * L::kStr + b * L::kStrBox, &tm_late, &bars[L::bLateFull + s], b * 64, srow, hs,
                      sq.bidx);
        issued_l = i + 1;
        if constexpr (MODE == kWideDQ) {
          // the next block's K and V towards L2 (their slots free up a block from now; measured: dQ 6 %
          // faster, while for dV and dK, whose streamed Q and dO are shared by fewer CTAs, it did not pay)
          if (i + 1 < niter) {
            const int nrow = (int)(col_tok0 + (int64_t)(cb_lo + cb) * kNB);
            for (int b = 0; b < L::kBoxes; ++b) {
              tma_prefetch_4d(&tm_late, b * 64, nrow, hk, sq.bidx);
              tma_prefetch_4d(&tm_early, b * 64, nrow, hk, sq.bidx);
            }
          }
        }
      }
      if (*abort_flag) {
        // Let copies that are still in flight land before the CTA gives its shared memory back.
        mbar_wait_quiet(&bars[L::bResFull], 0, abort_flag);
        for (int i = max(0, issued_l - 2); i < issued_l; ++i)
          mbar_wait_quiet(&bars[L::bLateFull + (i & 1)], (uint32_t)(i >> 1) & 1u, abort_flag);
        for (int i = max(drop_first ? 1 : 0, issued_e - kEarlyStages); i < issued_e; ++i)
          mbar_wait_quiet(&bars[L::bEarlyFull + i % kEarlyStages], (uint32_t)(i / kEarlyStages) & 1u, abort_flag);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================================= MMA issuer ====================================
    // Contractions over a head dimension run over it rounded up to 16, the accumulating GEMM
    // produces it rounded up to 16 (the copies zero-fill up to the 64-column box).
    constexpr uint32_t kIdescS = instr_desc_f16(Fmt<T>::code, 128, kNB, 0, 0);
    const uint32_t idesc_acc = instr_desc_f16(Fmt<T>::code, 128, (uint32_t)((d_out + 15) & ~15), 0, 1);
    const int ksteps_qk = (p.dqk + 15) >> 4, ksteps_vo = (p.dvo + 15) >> 4;
    const uint64_t r1_km = smem_desc_sw128(smem_u32(smem + L::kResA), 16, 1024);
    const uint64_t r2_km = smem_desc_sw128(smem_u32(smem + L::kResB), 16, 1024);
    const uint64_t late_km = smem_desc_sw128(smem_u32(smem + L::kLate), 16, 1024);
    const uint64_t late_mn = smem_desc_sw128(smem_u32(smem + L::kLate), L::kStrBox, 1024);
    const uint64_t early_km = smem_desc_sw128(smem_u32(smem + kEarlyBase), 16, 1024);
    constexpr uint32_t kStageStep = L::kStr >> 4;
    // k-step kk of a K-major tile: head-dim columns 16kk..16kk+15 (box kk / 4, 32 bytes per step inside it)
    auto res_step = [](int kk) { return (uint32_t)(kk >> 2) * (uint32_t)(L::kResBox >> 4) + (uint32_t)(kk & 3) * 2u; };
    auto str_step = [](int kk) { return (uint32_t)(kk >> 2) * (uint32_t)(L::kStrBox >> 4) + (uint32_t)(kk & 3) * 2u; };
    auto wait = [&](int bar, uint32_t parity, uint32_t where) {
      return __all_sync(0xffffffffu, mbar_wait(&bars[bar], parity, abort_flag, status, where)) != 0;
    };
    // rows of streamed block i that belong to the sequence (a partial last block holds a neighbour's
    // tokens or padding beyond them, which must not reach a product: they are zeroed in place)
    auto valid_rows = [&](int i) { return cols_total - (cb_lo + (kKeys ? i % ncb : i)) * kNB; };
    // the GEMMs that only need the block's tiles: dP'_i into dP buffer i & 1, then S'_i into the one S'
    // buffer once the compute warps have copied S'_{i-1} out.  (dP' goes first: the late tile S' reads
    // was requested only when the accumulating GEMM of block i-2 had finished, and dP' gives that copy
    // time to land.)
    auto issue_early = [&](int i) -> bool {
      const uint32_t s = (uint32_t)i & 1u;
      const uint32_t es = (uint32_t)(i % kEarlyStages), epar = (uint32_t)(i / kEarlyStages) & 1u;
      if constexpr (MODE == kWideDV) {
        if (i > 0 && !wait(L::bSRead, (uint32_t)(i - 1) & 1u, 0x3800)) return false;
        if (!wait(L::bEarlyFull + es, epar, 0x3200)) return false;
        tc_fence_after();
        const uint64_t ea = early_km + (uint64_t)(es * kStageStep);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 16; ++kk)
            if (kk < ksteps_qk) mma_ss(tmem_base + kWColS, r1_km + res_step(kk), ea + str_step(kk), kIdescS, kk > 0 ? 1u : 0u);
          mma_commit(&bars[L::bSFull]);
          mma_commit(&bars[L::bEarlyEmpty + es]);
          // the accumulating GEMM of block i-2 has run: its P' buffer can be written again
          mma_commit(&bars[L::bDpFull + s]);
        }
        __syncwarp();
      } else {
        const int valid = valid_rows(i);
        if (!wait(L::bEarlyFull + es, epar, 0x3400)) return false;
        if (valid < kNB) zero_tail_rows_streamed(smem + kEarlyBase + es * L::kStr, valid, lane);
        tc_fence_after();
        const uint64_t ea = early_km + (uint64_t)(es * kStageStep);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 16; ++kk)
            if (kk < ksteps_vo)
              mma_ss(tmem_base + kWColDP + s * 64u, r2_km + res_step(kk), ea + str_step(kk), kIdescS, kk > 0 ? 1u : 0u);
          mma_commit(&bars[L::bDpFull + s]);
          mma_commit(&bars[L::bEarlyEmpty + es]);
        }
        __syncwarp();
        if (i > 0 && !wait(L::bSRead, (uint32_t)(i - 1) & 1u, 0x3800)) return false;
        if (!wait(L::bLateFull + s, (uint32_t)(i >> 1) & 1u, 0x3300)) return false;
        if (valid < kNB) zero_tail_rows_streamed(smem + L::kLate + s * L::kStr, valid, lane);
        tc_fence_after();
        const uint64_t la = late_km + (uint64_t)(s * kStageStep);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 16; ++kk)
            if (kk < ksteps_qk) mma_ss(tmem_base + kWColS, r1_km + res_step(kk), la + str_step(kk), kIdescS, kk > 0 ? 1u : 0u);
          mma_commit(&bars[L::bSFull]);
        }
        __syncwarp();
      }
      return true;
    };
    // accumulator += A'_i (packed 16-bit, in dP buffer i & 1) x late tile of block i, its 64 rows contracted
    auto issue_acc = [&](int i) -> bool {
      const uint32_t s = (uint32_t)i & 1u;
      if (!wait(L::bDsFull + s, (uint32_t)(i >> 1) & 1u, 0x3500)) return false;
      if constexpr (MODE == kWideDV) {
        if (!wait(L::bLateFull + s, (uint32_t)(i >> 1) & 1u, 0x3600)) return false;
        const int valid = valid_rows(i);
        if (valid < kNB) zero_tail_rows_streamed(smem + L::kLate + s * L::kStr, valid, lane);
      }
      tc_fence_after();
      const uint64_t lb = late_mn + (uint64_t)(s * kStageStep);
      const uint32_t a_col = tmem_base + kWColDP + s * 64u;
      const uint32_t first = i > 0 ? 1u : 0u;
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < kNB / 16; ++kk)
          mma_ts(tmem_base + kWColAcc, a_col + split_a_col(kk), lb + (uint32_t)kk * (2048u >> 4), idesc_acc, kk > 0 ? 1u : first);
        mma_commit(&bars[L::bLateEmpty + s]);
        if (i + 1 == niter) mma_commit(&bars[L::bAccDone]);
      }
      __syncwarp();
      return true;
    };
    // order on the tensor pipe:  dP'_{i+1} S'_{i+1} | acc_i   (S' has one buffer: S'_{i+1} follows the
    // compute warps' copy of S'_i into registers; dP'_{i+1} takes the buffer acc_{i-1} has read)
    bool ok = wait(L::bResFull, 0, 0x3700);
    if (ok) ok = issue_early(0);
    for (int i = 0; ok && i < niter; ++i) {
      if (i + 1 < niter && !(ok = issue_early(i + 1))) break;
      ok = issue_acc(i);
    }
  } else if (warp == 2) {
    // logsumexp (in log2 units) and delta of the streamed query blocks (dV, dK), staged negated
    if constexpr (kKeys) {
      for (int i = 0, hg = 0, cb = 0; i < niter; ++i) {
        const int s = i & 1;
        if (!mbar_wait_relaxed(&bars[L::bAuxEmpty + s], ((uint32_t)(i >> 1) & 1u) ^ 1u, abort_flag, status, 0x3900)) break;
        const int h = hk * p.group + hg;
        const int mbase = (cb_lo + cb) * kNB;
        if (++cb == ncb) { cb = 0; ++hg; }
        const int64_t lrow = lse_offset(p, sq, h);
        float* dst = aux + s * (2 * kNB);
        float l2[2], dl[2];
        bool huge = false;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          const int m = mbase + lane * 2 + t;
          const bool in = m < sq.sq;
          l2[t] = in ? __ldg(p.lse + lrow + m) : INFINITY;
          dl[t] = in ? __ldg(p.delta + lrow + m) : 0.f;
        }
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          l2[t] *= kLog2e;
          huge = huge || (fabsf(l2[t]) > 1.0e6f && l2[t] != INFINITY);
        }
        *reinterpret_cast<float2*>(dst + lane * 2) = make_float2(-l2[0], -l2[1]);
        *reinterpret_cast<float2*>(dst + kNB + lane * 2) = make_float2(-dl[0], -dl[1]);
        const bool any_huge = __any_sync(0xffffffffu, huge);
        if (lane == 0) aux_flag[s] = any_huge ? 1u : 0u;
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[L::bAuxFull + s]);
      }
    }
  } else if (warp >= 4) {
    // ================================== compute ======================================
    const int quarter = warp & 3, wg = (warp - 4) >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int cbase = kWgCols * wg;
    const int row = r0 + r;                       // key (dV, dK) or query (dQ) of this thread
    // columns this row may see
    int v_lo = 0, v_hi = cols_total - 1;
    if (p.causal) {
      const int64_t lo = (int64_t)row - (kKeys ? sq.wr : sq.wl), hi = (int64_t)row + (kKeys ? sq.wl : sq.wr);
      if (lo > v_lo) v_lo = (int)(lo > 0x7fffffffLL ? 0x7fffffffLL : lo);
      if (hi < v_hi) v_hi = (int)(hi < -1 ? -1 : hi);
    }
    if (row >= rows_total) { v_lo = 1; v_hi = 0; }
    // the tightest bounds over the warp's rows: a block needs masking iff it is not inside them
    const int warp_lo = __reduce_max_sync(0xffffffffu, v_lo), warp_hi = __reduce_min_sync(0xffffffffu, v_hi);
    bool ok = true;
    // Philox seed and offset are read once; the round keys depend on the seed only
    const uint64_t ph_seed = (p.dropout_on && p.seed_ptr) ? *p.seed_ptr : 0ull;
    const uint64_t ph_off = p.off2 + ((p.dropout_on && p.off1_ptr) ? *p.off1_ptr : 0ull);
    PhiloxKeys pkeys;
    if (p.dropout_on) pkeys = philox_keys(ph_seed);
    if constexpr (kKeys) {
      const int n = row;
      for (int i = 0, hg = 0, cb = 0; i < niter; ++i) {
        const int s = i & 1;
        const uint32_t par2 = (uint32_t)(i >> 1) & 1u;
        const int h = hk * p.group + hg;
        const int mbase = (cb_lo + cb) * kNB + cbase;      // first query row of this thread's columns
        if (++cb == ncb) { cb = 0; ++hg; }
        const uint32_t lse2 = aux_s + (uint32_t)(s * 2 * kNB + cbase) * 4u;      // shared-space addresses
        const uint32_t dlt = lse2 + (uint32_t)kNB * 4u;
        if (p.has_bias && p.bias_vec)      // the warp's 32 x 32 bias tile, one 64-byte row per lane, towards L2
          asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const T*>(p.bias.ptr) + (int64_t)sq.bidx * p.bias.s[0] +
                                                       (int64_t)h * p.bias.s[1] + (int64_t)min(mbase + lane, sq.sq - 1) * p.bias.s[2] +
                                                       (r0 + quarter * 32)));
        if (!mbar_wait(&bars[L::bSFull], (uint32_t)i & 1u, abort_flag, status, 0x3A00)) { ok = false; break; }
        if (!mbar_wait(&bars[L::bAuxFull + s], par2, abort_flag, status, 0x3A80)) { ok = false; break; }
        tc_fence_after();
        float pr[32];
        tmem_ld32f(tmem_base + lane_addr + kWColS + cbase, pr);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[L::bSRead]);
        const bool any_mask = !(mbase >= warp_lo && mbase + kWgCols - 1 <= warp_hi);
        if (!p.has_bias && aux_flag[s] == 0) {
          const float2 sc2 = make_float2(p.qk_scale, p.qk_scale);
#pragma unroll
          for (int c4 = 0; c4 < 8; ++c4) {
            const float4 l4 = lds128(lse2 + 16u * c4);
            const float2 a = fma2(make_float2(pr[4 * c4], pr[4 * c4 + 1]), sc2, make_float2(l4.x, l4.y));
            const float2 b = fma2(make_float2(pr[4 * c4 + 2], pr[4 * c4 + 3]), sc2, make_float2(l4.z, l4.w));
            pr[4 * c4 + 0] = ex2(a.x);
            pr[4 * c4 + 1] = ex2(a.y);
            pr[4 * c4 + 2] = ex2(b.x);
            pr[4 * c4 + 3] = ex2(b.y);
          }
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) pr[c] *= p.qk_scale;
          if (p.has_bias && p.bias_vec && mbase + 32 <= sq.sq && r0 + quarter * 32 + 32 <= sq.sk) {
            // the warp's whole 32 x 32 bias tile is inside the sequence: vector loads and a transpose
            add_bias_column32<T>(pr, reinterpret_cast<const T*>(p.bias.ptr) + (int64_t)sq.bidx * p.bias.s[0] +
                                         (int64_t)h * p.bias.s[1] + (int64_t)mbase * p.bias.s[2] + (r0 + quarter * 32),
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
            pr[c] = (m >= v_lo && m <= v_hi) ? pr[c] : 0.f;
          }
        }
        uint32_t keep = 0xffffffffu;
        if (p.dropout_on) {
          // One Philox counter serves four consecutive keys of one query row, and the four lanes of
          // a quad own exactly such keys: lane q4 of the quad draws the counters of query rows
          // mbase + q4 + 4k (k = 0..7) for all four keys, then the quad exchanges them.
          const DropoutCtx dctx = dropout_ctx_from(p, ph_seed, ph_off, z, h);
          const int q4 = lane & 3;
          uint32_t mine = 0u;
#pragma unroll
          for (int k = 0; k < 8; ++k)
            mine |= dropout_keep4_keys(dctx, pkeys, min(mbase + q4 + 4 * k, p.max_sq - 1), n >> 2) << (4 * k);
          keep = 0u;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t w = __shfl_sync(0xffffffffu, mine, (lane & ~3) | j);
            keep |= ((w >> q4) & 0x11111111u) << j;      // this lane's key, query rows mbase + j + 4k -> bit 4k + j
          }
        }
        // dP' of this block is there (dK); for dV the same barrier says that the buffer's previous
        // P' has been consumed
        if (!mbar_wait(&bars[L::bDpFull + s], par2, abort_flag, status, 0x3B00)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_col = tmem_base + lane_addr + kWColDP + (uint32_t)s * 64u + cbase;
        uint32_t pk[16];
        if constexpr (MODE == kWideDV) {
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            float a = pr[2 * c], b = pr[2 * c + 1];
            if (p.dropout_on) {
              a = ((keep >> (2 * c)) & 1u) ? a * p.dropout_scale : 0.f;
              b = ((keep >> (2 * c + 1)) & 1u) ? b * p.dropout_scale : 0.f;
            }
            pk[c] = pack2<T>(a, b);
          }
        } else {
          float dp[32];
          tmem_ld32f(a_col, dp);
          tmem_wait_ld();
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
        }
        tmem_st16(a_col, pk);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars[L::bDsFull + s]);
          mbar_arrive(&bars[L::bAuxEmpty + s]);
        }
      }
    } else {
      const int m = row;
      const int64_t lrow = lse_offset(p, sq, hrow);
      const float lse2 = (m < sq.sq) ? p.lse[lrow + m] * kLog2e : INFINITY;
      const float dlt = (m < sq.sq) ? p.delta[lrow + m] : 0.f;
      const bool simple = !p.has_bias && !__any_sync(0xffffffffu, fabsf(lse2) > 1.0e6f && lse2 != INFINITY);
      DropoutCtx dctx;
      if (p.dropout_on) dctx = dropout_ctx_from(p, ph_seed, ph_off, z, hrow);
      const int mm = min(m, sq.sq - 1);
      const T* bias_row = p.has_bias ? reinterpret_cast<const T*>(p.bias.ptr) + (int64_t)sq.bidx * p.bias.s[0] +
                                           (int64_t)hrow * p.bias.s[1] + (int64_t)mm * p.bias.s[2]
                                     : nullptr;
      T* db_row = p.has_dbias ? reinterpret_cast<T*>(p.dbias.ptr) + (int64_t)sq.bidx * p.dbias.s[0] +
                                    (int64_t)hrow * p.dbias.s[1] + (int64_t)mm * p.dbias.s[2]
                              : nullptr;
      for (int i = 0; i < niter; ++i) {
        const int s = i & 1;
        const uint32_t par2 = (uint32_t)(i >> 1) & 1u;
        const int nbase = (cb_lo + i) * kNB + cbase;     // first key of this thread's columns
        if (p.has_bias && p.bias_vec) asm volatile("prefetch.global.L2 [%0];" ::"l"(bias_row + nbase));
        if (!mbar_wait(&bars[L::bSFull], (uint32_t)i & 1u, abort_flag, status, 0x3C00)) { ok = false; break; }
        tc_fence_after();
        float pr[32];
        tmem_ld32f(tmem_base + lane_addr + kWColS + cbase, pr);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[L::bSRead]);
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
                for (int j = 0; j < 8; ++j) pr[u * 8 + j] = fmaf(to_f32<T>(e[j]), kLog2e, pr[u * 8 + j]);
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
            pr[c] = (n >= v_lo && n <= v_hi) ? pr[c] : 0.f;
          }
        }
        uint32_t keep = 0xffffffffu;
        if (p.dropout_on) {
          keep = 0u;
          const int md = min(m, p.max_sq - 1);
#pragma unroll
          for (int c4 = 0; c4 < 8; ++c4) keep |= dropout_keep4_keys(dctx, pkeys, md, (nbase >> 2) + c4) << (4 * c4);
        }
        const uint32_t a_col = tmem_base + lane_addr + kWColDP + (uint32_t)s * 64u + cbase;
        if (!mbar_wait(&bars[L::bDpFull + s], par2, abort_flag, status, 0x3D00)) { ok = false; break; }
        tc_fence_after();
        {
          float dp[32];
          tmem_ld32f(a_col, dp);
          tmem_wait_ld();
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
          tmem_st16(a_col, pk);
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
        if (lane == 0) mbar_arrive(&bars[L::bDsFull + s]);
      }
    }
    // ---- write-out: the accumulator through the (now idle) first resident tile, so that the global
    // stores are 64-byte row segments ----
    if (ok) ok = mbar_wait(&bars[L::bAccDone], 0, abort_flag, status, 0x3E00);
    if (ok) {
      tc_fence_after();
      uint8_t* stage = smem + L::kResA;
      const int nrows = min(kBlk, rows_total - r0);
      T* dst = reinterpret_cast<T*>(outv.ptr) + (int64_t)sq.bidx * outv.s[0] + (int64_t)hrow * outv.s[1] +
               (row_tok0 + r0) * outv.s[2];
      const float scale = MODE == kWideDV ? 1.0f : p.sm_scale;
      for (int c = wg; c * 32 < d_out; c += 2) {
        float v[32];
        tmem_ld32f(tmem_base + lane_addr + kWColAcc + c * 32, v);
        tmem_wait_ld();
        stage_put32<T>(stage, r, c * 32, v, scale, 512);
        __syncwarp();
        warp_copy_out<T, 4>(stage, dst, outv.s[2], nrows, d_out, quarter * 32, c * 4, lane, 512);
        __syncwarp();
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

// which: 1 dV and dK (two launches), 2 dQ(+dBias)
template <typename T>
cudaError_t launch_bwd_wide_T(int which, const Params& p, cudaStream_t st) {
  using L = WideSmem;
  CUtensorMap q128, k128, v128, do128, q64, k64, v64, do64;
  if (which == 1) {
    if (!make_tile_map_16bit(&k128, p.k, p.dqk, p.k.n[2], kBlk) || !make_tile_map_16bit(&v128, p.v, p.dvo, p.v.n[2], kBlk) ||
        !make_tile_map_16bit(&q64, p.q, p.dqk, p.q.n[2], kNB) || !make_tile_map_16bit(&do64, p.dout, p.dvo, p.dout.n[2], kNB))
      return cudaErrorInvalidValue;
  } else {
    if (!make_tile_map_16bit(&q128, p.q, p.dqk, p.q.n[2], kBlk) ||
        !make_tile_map_16bit(&do128, p.dout, p.dvo, p.dout.n[2], kBlk) ||
        !make_tile_map_16bit(&k64, p.k, p.dqk, p.k.n[2], kNB) || !make_tile_map_16bit(&v64, p.v, p.dvo, p.v.n[2], kNB))
      return cudaErrorInvalidValue;
  }
  static std::atomic<unsigned int*> status_of[64];
  static std::atomic<bool> attr_set[64][3];
  int dev = 0;
  cudaError_t e = host().get_device(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  const bool pretend = host_pretends();      // (a pretended device's facts are not remembered)
  unsigned int* status = pretend ? nullptr : status_of[dev].load(std::memory_order_acquire);
  if (status == nullptr) {
    if ((e = host().symbol_address(reinterpret_cast<void**>(&status), reinterpret_cast<const void*>(&g_sm100_bwd_status))) != cudaSuccess) return e;
    if (!pretend) status_of[dev].store(status, std::memory_order_release);
  }
  auto set_smem = [&](int slot, const void* fn) -> cudaError_t {
    if (!pretend && attr_set[dev][slot].load(std::memory_order_acquire)) return cudaSuccess;
    cudaError_t r = host().func_set_smem(fn, L::kDynamic);
    if (r == cudaSuccess && !pretend) attr_set[dev][slot].store(true, std::memory_order_release);
    return r;
  };
  if (which == 1) {
    auto kern_dv = sm100_bwd_wide_kernel<T, kWideDV>;
    auto kern_dk = sm100_bwd_wide_kernel<T, kWideDK>;
    if ((e = set_smem(0, reinterpret_cast<const void*>(kern_dv))) != cudaSuccess) return e;
    if ((e = set_smem(1, reinterpret_cast<const void*>(kern_dk))) != cudaSuccess) return e;
    dim3 grid((p.max_sk + kBlk - 1) / kBlk, p.hk, p.batch);
    e = launch_kernel(kern_dv, grid, dim3(kWideThreads), L::kDynamic, st, p, k128, k128, do64, q64, status);
    if (e != cudaSuccess) return e;
    count_launch();
    e = launch_kernel(kern_dk, grid, dim3(kWideThreads), L::kDynamic, st, p, k128, v128, q64, do64, status);
  } else {
    auto kern_dq = sm100_bwd_wide_kernel<T, kWideDQ>;
    if ((e = set_smem(2, reinterpret_cast<const void*>(kern_dq))) != cudaSuccess) return e;
    dim3 grid((p.max_sq + kBlk - 1) / kBlk, p.hq, p.batch);
    e = launch_kernel(kern_dq, grid, dim3(kWideThreads), L::kDynamic, st, p, q128, do128, k64, v64, status);
  }
  if (e == cudaSuccess) count_launch();
  return e;
}
