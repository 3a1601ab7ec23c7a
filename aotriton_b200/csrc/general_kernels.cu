// General (any head dim <= 512, any of fp32/fp16/bf16, any stride) attention
// kernels.  They cover every feature of the operator -- GQA, windows, varlen in all
// three flavours, bias/dBias, dropout, Dqk != Dvo -- with plain CUDA cores and fp32
// math, and back the shapes the tcgen05 kernels do not take.
//
// All three matmul-bearing kernels share one scheme.  A CTA of 256 threads owns a
// 16x16 tile of (query, key) pairs:
//   pair phase        thread (r, c) computes the dot products of query r with key c
//                     from fp32 tiles staged in shared memory, applies scale, bias,
//                     mask, softmax pieces and dropout;
//   accumulate phase  warp w owns two rows (or two keys) of the output tile, each lane
//                     owns the head-dim columns lane, lane+32, ...; the P / dS values
//                     are read back from shared memory as broadcasts.
//
// Arithmetic follows ROCm/aotriton modules/flash/kernel/fwd_kernel_inner.py:126-277,
// fwd_kernel.py:573-620, bwd_inner_dk_dv.py:117-256, bwd_inner_dq.py:117-205,
// bwd_preprocess.py:118-133 and dropout_rng.py:86-126.
#include "common.cuh"
#include "launch.h"

namespace ab200 {

namespace {

constexpr int kTile = 16;       // rows and keys per tile
constexpr int kThreads = 256;
constexpr int kPad = 4;         // floats of padding per staged row (keeps float4 alignment)

template <typename T>
__device__ __forceinline__ const T* row_ptr(const View4& v, int b, int h, int64_t tok) {
  return reinterpret_cast<const T*>(v.ptr) + (int64_t)b * v.s[0] + (int64_t)h * v.s[1] + tok * v.s[2];
}
template <typename T>
__device__ __forceinline__ T* row_ptr_mut(const View4& v, int b, int h, int64_t tok) {
  return reinterpret_cast<T*>(v.ptr) + (int64_t)b * v.s[0] + (int64_t)h * v.s[1] + tok * v.s[2];
}

// Stage `kTile` rows starting at token tok0+row0 into dst[kTile][ld] as fp32; rows >= nrows
// and columns >= d are zero.
template <typename T>
__device__ __forceinline__ void stage_rows(float* dst, int ld, int dpad, const View4& v, int b, int h,
                                           int64_t tok0, int row0, int nrows, int d) {
  for (int idx = threadIdx.x; idx < kTile * dpad; idx += kThreads) {
    int r = idx / dpad, c = idx - r * dpad;
    float x = 0.f;
    int row = row0 + r;
    if (row < nrows && c < d) x = to_f32<T>(row_ptr<T>(v, b, h, tok0 + row)[c]);
    dst[r * ld + c] = x;
  }
}

__device__ __forceinline__ float dot_rows(const float* a, const float* b, int dpad) {
  float acc = 0.f;
  for (int c = 0; c < dpad; c += 4) {
    float4 x = *reinterpret_cast<const float4*>(a + c);
    float4 y = *reinterpret_cast<const float4*>(b + c);
    acc = fmaf(x.x, y.x, acc); acc = fmaf(x.y, y.y, acc);
    acc = fmaf(x.z, y.z, acc); acc = fmaf(x.w, y.w, acc);
  }
  return acc;
}

__device__ __forceinline__ float half_warp_max(float x) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float half_warp_sum(float x) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// ---------------------------------------------------------------------------
// Forward.  grid = (cdiv(max_sq, 16), Hq, batch)
template <typename T, int DJ>
__global__ void __launch_bounds__(kThreads) general_fwd_kernel(const __grid_constant__ Params p) {
  extern __shared__ float smem[];
  constexpr int DPAD = DJ * 32;
  constexpr int LD = DPAD + kPad;
  float* Qs = smem;                    // [16][LD]
  float* Ks = Qs + kTile * LD;         // [16][LD]
  float* Vs = Ks + kTile * LD;         // [16][LD]
  float* Ps = Vs + kTile * LD;         // [16][16]
  float* alpha_s = Ps + kTile * kTile; // [16]
  float* l_s = alpha_s + kTile;        // [16]

  const int z = blockIdx.z, h = blockIdx.y, m0 = blockIdx.x * kTile;
  // One thread of the grid reports the seed and offset actually used, before any early exit
  // (the first sequence of a varlen batch may be empty).
  if (p.dropout_on && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) {
    uint64_t seed = p.seed_ptr ? *p.seed_ptr : 0ull;
    uint64_t base = p.off2 + (p.off1_ptr ? *p.off1_ptr : 0ull);
    if (p.seed_out) *p.seed_out = seed;
    if (p.off_out) *p.off_out = base;
  }
  const Seq sq = resolve_seq(p, z);
  if (m0 >= sq.sq) return;
  const int hk = h / p.group;
  const int tid = threadIdx.x, r = tid >> 4, c = tid & 15, warp = tid >> 5, lane = tid & 31;
  DropoutCtx dctx;
  if (p.dropout_on) dctx = dropout_ctx(p, z, h);

  stage_rows<T>(Qs, LD, DPAD, p.q, sq.bidx, h, sq.q0, m0, sq.sq, p.dqk);

  float m_i = -INFINITY, l_i = 0.f;
  float acc[2][DJ];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < DJ; ++j) acc[i][j] = 0.f;

  int n_lo, n_hi;
  key_range(p, sq, m0, min(m0 + kTile, sq.sq) - 1, n_lo, n_hi);
  const int m = m0 + r;
  for (int nb = n_lo / kTile; nb * kTile <= n_hi; ++nb) {
    const int n0 = nb * kTile;
    __syncthreads();   // previous accumulate phase done (and Qs staged on first trip)
    stage_rows<T>(Ks, LD, DPAD, p.k, sq.bidx, hk, sq.k0, n0, sq.sk, p.dqk);
    stage_rows<T>(Vs, LD, DPAD, p.v, sq.bidx, hk, sq.k0, n0, sq.sk, p.dvo);
    __syncthreads();
    const int n = n0 + c;
    float s = -INFINITY;
    if (score_valid(p, sq, m, n)) {
      s = dot_rows(Qs + r * LD, Ks + c * LD, DPAD) * p.qk_scale;
      if (p.has_bias) {
        const T* bp = reinterpret_cast<const T*>(p.bias.ptr) + (int64_t)sq.bidx * p.bias.s[0] +
                      (int64_t)h * p.bias.s[1] + (int64_t)m * p.bias.s[2] + (int64_t)n * p.bias.s[3];
        s += to_f32<T>(*bp) * kLog2e;
      }
    }
    float m_new = fmaxf(m_i, half_warp_max(s));
    float pv = 0.f, alpha = 1.f;
    if (m_new != -INFINITY) {
      pv = exp2f(s - m_new);
      alpha = exp2f(m_i - m_new);   // m_i == -inf -> 0
    }
    l_i = l_i * alpha + half_warp_sum(pv);
    m_i = m_new;
    if (p.dropout_on && !dropout_keep(dctx, m, n)) pv = 0.f;
    Ps[r * kTile + c] = round_to<T>(pv);
    if (c == 0) alpha_s[r] = alpha;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = warp * 2 + i;
      const float a = alpha_s[row];
#pragma unroll
      for (int j = 0; j < DJ; ++j) acc[i][j] *= a;
      for (int kk = 0; kk < kTile; ++kk) {
        const float pk = Ps[row * kTile + kk];
#pragma unroll
        for (int j = 0; j < DJ; ++j) acc[i][j] = fmaf(pk, Vs[kk * LD + lane + 32 * j], acc[i][j]);
      }
    }
  }
  if (c == 0) {
    l_s[r] = l_i;
    if (p.lse != nullptr && m < sq.sq) {
      // natural-log LSE of the scaled, biased logits; rows without any valid key get +inf
      float lse = (l_i > 0.f) ? (m_i + log2f(l_i)) * kLn2 : INFINITY;
      p.lse[lse_offset(p, sq, h) + m] = lse;
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = m0 + warp * 2 + i;
    if (row >= sq.sq) continue;
    const float l = l_s[warp * 2 + i];
    const float inv = (l > 0.f) ? (1.f / l) * p.dropout_scale : 0.f;
    T* op = row_ptr_mut<T>(p.out, sq.bidx, h, sq.q0 + row);
#pragma unroll
    for (int j = 0; j < DJ; ++j) {
      const int d = lane + 32 * j;
      if (d < p.dvo) op[d] = from_f32<T>(acc[i][j] * inv);
    }
  }
}

// ---------------------------------------------------------------------------
// Pair phase shared by both backward kernels: recompute P, dP and dS for pair (m, n).
// pd_out = dropped-and-scaled P (for dV), ds_out = dS (for dK, dQ, dBias).
template <typename T>
__device__ __forceinline__ void bwd_pair(const Params& p, const Seq& sq, const DropoutCtx& dctx, int h,
                                         int m, int n, const float* qrow, const float* krow,
                                         const float* dorow, const float* vrow, int dpad,
                                         float lse_m, float delta_m, float& pd_out, float& ds_out) {
  pd_out = 0.f; ds_out = 0.f;
  if (!score_valid(p, sq, m, n)) return;
  float s = dot_rows(qrow, krow, dpad) * p.qk_scale;
  if (p.has_bias) {
    const T* bp = reinterpret_cast<const T*>(p.bias.ptr) + (int64_t)sq.bidx * p.bias.s[0] +
                  (int64_t)h * p.bias.s[1] + (int64_t)m * p.bias.s[2] + (int64_t)n * p.bias.s[3];
    s += to_f32<T>(*bp) * kLog2e;
  }
  float pr = exp2f(s - lse_m * kLog2e);      // lse = +inf on dead rows -> 0
  float dp = dot_rows(dorow, vrow, dpad);
  float pd = pr;
  if (p.dropout_on) {
    bool keep = dropout_keep(dctx, m, n);
    pd = keep ? pr * p.dropout_scale : 0.f;
    dp = keep ? dp * p.dropout_scale : 0.f;
  }
  pd_out = pd;
  ds_out = pr * (dp - delta_m);
}

// dK / dV.  grid = (cdiv(max_sk, 16), Hk, batch)
template <typename T, int DJ>
__global__ void __launch_bounds__(kThreads) general_bwd_dkdv_kernel(const __grid_constant__ Params p) {
  extern __shared__ float smem[];
  constexpr int DPAD = DJ * 32;
  constexpr int LD = DPAD + kPad;
  float* Ks = smem;
  float* Vs = Ks + kTile * LD;
  float* Qs = Vs + kTile * LD;
  float* dOs = Qs + kTile * LD;
  float* Ps = dOs + kTile * LD;        // [16 rows][16 keys]  dropped P
  float* dSs = Ps + kTile * kTile;     // [16][16]
  float* lse_s = dSs + kTile * kTile;  // [16]
  float* dl_s = lse_s + kTile;         // [16]

  const int z = blockIdx.z, hk = blockIdx.y, n0 = blockIdx.x * kTile;
  const Seq sq = resolve_seq(p, z);
  if (n0 >= sq.sk) return;
  const int tid = threadIdx.x, r = tid >> 4, c = tid & 15, warp = tid >> 5, lane = tid & 31;

  stage_rows<T>(Ks, LD, DPAD, p.k, sq.bidx, hk, sq.k0, n0, sq.sk, p.dqk);
  stage_rows<T>(Vs, LD, DPAD, p.v, sq.bidx, hk, sq.k0, n0, sq.sk, p.dvo);

  float adv[2][DJ], adk[2][DJ];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < DJ; ++j) { adv[i][j] = 0.f; adk[i][j] = 0.f; }

  int m_lo, m_hi;
  query_range(p, sq, n0, min(n0 + kTile, sq.sk) - 1, m_lo, m_hi);
  for (int g = 0; g < p.group; ++g) {
    const int h = hk * p.group + g;
    DropoutCtx dctx;
    if (p.dropout_on) dctx = dropout_ctx(p, z, h);
    const int64_t lrow = lse_offset(p, sq, h);
    for (int mb = m_lo / kTile; mb * kTile <= m_hi; ++mb) {
      const int m0 = mb * kTile;
      __syncthreads();
      stage_rows<T>(Qs, LD, DPAD, p.q, sq.bidx, h, sq.q0, m0, sq.sq, p.dqk);
      stage_rows<T>(dOs, LD, DPAD, p.dout, sq.bidx, h, sq.q0, m0, sq.sq, p.dvo);
      if (tid < kTile) {
        int mm = m0 + tid;
        lse_s[tid] = mm < sq.sq ? p.lse[lrow + mm] : 0.f;
        dl_s[tid] = mm < sq.sq ? p.delta[lrow + mm] : 0.f;
      }
      __syncthreads();
      float pd, ds;
      bwd_pair<T>(p, sq, dctx, h, m0 + r, n0 + c, Qs + r * LD, Ks + c * LD, dOs + r * LD, Vs + c * LD, DPAD,
                  lse_s[r], dl_s[r], pd, ds);
      Ps[r * kTile + c] = round_to<T>(pd);
      dSs[r * kTile + c] = round_to<T>(ds);
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int key = warp * 2 + i;
        for (int rr = 0; rr < kTile; ++rr) {
          const float pv = Ps[rr * kTile + key], dv = dSs[rr * kTile + key];
#pragma unroll
          for (int j = 0; j < DJ; ++j) {
            adv[i][j] = fmaf(pv, dOs[rr * LD + lane + 32 * j], adv[i][j]);
            adk[i][j] = fmaf(dv, Qs[rr * LD + lane + 32 * j], adk[i][j]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int n = n0 + warp * 2 + i;
    if (n >= sq.sk) continue;
    T* dkp = row_ptr_mut<T>(p.dk, sq.bidx, hk, sq.k0 + n);
    T* dvp = row_ptr_mut<T>(p.dv, sq.bidx, hk, sq.k0 + n);
#pragma unroll
    for (int j = 0; j < DJ; ++j) {
      const int d = lane + 32 * j;
      if (d < p.dqk) dkp[d] = from_f32<T>(adk[i][j] * p.sm_scale);
      if (d < p.dvo) dvp[d] = from_f32<T>(adv[i][j]);
    }
  }
}

// dQ (+ dBias).  grid = (cdiv(max_sq, 16), Hq, batch)
template <typename T, int DJ>
__global__ void __launch_bounds__(kThreads) general_bwd_dq_kernel(const __grid_constant__ Params p) {
  extern __shared__ float smem[];
  constexpr int DPAD = DJ * 32;
  constexpr int LD = DPAD + kPad;
  float* Qs = smem;
  float* dOs = Qs + kTile * LD;
  float* Ks = dOs + kTile * LD;
  float* Vs = Ks + kTile * LD;
  float* dSs = Vs + kTile * LD;        // [16][16]
  float* lse_s = dSs + kTile * kTile;
  float* dl_s = lse_s + kTile;

  const int z = blockIdx.z, h = blockIdx.y, m0 = blockIdx.x * kTile;
  const Seq sq = resolve_seq(p, z);
  if (m0 >= sq.sq) return;
  const int hk = h / p.group;
  const int tid = threadIdx.x, r = tid >> 4, c = tid & 15, warp = tid >> 5, lane = tid & 31;
  DropoutCtx dctx;
  if (p.dropout_on) dctx = dropout_ctx(p, z, h);

  stage_rows<T>(Qs, LD, DPAD, p.q, sq.bidx, h, sq.q0, m0, sq.sq, p.dqk);
  stage_rows<T>(dOs, LD, DPAD, p.dout, sq.bidx, h, sq.q0, m0, sq.sq, p.dvo);
  const int64_t lrow = lse_offset(p, sq, h);
  if (tid < kTile) {
    int mm = m0 + tid;
    lse_s[tid] = mm < sq.sq ? p.lse[lrow + mm] : 0.f;
    dl_s[tid] = mm < sq.sq ? p.delta[lrow + mm] : 0.f;
  }

  float adq[2][DJ];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < DJ; ++j) adq[i][j] = 0.f;

  int n_lo, n_hi;
  key_range(p, sq, m0, min(m0 + kTile, sq.sq) - 1, n_lo, n_hi);
  if (n_hi >= n_lo) zero_dbias_outside<T>(p, sq, h, m0, kTile, (n_lo / kTile) * kTile, (n_hi / kTile + 1) * kTile);
  else zero_dbias_outside<T>(p, sq, h, m0, kTile, 0, 0);
  const int m = m0 + r;
  for (int nb = n_lo / kTile; nb * kTile <= n_hi; ++nb) {
    const int n0 = nb * kTile;
    __syncthreads();
    stage_rows<T>(Ks, LD, DPAD, p.k, sq.bidx, hk, sq.k0, n0, sq.sk, p.dqk);
    stage_rows<T>(Vs, LD, DPAD, p.v, sq.bidx, hk, sq.k0, n0, sq.sk, p.dvo);
    __syncthreads();
    const int n = n0 + c;
    float pd, ds;
    bwd_pair<T>(p, sq, dctx, h, m, n, Qs + r * LD, Ks + c * LD, dOs + r * LD, Vs + c * LD, DPAD, lse_s[r],
                dl_s[r], pd, ds);
    if (p.has_dbias && m < sq.sq && n < sq.sk) {
      T* dbp = reinterpret_cast<T*>(p.dbias.ptr) + (int64_t)sq.bidx * p.dbias.s[0] + (int64_t)h * p.dbias.s[1] +
               (int64_t)m * p.dbias.s[2] + (int64_t)n * p.dbias.s[3];
      *dbp = from_f32<T>(ds);
    }
    dSs[r * kTile + c] = round_to<T>(ds);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = warp * 2 + i;
      for (int kk = 0; kk < kTile; ++kk) {
        const float dv = dSs[row * kTile + kk];
#pragma unroll
        for (int j = 0; j < DJ; ++j) adq[i][j] = fmaf(dv, Ks[kk * LD + lane + 32 * j], adq[i][j]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = m0 + warp * 2 + i;
    if (row >= sq.sq) continue;
    T* dqp = row_ptr_mut<T>(p.dq, sq.bidx, h, sq.q0 + row);
#pragma unroll
    for (int j = 0; j < DJ; ++j) {
      const int d = lane + 32 * j;
      if (d < p.dqk) dqp[d] = from_f32<T>(adq[i][j] * p.sm_scale);
    }
  }
}

// ---------------------------------------------------------------------------
// delta[m] = sum_d O[m,d] * dO[m,d] in fp32, written with the LSE layout.  HBM-bound.
// grid = (cdiv(max_sq, 128), Hq, batch); a CTA of 8 warps owns 128 rows of one (sequence, head).
// Fast path (16-bit types, D in {64,128,256}, 16-byte aligned rows): D/8 lanes share a row with
// one 16-byte load each from O and dO, four rows in flight per lane group.  Otherwise one warp
// per row with scalar loads.
template <typename T>
__global__ void __launch_bounds__(256) bwd_preprocess_kernel(const __grid_constant__ Params p) {
  const int z = blockIdx.z, h = blockIdx.y;
  const Seq sq = resolve_seq(p, z);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int d = p.dvo;
  const int row0 = blockIdx.x * 128;
  if (row0 >= sq.sq) return;
  const int64_t lrow = lse_offset(p, sq, h);
  const bool vec_ok = (sizeof(T) == 2) && (d == 64 || d == 128 || d == 256) &&
                      ((reinterpret_cast<uintptr_t>(p.out.ptr) | reinterpret_cast<uintptr_t>(p.dout.ptr)) % 16 == 0) &&
                      (p.out.s[0] % 8 == 0) && (p.out.s[1] % 8 == 0) && (p.out.s[2] % 8 == 0) &&
                      (p.dout.s[0] % 8 == 0) && (p.dout.s[1] % 8 == 0) && (p.dout.s[2] % 8 == 0);
  if (vec_ok) {
    const int lpr = d >> 3;                 // lanes per row: 8, 16 or 32
    const int rpw = 32 / lpr;               // rows per warp pass
    const int sub = lane / lpr, col = (lane % lpr) * 8;
    // warp w covers rows row0 + 16w .. +15 in passes of rpw rows, four passes in flight
    const int wrow0 = row0 + warp * 16;
    for (int pass = 0; pass < 16 / rpw; pass += 4) {
      uint4 a[4], b[4];
      int rows[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        rows[u] = wrow0 + (pass + u) * rpw + sub;
        const bool in = (pass + u) * rpw < 16 && rows[u] < sq.sq;
        if (in) {
          a[u] = *reinterpret_cast<const uint4*>(row_ptr<T>(p.out, sq.bidx, h, sq.q0 + rows[u]) + col);
          b[u] = *reinterpret_cast<const uint4*>(row_ptr<T>(p.dout, sq.bidx, h, sq.q0 + rows[u]) + col);
        } else {
          a[u] = make_uint4(0, 0, 0, 0);
          b[u] = make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const T* ae = reinterpret_cast<const T*>(&a[u]);
        const T* be = reinterpret_cast<const T*>(&b[u]);
        float acc = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc = fmaf(to_f32<T>(ae[e]), to_f32<T>(be[e]), acc);
        for (int o = lpr >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if ((lane % lpr) == 0 && (pass + u) * rpw < 16 && rows[u] < sq.sq) p.delta[lrow + rows[u]] = acc;
      }
    }
    return;
  }
  for (int m = row0 + warp; m < min(sq.sq, row0 + 128); m += 8) {
    const T* op = row_ptr<T>(p.out, sq.bidx, h, sq.q0 + m);
    const T* gp = row_ptr<T>(p.dout, sq.bidx, h, sq.q0 + m);
    float acc = 0.f;
    for (int c = lane; c < d; c += 32) acc = fmaf(to_f32<T>(op[c]), to_f32<T>(gp[c]), acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) p.delta[lrow + m] = acc;
  }
}

// ---------------------------------------------------------------------------
// dQ = cast(sm_scale * accumulator): the conversion that follows the fused backward, whose dQ partials
// were summed in fp32 (ROCm/aotriton modules/flash/kernel/bwd_postprocess.py:14-84).  The
// accumulator is contiguous in dQ's logical (batch, head, token, head-dim) order; dQ has its own
// strides.  HBM-bound: 4 bytes read and 2 written per element.  One thread per 8 elements when the
// rows allow 16-byte stores.  grid = (cdiv(tokens * D / 8, 256), H, B)
template <typename T>
__global__ void __launch_bounds__(256) bwd_postprocess_kernel(View4 dq, const float* __restrict__ acc, float scale,
                                                              int vec) {
  const int64_t tokens = dq.n[2], d = dq.n[3];
  const int b = blockIdx.z, h = blockIdx.y;
  const float* src = acc + ((int64_t)b * dq.n[1] + h) * tokens * d;
  T* dst = reinterpret_cast<T*>(dq.ptr) + (int64_t)b * dq.s[0] + (int64_t)h * dq.s[1];
  const int64_t i = ((int64_t)blockIdx.x * 256 + threadIdx.x) * 8;
  if (i >= tokens * d) return;
  if (vec) {
    const int64_t row = i / d, col = i - row * d;      // d % 8 == 0: the 8 elements share a row
    const float4 lo = __ldcs(reinterpret_cast<const float4*>(src + i));
    const float4 hi = __ldcs(reinterpret_cast<const float4*>(src + i + 4));
    const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    union { uint4 u; T e[8]; } w;
#pragma unroll
    for (int k = 0; k < 8; ++k) w.e[k] = from_f32<T>(v[k] * scale);
    *reinterpret_cast<uint4*>(dst + row * dq.s[2] + col) = w.u;
  } else {
    for (int k = 0; k < 8 && i + k < tokens * d; ++k) {
      const int64_t row = (i + k) / d, col = (i + k) - row * d;
      dst[row * dq.s[2] + col] = from_f32<T>(src[i + k] * scale);
    }
  }
}

// ---------------------------------------------------------------------------
// r[z,h,m,n] = keep ? +0.5 : -0.5 over the whole rows x cols rectangle.
// One thread per (row, 4 columns) = one Philox counter.  grid = (cdiv(cols/4 * rows, 256), H, B)
template <typename T>
__global__ void __launch_bounds__(256) dropout_sign_kernel(View4 r, int rows, int cols, int num_head, DropoutCtx base,
                                                           const uint64_t* seed_ptr, const uint64_t* off1_ptr,
                                                           uint64_t off2) {
  const int z = blockIdx.z, h = blockIdx.y;
  const uint32_t stride = (uint32_t)((cols + 3) / 4);
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)rows * stride) return;
  const int m = (int)(idx / stride), c4 = (int)(idx - (int64_t)m * stride);
  DropoutCtx d = base;
  d.seed = seed_ptr ? *seed_ptr : 0ull;
  d.stride = stride;
  d.base = off2 + (off1_ptr ? *off1_ptr : 0ull) + ((uint64_t)z * num_head + h) * (uint64_t)rows * stride;
  uint32_t keep = dropout_keep4(d, m, c4);
  T* out = reinterpret_cast<T*>(r.ptr) + (int64_t)z * r.s[0] + (int64_t)h * r.s[1] + (int64_t)m * r.s[2];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int n = c4 * 4 + j;
    if (n < cols) out[(int64_t)n * r.s[3]] = from_f32<T>((keep >> j) & 1u ? 0.5f : -0.5f);
  }
}

template <typename T, int DJ>
size_t fwd_smem() { return (3 * kTile * (DJ * 32 + kPad) + kTile * kTile + 2 * kTile) * sizeof(float); }
template <typename T, int DJ>
size_t bwd_smem() { return (4 * kTile * (DJ * 32 + kPad) + 2 * kTile * kTile + 2 * kTile) * sizeof(float); }

template <typename K>
cudaError_t set_smem(K kernel, size_t bytes) {
  if (bytes <= 48 * 1024) return cudaSuccess;
  return host().func_set_smem(reinterpret_cast<const void*>(kernel), (int)bytes);
}

template <typename T, int DJ>
cudaError_t launch_general_T(int which, const Params& p, cudaStream_t st) {
  cudaError_t e;
  if (which == 0) {
    size_t sm = fwd_smem<T, DJ>();
    if ((e = set_smem(general_fwd_kernel<T, DJ>, sm)) != cudaSuccess) return e;
    dim3 grid((p.max_sq + kTile - 1) / kTile, p.hq, p.batch);
    e = launch_kernel(general_fwd_kernel<T, DJ>, dim3(grid), dim3(kThreads), sm, st, p);
  } else if (which == 1) {
    size_t sm = bwd_smem<T, DJ>();
    if ((e = set_smem(general_bwd_dkdv_kernel<T, DJ>, sm)) != cudaSuccess) return e;
    dim3 grid((p.max_sk + kTile - 1) / kTile, p.hk, p.batch);
    e = launch_kernel(general_bwd_dkdv_kernel<T, DJ>, dim3(grid), dim3(kThreads), sm, st, p);
  } else {
    size_t sm = bwd_smem<T, DJ>();
    if ((e = set_smem(general_bwd_dq_kernel<T, DJ>, sm)) != cudaSuccess) return e;
    dim3 grid((p.max_sq + kTile - 1) / kTile, p.hq, p.batch);
    e = launch_kernel(general_bwd_dq_kernel<T, DJ>, dim3(grid), dim3(kThreads), sm, st, p);
  }
  if (e == cudaSuccess) count_launch();
  return e;
}

template <typename T>
cudaError_t launch_general_D(int which, const Params& p, cudaStream_t st) {
  int d = p.dqk > p.dvo ? p.dqk : p.dvo;
  if (d <= 64) return launch_general_T<T, 2>(which, p, st);
  if (d <= 128) return launch_general_T<T, 4>(which, p, st);
  if (d <= 256) return launch_general_T<T, 8>(which, p, st);
  return launch_general_T<T, 16>(which, p, st);
}

}  // namespace

cudaError_t launch_general(int which, int dtype, const Params& p, cudaStream_t st) {
  if (p.max_sq <= 0 || p.max_sk <= 0 || p.batch <= 0) return cudaSuccess;
  switch (dtype) {
    case 1: return launch_general_D<float>(which, p, st);
    case 2: return launch_general_D<__half>(which, p, st);
    case 3: return launch_general_D<__nv_bfloat16>(which, p, st);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_preprocess(int dtype, const Params& p, cudaStream_t st) {
  if (p.max_sq <= 0 || p.batch <= 0) return cudaSuccess;
  dim3 grid((p.max_sq + 127) / 128, p.hq, p.batch);
  cudaError_t e = cudaSuccess;
  switch (dtype) {
    case 1: e = launch_kernel(bwd_preprocess_kernel<float>, dim3(grid), dim3(256), 0, st, p); break;
    case 2: e = launch_kernel(bwd_preprocess_kernel<__half>, dim3(grid), dim3(256), 0, st, p); break;
    case 3: e = launch_kernel(bwd_preprocess_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, p); break;
    default: return cudaErrorInvalidValue;
  }
  if (e == cudaSuccess) count_launch();
  return e;
}

cudaError_t launch_postprocess(int dtype, const View4& dq, const float* acc, float scale, cudaStream_t st) {
  if (dq.ptr == nullptr || acc == nullptr) return cudaErrorInvalidValue;
  if (dq.n[0] <= 0 || dq.n[1] <= 0 || dq.n[2] <= 0 || dq.n[3] <= 0) return cudaSuccess;
  const int64_t per = dq.n[2] * dq.n[3];
  dim3 grid((unsigned)((per / 8 + 256) / 256), (unsigned)dq.n[1], (unsigned)dq.n[0]);
  const int vec = (dtype != 1) && dq.n[3] % 8 == 0 && (reinterpret_cast<uintptr_t>(dq.ptr) & 15u) == 0 &&
                  dq.s[0] % 8 == 0 && dq.s[1] % 8 == 0 && dq.s[2] % 8 == 0 && dq.s[3] == 1 &&
                  (reinterpret_cast<uintptr_t>(acc) & 15u) == 0;
  cudaError_t e = cudaSuccess;
  switch (dtype) {
    case 1: e = launch_kernel(bwd_postprocess_kernel<float>, dim3(grid), dim3(256), 0, st, dq, acc, scale, 0); break;
    case 2: e = launch_kernel(bwd_postprocess_kernel<__half>, dim3(grid), dim3(256), 0, st, dq, acc, scale, vec); break;
    case 3: e = launch_kernel(bwd_postprocess_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, dq, acc, scale, vec); break;
    default: return cudaErrorInvalidValue;
  }
  if (e == cudaSuccess) count_launch();
  return e;
}

cudaError_t launch_dropout_sign(int dtype, const View4& r, int batch, int heads, int rows, int cols, float dropout_p,
                                const uint64_t* seed, const uint64_t* off1, uint64_t off2, cudaStream_t st) {
  if (rows <= 0 || cols <= 0 || batch <= 0 || heads <= 0) return cudaSuccess;
  DropoutCtx d{};
  d.threshold = dropout_threshold(dropout_p);
  int64_t per = (int64_t)rows * ((cols + 3) / 4);
  dim3 grid((unsigned)((per + 255) / 256), heads, batch);
  cudaError_t e = cudaSuccess;
  switch (dtype) {
    case 1: e = launch_kernel(dropout_sign_kernel<float>, dim3(grid), dim3(256), 0, st, r, rows, cols, heads, d, seed, off1, off2); break;
    case 2: e = launch_kernel(dropout_sign_kernel<__half>, dim3(grid), dim3(256), 0, st, r, rows, cols, heads, d, seed, off1, off2); break;
    case 3: e = launch_kernel(dropout_sign_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, r, rows, cols, heads, d, seed, off1, off2); break;
    default: return cudaErrorInvalidValue;
  }
  if (e == cudaSuccess) count_launch();
  return e;
}

}  // namespace ab200
