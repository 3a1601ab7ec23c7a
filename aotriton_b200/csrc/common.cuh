// Device-side problem description and the arithmetic every attention kernel of
// this library shares: per-sequence geometry (dense / compact / padded / strided
// varlen), window parsing, the Philox dropout keep bit and dtype conversion.
//
// The formulas restate the behaviour of ROCm/aotriton's kernels:
//   sequence geometry   modules/flash/kernel/fwd_kernel.py:247-287
//   LSE / delta layout  modules/flash/kernel/fwd_kernel_inner.py:38-43
//   window parsing      modules/flash/kernel/masked_load_store.py:43-63
//   mask predicate      modules/flash/kernel/fwd_kernel_inner.py:127-150
//   dropout keep bit    modules/flash/kernel/dropout.py:16-70 (Philox4x32-10 as in
//                       triton/language/random.py:12-43)
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace ab200 {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471824645996f;

struct View4 {
  void* ptr;
  int64_t n[4];   // extents
  int64_t s[4];   // strides in elements
};

// Everything a kernel needs, passed by value as a __grid_constant__ parameter.
struct Params {
  View4 q, k, v, bias, out, dout, dq, dk, dv, dbias;
  float* lse;          // written by forward, read by backward
  float* delta;        // backward scratch
  int32_t batch, hq, hk, group;
  int32_t max_sq, max_sk, dqk, dvo;
  float sm_scale, qk_scale;       // qk_scale = sm_scale * log2(e)
  float dropout_p, dropout_scale; // dropout_scale = 1 / (1 - p)
  int32_t idropout;               // integer keep threshold
  int32_t dropout_on;
  int32_t causal;                 // causal_type != 0
  int32_t causal_type, window_left, window_right;
  int32_t varlen_mode;            // 0 dense, 1 compact/strided (THD), 2 padded (BHSD)
  const int32_t *cu_q, *cu_k, *ss_q, *ss_k;
  const uint64_t *seed_ptr, *off1_ptr;
  uint64_t off2;
  uint64_t *seed_out, *off_out;
  int32_t philox_head_offset, philox_hq;
  int32_t has_bias, has_dbias;
  int32_t bias_vec;               // bias rows are 16-byte aligned and unit-stride: read eight values per load
  uint32_t wait_limit_kcycles;    // bound of every in-kernel wait, in units of 1024 SM cycles (0 = about a second)
  int32_t drop_copy;              // test hook of the bounded waits: the producer leaves out one tile copy
                                  // (1 = first V block of the forward, 2 = first Q/dO block of dK/dV, 3 = first V block of dQ)
};

// Geometry of one (sequence z) slice.
struct Seq {
  int32_t sq, sk;        // actual lengths
  int64_t q0, k0;        // first token along the sequence axis
  int32_t bidx;          // index along the batch axis of the tensors
  int64_t lse_row;       // lse offset is (bidx*Hq + h) * lse_row + q0 + m
  int32_t wl, wr;        // parsed window (only meaningful when causal)
};

__device__ __forceinline__ Seq resolve_seq(const Params& p, int z) {
  Seq s;
  if (p.varlen_mode == 0) {
    s.sq = p.max_sq; s.sk = p.max_sk; s.q0 = 0; s.k0 = 0; s.bidx = z; s.lse_row = p.max_sq;
  } else {
    int q_lo = p.cu_q[z], q_hi = p.cu_q[z + 1];
    int k_lo = p.cu_k[z], k_hi = p.cu_k[z + 1];
    s.sq = q_hi - q_lo;
    s.sk = k_hi - k_lo;
    if (p.varlen_mode == 2) {          // padded: rank-4 tensors, lengths from cu_seqlens
      s.q0 = 0; s.k0 = 0; s.bidx = z; s.lse_row = p.max_sq;
    } else if (p.ss_q != nullptr) {    // strided THD: offsets from seq_strides
      s.q0 = p.ss_q[z]; s.k0 = p.ss_k[z]; s.bidx = 0; s.lse_row = p.ss_q[p.batch];
    } else {                           // compact THD
      s.q0 = q_lo; s.k0 = k_lo; s.bidx = 0; s.lse_row = p.cu_q[p.batch];
    }
  }
  const int32_t kTopLeft = -2147483647, kBottomRight = -2147483646;
  if (p.causal_type == 1 || p.window_left == kTopLeft) s.wl = s.sq;
  else if (p.causal_type == 2 || p.window_left == kBottomRight) s.wl = s.sq;
  else s.wl = p.window_left;
  if (p.causal_type == 1 || p.window_right == kTopLeft) s.wr = 0;
  else if (p.causal_type == 2 || p.window_right == kBottomRight) s.wr = s.sk - s.sq;
  else s.wr = p.window_right;
  return s;
}

__device__ __forceinline__ int64_t lse_offset(const Params& p, const Seq& s, int h) {
  return ((int64_t)s.bidx * p.hq + h) * s.lse_row + s.q0;
}

// (m, n) relative to the sequence; true when the score takes part in the softmax.
__device__ __forceinline__ bool score_valid(const Params& p, const Seq& s, int m, int n) {
  bool ok = (m < s.sq) && (n < s.sk);
  if (p.causal) ok = ok && (n <= m + s.wr) && (n >= m - s.wl);
  return ok;
}

// Closed range of key indices that can be valid for query rows [m_lo, m_hi].
__device__ __forceinline__ void key_range(const Params& p, const Seq& s, int m_lo, int m_hi, int& n_lo, int& n_hi) {
  n_lo = 0; n_hi = s.sk - 1;
  if (p.causal) {
    int64_t lo = (int64_t)m_lo - s.wl, hi = (int64_t)m_hi + s.wr;
    if (lo > n_lo) n_lo = (int)(lo > 2147483647LL ? 2147483647LL : lo);
    if (hi < n_hi) n_hi = (int)(hi < -1 ? -1 : hi);
  }
}

// Closed range of query rows that can be valid for keys [n_lo, n_hi].
__device__ __forceinline__ void query_range(const Params& p, const Seq& s, int n_lo, int n_hi, int& m_lo, int& m_hi) {
  m_lo = 0; m_hi = s.sq - 1;
  if (p.causal) {
    int64_t lo = (int64_t)n_lo - s.wr, hi = (int64_t)n_hi + s.wl;
    if (lo > m_lo) m_lo = (int)(lo > 2147483647LL ? 2147483647LL : lo);
    if (hi < m_hi) m_hi = (int)(hi < -1 ? -1 : hi);
  }
}

// ---------------------------------------------------------------------------
// Philox4x32-10, counter = (offset lo, offset hi, 0, 0), key = (seed lo, seed hi).
struct Philox4 { uint32_t w[4]; };

__host__ __device__ __forceinline__ Philox4 philox4x32_10(uint64_t seed, uint64_t offset) {
  const uint32_t kA = 0xD2511F53u, kB = 0xCD9E8D57u, kKA = 0x9E3779B9u, kKB = 0xBB67AE85u;
  uint32_t c0 = (uint32_t)offset, c1 = (uint32_t)(offset >> 32), c2 = 0u, c3 = 0u;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    uint64_t pa = (uint64_t)kA * c0, pb = (uint64_t)kB * c2;
    uint32_t n0 = (uint32_t)(pb >> 32) ^ c1 ^ k0;
    uint32_t n2 = (uint32_t)(pa >> 32) ^ c3 ^ k1;
    c1 = (uint32_t)pb; c3 = (uint32_t)pa; c0 = n0; c2 = n2;
    k0 += kKA; k1 += kKB;
  }
  Philox4 r; r.w[0] = c0; r.w[1] = c1; r.w[2] = c2; r.w[3] = c3;
  return r;
}

// Dropout state of one (sequence, q-head): everything but the row/column part of the counter.
struct DropoutCtx {
  uint64_t seed, base;
  uint32_t stride;      // counters per row = ceil(max_seqlen_k / 4)
  int32_t threshold;
};

// `seed` and `offset` (= philox_offset1 + philox_offset2) as read from the device scalars: a kernel
// that walks several heads reads them once and builds each head's context from the values.
__device__ __forceinline__ DropoutCtx dropout_ctx_from(const Params& p, uint64_t seed, uint64_t offset, int z, int h) {
  DropoutCtx d;
  d.seed = seed;
  d.stride = (uint32_t)((p.max_sk + 3) / 4);
  int hq_total = p.philox_hq > 0 ? p.philox_hq : p.hq;
  uint64_t zh = (uint64_t)z * hq_total + (uint64_t)(h + p.philox_head_offset);
  d.base = offset + zh * (uint64_t)p.max_sq * d.stride;
  d.threshold = p.idropout;
  return d;
}

__device__ __forceinline__ DropoutCtx dropout_ctx(const Params& p, int z, int h) {
  return dropout_ctx_from(p, p.seed_ptr ? *p.seed_ptr : 0ull, p.off2 + (p.off1_ptr ? *p.off1_ptr : 0ull), z, h);
}

// The four 32-bit words of one counter serve columns 4c..4c+3 in the order w0, w2, w1, w3.
__device__ __forceinline__ uint32_t philox_word_for_column(const Philox4& r, int n) {
  int j = n & 3;
  return j == 0 ? r.w[0] : (j == 1 ? r.w[2] : (j == 2 ? r.w[1] : r.w[3]));
}

__device__ __forceinline__ bool dropout_keep(const DropoutCtx& d, int m, int n) {
  Philox4 r = philox4x32_10(d.seed, d.base + (uint64_t)m * d.stride + (uint64_t)(n >> 2));
  return (int32_t)philox_word_for_column(r, n) > d.threshold;
}

// Keep bits of columns 4c..4c+3 of row m as a 4-bit mask (bit j = column 4c+j).
__device__ __forceinline__ uint32_t dropout_keep4(const DropoutCtx& d, int m, int c) {
  Philox4 r = philox4x32_10(d.seed, d.base + (uint64_t)m * d.stride + (uint64_t)c);
  uint32_t k = 0;
  k |= ((int32_t)r.w[0] > d.threshold) ? 1u : 0u;
  k |= ((int32_t)r.w[2] > d.threshold) ? 2u : 0u;
  k |= ((int32_t)r.w[1] > d.threshold) ? 4u : 0u;
  k |= ((int32_t)r.w[3] > d.threshold) ? 8u : 0u;
  return k;
}

// The same generator with its ten round keys precomputed (they depend on the seed only): a thread
// that draws many counters saves the two key additions of every round.
struct PhiloxKeys { uint32_t k0[10], k1[10]; };

__device__ __forceinline__ PhiloxKeys philox_keys(uint64_t seed) {
  PhiloxKeys r;
  uint32_t a = (uint32_t)seed, b = (uint32_t)(seed >> 32);
#pragma unroll
  for (int i = 0; i < 10; ++i) { r.k0[i] = a; r.k1[i] = b; a += 0x9E3779B9u; b += 0xBB67AE85u; }
  return r;
}

__device__ __forceinline__ Philox4 philox4x32_10_keys(const PhiloxKeys& ks, uint64_t offset) {
  const uint32_t kA = 0xD2511F53u, kB = 0xCD9E8D57u;
  uint32_t c0 = (uint32_t)offset, c1 = (uint32_t)(offset >> 32), c2 = 0u, c3 = 0u;
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const uint64_t pa = (uint64_t)kA * c0, pb = (uint64_t)kB * c2;
    const uint32_t n0 = (uint32_t)(pb >> 32) ^ c1 ^ ks.k0[i];
    const uint32_t n2 = (uint32_t)(pa >> 32) ^ c3 ^ ks.k1[i];
    c1 = (uint32_t)pb; c3 = (uint32_t)pa; c0 = n0; c2 = n2;
  }
  Philox4 r; r.w[0] = c0; r.w[1] = c1; r.w[2] = c2; r.w[3] = c3;
  return r;
}

// Zero the dropped ones of the four scores v[0..3] = columns 4c..4c+3 of row m, straight from the
// comparisons (no keep mask in between: for a consumer that applies the bits at once).
__device__ __forceinline__ void dropout_zero4_keys(const DropoutCtx& d, const PhiloxKeys& ks, int m, int c, float* v) {
  const Philox4 r = philox4x32_10_keys(ks, d.base + (uint64_t)m * d.stride + (uint64_t)c);
  v[0] = ((int32_t)r.w[0] > d.threshold) ? v[0] : 0.f;
  v[1] = ((int32_t)r.w[2] > d.threshold) ? v[1] : 0.f;
  v[2] = ((int32_t)r.w[1] > d.threshold) ? v[2] : 0.f;
  v[3] = ((int32_t)r.w[3] > d.threshold) ? v[3] : 0.f;
}

__device__ __forceinline__ uint32_t dropout_keep4_keys(const DropoutCtx& d, const PhiloxKeys& ks, int m, int c) {
  const Philox4 r4 = philox4x32_10_keys(ks, d.base + (uint64_t)m * d.stride + (uint64_t)c);
  const uint32_t c0 = r4.w[0], c1 = r4.w[1], c2 = r4.w[2], c3 = r4.w[3];
  uint32_t k = 0;
  k |= ((int32_t)c0 > d.threshold) ? 1u : 0u;
  k |= ((int32_t)c2 > d.threshold) ? 2u : 0u;
  k |= ((int32_t)c1 > d.threshold) ? 4u : 0u;
  k |= ((int32_t)c3 > d.threshold) ? 8u : 0u;
  return k;
}

// ---------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// dBias of query rows [m0, m0 + rows) outside the key columns [c_lo, c_hi) that the calling CTA's
// block loop visits.  A causal or windowed problem skips whole key blocks; the gradient of the bias
// there is zero, and it is written, so that dBias is defined everywhere inside the sequence.  (The
// reference leaves those entries as they were: modules/flash/kernel/bwd_inner_dq.py:200-204 stores
// dB only in the blocks its loop visits.)  Called by all threads of the CTA.
template <typename T>
__device__ __forceinline__ void zero_dbias_outside(const Params& p, const Seq& sq, int h, int m0, int rows, int c_lo,
                                                   int c_hi) {
  if (!p.has_dbias || !p.causal) return;
  const int lane = threadIdx.x & 31, nwarps = (int)blockDim.x >> 5;
  for (int r = (int)threadIdx.x >> 5; r < rows; r += nwarps) {
    const int m = m0 + r;
    if (m >= sq.sq) break;
    T* rowp = reinterpret_cast<T*>(p.dbias.ptr) + (int64_t)sq.bidx * p.dbias.s[0] + (int64_t)h * p.dbias.s[1] +
              (int64_t)m * p.dbias.s[2];
    for (int n = lane; n < min(c_lo, sq.sk); n += 32) rowp[(int64_t)n * p.dbias.s[3]] = from_f32<T>(0.f);
    for (int n = max(c_hi, 0) + lane; n < sq.sk; n += 32) rowp[(int64_t)n * p.dbias.s[3]] = from_f32<T>(0.f);
  }
}

// Round through the storage type, the way the reference casts P and dS before its GEMMs.
template <typename T> __device__ __forceinline__ float round_to(float x) { return to_f32<T>(from_f32<T>(x)); }

}  // namespace ab200
