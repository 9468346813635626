// _softmax / _log_softmax / native_layer_norm / sum.dim_IntList / argmax.
//
// The input is contiguous, viewed as [outer, dim, inner], the op runs along `dim`.
//   inner == 1, row fits in registers : "resident" kernels -- the row is read from HBM
//       exactly once with 16-byte streaming loads, held as fp32 in registers by one
//       warp (short rows) or one CTA (long rows), reduced with warp shuffles (+ one
//       shared-memory hop for CTA rows) and written once: 1 read + 1 write per element.
//   inner == 1, anything else        : "streaming" kernels, one CTA per row, scalar
//       accesses, re-reads served by L2.
//   inner  > 1                        : one thread per (outer, inner) column, coalesced
//       across `inner`, sequential along `dim`.
// sum and argmax are single-pass; when few outputs face a long reduction the reduction
// is split over gridDim.y CTAs and finished by a second tiny kernel from scratch memory.
#include <math_constants.h>

#include <mutex>

#include "b200_common.cuh"

namespace b200 {

constexpr float kLog2e = 1.4426950408889634f;

template <typename T> constexpr int dtype_of();
template <> constexpr int dtype_of<float>() { return B200_F32; }
template <> constexpr int dtype_of<__nv_bfloat16>() { return B200_BF16; }
template <> constexpr int dtype_of<__half>() { return B200_F16; }

// ---- group = one warp (WARP) or the whole CTA: reductions over the threads of a row
template <bool WARP, typename F>
__device__ __forceinline__ float group_reduce(float v, F f, float identity, float* smem, int phase) {
  if (WARP) return warp_reduce(v, f);
  return block_reduce_once(v, f, identity, smem, phase);
}

// Store VE fp32 values at element offset `e0` of `out`, as T (16-byte store) or as fp32.
template <typename T>
__device__ __forceinline__ void store_row_vec(void* out, int64_t e0, const float* f, bool out_f32) {
  constexpr int VE = Vec<T>::N;
  if (sizeof(T) == 4 || out_f32) {
    float* o = static_cast<float*>(out) + e0;
#pragma unroll
    for (int q = 0; q < VE / 4; ++q) st_stream(o + 4 * q, make_uint4(__float_as_uint(f[4 * q]), __float_as_uint(f[4 * q + 1]), __float_as_uint(f[4 * q + 2]), __float_as_uint(f[4 * q + 3])));
  } else {
    st_stream(static_cast<T*>(out) + e0, narrow<T>(f));
  }
}

// Load VE weights (dtype TW) starting at element e0 as fp32; weights are re-read by
// every row, so they take the cached read-only path.
template <int VE, typename TW>
__device__ __forceinline__ void load_weights(const TW* w, int e0, float* f) {
  constexpr int PER = 16 / sizeof(TW);
#pragma unroll
  for (int q = 0; q < VE / PER; ++q) {
    widen<TW>(ld_keep(w + e0 + q * PER), f + q * PER);
  }
}

// ------------------------------------------------------------------ softmax, resident
// One row by one group of threads (a warp, or the whole CTA).
template <typename T, int VPT, bool WARP, bool IS_LOG>
__device__ __forceinline__ void softmax_row(const T* __restrict__ xr, void* __restrict__ out, int64_t out_e0, int nvec, int t, int tpr, int out_f32, float* red) {
  constexpr int VE = Vec<T>::N;
  float f[VPT][VE];
  float m = -CUDART_INF_F;
#pragma unroll
  for (int u = 0; u < VPT; ++u) {
    const int j = t + u * tpr;
    if (j < nvec) {
      widen<T>(ld_stream(xr + static_cast<int64_t>(j) * VE), f[u]);
#pragma unroll
      for (int e = 0; e < VE; ++e) m = fmaxf(m, f[u][e]);
    }
  }
  m = group_reduce<WARP>(m, MaxF{}, -CUDART_INF_F, red, 0);
  float s = 0.f;
  // softmax: 2^(x*log2(e) - c) with c = m*log2(e) rounded once; the rounding of c scales
  // every term of the row alike and cancels in the quotient. Not when c would overflow,
  // and not for log_softmax, which needs x - m itself.
  if (!IS_LOG && fabsf(m) < 1e37f) {
    const float c = m * kLog2e;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      if (t + u * tpr < nvec) {
#pragma unroll
        for (int e = 0; e < VE; ++e) {
          f[u][e] = ex2_approx(fmaf(f[u][e], kLog2e, -c));
          s += f[u][e];
        }
      }
    }
  } else {
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      if (t + u * tpr < nvec) {
#pragma unroll
        for (int e = 0; e < VE; ++e) {
          const float d = f[u][e] - m;
          const float ex = ex2_approx(d * kLog2e);
          s += ex;
          f[u][e] = IS_LOG ? d : ex;
        }
      }
    }
  }
  s = group_reduce<WARP>(s, SumF{}, 0.f, red, 1);
  const float k = IS_LOG ? logf(s) : 1.f / s;
#pragma unroll
  for (int u = 0; u < VPT; ++u) {
    const int j = t + u * tpr;
    if (j < nvec) {
#pragma unroll
      for (int e = 0; e < VE; ++e) f[u][e] = IS_LOG ? f[u][e] - k : f[u][e] * k;
      store_row_vec<T>(out, out_e0 + static_cast<int64_t>(j) * VE, f[u], out_f32 != 0);
    }
  }
}

template <typename T, int VPT, bool WARP, bool IS_LOG>
__global__ void __launch_bounds__(WARP ? 128 : 1024)
softmax_resident(const T* __restrict__ x, void* __restrict__ out, int64_t rows, int cols, int out_f32) {
  __shared__ float red[64];
  const int tpr = WARP ? 32 : blockDim.x;
  const int t = WARP ? (threadIdx.x & 31) : threadIdx.x;
  const int64_t row = WARP ? static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5) : blockIdx.x;
  if (WARP && row >= rows) return;
  softmax_row<T, VPT, WARP, IS_LOG>(x + row * cols, out, row * cols, cols / Vec<T>::N, t, tpr, out_f32, red);
}

// ------------------------------------------------------------------ softmax / log_softmax backward
// aten._softmax_backward_data:      gin = (g - sum(g * y)) * y
// aten._log_softmax_backward_data:  gin = g - exp(y) * sum(g)
// with y the forward output, along `dim` of [outer, dim, inner]. Resident kernel: the rows
// of g and y are read once with 16-byte loads and held in registers (one warp or one CTA
// per row), one reduction, one write -- the forward kernel's geometry with two inputs.
template <typename T, int VPT, bool WARP, bool IS_LOG>
__global__ void __launch_bounds__(WARP ? 128 : 1024)
softmax_bwd_resident(const T* __restrict__ g, const T* __restrict__ y, void* __restrict__ out, int64_t rows, int cols, int out_f32) {
  constexpr int VE = Vec<T>::N;
  __shared__ float red[64];
  const int tpr = WARP ? 32 : blockDim.x;
  const int t = WARP ? (threadIdx.x & 31) : threadIdx.x;
  const int64_t row = WARP ? static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5) : blockIdx.x;
  if (WARP && row >= rows) return;
  const int nvec = cols / VE;
  const T* gr = g + row * cols;
  const T* yr = y + row * cols;
  float fg[VPT][VE], fy[VPT][VE];
  float s = 0.f;
#pragma unroll
  for (int u = 0; u < VPT; ++u) {
    const int j = t + u * tpr;
    if (j < nvec) {
      widen<T>(ld_stream(gr + j * VE), fg[u]);
      widen<T>(ld_stream(yr + j * VE), fy[u]);
#pragma unroll
      for (int e = 0; e < VE; ++e) s += IS_LOG ? fg[u][e] : fg[u][e] * fy[u][e];
    }
  }
  s = group_reduce<WARP>(s, SumF{}, 0.f, red, 0);
#pragma unroll
  for (int u = 0; u < VPT; ++u) {
    const int j = t + u * tpr;
    if (j < nvec) {
#pragma unroll
      for (int e = 0; e < VE; ++e) fg[u][e] = IS_LOG ? fg[u][e] - ex2_approx(fy[u][e] * kLog2e) * s : (fg[u][e] - s) * fy[u][e];
      store_row_vec<T>(out, row * cols + static_cast<int64_t>(j) * VE, fg[u], out_f32 != 0);
    }
  }
}

// Any geometry and alignment: one warp per (outer, inner) line, elements `inner` apart,
// two passes over the line (the second from cache).
template <typename T, bool IS_LOG>
__global__ void __launch_bounds__(128) softmax_bwd_lines(const T* __restrict__ g, const T* __restrict__ y, void* __restrict__ out, int64_t outer, int64_t dim, int64_t inner, int dto) {
  const int lane = threadIdx.x & 31;
  const int64_t line = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (line >= outer * inner) return;
  const int64_t o = line / inner, i = line - o * inner, base = o * dim * inner + i;
  float s = 0.f;
  for (int64_t k = lane; k < dim; k += 32) s += IS_LOG ? to_f32(g[base + k * inner]) : to_f32(g[base + k * inner]) * to_f32(y[base + k * inner]);
  s = warp_reduce(s, SumF{});
  for (int64_t k = lane; k < dim; k += 32) {
    const float gv = to_f32(g[base + k * inner]), yv = to_f32(y[base + k * inner]);
    store_from_f32(out, base + k * inner, dto, IS_LOG ? gv - ex2_approx(yv * kLog2e) * s : (gv - s) * yv);
  }
}

// ------------------------------------------------------------------ softmax, streaming
// One CTA per row, three scalar passes (max, sum of exponentials, write); the second
// and third read come from L2. Any `cols`, any alignment. NaN / inf rows behave as in
// the resident kernel: the arithmetic is the same, only the data path differs.
template <typename T>
__global__ void __launch_bounds__(256) softmax_stream(const T* __restrict__ x, void* __restrict__ out, int64_t cols, int dto, int is_log) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * cols;
  float m = -CUDART_INF_F;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, to_f32(xr[c]));
  m = block_reduce(m, MaxF{}, -CUDART_INF_F, red);
  float s = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s += exp2f((to_f32(xr[c]) - m) * kLog2e);
  s = block_reduce(s, SumF{}, 0.f, red);
  const float k = is_log ? logf(s) : 1.f / s;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    const float d = to_f32(xr[c]) - m;
    store_from_f32(out, row * cols + c, dto, is_log ? d - k : exp2f(d * kLog2e) * k);
  }
}

// Long rows (more than the registers of a CTA hold) and rows whose start is off the 16-byte
// grid, with 16-byte accesses all the same: the CTA walks the aligned span that covers its
// row -- from `head` elements before the row's first element, inside the first element's
// own 16-byte block, to the end of the last element's block -- and masks what lies outside
// the row. Pass 1 keeps a running (max, sum of exponentials relative to it) per thread and
// merges them over the CTA; pass 2 re-reads the row (from L2 for rows up to some hundreds
// of KB), writes whole 16-byte vectors inside the row and single elements in the first and
// last block. Measured on vocabulary-size bf16 rows: 4.4-4.6 TB/s of 1 read + 1 write;
// prefetching through a cp.async ring gave the same, and holding the row in shared memory
// between the passes (one 1024-thread CTA per SM) was slower, 3.9 TB/s. The output row must sit at the same offset inside its 16-byte block as the
// input row and have the input's type. max.NaN makes a NaN element the maximum, hence the
// whole row NaN, as the three-pass kernel above does through its sum.
__device__ __forceinline__ float max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
// (m, s): s = sum of 2^((x - m) log2 e) over the elements seen; m = -inf means none yet (s = 0)
__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float mn = max_nan(m, m2);
  const float a = m == -CUDART_INF_F ? 0.f : s * ex2_approx((m - mn) * kLog2e);
  const float b = m2 == -CUDART_INF_F ? 0.f : s2 * ex2_approx((m2 - mn) * kLog2e);
  m = mn;
  s = a + b;
}
// one 16-byte vector into a thread's running (m, s); `masked`: the vector reaches outside the row
template <typename T, bool MASKED>
__device__ __forceinline__ void online_take(uint4 v, int j, int head, int cols, float& m, float& s) {
  constexpr int VE = Vec<T>::N;
  float f[VE];
  widen<T>(v, f);
  if (MASKED) {
    const int c0 = j * VE - head;
#pragma unroll
    for (int e = 0; e < VE; ++e)
      if (c0 + e < 0 || c0 + e >= cols) f[e] = -CUDART_INF_F;
  }
  float lm = f[0];
#pragma unroll
  for (int e = 1; e < VE; ++e) lm = max_nan(lm, f[e]);
  const float mn = max_nan(m, lm);
  if (mn != m) {  // a new maximum (or a NaN): bring the sum so far onto it; 0 * 2^-inf when there was none
    s *= ex2_approx((m - mn) * kLog2e);
    m = mn;
  }
  if (fabsf(m) < 1e37f) {  // 2^(x log2e - m log2e) in one fused multiply-add per element
    const float c = m * kLog2e;
#pragma unroll
    for (int e = 0; e < VE; ++e) s += ex2_approx(fmaf(f[e], kLog2e, -c));
  } else if (m != -CUDART_INF_F) {
#pragma unroll
    for (int e = 0; e < VE; ++e) s += ex2_approx((f[e] - m) * kLog2e);
  }
}
template <typename T, bool IS_LOG, bool MASKED>
__device__ __forceinline__ void online_write(uint4 v, T* __restrict__ orow, int j, int head, int cols, float m, float k, bool fused) {
  constexpr int VE = Vec<T>::N;
  float f[VE];
  widen<T>(v, f);
  if (fused) {  // |m| < 1e37: log: x - (m + log s); softmax: 2^(x log2e - m log2e) / s
    const float c = IS_LOG ? m + k : m * kLog2e;
#pragma unroll
    for (int e = 0; e < VE; ++e) f[e] = IS_LOG ? f[e] - c : ex2_approx(fmaf(f[e], kLog2e, -c)) * k;
  } else {
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      const float d = f[e] - m;
      f[e] = IS_LOG ? d - k : ex2_approx(d * kLog2e) * k;
    }
  }
  const int c0 = j * VE - head;
  if (!MASKED) {
    store_row_vec<T>(orow, c0, f, false);
  } else {
#pragma unroll
    for (int e = 0; e < VE; ++e)
      if (c0 + e >= 0 && c0 + e < cols) orow[c0 + e] = from_f32<T>(f[e]);
  }
}
template <typename T, bool IS_LOG>
__global__ void __launch_bounds__(1024) softmax_stream_vec(const T* __restrict__ x, T* __restrict__ out, int cols) {
  constexpr int VE = Vec<T>::N;
  __shared__ float red_m[32], red_s[32];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * cols;
  const int head = static_cast<int>((reinterpret_cast<uintptr_t>(xr) & 15u) / sizeof(T));
  const T* xa = xr - head;
  const int nvec = (head + cols + VE - 1) / VE;
  const int tid = threadIdx.x, nth = blockDim.x;
  const int last = nvec - 1;  // interior vectors are 1 .. last - 1: they never reach outside the row
  float m = -CUDART_INF_F, s = 0.f;
  if (tid == 0) online_take<T, true>(ld_keep(xa), 0, head, cols, m, s);
  if (tid == 32 && nvec > 1) online_take<T, true>(ld_keep(xa + static_cast<int64_t>(last) * VE), last, head, cols, m, s);
  for (int j = 1 + tid; j < last; j += nth) online_take<T, false>(ld_keep(xa + static_cast<int64_t>(j) * VE), j, head, cols, m, s);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) online_merge(m, s, __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
  const int lane = tid & 31, warp = tid >> 5, nwarps = nth >> 5;
  if (lane == 0) { red_m[warp] = m; red_s[warp] = s; }
  __syncthreads();
  m = lane < nwarps ? red_m[lane] : -CUDART_INF_F;
  s = lane < nwarps ? red_s[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) online_merge(m, s, __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
  const float k = IS_LOG ? logf(s) : 1.f / s;
  const bool fused = fabsf(m) < 1e37f && (!IS_LOG || fabsf(k) < 1e37f);
  T* orow = out + row * cols;
  if (tid == 0) online_write<T, IS_LOG, true>(ld_stream(xa), orow, 0, head, cols, m, k, fused);
  if (tid == 32 && nvec > 1) online_write<T, IS_LOG, true>(ld_stream(xa + static_cast<int64_t>(last) * VE), orow, last, head, cols, m, k, fused);
  for (int j = 1 + tid; j < last; j += nth) online_write<T, IS_LOG, false>(ld_stream(xa + static_cast<int64_t>(j) * VE), orow, j, head, cols, m, k, fused);
}

// ------------------------------------------------------------------ ragged rows, one warp each
// Rows of 33 ... 32 * NPL elements whose length or base is off the 16-byte grid (the vector
// kernels cannot take them, and a CTA per row would idle most of its threads): a warp reads
// its row with coalesced scalar loads, lane l holding elements l, l + 32, ..., in registers,
// and does the same arithmetic as the resident kernels.
template <typename T, int NPL, bool IS_LOG>
__global__ void __launch_bounds__(128) softmax_warp_ragged(const T* __restrict__ x, void* __restrict__ out, int64_t rows, int cols, int dto) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * cols;
  float f[NPL];
  float m = -CUDART_INF_F;
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int c = lane + 32 * i;
    f[i] = c < cols ? to_f32(xr[c]) : -CUDART_INF_F;
    m = fmaxf(m, f[i]);
  }
  m = warp_reduce(m, MaxF{});
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const float d = f[i] - m;
    const float ex = lane + 32 * i < cols ? ex2_approx(d * kLog2e) : 0.f;
    s += ex;
    f[i] = IS_LOG ? d : ex;
  }
  s = warp_reduce(s, SumF{});
  const float k = IS_LOG ? logf(s) : 1.f / s;
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int c = lane + 32 * i;
    if (c < cols) store_from_f32(out, row * cols + c, dto, IS_LOG ? f[i] - k : f[i] * k);
  }
}

template <typename T, int NPL>
__global__ void __launch_bounds__(128) layernorm_warp_ragged(const T* __restrict__ x, const void* __restrict__ w, const void* __restrict__ b, T* __restrict__ y, void* __restrict__ mean,
                                                             void* __restrict__ rstd, int64_t rows, int cols, float eps, int dt_wb, int dt_stat) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * cols;
  float f[NPL];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int c = lane + 32 * i;
    f[i] = c < cols ? to_f32(xr[c]) : 0.f;
    s += f[i];
  }
  s = warp_reduce(s, SumF{});
  float mu = s / static_cast<float>(cols);
  if (!isfinite(mu)) mu = CUDART_NAN_F;  // same non-finite rule as the resident kernel
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const float d = lane + 32 * i < cols ? f[i] - mu : 0.f;
    q = fmaf(d, d, q);
  }
  q = warp_reduce(q, SumF{});
  const float rs = rsqrtf(q / static_cast<float>(cols) + eps);
  if (lane == 0) {
    store_from_f32(mean, row, dt_stat, mu);
    store_from_f32(rstd, row, dt_stat, rs);
  }
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int c = lane + 32 * i;
    if (c < cols) {
      float r = (f[i] - mu) * rs;
      if (w) r *= load_as_f32(w, c, dt_wb);
      if (b) r += load_as_f32(b, c, dt_wb);
      y[row * cols + c] = from_f32<T>(r);
    }
  }
}

// NPL for a ragged row of `cols` elements: 2, 4, ..., 32 elements per lane (cols <= 1024)
#define B200_DISPATCH_NPL(COLS, BODY)                       \
  if ((COLS) <= 64) { constexpr int NPL = 2; BODY; }        \
  else if ((COLS) <= 128) { constexpr int NPL = 4; BODY; }  \
  else if ((COLS) <= 256) { constexpr int NPL = 8; BODY; }  \
  else if ((COLS) <= 512) { constexpr int NPL = 16; BODY; } \
  else { constexpr int NPL = 32; BODY; }
constexpr int kRaggedMaxCols = 1024;

// ------------------------------------------------------------------ softmax, inner > 1
template <typename T>
__global__ void __launch_bounds__(128) softmax_cols(const T* __restrict__ x, void* __restrict__ out, int64_t dim, int64_t inner, int dto, int is_log) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= inner) return;
  const int64_t base = static_cast<int64_t>(blockIdx.y) * dim * inner + i;
  float m = -CUDART_INF_F;
  for (int64_t k = 0; k < dim; ++k) m = fmaxf(m, to_f32(x[base + k * inner]));
  float s = 0.f;
  for (int64_t k = 0; k < dim; ++k) s += exp2f((to_f32(x[base + k * inner]) - m) * kLog2e);
  const float kk = is_log ? logf(s) : 1.f / s;
  for (int64_t k = 0; k < dim; ++k) {
    const float d = to_f32(x[base + k * inner]) - m;
    store_from_f32(out, base + k * inner, dto, is_log ? d - kk : exp2f(d * kLog2e) * kk);
  }
}

// ------------------------------------------------------------------ layer norm, resident
// HOLD: the row is widened to fp32 once and held in registers (VE floats per vector);
// otherwise it stays in its storage type (16 bytes per vector) and is widened again in
// each of the three passes, which for 16-bit rows halves the registers held across the two
// reductions. AFFINE: weight and bias are both present (the usual call), so the last pass
// is one fused multiply-add per element with no per-element tests.
template <typename T, typename TW, int VPT, bool WARP, bool HOLD, bool AFFINE>
__global__ void __launch_bounds__(WARP ? 128 : 1024)
layernorm_resident(const T* __restrict__ x, const TW* __restrict__ w, const TW* __restrict__ b, T* __restrict__ y,
                   void* __restrict__ mean, void* __restrict__ rstd, int64_t rows, int cols, float inv_cols, float eps, int dt_stat) {
  constexpr int VE = Vec<T>::N;
  __shared__ float red[64];
  const int tpr = WARP ? 32 : blockDim.x;
  const int t = WARP ? (threadIdx.x & 31) : threadIdx.x;
  const int64_t row = WARP ? static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5) : blockIdx.x;
  if (WARP && row >= rows) return;
  const int nvec = cols / VE;
  const T* xr = x + row * cols;
  T* yr = y + row * cols;
  uint4 raw[HOLD ? 1 : VPT];
  float f[HOLD ? VPT : 1][VE];
  float s = 0.f;
  if (HOLD) {
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const int j = t + u * tpr;
      if (j < nvec) {
        widen<T>(ld_stream(xr + j * VE), f[HOLD ? u : 0]);
#pragma unroll
        for (int e = 0; e < VE; ++e) s += f[HOLD ? u : 0][e];
      }
    }
  } else {
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const int j = t + u * tpr;
      if (j < nvec) raw[HOLD ? 0 : u] = ld_stream(xr + j * VE);
    }
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      if (t + u * tpr < nvec) vec_accumulate<T>(s, raw[HOLD ? 0 : u]);
    }
  }
  s = group_reduce<WARP>(s, SumF{}, 0.f, red, 0);
  float mu = s * inv_cols;
  // a row holding NaN or inf has NaN statistics in aten (its running moments turn inf
  // into NaN once another element follows), not mean = inf
  if (!isfinite(mu)) mu = CUDART_NAN_F;
  float q = 0.f;
#pragma unroll
  for (int u = 0; u < VPT; ++u) {
    if (t + u * tpr < nvec) {
      float d[VE];
      if (HOLD) {
#pragma unroll
        for (int e = 0; e < VE; ++e) d[e] = f[HOLD ? u : 0][e] - mu;
      } else {
        vec_minus<T>(raw[HOLD ? 0 : u], mu, d);
      }
#pragma unroll
      for (int e = 0; e < VE; ++e) q = fmaf(d[e], d[e], q);
    }
  }
  q = group_reduce<WARP>(q, SumF{}, 0.f, red, 1);
  const float rs = rsqrtf(fmaf(q, inv_cols, eps));
  if (t == 0) {
    store_from_f32(mean, row, dt_stat, mu);
    store_from_f32(rstd, row, dt_stat, rs);
  }
#pragma unroll
  for (int u = 0; u < VPT; ++u) {
    const int j = t + u * tpr;
    if (j < nvec) {
      float o[VE], wv[VE], bv[VE], d[VE];
      if (HOLD) {
#pragma unroll
        for (int e = 0; e < VE; ++e) d[e] = f[HOLD ? u : 0][e] - mu;
      } else {
        vec_minus<T>(raw[HOLD ? 0 : u], mu, d);
      }
      if (AFFINE || w) load_weights<VE, TW>(w, j * VE, wv);
      if (AFFINE || b) load_weights<VE, TW>(b, j * VE, bv);
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        float r = d[e] * rs;
        if (AFFINE) {
          r = fmaf(r, wv[e], bv[e]);
        } else {
          if (w) r *= wv[e];
          if (b) r += bv[e];
        }
        o[e] = r;
      }
      st_stream(yr + j * VE, narrow<T>(o));
    }
  }
}

// The same for many 16-bit rows with weight and bias: persistent CTAs. A thread owns the same
// columns of every row its CTA sees, so it widens its share of weight and bias ONCE (the
// per-row kernel above fetched and unpacked 16 KB of them for every 8 KB row: two of its
// eighteen instructions per element, and more L2-to-SM traffic than the rows themselves), and
// the next row's vectors are requested before this row's two reductions.
template <typename T, typename TW, int VPT>
__global__ void __launch_bounds__(256, 4)
layernorm_persistent(const T* __restrict__ x, const TW* __restrict__ w, const TW* __restrict__ b, T* __restrict__ y, void* __restrict__ mean, void* __restrict__ rstd, int64_t rows, int cols,
                     float inv_cols, float eps, int dt_stat) {
  constexpr int VE = Vec<T>::N;
  __shared__ float red[64];
  const int t = threadIdx.x, tpr = blockDim.x;
  const int nvec = cols / VE;
  float wv[VPT][VE], bv[VPT][VE];
#pragma unroll
  for (int u = 0; u < VPT; ++u) {
    const int j = t + u * tpr;
    if (j < nvec) {
      load_weights<VE, TW>(w, j * VE, wv[u]);
      load_weights<VE, TW>(b, j * VE, bv[u]);
    }
  }
  uint4 nxt[VPT];
  int64_t row = blockIdx.x;
  if (row < rows) {
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const int j = t + u * tpr;
      if (j < nvec) nxt[u] = ld_stream(x + row * cols + j * VE);
    }
  }
  for (; row < rows; row += gridDim.x) {
    // the row stays packed (16 bytes per vector) and is widened again in each of the three
    // passes: held as fp32 it costs a CTA per SM (three instead of four) and ran 7 % slower
    uint4 raw[VPT];
#pragma unroll
    for (int u = 0; u < VPT; ++u) raw[u] = nxt[u];
    const int64_t nrow = row + gridDim.x;
    if (nrow < rows) {
#pragma unroll
      for (int u = 0; u < VPT; ++u) {
        const int j = t + u * tpr;
        if (j < nvec) nxt[u] = ld_stream(x + nrow * cols + j * VE);
      }
    }
    float s = 0.f;
#pragma unroll
    for (int u = 0; u < VPT; ++u)
      if (t + u * tpr < nvec) vec_accumulate<T>(s, raw[u]);
    s = block_reduce_once(s, SumF{}, 0.f, red, 0);
    float mu = s * inv_cols;
    if (!isfinite(mu)) mu = CUDART_NAN_F;  // as the per-row kernel: NaN statistics for a row holding NaN or inf
    float q = 0.f;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      if (t + u * tpr < nvec) {
        float d[VE];
        vec_minus<T>(raw[u], mu, d);
#pragma unroll
        for (int e = 0; e < VE; ++e) q = fmaf(d[e], d[e], q);
      }
    }
    q = block_reduce_once(q, SumF{}, 0.f, red, 1);
    const float rs = rsqrtf(fmaf(q, inv_cols, eps));
    if (t == 0) {
      store_from_f32(mean, row, dt_stat, mu);
      store_from_f32(rstd, row, dt_stat, rs);
    }
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const int j = t + u * tpr;
      if (j < nvec) {
        float d[VE], o[VE];
        vec_minus<T>(raw[u], mu, d);
#pragma unroll
        for (int e = 0; e < VE; ++e) o[e] = fmaf(d[e] * rs, wv[u][e], bv[u][e]);
        st_stream(y + row * cols + j * VE, narrow<T>(o));
      }
    }
  }
}

// ------------------------------------------------------------------ layer norm backward
// aten.native_layer_norm_backward: with xhat = (x - mean) * rstd and gy = dy * w per row,
//   dx = rstd * (gy - mean_j(gy) - xhat * mean_j(gy * xhat))
//   dw = sum_rows dy * xhat,  db = sum_rows dy.
// Fused kernel (row length a multiple of the 16-byte vector, everything aligned): persistent
// CTAs, one row at a time per CTA; a thread owns the same columns of every row it sees, so it
// carries its share of dw / db in registers across rows and writes one partial per CTA at
// the end (dy and x are read once for all three results). A small second kernel adds the
// per-CTA partials in order. fp32 arithmetic throughout.
template <typename T, typename TW, int VPT>
__global__ void __launch_bounds__(1024)
layernorm_bwd_fused(const T* __restrict__ dy, const T* __restrict__ x, const TW* __restrict__ w, const void* __restrict__ mean, const void* __restrict__ rstd, T* __restrict__ dx,
                    float* __restrict__ part_w, float* __restrict__ part_b, int64_t rows, int cols, int dt_stat) {
  constexpr int VE = Vec<T>::N;
  __shared__ float red[64];
  const int t = threadIdx.x, tpr = blockDim.x;
  const int nvec = cols / VE;
  const float inv_cols = 1.f / static_cast<float>(cols);
  float wv[VPT][VE], aw[VPT][VE], ab[VPT][VE];
#pragma unroll
  for (int u = 0; u < VPT; ++u) {
    const int j = t + u * tpr;
#pragma unroll
    for (int e = 0; e < VE; ++e) { wv[u][e] = 1.f; aw[u][e] = 0.f; ab[u][e] = 0.f; }
    if (w && j < nvec) load_weights<VE, TW>(w, j * VE, wv[u]);
  }
  // the vectors of the next row are requested before this row is worked on: twice the bytes in flight per thread
  uint4 ndy[VPT], nx[VPT];
  if (static_cast<int64_t>(blockIdx.x) < rows) {
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const int j = t + u * tpr;
      if (j < nvec) {
        ndy[u] = ld_stream(dy + static_cast<int64_t>(blockIdx.x) * cols + j * VE);
        nx[u] = ld_stream(x + static_cast<int64_t>(blockIdx.x) * cols + j * VE);
      }
    }
  }
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mu = load_as_f32(mean, row, dt_stat), rs = load_as_f32(rstd, row, dt_stat);
    float g[VPT][VE], h[VPT][VE];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      widen<T>(ndy[u], g[u]);
      widen<T>(nx[u], h[u]);
    }
    const int64_t next = row + gridDim.x;
    if (next < rows) {
#pragma unroll
      for (int u = 0; u < VPT; ++u) {
        const int j = t + u * tpr;
        if (j < nvec) {
          ndy[u] = ld_stream(dy + next * cols + j * VE);
          nx[u] = ld_stream(x + next * cols + j * VE);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const int j = t + u * tpr;
      if (j < nvec) {
#pragma unroll
        for (int e = 0; e < VE; ++e) {
          const float xhat = (h[u][e] - mu) * rs;
          ab[u][e] += g[u][e];
          aw[u][e] = fmaf(g[u][e], xhat, aw[u][e]);
          const float gy = g[u][e] * wv[u][e];
          s1 += gy;
          s2 = fmaf(gy, xhat, s2);
          g[u][e] = gy;
          h[u][e] = xhat;
        }
      }
    }
    s1 = block_reduce_once(s1, SumF{}, 0.f, red, 0);
    s2 = block_reduce_once(s2, SumF{}, 0.f, red, 1);
    const float c1 = s1 * inv_cols, c2 = s2 * inv_cols;
    if (dx) {
#pragma unroll
      for (int u = 0; u < VPT; ++u) {
        const int j = t + u * tpr;
        if (j < nvec) {
          float o[VE];
#pragma unroll
          for (int e = 0; e < VE; ++e) o[e] = rs * (g[u][e] - c1 - h[u][e] * c2);
          st_stream(dx + row * cols + j * VE, narrow<T>(o));
        }
      }
    }
  }
  if (part_w) {
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const int j = t + u * tpr;
      if (j < nvec) {
        float* pw = part_w + static_cast<int64_t>(blockIdx.x) * cols + j * VE;
        float* pb = part_b + static_cast<int64_t>(blockIdx.x) * cols + j * VE;
#pragma unroll
        for (int e = 0; e < VE; ++e) { pw[e] = aw[u][e]; pb[e] = ab[u][e]; }
      }
    }
  }
}

// Any row length and alignment. dx: one CTA per row, scalar, three passes (the second and
// third from cache). dw / db partials: one thread per column walking a chunk of rows
// (coalesced across columns), one partial row per chunk.
__global__ void __launch_bounds__(256) layernorm_bwd_dx_lines(const void* __restrict__ dy, const void* __restrict__ x, const void* __restrict__ w, const void* __restrict__ mean,
                                                              const void* __restrict__ rstd, void* __restrict__ dx, int64_t rows, int64_t cols, int dt, int dt_wb, int dt_stat) {
  __shared__ float red[64];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mu = load_as_f32(mean, row, dt_stat), rs = load_as_f32(rstd, row, dt_stat);
    const int64_t base = row * cols;
    float s1 = 0.f, s2 = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
      const float gy = load_as_f32(dy, base + c, dt) * (w ? load_as_f32(w, c, dt_wb) : 1.f);
      s1 += gy;
      s2 = fmaf(gy, (load_as_f32(x, base + c, dt) - mu) * rs, s2);
    }
    __syncthreads();  // the reduction buffers of the row before are free
    s1 = block_reduce_once(s1, SumF{}, 0.f, red, 0);
    s2 = block_reduce_once(s2, SumF{}, 0.f, red, 1);
    const float c1 = s1 / static_cast<float>(cols), c2 = s2 / static_cast<float>(cols);
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
      const float gy = load_as_f32(dy, base + c, dt) * (w ? load_as_f32(w, c, dt_wb) : 1.f);
      const float xhat = (load_as_f32(x, base + c, dt) - mu) * rs;
      store_from_f32(dx, base + c, dt, rs * (gy - c1 - xhat * c2));
    }
  }
}
__global__ void __launch_bounds__(256) layernorm_bwd_wb_lines(const void* __restrict__ dy, const void* __restrict__ x, const void* __restrict__ mean, const void* __restrict__ rstd,
                                                              float* __restrict__ part_w, float* __restrict__ part_b, int64_t rows, int64_t cols, int64_t rows_per, int dt, int dt_stat) {
  const int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * rows_per, r1 = r0 + rows_per < rows ? r0 + rows_per : rows;
  float aw = 0.f, ab = 0.f;
  for (int64_t r = r0; r < r1; ++r) {
    const float g = load_as_f32(dy, r * cols + c, dt);
    ab += g;
    aw = fmaf(g, (load_as_f32(x, r * cols + c, dt) - load_as_f32(mean, r, dt_stat)) * load_as_f32(rstd, r, dt_stat), aw);
  }
  part_w[static_cast<int64_t>(blockIdx.y) * cols + c] = aw;
  part_b[static_cast<int64_t>(blockIdx.y) * cols + c] = ab;
}
// dw[c] = sum over the `parts` partial rows, same for db: a CTA takes 32 columns, its 32
// warps take every 32nd partial row each (coalesced 128-byte reads), and the 32 slice sums
// of a column are added in slice order -- a fixed order, so the result is reproducible.
__global__ void __launch_bounds__(1024) layernorm_bwd_finalize(const float* __restrict__ part_w, const float* __restrict__ part_b, void* __restrict__ dw, void* __restrict__ db, int64_t parts,
                                                               int64_t cols, int dt_wb) {
  __shared__ float sw[32][33], sb[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t c = static_cast<int64_t>(blockIdx.x) * 32 + tx;
  float aw = 0.f, ab = 0.f;
  if (c < cols)
    for (int64_t p = ty; p < parts; p += 32) {
      aw += part_w[p * cols + c];
      ab += part_b[p * cols + c];
    }
  sw[ty][tx] = aw;
  sb[ty][tx] = ab;
  __syncthreads();
  if (ty == 0 && c < cols) {
    float tw = 0.f, tb = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      tw += sw[k][tx];
      tb += sb[k][tx];
    }
    if (dw) store_from_f32(dw, c, dt_wb, tw);
    if (db) store_from_f32(db, c, dt_wb, tb);
  }
}

// layer norm, streaming: one CTA per row, three scalar passes (second and third from L2).
__global__ void __launch_bounds__(256) layernorm_stream(const void* __restrict__ x, const void* __restrict__ w, const void* __restrict__ b, void* __restrict__ y,
                                                        void* __restrict__ mean, void* __restrict__ rstd, int64_t cols, float eps, int dt, int dt_wb, int dt_stat) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x, base = row * cols;
  float s = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s += load_as_f32(x, base + c, dt);
  s = block_reduce(s, SumF{}, 0.f, red);
  float mu = s / static_cast<float>(cols);
  if (!isfinite(mu)) mu = CUDART_NAN_F;  // same non-finite rule as the resident kernel
  float q = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    const float d = load_as_f32(x, base + c, dt) - mu;
    q = fmaf(d, d, q);
  }
  q = block_reduce(q, SumF{}, 0.f, red);
  const float rs = rsqrtf(q / static_cast<float>(cols) + eps);
  if (threadIdx.x == 0) {
    store_from_f32(mean, row, dt_stat, mu);
    store_from_f32(rstd, row, dt_stat, rs);
  }
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    float r = (load_as_f32(x, base + c, dt) - mu) * rs;
    if (w) r *= load_as_f32(w, c, dt_wb);
    if (b) r += load_as_f32(b, c, dt_wb);
    store_from_f32(y, base + c, dt, r);
  }
}

// ------------------------------------------------------------------ sum / argmax
// argmax order: NaN beats everything, then larger value, then smaller index.
struct ArgPair {
  float v;
  int64_t i;
};
__device__ __forceinline__ bool arg_better(float v, int64_t i, float bv, int64_t bi) {
  const bool vn = v != v, bn = bv != bv;
  if (vn || bn) return vn && (!bn || i < bi);
  return v > bv || (v == bv && i < bi);
}
__device__ __forceinline__ void arg_take(ArgPair& a, float v, int64_t i) {
  if (a.i < 0 || arg_better(v, i, a.v, a.i)) { a.v = v; a.i = i; }
}
// Streaming form for a thread that visits its elements in ASCENDING index order: one
// compare per element on the common path. `v <= best` is false when v is larger, when v is
// NaN, or when best is already NaN; only then the slow test runs (a NaN best is final:
// the first NaN wins; otherwise v is larger or NaN and, being the earliest such, is taken).
__device__ __forceinline__ void arg_take_ascending(ArgPair& a, float v, int64_t i) {
  if (!(v <= a.v)) {
    if (a.i < 0 || a.v == a.v) { a.v = v; a.i = i; }
  }
}
// A whole vector of consecutive elements at once: when none of them exceeds the best so far
// and none is NaN, nothing changes and no index is computed. The largest element is found
// with fmaxf, which skips NaN, so the sum of the vector stands guard for it (a sum that is
// NaN without a NaN element, +inf with -inf, only sends the vector the long way).
template <int VE>
__device__ __forceinline__ void arg_take_vector(ArgPair& a, const float* fw, int64_t i0) {
  float m = fw[0], s = fw[0];
#pragma unroll
  for (int e = 1; e < VE; ++e) {
    m = fmaxf(m, fw[e]);
    s += fw[e];
  }
  if (m <= a.v && s == s && a.i >= 0) return;
#pragma unroll
  for (int e = 0; e < VE; ++e) arg_take_ascending(a, fw[e], i0 + e);
}
__device__ __forceinline__ ArgPair arg_warp_reduce(ArgPair a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float v = __shfl_xor_sync(0xffffffffu, a.v, o);
    const int64_t i = __shfl_xor_sync(0xffffffffu, a.i, o);
    if (i >= 0) arg_take(a, v, i);
  }
  return a;
}

// Row reduction (inner == 1). grid = (row groups, splits). A row's [c0, c1) slice of
// split blockIdx.y is consumed by one warp (WARP) or one CTA with 16-byte loads when
// VECOK (row pitch and base 16-byte aligned), else scalar loads.
template <typename T, bool WARP, bool ARG, bool VECOK>
__global__ void __launch_bounds__(256) reduce_rows(const T* __restrict__ x, void* __restrict__ out, float* __restrict__ part_v, int64_t* __restrict__ part_i,
                                                   int64_t rows, int64_t cols, int64_t chunk, int dto) {
  constexpr int VE = Vec<T>::N;
  __shared__ float red[33];
  __shared__ float av[32];
  __shared__ int64_t ai[32];
  const int tpr = WARP ? 32 : blockDim.x;
  const int t = WARP ? (threadIdx.x & 31) : threadIdx.x;
  const int64_t row = WARP ? static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5) : blockIdx.x;
  if (WARP && row >= rows) return;
  const int64_t c0 = static_cast<int64_t>(blockIdx.y) * chunk;
  const int64_t c1 = c0 + chunk < cols ? c0 + chunk : cols;
  const T* xr = x + row * cols;
  float s = 0.f;
  ArgPair a{CUDART_NAN_F, -1};  // NaN start: the first element fails `v <= NaN` and is taken through a.i < 0
  if (VECOK) {
    // chunk is a multiple of VE, so every slice starts on a vector boundary
    const int64_t v0 = c0 / VE, v1 = c1 / VE;
    int64_t j = v0 + t;
    for (; j + 3 * tpr < v1; j += 4 * tpr) {
      Vec<T> v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u].raw = ld_stream(xr + (j + u * tpr) * VE);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (ARG) {
          float fw[VE];
          widen<T>(v[u].raw, fw);
          arg_take_vector<VE>(a, fw, (j + u * tpr) * VE);
        } else {
          vec_accumulate<T>(s, v[u].raw);  // 16-bit elements are widened inside the add
        }
      }
    }
    for (; j < v1; j += tpr) {
      const uint4 raw = ld_stream(xr + j * VE);
      if (ARG) {
        float fw[VE];
        widen<T>(raw, fw);
        arg_take_vector<VE>(a, fw, j * VE);
      } else {
        vec_accumulate<T>(s, raw);
      }
    }
    for (int64_t c = v1 * VE + t; c < c1; c += tpr) {  // ragged end of the last slice
      const float fv = to_f32(xr[c]);
      if (ARG) arg_take_ascending(a, fv, c);
      else s += fv;
    }
  } else {
    for (int64_t c = c0 + t; c < c1; c += tpr) {
      const float fv = to_f32(xr[c]);
      if (ARG) arg_take_ascending(a, fv, c);
      else s += fv;
    }
  }
  const bool split = gridDim.y > 1;
  const int64_t slot = static_cast<int64_t>(blockIdx.y) * rows + row;
  if (!ARG) {
    s = WARP ? warp_reduce(s, SumF{}) : block_reduce(s, SumF{}, 0.f, red);
    if (t == 0) {
      if (split) part_v[slot] = s;
      else store_from_f32(out, row, dto, s);
    }
  } else {
    a = arg_warp_reduce(a);
    if (!WARP) {
      const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
      if (lane == 0) { av[warp] = a.v; ai[warp] = a.i; }
      __syncthreads();
      if (warp == 0) {
        a.v = lane < (blockDim.x >> 5) ? av[lane] : 0.f;
        a.i = lane < (blockDim.x >> 5) ? ai[lane] : -1;
        a = arg_warp_reduce(a);
      }
    }
    if (threadIdx.x == 0 || (WARP && t == 0)) {
      if (split) { part_v[slot] = a.v; part_i[slot] = a.i; }
      else static_cast<int64_t*>(out)[row] = a.i;
    }
  }
}

// Column reduction (inner > 1): thread per inner element, grid = (inner tiles, outer, splits).
template <typename T, bool ARG>
__global__ void __launch_bounds__(256) reduce_cols(const T* __restrict__ x, void* __restrict__ out, float* __restrict__ part_v, int64_t* __restrict__ part_i,
                                                   int64_t outer, int64_t dim, int64_t inner, int64_t chunk, int dto) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= inner) return;
  const int64_t o = blockIdx.y;
  const int64_t k0 = static_cast<int64_t>(blockIdx.z) * chunk;
  const int64_t k1 = k0 + chunk < dim ? k0 + chunk : dim;
  const T* p = x + o * dim * inner + i;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  ArgPair a{0.f, -1};
  int64_t k = k0;
  if (!ARG) {
    for (; k + 3 < k1; k += 4) {
      s0 += to_f32(p[k * inner]);
      s1 += to_f32(p[(k + 1) * inner]);
      s2 += to_f32(p[(k + 2) * inner]);
      s3 += to_f32(p[(k + 3) * inner]);
    }
  } else {
    for (; k + 7 < k1; k += 8) {  // eight rows requested before the first comparison
      T f[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) f[u] = p[(k + u) * inner];
#pragma unroll
      for (int u = 0; u < 8; ++u) arg_take(a, to_f32(f[u]), k + u);
    }
  }
  for (; k < k1; ++k) {
    const float fv = to_f32(p[k * inner]);
    if (ARG) arg_take(a, fv, k);
    else s0 += fv;
  }
  const float s = (s0 + s1) + (s2 + s3);
  const int64_t oi = o * inner + i;
  if (gridDim.z > 1) {
    const int64_t slot = static_cast<int64_t>(blockIdx.z) * outer * inner + oi;
    if (ARG) { part_v[slot] = a.v; part_i[slot] = a.i; }
    else part_v[slot] = s;
  } else {
    if (ARG) static_cast<int64_t*>(out)[oi] = a.i;
    else store_from_f32(out, oi, dto, s);
  }
}

// Column reduction with at most 32 columns (the bias-gradient shape: many rows, few columns):
// a thread per column would leave most lanes of a warp without work, so the lanes of a warp
// tile rows x columns instead -- W = the next power of two above `inner` columns, 32 / W rows
// per warp and trip, i.e. a warp reads 32 consecutive elements when inner == W -- and the
// row-lanes are folded by shuffles, the CTA's 8 warps through shared memory, in a fixed order.
template <typename T, bool ARG>
__global__ void __launch_bounds__(256) reduce_cols_narrow(const T* __restrict__ x, void* __restrict__ out, float* __restrict__ part_v, int64_t* __restrict__ part_i,
                                                          int64_t outer, int64_t dim, int inner, int W, int64_t chunk, int dto) {
  __shared__ float sh_v[8][32];
  __shared__ int64_t sh_i[ARG ? 8 : 1][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = lane & (W - 1), rsub = lane / W, rpw = 32 / W;
  const int64_t o = blockIdx.y;
  const int64_t k0 = static_cast<int64_t>(blockIdx.z) * chunk;
  const int64_t k1 = k0 + chunk < dim ? k0 + chunk : dim;
  const T* p = x + o * dim * inner + col;
  const int64_t step = 8 * rpw;
  float s0 = 0.f, s1 = 0.f;
  ArgPair a{0.f, -1};
  if (col < inner) {
    int64_t k = k0 + warp * rpw + rsub;
    if (!ARG) {
      for (; k + step < k1; k += 2 * step) {
        s0 += to_f32(p[k * inner]);
        s1 += to_f32(p[(k + step) * inner]);
      }
    }
    for (; k < k1; k += step) {
      const float fv = to_f32(p[k * inner]);
      if (ARG) arg_take(a, fv, k);
      else s0 += fv;
    }
  }
  float s = s0 + s1;
  for (int off = W; off < 32; off <<= 1) {  // fold the row-lanes of the warp onto lanes 0 .. W-1
    if (ARG) {
      const float v = __shfl_xor_sync(0xffffffffu, a.v, off);
      const int64_t i = __shfl_xor_sync(0xffffffffu, a.i, off);
      if (i >= 0) arg_take(a, v, i);
    } else {
      s += __shfl_xor_sync(0xffffffffu, s, off);
    }
  }
  if (lane < W) {
    sh_v[warp][lane] = ARG ? a.v : s;
    if (ARG) sh_i[warp][lane] = a.i;
  }
  __syncthreads();
  if (warp == 0 && lane < inner) {
    float t = 0.f;
    ArgPair b{0.f, -1};
    for (int w = 0; w < 8; ++w) {
      if (ARG) { if (sh_i[w][lane] >= 0) arg_take(b, sh_v[w][lane], sh_i[w][lane]); }
      else t += sh_v[w][lane];
    }
    const int64_t oi = o * inner + lane;
    if (gridDim.z > 1) {
      const int64_t slot = static_cast<int64_t>(blockIdx.z) * outer * inner + oi;
      if (ARG) { part_v[slot] = b.v; part_i[slot] = b.i; }
      else part_v[slot] = t;
    } else {
      if (ARG) static_cast<int64_t*>(out)[oi] = b.i;
      else store_from_f32(out, oi, dto, t);
    }
  }
}

// Second stage of a split reduction: n outputs, `splits` partials each, ascending split
// order (so the earliest index wins argmax ties and sums are run-to-run identical).
template <bool ARG>
__global__ void __launch_bounds__(256) reduce_finalize(const float* __restrict__ part_v, const int64_t* __restrict__ part_i, void* __restrict__ out, int64_t n, int splits, int dto) {
  const int64_t o = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (o >= n) return;
  // eight partials are requested before the first one is combined: a thread that waited for
  // each in turn spent a round trip to L2 per partial (1059 x 3072 argmax over dim 0: 12 us)
  if (ARG) {
    ArgPair a{0.f, -1};
    for (int s0 = 0; s0 < splits; s0 += 8) {
      int64_t i[8];
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const bool in = s0 + u < splits;
        i[u] = in ? part_i[(s0 + u) * n + o] : -1;
        v[u] = in ? part_v[(s0 + u) * n + o] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (i[u] >= 0) arg_take(a, v[u], i[u]);
    }
    static_cast<int64_t*>(out)[o] = a.i;
  } else {
    float s = 0.f;
    for (int k0 = 0; k0 < splits; k0 += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = k0 + u < splits ? part_v[(k0 + u) * n + o] : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (k0 + u < splits) s += v[u];  // the same order of additions as one by one
    }
    store_from_f32(out, o, dto, s);
  }
}

// The same with one warp per output, for many partials of few outputs (a whole-tensor
// reduction): lanes take partials s = lane, lane + 32, ... and combine by shuffles. The
// order of the additions is fixed by (lane, shuffle tree), so sums stay run-to-run
// identical; argmax combines by (NaN, value, index), which is order-free.
template <bool ARG>
__global__ void __launch_bounds__(256) reduce_finalize_warp(const float* __restrict__ part_v, const int64_t* __restrict__ part_i, void* __restrict__ out, int64_t n, int splits, int dto) {
  const int64_t o = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (o >= n) return;
  if (ARG) {
    ArgPair a{0.f, -1};
    for (int s = lane; s < splits; s += 32) {
      const int64_t i = part_i[s * n + o];
      if (i >= 0) arg_take(a, part_v[s * n + o], i);
    }
    a = arg_warp_reduce(a);
    if (lane == 0) static_cast<int64_t*>(out)[o] = a.i;
  } else {
    float s = 0.f;
    for (int k = lane; k < splits; k += 32) s += part_v[k * n + o];
    s = warp_reduce(s, SumF());
    if (lane == 0) store_from_f32(out, o, dto, s);
  }
}

__global__ void fill_zero_typed(void* out, int64_t n, int dto) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) store_from_f32(out, i, dto, 0.f);
}

// ------------------------------------------------------------------ very short rows (dim <= 32, inner == 1)
// Millions of rows of a handful of elements: one THREAD per row, the row in registers (NC
// slots, the next multiple of 8 above the row length). A CTA owns 256 consecutive rows, one
// contiguous span of memory, and reaches it in one of three ways.
//   direct: each thread loads and stores its own row element by element. A warp-wide access
//     then touches one 32-byte sector per lane, and the load/store unit spends a cycle per
//     sector: the cost is ~2 x 32 x cols cycles per warp, far above the bytes moved. Kept
//     for bases off the 16-byte grid and outputs of another element size.
//   vector: rows that are whole 16-byte vectors are loaded and stored as such.
//   staged: any other row length. The CTA copies its span into shared memory with 16-byte
//     accesses, threads read and overwrite their rows there (the stride is not a multiple of
//     16 bytes, so at most two lanes of a quarter-warp meet in a bank), and the span goes
//     back out the same way.
constexpr int kSmallRow = 32;
constexpr int kSmallRows = 256;  // rows (threads) per CTA
enum { SMALL_SOFTMAX = 0, SMALL_LOGSOFTMAX = 1, SMALL_SUM = 2, SMALL_ARGMAX = 3, SMALL_LAYERNORM = 4 };
enum { SMALL_DIRECT = 0, SMALL_STAGED = 1, SMALL_VECTOR = 2 };

template <typename T, int OP, int NC, int MODE>
__global__ void __launch_bounds__(kSmallRows) rows_small(const T* __restrict__ x, void* __restrict__ out, int64_t rows, int cols, int dto, const void* __restrict__ w,
                                                         const void* __restrict__ b, int dt_wb, void* __restrict__ mean, void* __restrict__ rstd, int dt_stat, float eps) {
  extern __shared__ __align__(16) unsigned char small_smem[];
  constexpr bool WRITES_ROWS = OP == SMALL_SOFTMAX || OP == SMALL_LOGSOFTMAX || OP == SMALL_LAYERNORM;
  constexpr bool STAGED = MODE == SMALL_STAGED, VECTOR = MODE == SMALL_VECTOR;
  constexpr int VE = 16 / static_cast<int>(sizeof(T));
  const int tid = threadIdx.x;
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * kSmallRows;
  const int64_t row = row0 + tid;
  const bool live = row < rows;
  T* sm = reinterpret_cast<T*>(small_smem);
  __shared__ float wb[2 * kSmallRow];  // layer norm: weight and bias as fp32 (1 and 0 when absent)
  if (OP == SMALL_LAYERNORM) {
    if (tid < cols) {
      wb[tid] = w ? load_as_f32(w, tid, dt_wb) : 1.f;
      wb[kSmallRow + tid] = b ? load_as_f32(b, tid, dt_wb) : 0.f;
    }
    if (!STAGED) __syncthreads();
  }
  int span = 0;
  if (STAGED) {
    const int64_t left = rows - row0;
    span = static_cast<int>(left < kSmallRows ? left : kSmallRows) * cols;  // elements this CTA owns
    const T* src = x + row0 * cols;
    const int nv = span / VE;
    for (int j = tid; j < nv; j += kSmallRows) reinterpret_cast<uint4*>(sm)[j] = ld_stream(src + static_cast<int64_t>(j) * VE);
    for (int j = nv * VE + tid; j < span; j += kSmallRows) sm[j] = src[j];
    __syncthreads();
  }
  const T* xr = STAGED ? sm + tid * cols : x + row * cols;
  T* orow = sm + tid * cols;  // staged results overwrite the row in shared memory
  float f[NC];
  auto put = [&](int c, float v) {
    if (STAGED) orow[c] = from_f32<T>(v);
    else if (VECTOR) f[c] = v;  // in place: slot c has been consumed; stored as vectors below
    else store_from_f32(out, row * cols + c, dto, v);
  };
  if (live) {
    if (VECTOR) {
#pragma unroll
      for (int v = 0; v < NC / VE; ++v) {
        if (v * VE < cols) {
          widen<T>(ld_stream(xr + v * VE), f + v * VE);
        } else {
#pragma unroll
          for (int e = 0; e < VE; ++e) f[v * VE + e] = 0.f;
        }
      }
    } else {
#pragma unroll
      for (int c = 0; c < NC; ++c) f[c] = c < cols ? to_f32(xr[c]) : 0.f;
    }
    if (OP == SMALL_SUM) {
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < NC; ++c) s += c < cols ? f[c] : 0.f;
      store_from_f32(out, row, dto, s);
    } else if (OP == SMALL_ARGMAX) {
      ArgPair a{CUDART_NAN_F, -1};
#pragma unroll
      for (int c = 0; c < NC; ++c)
        if (c < cols) arg_take_ascending(a, f[c], c);
      static_cast<int64_t*>(out)[row] = a.i;
    } else if (OP == SMALL_LAYERNORM) {
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < NC; ++c) s += c < cols ? f[c] : 0.f;
      float mu = s / static_cast<float>(cols);
      if (!isfinite(mu)) mu = CUDART_NAN_F;
      float q = 0.f;
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const float d = f[c] - mu;
        q = c < cols ? fmaf(d, d, q) : q;
      }
      const float rs = rsqrtf(q / static_cast<float>(cols) + eps);
      store_from_f32(mean, row, dt_stat, mu);
      store_from_f32(rstd, row, dt_stat, rs);
#pragma unroll
      for (int c = 0; c < NC; ++c)
        if (c < cols) put(c, (f[c] - mu) * rs * wb[c] + wb[kSmallRow + c]);
    } else {
      float m = -CUDART_INF_F;
#pragma unroll
      for (int c = 0; c < NC; ++c) m = c < cols ? fmaxf(m, f[c]) : m;
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const float d = f[c] - m;
        const float ex = ex2_approx(d * kLog2e);
        s += c < cols ? ex : 0.f;
        f[c] = OP == SMALL_LOGSOFTMAX ? d : ex;
      }
      const float k = OP == SMALL_LOGSOFTMAX ? logf(s) : 1.f / s;
#pragma unroll
      for (int c = 0; c < NC; ++c)
        if (c < cols) put(c, OP == SMALL_LOGSOFTMAX ? f[c] - k : f[c] * k);
    }
    if (VECTOR && WRITES_ROWS) {
#pragma unroll
      for (int v = 0; v < NC / VE; ++v)
        if (v * VE < cols) store_row_vec<T>(out, row * cols + v * VE, f + v * VE, false);
    }
  }
  if (STAGED && WRITES_ROWS) {
    __syncthreads();
    T* dst = static_cast<T*>(out) + row0 * cols;
    const int nv = span / VE;
    for (int j = tid; j < nv; j += kSmallRows) st_stream(dst + static_cast<int64_t>(j) * VE, reinterpret_cast<const uint4*>(sm)[j]);
    for (int j = nv * VE + tid; j < span; j += kSmallRows) dst[j] = sm[j];
  }
}

template <typename T, int OP, int NC>
static void launch_rows_small_nc(const void* x, void* out, int64_t rows, int cols, int dti, int dto, const void* w, const void* b, int dt_wb, void* mean, void* rstd, int dt_stat, float eps,
                                 cudaStream_t st) {
  constexpr bool WRITES_ROWS = OP == SMALL_SOFTMAX || OP == SMALL_LOGSOFTMAX || OP == SMALL_LAYERNORM;
  const int g = grid_for(rows, kSmallRows);
  // 16-byte accesses need 16-byte aligned bases and, for row results, an output of the input's type
  const bool wide = aligned16(x) && (!WRITES_ROWS || (dto == dti && aligned16(out)));
  const T* px = static_cast<const T*>(x);
  if (wide && (cols * sizeof(T)) % 16 == 0) {
    rows_small<T, OP, NC, SMALL_VECTOR><<<g, kSmallRows, 0, st>>>(px, out, rows, cols, dto, w, b, dt_wb, mean, rstd, dt_stat, eps);
  } else if (wide) {
    const size_t smem = (static_cast<size_t>(kSmallRows) * cols * sizeof(T) + 15) / 16 * 16;
    rows_small<T, OP, NC, SMALL_STAGED><<<g, kSmallRows, smem, st>>>(px, out, rows, cols, dto, w, b, dt_wb, mean, rstd, dt_stat, eps);
  } else {
    rows_small<T, OP, NC, SMALL_DIRECT><<<g, kSmallRows, 0, st>>>(px, out, rows, cols, dto, w, b, dt_wb, mean, rstd, dt_stat, eps);
  }
}

template <typename T, int OP>
static void launch_rows_small_T(const void* x, void* out, int64_t rows, int cols, int dti, int dto, const void* w, const void* b, int dt_wb, void* mean, void* rstd, int dt_stat, float eps,
                                cudaStream_t st) {
  if (cols <= 8) launch_rows_small_nc<T, OP, 8>(x, out, rows, cols, dti, dto, w, b, dt_wb, mean, rstd, dt_stat, eps, st);
  else if (cols <= 16) launch_rows_small_nc<T, OP, 16>(x, out, rows, cols, dti, dto, w, b, dt_wb, mean, rstd, dt_stat, eps, st);
  else if (cols <= 24) launch_rows_small_nc<T, OP, 24>(x, out, rows, cols, dti, dto, w, b, dt_wb, mean, rstd, dt_stat, eps, st);
  else launch_rows_small_nc<T, OP, 32>(x, out, rows, cols, dti, dto, w, b, dt_wb, mean, rstd, dt_stat, eps, st);
}

template <int OP>
static int launch_rows_small(const void* x, void* out, int64_t rows, int cols, int dti, int dto, const void* w, const void* b, int dt_wb, void* mean, void* rstd, int dt_stat, float eps,
                             cudaStream_t st) {
  switch (dti) {
    case B200_F32: launch_rows_small_T<float, OP>(x, out, rows, cols, dti, dto, w, b, dt_wb, mean, rstd, dt_stat, eps, st); break;
    case B200_BF16: launch_rows_small_T<__nv_bfloat16, OP>(x, out, rows, cols, dti, dto, w, b, dt_wb, mean, rstd, dt_stat, eps, st); break;
    default: launch_rows_small_T<__half, OP>(x, out, rows, cols, dti, dto, w, b, dt_wb, mean, rstd, dt_stat, eps, st); break;
  }
  return check_launch();
}

// ------------------------------------------------------------------ host-side planning
struct ReducePlan {
  int splits;
  int64_t chunk;  // elements of `dim` per split (a multiple of 64 for rows, of 16 for columns)
};

static ReducePlan plan_reduce(int64_t outer, int64_t dim, int64_t inner) {
  // CTAs available without splitting
  int64_t ctas = inner == 1 ? outer : outer * ((inner + 255) / 256);
  ReducePlan p{1, dim};
  const int64_t want = 2LL * kNumSMs;
  // A row reduction (inner == 1) is worth splitting from 4096 elements, 1024 per split. A
  // column reduction walks `dim` one row per iteration, every row a coalesced read, and with
  // few columns it has few threads: split it from 64 rows, 16 per split (argmax over 112
  // rows of 6144 columns: 24 CTAs unsplit).
  const int64_t min_dim = inner == 1 ? 4096 : 64, min_chunk = inner == 1 ? 1024 : 16;
  if (ctas >= want || dim < min_dim) return p;
  int64_t s = (want + ctas - 1) / ctas;
  const int64_t max_s = dim / min_chunk;
  if (s > max_s) s = max_s;
  if (s > 1024) s = 1024;
  if (s <= 1) return p;
  int64_t chunk = (dim + s - 1) / s;
  const int64_t gran = inner == 1 ? 64 : 16;  // row chunks stay on the 16-byte grid of any element type
  chunk = (chunk + gran - 1) / gran * gran;
  p.splits = static_cast<int>((dim + chunk - 1) / chunk);
  p.chunk = chunk;
  return p;
}

template <typename T, bool ARG>
static int launch_reduce_T(const void* x, void* out, int64_t outer, int64_t dim, int64_t inner, int dto, void* scratch, int64_t scratch_bytes, cudaStream_t st) {
  const ReducePlan p = plan_reduce(outer, dim, inner);
  const int64_t nout = outer * inner;
  float* pv = nullptr;
  int64_t* pi = nullptr;
  if (p.splits > 1) {
    const int64_t need = static_cast<int64_t>(p.splits) * nout * 16;
    if (!scratch || scratch_bytes < need) return B200_ESCRATCH;
    pi = static_cast<int64_t*>(scratch);  // int64 block first keeps it 8-byte aligned
    pv = reinterpret_cast<float*>(pi + static_cast<int64_t>(p.splits) * nout);
  }
  const T* px = static_cast<const T*>(x);
  if (inner == 1) {
    constexpr int VE = Vec<T>::N;
    const bool vecok = aligned16(x) && (dim % VE == 0);
    const bool warp = p.splits == 1 && dim * static_cast<int64_t>(sizeof(T)) <= 8192;
    if (!warp && outer > 0x7fffffffLL) return B200_EINVAL;
    if (warp) {
      dim3 g(grid_for(outer, 8), 1);
      if (vecok) reduce_rows<T, true, ARG, true><<<g, 256, 0, st>>>(px, out, pv, pi, outer, dim, p.chunk, dto);
      else reduce_rows<T, true, ARG, false><<<g, 256, 0, st>>>(px, out, pv, pi, outer, dim, p.chunk, dto);
    } else {
      dim3 g(static_cast<unsigned>(outer), p.splits);
      if (vecok) reduce_rows<T, false, ARG, true><<<g, 256, 0, st>>>(px, out, pv, pi, outer, dim, p.chunk, dto);
      else reduce_rows<T, false, ARG, false><<<g, 256, 0, st>>>(px, out, pv, pi, outer, dim, p.chunk, dto);
    }
  } else {
    if (outer > 65535) {
      // grid.y limit: fold by launching per slab of 65535 outer rows
      for (int64_t o0 = 0; o0 < outer; o0 += 65535) {
        const int64_t on = outer - o0 < 65535 ? outer - o0 : 65535;
        dim3 g(grid_for(inner, 256), static_cast<unsigned>(on), 1);
        void* o_ptr = ARG ? static_cast<void*>(static_cast<int64_t*>(out) + o0 * inner) : static_cast<void*>(static_cast<char*>(out) + o0 * inner * dtype_size(dto));
        reduce_cols<T, ARG><<<g, 256, 0, st>>>(px + o0 * dim * inner, o_ptr, nullptr, nullptr, on, dim, inner, dim, dto);
      }
      return check_launch();
    }
    if (inner <= 32 && dim >= 64) {
      int W = 1;
      while (W < inner) W <<= 1;
      dim3 g(1, static_cast<unsigned>(outer), p.splits);
      reduce_cols_narrow<T, ARG><<<g, 256, 0, st>>>(px, out, pv, pi, outer, dim, static_cast<int>(inner), W, p.chunk, dto);
    } else {
      dim3 g(grid_for(inner, 256), static_cast<unsigned>(outer), p.splits);
      reduce_cols<T, ARG><<<g, 256, 0, st>>>(px, out, pv, pi, outer, dim, inner, p.chunk, dto);
    }
  }
  if (p.splits >= 64 && nout <= 8LL * kNumSMs * 8) reduce_finalize_warp<ARG><<<grid_for(nout, 8), 256, 0, st>>>(pv, pi, out, nout, p.splits, dto);
  else if (p.splits > 1) reduce_finalize<ARG><<<grid_for(nout, 256), 256, 0, st>>>(pv, pi, out, nout, p.splits, dto);
  return check_launch(p.splits > 1 ? 2 : 1);
}

// Resident-kernel geometry for `nvec` 16-byte vectors per row.
struct ResidentCfg {
  bool ok, warp;
  int vpt, threads;
};
static ResidentCfg resident_cfg(int64_t nvec, int max_vpt, int target_vpt = 2) {
  ResidentCfg c{false, false, 1, 128};
  if (nvec <= 0) return c;
  auto pow2_at_least = [](int64_t v) { int64_t p = 1; while (p < v) p <<= 1; return p; };
  if (nvec <= 32LL * max_vpt && nvec <= 256) {
    c.ok = true; c.warp = true; c.threads = 128;
    c.vpt = static_cast<int>(pow2_at_least((nvec + 31) / 32));
    return c;
  }
  // two 16-byte vectors per thread (fewer registers, more resident warps), except fp32
  // layer norm: four (its two CTA-wide reductions cost more with many warps)
  int64_t th = pow2_at_least((nvec + target_vpt - 1) / target_vpt);
  if (th < 128) th = 128;
  if (th > 1024) th = 1024;
  const int64_t vpt = pow2_at_least((nvec + th - 1) / th);
  if (vpt > max_vpt) return c;
  c.ok = true; c.warp = false; c.threads = static_cast<int>(th); c.vpt = static_cast<int>(vpt);
  return c;
}

#define B200_DISPATCH_VPT(VPT_VALUE, MAXV, BODY)                     \
  switch (VPT_VALUE) {                                               \
    case 1: { constexpr int VPT = 1; BODY; } break;                  \
    case 2: { constexpr int VPT = 2; BODY; } break;                  \
    case 4: { constexpr int VPT = 4; BODY; } break;                  \
    default: { constexpr int VPT = (MAXV) >= 8 ? 8 : 4; BODY; } break; \
  }

template <typename T, int VPT, bool WARP>
static void softmax_launch(unsigned grid, int threads, cudaStream_t st, int is_log, const T* x, void* out, int64_t rows, int cols, int out_f32) {
  if (is_log) softmax_resident<T, VPT, WARP, true><<<grid, threads, 0, st>>>(x, out, rows, cols, out_f32);
  else softmax_resident<T, VPT, WARP, false><<<grid, threads, 0, st>>>(x, out, rows, cols, out_f32);
}
template <typename T>
static int softmax_T(const void* x, void* out, int64_t outer, int64_t dim, int64_t inner, int dto, int is_log, cudaStream_t st) {
  constexpr int VE = Vec<T>::N;
  constexpr int MAXV = 32 / VE;  // at most 32 fp32 registers of row data per thread
  const T* px = static_cast<const T*>(x);
  const int out_f32 = dto == B200_F32;
  if (inner == 1) {
    const ResidentCfg c = (dim % VE == 0 && aligned16(x) && aligned16(out) && dim < (1LL << 30)) ? resident_cfg(dim / VE, MAXV) : ResidentCfg{false, false, 1, 128};
    // 16-bit rows past 16384 elements leave a 1024-thread CTA with 3-4 vectors per thread and
    // one CTA per SM; the two-pass streaming kernel (two CTAs per SM, the second read from L2)
    // measured faster there: 3.6-4.1 TB/s against 3.1-3.5 at 24576 and 32768 bf16 columns
    const bool same_phase = dto == dtype_of<T>() && ((reinterpret_cast<uintptr_t>(x) ^ reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    const bool prefer_stream = sizeof(T) == 2 && dim / VE > 2048 && same_phase;
    if (c.ok && outer <= 0x7fffffffLL && !prefer_stream) {
      if (c.warp) {
        B200_DISPATCH_VPT(c.vpt, MAXV, (softmax_launch<T, VPT, true>(grid_for(outer, 4), 128, st, is_log, px, out, outer, static_cast<int>(dim), out_f32)))
      } else {
        B200_DISPATCH_VPT(c.vpt, MAXV, (softmax_launch<T, VPT, false>(static_cast<unsigned>(outer), c.threads, st, is_log, px, out, outer, static_cast<int>(dim), out_f32)))
      }
    } else if (dim <= kRaggedMaxCols && outer >= 64) {
      const unsigned g = grid_for(outer, 4);
      if (is_log) { B200_DISPATCH_NPL(dim, (softmax_warp_ragged<T, NPL, true><<<g, 128, 0, st>>>(px, out, outer, static_cast<int>(dim), dto))) }
      else { B200_DISPATCH_NPL(dim, (softmax_warp_ragged<T, NPL, false><<<g, 128, 0, st>>>(px, out, outer, static_cast<int>(dim), dto))) }
    } else {
      if (outer > 0x7fffffffLL) return B200_EINVAL;
      if (same_phase && dim < (1LL << 30)) {  // same type out, and rows of x and out at the same offset inside their 16-byte blocks
        int64_t th = (dim / VE + 31) / 32 * 32;
        th = th < 128 ? 128 : (th > 1024 ? 1024 : th);
        auto go = [&](auto kernel) { kernel<<<static_cast<unsigned>(outer), static_cast<unsigned>(th), 0, st>>>(px, static_cast<T*>(out), static_cast<int>(dim)); };
        if (is_log) go(softmax_stream_vec<T, true>);
        else go(softmax_stream_vec<T, false>);
      } else {
        softmax_stream<T><<<static_cast<unsigned>(outer), 256, 0, st>>>(px, out, dim, dto, is_log);
      }
    }
  } else {
    for (int64_t o0 = 0; o0 < outer; o0 += 65535) {
      const int64_t on = outer - o0 < 65535 ? outer - o0 : 65535;
      dim3 g(grid_for(inner, 128), static_cast<unsigned>(on));
      softmax_cols<T><<<g, 128, 0, st>>>(px + o0 * dim * inner, static_cast<char*>(out) + o0 * dim * inner * dtype_size(dto), dim, inner, dto, is_log);
    }
  }
  return check_launch();
}

template <typename T>
static int softmax_bwd_T(const void* g, const void* y, void* out, int64_t outer, int64_t dim, int64_t inner, int dti, int dto, int is_log, cudaStream_t st) {
  constexpr int VE = Vec<T>::N;
  constexpr int MAXV = 16 / VE;  // two rows are held: at most 16 fp32 registers of each per thread
  const T* pg = static_cast<const T*>(g);
  const T* py = static_cast<const T*>(y);
  const int out_f32 = dto == B200_F32;
  const bool out_ok = dto == B200_F32 || dto == dti;  // the vector store writes T or fp32
  if (inner == 1 && out_ok && dim % VE == 0 && aligned16(g) && aligned16(y) && aligned16(out) && dim < (1LL << 30) && outer <= 0x7fffffffLL) {
    const ResidentCfg c = resident_cfg(dim / VE, MAXV);
    if (c.ok) {
      const int cols = static_cast<int>(dim);
      if (c.warp) {
        const unsigned gr = grid_for(outer, 4);
        if (is_log) { B200_DISPATCH_VPT(c.vpt, MAXV, (softmax_bwd_resident<T, VPT, true, true><<<gr, 128, 0, st>>>(pg, py, out, outer, cols, out_f32))) }
        else { B200_DISPATCH_VPT(c.vpt, MAXV, (softmax_bwd_resident<T, VPT, true, false><<<gr, 128, 0, st>>>(pg, py, out, outer, cols, out_f32))) }
      } else {
        const unsigned gr = static_cast<unsigned>(outer);
        if (is_log) { B200_DISPATCH_VPT(c.vpt, MAXV, (softmax_bwd_resident<T, VPT, false, true><<<gr, c.threads, 0, st>>>(pg, py, out, outer, cols, out_f32))) }
        else { B200_DISPATCH_VPT(c.vpt, MAXV, (softmax_bwd_resident<T, VPT, false, false><<<gr, c.threads, 0, st>>>(pg, py, out, outer, cols, out_f32))) }
      }
      return check_launch();
    }
  }
  const int64_t lines = outer * inner;
  if ((lines + 3) / 4 > 0x7fffffffLL) return B200_EINVAL;
  if (is_log) softmax_bwd_lines<T, true><<<grid_for(lines, 4), 128, 0, st>>>(pg, py, out, outer, dim, inner, dto);
  else softmax_bwd_lines<T, false><<<grid_for(lines, 4), 128, 0, st>>>(pg, py, out, outer, dim, inner, dto);
  return check_launch();
}

template <typename T, typename TW, bool HOLD, bool AFFINE>
static int layernorm_launch(const T* px, const TW* pw, const TW* pb, T* py, void* mean, void* rstd, int64_t rows, int64_t cols, float eps, int dt_stat, const ResidentCfg& c, cudaStream_t st) {
  constexpr int VE = Vec<T>::N;
  constexpr int MAXV = 32 / VE;
  const float inv_cols = 1.f / static_cast<float>(cols);
  if (c.warp) {
    B200_DISPATCH_VPT(c.vpt, MAXV, (layernorm_resident<T, TW, VPT, true, HOLD, AFFINE><<<grid_for(rows, 4), 128, 0, st>>>(px, pw, pb, py, mean, rstd, rows, static_cast<int>(cols), inv_cols, eps, dt_stat)))
  } else if (AFFINE && !HOLD && c.vpt <= 2 && c.threads <= 256 && rows >= 8LL * kNumSMs) {
    // many 16-bit rows: persistent CTAs that keep weight and bias in registers (four CTAs per SM)
    const unsigned grid = static_cast<unsigned>(4 * kNumSMs);
    if (c.vpt == 1) layernorm_persistent<T, TW, 1><<<grid, c.threads, 0, st>>>(px, pw, pb, py, mean, rstd, rows, static_cast<int>(cols), inv_cols, eps, dt_stat);
    else layernorm_persistent<T, TW, 2><<<grid, c.threads, 0, st>>>(px, pw, pb, py, mean, rstd, rows, static_cast<int>(cols), inv_cols, eps, dt_stat);
  } else {
    B200_DISPATCH_VPT(c.vpt, MAXV, (layernorm_resident<T, TW, VPT, false, HOLD, AFFINE><<<static_cast<unsigned>(rows), c.threads, 0, st>>>(px, pw, pb, py, mean, rstd, rows, static_cast<int>(cols), inv_cols, eps, dt_stat)))
  }
  return check_launch();
}

template <typename T, typename TW>
static int layernorm_T(const void* x, const void* w, const void* b, void* y, void* mean, void* rstd, int64_t rows, int64_t cols, float eps, int dt_stat, const ResidentCfg& c, cudaStream_t st) {
  const T* px = static_cast<const T*>(x);
  const TW* pw = static_cast<const TW*>(w);
  const TW* pb = static_cast<const TW*>(b);
  T* py = static_cast<T*>(y);
  constexpr bool hold = sizeof(T) == 4;  // 16-bit rows stay packed: fewer registers, more resident warps
  const bool affine = w && b;
  return affine ? layernorm_launch<T, TW, hold, true>(px, pw, pb, py, mean, rstd, rows, cols, eps, dt_stat, c, st) : layernorm_launch<T, TW, hold, false>(px, pw, pb, py, mean, rstd, rows, cols, eps, dt_stat, c, st);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_softmax(const void* x, void* out, int64_t outer, int64_t dim, int64_t inner, int dti, int dto, int is_log, void* stream) {
  if (outer < 0 || dim < 0 || inner < 0) return B200_EINVAL;
  if (!is_float_dtype(dti) || !(dto == dti || dto == B200_F32)) return B200_EDTYPE;
  if (outer == 0 || dim == 0 || inner == 0) return B200_OK;
  if (!x || !out) return B200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (inner == 1 && dim <= kSmallRow && outer >= 4096)
    return is_log ? launch_rows_small<SMALL_LOGSOFTMAX>(x, out, outer, static_cast<int>(dim), dti, dto, nullptr, nullptr, 0, nullptr, nullptr, 0, 0.f, st)
                  : launch_rows_small<SMALL_SOFTMAX>(x, out, outer, static_cast<int>(dim), dti, dto, nullptr, nullptr, 0, nullptr, nullptr, 0, 0.f, st);
  switch (dti) {
    case B200_F32: return softmax_T<float>(x, out, outer, dim, inner, dto, is_log, st);
    case B200_BF16: return softmax_T<__nv_bfloat16>(x, out, outer, dim, inner, dto, is_log, st);
    default: return softmax_T<__half>(x, out, outer, dim, inner, dto, is_log, st);
  }
}

extern "C" int b200_softmax_backward(const void* grad, const void* output, void* grad_input, int64_t outer, int64_t dim, int64_t inner, int dti, int dto, int is_log, void* stream) {
  if (outer < 0 || dim < 0 || inner < 0) return B200_EINVAL;
  if (!is_float_dtype(dti) || !is_float_dtype(dto)) return B200_EDTYPE;
  if (outer == 0 || dim == 0 || inner == 0) return B200_OK;
  if (!grad || !output || !grad_input) return B200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dti) {
    case B200_F32: return softmax_bwd_T<float>(grad, output, grad_input, outer, dim, inner, dti, dto, is_log, st);
    case B200_BF16: return softmax_bwd_T<__nv_bfloat16>(grad, output, grad_input, outer, dim, inner, dti, dto, is_log, st);
    default: return softmax_bwd_T<__half>(grad, output, grad_input, outer, dim, inner, dti, dto, is_log, st);
  }
}

extern "C" int64_t b200_reduce_scratch_bytes(int64_t outer, int64_t dim, int64_t inner) {
  if (outer <= 0 || dim <= 0 || inner <= 0) return 0;
  const ReducePlan p = plan_reduce(outer, dim, inner);
  return p.splits > 1 ? static_cast<int64_t>(p.splits) * outer * inner * 16 : 0;
}

extern "C" int b200_sum(const void* x, void* out, int64_t outer, int64_t dim, int64_t inner, int dti, int dto, void* scratch, int64_t scratch_bytes, void* stream) {
  if (outer < 0 || dim < 0 || inner < 0) return B200_EINVAL;
  if (!is_float_dtype(dti) || !is_float_dtype(dto)) return B200_EDTYPE;
  if (outer == 0 || inner == 0) return B200_OK;
  if (!out) return B200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dim == 0) {  // empty reduction: the sum is 0
    fill_zero_typed<<<grid_for(outer * inner, 256), 256, 0, st>>>(out, outer * inner, dto);
    return check_launch();
  }
  if (!x) return B200_EINVAL;
  if (inner == 1 && dim <= kSmallRow && outer >= 4096) return launch_rows_small<SMALL_SUM>(x, out, outer, static_cast<int>(dim), dti, dto, nullptr, nullptr, 0, nullptr, nullptr, 0, 0.f, st);
  switch (dti) {
    case B200_F32: return launch_reduce_T<float, false>(x, out, outer, dim, inner, dto, scratch, scratch_bytes, st);
    case B200_BF16: return launch_reduce_T<__nv_bfloat16, false>(x, out, outer, dim, inner, dto, scratch, scratch_bytes, st);
    default: return launch_reduce_T<__half, false>(x, out, outer, dim, inner, dto, scratch, scratch_bytes, st);
  }
}

extern "C" int b200_argmax(const void* x, int64_t* out, int64_t outer, int64_t dim, int64_t inner, int dt, void* scratch, int64_t scratch_bytes, void* stream) {
  if (outer < 0 || dim <= 0 || inner < 0) return B200_EINVAL;
  if (!is_float_dtype(dt)) return B200_EDTYPE;
  if (outer == 0 || inner == 0) return B200_OK;
  if (!x || !out) return B200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (inner == 1 && dim <= kSmallRow && outer >= 4096) return launch_rows_small<SMALL_ARGMAX>(x, out, outer, static_cast<int>(dim), dt, B200_I64, nullptr, nullptr, 0, nullptr, nullptr, 0, 0.f, st);
  switch (dt) {
    case B200_F32: return launch_reduce_T<float, true>(x, out, outer, dim, inner, B200_I64, scratch, scratch_bytes, st);
    case B200_BF16: return launch_reduce_T<__nv_bfloat16, true>(x, out, outer, dim, inner, B200_I64, scratch, scratch_bytes, st);
    default: return launch_reduce_T<__half, true>(x, out, outer, dim, inner, B200_I64, scratch, scratch_bytes, st);
  }
}

extern "C" int b200_layer_norm(const void* x, const void* w, const void* b, void* y, void* mean, void* rstd, int64_t rows, int64_t cols, double eps, int dt, int dt_wb, int dt_stat, void* stream) {
  if (rows < 0 || cols < 0) return B200_EINVAL;
  if (!is_float_dtype(dt) || !is_float_dtype(dt_stat) || ((w || b) && !is_float_dtype(dt_wb))) return B200_EDTYPE;
  if (rows == 0) return B200_OK;
  if (!mean || !rstd) return B200_EINVAL;
  if (cols > 0 && (!x || !y)) return B200_EINVAL;
  if (rows > 0x7fffffffLL) return B200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float e = static_cast<float>(eps);
  if (cols > 0 && cols <= kSmallRow && rows >= 4096) return launch_rows_small<SMALL_LAYERNORM>(x, y, rows, static_cast<int>(cols), dt, dt, w, b, dt_wb, mean, rstd, dt_stat, e, st);
  const int ve = 16 / dtype_size(dt);
  const bool wb_ok = (!w && !b) || dt_wb == dt || dt_wb == B200_F32;
  const bool al = aligned16(x) && aligned16(y) && (!w || aligned16(w)) && (!b || aligned16(b));
  ResidentCfg c{false, false, 1, 128};
  if (cols > 0 && cols % ve == 0 && (dt_wb != B200_F32 || cols % 4 == 0) && al && wb_ok && cols < (1LL << 30)) c = resident_cfg(cols / ve, 32 / ve, ve == 4 ? 4 : 2);
  if (!c.ok && cols > 0 && cols <= kRaggedMaxCols && rows >= 64) {
    const unsigned g = grid_for(rows, 4);
    const int ci = static_cast<int>(cols);
    switch (dt) {
      case B200_F32: B200_DISPATCH_NPL(cols, (layernorm_warp_ragged<float, NPL><<<g, 128, 0, st>>>(static_cast<const float*>(x), w, b, static_cast<float*>(y), mean, rstd, rows, ci, e, dt_wb, dt_stat))) break;
      case B200_BF16: B200_DISPATCH_NPL(cols, (layernorm_warp_ragged<__nv_bfloat16, NPL><<<g, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(x), w, b, static_cast<__nv_bfloat16*>(y), mean, rstd, rows, ci, e, dt_wb, dt_stat))) break;
      default: B200_DISPATCH_NPL(cols, (layernorm_warp_ragged<__half, NPL><<<g, 128, 0, st>>>(static_cast<const __half*>(x), w, b, static_cast<__half*>(y), mean, rstd, rows, ci, e, dt_wb, dt_stat))) break;
    }
    return check_launch();
  }
  if (!c.ok) {
    layernorm_stream<<<static_cast<unsigned>(rows), 256, 0, st>>>(x, w, b, y, mean, rstd, cols, e, dt, dt_wb, dt_stat);
    return check_launch();
  }
  const bool wf32 = (w || b) && dt_wb == B200_F32;
  switch (dt) {
    case B200_F32: return layernorm_T<float, float>(x, w, b, y, mean, rstd, rows, cols, e, dt_stat, c, st);
    case B200_BF16:
      return wf32 ? layernorm_T<__nv_bfloat16, float>(x, w, b, y, mean, rstd, rows, cols, e, dt_stat, c, st)
                  : layernorm_T<__nv_bfloat16, __nv_bfloat16>(x, w, b, y, mean, rstd, rows, cols, e, dt_stat, c, st);
    default:
      return wf32 ? layernorm_T<__half, float>(x, w, b, y, mean, rstd, rows, cols, e, dt_stat, c, st)
                  : layernorm_T<__half, __half>(x, w, b, y, mean, rstd, rows, cols, e, dt_stat, c, st);
  }
}

// ---- layer norm backward: host side
static const int64_t kLnBwdMaxParts = 8LL * kNumSMs;  // partial rows of dw / db in scratch

extern "C" int64_t b200_layer_norm_backward_scratch_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return 0;
  const int64_t parts = rows < kLnBwdMaxParts ? rows : kLnBwdMaxParts;
  return parts * cols * 2 * 4;
}

template <typename T, typename TW>
static int layernorm_bwd_fused_launch(const void* dy, const void* x, const void* w, const void* mean, const void* rstd, void* dx, float* pw, float* pb, int64_t rows, int64_t cols, int dt_stat,
                                      int threads, int vpt, int grid, cudaStream_t st) {
  const T* pdy = static_cast<const T*>(dy);
  const T* px = static_cast<const T*>(x);
  const TW* pwt = static_cast<const TW*>(w);
  T* pdx = static_cast<T*>(dx);
  const int ci = static_cast<int>(cols);
  switch (vpt) {
    case 1: layernorm_bwd_fused<T, TW, 1><<<grid, threads, 0, st>>>(pdy, px, pwt, mean, rstd, pdx, pw, pb, rows, ci, dt_stat); break;
    default: layernorm_bwd_fused<T, TW, 2><<<grid, threads, 0, st>>>(pdy, px, pwt, mean, rstd, pdx, pw, pb, rows, ci, dt_stat); break;
  }
  return B200_OK;
}
// CTAs of the fused kernel one SM holds at this block size (registers decide).
template <typename T, typename TW>
static int layernorm_bwd_fused_per_sm(int threads, int vpt) {
  int n = 0;
  const cudaError_t e = vpt == 1 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, layernorm_bwd_fused<T, TW, 1>, threads, 0)
                                 : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, layernorm_bwd_fused<T, TW, 2>, threads, 0);
  return e == cudaSuccess && n > 0 ? n : 1;
}

extern "C" int b200_layer_norm_backward(const void* dy, const void* x, const void* mean, const void* rstd, const void* w, void* dx, void* dw, void* db, int64_t rows, int64_t cols, int dt,
                                        int dt_wb, int dt_stat, void* scratch, int64_t scratch_bytes, void* stream) {
  if (rows < 0 || cols < 0) return B200_EINVAL;
  if (!is_float_dtype(dt) || !is_float_dtype(dt_stat) || ((w || dw || db) && !is_float_dtype(dt_wb))) return B200_EDTYPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cols == 0) return B200_OK;
  if (rows == 0) {  // nothing to sum: the parameter gradients are zero
    if (dw) fill_zero_typed<<<grid_for(cols, 256), 256, 0, st>>>(dw, cols, dt_wb);
    if (db) fill_zero_typed<<<grid_for(cols, 256), 256, 0, st>>>(db, cols, dt_wb);
    return check_launch();
  }
  if (!dy || !x || !mean || !rstd) return B200_EINVAL;
  const bool need_wb = dw || db;
  const int64_t parts_max = rows < kLnBwdMaxParts ? rows : kLnBwdMaxParts;
  float* pw = nullptr;
  float* pb = nullptr;
  if (need_wb) {
    if (!scratch || scratch_bytes < b200_layer_norm_backward_scratch_bytes(rows, cols)) return B200_ESCRATCH;
    pw = static_cast<float*>(scratch);
    pb = pw + parts_max * cols;
  }
  const int ve = 16 / dtype_size(dt);
  const bool wb_ok = !w || dt_wb == dt || dt_wb == B200_F32;
  const bool al = aligned16(dy) && aligned16(x) && (!dx || aligned16(dx)) && (!w || aligned16(w));
  int64_t parts = 0;
  // a thread keeps five values per owned column in registers (dy, xhat, w, and its share of dw
  // and db): one 16-byte vector of a 16-bit row, two of an fp32 row -- rows of up to 8192
  // elements; longer ones would spill
  const int target = ve == 4 ? 2 : 1;
  if (cols % ve == 0 && (dt_wb != B200_F32 || !w || cols % 4 == 0) && al && wb_ok && cols / ve <= 1024 * target) {
    const int64_t nvec = cols / ve;
    int threads = 32;
    while (threads < 1024 && threads * target < nvec) threads <<= 1;
    const int vpt = static_cast<int>((nvec + threads - 1) / threads);
    const bool wf32 = w && dt_wb == B200_F32;
    int per_sm = 1;
    switch (dt) {
      case B200_F32: per_sm = layernorm_bwd_fused_per_sm<float, float>(threads, vpt); break;
      case B200_BF16: per_sm = wf32 ? layernorm_bwd_fused_per_sm<__nv_bfloat16, float>(threads, vpt) : layernorm_bwd_fused_per_sm<__nv_bfloat16, __nv_bfloat16>(threads, vpt); break;
      default: per_sm = wf32 ? layernorm_bwd_fused_per_sm<__half, float>(threads, vpt) : layernorm_bwd_fused_per_sm<__half, __half>(threads, vpt); break;
    }
    if (per_sm > 8) per_sm = 8;
    parts = static_cast<int64_t>(per_sm) * kNumSMs;  // a persistent grid: exactly what the device holds at once
    if (parts > parts_max) parts = parts_max;
    const int grid = static_cast<int>(parts);
    switch (dt) {
      case B200_F32: layernorm_bwd_fused_launch<float, float>(dy, x, w, mean, rstd, dx, pw, pb, rows, cols, dt_stat, threads, vpt, grid, st); break;
      case B200_BF16:
        if (wf32) layernorm_bwd_fused_launch<__nv_bfloat16, float>(dy, x, w, mean, rstd, dx, pw, pb, rows, cols, dt_stat, threads, vpt, grid, st);
        else layernorm_bwd_fused_launch<__nv_bfloat16, __nv_bfloat16>(dy, x, w, mean, rstd, dx, pw, pb, rows, cols, dt_stat, threads, vpt, grid, st);
        break;
      default:
        if (wf32) layernorm_bwd_fused_launch<__half, float>(dy, x, w, mean, rstd, dx, pw, pb, rows, cols, dt_stat, threads, vpt, grid, st);
        else layernorm_bwd_fused_launch<__half, __half>(dy, x, w, mean, rstd, dx, pw, pb, rows, cols, dt_stat, threads, vpt, grid, st);
        break;
    }
  } else {
    if (dx) {
      const int64_t g = rows < 8LL * kNumSMs ? rows : 8LL * kNumSMs;
      layernorm_bwd_dx_lines<<<static_cast<int>(g), 256, 0, st>>>(dy, x, w, mean, rstd, dx, rows, cols, dt, dt_wb, dt_stat);
    }
    if (need_wb) {
      parts = parts_max < 64 ? parts_max : 64;
      const int64_t rows_per = (rows + parts - 1) / parts;
      parts = (rows + rows_per - 1) / rows_per;
      const int64_t gx = (cols + 255) / 256;
      if (gx > 0x7fffffffLL) return B200_EINVAL;
      layernorm_bwd_wb_lines<<<dim3(static_cast<unsigned>(gx), static_cast<unsigned>(parts)), 256, 0, st>>>(dy, x, mean, rstd, pw, pb, rows, cols, rows_per, dt, dt_stat);
    }
  }
  if (need_wb) layernorm_bwd_finalize<<<grid_for(cols, 32), 1024, 0, st>>>(pw, pb, dw, db, parts, cols, dt_wb);
  return check_launch(need_wb ? 2 : 1);
}

// ------------------------------------------------------------------ sum without any allocation
// Scratch for the split-reduction partials of b200_sum_static. It lives in the library
// image: every GPU that loads the library holds these bytes until the process exits.
static __device__ __align__(256) unsigned char g_sum_static_scratch[B200_STATIC_SCRATCH_BYTES];

// Device address of the array above on the CURRENT device. In host code the array's name
// is only a handle, not something a kernel can dereference, so the address is asked for
// once per device (cudaGetSymbolAddress, return code checked) and remembered.
static void* sum_static_scratch_address(void) {
  static std::mutex mu;
  static void* per_device[64] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    set_last_cuda_error(e != cudaSuccess ? e : cudaErrorInvalidDevice);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!per_device[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_sum_static_scratch);
    if (e != cudaSuccess || !p) {
      set_last_cuda_error(e);
      return nullptr;
    }
    per_device[dev] = p;
  }
  return per_device[dev];
}

extern "C" int b200_sum_static(const void* x, void* out, int64_t outer, int64_t dim, int64_t inner, int dti, int dto, void* stream) {
  const int64_t need = b200_reduce_scratch_bytes(outer, dim, inner);
  if (need > B200_STATIC_SCRATCH_BYTES) return B200_ESCRATCH;
  void* scratch = nullptr;
  if (need > 0) {
    scratch = sum_static_scratch_address();
    if (!scratch) return B200_ELAUNCH;
  }
  // every partial slot is written by the first stage before the second stage reads it, so
  // whatever an earlier call left in the array never needs clearing
  return b200_sum(x, out, outer, dim, inner, dti, dto, scratch, need > 0 ? B200_STATIC_SCRATCH_BYTES : 0, stream);
}
