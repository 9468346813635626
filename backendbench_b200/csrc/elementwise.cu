// relu / add / mul / where / strided copy: HBM-bound streaming kernels.
//
// Fast path: every operand contiguous (or a single broadcast scalar), same dtype,
// 16-byte aligned -> each thread moves kUnroll independent 16-byte vectors per operand
// so ~128 KB per SM is in flight, accesses are fully coalesced and marked streaming.
// Slow path: TensorIterator-style strided indexing with runtime dtypes (broadcasts,
// transposes, mixed-precision promotion); correctness first, one element per thread.
#include "b200_common.cuh"

namespace b200 {

constexpr int kEwThreads = 256;
constexpr int kUnroll = 4;

struct ReluOp { __device__ __forceinline__ float operator()(float x) const { return x <= 0.f ? 0.f : x; } };
struct AddOp {
  float alpha;
  __device__ __forceinline__ float operator()(float a, float b) const { return fmaf(alpha, b, a); }
};
struct AddConstOp { float c; __device__ __forceinline__ float operator()(float x) const { return x + c; } };
struct MulConstOp { float c; __device__ __forceinline__ float operator()(float x) const { return x * c; } };
struct MulOp { __device__ __forceinline__ float operator()(float a, float b) const { return a * b; } };

template <typename T, typename Op>
__global__ void __launch_bounds__(kEwThreads) ew_unary_vec(const T* __restrict__ x, T* __restrict__ out, int64_t n, Op op) {
  constexpr int VE = Vec<T>::N;
  const int64_t nvec = n / VE;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * (kEwThreads * kUnroll) + threadIdx.x;
  Vec<T> v[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t i = base + u * kEwThreads;
    if (i < nvec) v[u].raw = ld_stream(x + i * VE);
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t i = base + u * kEwThreads;
    if (i < nvec) {
      float f[VE];
      widen<T>(v[u].raw, f);
#pragma unroll
      for (int e = 0; e < VE; ++e) f[e] = op(f[e]);
      st_stream(out + i * VE, narrow<T>(f));
    }
  }
  // ragged tail (< VE elements): the last block's first threads
  if (blockIdx.x == gridDim.x - 1) {
    const int64_t i = nvec * VE + threadIdx.x;
    if (i < n) out[i] = from_f32<T>(op(to_f32(x[i])));
  }
}

// MODE 0: a[i] op b[i]; MODE 1: a[i] op b[0]; MODE 2: a[0] op b[i]
template <typename T, typename Op, int MODE>
__global__ void __launch_bounds__(kEwThreads) ew_binary_vec(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t n, Op op) {
  constexpr int VE = Vec<T>::N;
  const int64_t nvec = n / VE;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * (kEwThreads * kUnroll) + threadIdx.x;
  Vec<T> va[kUnroll], vb[kUnroll];
  float sa = 0.f, sb = 0.f;
  if (MODE == 1) sb = to_f32(b[0]);
  if (MODE == 2) sa = to_f32(a[0]);
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t i = base + u * kEwThreads;
    if (i < nvec) {
      if (MODE != 2) va[u].raw = ld_stream(a + i * VE);
      if (MODE != 1) vb[u].raw = ld_stream(b + i * VE);
    }
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t i = base + u * kEwThreads;
    if (i < nvec) {
      float fa[VE], fb[VE];
      if (MODE != 2) widen<T>(va[u].raw, fa);
      if (MODE != 1) widen<T>(vb[u].raw, fb);
#pragma unroll
      for (int e = 0; e < VE; ++e) fa[e] = op(MODE == 2 ? sa : fa[e], MODE == 1 ? sb : fb[e]);
      st_stream(out + i * VE, narrow<T>(fa));
    }
  }
  if (blockIdx.x == gridDim.x - 1) {
    const int64_t i = nvec * VE + threadIdx.x;
    if (i < n) {
      const float fa = MODE == 2 ? sa : to_f32(a[i]);
      const float fb = MODE == 1 ? sb : to_f32(b[i]);
      out[i] = from_f32<T>(op(fa, fb));
    }
  }
}

// where on contiguous same-size operands: U is an unsigned type of the element size
// (pure bit select, so NaN payloads and -0 survive untouched).
template <typename U>
__global__ void __launch_bounds__(kEwThreads) ew_where_vec(const uint8_t* __restrict__ c, const U* __restrict__ x, const U* __restrict__ y, U* __restrict__ out, int64_t n) {
  constexpr int VE = 16 / sizeof(U);
  const int64_t nvec = n / VE;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * (kEwThreads * kUnroll) + threadIdx.x;
  Vec<U> vx[kUnroll], vy[kUnroll];
  uint8_t cc[kUnroll][VE];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t i = base + u * kEwThreads;
    if (i < nvec) {
      vx[u].raw = ld_stream(x + i * VE);
      vy[u].raw = ld_stream(y + i * VE);
      if (VE == 4) {
        *reinterpret_cast<uint32_t*>(cc[u]) = __ldcs(reinterpret_cast<const uint32_t*>(c + i * VE));
      } else if (VE == 8) {
        *reinterpret_cast<uint2*>(cc[u]) = __ldcs(reinterpret_cast<const uint2*>(c + i * VE));
      } else {
#pragma unroll
        for (int e = 0; e < VE; ++e) cc[u][e] = c[i * VE + e];
      }
    }
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int64_t i = base + u * kEwThreads;
    if (i < nvec) {
      Vec<U> r;
#pragma unroll
      for (int e = 0; e < VE; ++e) r.set(e, cc[u][e] ? vx[u].get(e) : vy[u].get(e));
      st_stream(out + i * VE, r.raw);
    }
  }
  if (blockIdx.x == gridDim.x - 1) {
    const int64_t i = nvec * VE + threadIdx.x;
    if (i < n) out[i] = c[i] ? x[i] : y[i];
  }
}

// ------------------------------------------------------------------ strided slow path
struct StridedArgs {
  int ndim;
  int64_t n;
  int64_t shape[B200_MAX_DIMS];
  int64_t s0[B200_MAX_DIMS], s1[B200_MAX_DIMS], s2[B200_MAX_DIMS];
};

__device__ __forceinline__ void unravel3(const StridedArgs& A, int64_t lin, int64_t& o0, int64_t& o1, int64_t& o2) {
  o0 = o1 = o2 = 0;
  if (A.n <= 0x7fffffffLL) {  // coordinates by 32-bit division (a 64-bit one costs ~5x the instructions)
    uint32_t l = static_cast<uint32_t>(lin);
    for (int d = A.ndim - 1; d >= 0; --d) {
      const uint32_t ext = static_cast<uint32_t>(A.shape[d]);
      const uint32_t q = l / ext, r = l - q * ext;
      o0 += r * A.s0[d];
      o1 += r * A.s1[d];
      o2 += r * A.s2[d];
      l = q;
    }
    return;
  }
  for (int d = A.ndim - 1; d >= 0; --d) {
    const int64_t q = lin / A.shape[d];
    const int64_t r = lin - q * A.shape[d];
    o0 += r * A.s0[d];
    o1 += r * A.s1[d];
    o2 += r * A.s2[d];
    lin = q;
  }
}

enum { OP_RELU = 0, OP_ADD = 1, OP_MUL = 2, OP_COPY = 3, OP_ADDC = 4, OP_MULC = 5 };

template <int OP>
__global__ void __launch_bounds__(kEwThreads) ew_strided(const void* a, const void* b, void* out, StridedArgs A, int dta, int dtb, int dto, float alpha) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kEwThreads + threadIdx.x; i < A.n; i += static_cast<int64_t>(gridDim.x) * kEwThreads) {
    int64_t oa, ob, oc;
    unravel3(A, i, oa, ob, oc);
    float r;
    if (OP == OP_RELU) {
      const float x = load_as_f32(a, oa, dta);
      r = x <= 0.f ? 0.f : x;
    } else if (OP == OP_COPY) {
      r = load_as_f32(a, oa, dta);
    } else if (OP == OP_ADDC) {
      r = load_as_f32(a, oa, dta) + alpha;
    } else if (OP == OP_MULC) {
      r = load_as_f32(a, oa, dta) * alpha;
    } else {
      const float x = load_as_f32(a, oa, dta), y = load_as_f32(b, ob, dtb);
      r = OP == OP_ADD ? fmaf(alpha, y, x) : x * y;
    }
    store_from_f32(out, i, dto, r);
  }
}

// Bit-exact strided copy for any element size (same dtype in and out).
template <typename U>
__global__ void __launch_bounds__(kEwThreads) copy_strided_bits(const U* x, U* out, StridedArgs A) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kEwThreads + threadIdx.x; i < A.n; i += static_cast<int64_t>(gridDim.x) * kEwThreads) {
    int64_t oa, ob, oc;
    unravel3(A, i, oa, ob, oc);
    out[i] = x[oa];
  }
}

// Bit-exact copy between two strided layouts of one shape (source offsets in s0, destination
// offsets in s1): how a result is written into a caller's non-contiguous `out` / `self`.
template <typename U>
__global__ void __launch_bounds__(kEwThreads) copy_between_strided(const U* x, U* out, StridedArgs A) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kEwThreads + threadIdx.x; i < A.n; i += static_cast<int64_t>(gridDim.x) * kEwThreads) {
    int64_t oa, ob, oc;
    unravel3(A, i, oa, ob, oc);
    out[ob] = x[oa];
  }
}

// where, strided: cond/x/y offsets in s0/s1/s2. Same-dtype operands are bit-selected;
// mixed float dtypes go through fp32 (exact: every bf16/f16 value is an fp32 value).
template <typename U, bool BITS>
__global__ void __launch_bounds__(kEwThreads) where_strided(const uint8_t* c, const void* x, const void* y, void* out, StridedArgs A, int dtx, int dty, int dto) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kEwThreads + threadIdx.x; i < A.n; i += static_cast<int64_t>(gridDim.x) * kEwThreads) {
    int64_t oc, ox, oy;
    unravel3(A, i, oc, ox, oy);
    const bool take = c[oc] != 0;
    if (BITS) {
      static_cast<U*>(out)[i] = take ? static_cast<const U*>(x)[ox] : static_cast<const U*>(y)[oy];
    } else {
      store_from_f32(out, i, dto, take ? load_as_f32(x, ox, dtx) : load_as_f32(y, oy, dty));
    }
  }
}

// [batch, rows, cols] gather from arbitrary element strides into a pitched destination
// (unit column stride): how the host gives a tensor-core GEMM operand a 16-byte-aligned
// row pitch when the caller's layout has none.
// One warp per row, lanes along the columns: no per-element index division (a flat index
// costs two 64-bit divisions per 2-byte element), coalesced on both sides when the source
// has unit column stride.
template <typename U>
__global__ void __launch_bounds__(kEwThreads) copy_pitched(const U* __restrict__ x, U* __restrict__ out, int64_t batch, int64_t rows, int64_t cols, int64_t sxb, int64_t sxr,
                                                           int64_t sxc, int64_t opb, int64_t opr) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (kEwThreads / 32);
  for (int64_t rr = static_cast<int64_t>(blockIdx.x) * (kEwThreads / 32) + (threadIdx.x >> 5); rr < batch * rows; rr += warps) {
    const int64_t b = rr / rows, r = rr - b * rows;
    const U* src = x + b * sxb + r * sxr;
    U* dst = out + b * opb + r * opr;
    int64_t c = lane;
    for (; c + 96 < cols; c += 128) {  // four independent loads in flight per lane
      const U v0 = src[c * sxc], v1 = src[(c + 32) * sxc], v2 = src[(c + 64) * sxc], v3 = src[(c + 96) * sxc];
      dst[c] = v0; dst[c + 32] = v1; dst[c + 64] = v2; dst[c + 96] = v3;
    }
    for (; c < cols; c += 32) dst[c] = src[c * sxc];
  }
}

// ------------------------------------------------------------------ transposed operands
// When an operand's unit stride runs along the second-to-last dim of the (coalesced)
// iteration shape -- a transposed view -- the strided kernel above reads it one 32-byte
// sector per element. These kernels walk 32 x 32 tiles of the last two dims instead: a
// transposed operand is read along ITS contiguous direction into shared memory and handed
// to the thread that needs it; everything else is read in place. Up to one leading batch
// dim (blockIdx.z).
struct TiledArgs {
  int64_t B, R, C;
  int64_t ab, ar, ac, bb, br, bc;  // element strides of the two operands: batch, row, column
  int a_t, b_t;                    // operand is read through the transposing tile
};
static bool transposed_view(int64_t s_row, int64_t s_col, int64_t rows, int64_t cols) { return s_row == 1 && s_col != 1 && s_col != 0 && rows >= 16 && cols >= 16; }

template <int OP>
__global__ void __launch_bounds__(256) ew_tiled(const void* a, const void* b, void* out, TiledArgs T, int dta, int dtb, int dto, float alpha) {
  __shared__ float ta[32][33], tb[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 32, c0 = static_cast<int64_t>(blockIdx.x) * 32, bz = blockIdx.z;
  constexpr bool kBinary = OP == OP_ADD || OP == OP_MUL;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int64_t r = r0 + tx, c = c0 + ty + 8 * j;  // consecutive threads along the operand's contiguous rows
    if (r < T.R && c < T.C) {
      if (T.a_t) ta[ty + 8 * j][tx] = load_as_f32(a, bz * T.ab + r * T.ar + c * T.ac, dta);
      if (kBinary && T.b_t) tb[ty + 8 * j][tx] = load_as_f32(b, bz * T.bb + r * T.br + c * T.bc, dtb);
    }
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int64_t r = r0 + ty + 8 * j, c = c0 + tx;
    if (r < T.R && c < T.C) {
      const float x = T.a_t ? ta[tx][ty + 8 * j] : load_as_f32(a, bz * T.ab + r * T.ar + c * T.ac, dta);
      float res;
      if (OP == OP_RELU) res = x <= 0.f ? 0.f : x;
      else if (OP == OP_COPY) res = x;
      else if (OP == OP_ADDC) res = x + alpha;
      else if (OP == OP_MULC) res = x * alpha;
      else {
        const float y = T.b_t ? tb[tx][ty + 8 * j] : load_as_f32(b, bz * T.bb + r * T.br + c * T.bc, dtb);
        res = OP == OP_ADD ? fmaf(alpha, y, x) : x * y;
      }
      store_from_f32(out, (bz * T.R + r) * T.C + c, dto, res);
    }
  }
}

// The same 32 x 32 walk for operands and result of one type T. The generic kernel above
// decides the element type per access and rebuilds every address from three 64-bit products
// (92 instructions per element in the profile of a transposed fp32 add); here the type is a
// template parameter and the offsets advance by additions.
template <typename T, int OP>
__global__ void __launch_bounds__(256) ew_tiled_typed(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, TiledArgs A, float alpha) {
  constexpr bool kBinary = OP == OP_ADD || OP == OP_MUL;
  __shared__ float ta[32][33];
  __shared__ float tb[kBinary ? 32 : 1][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 32, c0 = static_cast<int64_t>(blockIdx.x) * 32, bz = blockIdx.z;
  const T* ap = a + bz * A.ab;
  const T* bp = kBinary ? b + bz * A.bb : nullptr;
  {
    const int64_t r = r0 + tx;  // consecutive threads along the transposed operand's contiguous direction
    int64_t c = c0 + ty;
    int64_t oa = r * A.ar + c * A.ac, ob = kBinary ? r * A.br + c * A.bc : 0;
#pragma unroll
    for (int j = 0; j < 4; ++j, c += 8, oa += 8 * A.ac, ob += 8 * A.bc) {
      if (r < A.R && c < A.C) {
        if (A.a_t) ta[ty + 8 * j][tx] = to_f32(ap[oa]);
        if (kBinary && A.b_t) tb[kBinary ? ty + 8 * j : 0][tx] = to_f32(bp[ob]);
      }
    }
  }
  __syncthreads();
  const int64_t c = c0 + tx;
  int64_t r = r0 + ty;
  int64_t oa = r * A.ar + c * A.ac, ob = kBinary ? r * A.br + c * A.bc : 0;
  T* op = out + (bz * A.R + r) * A.C + c;
#pragma unroll
  for (int j = 0; j < 4; ++j, r += 8, oa += 8 * A.ar, ob += 8 * A.br, op += 8 * A.C) {
    if (r < A.R && c < A.C) {
      const float x = A.a_t ? ta[tx][ty + 8 * j] : to_f32(ap[oa]);
      float res;
      if (OP == OP_RELU) res = x <= 0.f ? 0.f : x;
      else if (OP == OP_COPY) res = x;
      else if (OP == OP_ADDC) res = x + alpha;
      else if (OP == OP_MULC) res = x * alpha;
      else {
        const float y = A.b_t ? tb[kBinary ? tx : 0][ty + 8 * j] : to_f32(bp[ob]);
        res = OP == OP_ADD ? fmaf(alpha, y, x) : x * y;
      }
      *op = from_f32<T>(res);
    }
  }
}

template <int OP>
static void launch_tiled(const void* a, const void* b, void* out, const TiledArgs& T, int dta, int dtb, int dto, float alpha, cudaStream_t st) {
  constexpr bool kBinary = OP == OP_ADD || OP == OP_MUL;
  const dim3 g(static_cast<unsigned>((T.C + 31) / 32), static_cast<unsigned>((T.R + 31) / 32), static_cast<unsigned>(T.B));
  if (dta == dto && (!kBinary || dtb == dto)) {
    switch (dto) {
      case B200_F32: ew_tiled_typed<float, OP><<<g, 256, 0, st>>>(static_cast<const float*>(a), static_cast<const float*>(b), static_cast<float*>(out), T, alpha); return;
      case B200_BF16: ew_tiled_typed<__nv_bfloat16, OP><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), static_cast<__nv_bfloat16*>(out), T, alpha); return;
      case B200_F16: ew_tiled_typed<__half, OP><<<g, 256, 0, st>>>(static_cast<const __half*>(a), static_cast<const __half*>(b), static_cast<__half*>(out), T, alpha); return;
      default: break;
    }
  }
  ew_tiled<OP><<<g, 256, 0, st>>>(a, b, out, T, dta, dtb, dto, alpha);
}

template <typename U>
__global__ void __launch_bounds__(256) copy_tiled_bits(const U* __restrict__ x, U* __restrict__ out, TiledArgs T) {
  __shared__ U t[32][32 + (sizeof(U) >= 4 ? 1 : (4 / sizeof(U)))];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 32, c0 = static_cast<int64_t>(blockIdx.x) * 32, bz = blockIdx.z;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int64_t r = r0 + tx, c = c0 + ty + 8 * j;
    if (r < T.R && c < T.C) t[ty + 8 * j][tx] = x[bz * T.ab + r * T.ar + c * T.ac];
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int64_t r = r0 + ty + 8 * j, c = c0 + tx;
    if (r < T.R && c < T.C) out[(bz * T.R + r) * T.C + c] = t[tx][ty + 8 * j];
  }
}

// Fills T and returns true when the iteration shape has 2 or 3 dims and at least one operand
// is a transposed view of its last two dims (and the grid fits).
static bool plan_tiled(TiledArgs& T, const StridedArgs& A, bool has_b) {
  if (A.ndim != 2 && A.ndim != 3) return false;
  const int dr = A.ndim - 2, dc = A.ndim - 1;
  T.B = A.ndim == 3 ? A.shape[0] : 1;
  T.R = A.shape[dr];
  T.C = A.shape[dc];
  T.ab = A.ndim == 3 ? A.s0[0] : 0; T.ar = A.s0[dr]; T.ac = A.s0[dc];
  T.bb = A.ndim == 3 ? A.s1[0] : 0; T.br = A.s1[dr]; T.bc = A.s1[dc];
  T.a_t = transposed_view(T.ar, T.ac, T.R, T.C) ? 1 : 0;
  T.b_t = has_b && transposed_view(T.br, T.bc, T.R, T.C) ? 1 : 0;
  if (!T.a_t && !T.b_t) return false;
  return T.B <= 65535 && (T.R + 31) / 32 <= 65535 && (T.C + 31) / 32 <= 0x7fffffffLL;
}
static dim3 tiled_grid(const TiledArgs& T) { return dim3(static_cast<unsigned>((T.C + 31) / 32), static_cast<unsigned>((T.R + 31) / 32), static_cast<unsigned>(T.B)); }

static int fill_args(StridedArgs& A, int ndim, const int64_t* shape, const int64_t* s0, const int64_t* s1, const int64_t* s2) {
  if (ndim < 0 || ndim > B200_MAX_DIMS || (ndim > 0 && !shape)) return B200_EINVAL;
  A.ndim = ndim;
  A.n = 1;
  for (int d = 0; d < ndim; ++d) {
    if (shape[d] < 0) return B200_EINVAL;
    A.shape[d] = shape[d];
    A.n *= shape[d];
    A.s0[d] = s0 ? s0[d] : 0;
    A.s1[d] = s1 ? s1[d] : 0;
    A.s2[d] = s2 ? s2[d] : 0;
  }
  return B200_OK;
}

static int strided_grid(int64_t n) {
  int64_t g = (n + kEwThreads - 1) / kEwThreads;
  const int64_t cap = static_cast<int64_t>(kNumSMs) * 32;
  return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

template <typename Op>
static int launch_unary_fast(const void* x, void* out, int64_t n, int dtype, Op op, cudaStream_t st) {
  const int per_block = kEwThreads * kUnroll;
  switch (dtype) {
    case B200_F32: ew_unary_vec<float, Op><<<grid_for(n / 4 + 1, per_block), kEwThreads, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(out), n, op); break;
    case B200_BF16: ew_unary_vec<__nv_bfloat16, Op><<<grid_for(n / 8 + 1, per_block), kEwThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), n, op); break;
    case B200_F16: ew_unary_vec<__half, Op><<<grid_for(n / 8 + 1, per_block), kEwThreads, 0, st>>>(static_cast<const __half*>(x), static_cast<__half*>(out), n, op); break;
    default: return B200_EDTYPE;
  }
  return check_launch();
}

template <typename T, typename Op>
static void launch_binary_T(const void* a, const void* b, void* out, int64_t n, int mode, Op op, cudaStream_t st) {
  const int g = grid_for(n / Vec<T>::N + 1, kEwThreads * kUnroll);
  const T* pa = static_cast<const T*>(a);
  const T* pb = static_cast<const T*>(b);
  T* po = static_cast<T*>(out);
  if (mode == 0) ew_binary_vec<T, Op, 0><<<g, kEwThreads, 0, st>>>(pa, pb, po, n, op);
  else if (mode == 1) ew_binary_vec<T, Op, 1><<<g, kEwThreads, 0, st>>>(pa, pb, po, n, op);
  else ew_binary_vec<T, Op, 2><<<g, kEwThreads, 0, st>>>(pa, pb, po, n, op);
}

// ------------------------------------------------------------------ rows with a broadcast partner
// out[r, c] = f(a[r, c], b[r, c]) over a contiguous [R, C] result, where each operand is
// either contiguous along c (column stride 1, any row stride, 0 included: a bias vector) or
// constant along c (column stride 0: one value per row). The bias add and the per-row scale
// of ordinary model code; the generic strided kernel would pay an index decomposition per
// element. A thread produces 16 bytes of a row (VEC: rows, bases and C on the 16-byte grid)
// or one element; one 32-bit division per thread and trip finds its row.
struct Rows2dArgs {
  int64_t R, C;
  int64_t ar, br;  // row strides, elements
  int a_c, b_c;    // column stride: 1 or 0
};
template <typename T, int OP, bool VEC>
__global__ void __launch_bounds__(256) ew_rows2d(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, Rows2dArgs A, float alpha) {
  constexpr int VE = VEC ? 16 / static_cast<int>(sizeof(T)) : 1;
  const int64_t per_row = A.C / VE, total = A.R * per_row;
  const bool small = total <= 0x7fffffffLL;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t r, g;
    if (small) {
      const uint32_t q = static_cast<uint32_t>(i) / static_cast<uint32_t>(per_row);
      r = q;
      g = static_cast<uint32_t>(i) - q * static_cast<uint32_t>(per_row);
    } else {
      r = i / per_row;
      g = i - r * per_row;
    }
    const int64_t c = g * VE;
    float x[VE], y[VE], res[VE];
    if (VEC) {
      if (A.a_c) widen<T>(ld_stream(a + r * A.ar + c), x);
      if (A.b_c) widen<T>(ld_stream(b + r * A.br + c), y);
    } else {
      if (A.a_c) x[0] = to_f32(a[r * A.ar + c]);
      if (A.b_c) y[0] = to_f32(b[r * A.br + c]);
    }
    if (!A.a_c) {
      const float v = to_f32(a[r * A.ar]);
#pragma unroll
      for (int e = 0; e < VE; ++e) x[e] = v;
    }
    if (!A.b_c) {
      const float v = to_f32(b[r * A.br]);
#pragma unroll
      for (int e = 0; e < VE; ++e) y[e] = v;
    }
#pragma unroll
    for (int e = 0; e < VE; ++e) res[e] = OP == OP_ADD ? fmaf(alpha, y[e], x[e]) : x[e] * y[e];
    if (VEC) st_stream(out + r * A.C + c, narrow<T>(res));
    else out[r * A.C + c] = from_f32<T>(res[0]);
  }
}

// Classifies one operand of an N-d elementwise call against a contiguous [R, C] result
// (C = the last extent): contiguous, a last-dim vector (all other strides 0), or -- for 2-d
// calls -- a column (one value per row). Returns false for anything else.
static bool rows2d_operand(int ndim, const int64_t* shape, const int64_t* s, int64_t C, int64_t& row_stride, int& col_stride) {
  if (is_contiguous(ndim, shape, s)) { row_stride = C; col_stride = 1; return true; }
  bool lead_zero = true;
  for (int d = 0; d + 1 < ndim; ++d) lead_zero = lead_zero && (s[d] == 0 || shape[d] == 1);
  if (lead_zero && (s[ndim - 1] == 1 || shape[ndim - 1] == 1)) { row_stride = 0; col_stride = 1; return true; }
  if (ndim == 2 && s[1] == 0) { row_stride = shape[0] == 1 ? 0 : s[0]; col_stride = 0; return true; }
  if (ndim == 2 && s[1] == 1 && s[0] >= shape[1]) { row_stride = s[0]; col_stride = 1; return true; }  // a row-pitched matrix
  return false;
}
template <typename T, int OP>
static void launch_rows2d_T(const void* a, const void* b, void* out, const Rows2dArgs& A, float alpha, cudaStream_t st) {
  constexpr int VE = 16 / static_cast<int>(sizeof(T));
  const bool a_ok = !A.a_c || (aligned16(a) && A.ar % VE == 0), b_ok = !A.b_c || (aligned16(b) && A.br % VE == 0);
  const bool vec = A.C % VE == 0 && aligned16(out) && a_ok && b_ok;
  const int64_t work = A.R * (vec ? A.C / VE : A.C);
  const int g = strided_grid(work);
  if (vec) ew_rows2d<T, OP, true><<<g, 256, 0, st>>>(static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), A, alpha);
  else ew_rows2d<T, OP, false><<<g, 256, 0, st>>>(static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), A, alpha);
}

template <typename Op, int OPCODE>
static int binary_entry(const void* a, const void* b, void* out, int ndim, const int64_t* shape, const int64_t* sa, const int64_t* sb, int dta, int dtb, int dto, Op op, float alpha, cudaStream_t st) {
  StridedArgs A;
  if (int rc = fill_args(A, ndim, shape, sa, sb, nullptr)) return rc;
  if (!is_float_dtype(dta) || !is_float_dtype(dtb) || !is_float_dtype(dto)) return B200_EDTYPE;
  if (A.n == 0) return B200_OK;
  if (!a || !b || !out) return B200_EINVAL;
  const bool same = dta == dtb && dtb == dto;
  const bool a_full = is_contiguous(ndim, shape, sa), b_full = is_contiguous(ndim, shape, sb);
  const bool a_scalar = all_zero_strides(ndim, shape, sa), b_scalar = all_zero_strides(ndim, shape, sb);
  int mode = -1;
  if (same && aligned16(out)) {
    if (a_full && b_full && aligned16(a) && aligned16(b)) mode = 0;
    else if (a_full && b_scalar && aligned16(a) && A.n > 1) mode = 1;
    else if (a_scalar && b_full && aligned16(b) && A.n > 1) mode = 2;
  }
  if (mode >= 0) {
    switch (dto) {
      case B200_F32: launch_binary_T<float, Op>(a, b, out, A.n, mode, op, st); break;
      case B200_BF16: launch_binary_T<__nv_bfloat16, Op>(a, b, out, A.n, mode, op, st); break;
      default: launch_binary_T<__half, Op>(a, b, out, A.n, mode, op, st); break;
    }
  } else {
    TiledArgs T;
    Rows2dArgs R2;
    R2.C = ndim > 0 ? shape[ndim - 1] : 1;
    R2.R = R2.C > 0 ? A.n / R2.C : 0;
    if (same && ndim >= 1 && R2.C > 0 && rows2d_operand(ndim, shape, sa, R2.C, R2.ar, R2.a_c) && rows2d_operand(ndim, shape, sb, R2.C, R2.br, R2.b_c)) {
      switch (dto) {
        case B200_F32: launch_rows2d_T<float, OPCODE>(a, b, out, R2, alpha, st); break;
        case B200_BF16: launch_rows2d_T<__nv_bfloat16, OPCODE>(a, b, out, R2, alpha, st); break;
        default: launch_rows2d_T<__half, OPCODE>(a, b, out, R2, alpha, st); break;
      }
    } else if (plan_tiled(T, A, true)) {
      launch_tiled<OPCODE>(a, b, out, T, dta, dtb, dto, alpha, st);
    } else {
      ew_strided<OPCODE><<<strided_grid(A.n), kEwThreads, 0, st>>>(a, b, out, A, dta, dtb, dto, alpha);
    }
  }
  return check_launch();
}

}  // namespace b200

using namespace b200;

extern "C" int b200_relu(const void* x, void* out, int ndim, const int64_t* shape, const int64_t* sx, int dtype, void* stream) {
  StridedArgs A;
  if (int rc = fill_args(A, ndim, shape, sx, nullptr, nullptr)) return rc;
  if (!is_float_dtype(dtype)) return B200_EDTYPE;
  if (A.n == 0) return B200_OK;
  if (!x || !out) return B200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_contiguous(ndim, shape, sx) && aligned16(x) && aligned16(out)) return launch_unary_fast(x, out, A.n, dtype, ReluOp{}, st);
  TiledArgs T;
  if (plan_tiled(T, A, false)) launch_tiled<OP_RELU>(x, nullptr, out, T, dtype, dtype, dtype, 0.f, st);
  else ew_strided<OP_RELU><<<strided_grid(A.n), kEwThreads, 0, st>>>(x, nullptr, out, A, dtype, dtype, dtype, 0.f);
  return check_launch();
}

template <typename Op, int OPCODE>
static int scalar_entry(const void* x, void* out, int ndim, const int64_t* shape, const int64_t* sx, int dtx, int dto, Op op, float c, cudaStream_t st) {
  StridedArgs A;
  if (int rc = fill_args(A, ndim, shape, sx, nullptr, nullptr)) return rc;
  if (!is_float_dtype(dtx) || !is_float_dtype(dto)) return B200_EDTYPE;
  if (A.n == 0) return B200_OK;
  if (!x || !out) return B200_EINVAL;
  if (dtx == dto && is_contiguous(ndim, shape, sx) && aligned16(x) && aligned16(out)) return launch_unary_fast(x, out, A.n, dtx, op, st);
  TiledArgs T;
  if (plan_tiled(T, A, false)) launch_tiled<OPCODE>(x, nullptr, out, T, dtx, dtx, dto, c, st);
  else ew_strided<OPCODE><<<strided_grid(A.n), kEwThreads, 0, st>>>(x, nullptr, out, A, dtx, dtx, dto, c);
  return check_launch();
}

extern "C" int b200_add_scalar(const void* x, void* out, int ndim, const int64_t* shape, const int64_t* sx, int dtx, int dto, double value, void* stream) {
  const float c = static_cast<float>(value);
  return scalar_entry<AddConstOp, OP_ADDC>(x, out, ndim, shape, sx, dtx, dto, AddConstOp{c}, c, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_mul_scalar(const void* x, void* out, int ndim, const int64_t* shape, const int64_t* sx, int dtx, int dto, double value, void* stream) {
  const float c = static_cast<float>(value);
  return scalar_entry<MulConstOp, OP_MULC>(x, out, ndim, shape, sx, dtx, dto, MulConstOp{c}, c, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_add(const void* a, const void* b, void* out, int ndim, const int64_t* shape, const int64_t* sa, const int64_t* sb, int dta, int dtb, int dto, double alpha, void* stream) {
  const float al = static_cast<float>(alpha);
  return binary_entry<AddOp, OP_ADD>(a, b, out, ndim, shape, sa, sb, dta, dtb, dto, AddOp{al}, al, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_mul(const void* a, const void* b, void* out, int ndim, const int64_t* shape, const int64_t* sa, const int64_t* sb, int dta, int dtb, int dto, void* stream) {
  return binary_entry<MulOp, OP_MUL>(a, b, out, ndim, shape, sa, sb, dta, dtb, dto, MulOp{}, 1.f, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_where(const void* cond, const void* x, const void* y, void* out, int ndim, const int64_t* shape, const int64_t* sc, const int64_t* sx, const int64_t* sy, int dtx, int dty, int dto, void* stream) {
  StridedArgs A;
  if (int rc = fill_args(A, ndim, shape, sc, sx, sy)) return rc;
  const int es = dtype_size(dto);
  if (es == 0 || dtype_size(dtx) == 0 || dtype_size(dty) == 0) return B200_EDTYPE;
  if (A.n == 0) return B200_OK;
  if (!cond || !x || !y || !out) return B200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint8_t* c = static_cast<const uint8_t*>(cond);
  const bool same = dtx == dty && dty == dto;
  if (!same && !(is_float_dtype(dtx) && is_float_dtype(dty) && is_float_dtype(dto))) return B200_EDTYPE;
  const bool contig = is_contiguous(ndim, shape, sc) && is_contiguous(ndim, shape, sx) && is_contiguous(ndim, shape, sy);
  if (same && contig && (es == 2 || es == 4) && aligned16(x) && aligned16(y) && aligned16(out) && (reinterpret_cast<uintptr_t>(cond) & 7u) == 0) {
    if (es == 4) ew_where_vec<uint32_t><<<grid_for(A.n / 4 + 1, kEwThreads * kUnroll), kEwThreads, 0, st>>>(c, static_cast<const uint32_t*>(x), static_cast<const uint32_t*>(y), static_cast<uint32_t*>(out), A.n);
    else ew_where_vec<uint16_t><<<grid_for(A.n / 8 + 1, kEwThreads * kUnroll), kEwThreads, 0, st>>>(c, static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(y), static_cast<uint16_t*>(out), A.n);
    return check_launch();
  }
  const int g = strided_grid(A.n);
  if (same) {
    switch (es) {
      case 1: where_strided<uint8_t, true><<<g, kEwThreads, 0, st>>>(c, x, y, out, A, dtx, dty, dto); break;
      case 2: where_strided<uint16_t, true><<<g, kEwThreads, 0, st>>>(c, x, y, out, A, dtx, dty, dto); break;
      case 4: where_strided<uint32_t, true><<<g, kEwThreads, 0, st>>>(c, x, y, out, A, dtx, dty, dto); break;
      default: where_strided<uint64_t, true><<<g, kEwThreads, 0, st>>>(c, x, y, out, A, dtx, dty, dto); break;
    }
  } else {
    where_strided<uint32_t, false><<<g, kEwThreads, 0, st>>>(c, x, y, out, A, dtx, dty, dto);
  }
  return check_launch();
}

extern "C" int b200_copy_strided(const void* x, void* out, int ndim, const int64_t* shape, const int64_t* sx, int dti, int dto, void* stream) {
  StridedArgs A;
  if (int rc = fill_args(A, ndim, shape, sx, nullptr, nullptr)) return rc;
  const int es = dtype_size(dti);
  if (es == 0 || dtype_size(dto) == 0) return B200_EDTYPE;
  if (A.n == 0) return B200_OK;
  if (!x || !out) return B200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int g = strided_grid(A.n);
  TiledArgs T;
  if (plan_tiled(T, A, false)) {
    if (dti != dto) {
      if (!is_float_dtype(dto)) return B200_EDTYPE;
      launch_tiled<OP_COPY>(x, nullptr, out, T, dti, dti, dto, 0.f, st);
    } else {
      switch (es) {
        case 1: copy_tiled_bits<uint8_t><<<tiled_grid(T), 256, 0, st>>>(static_cast<const uint8_t*>(x), static_cast<uint8_t*>(out), T); break;
        case 2: copy_tiled_bits<uint16_t><<<tiled_grid(T), 256, 0, st>>>(static_cast<const uint16_t*>(x), static_cast<uint16_t*>(out), T); break;
        case 4: copy_tiled_bits<uint32_t><<<tiled_grid(T), 256, 0, st>>>(static_cast<const uint32_t*>(x), static_cast<uint32_t*>(out), T); break;
        default: copy_tiled_bits<uint64_t><<<tiled_grid(T), 256, 0, st>>>(static_cast<const uint64_t*>(x), static_cast<uint64_t*>(out), T); break;
      }
    }
    return check_launch();
  }
  if (dti == dto) {
    switch (es) {
      case 1: copy_strided_bits<uint8_t><<<g, kEwThreads, 0, st>>>(static_cast<const uint8_t*>(x), static_cast<uint8_t*>(out), A); break;
      case 2: copy_strided_bits<uint16_t><<<g, kEwThreads, 0, st>>>(static_cast<const uint16_t*>(x), static_cast<uint16_t*>(out), A); break;
      case 4: copy_strided_bits<uint32_t><<<g, kEwThreads, 0, st>>>(static_cast<const uint32_t*>(x), static_cast<uint32_t*>(out), A); break;
      default: copy_strided_bits<uint64_t><<<g, kEwThreads, 0, st>>>(static_cast<const uint64_t*>(x), static_cast<uint64_t*>(out), A); break;
    }
  } else {
    if (!is_float_dtype(dto)) return B200_EDTYPE;
    ew_strided<OP_COPY><<<g, kEwThreads, 0, st>>>(x, nullptr, out, A, dti, dti, dto, 0.f);
  }
  return check_launch();
}

extern "C" int b200_copy_pitched(const void* x, void* out, int64_t batch, int64_t rows, int64_t cols, int64_t sxb, int64_t sxr, int64_t sxc, int64_t out_batch_pitch,
                                 int64_t out_row_pitch, int elem_size, void* stream) {
  if (batch < 0 || rows < 0 || cols < 0 || out_row_pitch < cols) return B200_EINVAL;
  if (batch == 0 || rows == 0 || cols == 0) return B200_OK;
  if (!x || !out) return B200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int64_t blocks = (batch * rows + kEwThreads / 32 - 1) / (kEwThreads / 32);
  if (blocks > kNumSMs * 16LL) blocks = kNumSMs * 16LL;
  const int g = static_cast<int>(blocks);
  switch (elem_size) {
    case 2: copy_pitched<uint16_t><<<g, kEwThreads, 0, st>>>(static_cast<const uint16_t*>(x), static_cast<uint16_t*>(out), batch, rows, cols, sxb, sxr, sxc, out_batch_pitch, out_row_pitch); break;
    case 4: copy_pitched<uint32_t><<<g, kEwThreads, 0, st>>>(static_cast<const uint32_t*>(x), static_cast<uint32_t*>(out), batch, rows, cols, sxb, sxr, sxc, out_batch_pitch, out_row_pitch); break;
    default: return B200_EDTYPE;
  }
  return check_launch();
}

extern "C" int b200_copy_into(const void* x, void* out, int ndim, const int64_t* shape, const int64_t* sx, const int64_t* so, int elem_size, void* stream) {
  StridedArgs A;
  if (int rc = fill_args(A, ndim, shape, sx, so, nullptr)) return rc;
  if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8) return B200_EDTYPE;
  if (A.n == 0) return B200_OK;
  if (!x || !out || !sx || !so) return B200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int g = strided_grid(A.n);
  switch (elem_size) {
    case 1: copy_between_strided<uint8_t><<<g, kEwThreads, 0, st>>>(static_cast<const uint8_t*>(x), static_cast<uint8_t*>(out), A); break;
    case 2: copy_between_strided<uint16_t><<<g, kEwThreads, 0, st>>>(static_cast<const uint16_t*>(x), static_cast<uint16_t*>(out), A); break;
    case 4: copy_between_strided<uint32_t><<<g, kEwThreads, 0, st>>>(static_cast<const uint32_t*>(x), static_cast<uint32_t*>(out), A); break;
    default: copy_between_strided<uint64_t><<<g, kEwThreads, 0, st>>>(static_cast<const uint64_t*>(x), static_cast<uint64_t*>(out), A); break;
  }
  return check_launch();
}
