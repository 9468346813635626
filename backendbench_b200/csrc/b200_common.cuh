// Shared device/host helpers for the libb200ops kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200ops.h"

namespace b200 {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

// ---------------------------------------------------------------- error plumbing
const char* set_last_cuda_error(cudaError_t e);
void note_launches(int n);  // feeds b200_launch_count()
inline int check_launch(int launches = 1) {
  note_launches(launches);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    return B200_ELAUNCH;
  }
  return B200_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int dtype_size(int dt) {
  switch (dt) {
    case B200_F32: case B200_I32: return 4;
    case B200_BF16: case B200_F16: case B200_I16: return 2;
    case B200_I64: case B200_F64: return 8;
    case B200_BOOL: case B200_U8: case B200_I8: return 1;
    default: return 0;
  }
}
inline bool is_float_dtype(int dt) { return dt == B200_F32 || dt == B200_BF16 || dt == B200_F16; }

// ---------------------------------------------------------------- scalar conversion
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// Runtime-typed scalar access for the strided (slow) paths.
__device__ __forceinline__ float load_as_f32(const void* p, int64_t i, int dt) {
  switch (dt) {
    case B200_F32: return static_cast<const float*>(p)[i];
    case B200_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    case B200_F16: return __half2float(static_cast<const __half*>(p)[i]);
    case B200_I32: return static_cast<float>(static_cast<const int32_t*>(p)[i]);
    case B200_I64: return static_cast<float>(static_cast<const int64_t*>(p)[i]);
    case B200_BOOL: case B200_U8: return static_cast<float>(static_cast<const uint8_t*>(p)[i]);
    case B200_I8: return static_cast<float>(static_cast<const int8_t*>(p)[i]);
    case B200_I16: return static_cast<float>(static_cast<const int16_t*>(p)[i]);
    case B200_F64: return static_cast<float>(static_cast<const double*>(p)[i]);
    default: return 0.f;
  }
}
__device__ __forceinline__ void store_from_f32(void* p, int64_t i, int dt, float v) {
  switch (dt) {
    case B200_F32: static_cast<float*>(p)[i] = v; break;
    case B200_BF16: static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v); break;
    case B200_F16: static_cast<__half*>(p)[i] = __float2half_rn(v); break;
    default: break;
  }
}

// ---------------------------------------------------------------- 16-byte vectors
// Vec<T> is one 16-byte global transaction worth of T.
template <typename T> struct Vec {
  static constexpr int N = 16 / sizeof(T);
  uint4 raw;
  __device__ __forceinline__ T get(int i) const { return reinterpret_cast<const T*>(&raw)[i]; }
  __device__ __forceinline__ void set(int i, T v) { reinterpret_cast<T*>(&raw)[i] = v; }
};

// Whole-vector conversions written on the packed words, so that each element costs one
// instruction on the way in (a shift or a mask for bf16, one convert for f16) and half an
// instruction on the way out (packed round-to-nearest-even converts).
template <typename T> __device__ __forceinline__ void widen(const uint4& raw, float* f);
template <> __device__ __forceinline__ void widen<float>(const uint4& raw, float* f) {
  f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
}
template <> __device__ __forceinline__ void widen<__nv_bfloat16>(const uint4& raw, float* f) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <> __device__ __forceinline__ void widen<__half>(const uint4& raw, float* f) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = p.x;
    f[2 * i + 1] = p.y;
  }
}
template <typename T> __device__ __forceinline__ uint4 narrow(const float* f);
template <> __device__ __forceinline__ uint4 narrow<float>(const float* f) {
  return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
}
template <> __device__ __forceinline__ uint4 narrow<__nv_bfloat16>(const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&p);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <> __device__ __forceinline__ uint4 narrow<__half>(const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 p = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&p);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Mixed-precision add / subtract (sm_100a): one 16-bit operand widened inside the
// instruction, so a packed row can feed fp32 arithmetic without a separate unpack. The
// result is that of widening first (the conversion is exact). `w` holds two elements;
// they are taken low half first, the order `widen` gives them.
template <typename T> struct Mixed;
template <> struct Mixed<__nv_bfloat16> {
  static __device__ __forceinline__ void add2(float& s, uint32_t w) {
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tadd.rn.f32.bf16 %0, lo, %0;\n\tadd.rn.f32.bf16 %0, hi, %0;\n\t}" : "+f"(s) : "r"(w));
  }
  static __device__ __forceinline__ void sub2(uint32_t w, float c, float& d0, float& d1) {
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tsub.rn.f32.bf16 %0, lo, %3;\n\tsub.rn.f32.bf16 %1, hi, %3;\n\t}" : "=f"(d0), "=f"(d1) : "r"(w), "f"(c));
  }
};
template <> struct Mixed<__half> {
  static __device__ __forceinline__ void add2(float& s, uint32_t w) {
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tadd.rn.f32.f16 %0, lo, %0;\n\tadd.rn.f32.f16 %0, hi, %0;\n\t}" : "+f"(s) : "r"(w));
  }
  static __device__ __forceinline__ void sub2(uint32_t w, float c, float& d0, float& d1) {
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tsub.rn.f32.f16 %0, lo, %3;\n\tsub.rn.f32.f16 %1, hi, %3;\n\t}" : "=f"(d0), "=f"(d1) : "r"(w), "f"(c));
  }
};
// sum += the elements of a packed vector; d[e] = element e - c
template <typename T> __device__ __forceinline__ void vec_accumulate(float& s, const uint4& raw) {
  if constexpr (sizeof(T) == 4) {
    s += __uint_as_float(raw.x); s += __uint_as_float(raw.y); s += __uint_as_float(raw.z); s += __uint_as_float(raw.w);
  } else {
    Mixed<T>::add2(s, raw.x); Mixed<T>::add2(s, raw.y); Mixed<T>::add2(s, raw.z); Mixed<T>::add2(s, raw.w);
  }
}
template <typename T> __device__ __forceinline__ void vec_minus(const uint4& raw, float c, float* d) {
  if constexpr (sizeof(T) == 4) {
    d[0] = __uint_as_float(raw.x) - c; d[1] = __uint_as_float(raw.y) - c; d[2] = __uint_as_float(raw.z) - c; d[3] = __uint_as_float(raw.w) - c;
  } else {
    Mixed<T>::sub2(raw.x, c, d[0], d[1]); Mixed<T>::sub2(raw.y, c, d[2], d[3]); Mixed<T>::sub2(raw.z, c, d[4], d[5]); Mixed<T>::sub2(raw.w, c, d[6], d[7]);
  }
}

// Streaming (evict-first) accesses: the memory-bound kernels touch every byte once.
__device__ __forceinline__ uint4 ld_stream(const void* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void st_stream(void* p, uint4 v) { __stcs(reinterpret_cast<uint4*>(p), v); }
// Read-only data that other CTAs re-read (weights, gather sources): keep in L2.
__device__ __forceinline__ uint4 ld_keep(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

// ---------------------------------------------------------------- warp / block reductions
template <typename F> __device__ __forceinline__ float warp_reduce(float v, F f) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = f(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
struct MaxF { __device__ __forceinline__ float operator()(float a, float b) const { return fmaxf(a, b); } };
// Maximum over the warp in one instruction; like fmaxf it passes over NaN inputs.
__device__ __forceinline__ float warp_reduce(float v, MaxF) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
struct SumF { __device__ __forceinline__ float operator()(float a, float b) const { return a + b; } };

// Reduce across the whole CTA; every thread gets the result. `smem` holds >= 33 floats.
template <typename F> __device__ __forceinline__ float block_reduce(float v, F f, float identity, float* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_reduce(v, f);
  __syncthreads();  // protect smem reuse between consecutive calls
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? smem[lane] : identity;
    t = warp_reduce(t, f);
    if (lane == 0) smem[32] = t;
  }
  __syncthreads();
  return smem[32];
}

// Same result with one barrier: every warp leaves its partial in shared memory and every
// warp then reduces the partials itself. `smem` holds >= 64 floats in two halves;
// consecutive calls in one kernel pass alternating `phase` (0, 1, 0, ...) so that a call
// never overwrites partials a slower warp is still reading from the call before.
template <typename F> __device__ __forceinline__ float block_reduce_once(float v, F f, float identity, float* smem, int phase) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  float* part = smem + 32 * phase;
  v = warp_reduce(v, f);
  if (lane == 0) part[warp] = v;
  __syncthreads();
  return warp_reduce(lane < nwarps ? part[lane] : identity, f);
}

// 2^x by the special-function unit alone (results below 2^-126 flush to zero).
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---------------------------------------------------------------- strided index math
struct Dims {
  int ndim;
  int64_t shape[B200_MAX_DIMS];
};
struct Strides {
  int64_t s[B200_MAX_DIMS];
};

inline bool is_contiguous(int ndim, const int64_t* shape, const int64_t* strides) {
  int64_t expect = 1;
  for (int d = ndim - 1; d >= 0; --d) {
    if (shape[d] == 1) continue;
    if (strides[d] != expect) return false;
    expect *= shape[d];
  }
  return true;
}
inline int64_t numel_of(int ndim, const int64_t* shape) {
  int64_t n = 1;
  for (int d = 0; d < ndim; ++d) n *= shape[d];
  return n;
}
inline bool all_zero_strides(int ndim, const int64_t* shape, const int64_t* strides) {
  for (int d = 0; d < ndim; ++d)
    if (shape[d] != 1 && strides[d] != 0) return false;
  return true;
}

inline int grid_for(int64_t work_items, int per_block) {
  int64_t g = (work_items + per_block - 1) / per_block;
  if (g < 1) g = 1;
  if (g > 0x7fffffffLL) g = 0x7fffffffLL;
  return static_cast<int>(g);
}

}  // namespace b200
