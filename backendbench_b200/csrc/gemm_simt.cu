// CUDA-core GEMM: the path for fp32 operands (full fp32 products, like aten's default
// with TF32 off) and for any layout the tensor-core kernel cannot take (odd strides,
// unaligned bases, K not a multiple of 8). Arbitrary element strides, fp32 accumulate,
// one rounding. 64x64 output tile per CTA, 16-deep K slices staged in shared memory,
// 4x4 outputs per thread.
#include "b200_common.cuh"

namespace b200 {

constexpr int kTM = 64, kTN = 64, kTK = 16;

struct GemmArgs {
  int64_t M, N, K;
  int64_t sAb, sAm, sAk, sBb, sBk, sBn, sbm, sbn;
  float alpha, beta;
};

template <typename T>
__global__ void __launch_bounds__(256) gemm_simt(const T* __restrict__ A, const T* __restrict__ B, const T* __restrict__ bias, T* __restrict__ C, GemmArgs g) {
  __shared__ float As[kTK][kTM + 4];
  __shared__ float Bs[kTK][kTN + 4];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kTM, n0 = static_cast<int64_t>(blockIdx.x) * kTN;
  const int64_t b = blockIdx.z;
  const T* Ab = A + b * g.sAb;
  const T* Bb = B + b * g.sBb;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < g.K; k0 += kTK) {
    // 64x16 A slice and 16x64 B slice: 1024 elements each, 4 per thread
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int e = tid + q * 256;
      {
        // A: consecutive threads walk k when A is k-contiguous, m otherwise
        const int kk = g.sAk == 1 ? (e & 15) : (e >> 6), mm = g.sAk == 1 ? (e >> 4) : (e & 63);
        const int64_t m = m0 + mm, k = k0 + kk;
        As[kk][mm] = (m < g.M && k < g.K) ? to_f32(Ab[m * g.sAm + k * g.sAk]) : 0.f;
      }
      {
        const int kk = g.sBn == 1 ? (e >> 6) : (e & 15), nn = g.sBn == 1 ? (e & 63) : (e >> 4);
        const int64_t n = n0 + nn, k = k0 + kk;
        Bs[kk][nn] = (n < g.N && k < g.K) ? to_f32(Bb[k * g.sBk + n * g.sBn]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTK; ++kk) {
      float a[4], bb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bb[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
    }
    __syncthreads();
  }
  T* Cb = C + b * g.M * g.N;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n >= g.N) continue;
      float r = g.alpha * acc[i][j];
      // beta == 0 drops the bias term entirely (a NaN bias must not leak through)
      if (bias && g.beta != 0.f) r = fmaf(g.beta, to_f32(bias[m * g.sbm + n * g.sbn]), r);
      Cb[m * g.N + n] = from_f32<T>(r);
    }
  }
}

template <typename T>
static int launch_simt(const void* A, const void* B, const void* bias, void* C, int64_t batch, const GemmArgs& g, cudaStream_t st) {
  const int64_t gx = (g.N + kTN - 1) / kTN, gy = (g.M + kTM - 1) / kTM;
  if (gx > 0x7fffffffLL || gy > 65535) return B200_EINVAL;
  for (int64_t b0 = 0; b0 < batch; b0 += 65535) {
    const int64_t bn = batch - b0 < 65535 ? batch - b0 : 65535;
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(bn));
    gemm_simt<T><<<grid, 256, 0, st>>>(static_cast<const T*>(A) + b0 * g.sAb, static_cast<const T*>(B) + b0 * g.sBb, static_cast<const T*>(bias), static_cast<T*>(C) + b0 * g.M * g.N, g);
  }
  return check_launch();
}

int gemm_simt_dispatch(const void* A, const void* B, const void* bias, void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk,
                       int64_t sBb, int64_t sBk, int64_t sBn, int64_t sbm, int64_t sbn, double alpha, double beta, int dtype, cudaStream_t st) {
  GemmArgs g{M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, sbm, sbn, static_cast<float>(alpha), static_cast<float>(beta)};
  switch (dtype) {
    case B200_F32: return launch_simt<float>(A, B, bias, C, batch, g, st);
    case B200_BF16: return launch_simt<__nv_bfloat16>(A, B, bias, C, batch, g, st);
    case B200_F16: return launch_simt<__half>(A, B, bias, C, batch, g, st);
    default: return B200_EDTYPE;
  }
}

}  // namespace b200
