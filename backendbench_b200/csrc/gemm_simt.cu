// CUDA-core GEMM: the path for fp32 operands (full fp32 products, like aten's default
// with TF32 off) and for any layout the tensor-core kernel cannot take (odd strides,
// unaligned bases, K not a multiple of 8). Arbitrary element strides, fp32 accumulate,
// one rounding. Output tile per CTA chosen by shape (128x128 down to 128x32 / 32x128),
// 16-deep K slices staged in shared memory.
#include "b200_common.cuh"

namespace b200 {

constexpr int kTK = 16;

struct GemmArgs {
  int64_t M, N, K;
  int64_t sAb, sAm, sAk, sBb, sBk, sBn, sbm, sbn;
  float alpha, beta;
  const uint32_t* gate;  // when not NULL: the kernel does its work only if this device word is non-zero
};

// TM x TN outputs per CTA (256 threads, (TM/16) x (TN/16) per thread), 16-deep K slices.
// The next slice is fetched from global memory into registers while the current one is
// multiplied out of shared memory, so one barrier pair per slice is the only serialisation.
// Tile shapes: 128x128 for large problems, 64x64 / 128x32 / 32x128 when M or N is small.
template <typename T, int kTM, int kTN>
__global__ void __launch_bounds__(256) gemm_simt(const T* __restrict__ A, const T* __restrict__ B, const T* __restrict__ bias, T* __restrict__ C, GemmArgs g) {
  __shared__ __align__(16) float As[kTK][kTM + 4];
  __shared__ __align__(16) float Bs[kTK][kTN + 4];
  if (g.gate && *g.gate == 0u) return;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kTM, n0 = static_cast<int64_t>(blockIdx.x) * kTN;
  const int64_t b = blockIdx.z;
  const T* Ab = A + b * g.sAb;
  const T* Bb = B + b * g.sBb;
  const bool a_kfast = g.sAk == 1, b_nfast = g.sBn == 1;
  constexpr int RM = kTM / 16, RN = kTN / 16;        // outputs per thread
  constexpr int QA = kTM * kTK / 256, QB = kTN * kTK / 256;  // slice elements per thread
  float acc[RM][RN] = {};
  float pa[QA], pb[QB];
  auto fetch = [&](int64_t k0) {
#pragma unroll
    for (int q = 0; q < QA; ++q) {
      const int e = tid + q * 256;
      // consecutive threads walk the contiguous direction of the operand
      const int kk = a_kfast ? (e & 15) : (e / kTM), mm = a_kfast ? (e >> 4) : (e % kTM);
      const int64_t m = m0 + mm, k = k0 + kk;
      pa[q] = (m < g.M && k < g.K) ? to_f32(Ab[m * g.sAm + k * g.sAk]) : 0.f;
    }
#pragma unroll
    for (int q = 0; q < QB; ++q) {
      const int e = tid + q * 256;
      const int kk = b_nfast ? (e / kTN) : (e & 15), nn = b_nfast ? (e % kTN) : (e >> 4);
      const int64_t n = n0 + nn, k = k0 + kk;
      pb[q] = (n < g.N && k < g.K) ? to_f32(Bb[k * g.sBk + n * g.sBn]) : 0.f;
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int q = 0; q < QA; ++q) {
      const int e = tid + q * 256;
      As[a_kfast ? (e & 15) : (e / kTM)][a_kfast ? (e >> 4) : (e % kTM)] = pa[q];
    }
#pragma unroll
    for (int q = 0; q < QB; ++q) {
      const int e = tid + q * 256;
      Bs[b_nfast ? (e / kTN) : (e & 15)][b_nfast ? (e % kTN) : (e >> 4)] = pb[q];
    }
  };
  fetch(0);
  for (int64_t k0 = 0; k0 < g.K; k0 += kTK) {
    stash();
    __syncthreads();
    if (k0 + kTK < g.K) fetch(k0 + kTK);
#pragma unroll
    for (int kk = 0; kk < kTK; ++kk) {
      float a[RM], bb[RN];
#pragma unroll
      for (int i = 0; i < RM; ++i) a[i] = As[kk][ty * RM + i];
#pragma unroll
      for (int j = 0; j < RN; ++j) bb[j] = Bs[kk][tx * RN + j];
#pragma unroll
      for (int i = 0; i < RM; ++i)
#pragma unroll
        for (int j = 0; j < RN; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
    }
    __syncthreads();
  }
  T* Cb = C + b * g.M * g.N;
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    const int64_t m = m0 + ty * RM + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < RN; ++j) {
      const int64_t n = n0 + tx * RN + j;
      if (n >= g.N) continue;
      float r = g.alpha * acc[i][j];
      // beta == 0 drops the bias term entirely (a NaN bias must not leak through)
      if (bias && g.beta != 0.f) r = fmaf(g.beta, to_f32(bias[m * g.sbm + n * g.sbn]), r);
      Cb[m * g.N + n] = from_f32<T>(r);
    }
  }
}

template <typename T, int kTM, int kTN>
static int launch_simt_tile(const void* A, const void* B, const void* bias, void* C, int64_t batch, const GemmArgs& g, cudaStream_t st) {
  const int64_t gx = (g.N + kTN - 1) / kTN, gy = (g.M + kTM - 1) / kTM;
  if (gx > 0x7fffffffLL || gy > 65535) return B200_EINVAL;
  for (int64_t b0 = 0; b0 < batch; b0 += 65535) {
    const int64_t bn = batch - b0 < 65535 ? batch - b0 : 65535;
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(bn));
    gemm_simt<T, kTM, kTN><<<grid, 256, 0, st>>>(static_cast<const T*>(A) + b0 * g.sAb, static_cast<const T*>(B) + b0 * g.sBb, static_cast<const T*>(bias), static_cast<T*>(C) + b0 * g.M * g.N, g);
  }
  return check_launch();
}

template <typename T>
static int launch_simt(const void* A, const void* B, const void* bias, void* C, int64_t batch, const GemmArgs& g, cudaStream_t st) {
  // big tiles only when they are mostly full and there are enough of them to fill the GPU
  const int64_t big_tiles = batch * ((g.M + 127) / 128) * ((g.N + 127) / 128);
  if (g.M >= 96 && g.N >= 96 && big_tiles >= kNumSMs) return launch_simt_tile<T, 128, 128>(A, B, bias, C, batch, g, st);
  if (g.N <= 40 && g.M >= 96) return launch_simt_tile<T, 128, 32>(A, B, bias, C, batch, g, st);
  if (g.M <= 40 && g.N >= 96) return launch_simt_tile<T, 32, 128>(A, B, bias, C, batch, g, st);
  return launch_simt_tile<T, 64, 64>(A, B, bias, C, batch, g, st);
}

int gemm_simt_dispatch(const void* A, const void* B, const void* bias, void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk,
                       int64_t sBb, int64_t sBk, int64_t sBn, int64_t sbm, int64_t sbn, double alpha, double beta, int dtype, cudaStream_t st, const uint32_t* gate) {
  GemmArgs g{M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, sbm, sbn, static_cast<float>(alpha), static_cast<float>(beta), gate};
  switch (dtype) {
    case B200_F32: return launch_simt<float>(A, B, bias, C, batch, g, st);
    case B200_BF16: return launch_simt<__nv_bfloat16>(A, B, bias, C, batch, g, st);
    case B200_F16: return launch_simt<__half>(A, B, bias, C, batch, g, st);
    default: return B200_EDTYPE;
  }
}

}  // namespace b200
