// Small 16-bit products (mm / addmm / bmm): a few dozen 64 x 64 tiles, K up to 256. The tcgen05 kernel pays about 5 us before its first result (tensor-memory
// allocation, barrier set-up, the first TMA round trip, the tile store) and computes 128-row
// tiles whatever M is; the CUDA-core kernel has no tensor cores at all. Here a CTA of four
// warps owns a 64 x 64 tile of C and walks K in slices of 64 through a four-stage ring of
// `cp.async` copies (16 bytes along each operand's contiguous direction: base and strides
// are on the 16-byte grid, or the product goes elsewhere); the warps read their
// fragments with `ldmatrix` (transposing where the operand is stored along M or N) and
// multiply with `mma.sync.m16n8k16` into fp32 accumulators. alpha, beta and the bias are
// applied in fp32 and the result is rounded once. C contiguous.
#include <type_traits>

#include "b200_common.cuh"

namespace b200 {

namespace {

constexpr int kMT = 64, kNT = 64, kKT = 64;  // tile of C, K slice
constexpr int kMmaThreads = 128;
constexpr int kMmaStages = 4;      // 256 k in flight per CTA: a product this small is a chain of global-memory round trips, nothing else
constexpr int kPitchK = kKT + 8;   // elements per row of a tile stored [mn][k]: 144 bytes
constexpr int kPitchMN = kMT + 8;  // elements per row of a tile stored [k][mn]: 144 bytes
constexpr int kOperandElems = kMT * kPitchK;  // one operand's 64 x 64 slice, either layout
static_assert(kMT == kNT && kMT == kKT, "one slice geometry for both operands and both layouts");
constexpr int kMmaSmem = kMmaStages * 2 * kOperandElems * 2;  // bytes (dynamic: above the 48 KB of static shared memory)

struct MmaArgs {
  int64_t M, N, K;
  int64_t sAb, sAm, sAk, sBb, sBk, sBn, sbm, sbn;
  float alpha, beta;
};

__device__ __forceinline__ void cp16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (std::is_same<T, __nv_bfloat16>::value) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// One operand's 64 x 64 slice into shared memory. `mn_fast`: the operand is contiguous along
// M (resp. N) and the tile is stored [k][mn]; otherwise it is stored [mn][k]. Eight elements
// (16 bytes) per copy along the contiguous direction, zero-filled past the edges.
template <typename T>
__device__ __forceinline__ void load_slice(T* tile, const T* base, int64_t s_mn, int64_t s_k, int64_t mn0, int64_t k0, int64_t mn_lim, int64_t k_lim, bool mn_fast, int tid) {
  // 512 chunks of 8 elements per slice, four per thread
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int e = tid + q * kMmaThreads;
    const int row = e >> 3, col8 = (e & 7) * 8;
    int64_t mn, k;
    if (mn_fast) {  // rows of the tile are k, eight mn per chunk
      k = k0 + row;
      mn = mn0 + col8;
    } else {  // rows of the tile are mn, eight k per chunk
      mn = mn0 + row;
      k = k0 + col8;
    }
    T* dst = tile + row * kPitchK + col8;
    const int64_t left = mn_fast ? (k < k_lim ? mn_lim - mn : 0) : (mn < mn_lim ? k_lim - k : 0);  // elements of this chunk that exist
    const int bytes = left >= 8 ? 16 : (left > 0 ? static_cast<int>(left) * 2 : 0);
    cp16(static_cast<uint32_t>(__cvta_generic_to_shared(dst)), bytes ? base + mn * s_mn + k * s_k : base, bytes);
  }
}

template <typename T>
__global__ void __launch_bounds__(kMmaThreads) gemm_mma_small(const T* __restrict__ A, const T* __restrict__ B, const T* __restrict__ bias, T* __restrict__ C, MmaArgs g) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T(*smem)[2][kOperandElems] = reinterpret_cast<T(*)[2][kOperandElems]>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 1, wn = warp & 1;  // the warp's 32 x 32 quarter of the tile
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kMT, n0 = static_cast<int64_t>(blockIdx.x) * kNT;
  const int64_t b = blockIdx.z;
  const T* Ab = A + b * g.sAb;
  const T* Bb = B + b * g.sBb;
  const bool a_mfast = g.sAm == 1 && g.sAk != 1, b_nfast = g.sBn == 1 && g.sBk != 1;  // an operand with both strides 1 counts as K-major
  const bool b_kfast_layout = !b_nfast;
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;
  const int nslices = static_cast<int>((g.K + kKT - 1) / kKT);
  // (Skipping the 16 x 16 blocks of a warp's quarter that are pure padding was tried: the tests
  // cost more registers and time than the multiplications they saved.)
  auto issue = [&](int s) {
    if (s < nslices) {
      const int st = s % kMmaStages;
      load_slice<T>(smem[st][0], Ab, g.sAm, g.sAk, m0, static_cast<int64_t>(s) * kKT, g.M, g.K, a_mfast, tid);
      load_slice<T>(smem[st][1], Bb, g.sBn, g.sBk, n0, static_cast<int64_t>(s) * kKT, g.N, g.K, b_nfast, tid);
    }
    cp_commit();  // an empty group past the end keeps the count in step
  };
#pragma unroll
  for (int s = 0; s < kMmaStages - 1; ++s) issue(s);
  for (int s = 0; s < nslices; ++s) {
    cp_wait<kMmaStages - 2>();  // this thread's copies of slice s have landed ...
    __syncthreads();            // ... and everybody's; the stage refilled below was consumed before this barrier
    issue(s + kMmaStages - 1);
    const T* at = smem[s % kMmaStages][0];
    const T* bt = smem[s % kMmaStages][1];
#pragma unroll
    for (int kk = 0; kk < kKT; kk += 16) {
      uint32_t af[2][4], bf[2][4];  // bf[p]: the two k halves of columns 16 p .. 16 p + 7 and 16 p + 8 .. 16 p + 15
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int mrow = wm * 32 + i * 16;
        if (a_mfast) {  // stored [k][m]: transposing read
          const int krow = kk + (lane & 7) + (lane >> 4) * 8, mcol = mrow + ((lane >> 3) & 1) * 8;
          ldsm_x4_trans(static_cast<uint32_t>(__cvta_generic_to_shared(at + krow * kPitchMN + mcol)), af[i]);
        } else {  // stored [m][k]
          const int row = mrow + (lane & 15), kcol = kk + (lane >> 4) * 8;
          ldsm_x4(static_cast<uint32_t>(__cvta_generic_to_shared(at + row * kPitchK + kcol)), af[i]);
        }
      }
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        const int ncol = wn * 32 + p * 16;
        if (b_kfast_layout) {  // stored [n][k]
          const int nrow = ncol + (lane & 7) + (lane >> 4) * 8, kcol = kk + ((lane >> 3) & 1) * 8;
          ldsm_x4(static_cast<uint32_t>(__cvta_generic_to_shared(bt + nrow * kPitchK + kcol)), bf[p]);
        } else {  // stored [k][n]: transposing read
          const int krow = kk + (lane & 7) + ((lane >> 3) & 1) * 8, nc = ncol + (lane >> 4) * 8;
          ldsm_x4_trans(static_cast<uint32_t>(__cvta_generic_to_shared(bt + krow * kPitchMN + nc)), bf[p]);
        }
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int p = 0; p < 2; ++p) {
          mma16816<T>(acc[i][2 * p], af[i], bf[p][0], bf[p][1]);
          mma16816<T>(acc[i][2 * p + 1], af[i], bf[p][2], bf[p][3]);
        }
    }
  }
  cp_wait<0>();
  // ---- epilogue: alpha, beta * bias, one rounding; a thread holds rows g, g + 8 and columns 2 t, 2 t + 1 of each 16 x 8 block
  T* Cb = C + b * g.M * g.N;
  const int gq = lane >> 2, tq = lane & 3;
  const bool with_bias = bias != nullptr && g.beta != 0.f;  // beta == 0 drops the bias term entirely (a NaN bias must not leak through)
  const bool pair_ok = (g.N & 1) == 0 && (reinterpret_cast<uintptr_t>(C) & 3u) == 0;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int64_t m = m0 + wm * 32 + i * 16 + gq + h * 8;
      if (m >= g.M) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int64_t n = n0 + wn * 32 + j * 8 + tq * 2;
        if (n >= g.N) continue;
        float v0 = g.alpha * acc[i][j][2 * h], v1 = g.alpha * acc[i][j][2 * h + 1];
        if (with_bias) {
          v0 = fmaf(g.beta, to_f32(bias[m * g.sbm + n * g.sbn]), v0);
          if (n + 1 < g.N) v1 = fmaf(g.beta, to_f32(bias[m * g.sbm + (n + 1) * g.sbn]), v1);
        }
        T* dst = Cb + m * g.N + n;
        if (pair_ok && n + 1 < g.N) {
          T pr[2] = {from_f32<T>(v0), from_f32<T>(v1)};
          *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(pr);
        } else {
          dst[0] = from_f32<T>(v0);
          if (n + 1 < g.N) dst[1] = from_f32<T>(v1);
        }
      }
    }
}

}  // namespace

// Worth it for a product of a few dozen tiles with a short contraction whose operands can be
// copied 16 bytes at a time; anything larger belongs to the tcgen05 kernel (or its K split),
// operands off the 16-byte grid to the CUDA-core kernel (this kernel's element-by-element
// staging is not pipelined: 227 x 256 x 65 took 13 us here against 8 us there).
static bool operand_on_grid(const void* base, int64_t s_mn, int64_t s_k, int64_t s_b) {
  const bool mn_fast = s_mn == 1 && s_k != 1;
  return (mn_fast ? s_k % 8 == 0 : (s_k == 1 && s_mn % 8 == 0)) && s_b % 8 == 0 && (reinterpret_cast<uintptr_t>(base) & 15u) == 0;
}
bool gemm_mma_small_preferred(const void* A, const void* B, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk, int64_t sBb, int64_t sBk, int64_t sBn,
                              int dtype) {
  if (dtype != B200_BF16 && dtype != B200_F16) return false;
  if (batch < 1 || M < 1 || N < 1 || K < 1 || batch > 65535) return false;
  const int64_t tiles = batch * ((M + kMT - 1) / kMT) * ((N + kNT - 1) / kNT);
  // (K = 512 in one tile took 9.5 us here against 6.1 us on the tcgen05 kernel: mma.sync is the slow
  // path of this part, about 0.8 us per 64 k of a tile; 16384 x 256 x 16, 256 tiles: 7.8 us both ways)
  if (!(tiles <= kNumSMs && K <= 256 && batch * M * N * K <= (1LL << 26) && (M + kMT - 1) / kMT <= 65535)) return false;
  return operand_on_grid(A, sAm, sAk, batch > 1 ? sAb : 0) && operand_on_grid(B, sBn, sBk, batch > 1 ? sBb : 0);
}

int gemm_mma_small_dispatch(const void* A, const void* B, const void* bias, void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk, int64_t sBb,
                            int64_t sBk, int64_t sBn, int64_t sbm, int64_t sbn, double alpha, double beta, int dtype, cudaStream_t st) {
  const MmaArgs g{M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, sbm, sbn, static_cast<float>(alpha), static_cast<float>(beta)};
  const dim3 grid(static_cast<unsigned>((N + kNT - 1) / kNT), static_cast<unsigned>((M + kMT - 1) / kMT), static_cast<unsigned>(batch));
  const cudaError_t ae = dtype == B200_BF16 ? cudaFuncSetAttribute(gemm_mma_small<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMmaSmem)
                                            : cudaFuncSetAttribute(gemm_mma_small<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMmaSmem);
  if (ae != cudaSuccess) { set_last_cuda_error(ae); return B200_ELAUNCH; }
  if (dtype == B200_BF16)
    gemm_mma_small<__nv_bfloat16><<<grid, kMmaThreads, kMmaSmem, st>>>(static_cast<const __nv_bfloat16*>(A), static_cast<const __nv_bfloat16*>(B), static_cast<const __nv_bfloat16*>(bias),
                                                                static_cast<__nv_bfloat16*>(C), g);
  else
    gemm_mma_small<__half><<<grid, kMmaThreads, kMmaSmem, st>>>(static_cast<const __half*>(A), static_cast<const __half*>(B), static_cast<const __half*>(bias), static_cast<__half*>(C), g);
  return check_launch();
}

}  // namespace b200
