// CUDA-core GEMM: the path for fp32 operands (full fp32 products, like aten's default
// with TF32 off) and for any layout the tensor-core kernel cannot take (odd strides,
// unaligned bases, K not a multiple of 8). Arbitrary element strides, fp32 accumulate,
// one rounding. Output tile per CTA chosen by shape (128x128 down to 128x32 / 32x128),
// 16-deep K slices staged in shared memory. A product with a long contraction and an output
// of only a few tiles is split along K over the CTAs of a thread-block cluster, which add
// their partial tiles through distributed shared memory in rank order (no scratch buffer,
// no atomics: the result does not depend on scheduling).
#include <cooperative_groups.h>

#include <cstdlib>
#include <type_traits>

#include "b200_common.cuh"

namespace b200 {
namespace cg = cooperative_groups;

constexpr int kTK = 16;

struct GemmArgs {
  int64_t M, N, K;
  int64_t sAb, sAm, sAk, sBb, sBk, sBn, sbm, sbn;
  float alpha, beta;
  const uint32_t* gate;  // when not NULL: the kernel does its work only if this device word is non-zero
  int ksplit;            // CTAs per cluster sharing one output tile (KSPLIT kernels), else 1
  int64_t kchunk;        // K elements per CTA of the cluster, a multiple of kTK
};

// Copies of 4 or 16 bytes global -> shared that complete in the background. `bytes` of the
// source are read (0 .. size), the rest of the destination is filled with zeros.
__device__ __forceinline__ void cp_async4_zfill(void* smem_dst, const void* gsrc, bool valid) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(gsrc), "r"(valid ? 4 : 0) : "memory");
}
__device__ __forceinline__ void cp_async16_zfill(void* smem_dst, const void* gsrc, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// K slices in flight per CTA for fp32 operands (16-bit operands go through registers, one
// slice ahead: they are converted on the way into shared memory)
template <typename T, int kTM, int kTN> struct SimtStages { static constexpr int value = 1; };
template <int kTM, int kTN> struct SimtStages<float, kTM, kTN> { static constexpr int value = (kTM + kTN > 192) ? 2 : 4; };

// TM x TN outputs per CTA (256 threads, (TM/16) x (TN/16) per thread), 16-deep K slices.
// fp32 operands: the slices arrive through a ring of `cp.async` stages (4 for the small
// tiles, 2 for 128 x 128), 16 bytes per copy where the operand is contiguous along the
// tile's row of shared memory and aligned, 4 bytes otherwise, zero-filled past the edges; one
// barrier per slice. A CTA that walked K one global-memory round trip per slice took 1.5 us a
// slice (21 x 1024 x 256 in 64 batches: 98 us). 16-bit operands: the next slice is fetched
// into registers while the current one is multiplied out of shared memory.
// Tile shapes: 128x128 for large problems, 64x64 / 128x32 / 32x128 when M or N is small.
// KSPLIT: launched as clusters of g.ksplit CTAs along z; CTA s of a cluster contracts the K
// range [s * kchunk, (s + 1) * kchunk) of the same output tile, leaves its partial tile in
// shared memory, and after a cluster barrier every CTA finishes a share of the tile's
// elements, adding the partials of ranks 0 .. ksplit-1 in that order.
// AROWS (fp32, A with unit K stride, rows and base on the 16-byte grid): a stage keeps A as
// [m][k] -- 16-byte copies along K, four k of a row per 16-byte read in the product -- instead
// of [k][m]; the common row-major A then costs kTM / 64 copies per thread and slice, not kTM / 16.
template <typename T, int kTM, int kTN, bool KSPLIT, bool AROWS = false>
__global__ void __launch_bounds__(256) gemm_simt(const T* __restrict__ A, const T* __restrict__ B, const T* __restrict__ bias, T* __restrict__ C, GemmArgs g) {
  constexpr bool kAsync = SimtStages<T, kTM, kTN>::value > 1;
  static_assert(!AROWS || kAsync, "the [m][k] stage layout belongs to the cp.async path");
  constexpr int kAPitch = AROWS ? kTK + 4 : kTM + 4;  // floats per row of the A part of a stage
  constexpr int kAFloats = AROWS ? kTM * kAPitch : kTK * kAPitch;
  constexpr int kStageFloats = kAFloats + kTK * (kTN + 4);
  constexpr int kS = (SimtStages<T, kTM, kTN>::value == 4 && 4 * kStageFloats * 4 > 48 * 1024) ? 3 : SimtStages<T, kTM, kTN>::value;  // static shared memory ends at 48 KB
  constexpr int kPartFloats = KSPLIT ? kTM * kTN : 4;
  // the partial tile of a K split reuses the stage ring once the contraction is done
  __shared__ __align__(16) float smem[(kS * kStageFloats > kPartFloats) ? kS * kStageFloats : kPartFloats];
  auto As = [&](int st) { return reinterpret_cast<float(*)[kAPitch]>(smem + st * kStageFloats); };
  auto Bs = [&](int st) { return reinterpret_cast<float(*)[kTN + 4]>(smem + st * kStageFloats + kAFloats); };
  float* part = smem;
  if (g.gate && *g.gate == 0u) return;  // the same word for every CTA: whole clusters leave together
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kTM, n0 = static_cast<int64_t>(blockIdx.x) * kTN;
  const int nsplit = KSPLIT ? g.ksplit : 1;
  const int64_t b = KSPLIT ? blockIdx.z / nsplit : blockIdx.z;
  const int rank = KSPLIT ? static_cast<int>(blockIdx.z % nsplit) : 0;
  const int64_t k_lo = KSPLIT ? rank * g.kchunk : 0;
  const int64_t k_hi = KSPLIT ? (k_lo + g.kchunk < g.K ? k_lo + g.kchunk : g.K) : g.K;
  const T* Ab = A + b * g.sAb;
  const T* Bb = B + b * g.sBb;
  const bool a_kfast = g.sAk == 1, b_nfast = g.sBn == 1;
  constexpr int RM = kTM / 16, RN = kTN / 16;        // outputs per thread
  constexpr int QA = kTM * kTK / 256, QB = kTN * kTK / 256;  // slice elements per thread
  float acc[RM][RN] = {};
  // Columns of C a thread owns: groups of four adjacent ones, 64 apart (one 16-byte read of a
  // B row per group; the 16 threads of a row of the CTA read 256 contiguous bytes), or every
  // 16th column for the 32-wide tile. Eight adjacent columns per thread, read one by one, put
  // the 16 threads on four banks (34 shared-memory wavefronts per k instead of 6:
  // 21 x 1024 x 256 in 64 batches took 98 us for that reason alone).
  auto col = [&](int j) { return (RN % 4 == 0) ? (j / 4) * 64 + tx * 4 + (j % 4) : tx + 16 * j; };
  auto load_b = [&](const float(*bs)[kTN + 4], int kk, float* bb) {
    if constexpr (RN % 4 == 0) {
#pragma unroll
      for (int j = 0; j < RN; j += 4) *reinterpret_cast<float4*>(bb + j) = *reinterpret_cast<const float4*>(&bs[kk][(j / 4) * 64 + tx * 4]);
    } else {
#pragma unroll
      for (int j = 0; j < RN; ++j) bb[j] = bs[kk][tx + 16 * j];
    }
  };
  auto multiply = [&](int st) {
    const float(*as)[kAPitch] = As(st);
    const float(*bs)[kTN + 4] = Bs(st);
    if constexpr (AROWS) {
#pragma unroll
      for (int k4 = 0; k4 < kTK; k4 += 4) {
        float a[RM][4];
#pragma unroll
        for (int i = 0; i < RM; ++i) *reinterpret_cast<float4*>(a[i]) = *reinterpret_cast<const float4*>(&as[ty * RM + i][k4]);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float bb[RN];
          load_b(bs, k4 + u, bb);
#pragma unroll
          for (int i = 0; i < RM; ++i)
#pragma unroll
            for (int j = 0; j < RN; ++j) acc[i][j] = fmaf(a[i][u], bb[j], acc[i][j]);
        }
      }
    } else {
#pragma unroll
      for (int kk = 0; kk < kTK; ++kk) {
        float a[RM], bb[RN];
        if constexpr (RM % 4 == 0) {
#pragma unroll
          for (int i = 0; i < RM; i += 4) *reinterpret_cast<float4*>(a + i) = *reinterpret_cast<const float4*>(&as[kk][ty * RM + i]);
        } else {
          *reinterpret_cast<float2*>(a) = *reinterpret_cast<const float2*>(&as[kk][ty * RM]);
        }
        load_b(bs, kk, bb);
#pragma unroll
        for (int i = 0; i < RM; ++i)
#pragma unroll
          for (int j = 0; j < RN; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
      }
    }
  };
  static_assert(RM == 2 || RM % 4 == 0, "rows per thread: 2, 4 or 8");
  if constexpr (kAsync) {
    // Every copy a thread issues has the same place in the tile for all slices: its source
    // pointer (advanced by one slice per issue), its destination offset inside a stage, its
    // first k inside the slice and whether its row / column exists are worked out once.
    // Rows of shared memory that are contiguous in global memory and on the 16-byte grid
    // there travel 16 bytes per copy (A along K with AROWS, A along M or B along N otherwise).
    struct Copy { const float* src; uint32_t dst; int kq; int bytes; };  // bytes: what exists of the copy's row (0 = zeros only, -1 = no such copy)
    const bool a_vec = !AROWS && g.sAm == 1 && g.sAk % 4 == 0 && g.sAb % 4 == 0 && (reinterpret_cast<uintptr_t>(A) & 15u) == 0;
    const bool b_vec = g.sBn == 1 && g.sBk % 4 == 0 && g.sBb % 4 == 0 && (reinterpret_cast<uintptr_t>(B) & 15u) == 0;
    constexpr int NA = AROWS ? (kTM * 4 + 255) / 256 : QA, NB = QB;
    Copy ca[NA], cb[NB];
    const uint32_t smem_a = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int na = AROWS ? NA : (a_vec ? (QA + 3) / 4 : QA), nb = b_vec ? (QB + 3) / 4 : QB;
#pragma unroll
    for (int q = 0; q < NA; ++q) {
      const int e = tid + q * 256;
      int kk, mm, span;  // span: elements along the copy's contiguous direction
      if (AROWS) { mm = e >> 2; kk = (e & 3) * 4; span = 1; }
      else if (a_vec) { kk = e / (kTM / 4); mm = (e % (kTM / 4)) * 4; span = 4; }
      else { kk = a_kfast ? (e & 15) : (e / kTM); mm = a_kfast ? (e >> 4) : (e % kTM); span = 1; }
      const bool in_tile = AROWS ? e < kTM * 4 : (a_vec ? e < kTM * kTK / 4 : true);
      const int64_t m = m0 + mm, left = g.M - m;
      ca[q].kq = kk;
      ca[q].bytes = !in_tile ? -1 : left > 0 ? (AROWS ? 16 : (left >= span ? span * 4 : static_cast<int>(left) * 4)) : 0;
      ca[q].src = ca[q].bytes > 0 ? Ab + m * g.sAm + (k_lo + kk) * g.sAk : Ab;
      ca[q].dst = smem_a + 4u * static_cast<uint32_t>(AROWS ? mm * kAPitch + kk : kk * kAPitch + mm);
    }
#pragma unroll
    for (int q = 0; q < NB; ++q) {
      const int e = tid + q * 256;
      int kk, nn, span;
      if (b_vec) { kk = e / (kTN / 4); nn = (e % (kTN / 4)) * 4; span = 4; }
      else { kk = b_nfast ? (e / kTN) : (e & 15); nn = b_nfast ? (e % kTN) : (e >> 4); span = 1; }
      const bool in_tile = b_vec ? e < kTN * kTK / 4 : true;
      const int64_t n = n0 + nn, left = g.N - n;
      cb[q].kq = kk;
      cb[q].bytes = !in_tile ? -1 : left > 0 ? (left >= span ? span * 4 : static_cast<int>(left) * 4) : 0;
      cb[q].src = cb[q].bytes > 0 ? Bb + (k_lo + kk) * g.sBk + n * g.sBn : Bb;
      cb[q].dst = smem_a + 4u * static_cast<uint32_t>(kAFloats + kk * (kTN + 4) + nn);
    }
    const int64_t a_step = kTK * g.sAk, b_step = kTK * g.sBk;
    auto cp16 = [](uint32_t dst, const void* src, int bytes) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory"); };
    auto cp4 = [](uint32_t dst, const void* src, int bytes) { asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory"); };
    auto issue = [&](int64_t k0, int st) {
      if (k0 < k_hi) {
        const int rem = static_cast<int>(k_hi - k0 < kTK ? k_hi - k0 : kTK);  // k of this slice that exist
        const uint32_t stage = static_cast<uint32_t>(st) * (kStageFloats * 4u);
#pragma unroll
        for (int q = 0; q < NA; ++q) {
          if (q < na && ca[q].bytes >= 0) {
            const int r = rem - ca[q].kq;
            if (AROWS) cp16(ca[q].dst + stage, ca[q].src, ca[q].bytes ? (r >= 4 ? 16 : (r > 0 ? r * 4 : 0)) : 0);
            else if (a_vec) cp16(ca[q].dst + stage, ca[q].src, r > 0 ? ca[q].bytes : 0);
            else cp4(ca[q].dst + stage, ca[q].src, r > 0 ? ca[q].bytes : 0);
            if (ca[q].bytes > 0) ca[q].src += a_step;
          }
        }
#pragma unroll
        for (int q = 0; q < NB; ++q) {
          if (q < nb && cb[q].bytes >= 0) {
            const int r = rem - cb[q].kq;
            if (b_vec) cp16(cb[q].dst + stage, cb[q].src, r > 0 ? cb[q].bytes : 0);
            else cp4(cb[q].dst + stage, cb[q].src, r > 0 ? cb[q].bytes : 0);
            if (cb[q].bytes > 0) cb[q].src += b_step;
          }
        }
      }
    cp_async_commit();  // an empty group past the end keeps the group count in step
    };
#pragma unroll
    for (int s = 0; s < kS - 1; ++s) issue(k_lo + s * kTK, s);
    int st = 0;
    for (int64_t k0 = k_lo; k0 < k_hi; k0 += kTK) {
      cp_async_wait<kS - 2>();  // this thread's copies of the current slice have landed ...
      __syncthreads();          // ... and everybody's; the stage refilled below was multiplied out before this barrier
      issue(k0 + (kS - 1) * kTK, st == 0 ? kS - 1 : st - 1);
      multiply(st);
      st = st + 1 == kS ? 0 : st + 1;
    }
    cp_async_wait<0>();
    __syncthreads();  // the ring is free (a K split reuses it for the partial tile)
  } else {
    // kD slices are on their way in registers at any time (four for the small tiles): a
    // contraction of a few slices -- most 16-bit products that come here are small -- costs
    // one global-memory round trip, not one per slice.
    constexpr int kD = (QA + QB <= 8) ? 4 : (QA + QB <= 12 ? 3 : 2);
    T pa[kD][QA], pb[kD][QB];
    auto fetch = [&](int64_t k0, T* ra, T* rb) {
#pragma unroll
      for (int q = 0; q < QA; ++q) {
        const int e = tid + q * 256;
        // consecutive threads walk the contiguous direction of the operand
        const int kk = a_kfast ? (e & 15) : (e / kTM), mm = a_kfast ? (e >> 4) : (e % kTM);
        const int64_t m = m0 + mm, k = k0 + kk;
        ra[q] = (m < g.M && k < k_hi) ? Ab[m * g.sAm + k * g.sAk] : from_f32<T>(0.f);
      }
#pragma unroll
      for (int q = 0; q < QB; ++q) {
        const int e = tid + q * 256;
        const int kk = b_nfast ? (e / kTN) : (e & 15), nn = b_nfast ? (e % kTN) : (e >> 4);
        const int64_t n = n0 + nn, k = k0 + kk;
        rb[q] = (n < g.N && k < k_hi) ? Bb[k * g.sBk + n * g.sBn] : from_f32<T>(0.f);
      }
    };
    auto stash = [&](const T* ra, const T* rb) {
      float(*as)[kTM + 4] = As(0);
      float(*bs)[kTN + 4] = Bs(0);
#pragma unroll
      for (int q = 0; q < QA; ++q) {
        const int e = tid + q * 256;
        as[a_kfast ? (e & 15) : (e / kTM)][a_kfast ? (e >> 4) : (e % kTM)] = to_f32(ra[q]);
      }
#pragma unroll
      for (int q = 0; q < QB; ++q) {
        const int e = tid + q * 256;
        bs[b_nfast ? (e / kTN) : (e & 15)][b_nfast ? (e % kTN) : (e >> 4)] = to_f32(rb[q]);
      }
    };
#pragma unroll
    for (int d = 0; d < kD; ++d)
      if (k_lo + d * kTK < k_hi) fetch(k_lo + d * kTK, pa[d], pb[d]);
    for (int64_t k0 = k_lo; k0 < k_hi; k0 += kD * kTK) {
#pragma unroll
      for (int d = 0; d < kD; ++d) {
        const int64_t kd = k0 + d * kTK;
        if (kd < k_hi) {  // uniform over the CTA
          stash(pa[d], pb[d]);
          __syncthreads();
          if (kd + kD * kTK < k_hi) fetch(kd + kD * kTK, pa[d], pb[d]);
          multiply(0);
          __syncthreads();
        }
      }
    }
  }
  T* Cb = C + b * g.M * g.N;
  if (KSPLIT) {
    cg::cluster_group cluster = cg::this_cluster();
#pragma unroll
    for (int i = 0; i < RM; ++i)
#pragma unroll
      for (int j = 0; j < RN; ++j) part[(ty * RM + i) * kTN + col(j)] = acc[i][j];
    cluster.sync();
    for (int e = rank * 256 + tid; e < kTM * kTN; e += nsplit * 256) {
      float sum = 0.f;
      for (int r = 0; r < nsplit; ++r) sum += cluster.map_shared_rank(part, r)[e];
      const int64_t m = m0 + e / kTN, n = n0 + e % kTN;
      if (m < g.M && n < g.N) {
        float r = g.alpha * sum;
        // beta == 0 drops the bias term entirely (a NaN bias must not leak through)
        if (bias && g.beta != 0.f) r = fmaf(g.beta, to_f32(bias[m * g.sbm + n * g.sbn]), r);
        Cb[m * g.N + n] = from_f32<T>(r);
      }
    }
    cluster.sync();  // nobody leaves while its partial tile may still be read
  } else {
#pragma unroll
    for (int i = 0; i < RM; ++i) {
      const int64_t m = m0 + ty * RM + i;
      if (m >= g.M) continue;
#pragma unroll
      for (int j = 0; j < RN; ++j) {
        const int64_t n = n0 + col(j);
        if (n >= g.N) continue;
        float r = g.alpha * acc[i][j];
        // beta == 0 drops the bias term entirely (a NaN bias must not leak through)
        if (bias && g.beta != 0.f) r = fmaf(g.beta, to_f32(bias[m * g.sbm + n * g.sbn]), r);
        Cb[m * g.N + n] = from_f32<T>(r);
      }
    }
  }
}

// Few output tiles and a long contraction: how many CTAs share a tile (1 = no split). One
// CTA walks K at a slice per global-memory round trip, so with under half the SMs busy the
// time falls with every CTA added (measured: 2 x 2048 x 256 fp32, 192 us unsplit, 41 us
// at 8). Between half a tile and one tile per SM two CTAs per tile still pay for the tiles of
// 64 rows or more (16384 x 1024 x 19: 60 -> 50 us, 16384 x 2060 x 32: 117 -> 87 us,
// 3991 x 4120 x 96: 185 -> 147 us) but not for the 32-row tile, whose CTAs stream a wide B
// and gain nothing from a shorter K (21 x 1024 x 256 in 64 batches: 52 us unsplit, 66-71 us
// split); from one tile per SM on, splitting only adds the exchange. Each CTA keeps at least
// four K slices and the cluster stays within the portable size of 8.
// B200_SIMT_SPLIT_BELOW / B200_SIMT_SPLIT_FILL override the two thresholds (for comparisons).
static int pick_ksplit(int64_t tiles, int64_t K, int tile_rows) {
  static const int64_t env_limit = []() { const char* e = getenv("B200_SIMT_SPLIT_BELOW"); return e ? atoll(e) : 0LL; }();
  static const int64_t env_want = []() { const char* e = getenv("B200_SIMT_SPLIT_FILL"); return e ? atoll(e) : 0LL; }();
  const int64_t limit = env_limit > 0 ? env_limit : (tile_rows >= 64 ? kNumSMs : kNumSMs / 2);
  const int64_t want = env_want > 0 ? env_want : (tiles >= kNumSMs / 2 ? 2 : 4);  // CTAs per SM aimed at
  if (tiles >= limit || K < 8 * kTK) return 1;
  int64_t s = K / (4 * kTK);
  const int64_t fill = (want * kNumSMs + tiles - 1) / tiles;
  if (s > fill) s = fill;
  if (s > 8) s = 8;
  return s < 2 ? 1 : static_cast<int>(s);
}

template <typename T, int kTM, int kTN, bool KSPLIT = false, bool AROWS = false>
static int launch_simt_tile(const void* A, const void* B, const void* bias, void* C, int64_t batch, GemmArgs g, cudaStream_t st) {
  if constexpr (std::is_same<T, float>::value && !AROWS) {
    // row-major fp32 A on the 16-byte grid: the variant that copies it 16 bytes at a time along K
    if (g.sAk == 1 && g.sAm % 4 == 0 && g.sAb % 4 == 0 && aligned16(A)) return launch_simt_tile<T, kTM, kTN, KSPLIT, true>(A, B, bias, C, batch, g, st);
  }
  const int64_t gx = (g.N + kTN - 1) / kTN, gy = (g.M + kTM - 1) / kTM;
  if (gx > 0x7fffffffLL || gy > 65535) return B200_EINVAL;
  const int64_t per_launch = 65535 / g.ksplit;  // batches per launch: grid z holds batch x ksplit
  for (int64_t b0 = 0; b0 < batch; b0 += per_launch) {
    const int64_t bn = batch - b0 < per_launch ? batch - b0 : per_launch;
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(bn * g.ksplit));
    const T* a = static_cast<const T*>(A) + b0 * g.sAb;
    const T* b = static_cast<const T*>(B) + b0 * g.sBb;
    const T* bs = static_cast<const T*>(bias);
    T* c = static_cast<T*>(C) + b0 * g.M * g.N;
    if (KSPLIT) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = grid;
      cfg.blockDim = dim3(256);
      cfg.stream = st;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 1;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = static_cast<unsigned>(g.ksplit);
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_simt<T, kTM, kTN, KSPLIT, AROWS>, a, b, bs, c, g);
      if (e != cudaSuccess) { set_last_cuda_error(e); return B200_ELAUNCH; }
    } else {
      gemm_simt<T, kTM, kTN, KSPLIT, AROWS><<<grid, 256, 0, st>>>(a, b, bs, c, g);
    }
  }
  return check_launch();
}

template <typename T, int kTM, int kTN>
static int launch_simt_small(const void* A, const void* B, const void* bias, void* C, int64_t batch, GemmArgs g, cudaStream_t st) {
  const int64_t tiles = batch * ((g.M + kTM - 1) / kTM) * ((g.N + kTN - 1) / kTN);
  g.ksplit = pick_ksplit(tiles, g.K, kTM);
  if (g.ksplit == 1) return launch_simt_tile<T, kTM, kTN, false>(A, B, bias, C, batch, g, st);
  const int64_t per = (g.K + g.ksplit - 1) / g.ksplit;
  g.kchunk = (per + kTK - 1) / kTK * kTK;
  return launch_simt_tile<T, kTM, kTN, true>(A, B, bias, C, batch, g, st);
}

// ------------------------------------------------------------------ many rows, a few columns
// C has at most 16 columns and A has many rows with unit K stride: the tile kernel above would
// compute mostly padding and walk A in 16-deep slices. Here a THREAD owns a row of C: it
// streams its row of A with 16-byte loads and multiplies by B from shared memory (every lane
// reads the same B element: a broadcast), NN accumulators in registers. A is read once, at
// the rate the load/store unit delivers one 32-byte sector per lane and load. It needs rows
// enough for about four warps per scheduler (one warp alone cannot hide its own shared-memory
// and global latencies: 16384 rows x 2060 x 32 ran 2.5x slower than the tile kernel), and at
// most 16 columns (measured: 524288 rows x 256 x 8 fp32, 0.33 ms on the tile kernel, 0.23 here).
constexpr int kSkinnyThreads = 128;
constexpr int kSkinnyBsFloats = 2048;  // 8 KB of B per K chunk
template <typename T, int NN>
__global__ void __launch_bounds__(kSkinnyThreads) gemm_skinny(const T* __restrict__ A, const T* __restrict__ B, const T* __restrict__ bias, T* __restrict__ C, GemmArgs g) {
  __shared__ __align__(16) float Bs[kSkinnyBsFloats];  // [kc][NN]
  constexpr int VE = 16 / static_cast<int>(sizeof(T));
  constexpr int kc = kSkinnyBsFloats / NN;  // a multiple of VE
  if (g.gate && *g.gate == 0u) return;
  const int64_t b = blockIdx.y;
  const int64_t m = static_cast<int64_t>(blockIdx.x) * kSkinnyThreads + threadIdx.x;
  const bool live = m < g.M;
  const T* arow = A + b * g.sAb + (live ? m : 0) * g.sAm;
  const T* Bb = B + b * g.sBb;
  float acc[NN];
#pragma unroll
  for (int n = 0; n < NN; ++n) acc[n] = 0.f;
  for (int64_t k0 = 0; k0 < g.K; k0 += kc) {
    const int kn = g.K - k0 < kc ? static_cast<int>(g.K - k0) : kc;
    __syncthreads();  // the previous chunk of B has been consumed
    for (int e = threadIdx.x; e < kn * NN; e += kSkinnyThreads) {
      const int kk = e / NN, n = e % NN;
      Bs[e] = n < g.N ? to_f32(Bb[(k0 + kk) * g.sBk + n * g.sBn]) : 0.f;
    }
    __syncthreads();
    if (live) {
      int kk = 0;
#pragma unroll 2
      for (; kk + VE <= kn; kk += VE) {
        float a[VE];
        widen<T>(ld_stream(arow + k0 + kk), a);
#pragma unroll
        for (int u = 0; u < VE; ++u) {
          const float* brow = Bs + (kk + u) * NN;
#pragma unroll
          for (int n = 0; n < NN; ++n) acc[n] = fmaf(a[u], brow[n], acc[n]);
        }
      }
      for (; kk < kn; ++kk) {
        const float a = to_f32(arow[k0 + kk]);
        const float* brow = Bs + kk * NN;
#pragma unroll
        for (int n = 0; n < NN; ++n) acc[n] = fmaf(a, brow[n], acc[n]);
      }
    }
  }
  if (!live) return;
  T* crow = C + (b * g.M + m) * g.N;
#pragma unroll
  for (int n = 0; n < NN; ++n) {
    if (n < g.N) {
      float r = g.alpha * acc[n];
      if (bias && g.beta != 0.f) r = fmaf(g.beta, to_f32(bias[m * g.sbm + n * g.sbn]), r);
      crow[n] = from_f32<T>(r);
    }
  }
}

// The same shape (C at most 16 columns wide, A row-major) with a WARP per row of A: the 32
// lanes read consecutive 16-byte pieces of the row (512 contiguous bytes per load, where the
// thread-per-row kernel above fetches 16 bytes from each of 32 rows), multiply them by B held
// in shared memory as [n][k] (a lane's four or eight k of one column are one 16-byte read, no
// bank conflicts), and fold the NN partial sums of the 32 lanes with a halving exchange: at
// each of the first log2(NN) levels a lane keeps half of its sums and hands the other half to
// its partner (NN - 1 shuffles in all, then one per remaining level), so that lanes 0, 32/NN,
// ... end up with one finished output each. The order of the additions is fixed.
// 8192 x 256 x 8 in 64 batches (fp32): 190 us by thread-per-row, 142 us here, against 83 us for
// reading A once. (16-bit products of this shape that the tensor-core path can load stay there:
// 16384 x 256 x 16 f16 took 12 us here against 7.6 us on the 128-wide tcgen05 tile.)
// One level of the halving exchange of gemm_skinny_warp: WIDTH sums per lane, partner lane ^ OFF.
template <int WIDTH, int OFF>
__device__ __forceinline__ void fold_lanes(float* acc, int lane, int& n_mine) {
  if constexpr (OFF >= 1) {
    if constexpr (WIDTH > 1) {
      constexpr int half = WIDTH / 2;
      const bool upper = (lane & OFF) != 0;
#pragma unroll
      for (int i = 0; i < half; ++i) {
        const float send = upper ? acc[i] : acc[i + half];
        const float keep = upper ? acc[i + half] : acc[i];
        acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, OFF);
      }
      if (upper) n_mine += half;
      fold_lanes<half, OFF / 2>(acc, lane, n_mine);
    } else {
      acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], OFF);
      fold_lanes<1, OFF / 2>(acc, lane, n_mine);
    }
  }
}

constexpr int kSkinnyWarpRows = 4;  // rows of A per warp and trip (their accumulators live in registers across K chunks)
template <typename T, int NN>
__global__ void __launch_bounds__(256, 2) gemm_skinny_warp(const T* __restrict__ A, const T* __restrict__ B, const T* __restrict__ bias, T* __restrict__ C, GemmArgs g) {
  constexpr int VE = 16 / static_cast<int>(sizeof(T));
  constexpr int kc = (kSkinnyBsFloats / NN < 32 * VE) ? 32 * VE : kSkinnyBsFloats / NN;  // k per chunk of B: at least one 16-byte piece per lane
  constexpr int kPitch = kc + 4;                                                       // floats per column of the chunk in shared memory
  __shared__ __align__(16) float Bs[NN * kPitch];
  if (g.gate && *g.gate == 0u) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t b = blockIdx.y;
  const T* Ab = A + b * g.sAb;
  const T* Bb = B + b * g.sBb;
  const int nchunks = static_cast<int>((g.K + kc - 1) / kc);
  const int64_t rows_per_cta = 8 * kSkinnyWarpRows;
  bool staged = false;
  for (int64_t m0 = static_cast<int64_t>(blockIdx.x) * rows_per_cta; m0 < g.M; m0 += static_cast<int64_t>(gridDim.x) * rows_per_cta) {
    float acc[kSkinnyWarpRows][NN];
#pragma unroll
    for (int r = 0; r < kSkinnyWarpRows; ++r)
#pragma unroll
      for (int n = 0; n < NN; ++n) acc[r][n] = 0.f;
    for (int ch = 0; ch < nchunks; ++ch) {
      const int64_t k0 = static_cast<int64_t>(ch) * kc;
      const int kn = g.K - k0 < kc ? static_cast<int>(g.K - k0) : kc;
      if (!(staged && nchunks == 1)) {  // a single chunk stays for every batch of rows of this CTA
        __syncthreads();                // the previous chunk has been consumed
        for (int e = threadIdx.x; e < kc * NN; e += 256) {
          const int kk = e / NN, n = e % NN;  // consecutive threads walk a row of B
          Bs[n * kPitch + kk] = (kk < kn && n < g.N) ? to_f32(Bb[(k0 + kk) * g.sBk + n * g.sBn]) : 0.f;
        }
        __syncthreads();
        staged = true;
      }
      // all 16-byte pieces of this chunk of the warp's rows are requested before the first is used
      constexpr int kPasses = kc / (32 * VE);  // 16-byte pieces of a row's chunk per lane: 2 (fp32), 1 or 2 (16-bit)
      uint4 piece[kSkinnyWarpRows][kPasses];
#pragma unroll
      for (int r = 0; r < kSkinnyWarpRows; ++r) {
        const int64_t m = m0 + warp * kSkinnyWarpRows + r;
        const T* arow = Ab + (m < g.M ? m : 0) * g.sAm + k0;
#pragma unroll
        for (int ps = 0; ps < kPasses; ++ps) {
          const int kk = (ps * 32 + lane) * VE;
          piece[r][ps] = make_uint4(0u, 0u, 0u, 0u);
          if (m < g.M && kk + VE <= kn) {
            piece[r][ps] = ld_stream(arow + kk);
          } else if (m < g.M && kk < kn) {  // the ragged end of K: element by element, zeros beyond
            T tail[VE];
#pragma unroll
            for (int u = 0; u < VE; ++u) tail[u] = kk + u < kn ? arow[kk + u] : from_f32<T>(0.f);
            piece[r][ps] = *reinterpret_cast<const uint4*>(tail);
          }
        }
      }
#pragma unroll
      for (int ps = 0; ps < kPasses; ++ps) {
        const int kk = (ps * 32 + lane) * VE;
        if (ps * 32 * VE < kn) {  // warp-uniform: this pass holds data
#pragma unroll
          for (int n = 0; n < NN; ++n) {
            float bv[VE];
#pragma unroll
            for (int q = 0; q < VE; q += 4) *reinterpret_cast<float4*>(bv + q) = *reinterpret_cast<const float4*>(&Bs[n * kPitch + kk + q]);
#pragma unroll
            for (int r = 0; r < kSkinnyWarpRows; ++r) {
              float a[VE];
              widen<T>(piece[r][ps], a);
#pragma unroll
              for (int u = 0; u < VE; ++u) acc[r][n] = fmaf(a[u], bv[u], acc[r][n]);
            }
          }
        }
      }
    }
    // fold the lanes' partial sums and write the rows
#pragma unroll
    for (int r = 0; r < kSkinnyWarpRows; ++r) {
      const int64_t m = m0 + warp * kSkinnyWarpRows + r;
      int n_mine = 0;
      fold_lanes<NN, 16>(acc[r], lane, n_mine);
      if ((lane & (32 / NN - 1)) == 0 && n_mine < g.N && m < g.M) {
        float v = g.alpha * acc[r][0];
        if (bias && g.beta != 0.f) v = fmaf(g.beta, to_f32(bias[m * g.sbm + n_mine * g.sbn]), v);
        C[(b * g.M + m) * g.N + n_mine] = from_f32<T>(v);
      }
    }
  }
}

template <typename T>
static bool skinny_warp_eligible(const void* A, int64_t batch, const GemmArgs& g) {
  constexpr int VE = 16 / static_cast<int>(sizeof(T));
  // fp32 only: the 16-bit form was measured slower than the kernels it would replace
  return std::is_same<T, float>::value && g.N <= 16 && g.sAk == 1 && g.K >= 32 * VE && g.sAm % VE == 0 && g.sAb % VE == 0 && aligned16(A) && batch <= 65535 && batch * g.M >= 8LL * kNumSMs;
}
template <typename T>
static int launch_skinny_warp(const void* A, const void* B, const void* bias, void* C, int64_t batch, const GemmArgs& g, cudaStream_t st) {
  const int64_t per_cta = 8 * kSkinnyWarpRows;
  int64_t gx = (g.M + per_cta - 1) / per_cta;
  const int64_t cap = (16LL * kNumSMs + batch - 1) / batch;  // about 16 CTAs per SM in all: a CTA with one chunk of B keeps it for all its rows
  if (gx > cap) gx = cap < 1 ? 1 : cap;
  const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(batch));
  const T* a = static_cast<const T*>(A);
  const T* b = static_cast<const T*>(B);
  const T* bs = static_cast<const T*>(bias);
  T* c = static_cast<T*>(C);
  if (g.N <= 8) gemm_skinny_warp<T, 8><<<grid, 256, 0, st>>>(a, b, bs, c, g);
  else gemm_skinny_warp<T, 16><<<grid, 256, 0, st>>>(a, b, bs, c, g);
  return check_launch();
}

template <typename T>
static bool skinny_eligible(const void* A, int64_t batch, const GemmArgs& g) {
  constexpr int VE = 16 / static_cast<int>(sizeof(T));
  return g.N <= 16 && g.sAk == 1 && g.K >= 16 && g.sAm % VE == 0 && g.sAb % VE == 0 && aligned16(A) && batch <= 65535 && batch * g.M >= 16LL * 32 * kNumSMs &&
         (g.M + kSkinnyThreads - 1) / kSkinnyThreads <= 0x7fffffffLL;
}
template <typename T>
static int launch_skinny(const void* A, const void* B, const void* bias, void* C, int64_t batch, const GemmArgs& g, cudaStream_t st) {
  const dim3 grid(static_cast<unsigned>((g.M + kSkinnyThreads - 1) / kSkinnyThreads), static_cast<unsigned>(batch));
  const T* a = static_cast<const T*>(A);
  const T* b = static_cast<const T*>(B);
  const T* bs = static_cast<const T*>(bias);
  T* c = static_cast<T*>(C);
  if (g.N <= 8) gemm_skinny<T, 8><<<grid, kSkinnyThreads, 0, st>>>(a, b, bs, c, g);
  else gemm_skinny<T, 16><<<grid, kSkinnyThreads, 0, st>>>(a, b, bs, c, g);
  return check_launch();
}

template <typename T>
static int launch_simt(const void* A, const void* B, const void* bias, void* C, int64_t batch, const GemmArgs& g, cudaStream_t st) {
  if (skinny_warp_eligible<T>(A, batch, g)) return launch_skinny_warp<T>(A, B, bias, C, batch, g, st);
  if (skinny_eligible<T>(A, batch, g)) return launch_skinny<T>(A, B, bias, C, batch, g, st);
  // big tiles only when they are mostly full and there are enough of them to fill the GPU
  const int64_t big_tiles = batch * ((g.M + 127) / 128) * ((g.N + 127) / 128);
  if (g.M >= 96 && g.N >= 96 && big_tiles >= kNumSMs) return launch_simt_tile<T, 128, 128>(A, B, bias, C, batch, g, st);
  if (g.N <= 40 && g.M >= 96) return launch_simt_small<T, 128, 32>(A, B, bias, C, batch, g, st);
  if (g.M <= 40 && g.N >= 96) return launch_simt_small<T, 32, 128>(A, B, bias, C, batch, g, st);
  return launch_simt_small<T, 64, 64>(A, B, bias, C, batch, g, st);
}

int gemm_simt_dispatch(const void* A, const void* B, const void* bias, void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk,
                       int64_t sBb, int64_t sBk, int64_t sBn, int64_t sbm, int64_t sbn, double alpha, double beta, int dtype, cudaStream_t st, const uint32_t* gate) {
  GemmArgs g{M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, sbm, sbn, static_cast<float>(alpha), static_cast<float>(beta), gate, 1, 0};
  switch (dtype) {
    case B200_F32: return launch_simt<float>(A, B, bias, C, batch, g, st);
    case B200_BF16: return launch_simt<__nv_bfloat16>(A, B, bias, C, batch, g, st);
    case B200_F16: return launch_simt<__half>(A, B, bias, C, batch, g, st);
    default: return B200_EDTYPE;
  }
}

}  // namespace b200
