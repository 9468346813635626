// embedding / index_select / gather: bit-exact data movement driven by integer indices.
//
// Rows (embedding, index_select dim 0) are copied with 16-byte accesses, one CTA per
// output row when rows are wide (>= 1 KB) and a flattened (row, vector) space when they
// are narrow, so loads within a row and all stores are coalesced. gather moves single
// elements: index reads and output writes are coalesced, source reads hit one 32-byte
// sector each and are served by L2 when the source fits there.
// An index outside [0, size) never faults: the element/row is written as zero and
// B200_DEV_INDEX_OOB is OR-ed into the caller's status word. Negative indices are out of
// range here, as they are for the aten CPU kernels.
#include <cstdlib>

#include "b200_common.cuh"
#include "tma_common.cuh"

namespace b200 {

__device__ __forceinline__ int64_t load_index(const void* idx, int64_t i, int idx_i32) {
  return idx_i32 ? static_cast<int64_t>(static_cast<const int32_t*>(idx)[i]) : static_cast<const int64_t*>(idx)[i];
}
__device__ __forceinline__ void flag_oob(uint32_t* status) {
  if (status) atomicOr(status, B200_DEV_INDEX_OOB);
}
// The gathered-from tensor is re-read at random while index and output stream through once:
// pin the former in L2 (evict_last) so the streams do not push it out.
__device__ __forceinline__ uint64_t l2_keep_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint32_t ld_keep_l2(const uint32_t* p, uint64_t pol) {
  uint32_t v;
  asm volatile("ld.global.nc.L2::cache_hint.u32 %0, [%1], %2;" : "=r"(v) : "l"(p), "l"(pol));
  return v;
}
__device__ __forceinline__ uint16_t ld_keep_l2(const uint16_t* p, uint64_t pol) {
  uint16_t v;
  asm volatile("ld.global.nc.L2::cache_hint.u16 %0, [%1], %2;" : "=h"(v) : "l"(p), "l"(pol));
  return v;
}
template <typename U> __device__ __forceinline__ U zero_of() { U z; memset(&z, 0, sizeof(U)); return z; }

// One CTA (128 threads) per output row; rows are `nvec` 16-byte vectors.
__global__ void __launch_bounds__(128) gather_rows_wide(const uint4* __restrict__ table, const void* __restrict__ idx, uint4* __restrict__ out,
                                                        int64_t table_rows, int64_t nvec, int64_t n_idx, int idx_i32, uint32_t* status) {
  for (int64_t r = blockIdx.x; r < n_idx; r += gridDim.x) {
    const int64_t src = load_index(idx, r, idx_i32);
    const bool ok = src >= 0 && src < table_rows;
    if (!ok && threadIdx.x == 0) flag_oob(status);
    const uint4* s = table + (ok ? src : 0) * nvec;
    uint4* d = out + r * nvec;
    int64_t j = threadIdx.x;
    for (; j + 3 * 128 < nvec; j += 4 * 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = ok ? __ldcs(s + j + u * 128) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < 4; ++u) __stcs(d + j + u * 128, v[u]);
    }
    for (; j < nvec; j += 128) __stcs(d + j, ok ? __ldcs(s + j) : make_uint4(0, 0, 0, 0));
  }
}

// Flattened index_select: x is [outer, dim_size, inner] in units of U, out is
// [outer, n_idx, inner]; one unit per thread iteration.
template <typename U>
__global__ void __launch_bounds__(256) index_select_flat(const U* __restrict__ x, const void* __restrict__ idx, U* __restrict__ out, int64_t outer, int64_t dim_size,
                                                         int64_t inner, int64_t n_idx, int idx_i32, uint32_t* status) {
  const int64_t total = outer * n_idx * inner;
  for (int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p < total; p += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t q = p / inner, i = p - q * inner;
    const int64_t o = q / n_idx, k = q - o * n_idx;
    const int64_t src = load_index(idx, k, idx_i32);
    if (src < 0 || src >= dim_size) {
      flag_oob(status);
      out[p] = zero_of<U>();
    } else {
      out[p] = x[(o * dim_size + src) * inner + i];
    }
  }
}

struct GatherArgs {
  int ndim, dim;
  int64_t n;
  int64_t shape[B200_MAX_DIMS], self_stride[B200_MAX_DIMS], idx_stride[B200_MAX_DIMS];
  int64_t self_dim_size;
};

template <typename U>
__global__ void __launch_bounds__(256) gather_generic(const U* __restrict__ self, const int64_t* __restrict__ index, U* __restrict__ out, GatherArgs A, uint32_t* status) {
  for (int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p < A.n; p += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t io = 0, so = 0;
    if (A.n <= 0x7fffffffLL) {  // coordinates by 32-bit division (a 64-bit one costs ~5x the instructions)
      uint32_t lin = static_cast<uint32_t>(p);
      for (int d = A.ndim - 1; d >= 0; --d) {
        const uint32_t ext = static_cast<uint32_t>(A.shape[d]);
        const uint32_t q = lin / ext, r = lin - q * ext;
        io += r * A.idx_stride[d];
        if (d != A.dim) so += r * A.self_stride[d];
        lin = q;
      }
    } else {
      int64_t lin = p;
      for (int d = A.ndim - 1; d >= 0; --d) {
        const int64_t q = lin / A.shape[d], r = lin - q * A.shape[d];
        io += r * A.idx_stride[d];
        if (d != A.dim) so += r * A.self_stride[d];
        lin = q;
      }
    }
    const int64_t k = index[io];
    if (k < 0 || k >= A.self_dim_size) {
      flag_oob(status);
      out[p] = zero_of<U>();
    } else {
      out[p] = self[so + k * A.self_stride[A.dim]];
    }
  }
}

// 2-D, dim 0, contiguous index [R, C] and unit column stride in self (row pitch
// `self_pitch`): each thread produces the 16 bytes of adjacent outputs (4 or 8 elements) --
// 16-byte index loads, one sector read per element, one 16-byte store. The columns are
// walked in blocks of `wcols` (blockIdx.y), chosen so that the slice of `self` a block of
// columns can touch (self_rows x wcols) stays L2-resident while index and output stream past
// it: every source sector then comes from DRAM once instead of once per eviction.
template <typename U>
__global__ void __launch_bounds__(256) gather_dim0_vec(const U* __restrict__ self, const int64_t* __restrict__ index, U* __restrict__ out, int64_t rows, int64_t cols,
                                                       int64_t self_pitch, int64_t self_rows, int64_t wcols, uint32_t* status) {
  constexpr int VE = 16 / static_cast<int>(sizeof(U));
  const int64_t j0 = static_cast<int64_t>(blockIdx.y) * wcols;
  const int64_t wb = cols - j0 < wcols ? cols - j0 : wcols;
  const int64_t gpr = wb / VE;  // 16-byte groups per row inside this column block
  const int64_t ngroup = rows * gpr;
  const uint64_t keep = l2_keep_policy();
  for (int64_t q = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; q < ngroup; q += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t i = q / gpr, col = j0 + (q - i * gpr) * VE;
    const int64_t p = i * cols + col;
    int64_t k[VE];
#pragma unroll
    for (int h = 0; h < VE / 2; ++h) {
      const longlong2 t = __ldcs(reinterpret_cast<const longlong2*>(index + p) + h);
      k[2 * h] = t.x;
      k[2 * h + 1] = t.y;
    }
    __align__(16) U v[VE];
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      if (k[e] < 0 || k[e] >= self_rows) {
        flag_oob(status);
        v[e] = zero_of<U>();
      } else {
        v[e] = ld_keep_l2(self + k[e] * self_pitch + col + e, keep);
      }
    }
    __stcs(reinterpret_cast<uint4*>(out + p), *reinterpret_cast<const uint4*>(v));
  }
}

// 2-D, along the LAST dim (out[i][j] = self[i][index[i][j]]), contiguous index and unit element
// stride in self: each thread produces the 16 bytes of adjacent outputs of one row -- 16-byte
// index loads, look-ups that stay inside the row (its lines are in L1 / L2 after the first
// touch), one 16-byte store, one 32-bit division per thread instead of a coordinate
// decomposition per element.
template <typename U>
__global__ void __launch_bounds__(256) gather_lastdim_vec(const U* __restrict__ self, const int64_t* __restrict__ index, U* __restrict__ out, int64_t rows, int64_t cols, int64_t self_pitch,
                                                          int64_t self_cols, uint32_t* status) {
  constexpr int VE = 16 / static_cast<int>(sizeof(U));
  const int64_t gpr = cols / VE, ngroup = rows * gpr;
  for (int64_t q = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; q < ngroup; q += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t i = ngroup <= 0x7fffffffLL ? static_cast<int64_t>(static_cast<uint32_t>(q) / static_cast<uint32_t>(gpr)) : q / gpr;
    const int64_t p = q * VE;  // = i * cols + first column of the group
    int64_t k[VE];
#pragma unroll
    for (int h = 0; h < VE / 2; ++h) {
      const longlong2 t = __ldcs(reinterpret_cast<const longlong2*>(index + p) + h);
      k[2 * h] = t.x;
      k[2 * h + 1] = t.y;
    }
    const U* row = self + i * self_pitch;
    __align__(16) U v[VE];
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      if (k[e] < 0 || k[e] >= self_cols) {
        flag_oob(status);
        v[e] = zero_of<U>();
      } else {
        v[e] = row[k[e]];
      }
    }
    __stcs(reinterpret_cast<uint4*>(out + p), *reinterpret_cast<const uint4*>(v));
  }
}

// The same gather when a strip of `self` -- all its rows, kStripW columns -- fits in shared
// memory: a CTA copies the strip in once (32-byte segments, each source sector read once)
// and then streams index rows past it, looking every element up in shared memory. Index
// and output move as 64- and 32-byte row segments; neighbouring CTAs work on neighbouring
// strips, so the segments of one row meet again in L2 / DRAM pages. What the L2-resident
// walk above pays per element -- a 32-byte sector crossing the L2-to-SM fabric for 4
// useful bytes -- is paid here once per source element.
// One CTA per strip, one CTA per SM at a time, so the strips go by in waves of as many
// CTAs as there are SMs. The strips of the last, partial wave are cut into `tail_split`
// row ranges each (blockIdx.x >= whole_strips), so that the wave's work spreads over all
// SMs instead of leaving most of them idle.
constexpr int kStripW = 8;
constexpr int kStripThreads = 1024;
constexpr int64_t kStripMaxSelfBytes = 200 * 1024;
// Which strip and which rows this CTA works on (the strips of the last partial wave are cut
// into `tail_split` row ranges).
struct StripWork {
  int64_t c0, r_begin, r_end;
};
__device__ __forceinline__ StripWork strip_work(int64_t rows, int whole_strips, int tail_split) {
  int64_t s = blockIdx.x, r_begin = 0, r_end = rows;
  if (static_cast<int>(blockIdx.x) >= whole_strips) {
    const int q = (blockIdx.x - whole_strips) / tail_split, piece = (blockIdx.x - whole_strips) % tail_split;
    const int64_t per = (rows + tail_split - 1) / tail_split;
    s = whole_strips + q;
    r_begin = piece * per;
    r_end = r_begin + per < rows ? r_begin + per : rows;
  }
  return StripWork{s * kStripW, r_begin, r_end};
}

// Four index segments in flight per thread and no more: keeping the next trip's segments
// in flight as well (with 1024, 768 or 512 threads) was measured 12-19 % SLOWER (62 -> 70-74
// us at 4096 x 4096) -- the 64-byte segments of different rows lie in different DRAM pages,
// and more of them outstanding at once cost more in page misses than the latency they hid.
// Holding neighbouring strips in lockstep (clusters of 2 / 4 / 8 CTAs, a cluster barrier per
// trip) did not help either: 68 -> 76 / 84 / 90 us on the same box.
constexpr int kStripU = 4;
constexpr int64_t kStripTrip = static_cast<int64_t>(kStripThreads / 32) * (8 * kStripU);  // rows one trip of the CTA covers

__device__ __forceinline__ void strip_fetch(const int64_t* __restrict__ index, int64_t cols, const StripWork& w, int64_t r0, int rsub, int cp, longlong2 (&k)[kStripU]) {
#pragma unroll
  for (int u = 0; u < kStripU; ++u) {
    const int64_t row = r0 + u * 8 + rsub;
    if (row < w.r_end) k[u] = __ldcs(reinterpret_cast<const longlong2*>(index + row * cols + w.c0 + cp));
  }
}
__device__ __forceinline__ void strip_emit(const uint32_t* strip, uint32_t* __restrict__ out, int64_t cols, const StripWork& w, int64_t r0, int rsub, int cp, int self_rows,
                                           const longlong2 (&k)[kStripU], uint32_t* status) {
#pragma unroll
  for (int u = 0; u < kStripU; ++u) {
    const int64_t row = r0 + u * 8 + rsub;
    if (row < w.r_end) {
      uint2 v = make_uint2(0u, 0u);
      if (k[u].x < 0 || k[u].x >= self_rows) flag_oob(status);
      else v.x = strip[static_cast<int>(k[u].x) * kStripW + cp];
      if (k[u].y < 0 || k[u].y >= self_rows) flag_oob(status);
      else v.y = strip[static_cast<int>(k[u].y) * kStripW + cp + 1];
      __stcs(reinterpret_cast<uint2*>(out + row * cols + w.c0 + cp), v);
    }
  }
}

__global__ void __launch_bounds__(kStripThreads, 1) gather_dim0_strip(const uint32_t* __restrict__ self, const int64_t* __restrict__ index, uint32_t* __restrict__ out,
                                                                      int64_t rows, int64_t cols, int64_t self_pitch, int self_rows, int whole_strips, int tail_split, uint32_t* status) {
  extern __shared__ __align__(128) uint32_t strip[];  // [self_rows][kStripW]
  const StripWork w = strip_work(rows, whole_strips, tail_split);
  for (int h = threadIdx.x; h < self_rows * 2; h += kStripThreads)  // half-rows: 16 bytes each
    reinterpret_cast<uint4*>(strip)[h] = ld_keep(self + static_cast<int64_t>(h >> 1) * self_pitch + w.c0 + (h & 1) * 4);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rsub = lane >> 2, cp = (lane & 3) * 2;  // a warp covers 8 rows x 8 columns per load
  for (int64_t r0 = w.r_begin + warp * (8 * kStripU); r0 < w.r_end; r0 += kStripTrip) {
    longlong2 k[kStripU];
    strip_fetch(index, cols, w, r0, rsub, cp, k);
    strip_emit(strip, out, cols, w, r0, rsub, cp, self_rows, k, status);
  }
}

// The same kernel with the strip brought in by the copy engine: one thread issues a tiled TMA
// load per 256 source rows (box 8 columns x 256 rows = 8 KB, rows beyond the source read as
// zero), all of them completing on one mbarrier, and every thread requests the index
// segments of its first trip BEFORE it waits for the strip -- the strip load costs the 1024
// threads no issue slots and overlaps the first index loads instead of preceding them. The
// wait is bounded: when it runs out the CTA raises B200_DEV_WAIT_TIMEOUT and leaves.
constexpr int kStripBoxRows = 256;
constexpr int kStripBoxBytes = kStripBoxRows * kStripW * 4;
__global__ void __launch_bounds__(kStripThreads, 1) gather_dim0_strip_tma(const __grid_constant__ CUtensorMap map_self, const int64_t* __restrict__ index, uint32_t* __restrict__ out, int64_t rows,
                                                                          int64_t cols, int self_rows, int whole_strips, int tail_split, uint32_t* status) {
  extern __shared__ __align__(128) uint32_t strip[];  // [boxes * 256][kStripW]
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t gave_up;
  const StripWork w = strip_work(rows, whole_strips, tail_split);
  const int boxes = (self_rows + kStripBoxRows - 1) / kStripBoxRows;
  if (threadIdx.x == 0) {
    gave_up = 0u;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_expect_tx(smem_u32(&bar), static_cast<uint32_t>(boxes) * kStripBoxBytes);
    for (int b = 0; b < boxes; ++b) tma_load_2d(smem_u32(strip) + b * kStripBoxBytes, &map_self, smem_u32(&bar), static_cast<int>(w.c0), b * kStripBoxRows);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rsub = lane >> 2, cp = (lane & 3) * 2;
  int64_t r0 = w.r_begin + warp * (8 * kStripU);
  longlong2 k[kStripU];
  if (r0 < w.r_end) strip_fetch(index, cols, w, r0, rsub, cp, k);  // in flight while the strip lands
  __syncthreads();                                                  // the barrier is initialised for everybody
  if (!mbar_wait(smem_u32(&bar), 0u, &gave_up, 2000000000ull)) {
    gave_up = 1u;
    if (status) atomicOr(status, B200_DEV_WAIT_TIMEOUT);
    for (int i = 0; i < 64; ++i) __nanosleep(1000);  // copies still under way may land before this CTA's shared memory is handed on
    return;
  }
  while (r0 < w.r_end) {
    strip_emit(strip, out, cols, w, r0, rsub, cp, self_rows, k, status);
    r0 += kStripTrip;
    if (r0 < w.r_end) strip_fetch(index, cols, w, r0, rsub, cp, k);
  }
}

static int capped_grid(int64_t items, int per_block, int waves) {
  int64_t g = (items + per_block - 1) / per_block;
  const int64_t cap = static_cast<int64_t>(kNumSMs) * waves;
  return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

// Largest power-of-two unit (<= 16 bytes) dividing `bytes` and every pointer's address.
static int common_unit(int64_t bytes, const void* a, const void* b) {
  uintptr_t m = static_cast<uintptr_t>(bytes) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b);
  int u = 16;
  while (u > 1 && (m & (u - 1))) u >>= 1;
  return u;
}

template <typename U>
static void launch_flat(const void* x, const void* idx, void* out, int64_t outer, int64_t dim_size, int64_t inner_units, int64_t n_idx, int idx_i32, uint32_t* status, cudaStream_t st) {
  const int64_t total = outer * n_idx * inner_units;
  index_select_flat<U><<<capped_grid(total, 256, 16), 256, 0, st>>>(static_cast<const U*>(x), idx, static_cast<U*>(out), outer, dim_size, inner_units, n_idx, idx_i32, status);
}

// index_select along the LAST dim (inner == 1): every output row is a permutation-with-
// repeats of one input row of at most 8 KB. A warp copies its input row to shared memory
// with coalesced loads and builds the output row from there with coalesced stores; the
// index list is narrowed to int32 once per CTA (-1 = out of range, reported and written as
// zero). Picking single elements straight from global memory, as the flat kernel does,
// fetches a 32-byte sector per element.
constexpr int kLastDimWarps = 8;
template <typename U>
__global__ void __launch_bounds__(kLastDimWarps * 32) index_select_lastdim(const U* __restrict__ x, const void* __restrict__ idx, U* __restrict__ out, int64_t outer, int dim, int n_idx, int row_pitch_bytes,
                                                                           int i32, int vec, uint32_t* status) {
  extern __shared__ __align__(16) unsigned char sm[];
  int* sidx = reinterpret_cast<int*>(sm);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned char* mine = sm + ((n_idx * 4 + 15) & ~15) + warp * row_pitch_bytes;
  for (int k = tid; k < n_idx; k += blockDim.x) {
    const int64_t v = load_index(idx, k, i32);
    const bool ok = v >= 0 && v < dim;
    if (!ok) flag_oob(status);
    sidx[k] = ok ? static_cast<int>(v) : -1;
  }
  __syncthreads();
  const U* row_s = reinterpret_cast<const U*>(mine);
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kLastDimWarps + warp; row < outer; row += static_cast<int64_t>(gridDim.x) * kLastDimWarps) {
    const U* xr = x + row * dim;
    if (vec) {
      const int nv = dim * static_cast<int>(sizeof(U)) / 16;
#pragma unroll 4
      for (int v = lane; v < nv; v += 32) reinterpret_cast<uint4*>(mine)[v] = ld_stream(reinterpret_cast<const uint4*>(xr) + v);
    } else {
      for (int c = lane; c < dim; c += 32) reinterpret_cast<U*>(mine)[c] = xr[c];
    }
    __syncwarp();
    U* orow = out + row * n_idx;
    for (int k = lane; k < n_idx; k += 32) {
      const int j = sidx[k];
      orow[k] = j >= 0 ? row_s[j] : zero_of<U>();
    }
    __syncwarp();  // the row buffer is rewritten in the next round
  }
}

template <typename U>
static void launch_lastdim(const void* x, const void* idx, void* out, int64_t outer, int64_t dim, int64_t n_idx, int i32, uint32_t* status, cudaStream_t st) {
  const int pitch = static_cast<int>((dim * sizeof(U) + 15) / 16 * 16);
  const size_t smem = ((n_idx * 4 + 15) & ~static_cast<size_t>(15)) + static_cast<size_t>(kLastDimWarps) * pitch;
  const int vec = (dim * sizeof(U)) % 16 == 0 && aligned16(x);
  cudaFuncSetAttribute(index_select_lastdim<U>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  index_select_lastdim<U><<<capped_grid(outer, kLastDimWarps, 8), kLastDimWarps * 32, smem, st>>>(static_cast<const U*>(x), idx, static_cast<U*>(out), outer, static_cast<int>(dim), static_cast<int>(n_idx), pitch,
                                                                                                 i32, vec, status);
}

static int index_select_bytes(const void* x, const void* idx, void* out, int64_t outer, int64_t dim_size, int64_t inner_bytes, int64_t n_idx, int idx_dtype, uint32_t* status, cudaStream_t st) {
  if (idx_dtype != B200_I32 && idx_dtype != B200_I64) return B200_EDTYPE;
  const int i32 = idx_dtype == B200_I32;
  const int unit = common_unit(inner_bytes, x, out);
  const int64_t units = inner_bytes / unit;
  if (outer == 1 && unit == 16 && units >= 64) {
    gather_rows_wide<<<capped_grid(n_idx, 1, 64), 128, 0, st>>>(static_cast<const uint4*>(x), idx, static_cast<uint4*>(out), dim_size, units, n_idx, i32, status);
    return check_launch();
  }
  if (units == 1 && unit <= 8 && dim_size * unit <= 8192 && dim_size >= 32 && n_idx >= 16 && n_idx <= 8192 && outer >= 256) {
    switch (unit) {
      case 8: launch_lastdim<uint64_t>(x, idx, out, outer, dim_size, n_idx, i32, status, st); break;
      case 4: launch_lastdim<uint32_t>(x, idx, out, outer, dim_size, n_idx, i32, status, st); break;
      case 2: launch_lastdim<uint16_t>(x, idx, out, outer, dim_size, n_idx, i32, status, st); break;
      default: launch_lastdim<uint8_t>(x, idx, out, outer, dim_size, n_idx, i32, status, st); break;
    }
    return check_launch();
  }
  switch (unit) {
    case 16: launch_flat<uint4>(x, idx, out, outer, dim_size, units, n_idx, i32, status, st); break;
    case 8: launch_flat<uint64_t>(x, idx, out, outer, dim_size, units, n_idx, i32, status, st); break;
    case 4: launch_flat<uint32_t>(x, idx, out, outer, dim_size, units, n_idx, i32, status, st); break;
    case 2: launch_flat<uint16_t>(x, idx, out, outer, dim_size, units, n_idx, i32, status, st); break;
    default: launch_flat<uint8_t>(x, idx, out, outer, dim_size, units, n_idx, i32, status, st); break;
  }
  return check_launch();
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gather_rows(const void* table, const void* idx, void* out, int64_t table_rows, int64_t row_bytes, int64_t n_idx, int idx_dtype, uint32_t* status, void* stream) {
  if (table_rows < 0 || row_bytes < 0 || n_idx < 0) return B200_EINVAL;
  if (n_idx == 0 || row_bytes == 0) return B200_OK;
  if (!idx || !out || (!table && table_rows > 0)) return B200_EINVAL;
  return index_select_bytes(table, idx, out, 1, table_rows, row_bytes, n_idx, idx_dtype, status, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_index_select(const void* x, const void* idx, void* out, int64_t outer, int64_t dim_size, int64_t inner, int64_t n_idx, int elem_size, int idx_dtype, uint32_t* status, void* stream) {
  if (outer < 0 || dim_size < 0 || inner < 0 || n_idx < 0 || elem_size <= 0) return B200_EINVAL;
  if (outer == 0 || inner == 0 || n_idx == 0) return B200_OK;
  if (!idx || !out || (!x && dim_size > 0)) return B200_EINVAL;
  return index_select_bytes(x, idx, out, outer, dim_size, inner * elem_size, n_idx, idx_dtype, status, static_cast<cudaStream_t>(stream));
}

// B200_GATHER_TMA=0 in the environment (read once) keeps the strip on plain loads: how the two are compared.
static bool strip_tma_enabled() {
  static const bool on = []() {
    const char* e = getenv("B200_GATHER_TMA");
    return !(e && e[0] == '0');
  }();
  return on;
}

extern "C" int b200_gather(const void* self, const void* index, void* out, int ndim, const int64_t* index_shape, const int64_t* self_strides, const int64_t* index_strides, int64_t self_dim_size, int dim, int elem_size, uint32_t* status, void* stream) {
  if (ndim < 1 || ndim > B200_MAX_DIMS || dim < 0 || dim >= ndim || !index_shape || !self_strides || !index_strides) return B200_EINVAL;
  GatherArgs A;
  A.ndim = ndim;
  A.dim = dim;
  A.n = 1;
  A.self_dim_size = self_dim_size;
  for (int d = 0; d < ndim; ++d) {
    if (index_shape[d] < 0) return B200_EINVAL;
    A.shape[d] = index_shape[d];
    A.self_stride[d] = self_strides[d];
    A.idx_stride[d] = index_strides[d];
    A.n *= index_shape[d];
  }
  if (A.n == 0) return B200_OK;
  if (!self || !index || !out) return B200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool idx_contig = is_contiguous(ndim, index_shape, index_strides);
  if (ndim == 2 && dim == 0 && elem_size == 4 && idx_contig && self_strides[1] == 1 && index_shape[1] % kStripW == 0 && self_strides[0] % 4 == 0 && aligned16(self) && aligned16(index) &&
      aligned16(out) && self_dim_size > 0 && self_dim_size * kStripW * 4 <= kStripMaxSelfBytes && index_shape[0] >= 512 && index_shape[0] * 2 >= self_dim_size && index_shape[1] / kStripW >= kNumSMs) {
    const size_t smem = static_cast<size_t>(self_dim_size) * kStripW * 4;
    {  // the attribute belongs to the current device: set it on every launch, as the other large-shared-memory kernels do
      const cudaError_t e = cudaFuncSetAttribute(gather_dim0_strip, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kStripMaxSelfBytes));
      if (e != cudaSuccess) { set_last_cuda_error(e); return B200_ELAUNCH; }
    }
    const int64_t strips = index_shape[1] / kStripW;
    const int64_t tail = strips % kNumSMs;
    int64_t tail_split = tail > 0 ? kNumSMs / tail : 1;
    if (tail_split > 8) tail_split = 8;  // every piece reloads the strip
    if (tail_split * 256 > index_shape[0]) tail_split = 1;
    const int64_t whole = tail_split > 1 ? strips - tail : strips;
    const int64_t grid = whole + (strips - whole) * tail_split;
    if (grid > 0x7fffffffLL) return B200_EINVAL;
    // the strip through the copy engine when a tensor map over `self` can be built (this GPU's own memory, no multicast)
    alignas(64) CUtensorMap map_self;
    bool tma = encode_fn() != nullptr && strip_tma_enabled();
    if (tma) {
      cuuint64_t dims[2] = {static_cast<cuuint64_t>(index_shape[1]), static_cast<cuuint64_t>(self_dim_size)};  // the columns this launch may touch x all source rows
      cuuint64_t strides[1] = {static_cast<cuuint64_t>(self_strides[0]) * 4};
      cuuint32_t box[2] = {kStripW, kStripBoxRows};
      cuuint32_t estr[2] = {1, 1};
      tma = encode_fn()(&map_self, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(self), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    if (tma) {
      const size_t smem_tma = static_cast<size_t>((self_dim_size + kStripBoxRows - 1) / kStripBoxRows) * kStripBoxBytes;
      const cudaError_t e2 = cudaFuncSetAttribute(gather_dim0_strip_tma, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kStripMaxSelfBytes));
      if (e2 != cudaSuccess) { set_last_cuda_error(e2); return B200_ELAUNCH; }
      gather_dim0_strip_tma<<<static_cast<unsigned>(grid), kStripThreads, smem_tma, st>>>(map_self, static_cast<const int64_t*>(index), static_cast<uint32_t*>(out), index_shape[0], index_shape[1],
                                                                                        static_cast<int>(self_dim_size), static_cast<int>(whole), static_cast<int>(tail_split), status);
      return check_launch();
    }
    gather_dim0_strip<<<static_cast<unsigned>(grid), kStripThreads, smem, st>>>(static_cast<const uint32_t*>(self), static_cast<const int64_t*>(index), static_cast<uint32_t*>(out), index_shape[0],
                                                                              index_shape[1], self_strides[0], static_cast<int>(self_dim_size), static_cast<int>(whole), static_cast<int>(tail_split), status);
    return check_launch();
  }
  const int ve = elem_size == 4 ? 4 : 8;  // outputs per 16 bytes
  if (ndim == 2 && dim == 0 && (elem_size == 4 || elem_size == 2) && idx_contig && self_strides[1] == 1 && index_shape[1] % ve == 0 && aligned16(index) && aligned16(out)) {
    // column block: about 16 MB of `self` (self_rows x wcols elements), a multiple of the group width
    int64_t wcols = (16LL << 20) / (elem_size * (self_dim_size > 0 ? self_dim_size : 1));
    wcols = wcols / ve * ve;
    if (wcols < 64) wcols = 64;
    if (wcols > index_shape[1]) wcols = index_shape[1];
    const int64_t nblocks = (index_shape[1] + wcols - 1) / wcols;
    if (nblocks <= 65535) {
      dim3 grid(capped_grid(index_shape[0] * wcols / ve, 256, 32), static_cast<unsigned>(nblocks));
      if (elem_size == 4)
        gather_dim0_vec<uint32_t><<<grid, 256, 0, st>>>(static_cast<const uint32_t*>(self), static_cast<const int64_t*>(index), static_cast<uint32_t*>(out), index_shape[0], index_shape[1], self_strides[0], self_dim_size, wcols, status);
      else
        gather_dim0_vec<uint16_t><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(self), static_cast<const int64_t*>(index), static_cast<uint16_t*>(out), index_shape[0], index_shape[1], self_strides[0], self_dim_size, wcols, status);
      return check_launch();
    }
  }
  if (ndim == 2 && dim == 1 && (elem_size == 4 || elem_size == 2) && idx_contig && self_strides[1] == 1 && index_shape[1] % ve == 0 && aligned16(index) && aligned16(out)) {
    const int g2 = capped_grid(A.n / ve, 256, 32);
    if (elem_size == 4)
      gather_lastdim_vec<uint32_t><<<g2, 256, 0, st>>>(static_cast<const uint32_t*>(self), static_cast<const int64_t*>(index), static_cast<uint32_t*>(out), index_shape[0], index_shape[1], self_strides[0], self_dim_size, status);
    else
      gather_lastdim_vec<uint16_t><<<g2, 256, 0, st>>>(static_cast<const uint16_t*>(self), static_cast<const int64_t*>(index), static_cast<uint16_t*>(out), index_shape[0], index_shape[1], self_strides[0], self_dim_size, status);
    return check_launch();
  }
  const int g = capped_grid(A.n, 256, 32);
  const int64_t* pi = static_cast<const int64_t*>(index);
  switch (elem_size) {
    case 1: gather_generic<uint8_t><<<g, 256, 0, st>>>(static_cast<const uint8_t*>(self), pi, static_cast<uint8_t*>(out), A, status); break;
    case 2: gather_generic<uint16_t><<<g, 256, 0, st>>>(static_cast<const uint16_t*>(self), pi, static_cast<uint16_t*>(out), A, status); break;
    case 4: gather_generic<uint32_t><<<g, 256, 0, st>>>(static_cast<const uint32_t*>(self), pi, static_cast<uint32_t*>(out), A, status); break;
    case 8: gather_generic<uint64_t><<<g, 256, 0, st>>>(static_cast<const uint64_t*>(self), pi, static_cast<uint64_t*>(out), A, status); break;
    default: return B200_EDTYPE;
  }
  return check_launch();
}
