// scatter_add with the aten CPU kernel's summation order (bit-identical fp results).
//
// For every destination element the contributions src[p] are added one after another in
// ascending p[dim], starting from self, in fp32 (bf16/f16 tensors accumulate in fp32 and
// round once at the end) -- exactly what the sequential CPU loop does. Atomics cannot
// reproduce that order, so ordering is made structural. self is viewed as
// [outer, rows, cols] with `rows` the scatter dimension:
//
//   strip kernel (cols > 1): a CTA owns a strip of 4 output columns and keeps it as fp32
//     in shared memory (column-major, so random destination rows spread over the banks;
//     64 KB at 4096 rows, so two CTAs share an SM). Source rows stream through a cp.async
//     ring of 128-row tiles (index and value segments of the 4 columns). Two warps share
//     one column, split by the parity of the destination row, and each walks a tile 32
//     source rows at a time, lane = source row. Whether two lanes of a step hit the same
//     destination is screened with a tiny per-warp tag table (each lane drops its id at a
//     slot hashed from the destination and reads it back); only on a clash is the rank of
//     every lane among EARLIER rows with the same destination computed with warp shuffles
//     and the additions applied rank by rank -- source-row order is kept without
//     __match_any_sync, whose throughput is ~250-500 cycles per call per SM.
//   row kernel (cols == 1, i.e. the scatter dimension is the last one): a warp owns two
//     rows of `outer`, their destination rows sit in shared memory, and the 16 lanes of a
//     row read 16 consecutive source positions (coalesced) with the same rank-by-shuffle
//     ordering.
//   Destinations that do not fit in shared memory are processed in windows (each window
//     re-scans the sources); HBM traffic is the algorithmic minimum otherwise: self, index
//     and src read once, out written once.
//   line kernel (any strides / ragged shapes): one thread per "line" applies its
//     contributions sequentially in global memory on an fp32 accumulator.
#include <cuda_pipeline.h>

#include <type_traits>

#include "b200_common.cuh"

namespace b200 {

constexpr int kStripCols = 4;
constexpr int kTileRows = 128;
constexpr int kStripThreads = 256;  // 8 warps: (column, destination parity)
constexpr int kSmemBudget = 220 * 1024;
constexpr int kStripSmemTarget = 110 * 1024;  // two strip CTAs per SM when the destination fits

// A CTA touches only a 16- or 32-byte segment of every row it reads (its 4 columns); the
// CTAs of the neighbouring strips read the neighbouring segments at about the same time.
// Asking L2 to fetch 256 bytes around each request turns those per-CTA slivers into full
// DRAM bursts: one CTA misses, its seven neighbours hit in L2.
__device__ __forceinline__ void cp_async8_wide(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global.L2::256B [%0], [%1], 8;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async4_wide(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global.L2::256B [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(gsrc) : "memory");
}
__device__ __forceinline__ uint4 ld_wide(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.L2::256B.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ld_wide(const uint2* p) {
  uint2 v;
  asm volatile("ld.global.L2::256B.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

__device__ __forceinline__ void flag_oob(uint32_t* status) {
  if (status) atomicOr(status, B200_DEV_INDEX_OOB);
}

// Rank of this lane among the EARLIER in-order elements of its own group of GROUP adjacent
// lanes that carry the same destination `k` (negative k = nothing to apply; made unique per
// lane so it never matches). `pos` is the lane's position inside its group.
template <int GROUP>
__device__ __forceinline__ int rank_among_earlier(int k, int pos) {
  int rank = 0;
#pragma unroll
  for (int d = 1; d < GROUP; ++d) {
    const int other = __shfl_up_sync(0xffffffffu, k, d);
    rank += (pos >= d && other == k) ? 1 : 0;
  }
  return rank;
}
// Same-destination lanes add one rank after the other, so the in-order sequence is kept.
__device__ __forceinline__ void apply_in_rank_order(float* col, int k, float v, int rank) {
  const int rounds = __reduce_max_sync(0xffffffffu, k >= 0 ? rank : 0);
  for (int t = 0; t <= rounds; ++t) {
    if (k >= 0 && rank == t) col[k] += v;
    __syncwarp();
  }
}

// One in-order step of a warp: GROUP adjacent lanes hold consecutive in-order elements of
// one independent unit (`unit` tells the groups of a warp apart), `col` is that unit's fp32
// destination array in shared memory. A cheap screen makes the shuffle ranking rare: every
// lane drops its lane id into a small per-warp table at a slot hashed from (destination,
// unit) and reads it back. If all lanes read their own id, no two lanes share a slot, hence
// no two lanes share a destination, and the additions are applied in one go. A clash (a
// real duplicate or a slot collision) falls back to ranking.
constexpr int kTagSlots = 2048;
template <int GROUP>
__device__ __forceinline__ void ordered_step(float* col, unsigned char* tags, int k, float v, int unit, int pos, int lane) {
  constexpr int kUnits = 32 / GROUP;  // groups per warp share one table: fold the unit into the slot
  const int slot = (k * kUnits + unit) & (kTagSlots - 1);
  if (k >= 0) tags[slot] = static_cast<unsigned char>(lane);
  __syncwarp();
  const bool lost = k >= 0 && tags[slot] != static_cast<unsigned char>(lane);
  if (!__any_sync(0xffffffffu, lost)) {  // the vote also orders these reads before the next step's writes
    if (k >= 0) col[k] += v;
    __syncwarp();
  } else {
    apply_in_rank_order(col, k, v, rank_among_earlier<GROUP>(k, pos));
  }
}

// ------------------------------------------------------------------ strip kernel (cols > 1)
struct StripArgs {
  int64_t outer, rows, cols;         // self / out: [outer, rows, cols] contiguous
  int64_t idx_outer, idx_rows, idx_cols;
  int64_t idx_so, idx_sr, src_so, src_sr;  // element strides of index / src (inner stride 1)
  int win_rows;                      // destination rows held in shared memory per pass
  int stages;                        // cp.async ring depth
};

template <typename T>
__global__ void __launch_bounds__(kStripThreads, 2)
scatter_add_strip(const T* __restrict__ self, const int64_t* __restrict__ index, const T* __restrict__ src, T* __restrict__ out, StripArgs A, uint32_t* status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int kIdxTile = kTileRows * kStripCols * 8, kSrcTile = kTileRows * kStripCols * static_cast<int>(sizeof(T));
  unsigned char* ring = smem_raw;                                                                             // stages x (idx tile, src tile)
  unsigned char* tags = smem_raw + static_cast<size_t>(A.stages) * (kIdxTile + kSrcTile) + (threadIdx.x >> 5) * kTagSlots;  // one screening table per warp
  float* strip = reinterpret_cast<float*>(smem_raw + static_cast<size_t>(A.stages) * (kIdxTile + kSrcTile) + (kStripThreads / 32) * kTagSlots);  // [8][win_rows]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int mycol = warp >> 1, myparity = warp & 1;
  using RowSeg = typename std::conditional<sizeof(T) == 4, uint4, uint2>::type;  // the 4 strip columns of one row
  const int64_t nstrips = A.cols / kStripCols;
  const int64_t ntiles = (A.idx_rows + kTileRows - 1) / kTileRows;

  for (int64_t item = blockIdx.x; item < A.outer * nstrips; item += gridDim.x) {
    const int64_t o = item / nstrips, j0 = (item - o * nstrips) * kStripCols;
    const T* self_o = self + o * A.rows * A.cols;
    T* out_o = out + o * A.rows * A.cols;
    const bool active = j0 < A.idx_cols && o < A.idx_outer && A.idx_rows > 0;
    for (int64_t r0 = 0; r0 < A.rows; r0 += A.win_rows) {
      const int wrows = static_cast<int>(A.rows - r0 < A.win_rows ? A.rows - r0 : A.win_rows);
      // ---- stage self[r0 : r0 + wrows, j0 : j0 + 4] column-major as fp32 (8 loads in flight per thread)
      for (int q0 = 0; q0 < wrows; q0 += kStripThreads * 8) {
        RowSeg seg[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int r = q0 + u * kStripThreads + tid;
          if (r < wrows) seg[u] = ld_wide(reinterpret_cast<const RowSeg*>(self_o + (r0 + r) * A.cols + j0));
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int r = q0 + u * kStripThreads + tid;
          if (r < wrows) {
            const T* e = reinterpret_cast<const T*>(&seg[u]);
#pragma unroll
            for (int c = 0; c < kStripCols; ++c) strip[c * A.win_rows + r] = to_f32(e[c]);
          }
        }
      }
      if (active) {
        // Tiles are staged TRANSPOSED ([column][row]) with 8-byte (index) and 4-byte (value)
        // cp.async granules: four adjacent threads still read one contiguous 32-byte index
        // segment of a source row, and a warp later reads its column with unit stride (no
        // bank conflicts). 16-bit values travel as column pairs.
        constexpr int kValCols = sizeof(T) == 4 ? kStripCols : kStripCols / 2;  // 4-byte granules per row
        const int64_t* idx_g = index + o * A.idx_so + j0;
        const uint32_t* src_g = reinterpret_cast<const uint32_t*>(src + o * A.src_so + j0);
        const int64_t src_sr32 = A.src_sr * static_cast<int64_t>(sizeof(T)) / 4;  // source row pitch in 4-byte units
        auto issue_tile = [&](int tile, int slot) {
          if (tile < ntiles) {
            int64_t* idx_s = reinterpret_cast<int64_t*>(ring + static_cast<size_t>(slot) * (kIdxTile + kSrcTile));
            uint32_t* src_s = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(idx_s) + kIdxTile);
            const int64_t i0 = static_cast<int64_t>(tile) * kTileRows;
            const int c = tid & 3, rbase = tid >> 2;  // 256 threads = 64 rows x 4 columns per sweep
#pragma unroll
            for (int u = 0; u < kTileRows / 64; ++u) {
              const int r = rbase + u * 64;
              if (i0 + r < A.idx_rows) {
                cp_async8_wide(idx_s + c * kTileRows + r, idx_g + (i0 + r) * A.idx_sr + c);
                if (c < kValCols) cp_async4_wide(src_s + c * kTileRows + r, src_g + (i0 + r) * src_sr32 + c);
              }
            }
          }
          __pipeline_commit();  // one group per tile slot, empty past the end, so the wait depth stays constant
        };
        const int nt = static_cast<int>(ntiles);
        for (int sidx = 0; sidx < A.stages - 1; ++sidx) issue_tile(sidx, sidx);
        float* col = strip + static_cast<int64_t>(mycol) * A.win_rows;
        int slot = 0, fill_slot = A.stages - 1;
        for (int tile = 0; tile < nt; ++tile) {
          __pipeline_wait_prior(A.stages - 2);  // this thread's copies of tile `tile` have landed
          __syncthreads();                      // ... everyone's have; all warps are also done with tile - 1
          issue_tile(tile + A.stages - 1, fill_slot);  // refills the slot that tile - 1 used
          const int64_t* idx_s = reinterpret_cast<const int64_t*>(ring + static_cast<size_t>(slot) * (kIdxTile + kSrcTile));
          const T* src_s = reinterpret_cast<const T*>(reinterpret_cast<const unsigned char*>(idx_s) + kIdxTile);
          const int64_t i0 = static_cast<int64_t>(tile) * kTileRows;
          constexpr int kSteps = kTileRows / 32;
          int k[kSteps];
          float v[kSteps];
#pragma unroll
          for (int st = 0; st < kSteps; ++st) {
            const int r = st * 32 + lane;
            k[st] = -1 - lane;
            v[st] = 0.f;
            if (i0 + r < A.idx_rows) {
              const int64_t key = idx_s[mycol * kTileRows + r];
              if (key < 0 || key >= A.rows) flag_oob(status);
              else if (key >= r0 && key < r0 + wrows && (static_cast<int>(key) & 1) == myparity) {
                k[st] = static_cast<int>(key - r0);
                // fp32: [column][row]; 16-bit: [column pair][row][2]
                v[st] = sizeof(T) == 4 ? to_f32(src_s[mycol * kTileRows + r]) : to_f32(src_s[((mycol >> 1) * kTileRows + r) * 2 + (mycol & 1)]);
              }
            }
          }
#pragma unroll
          for (int st = 0; st < kSteps; ++st) ordered_step<32>(col, tags, k[st], v[st], 0, lane, lane);
          if (++slot == A.stages) slot = 0;
          if (++fill_slot == A.stages) fill_slot = 0;
        }
        __pipeline_wait_prior(0);
      }
      __syncthreads();
      // ---- write the window back, rounding once
      for (int r = tid; r < wrows; r += kStripThreads) {
        RowSeg seg;
        T* e = reinterpret_cast<T*>(&seg);
#pragma unroll
        for (int c = 0; c < kStripCols; ++c) e[c] = from_f32<T>(strip[c * A.win_rows + r]);
        __stcs(reinterpret_cast<RowSeg*>(out_o + (r0 + r) * A.cols + j0), seg);
      }
      __syncthreads();  // the strip is rewritten by the next window / item
    }
  }
}

// ------------------------------------------------------------------ row kernel (scatter along the last dim)
struct RowArgs {
  int64_t outer, rows;               // self / out: [outer, rows] contiguous, scatter along `rows`
  int64_t idx_outer, idx_len;        // index / src: [idx_outer, idx_len], inner stride 1
  int64_t idx_so, src_so;
  int win_rows;
};

template <typename T>
__global__ void __launch_bounds__(256) scatter_add_rows(const T* __restrict__ self, const int64_t* __restrict__ index, const T* __restrict__ src, T* __restrict__ out, RowArgs A,
                                                        uint32_t* status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int half = lane >> 4, p16 = lane & 15;  // lanes 0-15: first row of the pair, 16-31: second
  unsigned char* tags = smem_raw + warp * kTagSlots;  // one screening table per warp, ahead of the destination rows
  float* mine = reinterpret_cast<float*>(smem_raw + nwarps * kTagSlots) + (static_cast<int64_t>(warp) * 2 + half) * A.win_rows;
  const int64_t npairs = (A.outer + 1) / 2;
  for (int64_t pair = static_cast<int64_t>(blockIdx.x) * nwarps + warp; pair < npairs; pair += static_cast<int64_t>(gridDim.x) * nwarps) {
    const int64_t o = pair * 2 + half;
    const bool row_ok = o < A.outer;
    const bool active = row_ok && o < A.idx_outer;
    for (int64_t r0 = 0; r0 < A.rows; r0 += A.win_rows) {
      const int wrows = static_cast<int>(A.rows - r0 < A.win_rows ? A.rows - r0 : A.win_rows);
      if (row_ok)
        for (int r = p16; r < wrows; r += 16) mine[r] = to_f32(self[o * A.rows + r0 + r]);
      __syncwarp();
      for (int64_t j0 = 0; j0 < A.idx_len; j0 += 64) {  // warp-uniform trip count
        int k[4];
        float v[4];
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          const int64_t j = j0 + s * 16 + p16;
          k[s] = -1 - lane;
          v[s] = 0.f;
          if (active && j < A.idx_len) {
            const int64_t key = index[o * A.idx_so + j];
            if (key < 0 || key >= A.rows) flag_oob(status);
            else if (key >= r0 && key < r0 + wrows) {
              k[s] = static_cast<int>(key - r0);
              v[s] = to_f32(src[o * A.src_so + j]);
            }
          }
        }
#pragma unroll
        for (int s = 0; s < 4; ++s) ordered_step<16>(mine, tags, k[s], v[s], half, p16, lane);
      }
      if (row_ok)
        for (int r = p16; r < wrows; r += 16) out[o * A.rows + r0 + r] = from_f32<T>(mine[r]);
      __syncwarp();
    }
  }
}

// ------------------------------------------------------------------ generic line kernel
struct ScatterArgs {
  int ndim, dim;
  int64_t nlines, dim_len, self_dim_size;
  int64_t shape[B200_MAX_DIMS];  // index shape with shape[dim] forced to 1
  int64_t out_stride[B200_MAX_DIMS], idx_stride[B200_MAX_DIMS], src_stride[B200_MAX_DIMS];
};

template <typename T>
__global__ void __launch_bounds__(128) scatter_add_lines(float* __restrict__ out, const int64_t* __restrict__ index, const T* __restrict__ src, ScatterArgs A, uint32_t* status) {
  const int64_t line = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (line >= A.nlines) return;
  int64_t lin = line, oo = 0, io = 0, so = 0;
  for (int d = A.ndim - 1; d >= 0; --d) {
    const int64_t q = lin / A.shape[d], r = lin - q * A.shape[d];
    oo += r * A.out_stride[d];
    io += r * A.idx_stride[d];
    so += r * A.src_stride[d];
    lin = q;
  }
  const int64_t os = A.out_stride[A.dim], is = A.idx_stride[A.dim], ss = A.src_stride[A.dim];
  for (int64_t k = 0; k < A.dim_len; ++k) {
    const int64_t key = index[io + k * is];
    if (key < 0 || key >= A.self_dim_size) {
      flag_oob(status);
      continue;
    }
    out[oo + key * os] += to_f32(src[so + k * ss]);
  }
}

template <typename T>
static int launch_strip(const void* self, const void* index, const void* src, void* out, StripArgs A, uint32_t* status, cudaStream_t st) {
  const int tile_bytes = kTileRows * kStripCols * (8 + static_cast<int>(sizeof(T)));
  const int tag_bytes = (kStripThreads / 32) * kTagSlots;
  // keep at least 4 stages of source tiles; the rest of the budget holds destination rows
  int64_t win = (kSmemBudget - tag_bytes - 4 * tile_bytes) / (kStripCols * 4);
  if (win > A.rows) win = A.rows;
  A.win_rows = static_cast<int>(win);
  // a destination that fits in half an SM's shared memory leaves room for a second CTA
  const int64_t budget = tag_bytes + win * kStripCols * 4 + 3 * tile_bytes <= kStripSmemTarget ? kStripSmemTarget : kSmemBudget;
  int stages = static_cast<int>((budget - tag_bytes - win * kStripCols * 4) / tile_bytes);
  if (stages > 8) stages = 8;  // the wait depth cp.async can express
  if (stages < 2) stages = 2;
  A.stages = stages;
  const size_t smem = static_cast<size_t>(stages) * tile_bytes + tag_bytes + static_cast<size_t>(win) * kStripCols * 4;
  const cudaError_t ae = cudaFuncSetAttribute(scatter_add_strip<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
  if (ae != cudaSuccess) { set_last_cuda_error(ae); return B200_ELAUNCH; }
  const int64_t items = A.outer * (A.cols / kStripCols);
  const int grid = static_cast<int>(items < 8LL * kNumSMs ? items : 8LL * kNumSMs);
  scatter_add_strip<T><<<grid, kStripThreads, smem, st>>>(static_cast<const T*>(self), static_cast<const int64_t*>(index), static_cast<const T*>(src), static_cast<T*>(out), A, status);
  return check_launch();
}

template <typename T>
static int launch_rows(const void* self, const void* index, const void* src, void* out, RowArgs A, uint32_t* status, cudaStream_t st) {
  // two destination rows per warp; shrink the CTA before windowing the destination
  int warps = 8;
  while (warps > 1 && static_cast<int64_t>(warps) * (2 * A.rows * 4 + kTagSlots) > 96 * 1024) warps >>= 1;
  int64_t win = A.rows;
  const int64_t dest_budget = kSmemBudget - static_cast<int64_t>(warps) * kTagSlots;
  if (static_cast<int64_t>(warps) * 2 * win * 4 > dest_budget) win = dest_budget / (warps * 2 * 4);
  A.win_rows = static_cast<int>(win);
  const size_t smem = static_cast<size_t>(warps) * (2 * win * 4 + kTagSlots);
  const cudaError_t ae = cudaFuncSetAttribute(scatter_add_rows<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
  if (ae != cudaSuccess) { set_last_cuda_error(ae); return B200_ELAUNCH; }
  const int64_t pairs = (A.outer + 1) / 2;
  int64_t blocks = (pairs + warps - 1) / warps;
  if (blocks > 16LL * kNumSMs) blocks = 16LL * kNumSMs;
  scatter_add_rows<T><<<static_cast<int>(blocks), warps * 32, smem, st>>>(static_cast<const T*>(self), static_cast<const int64_t*>(index), static_cast<const T*>(src), static_cast<T*>(out), A, status);
  return check_launch();
}

}  // namespace b200

using namespace b200;

extern "C" int b200_scatter_add(const void* self, const void* index, const void* src, void* out, int ndim, const int64_t* self_shape, const int64_t* index_shape,
                                const int64_t* index_strides, const int64_t* src_strides, int dim, int dtype, void* scratch, int64_t scratch_bytes, uint32_t* status, void* stream) {
  if (ndim < 1 || ndim > B200_MAX_DIMS || dim < 0 || dim >= ndim || !self_shape || !index_shape || !index_strides || !src_strides) return B200_EINVAL;
  if (!is_float_dtype(dtype)) return B200_EDTYPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t n_self = numel_of(ndim, self_shape);
  const int64_t n_idx = numel_of(ndim, index_shape);
  for (int d = 0; d < ndim; ++d)
    if (self_shape[d] < 0 || index_shape[d] < 0 || (d != dim && index_shape[d] > self_shape[d])) return B200_EINVAL;
  if (n_self == 0) return B200_OK;
  if (!self || !out) return B200_EINVAL;
  const int es = dtype_size(dtype);

  // ---- [outer, rows, cols] view; index / src must be plain row-major views of it
  if (n_idx > 0 && index && src && aligned16(self) && aligned16(out) && aligned16(index) && aligned16(src)) {
    int64_t outer = 1, cols = 1, idx_outer = 1, idx_cols = 1;
    for (int d = 0; d < dim; ++d) { outer *= self_shape[d]; idx_outer *= index_shape[d]; }
    for (int d = dim + 1; d < ndim; ++d) { cols *= self_shape[d]; idx_cols *= index_shape[d]; }
    const int64_t rows = self_shape[dim], idx_rows = index_shape[dim];
    // collapsible only when at most one leading and one trailing dim are non-trivial
    int lead = 0, trail = 0, dl = -1, dt = -1;
    for (int d = 0; d < dim; ++d)
      if (self_shape[d] > 1 || index_shape[d] > 1) { ++lead; dl = d; }
    for (int d = dim + 1; d < ndim; ++d)
      if (self_shape[d] > 1 || index_shape[d] > 1) { ++trail; dt = d; }
    if (lead <= 1 && trail <= 1 && rows < 0x7fffffffLL) {
      const int64_t idx_so = dl >= 0 ? index_strides[dl] : 0, src_so = dl >= 0 ? src_strides[dl] : 0;
      if (dt >= 0) {
        const bool inner_ok = index_strides[dt] == 1 && src_strides[dt] == 1;
        const bool shape_ok = cols % kStripCols == 0 && idx_cols % kStripCols == 0;
        const bool stride_ok = (src_strides[dim] * es) % 4 == 0 && (src_so * es) % 4 == 0;  // 4-byte value granules
        if (inner_ok && shape_ok && stride_ok) {
          StripArgs A{outer, rows, cols, idx_outer, idx_rows, idx_cols, idx_so, index_strides[dim], src_so, src_strides[dim], 0, 0};
          switch (dtype) {
            case B200_F32: return launch_strip<float>(self, index, src, out, A, status, st);
            case B200_BF16: return launch_strip<__nv_bfloat16>(self, index, src, out, A, status, st);
            default: return launch_strip<__half>(self, index, src, out, A, status, st);
          }
        }
      } else if (index_strides[dim] == 1 && src_strides[dim] == 1) {
        RowArgs A{outer, rows, idx_outer, idx_rows, idx_so, src_so, 0};
        switch (dtype) {
          case B200_F32: return launch_rows<float>(self, index, src, out, A, status, st);
          case B200_BF16: return launch_rows<__nv_bfloat16>(self, index, src, out, A, status, st);
          default: return launch_rows<__half>(self, index, src, out, A, status, st);
        }
      }
    }
  }

  // ---- generic: acc = fp32(self), ordered lines on acc, out = round(acc)
  const bool wide = dtype == B200_F32;
  float* acc = wide ? static_cast<float*>(out) : static_cast<float*>(scratch);
  if (!wide && (!scratch || scratch_bytes < n_self * 4)) return B200_ESCRATCH;
  if (wide) {
    if (out != self) {
      const cudaError_t ce = cudaMemcpyAsync(out, self, static_cast<size_t>(n_self) * es, cudaMemcpyDeviceToDevice, st);
      if (ce != cudaSuccess) { set_last_cuda_error(ce); return B200_ELAUNCH; }
    }
  } else {
    const int64_t one = 1;
    if (int rc = b200_copy_strided(self, acc, 1, &n_self, &one, dtype, B200_F32, stream)) return rc;
  }
  if (n_idx > 0) {
    if (!index || !src) return B200_EINVAL;
    ScatterArgs A;
    A.ndim = ndim;
    A.dim = dim;
    A.dim_len = index_shape[dim];
    A.self_dim_size = self_shape[dim];
    A.nlines = 1;
    int64_t st_out = 1;
    for (int d = ndim - 1; d >= 0; --d) {
      A.shape[d] = d == dim ? 1 : index_shape[d];
      A.nlines *= A.shape[d];
      A.out_stride[d] = st_out;
      st_out *= self_shape[d];
      A.idx_stride[d] = index_strides[d];
      A.src_stride[d] = src_strides[d];
    }
    const int g = grid_for(A.nlines, 128);
    const int64_t* pi = static_cast<const int64_t*>(index);
    switch (dtype) {
      case B200_F32: scatter_add_lines<float><<<g, 128, 0, st>>>(acc, pi, static_cast<const float*>(src), A, status); break;
      case B200_BF16: scatter_add_lines<__nv_bfloat16><<<g, 128, 0, st>>>(acc, pi, static_cast<const __nv_bfloat16*>(src), A, status); break;
      default: scatter_add_lines<__half><<<g, 128, 0, st>>>(acc, pi, static_cast<const __half*>(src), A, status); break;
    }
    if (int rc = check_launch()) return rc;
  }
  if (!wide) {
    const int64_t one = 1;
    return b200_copy_strided(acc, out, 1, &n_self, &one, B200_F32, dtype, stream);
  }
  return B200_OK;
}
