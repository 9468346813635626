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
#include "tma_common.cuh"

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
template <int GROUP, int SLOTS = kTagSlots>
__device__ __forceinline__ void ordered_step(float* col, unsigned char* tags, int k, float v, int unit, int pos, int lane) {
  constexpr int kUnits = 32 / GROUP;  // groups per warp share one table: fold the unit into the slot
  const int slot = (k * kUnits + unit) & (SLOTS - 1);
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

// ------------------------------------------------------------------ wide strip kernel
// The strip kernel again, for destinations of at most 4096 rows, sized for the memory
// system instead of for occupancy. A CTA owns EIGHT columns (its fp32 strip is 128 KB at
// 4096 rows: one CTA per SM), so every source row contributes a 64-byte index segment and
// a 32-byte (fp32) value segment -- whole sectors.
// Source rows arrive in tiles of 128 rows through a ring filled by the copy engine: a ninth
// warp issues two tiled TMA loads per tile (index box 8 x 128 int64 with the 64-byte swizzle,
// value box 8 x 128 with the 32-byte swizzle: the 16-byte chunks of a staged row are XORed
// with the row number, so the 32 rows a warp reads of one column spread over the banks) onto
// the tile's `full` mbarrier, as soon as the eight compute warps have released the slot on its
// `empty` mbarrier. The compute warps never meet at a CTA-wide barrier inside a strip: each
// owns one column, waits for a tile, walks it 32 source rows at a time (lane = source row) and
// releases it, so a warp that met more clashes than its neighbours falls behind by a few
// tiles instead of holding all of them up, and the next strip's first tiles load while this
// strip is written back. Every wait is bounded (a wait that runs out raises
// B200_DEV_WAIT_TIMEOUT, and the CTA finishes its barriers and leaves).
// With one or two warps per scheduler the kernel runs at the speed of its dependent
// instruction chain, so the step is kept to a couple of dozen instructions: every offset
// that depends only on the lane is computed once, row-bound tests exist only for the
// ragged last tile, and the steps are software-pipelined by hand (the compiler must assume
// that the tag table and the strip alias): while step st waits for its tag read-back and
// for the strip value it read ahead, keys, values and tags of step st + 1 are under way.
constexpr int kWideCols = 8;
constexpr int kWideTileRows = 128;
constexpr int kWideComputeThreads = 256;  // eight warps: one column each
constexpr int kWideThreads = 288;         // ... and the warp that feeds the ring
constexpr int kWideTagSlots = 4096;       // one table per warp, exact up to 4096 destinations ...
constexpr int kWideDummies = 32;          // ... plus a slot (and a strip element) per lane for rows that have nothing to add
constexpr int kWideSelfRows = 256;        // rows of the destination strip per ring slot on its way in (the largest TMA box)
constexpr int kWideOutRows = 32;          // rows of the destination strip per tiled store on its way out: a warp's share of a slab
constexpr int kWideOutBlocks = 4;         // staging blocks per warp for those stores
constexpr int kWideStages = 5;            // 12 KB tiles (fp32): 48 KB of source rows in flight per SM
constexpr int kWideMaxRows = 4096;
constexpr uint64_t kWideWaitLimitNs = 2000000000ull;

__device__ __forceinline__ void compute_warps_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kWideComputeThreads) : "memory"); }

template <typename T>
__global__ void __launch_bounds__(kWideThreads, 1)
scatter_add_strip_wide(const __grid_constant__ CUtensorMap map_idx, const __grid_constant__ CUtensorMap map_src, const __grid_constant__ CUtensorMap map_self, const __grid_constant__ CUtensorMap map_out, StripArgs A, uint32_t* status) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem_raw = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));  // the swizzle patterns repeat every 512 bytes
  constexpr int kIdxTile = kWideTileRows * kWideCols * 8;                            // 8 KB: [row][4 chunks of 2 indices]
  constexpr int kSrcRow = kWideCols * static_cast<int>(sizeof(T));                   // 32 or 16 bytes of values per row
  constexpr int kSrcTile = kWideTileRows * kSrcRow;
  constexpr int kSrcChunks = kSrcRow / 16;                                           // 16-byte chunks per value row: 2 or 1
  constexpr int kTile = kIdxTile + kSrcTile;                                         // 12 KB / 10 KB: every slot starts on a 1 KB boundary
  unsigned char* ring = smem_raw;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned char* tags = smem_raw + kWideStages * kTile + (warp & 7) * (kWideTagSlots + kWideDummies);
  float* strip = reinterpret_cast<float*>(smem_raw + kWideStages * kTile + 8 * (kWideTagSlots + kWideDummies));  // [8][rows + 32]
  const int rows = static_cast<int>(A.rows);
  const int cstride = rows + kWideDummies;  // a column of the strip, then one dummy element per lane
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(strip) + static_cast<size_t>(kWideMaxRows + kWideDummies) * kWideCols * 4);  // full[S], empty[S]
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 2 * kWideStages);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kWideStages + s); };
  const int64_t nstrips = A.cols / kWideCols;
  const int ntiles = static_cast<int>((A.idx_rows + kWideTileRows - 1) / kWideTileRows);
  constexpr int kSegsPerRow = kSrcRow / 16, kPerSeg = 16 / static_cast<int>(sizeof(T));  // 16-byte segments of a destination row
  constexpr int kSelfBytes = kWideSelfRows * kSrcRow;  // a slab of the destination strip fits a ring slot
  static_assert(kSelfBytes <= kTile, "a slab of the destination strip travels in one ring slot");
  static_assert(8 * kWideOutBlocks * kWideOutRows * 32 <= 8 * (kWideTagSlots + kWideDummies), "the blocks on their way out are staged in the tag tables");
  static_assert(kWideSelfRows == kWideComputeThreads && kWideOutRows == 32, "thread t owns row t of every slab, on the way in and on the way out");
  const int nslabs = (static_cast<int>(A.rows) + kWideSelfRows - 1) / kWideSelfRows;

  if (tid == 0) {
    for (int s = 0; s < kWideStages; ++s) {
      mbar_init(full_bar(s), 1);   // the producer's expect_tx arrival; the copies complete the bytes
      mbar_init(empty_bar(s), 8);  // one arrival per compute warp
    }
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == 8) {
    // ------------------------------------------------------------ producer: the ring, tile after tile, strip after strip
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t item = blockIdx.x; item < A.outer * nstrips && ok; item += gridDim.x) {
        const int64_t o = item / nstrips, j0 = (item - o * nstrips) * kWideCols;
        for (int slab = 0; slab < nslabs && ok; ++slab) {  // self[:, j0 : j0 + 8], 256 rows per slot
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, kWideWaitLimitNs)) { ok = false; break; }
          mbar_expect_tx(full_bar(stage), kSelfBytes);
          tma_load_3d(smem_u32(ring) + stage * kTile, &map_self, full_bar(stage), static_cast<int>(j0), slab * kWideSelfRows, static_cast<int>(o));
          if (++stage == kWideStages) { stage = 0; phase ^= 1u; }
        }
        if (!(j0 < A.idx_cols && o < A.idx_outer && ntiles > 0)) continue;
        for (int tile = 0; tile < ntiles && ok; ++tile) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, kWideWaitLimitNs)) { ok = false; break; }
          const uint32_t dst = smem_u32(ring) + stage * kTile;
          mbar_expect_tx(full_bar(stage), kTile);  // a box counts in full, rows past the end of the tensor arrive as zeros
          tma_load_3d(dst, &map_idx, full_bar(stage), static_cast<int>(j0), tile * kWideTileRows, static_cast<int>(o));
          tma_load_3d(dst + kIdxTile, &map_src, full_bar(stage), static_cast<int>(j0), tile * kWideTileRows, static_cast<int>(o));
          if (++stage == kWideStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        *abort_flag = 1u;
        if (status) atomicOr(status, B200_DEV_WAIT_TIMEOUT);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ compute warps: lane reads row `lane` (+ 32 per step) of column `warp`
    const int c_idx_off = lane * 64 + (((warp >> 1) ^ ((lane >> 1) & 3)) << 4) + (warp & 1) * 8;
    const int c_src_off = kIdxTile + lane * kSrcRow + (kSrcChunks == 2 ? (((warp >> 2) ^ ((lane >> 2) & 1)) << 4) : 0) + (warp & (kPerSeg - 1)) * static_cast<int>(sizeof(T));
    float* col = strip + warp * cstride;
    const int dummy = rows + lane;  // where a lane with nothing to add "adds" zero: its own slot, so it never clashes
    const uint32_t ring_a = smem_u32(ring), tags_a = smem_u32(tags), col_a = smem_u32(col), strip_a = smem_u32(strip);
    const uint32_t out_stage_a = ring_a + kWideStages * kTile + warp * (kWideOutBlocks * kWideOutRows * 32);  // four blocks of 32 rows per warp inside the tag tables
    int out_parity = 0;
    // Rows r0 .. r0 + 31 of the finished strip (this warp's share of a slab) leave for
    // out[po, r0 .., pj0 : pj0 + 8], rounded once: back to rows of 8 values in one of the warp's
    // four staging blocks inside the tag tables (idle between tile loops), then one tiled store,
    // which clips at the last row. The warp only waits for the engine to have read the block it
    // staged four stores ago.
    auto store_rows = [&](int r0, int64_t pj0, int64_t po) {
      if (r0 >= rows) return;
      if (lane == 0) tma_store_wait_read_but<kWideOutBlocks - 1>();
      __syncwarp();
      const int r = r0 + lane < rows ? r0 + lane : rows - 1;  // rows past the end are clipped by the store
      const uint32_t block_a = out_stage_a + out_parity * (kWideOutRows * 32);
      float f[kWideCols];
#pragma unroll
      for (int c = 0; c < kWideCols; ++c) asm volatile("ld.shared.f32 %0, [%1];" : "=f"(f[c]) : "r"(strip_a + 4u * static_cast<uint32_t>(c * cstride + r)) : "memory");
#pragma unroll
      for (int h = 0; h < kSegsPerRow; ++h) {
        const uint4 seg = narrow<T>(f + h * kPerSeg);
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(block_a + lane * kSrcRow + h * 16), "r"(seg.x), "r"(seg.y), "r"(seg.z), "r"(seg.w) : "memory");
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_3d(&map_out, block_a, static_cast<int>(pj0), r0, static_cast<int>(po));
        tma_store_commit();
      }
      out_parity = (out_parity + 1) & (kWideOutBlocks - 1);
    };
    bool have_prev = false;
    int64_t prev_j0 = 0, prev_o = 0;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int64_t item = blockIdx.x; item < A.outer * nstrips; item += gridDim.x) {
      const int64_t o = item / nstrips, j0 = (item - o * nstrips) * kWideCols;
      const bool active = j0 < A.idx_cols && o < A.idx_outer && ntiles > 0;

      // ---- one pass over the strip, 256 rows at a time: the previous item's result leaves, and
      // self[:, j0 : j0 + 8] of this item, which arrives through the ring (256 rows per slot),
      // takes its place column-major as fp32. Thread t owns row t of every slab in both
      // directions, so nothing orders the two but the thread's own program; the 32 lanes of a
      // warp read and write 32 adjacent rows of one column.
      for (int slab = 0; slab < nslabs && ok; ++slab) {
        if (have_prev) store_rows(slab * kWideSelfRows + warp * 32, prev_j0, prev_o);
        int got = 0;
        if (lane == 0) got = mbar_wait(full_bar(stage), phase, abort_flag, kWideWaitLimitNs) ? 1 : 0;
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) {
          ok = false;
          if (lane == 0) {
            *abort_flag = 1u;
            if (status) atomicOr(status, B200_DEV_WAIT_TIMEOUT);
          }
          break;
        }
        const uint32_t slab_a = ring_a + stage * kTile + tid * kSrcRow;
        const int r = slab * kWideSelfRows + tid;
#pragma unroll
        for (int h = 0; h < kSegsPerRow; ++h) {
          uint4 seg;
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(seg.x), "=r"(seg.y), "=r"(seg.z), "=r"(seg.w) : "r"(slab_a + h * 16));
          float f[kPerSeg];
          widen<T>(seg, f);
          if (r < rows) {
#pragma unroll
            for (int c = 0; c < kPerSeg; ++c) asm volatile("st.shared.f32 [%0], %1;" ::"r"(strip_a + 4u * static_cast<uint32_t>((h * kPerSeg + c) * cstride + r)), "f"(f[c]) : "memory");
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(stage));
        if (++stage == kWideStages) { stage = 0; phase ^= 1u; }
      }
      if (lane == 0) tma_store_wait_read();  // the tag tables are free again
      compute_warps_barrier();               // the strip is staged

      if (active) {
        for (int tile = 0; tile < ntiles && ok; ++tile) {
          int got = 0;
          if (lane == 0) got = mbar_wait(full_bar(stage), phase, abort_flag, kWideWaitLimitNs) ? 1 : 0;
          got = __shfl_sync(0xffffffffu, got, 0);
          if (!got) {
            ok = false;
            if (lane == 0) {
              *abort_flag = 1u;
              if (status) atomicOr(status, B200_DEV_WAIT_TIMEOUT);
            }
            break;
          }
          // shared-memory accesses of the step by 32-bit shared addresses (the ring, the tag table
          // and the strip are carved out of one aligned buffer, which hides their address space
          // from the compiler: generic accesses would cost 64-bit address arithmetic per access)
          const uint32_t tile_a = ring_a + stage * kTile;
          const int valid_rows = static_cast<int>(A.idx_rows - static_cast<int64_t>(tile) * kWideTileRows);  // >= 128 except in the last tile
          const bool ragged = valid_rows < kWideTileRows;
          constexpr int kSteps = kWideTileRows / 32;
          unsigned oob = 0u;
          // Every lane always has a destination: a row past the end of the tensor, or an index
          // out of range (reported once per tile), adds zero to the lane's own dummy element.
          // The step below therefore has no per-lane conditions at all -- with two warps per
          // scheduler the kernel runs at the speed of its instruction chain, and every
          // `if (k >= 0)` cost a branch and its reconvergence bookkeeping.
          auto fetch = [&](int st, int& k, float& v) {
            uint32_t lo, hi;
            asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(tile_a + c_idx_off + st * (32 * 64)));
            float val;
            if (sizeof(T) == 4) {
              asm volatile("ld.shared.f32 %0, [%1];" : "=f"(val) : "r"(tile_a + c_src_off + st * (32 * kSrcRow)));
            } else {
              unsigned short raw;
              asm volatile("ld.shared.u16 %0, [%1];" : "=h"(raw) : "r"(tile_a + c_src_off + st * (32 * kSrcRow)));
              val = to_f32(*reinterpret_cast<const T*>(&raw));
            }
            const bool in_range = hi == 0u && lo < static_cast<uint32_t>(rows);
            const bool in_tensor = !ragged || st * 32 + lane < valid_rows;
            oob |= (in_tensor && !in_range) ? 1u : 0u;
            const bool use = in_tensor && in_range;
            k = use ? static_cast<int>(lo) : dummy;
            v = use ? val : 0.f;
          };
          auto tag_put = [&](int k) { asm volatile("st.shared.u8 [%0], %1;" ::"r"(tags_a + k), "r"(lane) : "memory"); };
          auto tag_get = [&](int k) {
            uint32_t w;
            asm volatile("ld.shared.u8 %0, [%1];" : "=r"(w) : "r"(tags_a + k) : "memory");
            return w;
          };
          auto col_get = [&](int k) {
            float f;
            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(f) : "r"(col_a + 4 * k) : "memory");
            return f;
          };
          auto col_put = [&](int k, float f) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(col_a + 4 * k), "f"(f) : "memory"); };
          int k[2];
          float v[2];
          fetch(0, k[0], v[0]);
          tag_put(k[0]);
#pragma unroll
          for (int st = 0; st < kSteps; ++st) {
            const int cur = st & 1, nxt = cur ^ 1;
            if (st + 1 < kSteps) fetch(st + 1, k[nxt], v[nxt]);
            __syncwarp();  // the tags of step st are written
            const unsigned winner = tag_get(k[cur]);
            const bool lost = winner != static_cast<unsigned>(lane);
            const float old = col_get(k[cur]);  // read ahead; used only by lanes that nothing clashes with
            if (st + 1 < kSteps) tag_put(k[nxt]);  // after this step's read-back, in program order
            const unsigned losers = __ballot_sync(0xffffffffu, lost);
            if (losers == 0u) {
              col_put(k[cur], old + v[cur]);
            } else {
              // All lanes that share a slot read the same tag: the one lane it names is not
              // lost, every other one is. So the lanes in a clash are exactly the losers and
              // the lanes they name; everybody else adds at once, and the few involved add one
              // after the other in lane order, which is source-row order.
              unsigned involved = losers | __reduce_or_sync(0xffffffffu, lost ? 1u << winner : 0u);
              if (__popc(involved) <= 8) {
                if (!((involved >> lane) & 1u)) col_put(k[cur], old + v[cur]);
                while (involved) {
                  const int l = __ffs(involved) - 1;
                  if (lane == l) col_put(k[cur], col_get(k[cur]) + v[cur]);
                  involved &= involved - 1;
                  __syncwarp();
                }
              } else {
                apply_in_rank_order(col, k[cur], v[cur], rank_among_earlier<32>(k[cur], lane));
              }
            }
          }
          if (__any_sync(0xffffffffu, oob != 0u) && lane == 0) flag_oob(status);
          __syncwarp();                                   // every lane is done with the tile ...
          if (lane == 0) mbar_arrive(empty_bar(stage));   // ... and this warp hands its share of the slot back
          if (++stage == kWideStages) { stage = 0; phase ^= 1u; }
        }
      }
      compute_warps_barrier();  // every column of the strip is final
      have_prev = true;
      prev_j0 = j0;
      prev_o = o;
    }
    if (have_prev)  // the last strip of this CTA
      for (int slab = 0; slab < nslabs; ++slab) store_rows(slab * kWideSelfRows + warp * 32, prev_j0, prev_o);
    if (lane == 0) tma_store_wait_all();
  }
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);  // copies still under way land before the shared memory is handed on
    __syncthreads();
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

// Few rows, long ones (17 x 2051: nine warps of the kernel above would walk 2051 sources
// each, one global-memory round trip per 64): the destinations of a row are cut into
// `slices` ranges and a warp owns one range of one row. It reads ALL sources of the row (32
// per step, the next step's loads in flight while this one is applied; the other warps of the
// row read the same lines out of L1 / L2) and applies those that fall into its range, in
// source order. The order of the additions into a destination is untouched.
template <typename T>
__global__ void __launch_bounds__(256) scatter_add_rows_sliced(const T* __restrict__ self, const int64_t* __restrict__ index, const T* __restrict__ src, T* __restrict__ out, RowArgs A,
                                                               int slices, int slice_rows, uint32_t* status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  unsigned char* tags = smem_raw + warp * kTagSlots;
  float* mine = reinterpret_cast<float*>(smem_raw + nwarps * kTagSlots) + static_cast<int64_t>(warp) * slice_rows;
  const int64_t items = A.outer * slices;
  for (int64_t item = static_cast<int64_t>(blockIdx.x) * nwarps + warp; item < items; item += static_cast<int64_t>(gridDim.x) * nwarps) {
    const int64_t o = item / slices;
    const int d = static_cast<int>(item - o * slices);
    const int64_t lo = static_cast<int64_t>(d) * slice_rows;
    const int n = static_cast<int>(A.rows - lo < slice_rows ? A.rows - lo : slice_rows);  // > 0 by the choice of slices
    for (int r = lane; r < n; r += 32) mine[r] = to_f32(self[o * A.rows + lo + r]);
    __syncwarp();
    if (o < A.idx_outer) {
      const int64_t* irow = index + o * A.idx_so;
      const T* srow = src + o * A.src_so;
      int64_t key = lane < A.idx_len ? irow[lane] : -1;
      T val = lane < A.idx_len ? srow[lane] : from_f32<T>(0.f);
      for (int64_t j0 = 0; j0 < A.idx_len; j0 += 32) {
        const int64_t jn = j0 + 32 + lane;
        const int64_t key_n = jn < A.idx_len ? irow[jn] : -1;
        const T val_n = jn < A.idx_len ? srow[jn] : from_f32<T>(0.f);
        const bool real = j0 + lane < A.idx_len;
        if (real && d == 0 && (key < 0 || key >= A.rows)) flag_oob(status);
        const bool take = real && key >= lo && key < lo + n;
        ordered_step<32>(mine, tags, take ? static_cast<int>(key - lo) : -1 - lane, take ? to_f32(val) : 0.f, 0, lane, lane);
        key = key_n;
        val = val_n;
      }
    }
    for (int r = lane; r < n; r += 32) out[o * A.rows + lo + r] = from_f32<T>(mine[r]);
    __syncwarp();
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

// ------------------------------------------------------------------ bucket path
// For shapes with little column / row parallelism (tall and narrow, ragged, strided) the
// sources are first grouped by DESTINATION: count per destination (integer atomics -- their
// order does not matter), exclusive scan, then every source drops (position along the
// scatter dimension, value) into its destination's segment at an arbitrary slot. One thread
// per destination finally replays its segment in ascending position, i.e. in the aten CPU
// order. Fully parallel over sources and destinations; ~3x the algorithmic traffic.
// Destinations with more than kLightMax contributions go to a CTA-cooperative replay.
constexpr int kLightMax = 32;
constexpr int kScanBlock = 256, kScanItems = 16, kScanTile = kScanBlock * kScanItems;
constexpr int kHeavyWindow = 4096;

struct BucketArgs {
  int ndim, dim;
  int64_t n_idx, n_self, dim_len, self_dim_size;
  int64_t shape[B200_MAX_DIMS];  // index shape
  int64_t out_stride[B200_MAX_DIMS], idx_stride[B200_MAX_DIMS], src_stride[B200_MAX_DIMS];
};

__device__ __forceinline__ bool bucket_decode(const BucketArgs& A, int64_t p, const int64_t* __restrict__ index, int64_t& dest, int64_t& so, int& pos, uint32_t* status) {
  int64_t oo = 0, io = 0;
  so = 0;
  pos = 0;
  if (A.n_idx <= 0x7fffffffLL) {  // coordinates by 32-bit division (a 64-bit one costs ~5x the instructions)
    uint32_t lin = static_cast<uint32_t>(p);
    for (int d = A.ndim - 1; d >= 0; --d) {
      const uint32_t ext = static_cast<uint32_t>(A.shape[d]);
      const uint32_t q = lin / ext, r = lin - q * ext;
      io += r * A.idx_stride[d];
      so += r * A.src_stride[d];
      if (d == A.dim) pos = static_cast<int>(r);
      else oo += r * A.out_stride[d];
      lin = q;
    }
  } else {
    int64_t lin = p;
    for (int d = A.ndim - 1; d >= 0; --d) {
      const int64_t q = lin / A.shape[d], r = lin - q * A.shape[d];
      io += r * A.idx_stride[d];
      so += r * A.src_stride[d];
      if (d == A.dim) pos = static_cast<int>(r);
      else oo += r * A.out_stride[d];
      lin = q;
    }
  }
  const int64_t key = index[io];
  if (key < 0 || key >= A.self_dim_size) {
    flag_oob(status);
    return false;
  }
  dest = oo + key * A.out_stride[A.dim];
  return true;
}

__global__ void __launch_bounds__(256) bucket_count(const int64_t* __restrict__ index, int* __restrict__ cnt, BucketArgs A, uint32_t* status) {
  for (int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p < A.n_idx; p += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t dest, so;
    int pos;
    if (bucket_decode(A, p, index, dest, so, pos, nullptr)) atomicAdd(&cnt[dest], 1);
  }
}

// Exclusive scan of cnt[0, n) in three launches: per-tile totals, scan of the totals by one
// CTA, per-tile rescan with the tile's prefix. Writes offs (in place) and a copy in cursor.
__global__ void __launch_bounds__(kScanBlock) scan_tile_totals(const int* __restrict__ cnt, int* __restrict__ totals, int64_t n) {
  __shared__ int red[kScanBlock / 32];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile;
  int s = 0;
  for (int i = threadIdx.x; i < kScanTile; i += kScanBlock)
    if (base + i < n) s += cnt[base + i];
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int w = 0; w < kScanBlock / 32; ++w) t += red[w];
    totals[blockIdx.x] = t;
  }
}
__global__ void __launch_bounds__(1024) scan_totals(int* __restrict__ totals, int64_t ntiles, int* __restrict__ grand_total) {
  __shared__ int warp_sums[32];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int64_t base = 0; base < ntiles; base += 1024) {
    const int64_t i = base + threadIdx.x;
    const int v = i < ntiles ? totals[i] : 0;
    int inc = v;
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, inc, o);
      if ((threadIdx.x & 31) >= o) inc += y;
    }
    if ((threadIdx.x & 31) == 31) warp_sums[threadIdx.x >> 5] = inc;
    __syncthreads();
    if (threadIdx.x < 32) {
      int w = warp_sums[threadIdx.x];
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, w, o);
        if (threadIdx.x >= o) w += y;
      }
      warp_sums[threadIdx.x] = w;
    }
    __syncthreads();
    const int warp_prefix = (threadIdx.x >> 5) ? warp_sums[(threadIdx.x >> 5) - 1] : 0;
    const int excl = carry + warp_prefix + inc - v;
    if (i < ntiles) totals[i] = excl;
    __syncthreads();
    if (threadIdx.x == 1023) carry = excl + v;
    __syncthreads();
  }
  if (threadIdx.x == 0) *grand_total = carry;
}
__global__ void __launch_bounds__(kScanBlock) scan_apply(int* __restrict__ cnt_offs, int* __restrict__ cursor, const int* __restrict__ totals, int64_t n) {
  __shared__ int warp_sums[kScanBlock / 32];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile + static_cast<int64_t>(threadIdx.x) * kScanItems;
  // a thread's 16 counters are 64 contiguous, 64-byte aligned bytes: four 16-byte accesses
  const bool whole = base + kScanItems <= n && ((reinterpret_cast<uintptr_t>(cnt_offs) | reinterpret_cast<uintptr_t>(cursor)) & 15u) == 0;
  int v[kScanItems], s = 0;
  if (whole) {
#pragma unroll
    for (int q = 0; q < kScanItems / 4; ++q) {
      const int4 t = reinterpret_cast<const int4*>(cnt_offs + base)[q];
      v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) v[k] = base + k < n ? cnt_offs[base + k] : 0;
  }
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) s += v[k];
  int inc = s;
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, inc, o);
    if ((threadIdx.x & 31) >= o) inc += y;
  }
  if ((threadIdx.x & 31) == 31) warp_sums[threadIdx.x >> 5] = inc;
  __syncthreads();
  int prefix = totals[blockIdx.x] + inc - s;
  for (int w = 0; w < (threadIdx.x >> 5); ++w) prefix += warp_sums[w];
  if (whole) {
#pragma unroll
    for (int q = 0; q < kScanItems / 4; ++q) {
      int4 t;
      t.x = prefix; prefix += v[4 * q];
      t.y = prefix; prefix += v[4 * q + 1];
      t.z = prefix; prefix += v[4 * q + 2];
      t.w = prefix; prefix += v[4 * q + 3];
      reinterpret_cast<int4*>(cnt_offs + base)[q] = t;
      reinterpret_cast<int4*>(cursor + base)[q] = t;
    }
    return;
  }
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    if (base + k < n) {
      cnt_offs[base + k] = prefix;
      cursor[base + k] = prefix;
    }
    prefix += v[k];
  }
}

template <typename T>
__global__ void __launch_bounds__(256) bucket_fill(const int64_t* __restrict__ index, const T* __restrict__ src, int* __restrict__ cursor, int2* __restrict__ seg,
                                                   BucketArgs A, uint32_t* status) {
  for (int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p < A.n_idx; p += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t dest, so;
    int pos;
    if (bucket_decode(A, p, index, dest, so, pos, status)) {
      const int slot = atomicAdd(&cursor[dest], 1);
      seg[slot] = make_int2(pos, __float_as_int(to_f32(src[so])));  // (position, value) in one 8-byte store
    }
  }
}

// One thread per destination: replay its segment in ascending source position.
template <typename T>
__global__ void __launch_bounds__(256) bucket_replay(const T* __restrict__ self, T* __restrict__ out, const int* __restrict__ offs, const int* __restrict__ grand_total,
                                                     const int2* __restrict__ seg, int64_t n_self, int* __restrict__ heavy_count,
                                                     int* __restrict__ heavy_list) {
  for (int64_t d = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; d < n_self; d += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int b = offs[d], e = d + 1 < n_self ? offs[d + 1] : *grand_total;
    const int c = e - b;
    if (c == 0) {
      out[d] = self[d];
    } else if (c <= kLightMax) {
      float acc = to_f32(self[d]);
      int last = -1;
      for (int i = 0; i < c; ++i) {
        int best = 0x7fffffff;
        float bv = 0.f;
        for (int j = b; j < e; ++j) {
          const int2 pv = seg[j];
          if (pv.x > last && pv.x < best) { best = pv.x; bv = __int_as_float(pv.y); }
        }
        acc += bv;
        last = best;
      }
      out[d] = from_f32<T>(acc);
    } else {
      heavy_list[atomicAdd(heavy_count, 1)] = static_cast<int>(d);
    }
  }
}

// Destinations with long segments: one CTA each. The segment is visited in windows of
// kHeavyWindow source positions; inside a window every element is parked at its position,
// the occupied slots are compacted in order with a block scan, and one thread adds them.
template <typename T>
__global__ void __launch_bounds__(256) bucket_replay_heavy(const T* __restrict__ self, T* __restrict__ out, const int* __restrict__ offs, const int* __restrict__ grand_total,
                                                           const int2* __restrict__ seg, int64_t n_self, int64_t dim_len,
                                                           const int* __restrict__ heavy_count, const int* __restrict__ heavy_list) {
  __shared__ float slot_val[kHeavyWindow];
  __shared__ unsigned char slot_set[kHeavyWindow];
  __shared__ float ordered[kHeavyWindow];
  __shared__ int warp_sums[8];
  __shared__ int window_count;
  __shared__ float acc_s;
  const int nheavy = *heavy_count;
  constexpr int kPer = kHeavyWindow / 256;
  for (int h = blockIdx.x; h < nheavy; h += gridDim.x) {
    const int64_t d = heavy_list[h];
    const int b = offs[d], e = d + 1 < n_self ? offs[d + 1] : *grand_total;
    if (threadIdx.x == 0) acc_s = to_f32(self[d]);
    for (int64_t w0 = 0; w0 < dim_len; w0 += kHeavyWindow) {
      for (int i = threadIdx.x; i < kHeavyWindow; i += 256) slot_set[i] = 0;
      __syncthreads();
      for (int j = b + threadIdx.x; j < e; j += 256) {
        const int2 pv = seg[j];
        const int64_t pj = pv.x;
        if (pj >= w0 && pj < w0 + kHeavyWindow) {
          slot_val[pj - w0] = __int_as_float(pv.y);
          slot_set[pj - w0] = 1;
        }
      }
      __syncthreads();
      int mine = 0;
#pragma unroll
      for (int k = 0; k < kPer; ++k) mine += slot_set[threadIdx.x * kPer + k];
      int inc = mine;
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, inc, o);
        if ((threadIdx.x & 31) >= o) inc += y;
      }
      if ((threadIdx.x & 31) == 31) warp_sums[threadIdx.x >> 5] = inc;
      __syncthreads();
      int prefix = inc - mine;
      for (int w = 0; w < (threadIdx.x >> 5); ++w) prefix += warp_sums[w];
      if (threadIdx.x == 255) window_count = prefix + mine;
#pragma unroll
      for (int k = 0; k < kPer; ++k)
        if (slot_set[threadIdx.x * kPer + k]) ordered[prefix++] = slot_val[threadIdx.x * kPer + k];
      __syncthreads();
      if (threadIdx.x == 0) {
        float acc = acc_s;
        const int n = window_count;
        for (int i = 0; i < n; ++i) acc += ordered[i];
        acc_s = acc;
      }
      __syncthreads();
    }
    if (threadIdx.x == 0) out[d] = from_f32<T>(acc_s);
    __syncthreads();
  }
}

struct BucketScratch {
  int64_t offs_bytes, cursor_bytes, pos_bytes, val_bytes, totals_bytes, heavy_bytes, total;
};
static BucketScratch bucket_scratch(int64_t n_self, int64_t n_idx) {
  auto up = [](int64_t b) { return (b + 255) / 256 * 256; };
  BucketScratch s;
  s.offs_bytes = up(4 * (n_self + 1));
  s.cursor_bytes = up(4 * n_self);
  s.pos_bytes = up(4 * n_idx);
  s.val_bytes = up(4 * n_idx);
  s.totals_bytes = up(4 * ((n_self + kScanTile - 1) / kScanTile + 2));
  s.heavy_bytes = up(4 * (n_idx / (kLightMax + 1) + 4));
  s.total = s.offs_bytes + s.cursor_bytes + s.pos_bytes + s.val_bytes + s.totals_bytes + s.heavy_bytes;
  return s;
}

template <typename T>
static int launch_bucket(const void* self, const void* index, const void* src, void* out, const BucketArgs& A, void* scratch, uint32_t* status, cudaStream_t st) {
  const BucketScratch S = bucket_scratch(A.n_self, A.n_idx);
  char* base = static_cast<char*>(scratch);
  int* offs = reinterpret_cast<int*>(base);
  int* cursor = reinterpret_cast<int*>(base + S.offs_bytes);
  int2* seg = reinterpret_cast<int2*>(base + S.offs_bytes + S.cursor_bytes);  // (source position, value bits) per contribution: pos_bytes + val_bytes
  int* totals = reinterpret_cast<int*>(base + S.offs_bytes + S.cursor_bytes + S.pos_bytes + S.val_bytes);
  int* heavy = reinterpret_cast<int*>(base + S.offs_bytes + S.cursor_bytes + S.pos_bytes + S.val_bytes + S.totals_bytes);  // [0] count, [1] grand total, [4..] list
  cudaError_t e = cudaMemsetAsync(offs, 0, static_cast<size_t>(S.offs_bytes), st);
  if (e == cudaSuccess) e = cudaMemsetAsync(heavy, 0, 16, st);
  if (e != cudaSuccess) { set_last_cuda_error(e); return B200_ELAUNCH; }
  const int64_t* pi = static_cast<const int64_t*>(index);
  auto grid = [](int64_t n, int per) { int64_t g = (n + per - 1) / per; const int64_t cap = 32LL * kNumSMs; return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g)); };
  const int64_t ntiles = (A.n_self + kScanTile - 1) / kScanTile;
  bucket_count<<<grid(A.n_idx, 256), 256, 0, st>>>(pi, offs, A, status);
  scan_tile_totals<<<static_cast<unsigned>(ntiles), kScanBlock, 0, st>>>(offs, totals, A.n_self);
  scan_totals<<<1, 1024, 0, st>>>(totals, ntiles, heavy + 1);
  scan_apply<<<static_cast<unsigned>(ntiles), kScanBlock, 0, st>>>(offs, cursor, totals, A.n_self);
  bucket_fill<T><<<grid(A.n_idx, 256), 256, 0, st>>>(pi, static_cast<const T*>(src), cursor, seg, A, status);
  bucket_replay<T><<<grid(A.n_self, 256), 256, 0, st>>>(static_cast<const T*>(self), static_cast<T*>(out), offs, heavy + 1, seg, A.n_self, heavy, heavy + 4);
  bucket_replay_heavy<T><<<2 * kNumSMs, 256, 0, st>>>(static_cast<const T*>(self), static_cast<T*>(out), offs, heavy + 1, seg, A.n_self, A.dim_len, heavy, heavy + 4);
  return check_launch(7);
}

// ------------------------------------------------------------------ embedding_dense_backward
// out[v, :] = sum over the positions i with indices[i] == v (and v != padding_idx) of
// grad[i, :], in ascending i, fp32 accumulation, one rounding: the bucket scheme above with
// whole rows as the unit. count per destination row -> exclusive scan -> fill the row's
// segment with its source positions (slot order arbitrary) -> replay. A row with at most 32
// contributions is replayed by one warp, which ranks the positions with shuffles; a heavier
// row by one CTA, which marks the positions in a shared-memory bitmap (a window of 2^18
// positions at a time, with a summary word per 32 bitmap words) and walks the bitmap in
// order -- ascending positions with no sort.
constexpr int kEmbWindowBits = 1 << 18;
constexpr int kEmbWindowWords = kEmbWindowBits / 32;

__device__ __forceinline__ int64_t emb_index(const void* idx, int64_t i, int i32) { return i32 ? static_cast<const int32_t*>(idx)[i] : static_cast<const int64_t*>(idx)[i]; }

__global__ void __launch_bounds__(256) emb_count(const void* __restrict__ idx, int i32, int64_t n, int64_t V, int64_t padding_idx, int* __restrict__ cnt, uint32_t* status) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t v = emb_index(idx, i, i32);
    if (v == padding_idx) continue;
    if (v < 0 || v >= V) { flag_oob(status); continue; }
    atomicAdd(&cnt[v], 1);
  }
}
__global__ void __launch_bounds__(256) emb_fill(const void* __restrict__ idx, int i32, int64_t n, int64_t V, int64_t padding_idx, int* __restrict__ cursor, int* __restrict__ seg_pos) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t v = emb_index(idx, i, i32);
    if (v == padding_idx || v < 0 || v >= V) continue;
    seg_pos[atomicAdd(&cursor[v], 1)] = static_cast<int>(i);
  }
}

// acc[0..VE) += grad[pos, col .. col + VE) (VE = 16 bytes of T when `vec`, else 1)
template <typename T, bool VEC>
__device__ __forceinline__ void emb_add_row(float* acc, const T* __restrict__ grad, int64_t pos, int64_t D, int64_t col) {
  if (VEC) {
    float f[Vec<T>::N];
    widen<T>(ld_stream(grad + pos * D + col), f);
#pragma unroll
    for (int e = 0; e < Vec<T>::N; ++e) acc[e] += f[e];
  } else {
    acc[0] += to_f32(grad[pos * D + col]);
  }
}
template <typename T, bool VEC>
__device__ __forceinline__ void emb_store(T* __restrict__ out, int64_t v, int64_t D, int64_t col, const float* acc) {
  if (VEC) st_stream(out + v * D + col, narrow<T>(acc));
  else out[v * D + col] = from_f32<T>(acc[0]);
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(256) emb_replay(const T* __restrict__ grad, T* __restrict__ out, const int* __restrict__ offs, const int* __restrict__ grand_total, const int* __restrict__ seg_pos,
                                                  int64_t V, int64_t D, int* __restrict__ heavy_count, int* __restrict__ heavy_list) {
  constexpr int VE = VEC ? Vec<T>::N : 1;
  __shared__ int sorted[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t units = D / VE;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * 8 + warp; v < V; v += static_cast<int64_t>(gridDim.x) * 8) {
    const int b = offs[v], e = v + 1 < V ? offs[v + 1] : *grand_total;
    const int c = e - b;
    if (c > 32) {
      if (lane == 0) heavy_list[atomicAdd(heavy_count, 1)] = static_cast<int>(v);
      continue;
    }
    // rank of this lane's position among the row's positions (all distinct)
    const int p = lane < c ? seg_pos[b + lane] : 0x7fffffff;
    int rank = 0;
#pragma unroll
    for (int k = 0; k < 32; ++k) rank += __shfl_sync(0xffffffffu, p, k) < p ? 1 : 0;
    __syncwarp();
    if (lane < c) sorted[warp][rank] = p;
    __syncwarp();
    for (int64_t u = lane; u < units; u += 32) {
      float acc[VE];
#pragma unroll
      for (int q = 0; q < VE; ++q) acc[q] = 0.f;
      for (int k = 0; k < c; ++k) emb_add_row<T, VEC>(acc, grad, sorted[warp][k], D, u * VE);
      emb_store<T, VEC>(out, v, D, u * VE, acc);
    }
  }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(256) emb_replay_heavy(const T* __restrict__ grad, T* __restrict__ out, const int* __restrict__ offs, const int* __restrict__ grand_total,
                                                        const int* __restrict__ seg_pos, int64_t V, int64_t D, int64_t n, const int* __restrict__ heavy_count, const int* __restrict__ heavy_list) {
  constexpr int VE = VEC ? Vec<T>::N : 1;
  __shared__ uint32_t bitmap[kEmbWindowWords];
  __shared__ uint32_t summary[kEmbWindowWords / 32];
  const int64_t units = D / VE;
  for (int h = blockIdx.x; h < *heavy_count; h += gridDim.x) {
    const int64_t v = heavy_list[h];
    const int b = offs[v], e = v + 1 < V ? offs[v + 1] : *grand_total;
    // the row's columns are taken blockDim.x vectors at a time; every pass walks all windows
    for (int64_t u0 = 0; u0 < units; u0 += blockDim.x) {
      const int64_t u = u0 + threadIdx.x;
      float acc[VE];
#pragma unroll
      for (int q = 0; q < VE; ++q) acc[q] = 0.f;
      for (int64_t w0 = 0; w0 < n; w0 += kEmbWindowBits) {
        __syncthreads();  // the bitmap of the window before has been read by everyone
        for (int i = threadIdx.x; i < kEmbWindowWords; i += blockDim.x) bitmap[i] = 0u;
        for (int i = threadIdx.x; i < kEmbWindowWords / 32; i += blockDim.x) summary[i] = 0u;
        __syncthreads();
        for (int j = b + threadIdx.x; j < e; j += blockDim.x) {
          const int64_t rel = static_cast<int64_t>(seg_pos[j]) - w0;
          if (rel >= 0 && rel < kEmbWindowBits) {
            atomicOr(&bitmap[rel >> 5], 1u << (rel & 31));
            atomicOr(&summary[rel >> 10], 1u << ((rel >> 5) & 31));
          }
        }
        __syncthreads();
        if (u < units) {
          for (int sw = 0; sw < kEmbWindowWords / 32; ++sw) {
            uint32_t words = summary[sw];
            while (words) {
              const int wi = sw * 32 + __ffs(words) - 1;
              words &= words - 1;
              uint32_t bits = bitmap[wi];
              while (bits) {
                const int64_t pos = w0 + wi * 32 + __ffs(bits) - 1;
                bits &= bits - 1;
                emb_add_row<T, VEC>(acc, grad, pos, D, u * VE);
              }
            }
          }
        }
      }
      if (u < units) emb_store<T, VEC>(out, v, D, u * VE, acc);
    }
  }
}

struct EmbScratch {
  int64_t offs_bytes, cursor_bytes, pos_bytes, totals_bytes, heavy_bytes, total;
};
static EmbScratch emb_scratch(int64_t V, int64_t n) {
  auto up = [](int64_t b) { return (b + 255) / 256 * 256; };
  EmbScratch s;
  s.offs_bytes = up(4 * (V + 1));
  s.cursor_bytes = up(4 * V);
  s.pos_bytes = up(4 * n);
  s.totals_bytes = up(4 * ((V + kScanTile - 1) / kScanTile + 2));
  s.heavy_bytes = up(4 * (n / 33 + 4));
  s.total = s.offs_bytes + s.cursor_bytes + s.pos_bytes + s.totals_bytes + s.heavy_bytes;
  return s;
}

template <typename T>
static int launch_embedding_backward(const void* grad, const void* idx, void* out, int64_t n, int64_t V, int64_t D, int64_t padding_idx, int i32, void* scratch, uint32_t* status, cudaStream_t st) {
  const EmbScratch S = emb_scratch(V, n);
  char* base = static_cast<char*>(scratch);
  int* offs = reinterpret_cast<int*>(base);
  int* cursor = reinterpret_cast<int*>(base + S.offs_bytes);
  int* seg_pos = reinterpret_cast<int*>(base + S.offs_bytes + S.cursor_bytes);
  int* totals = reinterpret_cast<int*>(base + S.offs_bytes + S.cursor_bytes + S.pos_bytes);
  int* heavy = reinterpret_cast<int*>(base + S.offs_bytes + S.cursor_bytes + S.pos_bytes + S.totals_bytes);  // [0] count, [1] grand total, [4..] list
  cudaError_t e = cudaMemsetAsync(offs, 0, static_cast<size_t>(S.offs_bytes), st);
  if (e == cudaSuccess) e = cudaMemsetAsync(heavy, 0, 16, st);
  if (e != cudaSuccess) { set_last_cuda_error(e); return B200_ELAUNCH; }
  auto grid = [](int64_t items, int per) { int64_t g = (items + per - 1) / per; const int64_t cap = 32LL * kNumSMs; return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g)); };
  const int64_t ntiles = (V + kScanTile - 1) / kScanTile;
  emb_count<<<grid(n, 256), 256, 0, st>>>(idx, i32, n, V, padding_idx, offs, status);
  scan_tile_totals<<<static_cast<unsigned>(ntiles), kScanBlock, 0, st>>>(offs, totals, V);
  scan_totals<<<1, 1024, 0, st>>>(totals, ntiles, heavy + 1);
  scan_apply<<<static_cast<unsigned>(ntiles), kScanBlock, 0, st>>>(offs, cursor, totals, V);
  emb_fill<<<grid(n, 256), 256, 0, st>>>(idx, i32, n, V, padding_idx, cursor, seg_pos);
  const T* g = static_cast<const T*>(grad);
  T* o = static_cast<T*>(out);
  const bool vec = (D * static_cast<int64_t>(sizeof(T))) % 16 == 0 && aligned16(grad) && aligned16(out);
  if (vec) {
    emb_replay<T, true><<<grid(V, 8), 256, 0, st>>>(g, o, offs, heavy + 1, seg_pos, V, D, heavy, heavy + 4);
    emb_replay_heavy<T, true><<<2 * kNumSMs, 256, 0, st>>>(g, o, offs, heavy + 1, seg_pos, V, D, n, heavy, heavy + 4);
  } else {
    emb_replay<T, false><<<grid(V, 8), 256, 0, st>>>(g, o, offs, heavy + 1, seg_pos, V, D, heavy, heavy + 4);
    emb_replay_heavy<T, false><<<2 * kNumSMs, 256, 0, st>>>(g, o, offs, heavy + 1, seg_pos, V, D, n, heavy, heavy + 4);
  }
  return check_launch(7);
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
static int launch_strip_wide(const void* self, const void* index, const void* src, void* out, const StripArgs& A, uint32_t* status, cudaStream_t st) {
  // tensor maps over the index and value tensors (this GPU's own memory, no multicast): boxes
  // of 8 columns x 128 rows, swizzled the way the compute warps read them
  if (!encode_fn()) return B200_EDRIVER;
  alignas(64) CUtensorMap map_idx, map_src;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(A.idx_cols), static_cast<cuuint64_t>(A.idx_rows), static_cast<cuuint64_t>(A.idx_outer)};
  const cuuint32_t box[3] = {kWideCols, kWideTileRows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  auto outer_stride = [&](int64_t so, int64_t sr, int64_t es) { return static_cast<cuuint64_t>((A.idx_outer > 1 && so > 0 ? so : sr * A.idx_rows) * es); };
  const cuuint64_t istr[2] = {static_cast<cuuint64_t>(A.idx_sr) * 8, outer_stride(A.idx_so, A.idx_sr, 8)};
  const int es = static_cast<int>(sizeof(T));
  const cuuint64_t sstr[2] = {static_cast<cuuint64_t>(A.src_sr) * es, outer_stride(A.src_so, A.src_sr, es)};
  if (istr[1] % 16 || sstr[1] % 16) return B200_EALIGN;
  if (encode_fn()(&map_idx, CU_TENSOR_MAP_DATA_TYPE_INT64, 3, const_cast<void*>(index), dims, istr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return B200_EDRIVER;
  const CUtensorMapDataType vt = std::is_same<T, float>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : std::is_same<T, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUtensorMapSwizzle vs = sizeof(T) == 4 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;  // 16-bit rows are one 16-byte chunk
  if (encode_fn()(&map_src, vt, 3, const_cast<void*>(src), dims, sstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, vs, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) !=
      CUDA_SUCCESS)
    return B200_EDRIVER;
  alignas(64) CUtensorMap map_self;  // the destination strip on its way in: 8 columns x 256 rows, rows as they lie
  {
    const cuuint64_t ddims[3] = {static_cast<cuuint64_t>(A.cols), static_cast<cuuint64_t>(A.rows), static_cast<cuuint64_t>(A.outer)};
    const cuuint64_t dstr[2] = {static_cast<cuuint64_t>(A.cols) * es, static_cast<cuuint64_t>(A.rows) * static_cast<cuuint64_t>(A.cols) * es};
    const cuuint32_t dbox[3] = {kWideCols, kWideSelfRows, 1};
    if (dstr[0] % 16 || (reinterpret_cast<uintptr_t>(self) & 15)) return B200_EALIGN;
    if (encode_fn()(&map_self, vt, 3, const_cast<void*>(self), ddims, dstr, dbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return B200_EDRIVER;
  }
  alignas(64) CUtensorMap map_out;  // ... and on its way out: 8 columns x 32 rows
  {
    const cuuint64_t ddims[3] = {static_cast<cuuint64_t>(A.cols), static_cast<cuuint64_t>(A.rows), static_cast<cuuint64_t>(A.outer)};
    const cuuint64_t dstr[2] = {static_cast<cuuint64_t>(A.cols) * es, static_cast<cuuint64_t>(A.rows) * static_cast<cuuint64_t>(A.cols) * es};
    const cuuint32_t dbox[3] = {kWideCols, kWideOutRows, 1};
    if (reinterpret_cast<uintptr_t>(out) & 15) return B200_EALIGN;
    if (encode_fn()(&map_out, vt, 3, out, ddims, dstr, dbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) !=
        CUDA_SUCCESS)
      return B200_EDRIVER;
  }
  // ring + tag tables + the strip at its largest + barriers + room to align the ring to 1 KB
  const size_t smem = static_cast<size_t>(kWideStages) * kWideTileRows * kWideCols * (8 + sizeof(T)) + 8 * (kWideTagSlots + kWideDummies) + static_cast<size_t>(kWideMaxRows + kWideDummies) * kWideCols * 4 + 128 + 1024;
  const cudaError_t ae = cudaFuncSetAttribute(scatter_add_strip_wide<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (ae != cudaSuccess) { set_last_cuda_error(ae); return B200_ELAUNCH; }
  const int64_t items = A.outer * (A.cols / kWideCols);
  const int grid = static_cast<int>(items < kNumSMs ? items : kNumSMs);  // one CTA per SM: a strip leaves while the next one comes in
  scatter_add_strip_wide<T><<<grid, kWideThreads, smem, st>>>(map_idx, map_src, map_self, map_out, A, status);
  return check_launch();
}

template <typename T>
static int launch_rows(const void* self, const void* index, const void* src, void* out, RowArgs A, uint32_t* status, cudaStream_t st) {
  // few long rows: several warps per row, each with a range of the row's destinations
  if (A.outer < 2LL * kNumSMs && A.idx_len >= 256 && A.rows >= 128) {
    int64_t slices = (4LL * kNumSMs + A.outer - 1) / A.outer;
    if (slices > A.rows / 64) slices = A.rows / 64;
    if (slices > 32) slices = 32;
    if (slices >= 2) {
      const int64_t slice_rows = (A.rows + slices - 1) / slices;
      slices = (A.rows + slice_rows - 1) / slice_rows;  // no empty range at the end
      int warps = 8;
      while (warps > 1 && static_cast<int64_t>(warps) * (slice_rows * 4 + kTagSlots) > 96 * 1024) warps >>= 1;
      const size_t smem = static_cast<size_t>(warps) * (slice_rows * 4 + kTagSlots);
      if (smem <= static_cast<size_t>(kSmemBudget)) {
        const cudaError_t ae = cudaFuncSetAttribute(scatter_add_rows_sliced<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
        if (ae != cudaSuccess) { set_last_cuda_error(ae); return B200_ELAUNCH; }
        const int64_t items = A.outer * slices;
        // one item per warp where the machine has room: spread the items over the SMs first
        int per_cta = static_cast<int>((items + kNumSMs - 1) / kNumSMs);
        if (per_cta > warps) per_cta = warps;
        if (per_cta < 1) per_cta = 1;
        const int64_t blocks = (items + per_cta - 1) / per_cta;
        scatter_add_rows_sliced<T><<<static_cast<int>(blocks), per_cta * 32, static_cast<size_t>(per_cta) * (slice_rows * 4 + kTagSlots), st>>>(
            static_cast<const T*>(self), static_cast<const int64_t*>(index), static_cast<const T*>(src), static_cast<T*>(out), A, static_cast<int>(slices), static_cast<int>(slice_rows), status);
        return check_launch();
      }
    }
  }
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

namespace b200 {

enum ScatterPath { kPathNone = 0, kPathStrip, kPathStripWide, kPathRows, kPathBucket, kPathLines };

struct ScatterPlan {
  ScatterPath path;
  int64_t n_self, n_idx, scratch_bytes;
  StripArgs strip;
  RowArgs rows;
};

// Decides which kernel family serves a geometry (shared by the launcher and the scratch
// query so that both always agree).
static ScatterPlan plan_scatter(const void* self, const void* index, const void* src, const void* out, int ndim, const int64_t* self_shape, const int64_t* index_shape,
                                const int64_t* index_strides, const int64_t* src_strides, int dim, int dtype) {
  ScatterPlan P{};
  P.n_self = numel_of(ndim, self_shape);
  P.n_idx = numel_of(ndim, index_shape);
  const int es = dtype_size(dtype);
  P.path = kPathLines;
  if (P.n_self == 0 || P.n_idx == 0) { P.path = kPathNone; return P; }
  const bool small = P.n_idx <= (1 << 16);  // launch-bound either way
  if (aligned16(self) && aligned16(out) && aligned16(index) && aligned16(src)) {
    int64_t outer = 1, cols = 1, idx_outer = 1, idx_cols = 1;
    for (int d = 0; d < dim; ++d) { outer *= self_shape[d]; idx_outer *= index_shape[d]; }
    for (int d = dim + 1; d < ndim; ++d) { cols *= self_shape[d]; idx_cols *= index_shape[d]; }
    const int64_t rows = self_shape[dim], idx_rows = index_shape[dim];
    int lead = 0, trail = 0, dl = -1, dt = -1;  // collapsible only with at most one non-trivial dim on each side
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
        const int64_t strips = outer * (cols / kStripCols);
        const bool fits = rows * kStripCols * 4 <= 2 * (kSmemBudget - 64 * 1024);  // at most two destination windows
        if (inner_ok && shape_ok && stride_ok && fits && (strips >= 32 || small)) {
          P.path = kPathStrip;
          P.strip = StripArgs{outer, rows, cols, idx_outer, idx_rows, idx_cols, idx_so, index_strides[dim], src_so, src_strides[dim], 0, 0};
          // eight columns per CTA when the whole destination strip fits and every staged chunk is 16-byte aligned
          const bool wide_shape = cols % kWideCols == 0 && idx_cols % kWideCols == 0 && rows <= kWideMaxRows && idx_rows >= 256 && idx_rows < 0x7fffffffLL && outer * (cols / kWideCols) >= kNumSMs / 2;
          const bool wide_align = index_strides[dim] % 2 == 0 && idx_so % 2 == 0 && (src_strides[dim] * es) % 16 == 0 && (src_so * es) % 16 == 0;
          if (wide_shape && wide_align) P.path = kPathStripWide;
          return P;
        }
      } else if (index_strides[dim] == 1 && src_strides[dim] == 1) {
        const bool fits = rows * 2 * 4 <= kSmemBudget - 16 * 1024;
        if (fits && (outer >= 64 || small)) {
          P.path = kPathRows;
          P.rows = RowArgs{outer, rows, idx_outer, idx_rows, idx_so, src_so, 0};
          return P;
        }
      }
    }
  }
  // short lines are cheapest walked by one thread each; anything longer is grouped by destination
  if (P.n_self < 0x7fffffffLL && P.n_idx < 0x7fffffffLL && index_shape[dim] < 0x7fffffffLL && index_shape[dim] > 64) {
    P.path = kPathBucket;
    P.scratch_bytes = bucket_scratch(P.n_self, P.n_idx).total;
    return P;
  }
  P.scratch_bytes = dtype == B200_F32 ? 0 : P.n_self * 4;  // fp32 accumulator of the line kernel
  return P;
}

}  // namespace b200

using namespace b200;

extern "C" int64_t b200_scatter_add_scratch_bytes(const void* self, const void* index, const void* src, const void* out, int ndim, const int64_t* self_shape,
                                                   const int64_t* index_shape, const int64_t* index_strides, const int64_t* src_strides, int dim, int dtype) {
  if (ndim < 1 || ndim > B200_MAX_DIMS || dim < 0 || dim >= ndim || !self_shape || !index_shape || !index_strides || !src_strides || !is_float_dtype(dtype)) return 0;
  return plan_scatter(self, index, src, out, ndim, self_shape, index_shape, index_strides, src_strides, dim, dtype).scratch_bytes;
}

extern "C" int b200_scatter_add(const void* self, const void* index, const void* src, void* out, int ndim, const int64_t* self_shape, const int64_t* index_shape,
                                const int64_t* index_strides, const int64_t* src_strides, int dim, int dtype, void* scratch, int64_t scratch_bytes, uint32_t* status, void* stream) {
  if (ndim < 1 || ndim > B200_MAX_DIMS || dim < 0 || dim >= ndim || !self_shape || !index_shape || !index_strides || !src_strides) return B200_EINVAL;
  if (!is_float_dtype(dtype)) return B200_EDTYPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (int d = 0; d < ndim; ++d)
    if (self_shape[d] < 0 || index_shape[d] < 0 || (d != dim && index_shape[d] > self_shape[d])) return B200_EINVAL;
  const int64_t n_self = numel_of(ndim, self_shape);
  const int64_t n_idx = numel_of(ndim, index_shape);
  if (n_self == 0) return B200_OK;
  if (!self || !out) return B200_EINVAL;
  if (n_idx > 0 && (!index || !src)) return B200_EINVAL;
  const int es = dtype_size(dtype);
  const ScatterPlan P = plan_scatter(self, index, src, out, ndim, self_shape, index_shape, index_strides, src_strides, dim, dtype);

  if (P.path == kPathNone) {  // nothing to add: the result is a copy of self (no scratch, whatever the dtype)
    if (out != self) {
      const cudaError_t ce = cudaMemcpyAsync(out, self, static_cast<size_t>(n_self) * es, cudaMemcpyDeviceToDevice, st);
      if (ce != cudaSuccess) { set_last_cuda_error(ce); return B200_ELAUNCH; }
    }
    return B200_OK;
  }
  if (P.path == kPathStrip) {
    switch (dtype) {
      case B200_F32: return launch_strip<float>(self, index, src, out, P.strip, status, st);
      case B200_BF16: return launch_strip<__nv_bfloat16>(self, index, src, out, P.strip, status, st);
      default: return launch_strip<__half>(self, index, src, out, P.strip, status, st);
    }
  }
  if (P.path == kPathStripWide) {
    switch (dtype) {
      case B200_F32: return launch_strip_wide<float>(self, index, src, out, P.strip, status, st);
      case B200_BF16: return launch_strip_wide<__nv_bfloat16>(self, index, src, out, P.strip, status, st);
      default: return launch_strip_wide<__half>(self, index, src, out, P.strip, status, st);
    }
  }
  if (P.path == kPathRows) {
    switch (dtype) {
      case B200_F32: return launch_rows<float>(self, index, src, out, P.rows, status, st);
      case B200_BF16: return launch_rows<__nv_bfloat16>(self, index, src, out, P.rows, status, st);
      default: return launch_rows<__half>(self, index, src, out, P.rows, status, st);
    }
  }
  if (P.path == kPathBucket) {
    if (!scratch || scratch_bytes < P.scratch_bytes) return B200_ESCRATCH;
    BucketArgs A;
    A.ndim = ndim;
    A.dim = dim;
    A.n_idx = n_idx;
    A.n_self = n_self;
    A.dim_len = index_shape[dim];
    A.self_dim_size = self_shape[dim];
    int64_t st_out = 1;
    for (int d = ndim - 1; d >= 0; --d) {
      A.shape[d] = index_shape[d];
      A.out_stride[d] = st_out;
      st_out *= self_shape[d];
      A.idx_stride[d] = index_strides[d];
      A.src_stride[d] = src_strides[d];
    }
    switch (dtype) {
      case B200_F32: return launch_bucket<float>(self, index, src, out, A, scratch, status, st);
      case B200_BF16: return launch_bucket<__nv_bfloat16>(self, index, src, out, A, scratch, status, st);
      default: return launch_bucket<__half>(self, index, src, out, A, scratch, status, st);
    }
  }

  // ---- line kernel: acc = fp32(self), ordered lines on acc, out = round(acc)
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

extern "C" int64_t b200_embedding_backward_scratch_bytes(int64_t n_indices, int64_t num_weights) {
  if (n_indices < 0 || num_weights <= 0) return 0;
  return emb_scratch(num_weights, n_indices).total;
}

extern "C" int b200_embedding_backward(const void* grad, const void* indices, void* out, int64_t n_indices, int64_t num_weights, int64_t row_len, int64_t padding_idx, int dtype, int idx_dtype,
                                       void* scratch, int64_t scratch_bytes, uint32_t* status, void* stream) {
  if (n_indices < 0 || num_weights < 0 || row_len < 0) return B200_EINVAL;
  if (!is_float_dtype(dtype)) return B200_EDTYPE;
  if (idx_dtype != B200_I32 && idx_dtype != B200_I64) return B200_EDTYPE;
  if (num_weights == 0 || row_len == 0) return B200_OK;
  if (!out || (n_indices > 0 && (!grad || !indices))) return B200_EINVAL;
  if (n_indices >= 0x7fffffffLL || num_weights >= 0x7fffffffLL) return B200_EINVAL;
  if (!scratch || scratch_bytes < b200_embedding_backward_scratch_bytes(n_indices, num_weights)) return B200_ESCRATCH;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int i32 = idx_dtype == B200_I32;
  switch (dtype) {
    case B200_F32: return launch_embedding_backward<float>(grad, indices, out, n_indices, num_weights, row_len, padding_idx, i32, scratch, status, st);
    case B200_BF16: return launch_embedding_backward<__nv_bfloat16>(grad, indices, out, n_indices, num_weights, row_len, padding_idx, i32, scratch, status, st);
    default: return launch_embedding_backward<__half>(grad, indices, out, n_indices, num_weights, row_len, padding_idx, i32, scratch, status, st);
  }
}
