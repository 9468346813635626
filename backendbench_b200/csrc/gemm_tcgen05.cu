// mm / addmm / bmm on the 5th-generation tensor cores (tcgen05) for bf16 / f16 operands.
//
//   C[b] (M x N, row-major) = alpha * A[b] (M x K) @ B[b] (K x N) + beta * bias
//
// One persistent CTA per SM walks 128 x 256 (or 128 x 128) output tiles. Roles by warp:
//   warp 0   : TMA producer -- one lane issues cp.async.bulk.tensor loads
//              of a 128 x 64 A slab and a 64 x 256 B slab per pipeline stage into
//              128-byte-swizzled shared memory, completion on an mbarrier.
//   warp 1   : owns tensor memory (allocates all 512 TMEM columns = two fp32 accumulators
//              of 128 lanes x 256 columns) and issues tcgen05.mma (kind::f16, M128 N256
//              K16, four per stage); tcgen05.commit releases the stage / publishes the
//              accumulator through mbarriers.
//   warps 2-9: epilogue -- tcgen05.ld the accumulator (a warp may read only the 32 TMEM
//              lanes of its quarter, so two warps share a quarter and split the 256
//              columns), scale / add bias in fp32, round once, 16-byte stores. While they
//              drain accumulator `a`, the MMA warp already fills accumulator `a ^ 1`.
// Tiles are walked in groups of 16 row-blocks x all column-blocks so that the CTAs running
// at the same time share A and B slabs in L2.
// Operands may be K-major or MN-major in global memory (A row- or column-major, B given
// as [K,N] or as a transposed [N,K] view): the layout goes into the shared-memory and
// instruction descriptors, nothing is copied or transposed. Ragged M / N / K edges rely on
// TMA zero fill for loads and predicated stores.
//
// CTA pairs (kPair): two CTAs of a 2-CTA cluster, on the two SMs of one TPC, share a 256 x 256
// tile. Each keeps the accumulator of ITS 128 rows in its own tensor memory and loads its own
// 128 x 64 A slab and HALF of the 64 x 256 B slab (32 KB per stage instead of 48, six stages);
// one thread of the even CTA issues tcgen05.mma.cta_group::2 (M256 N256 K16), which reads A
// from both shared memories and each half of B from its own. The odd CTA's copies complete on
// the even CTA's barrier, and tcgen05.commit.cta_group::2 hands stages and accumulators back
// to both. Per FLOP a third fewer operand bytes cross the L2-to-SM fabric, which is what the
// single-CTA kernel waits on at large shapes. No cluster multicast is used anywhere: every
// CTA fetches its own tiles.
//
// Every mbarrier wait is bounded: when a wait gives up the CTA sets an abort flag, ORs
// B200_DEV_WAIT_TIMEOUT into the caller's status word, lets outstanding copies land, frees
// its tensor memory and returns -- a protocol bug can produce a wrong result plus an error
// status, never a hung GPU.
#include <cuda.h>

#include <cstdlib>

#include "b200_common.cuh"
#include "tma_common.cuh"

namespace b200 {

constexpr int kBM = 128, kBK = 64;                      // tile: 128 x BN outputs (BN = 256 or 128), 64-deep K slabs
constexpr int kABytes = kBM * kBK * 2;                  // 16 KB
constexpr int kTmemCols = 512;                          // 512 / BN fp32 accumulators of 128 lanes x BN columns
// BN = 256: 48 KB stages x 4, two accumulators (compute-bound shapes).
// BN = 128: 32 KB stages x 6, four accumulators, for C no wider than 128 columns.
// A CTA of a pair holds half of the B slab: 32 KB stages x 6, two accumulators.
template <int BN, bool PAIR = false> struct TileCfg {
  static constexpr int kBRows = PAIR ? BN / 2 : BN;      // rows (N) of the B slab in THIS CTA's shared memory
  static constexpr int kBBytes = kBRows * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = kStageBytes == 49152 ? 4 : 6;
  static constexpr int kAccs = kTmemCols / BN;
};
constexpr int kGemmThreads = 320;                       // TMA warp, MMA warp, 8 epilogue warps
constexpr int kGroupM = 16;                             // row-blocks per rasterisation group
constexpr uint64_t kWaitLimitNs = 2000000000ull;        // every mbarrier wait gives up after 2 s
constexpr int kEpiWarps = 8;
constexpr int kEpiStageBytes = 32 * 128;                // per epilogue warp: 32 rows x 64 16-bit outputs, TMA-store staging
constexpr size_t kGemmSmem = static_cast<size_t>(4) * (kABytes + 256 * kBK * 2) + kEpiWarps * kEpiStageBytes + 1024 /*align*/ + 256 /*barriers*/;  // same for both tile shapes (6 x 32 KB = 4 x 48 KB)

// ------------------------------------------------------------------ PTX wrappers (mbarrier and timer helpers: tma_common.cuh)
// The same load issued by a CTA of a pair: the destination is this CTA's shared memory, the
// mbarrier (a shared::cluster address) may be the peer CTA's.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0),
               "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) { return map_to_cta_addr(addr, rank); }
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) { asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory"); }
__device__ __forceinline__ void cluster_sync_all() { cluster_barrier(); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) { asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// pair forms: the barrier address is a shared::cluster address (own or peer CTA)
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster) { asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster) : "memory"); }
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  const uint32_t z = 0u;  // no output lane is disabled
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tc_ld_32x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
        "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (128-byte swizzle, sm_100 format): start address,
// leading-dimension byte offset and stride byte offset in 16-byte units, version 1.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3fffu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= 1ull << 46;  // descriptor version for sm_100
  d |= 2ull << 61;  // SWIZZLE_128B
  return d;
}

struct GemmTcParams {
  int64_t M, N, K, batch;
  int64_t sbm, sbn;  // bias strides in elements (0 = broadcast)
  float alpha, beta;
  int a_mn_major, b_mn_major;  // 0: K contiguous in global memory, 1: M (resp. N) contiguous
  int is_bf16;
  int has_bias;
  int tma_store;    // 1 = C goes out through TMA tile stores (N % 8 == 0, aligned), 0 = plain stores
  int col_fastest;  // tile order: 1 = column-block fastest (write-bound shapes), 0 = grouped row-block fastest
  int split_slabs;  // 0, or K slabs per plane of fp32 operands split into three bf16 planes (see gemm_f32_split_dispatch)
  const uint32_t* skip_if_set;  // when not NULL: the kernel returns at once if this device word is non-zero
  uint64_t wait_limit_ns;       // every mbarrier wait gives up after this long (kWaitLimitNs in ordinary calls)
  int withhold_first_slab;      // wait probe only: the producer never loads the first K slab of a CTA's first tile
  int group_m;                  // row-blocks per rasterisation group (see tile_coords)
};

// Tile t of one batch entry -> (row-block, column-block): column-block fastest, or groups of
// kGroupM row-blocks with the row-block fastest inside a group.
__device__ __forceinline__ void tile_coords(int64_t rem, int64_t mt, int64_t nt, int& mb, int& nb, int col_fastest, int group_m = kGroupM) {
  if (col_fastest) {
    mb = static_cast<int>(rem / nt);
    nb = static_cast<int>(rem - static_cast<int64_t>(mb) * nt);
    return;
  }
  const int64_t per_group = static_cast<int64_t>(group_m) * nt;
  const int64_t g = rem / per_group, in_g = rem - g * per_group;
  const int64_t gm = (mt - g * group_m) < group_m ? (mt - g * group_m) : group_m;  // the last group may be short
  mb = static_cast<int>(g * group_m + in_g % gm);
  nb = static_cast<int>(in_g / gm);
}

// T: operand type in shared memory (bf16 / f16). TO: type of C and of the bias -- T itself,
// or float when the operands are the bf16 planes of split fp32 matrices.
template <typename T, int kBN, typename TO, bool kPair = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c, const TO* __restrict__ bias, TO* __restrict__ C, GemmTcParams p,
                    uint32_t* __restrict__ status) {
  using Cfg = TileCfg<kBN, kPair>;
  constexpr int kStages = Cfg::kStages, kStageBytes = Cfg::kStageBytes, kAccs = Cfg::kAccs, kBRows = Cfg::kBRows;
  constexpr int kTileM = kPair ? 2 * kBM : kBM;  // rows of C one tile covers (both CTAs of a pair)
  static_assert(!kPair || kBN == 256, "CTA pairs work on 256 x 256 tiles");
  if (p.skip_if_set && *p.skip_if_set != 0u) return;  // every thread of every CTA reads the same word: a uniform exit before any barrier or TMEM set-up
  extern __shared__ unsigned char smem_raw[];
  // 1024-byte alignment: the 128B swizzle pattern repeats every 8 rows x 128 bytes
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  unsigned char* epi_stage = smem + kStages * kStageBytes;  // kEpiWarps x 4 KB, each 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes + kEpiWarps * kEpiStageBytes);
  // barrier slots: [0,S) full, [S,2S) empty, [2S,2S+2) tmem_full, [2S+2,2S+4) tmem_empty
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 2 * kAccs);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + kAccs + a); };

  // pair: rank of this CTA in its 2-CTA cluster (0 = the CTA that issues the MMAs), and the
  // shared::cluster addresses of the even CTA's barriers that both CTAs signal
  const uint32_t cta_rank = kPair ? cluster_ctarank() : 0u;
  if (threadIdx.x == 64) {
    // the copy engine's descriptors are on their way while the barriers and the tensor memory are set up
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
    if (p.tma_store) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_c)) : "memory");
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);   // pair: only the even CTA's is used (its producer arms it for both CTAs' bytes)
      mbar_init(empty_bar(s), 1);  // one tcgen05.commit per use (pair: the even CTA commits to both CTAs')
    }
    for (int a = 0; a < kAccs; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), kPair ? 16 : 8);  // one arrival per epilogue warp (pair: of both CTAs, on the even CTA's)
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if (kPair) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)), "r"(kTmemCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)), "r"(kTmemCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (kPair) cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  const int64_t mt = (p.M + kTileM - 1) / kTileM, nt = (p.N + kBN - 1) / kBN;
  const int64_t tiles = p.batch * mt * nt;
  const int64_t tile_first = kPair ? (blockIdx.x >> 1) : blockIdx.x, tile_step = kPair ? (gridDim.x >> 1) : gridDim.x;
  // Split operands: plane q of an operand occupies K coordinates [q * Kp, q * Kp + K) of its
  // tensor map, Kp = 64 * split_slabs. One slab of the product needs the six plane pairs
  // whose product is not below fp32 resolution: (0,0) (0,1) (1,0) (0,2) (1,1) (2,0).
  // They are walked pair by pair over all slabs (see the producer).
  const int num_kb = p.split_slabs ? 6 * p.split_slabs : static_cast<int>((p.K + kBK - 1) / kBK);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t t = tile_first; t < tiles && ok; t += tile_step) {
        const int64_t b = t / (mt * nt), rem = t - b * (mt * nt);
        int mb, nb;
        tile_coords(rem, mt, nt, mb, nb, p.col_fastest, p.group_m);
        // pair: this CTA's 128 rows of A and its half of the B slab's 256 rows
        const int m0 = mb * kTileM + static_cast<int>(cta_rank) * kBM, n0 = nb * kBN + static_cast<int>(cta_rank) * (kPair ? kBRows : 0);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.wait_limit_ns)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * kStageBytes, b_dst = a_dst + kABytes;
          if (!kPair && p.withhold_first_slab && t == blockIdx.x && kb == 0) {
            // wait probe: this stage is never armed and never filled, so the MMA warp's wait on
            // it must run into its limit; the producer carries on until it needs the stage back
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
            continue;
          }
          // pair: every copy of both CTAs completes on the even CTA's barrier, which its
          // producer arms for the bytes of both
          const uint32_t fbar = kPair ? map_to_cta(full_bar(stage), 0u) : full_bar(stage);
          if (!kPair) mbar_expect_tx(full_bar(stage), kStageBytes);
          else if (cta_rank == 0u) mbar_expect_tx(full_bar(stage), 2 * kStageBytes);
          auto load = [&](uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2) {
            if (kPair) tma_load_3d_pair(dst, map, fbar, c0, c1, c2);
            else tma_load_3d(dst, map, fbar, c0, c1, c2);
          };
          int ka = kb * kBK, kbb = kb * kBK;
          if (p.split_slabs) {
            // pairs (2,0) (1,1) (0,2) (1,0) (0,1) over all slabs first, then (0,0): the tensor
            // core truncates when it adds into the accumulator, by half a unit in the last
            // place of the running sum on average, so the small products go in while the sum
            // is still small and only the K/16 steps of the leading product pay full price
            const int pair = kb / p.split_slabs, slab = kb - pair * p.split_slabs;
            ka = (((0x001012 >> (4 * pair)) & 0xf) * p.split_slabs + slab) * kBK;
            kbb = (((0x010210 >> (4 * pair)) & 0xf) * p.split_slabs + slab) * kBK;
          }
          if (!p.a_mn_major) {
            load(a_dst, &map_a, ka, m0, static_cast<int>(b));  // box [128 rows][64 k]
          } else {
#pragma unroll
            for (int c = 0; c < kBM / 64; ++c) load(a_dst + c * 8192, &map_a, m0 + c * 64, ka, static_cast<int>(b));  // box [64 k][64 m]
          }
          if (!p.b_mn_major) {
            load(b_dst, &map_b, kbb, n0, static_cast<int>(b));  // box [kBRows rows][64 k]
          } else {
#pragma unroll
            for (int c = 0; c < kBRows / 64; ++c) load(b_dst + c * 8192, &map_b, n0 + c * 64, kbb, static_cast<int>(b));  // box [64 k][64 n]
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (kPair && ok) {
        // tail: the even CTA's commits arrive on THIS CTA's empty barriers from afar; wait for
        // the ones still outstanding so that none lands after this CTA's shared memory is gone
        for (int i = 0; i < kStages && ok; ++i) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.wait_limit_ns)) ok = false;
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        if (status) atomicOr(status, B200_DEV_WAIT_TIMEOUT);
      }
    }
    __syncwarp();  // lanes 1..31 rejoin lane 0 before the CTA-wide barrier below
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0u) {  // pair: the even CTA issues for both
      // instruction descriptor: fp32 accumulate, A/B format, majors, N >> 3, M >> 4
      const uint32_t fmt = p.is_bf16 ? 1u : 0u;
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(p.a_mn_major) << 15) | (static_cast<uint32_t>(p.b_mn_major) << 16) |
                             (static_cast<uint32_t>(kBN >> 3) << 17) | (static_cast<uint32_t>(kTileM >> 4) << 24);
      // per-UMMA (K = 16) advance of the start address and the two byte offsets per layout
      const uint32_t a_adv = p.a_mn_major ? 2048u : 32u, b_adv = p.b_mn_major ? 2048u : 32u;
      const uint32_t a_lbo = p.a_mn_major ? 8192u : 16u, b_lbo = p.b_mn_major ? 8192u : 16u;
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int64_t t = tile_first; t < tiles && ok; t += tile_step) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.wait_limit_ns)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kBN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.wait_limit_ns)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * kStageBytes, b_addr = a_addr + kABytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t da = smem_desc(a_addr + k * a_adv, a_lbo, 1024u);
            const uint64_t db = smem_desc(b_addr + k * b_adv, b_lbo, 1024u);
            if (kPair) tc_mma_f16_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
            else tc_mma_f16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // the stage is free once these MMAs have read it (pair: in both CTAs)
          if (kPair) {
            tc_commit_pair(map_to_cta(empty_bar(stage), 0u));
            tc_commit_pair(map_to_cta(empty_bar(stage), 1u));
          } else {
            tc_commit(empty_bar(stage));
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        // accumulator complete (pair: each CTA's epilogue waits on its own barrier)
        if (kPair) {
          tc_commit_pair(map_to_cta(tfull_bar(acc), 0u));
          tc_commit_pair(map_to_cta(tfull_bar(acc), 1u));
        } else {
          tc_commit(tfull_bar(acc));
        }
        if (++acc == kAccs) { acc = 0; acc_phase ^= 1u; }
      }
      if (!ok) {
        *abort_flag = 1;
        if (status) atomicOr(status, B200_DEV_WAIT_TIMEOUT);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    const int q = warp & 3;             // TMEM lane quarter this warp may read: lanes [32q, 32q + 32)
    const int chalf = (warp - 2) >> 2;  // which 128 of the 256 columns
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    constexpr int kOutVec = 16 / static_cast<int>(sizeof(TO));  // outputs per 16-byte store
    const bool vec_ok = (p.N % kOutVec == 0) && ((reinterpret_cast<uintptr_t>(C) & 15u) == 0);
    const uint32_t tempty_target = kPair ? map_to_cta(tempty_bar(0), 0u) : 0u;  // the even CTA's tmem_empty[0]
    for (int64_t t = tile_first; t < tiles && ok; t += tile_step) {
      const int64_t b = t / (mt * nt), rem = t - b * (mt * nt);
      int mb, nb_blk;
      tile_coords(rem, mt, nt, mb, nb_blk, p.col_fastest, p.group_m);
      const int64_t m0 = static_cast<int64_t>(mb) * kTileM + static_cast<int64_t>(cta_rank) * kBM, n0 = static_cast<int64_t>(nb_blk) * kBN + chalf * (kBN / 2);
      int got = 0;
      if (lane == 0) got = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.wait_limit_ns) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) { ok = false; break; }
      tc_fence_after();
      const int64_t m = m0 + q * 32 + lane;
      const uint32_t t_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * kBN + chalf * (kBN / 2));
      // the 64-column chunks of this warp's half are double-buffered in registers: the
      // tensor-memory load of the next chunk is in flight while this one is converted and stored
      constexpr int kChunks = kBN / 2 / 64;
      uint32_t r[kChunks > 1 ? 2 : 1][64];
      tc_ld_32x32(t_base, r[0]);
      tc_ld_32x32(t_base + 32, r[0] + 32);
      const bool plain = p.alpha == 1.f && !p.has_bias;  // C = A x B: nothing to do but round
      const bool unit_scales = p.alpha == 1.f && p.beta == 1.f;
      const bool bias_vec = sizeof(TO) == sizeof(T) && p.has_bias && p.sbn == 1 && p.sbm % 8 == 0 && (reinterpret_cast<uintptr_t>(bias) & 15u) == 0;
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        tc_ld_wait();
        if (c + 1 < kChunks) {
          tc_ld_32x32(t_base + (c + 1) * 64, r[(c + 1) & 1]);
          tc_ld_32x32(t_base + (c + 1) * 64 + 32, r[(c + 1) & 1] + 32);
        } else {
          // every value of the accumulator is in registers: hand it back to the MMA warp now
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (kPair) mbar_arrive_cluster(tempty_target + 8u * acc);
            else mbar_arrive(tempty_bar(acc));
          }
        }
        const uint32_t* rc = r[c & 1];
        const int64_t nb = n0 + c * 64;
        if (p.tma_store) {
          // scale / bias in fp32, round once, park the lane's 64 outputs of its row in this
          // warp's 32 x 128-byte buffer in the 128-byte-swizzle layout (16-byte chunk index
          // XOR row) -- conflict-free to write and exactly what a SWIZZLE_128B tiled store
          // reads -- then one lane hands the 32 x 64 tile to the copy engine, which writes
          // whole lines and clips at the edges of C.
          unsigned char* mine = epi_stage + (warp - 2) * kEpiStageBytes;
          if (lane == 0) tma_store_wait_read();  // the previous tile store has finished reading the buffer
          __syncwarp();
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const int64_t n = nb + g * 8;
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(rc[g * 8 + e]);
            if (!plain) {
              if (bias_vec && m < p.M && n + 8 <= p.N) {
                // unit-stride bias (a row vector, or a matrix like C): eight values in one load
                float bv[8];
                widen<T>(ld_keep(bias + m * p.sbm + n), bv);  // TO is T on this path
                if (unit_scales) {  // addmm as models call it: one add per value
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[e] += bv[e];
                } else {
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[e] = fmaf(p.beta, bv[e], p.alpha * v[e]);
                }
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  v[e] *= p.alpha;
                  if (p.has_bias && m < p.M && n + e < p.N) v[e] = fmaf(p.beta, to_f32(bias[m * p.sbm + (n + e) * p.sbn]), v[e]);
                }
              }
            }
            *reinterpret_cast<uint4*>(mine + lane * 128 + ((g ^ (lane & 7)) << 4)) = narrow<T>(v);
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0 && nb < p.N && m0 + q * 32 < p.M) {
            tma_store_3d(&map_c, smem_u32(mine), static_cast<int>(nb), static_cast<int>(m0 + q * 32), static_cast<int>(b));
            tma_store_commit();
          }
        } else if (sizeof(TO) == 2) {
          // 16-bit C whose rows are off the 16-byte grid (N not a multiple of 8): a lane owns a
          // row, so storing from registers would put every lane of a store in another row, one
          // 32-byte sector per 2-byte element. Park the chunk in the warp's buffer as above and
          // write it out row by row, 64 contiguous bytes per store.
          unsigned char* mine = epi_stage + (warp - 2) * kEpiStageBytes;
          __syncwarp();  // the previous chunk has been read out of the buffer
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const int64_t n = nb + g * 8;
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              v[e] = p.alpha * __uint_as_float(rc[g * 8 + e]);
              if (p.has_bias && m < p.M && n + e < p.N) v[e] = fmaf(p.beta, to_f32(bias[m * p.sbm + (n + e) * p.sbn]), v[e]);
            }
            *reinterpret_cast<uint4*>(mine + lane * 128 + ((g ^ (lane & 7)) << 4)) = narrow<T>(v);
          }
          __syncwarp();
          const int64_t left = p.N - nb;
          const int ncols = left < 64 ? static_cast<int>(left) : 64;  // <= 0: the chunk lies right of C
          for (int rr = 0; rr < 32; ++rr) {
            const int64_t mr = m0 + q * 32 + rr;
            if (mr >= p.M) break;
            TO* crow = C + (b * p.M + mr) * p.N + nb;
            for (int cc = lane; cc < ncols; cc += 32)
              crow[cc] = *reinterpret_cast<const TO*>(mine + rr * 128 + (((cc >> 3) ^ (rr & 7)) << 4) + (cc & 7) * 2);
          }
        } else if (m < p.M && nb < p.N) {
          TO* crow = C + (b * p.M + m) * p.N;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const int64_t n = nb + g * 8;
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              v[e] = p.alpha * __uint_as_float(rc[g * 8 + e]);
              if (p.has_bias && n + e < p.N) v[e] = fmaf(p.beta, to_f32(bias[m * p.sbm + (n + e) * p.sbn]), v[e]);
            }
            if (vec_ok && n + 8 <= p.N) {
#pragma unroll
              for (int h = 0; h < 8 / kOutVec; ++h) *reinterpret_cast<uint4*>(crow + n + h * kOutVec) = narrow<TO>(v + h * kOutVec);
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e)
                if (n + e < p.N) crow[n + e] = from_f32<TO>(v[e]);
            }
          }
        }
      }
      if (++acc == kAccs) { acc = 0; acc_phase ^= 1u; }
    }
    if (lane == 0) tma_store_wait_read();  // the tile stores have read their shared memory: the CTA may exit (the writes complete on their own)
    if (!ok && lane == 0) {
      *abort_flag = 1;
      if (status) atomicOr(status, B200_DEV_WAIT_TIMEOUT);
    }
    __syncwarp();
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*abort_flag) {
    // give copies that are still in flight time to land before the shared memory goes away
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (kPair) cluster_sync_all();  // neither CTA leaves while the other may still signal its barriers or read its operands
  if (warp == 1) {
    if (kPair) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------ host side
struct OperandLayout {
  bool ok, mn_major;
};
// An operand [rows(MN), K] with element strides (s_mn, s_k) is TMA-loadable when one of
// the two strides is 1 and the other (and the batch stride) keeps 16-byte alignment.
static OperandLayout operand_layout(int64_t mn, int64_t k, int64_t s_mn, int64_t s_k, int64_t s_b, int64_t batch, const void* base) {
  OperandLayout r{false, false};
  if (!aligned16(base)) return r;
  if (batch > 1 && (s_b % 8 != 0 || s_b <= 0)) return r;
  if (s_k == 1 && (s_mn % 8 == 0) && s_mn >= k) { r.ok = true; r.mn_major = false; return r; }
  if (s_mn == 1 && (s_k % 8 == 0) && s_k >= mn) { r.ok = true; r.mn_major = true; return r; }
  // a single row / column is contiguous either way
  if (mn == 1 && s_k == 1) { r.ok = true; r.mn_major = false; return r; }
  return r;
}

int gemm_simt_dispatch(const void* A, const void* B, const void* bias, void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk,
                       int64_t sBb, int64_t sBk, int64_t sBn, int64_t sbm, int64_t sbn, double alpha, double beta, int dtype, cudaStream_t st, const uint32_t* gate);

bool gemm_tc_eligible(int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk, int64_t sBb, int64_t sBk, int64_t sBn, int dtype, const void* A,
                      const void* B, const void* C) {
  if (dtype != B200_BF16 && dtype != B200_F16) return false;
  if (batch < 1 || M < 1 || N < 1 || K < 1) return false;
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL || batch > 0x7fffffffLL) return false;
  // tiny problems are launch-bound either way; the CUDA-core kernel has no TMEM / barrier set-up
  if (M * N * K < (1LL << 15)) return false;
  if (!operand_layout(M, K, sAm, sAk, sAb, batch, A).ok) return false;
  if (!operand_layout(N, K, sBn, sBk, sBb, batch, B).ok) return false;
  if (!C) return false;
  return encode_fn() != nullptr;
}

static bool encode_operand(CUtensorMap* map, const void* base, int dtype, bool mn_major, int64_t mn, int64_t k, int64_t s_mn, int64_t s_k, int64_t s_b, int64_t batch, int tile_mn) {
  const cuuint64_t inner = mn_major ? mn : k, outer = mn_major ? k : mn;
  int64_t outer_stride = mn_major ? s_k : s_mn;  // elements
  if (outer == 1 && outer_stride % 8 != 0) outer_stride = (static_cast<int64_t>(inner) + 7) / 8 * 8;  // never dereferenced beyond row 0
  int64_t batch_stride = batch > 1 ? s_b : outer_stride * static_cast<int64_t>(outer);
  if (batch_stride % 8 != 0 || batch_stride <= 0) batch_stride = (batch_stride / 8 + 1) * 8;
  cuuint64_t dims[3] = {inner, outer, static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(outer_stride) * 2, static_cast<cuuint64_t>(batch_stride) * 2};
  cuuint32_t box[3] = {64, static_cast<cuuint32_t>(mn_major ? kBK : tile_mn), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = dtype == B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = encode_fn()(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Rows of C per rasterisation group: the CTAs that run together walk the column blocks of one
// group of row blocks, so the group's A panel (rows x K 16-bit values) stays in L2 while B
// streams past it once per group. The panel is sized to a fraction of the 126 MB L2; fewer
// groups mean fewer passes over B (at 8192 x 4096 x 11008 groups of 2048 rows read B four
// times: 441 MB of DRAM reads for 157 MB of operands).
#ifndef B200_GEMM_PANEL_MB
#define B200_GEMM_PANEL_MB 32
#endif
static int group_rows_for(int64_t k_elems) {
  int64_t rows = (static_cast<int64_t>(B200_GEMM_PANEL_MB) << 20) / (2 * (k_elems > 0 ? k_elems : 1));
  rows = rows / 256 * 256;
  if (rows < 2048) rows = 2048;    // never smaller than the groups the kernel always used
  if (rows > 65536) rows = 65536;
  return static_cast<int>(rows);
}

// One launch of the kernel: a plain grid, or 2-CTA clusters for the pair variant.
template <typename Kernel, typename TB, typename TC>
static int launch_tc(Kernel kernel, bool pair, int grid, cudaStream_t st, const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_c, const TB* bias_t, TC* c_t,
                     const GemmTcParams& p, uint32_t* status) {
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kGemmSmem));
  if (e != cudaSuccess) { set_last_cuda_error(e); return B200_ELAUNCH; }
  if (!pair) {
    kernel<<<grid, kGemmThreads, kGemmSmem, st>>>(map_a, map_b, map_c, bias_t, c_t, p, status);
    return B200_OK;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = kGemmSmem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t le = cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, map_c, bias_t, c_t, p, status);
  if (le != cudaSuccess) { set_last_cuda_error(le); return B200_ELAUNCH; }
  return B200_OK;
}

// CTA pairs can be switched off with B200_GEMM_PAIR=0 in the environment (read once): the
// single-CTA kernel then serves every shape, which is how the two are compared.
static bool pair_launch_ok() {
  static const bool on = []() {
    const char* e = getenv("B200_GEMM_PAIR");
    return !(e && e[0] == '0');
  }();
  return on;
}

int gemm_tc_dispatch(const void* A, const void* B, const void* bias, void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk, int64_t sBb,
                     int64_t sBk, int64_t sBn, int64_t sbm, int64_t sbn, double alpha, double beta, int dtype, uint32_t* status, cudaStream_t st, uint64_t wait_probe_limit_ns,
                     bool allow_pair) {
  const OperandLayout la = operand_layout(M, K, sAm, sAk, sAb, batch, A);
  const OperandLayout lb = operand_layout(N, K, sBn, sBk, sBb, batch, B);
  if (!la.ok || !lb.ok || !encode_fn()) return B200_EALIGN;
  alignas(64) CUtensorMap map_a, map_b;
  if (!encode_operand(&map_a, A, dtype, la.mn_major, M, K, sAm, sAk, sAb, batch, kBM)) return B200_EDRIVER;
  // CTA pairs on 256 x 256 tiles whenever C has more than one 128-row block and is not narrow;
  // the wait probe stays on the single-CTA kernel
  // (with four K slabs or fewer the kernel is bound by writing C and the pair is slower:
  // bmm 32 x 2048 x 128 x 2048 0.087 ms against 0.061 ms)
  const bool pair = allow_pair && M > kBM && N > 128 && (K + kBK - 1) / kBK > 4 && wait_probe_limit_ns == 0 && pair_launch_ok();
  const int bn_box = (N <= 128 || pair) ? 128 : 256;  // rows of the B box: must match the tile shape chosen below
  if (!encode_operand(&map_b, B, dtype, lb.mn_major, N, K, sBn, sBk, sBb, batch, bn_box)) return B200_EDRIVER;
  alignas(64) CUtensorMap map_c;
  const bool tma_store = (N % 8 == 0) && aligned16(C);
  if (tma_store) {
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(M), static_cast<cuuint64_t>(batch)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(N) * 2, static_cast<cuuint64_t>(M) * static_cast<cuuint64_t>(N) * 2};
    cuuint32_t box[3] = {64, 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapDataType dt = dtype == B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (encode_fn()(&map_c, dt, 3, C, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return B200_EDRIVER;
  } else {
    map_c = map_a;  // unused by the kernel in this mode
  }
  GemmTcParams p;
  p.tma_store = tma_store ? 1 : 0;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.sbm = sbm; p.sbn = sbn;
  p.alpha = static_cast<float>(alpha);
  p.beta = static_cast<float>(beta);
  p.a_mn_major = la.mn_major ? 1 : 0;
  p.b_mn_major = lb.mn_major ? 1 : 0;
  p.is_bf16 = dtype == B200_BF16 ? 1 : 0;
  p.has_bias = (bias != nullptr && p.beta != 0.f) ? 1 : 0;
  // few K slabs per tile: the kernel is bound by writing C, so CTAs that run together should
  // write neighbouring column blocks of the same rows (whole DRAM pages); otherwise order
  // tiles for operand reuse in L2
  p.col_fastest = (K + kBK - 1) / kBK <= 4 ? 1 : 0;
  p.split_slabs = 0;
  p.skip_if_set = nullptr;
  p.wait_limit_ns = wait_probe_limit_ns ? wait_probe_limit_ns : kWaitLimitNs;
  p.withhold_first_slab = wait_probe_limit_ns ? 1 : 0;
  p.group_m = group_rows_for(K) / (pair ? 2 * kBM : kBM);
  // a narrow C takes the 128-wide tile. (Write-bound shapes with few K slabs were measured
  // slower on it: 256-byte row segments instead of 512-byte ones cost more in DRAM than the
  // deeper pipeline gains -- bmm 32x2048x128x2048: 0.162 ms vs 0.116 ms.)
  const bool narrow = N <= 128;
  const int bn = narrow ? 128 : 256;
  const int tile_m = pair ? 2 * kBM : kBM;
  const int64_t tiles = batch * ((M + tile_m - 1) / tile_m) * ((N + bn - 1) / bn);
  const int64_t slots = pair ? kNumSMs / 2 : kNumSMs;  // persistent: one CTA (or CTA pair) per SM (or TPC)
  const int grid = static_cast<int>(tiles < slots ? tiles : slots) * (pair ? 2 : 1);
  auto launch = [&](auto kernel, auto* bias_t, auto* c_t) -> int { return launch_tc(kernel, pair, grid, st, map_a, map_b, map_c, bias_t, c_t, p, status); };
  int rc;
  if (dtype == B200_BF16) {
    const __nv_bfloat16* bt = static_cast<const __nv_bfloat16*>(bias);
    __nv_bfloat16* ct = static_cast<__nv_bfloat16*>(C);
    rc = pair ? launch(gemm_tcgen05_kernel<__nv_bfloat16, 256, __nv_bfloat16, true>, bt, ct)
              : narrow ? launch(gemm_tcgen05_kernel<__nv_bfloat16, 128, __nv_bfloat16>, bt, ct) : launch(gemm_tcgen05_kernel<__nv_bfloat16, 256, __nv_bfloat16>, bt, ct);
  } else {
    const __half* bt = static_cast<const __half*>(bias);
    __half* ct = static_cast<__half*>(C);
    rc = pair ? launch(gemm_tcgen05_kernel<__half, 256, __half, true>, bt, ct)
              : narrow ? launch(gemm_tcgen05_kernel<__half, 128, __half>, bt, ct) : launch(gemm_tcgen05_kernel<__half, 256, __half>, bt, ct);
  }
  if (rc == B200_ELAUNCH && pair) {
    // the cluster launch was refused (a device or a partition without thread-block clusters):
    // the same product on single CTAs
    (void)cudaGetLastError();
    return gemm_tc_dispatch(A, B, bias, C, batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, sbm, sbn, alpha, beta, dtype, status, st, wait_probe_limit_ns, false);
  }
  if (rc) return rc;
  return check_launch();
}

// ------------------------------------------------------------------ long contraction, few output tiles
// A 16-bit product whose C is a handful of tiles leaves most SMs idle while one CTA per tile
// walks all of K (5 x 4096 x 512: two CTAs, 64 K slabs each, 26 us). Here the contraction is
// cut into S equal ranges that the kernel above sees as S batch entries -- A as [S][M][K/S],
// B as [S][K/S][N], both only a different tensor map over the same memory -- and writes as
// fp32 partial products [S][M][N] into caller scratch; a second kernel adds the S partials of
// every element in the order 0 .. S-1, applies alpha, beta and the bias and rounds once. No
// atomics: the result does not depend on scheduling.
struct SplitKPlan {
  int splits;      // 1 = not worth it / not possible
  int64_t kchunk;  // K / splits
};
static SplitKPlan plan_splitk(int64_t batch, int64_t M, int64_t N, int64_t K) {
  SplitKPlan r{1, K};
  if (batch != 1) return r;
  const int bn = N <= 128 ? 128 : 256;
  const int64_t tiles = ((M + kBM - 1) / kBM) * ((N + bn - 1) / bn), slabs = (K + kBK - 1) / kBK;
  // (more tiles than a quarter of the SMs: 5722 x 4096 x 256, 45 tiles, ran 30 us in two ranges against 26 us whole)
  if (tiles > kNumSMs / 4 || slabs < 24) return r;  // (16 slabs: 104 x 1024 x 1024 took 12 us either way)
  int64_t s = kNumSMs / tiles;
  if (s > slabs / 4) s = slabs / 4;  // every range keeps at least four K slabs
  if (s > 32) s = 32;
  for (; s >= 2; --s)
    if (K % (8 * s) == 0) break;     // ranges start on the 16-byte grid of a K-major operand
  if (s < 2) return r;
  r.splits = static_cast<int>(s);
  r.kchunk = K / s;
  return r;
}

int64_t gemm_tc_splitk_scratch_bytes(int64_t batch, int64_t M, int64_t N, int64_t K) {
  const SplitKPlan pl = plan_splitk(batch, M, N, K);
  return pl.splits < 2 ? 0 : static_cast<int64_t>(pl.splits) * M * N * 4 + 256;
}

template <typename T>
__global__ void __launch_bounds__(256) splitk_reduce(const float* __restrict__ part, int splits, int64_t M, int64_t N, const T* __restrict__ bias, int64_t sbm, int64_t sbn, float alpha, float beta,
                                                     T* __restrict__ C) {
  const int64_t total = M * N;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float sum = 0.f;
    for (int s = 0; s < splits; ++s) sum += part[s * total + i];
    float r = alpha * sum;
    if (bias && beta != 0.f) {
      const int64_t m = i / N, n = i - m * N;
      r = fmaf(beta, to_f32(bias[m * sbm + n * sbn]), r);
    }
    C[i] = from_f32<T>(r);
  }
}

int gemm_tc_splitk_dispatch(const void* A, const void* B, const void* bias, void* C, int64_t M, int64_t N, int64_t K, int64_t sAm, int64_t sAk, int64_t sBk, int64_t sBn, int64_t sbm,
                            int64_t sbn, double alpha, double beta, int dtype, void* scratch, int64_t scratch_bytes, uint32_t* status, cudaStream_t st) {
  const SplitKPlan pl = plan_splitk(1, M, N, K);
  if (pl.splits < 2) return B200_EINVAL;
  if (!scratch || scratch_bytes < gemm_tc_splitk_scratch_bytes(1, M, N, K)) return B200_ESCRATCH;
  float* part = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(scratch) + 255) & ~static_cast<uintptr_t>(255));
  const int64_t S = pl.splits, Kc = pl.kchunk;
  const int64_t sAb = Kc * sAk, sBb = Kc * sBk;  // range s of the contraction starts s * Kc further along K
  const OperandLayout la = operand_layout(M, Kc, sAm, sAk, sAb, S, A);
  const OperandLayout lb = operand_layout(N, Kc, sBn, sBk, sBb, S, B);
  if (!la.ok || !lb.ok || !encode_fn()) return B200_EALIGN;
  const int bn = N <= 128 ? 128 : 256;
  alignas(64) CUtensorMap map_a, map_b;
  if (!encode_operand(&map_a, A, dtype, la.mn_major, M, Kc, sAm, sAk, sAb, S, kBM)) return B200_EDRIVER;
  if (!encode_operand(&map_b, B, dtype, lb.mn_major, N, Kc, sBn, sBk, sBb, S, bn)) return B200_EDRIVER;
  GemmTcParams p;
  p.tma_store = 0;
  p.M = M; p.N = N; p.K = Kc; p.batch = S;
  p.sbm = 0; p.sbn = 0;
  p.alpha = 1.f;
  p.beta = 0.f;
  p.a_mn_major = la.mn_major ? 1 : 0;
  p.b_mn_major = lb.mn_major ? 1 : 0;
  p.is_bf16 = dtype == B200_BF16 ? 1 : 0;
  p.has_bias = 0;
  p.col_fastest = 1;
  p.split_slabs = 0;
  p.skip_if_set = nullptr;
  p.wait_limit_ns = kWaitLimitNs;
  p.withhold_first_slab = 0;
  p.group_m = group_rows_for(Kc) / kBM;
  const int64_t tiles = S * ((M + kBM - 1) / kBM) * ((N + bn - 1) / bn);
  const int grid = static_cast<int>(tiles < kNumSMs ? tiles : kNumSMs);
  auto launch = [&](auto kernel) -> int { return launch_tc(kernel, false, grid, st, map_a, map_b, map_a, static_cast<const float*>(nullptr), part, p, status); };
  int rc;
  if (dtype == B200_BF16) rc = bn == 128 ? launch(gemm_tcgen05_kernel<__nv_bfloat16, 128, float>) : launch(gemm_tcgen05_kernel<__nv_bfloat16, 256, float>);
  else rc = bn == 128 ? launch(gemm_tcgen05_kernel<__half, 128, float>) : launch(gemm_tcgen05_kernel<__half, 256, float>);
  if (rc) return rc;
  int64_t blocks = (M * N + 255) / 256;
  if (blocks > kNumSMs * 8) blocks = kNumSMs * 8;
  const float al = static_cast<float>(alpha), be = static_cast<float>(beta);
  if (dtype == B200_BF16)
    splitk_reduce<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, st>>>(part, static_cast<int>(S), M, N, static_cast<const __nv_bfloat16*>(bias), sbm, sbn, al, be, static_cast<__nv_bfloat16*>(C));
  else
    splitk_reduce<__half><<<static_cast<int>(blocks), 256, 0, st>>>(part, static_cast<int>(S), M, N, static_cast<const __half*>(bias), sbm, sbn, al, be, static_cast<__half*>(C));
  return check_launch(2);
}

// ------------------------------------------------------------------ fp32 operands on the tensor cores
// An fp32 value is the sum of three bf16 values to within 2^-25 of itself (x1 = bf16(x),
// x2 = bf16(x - x1), x3 = bf16(x - x1 - x2); the subtractions are exact). A product of fp32
// matrices is therefore, to fp32 accuracy, the sum of the six bf16 products
// A1B1 + A1B2 + A2B1 + A1B3 + A2B2 + A3B1 (the three left out are below 2^-25 relative) --
// every one exact in the tensor core's fp32 accumulator. The kernel above runs them as one
// contraction of depth 6 K: the operands are split once into planes laid side by side along
// K, and the producer warp walks the six plane pairs of every K slab.
//
// split_f32_planes: x [batch, mn, k] (any strides) -> bf16 planes. K-major form (src K
// stride 1, or neither stride 1): out[b][mn][q * Kp + k]; MN-major form (src MN stride 1):
// out[b][q * Kp + k][mn]. Kp = K rounded up to 64; the pad [K, Kp) is written as zero.
// Infinities and NaN stay in plane 0 alone (x - x1 would be NaN); a value whose bf16
// rounding overflows is truncated instead. An infinity still meets the residual planes of
// the other operand, whose signs are arbitrary (inf - inf = NaN where fp32 arithmetic gives
// inf), so the split raises a device flag when it meets a non-finite value: the tensor-core
// kernel returns at once when the flag is up and the CUDA-core kernel, launched behind it
// and gated the other way, computes that product in plain fp32.
struct SplitArgs {
  int64_t batch, mn, k, kp;
  int64_t s_b, s_mn, s_k;        // source strides, elements
  int64_t o_b, o_row;            // output batch stride and row pitch, elements
  int mn_major;                  // output form
  uint32_t* any_flag;            // set when the operand holds an infinity or a NaN
};
__device__ __forceinline__ void split3(float x, __nv_bfloat16& a, __nv_bfloat16& b, __nv_bfloat16& c) {
  if (!isfinite(x)) { a = __float2bfloat16_rn(x); b = c = __float2bfloat16_rn(0.f); return; }
  float x1 = __bfloat162float(__float2bfloat16_rn(x));
  if (!isfinite(x1)) x1 = __uint_as_float(__float_as_uint(x) & 0xffff0000u);
  const float r1 = x - x1;
  const float x2 = __bfloat162float(__float2bfloat16_rn(r1));
  const float r2 = r1 - x2;
  a = __float2bfloat16_rn(x1);
  b = __float2bfloat16_rn(x2);
  c = __float2bfloat16_rn(r2);
}
__global__ void __launch_bounds__(256) split_f32_planes(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, SplitArgs A) {
  // A thread produces 8 consecutive elements along the contiguous dimension of the output
  // (k in the K-major form, mn in the MN-major form): two 16-byte loads when the source is
  // contiguous and aligned there, three 16-byte stores.
  const int64_t inner = A.mn_major ? A.mn : A.kp, outer = A.mn_major ? A.kp : A.mn;
  const int64_t groups = (inner + 7) / 8;  // kp is a multiple of 8; a ragged mn tail is a partial group
  const int64_t per_batch = groups * outer;
  const int64_t total = A.batch * per_batch;
  const int64_t s_in = A.mn_major ? A.s_mn : A.s_k, s_out = A.mn_major ? A.s_k : A.s_mn;  // source strides along inner / outer
  const int64_t lim_in = A.mn_major ? A.mn : A.k, lim_out = A.mn_major ? A.k : A.mn;      // where real data ends
  const bool vec = s_in == 1 && s_out % 4 == 0 && A.s_b % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t b = i / per_batch, r = i - b * per_batch;
    const int64_t o = r / groups, in0 = (r - o * groups) * 8;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = 0.f;
    if (o < lim_out) {
      const float* src = x + b * A.s_b + o * s_out + in0 * s_in;
      if (vec && in0 + 8 <= lim_in) {
        const float4 lo = __ldcs(reinterpret_cast<const float4*>(src)), hi = __ldcs(reinterpret_cast<const float4*>(src) + 1);
        v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (in0 + e < lim_in) v[e] = src[e * s_in];
      }
    }
    __nv_bfloat16 q0[8], q1[8], q2[8];
    bool bad = false;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      split3(v[e], q0[e], q1[e], q2[e]);
      bad |= !isfinite(v[e]);
    }
    if (bad) *A.any_flag = 1u;
    // o_row is a multiple of 8 and so are in0 and kp: every store below is 16-byte aligned
    __nv_bfloat16* ob = out + b * A.o_b;
    if (A.mn_major) {
      *reinterpret_cast<uint4*>(ob + o * A.o_row + in0) = *reinterpret_cast<const uint4*>(q0);
      *reinterpret_cast<uint4*>(ob + (A.kp + o) * A.o_row + in0) = *reinterpret_cast<const uint4*>(q1);
      *reinterpret_cast<uint4*>(ob + (2 * A.kp + o) * A.o_row + in0) = *reinterpret_cast<const uint4*>(q2);
    } else {
      *reinterpret_cast<uint4*>(ob + o * A.o_row + in0) = *reinterpret_cast<const uint4*>(q0);
      *reinterpret_cast<uint4*>(ob + o * A.o_row + A.kp + in0) = *reinterpret_cast<const uint4*>(q1);
      *reinterpret_cast<uint4*>(ob + o * A.o_row + 2 * A.kp + in0) = *reinterpret_cast<const uint4*>(q2);
    }
  }
}

static inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

int64_t gemm_f32_split_scratch_bytes(int64_t batch, int64_t M, int64_t N, int64_t K) {
  const int64_t kp = round_up(K, kBK);
  return batch * 3 * kp * (round_up(M, 8) + round_up(N, 8)) * 2 + 256 + 512;
}

bool gemm_f32_split_eligible(int64_t batch, int64_t M, int64_t N, int64_t K) {
  if (batch < 1 || M < 1 || N < 1 || K < 1) return false;
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || 3 * round_up(K, kBK) > 0x7fffffffLL || batch > 0x7fffffffLL) return false;
  return encode_fn() != nullptr;
}

int gemm_f32_split_dispatch(const void* A, const void* B, const void* bias, void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk, int64_t sBb,
                            int64_t sBk, int64_t sBn, int64_t sbm, int64_t sbn, double alpha, double beta, void* scratch, int64_t scratch_bytes, uint32_t* status, cudaStream_t st) {
  if (!gemm_f32_split_eligible(batch, M, N, K)) return B200_EINVAL;
  if (!scratch || scratch_bytes < gemm_f32_split_scratch_bytes(batch, M, N, K)) return B200_ESCRATCH;
  const int64_t kp = round_up(K, kBK);
  // scratch: [flag word, padded to 256 bytes] [planes of A] [planes of B]
  unsigned char* flags = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(scratch) + 255) & ~static_cast<uintptr_t>(255));
  const int64_t flag_bytes = 256;
  uint32_t* any_flag = reinterpret_cast<uint32_t*>(flags);
  const cudaError_t me = cudaMemsetAsync(flags, 0, 4, st);
  if (me != cudaSuccess) { set_last_cuda_error(me); return B200_ELAUNCH; }
  auto* pa = reinterpret_cast<__nv_bfloat16*>(flags + flag_bytes);
  const bool a_mn = sAm == 1 && sAk != 1 && M > 1, b_mn = sBn == 1 && sBk != 1 && N > 1;  // keep the contiguous dimension of each source
  const int64_t a_row = a_mn ? round_up(M, 8) : 3 * kp, a_rows = a_mn ? 3 * kp : M;
  const int64_t b_row = b_mn ? round_up(N, 8) : 3 * kp, b_rows = b_mn ? 3 * kp : N;
  __nv_bfloat16* pb = pa + batch * a_rows * a_row;  // a multiple of 8 elements: stays 16-byte aligned
  const SplitArgs sa{batch, M, K, kp, sAb, sAm, sAk, a_rows * a_row, a_row, a_mn ? 1 : 0, any_flag};
  const SplitArgs sb{batch, N, K, kp, sBb, sBn, sBk, b_rows * b_row, b_row, b_mn ? 1 : 0, any_flag};
  auto blocks = [](int64_t n) { const int64_t b = (n + 255) / 256; return static_cast<int>(b < 1 ? 1 : (b > kNumSMs * 32LL ? kNumSMs * 32LL : b)); };
  split_f32_planes<<<blocks(batch * a_rows * a_row / 24), 256, 0, st>>>(static_cast<const float*>(A), pa, sa);
  split_f32_planes<<<blocks(batch * b_rows * b_row / 24), 256, 0, st>>>(static_cast<const float*>(B), pb, sb);
  const cudaError_t se = cudaGetLastError();
  if (se != cudaSuccess) { set_last_cuda_error(se); return B200_ELAUNCH; }

  // the planes as [rows, 3 Kp] (K-major) or [3 Kp, rows] (MN-major) bf16 operands
  alignas(64) CUtensorMap map_a, map_b;
  const int bn = N <= 128 ? 128 : 256;
  const bool pair = M > kBM && N > 128 && pair_launch_ok();  // the contraction is six planes deep: never write-bound
  if (!encode_operand(&map_a, pa, B200_BF16, a_mn, M, 3 * kp, a_mn ? 1 : a_row, a_mn ? a_row : 1, a_rows * a_row, batch, kBM)) return B200_EDRIVER;
  if (!encode_operand(&map_b, pb, B200_BF16, b_mn, N, 3 * kp, b_mn ? 1 : b_row, b_mn ? b_row : 1, b_rows * b_row, batch, pair ? 128 : bn)) return B200_EDRIVER;
  GemmTcParams p;
  p.tma_store = 0;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.sbm = sbm; p.sbn = sbn;
  p.alpha = static_cast<float>(alpha);
  p.beta = static_cast<float>(beta);
  p.a_mn_major = a_mn ? 1 : 0;
  p.b_mn_major = b_mn ? 1 : 0;
  p.is_bf16 = 1;
  p.has_bias = (bias != nullptr && p.beta != 0.f) ? 1 : 0;
  p.split_slabs = static_cast<int>(kp / kBK);
  p.skip_if_set = any_flag;
  p.wait_limit_ns = kWaitLimitNs;
  p.withhold_first_slab = 0;
  p.col_fastest = 6 * p.split_slabs <= 4 ? 1 : 0;
  p.group_m = group_rows_for(3 * kp) / (pair ? 2 * kBM : kBM);
  const int tile_m = pair ? 2 * kBM : kBM;
  const int64_t tiles = batch * ((M + tile_m - 1) / tile_m) * ((N + bn - 1) / bn);
  const int64_t slots = pair ? kNumSMs / 2 : kNumSMs;
  const int grid = static_cast<int>(tiles < slots ? tiles : slots) * (pair ? 2 : 1);
  auto launch = [&](auto kernel) -> int { return launch_tc(kernel, pair, grid, st, map_a, map_b, map_a, static_cast<const float*>(bias), static_cast<float*>(C), p, status); };
  const int rc = pair ? launch(gemm_tcgen05_kernel<__nv_bfloat16, 256, float, true>)
                      : bn == 128 ? launch(gemm_tcgen05_kernel<__nv_bfloat16, 128, float>) : launch(gemm_tcgen05_kernel<__nv_bfloat16, 256, float>);
  if (rc) return rc;
  // the same product on the CUDA cores, run only when the split met an infinity or a NaN
  const int rs = gemm_simt_dispatch(A, B, bias, C, batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, sbm, sbn, alpha, beta, B200_F32, st, any_flag);
  if (rs) return rs;
  return check_launch(3);
}

}  // namespace b200
