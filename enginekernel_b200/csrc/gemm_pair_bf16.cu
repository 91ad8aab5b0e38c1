// out = x . w^T for many rows (prompts) on pairs of SMs: tcgen05.mma.cta_group::2 with a
// 256 x 256 tile a pair.  x [M, K] and w [N, K] are bfloat16 and K-major.
//
// Two blocks form a cluster and share one MMA: each stages HALF of both operands (128 rows of x,
// 128 rows of w, 64 values of K a stage, by TMA with the 128-byte swizzle), the first block's
// thread issues the MMAs for both, and each block's tensor memory receives the 128 rows of the
// tile that it staged, 256 columns wide.  Against one block a tile this halves what an SM has to
// fetch per multiply-add (32 KB instead of 48 KB for 128 x 256 x 64), which is what limits a
// tcgen05 product whose operands come from L2.
//
// The kernel is persistent: the pairs that fit the GPU walk the list of tiles (groups of 8 row
// tiles, so that the pairs running together share operands in L2).  Roles in a block:
//   warps 0..7       epilogue: two threads a row (TMEM lane) of the block's half tile, one for
//                    each half of the tile's columns (warps w and w + 4 reach the same lanes)
//   warp 8, 1 thread TMA producer of this block's operand halves (ring of five or six stages); the
//                    copies of both blocks complete on the FIRST block's barrier
//   warp 9, 1 thread (first block only) MMA issuer; frees a stage in both blocks and hands a
//                    finished accumulator to both blocks' epilogues by tcgen05.commit to both
// Two accumulators of 256 columns fill the tensor memory, so the epilogue of a tile runs under the
// MMAs of the next.  Epilogues: bfloat16 result; 32-bit result ADDED to a residual stream;
// SwiGLU (the first block stages 128 gate rows and the second the matching 128 up rows, so the
// tile's columns j and 128 + j are one output's gate and up); and for the q/k/v product of an
// attention layer with heads of 128 the per-head RMSNorm of q and k, the rotation by the token's
// position and the write of k and v into the paged cache (a tile is two whole heads of 256 tokens
// and a thread holds one token's row of one of them, so norm and rotation need no exchange; same
// arithmetic as qk_norm_rope_kv_wide_kernel, on the 32-bit sums, with one rounding).  That form
// takes a few neighbouring column tiles of a row tile in a row and keeps the cosines and sines of
// its 128 tokens' positions in shared memory meanwhile (in place of the ring's sixth stage).
//
// Every barrier wait is bounded; a wait that runs out records a code in `status`, the block stops
// taking tiles, and both blocks of the pair still meet at the end before the tensor memory is
// freed.  The reference calls cuBLAS for these products (engine/ek_model.py:203-209, 298, 311).
#include "tc_common.cuh"

namespace ek {

enum { PAIR_EPI_BF16 = 0, PAIR_EPI_ADD_F32 = 1, PAIR_EPI_SWIGLU = 2, PAIR_EPI_QKV_ROPE = 3 };

constexpr int kPairRows = 128;                 // rows of x and of w that ONE block stages
constexpr int kPairTile = 256;                 // the pair's tile: 256 rows of x by 256 rows of w
// Stages of the operand ring: six of 32 KB, or five for the q/k/v form, which keeps its tokens' angles
// in shared memory beside the ring (the sixth stage is worth 1 % to the products).
__host__ __device__ constexpr int pair_stages(int epi) { return epi == 3 ? 5 : 6; }
constexpr int kPairThreads = 320;
constexpr int kPairEpilogueWarps = 8;
constexpr int kPairGroup = 8;                  // row tiles walked together
constexpr uint32_t kPairHalfBytes = kPairRows * kTcBK * 2;          // one operand half of a stage
constexpr uint32_t kPairStageBytes = 2 * kPairHalfBytes;            // x half + w half
constexpr uint32_t kPairTxBytes = 2 * kPairStageBytes;              // both blocks' copies
// The q/k/v form's angles: for each of the block's 128 tokens the 64 cosines and 64 sines of its
// position, rows 4 floats apart from a multiple of 32 so that a warp's 16-byte accesses, a row a lane,
// meet no bank twice.
constexpr int kPairTabRow = 132;
constexpr size_t kPairTabBytes = (size_t)kPairRows * kPairTabRow * 4;
// barriers: full[S], empty[S], acc_full[2], acc_empty[2], and for each quarter of the rows "angles
// there" and "angles no longer needed"
__host__ __device__ constexpr size_t pair_smem(int epi) {
  return (size_t)pair_stages(epi) * kPairStageBytes + (epi == 3 ? kPairTabBytes : 0) +
         (2 * pair_stages(epi) + 4 + 8) * 8 + 16;
}

struct PairParams {
  void* out;          // bfloat16 [M, N] (or [M, N / 2] with SwiGLU), or the 32-bit stream [M, N]
  int ldo;
  int M, N;           // rows of x; rows of w (both halves together with SwiGLU)
  int k_blocks;
  int tiles_m, tiles_n, n_pairs;
  int chunk, n_chunks;  // a pair takes `chunk` neighbouring column tiles of one row tile in a row (a unit)
  int swiglu_half;    // row of w where the up half starts
  int wide;           // rows of `out` (and of the cache pages) are 32-byte aligned
  int* status;
  // PAIR_EPI_QKV_ROPE: out is the q/k/v buffer [M, (NQ + 2 NKV) * 128], of which only q is written
  const int* positions;     // [M]; a negative position: the row is skipped
  const int* slots;         // [M]
  const float* q_gain;      // [128] or null
  const float* k_gain;
  const float* cos_tab;     // [positions][64]
  const float* sin_tab;
  PagedKV cache;
  int n_q_heads;
  int write_kv;
  float qk_eps;
};

// 16 values, rounded to bfloat16, to 32 bytes at `dst`: one 32-byte store where `dst` is 32-byte
// aligned (`wide`), else two of 16 bytes.  A thread of the epilogue writes its own row, so a warp's
// store touches 32 rows; with 32 bytes a thread every store fills whole 32-byte sectors of L2
// (half as many transactions as 16-byte stores, which a product with a short K is bound by).
__device__ __forceinline__ void store_bf16x16(bf16* dst, const float* v, bool wide) {
  uint32_t w[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
    w[e] = *reinterpret_cast<uint32_t*>(&h);
  }
  if (wide) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(w[0]), "r"(w[1]),
                 "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
  } else {
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint4*>(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

// Eight consecutive floats (32-byte aligned) with one load: a thread of the epilogue reads its own
// token's row of a table, so a warp's load touches 32 rows, and what that costs is the number of
// 32-byte sectors asked of L2, not the bytes.
__device__ __forceinline__ void load_f32x8(const float* p, float4& a, float4& b) {
  asm volatile("ld.global.nc.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w), "=f"(b.x), "=f"(b.y), "=f"(b.z), "=f"(b.w) : "l"(p));
}

// bfloat16 x bfloat16 -> float, both K-major, M = 256 over the pair, N = 256.
__host__ __device__ constexpr uint32_t pair_idesc() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kPairTile >> 3) << 17) | ((uint32_t)(kPairTile >> 4) << 24);
}

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address of the same shared-memory place in block `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t own, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(own), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// A tile of this block's shared memory whose bytes complete on a barrier that may stand in the
// other block of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// All MMAs issued so far by this thread: when they are done, one arrival on the barrier at this
// place in BOTH blocks of the pair.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}

// One stage of the pair's product in one piece of PTX: ask the NEXT stage's barrier (test_wait: it
// answers at once and never suspends the thread, unlike try_wait), issue this stage's four MMAs (K = 16 each, 32 bytes further along the swizzled row), commit them to this stage's "empty"
// barrier in both blocks, and only then look at the barrier's answer - the thread does not wait for it
// before the MMAs are on their way.  Returns whether the next stage is full.
__device__ __forceinline__ uint32_t mma_stage_pair(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc,
                                                   uint32_t accumulate, uint32_t empty_bar, uint32_t next_full,
                                                   uint32_t next_parity) {
  uint32_t ready;
  asm volatile(
      "{\n\t.reg .pred p, q, t;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 q, [%8], %9;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "setp.eq.b32 t, %6, %6;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%1], %2, %3, %4, {%6, %6, %6, %6, %6, %6, %6, %6}, p;\n\t"
      "add.u64 %2, %2, 2;\n\tadd.u64 %3, %3, 2;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%1], %2, %3, %4, {%6, %6, %6, %6, %6, %6, %6, %6}, t;\n\t"
      "add.u64 %2, %2, 2;\n\tadd.u64 %3, %3, 2;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%1], %2, %3, %4, {%6, %6, %6, %6, %6, %6, %6, %6}, t;\n\t"
      "add.u64 %2, %2, 2;\n\tadd.u64 %3, %3, 2;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%1], %2, %3, %4, {%6, %6, %6, %6, %6, %6, %6, %6}, t;\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%7], %10;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(ready), "+r"(d_tmem), "+l"(da), "+l"(db)
      : "r"(idesc), "r"(accumulate), "r"(0u), "r"(empty_bar), "r"(next_full), "r"(next_parity), "h"((uint16_t)3)
      : "memory");
  return ready;
}

// The u-th unit of the list: a row tile and a chunk of `chunk` neighbouring column tiles.  Row tiles
// go in groups of kPairGroup, inside a group the row tile runs fastest, so that pairs working side by
// side share rows of x and of w.  (With chunk = 1 a unit is a tile.)
__device__ __forceinline__ void pair_unit(const PairParams& prm, int u, int& tile_m, int& chunk_n) {
  const int per_group = kPairGroup * prm.n_chunks;
  const int g = u / per_group, r = u - g * per_group;
  const int rows = min(kPairGroup, prm.tiles_m - g * kPairGroup);
  chunk_n = r / rows;
  tile_m = g * kPairGroup + (r - chunk_n * rows);
}

template <int EPI>
__global__ void __launch_bounds__(kPairThreads, 1)
gemm_pair_bf16_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                      const PairParams prm) {
  constexpr int kPairStages = pair_stages(EPI);
  extern __shared__ __align__(1024) unsigned char smem[];
  float* tab = (float*)(smem + (size_t)kPairStages * kPairStageBytes);          // (q/k/v form only)
  uint64_t* bars = (uint64_t*)(smem + (size_t)kPairStages * kPairStageBytes +
                               (EPI == PAIR_EPI_QKV_ROPE ? kPairTabBytes : 0));
  // full[S] (used in the first block), empty[S], acc_full[2], acc_empty[2] (used in the first block),
  // tab_full[4], tab_free[4]
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kPairStages),
                 acc_full0 = smem_u32(bars + 2 * kPairStages), acc_empty0 = smem_u32(bars + 2 * kPairStages + 2),
                 tab_full0 = smem_u32(bars + 2 * kPairStages + 4), tab_free0 = smem_u32(bars + 2 * kPairStages + 8);
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * kPairStages + 12);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1;
  const int n_units = prm.tiles_m * prm.n_chunks;

  if (tid == 0) {
    tma_prefetch_map(&map_x);
    tma_prefetch_map(&map_w);
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 2 * kPairEpilogueWarps);   // a lane of each epilogue warp of both blocks
    }
    for (int q = 0; q < 8; ++q) mbar_init(tab_full0 + 8 * q, 2);   // the two warps that share a quarter of the rows
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kPairEpilogueWarps) tmem_alloc_pair(smem_u32(tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  cluster_sync();                              // the other block's barriers exist before anything reaches them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();

  bool ok = (smem_u32(smem) & 1023u) == 0;
  if (!ok && tid == 0) atomicCAS(prm.status, 0, 49);

  if (tid == 32 * kPairEpilogueWarps) {
    // ------------------------------------------------------------------ TMA producer
    const uint32_t full_first = map_to_rank(full0, 0);       // the first block's barriers
    int c = 0;                                                // stage fillings so far
    for (int u = pair; u < n_units && ok; u += prm.n_pairs) {
      int tile_m, chunk_n;
      pair_unit(prm, u, tile_m, chunk_n);
      const int x_row = tile_m * kPairTile + (int)rank * kPairRows;
      for (int j = 0; j < prm.chunk && ok; ++j) {
        const int tile_n = chunk_n * prm.chunk + j;
        if (tile_n >= prm.tiles_n) break;
        const int w_row = EPI == PAIR_EPI_SWIGLU ? (int)rank * prm.swiglu_half + tile_n * kPairRows
                                                 : tile_n * kPairTile + (int)rank * kPairRows;
        for (int kb = 0; kb < prm.k_blocks; ++kb, ++c) {
          const int s = c % kPairStages;
          if (c >= kPairStages) {
            ok = mbar_wait(empty0 + 8 * s, ((c / kPairStages) & 1) ^ 1, prm.status, 41);
            if (!ok) break;
          }
          if (rank == 0) mbar_expect_tx(full0 + 8 * s, kPairTxBytes);
          const uint32_t dst = smem_u32(smem + (size_t)s * kPairStageBytes);
          tma_load_2d_pair(dst, &map_x, kb * kTcBK, x_row, full_first + 8 * s);
          tma_load_2d_pair(dst + kPairHalfBytes, &map_w, kb * kTcBK, w_row, full_first + 8 * s);
        }
      }
    }
  } else if (tid == 32 * (kPairEpilogueWarps + 1) && rank == 0) {
    // ------------------------------------------------------------------ MMA issuer (first block)
    // This thread is the pace of the kernel: a stage's four MMAs keep the tensor cores of both SMs
    // busy for 512 cycles, and reading the stage's barrier (about 220 cycles until the answer is
    // there), issuing them and committing took it longer than that.  So the barrier of the NEXT stage
    // is asked before this stage's MMAs are issued and its answer looked at after them; the bounded
    // wait is only entered when that answer was "not yet".
    constexpr uint32_t idesc = pair_idesc();
    const uint32_t stage0 = smem_u32(smem);
    int c = 0, i = 0;                          // stages consumed, tiles done
    uint32_t ready = 0;                        // the stage c is known to be full
    for (int u = pair; u < n_units && ok; u += prm.n_pairs) {
      int tile_m, chunk_n;
      pair_unit(prm, u, tile_m, chunk_n);
      for (int j = 0; j < prm.chunk && ok && chunk_n * prm.chunk + j < prm.tiles_n; ++j, ++i) {
        const int buf = i & 1;
        if (i >= 2) {                            // the epilogues of tile i - 2 have read this accumulator
          ok = mbar_wait(acc_empty0 + 8 * buf, ((i >> 1) & 1) ^ 1, prm.status, 42);
          if (!ok) break;
          tc_fence_after();
        }
        const uint32_t acc = tmem_base + (uint32_t)(buf * kPairTile);
        for (int kb = 0; kb < prm.k_blocks; ++kb, ++c) {
          const int s = c % kPairStages;
          if (!ready) {
            ok = mbar_wait(full0 + 8 * s, (c / kPairStages) & 1, prm.status, 43);
            if (!ok) break;
          }
          tc_fence_after();
          const int s_next = (c + 1) % kPairStages;
          const uint32_t base = stage0 + (uint32_t)s * kPairStageBytes;
          static_assert(kTcBK == 64, "mma_stage_pair issues four MMAs of K = 16");
          ready = mma_stage_pair(acc, smem_desc_k_sw128(base), smem_desc_k_sw128(base + kPairHalfBytes), idesc,
                                 kb ? 1u : 0u, empty0 + 8 * s, full0 + 8 * s_next,
                                 ((c + 1) / kPairStages) & 1);
        }
        if (!ok) break;
        tc_commit_pair(acc_full0 + 8 * buf);     // the tile's accumulator is complete in both blocks
      }
    }
  } else if (warp < kPairEpilogueWarps) {
    // ------------------------------------------------------------------ epilogue
    const uint32_t acc_empty_first = map_to_rank(acc_empty0, 0);
    const int quarter = warp & 3, side = warp >> 2;       // lanes 32 quarter ..., columns' half
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    int i = 0, units = 0;
    for (int u = pair; u < n_units && ok; u += prm.n_pairs, ++units) {
      int tile_m, chunk_n;
      pair_unit(prm, u, tile_m, chunk_n);
      const int m = tile_m * kPairTile + (int)rank * kPairRows + quarter * 32 + lane;
      // q/k/v form: what depends on the token alone is fetched once for the unit's column tiles - its
      // position, its cache page, and the cosines and sines of its position, which go to shared
      // memory: the two warps that share these 32 rows (one head each) bring one table each and use
      // both.  (Fetched per head and tile by every thread, a row a lane, the angles were a third of the
      // launch: 512 bytes for each of 24 to 40 heads of every token, asked of L2 sector by sector.)
      int pos = -1, page = 0;
      float* my_tab = tab + (size_t)(quarter * 32 + lane) * kPairTabRow;
      if (EPI == PAIR_EPI_QKV_ROPE) {
        pos = m < prm.M ? prm.positions[m] : -1;
        if (pos >= 0 && prm.write_kv)
          page = prm.cache.block_table[(size_t)prm.slots[m] * prm.cache.table_stride + pos / EK_PAGE];
        // the angles of the unit before are no longer read by either warp
        if (units > 0) ok = mbar_wait(tab_free0 + 8 * quarter, (units - 1) & 1, prm.status, 45);
        if (!ok) break;
        if (pos >= 0) {
          const float* src = (side == 0 ? prm.cos_tab : prm.sin_tab) + (size_t)pos * 64;
          float* to = my_tab + 64 * side;
#pragma unroll
          for (int e = 0; e < 64; e += 8) {
            float4 a, b;
            load_f32x8(src + e, a, b);
            *reinterpret_cast<float4*>(to + e) = a;
            *reinterpret_cast<float4*>(to + e + 4) = b;
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(tab_full0 + 8 * quarter);
        ok = mbar_wait(tab_full0 + 8 * quarter, units & 1, prm.status, 46);
        if (!ok) break;
      }
      for (int j = 0; j < prm.chunk && ok && chunk_n * prm.chunk + j < prm.tiles_n; ++j, ++i) {
        const int tile_n = chunk_n * prm.chunk + j;
        const int buf = i & 1;
        bf16* dst = nullptr;
        bool is_q = false, is_k = false, is_v = false;
        if (EPI == PAIR_EPI_QKV_ROPE) {
          const int n_kv = prm.cache.heads, nq = prm.n_q_heads;
          const int head = 2 * tile_n + side;     // columns 0..127 of the tile: warps 0..3; 128..255: warps 4..7
          is_q = head < nq;
          is_k = !is_q && head < nq + n_kv;
          is_v = !is_q && !is_k && head < nq + 2 * n_kv;
          if (is_q) {
            dst = (bf16*)prm.out + (size_t)m * prm.ldo + (size_t)head * 128;
          } else if ((is_k || is_v) && prm.write_kv && pos >= 0) {
            const int kv_head = is_k ? head - nq : head - nq - n_kv;
            dst = (bf16*)(is_k ? prm.cache.k : prm.cache.v) + page_offset(prm.cache, page, kv_head, pos);
          }
        }
        ok = mbar_wait(acc_full0 + 8 * buf, (i >> 1) & 1, prm.status, 44);
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc = lane_addr + (uint32_t)(buf * kPairTile);
        // This thread's 128 columns of the accumulator in one go (one wait for tensor memory instead of
        // one a chunk: with the MMAs of the next tile running, each such wait takes about a microsecond),
        // then the accumulator is handed back and the rest works from registers.
        float v[128];
        {
          const uint32_t first = EPI == PAIR_EPI_SWIGLU ? acc + (uint32_t)(side * 64) : acc + (uint32_t)(side * 128);
          tmem_ld32_nowait(first, v);
          tmem_ld32_nowait(first + 32, v + 32);
          if (EPI == PAIR_EPI_SWIGLU) {            // gate columns 64 side .. + 63, then their up columns
            tmem_ld32_nowait(first + 128, v + 64);
            tmem_ld32_nowait(first + 160, v + 96);
          } else {
            tmem_ld32_nowait(first + 64, v + 64);
            tmem_ld32_nowait(first + 96, v + 96);
          }
          tmem_ld_wait();
        }
        tc_fence_before();                       // read: the MMAs of tile i + 2 may overwrite the accumulator
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_first + 8 * buf);

        if (EPI == PAIR_EPI_SWIGLU) {
          const int n0 = tile_n * kPairRows + side * 64;     // this thread's outputs: n0 .. n0 + 63
          bf16* o = (bf16*)prm.out + (size_t)m * prm.ldo + n0;
          if (m < prm.M) {
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 16) {
#pragma unroll
              for (int e = 0; e < 16; ++e)
                v[c0 + e] = __fdividef(v[c0 + e], 1.f + __expf(-v[c0 + e])) * v[64 + c0 + e];
              if (n0 + c0 + 16 <= prm.swiglu_half) {
                store_bf16x16(o + c0, v + c0, prm.wide);
              } else {
                for (int e = 0; e < 16; ++e)
                  if (n0 + c0 + e < prm.swiglu_half) o[c0 + e] = __float2bfloat16_rn(v[c0 + e]);
              }
            }
          }
        } else if (EPI == PAIR_EPI_QKV_ROPE) {
          // the tile holds two heads of this thread's token, one for each half of the epilogue warps
          const bool store = pos >= 0 && dst != nullptr;
          if (is_v && prm.write_kv) {               // values: rounded and stored
            if (store) {
#pragma unroll
              for (int c0 = 0; c0 < 128; c0 += 16) store_bf16x16(dst + c0, v + c0, prm.wide);
            }
          } else if (store && (is_q || is_k)) {
            const float* gain = is_q ? prm.q_gain : prm.k_gain;
            float rstd = 1.f;
            if (gain) {
              float ss[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
              for (int e = 0; e < 128; ++e) ss[e & 3] = fmaf(v[e], v[e], ss[e & 3]);
              rstd = rsqrtf(((ss[0] + ss[1]) + (ss[2] + ss[3])) * (1.f / 128.f) + prm.qk_eps);
            }
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 16) {
#pragma unroll
              for (int e = 0; e < 16; e += 4) {
                float4 gl = make_float4(rstd, rstd, rstd, rstd), gh = gl;
                if (gain) {
                  const float4 a = *reinterpret_cast<const float4*>(gain + c0 + e);
                  const float4 b = *reinterpret_cast<const float4*>(gain + 64 + c0 + e);
                  gl = make_float4(a.x * rstd, a.y * rstd, a.z * rstd, a.w * rstd);
                  gh = make_float4(b.x * rstd, b.y * rstd, b.z * rstd, b.w * rstd);
                }
                const float4 cc = *reinterpret_cast<const float4*>(my_tab + c0 + e);
                const float4 sv = *reinterpret_cast<const float4*>(my_tab + 64 + c0 + e);
                const float cv[4] = {cc.x, cc.y, cc.z, cc.w}, sw[4] = {sv.x, sv.y, sv.z, sv.w};
                const float g0[4] = {gl.x, gl.y, gl.z, gl.w}, g1[4] = {gh.x, gh.y, gh.z, gh.w};
#pragma unroll
                for (int i2 = 0; i2 < 4; ++i2) {
                  const float x = v[c0 + e + i2] * g0[i2], y = v[64 + c0 + e + i2] * g1[i2];   // gain * x / rms
                  v[c0 + e + i2] = x * cv[i2] - y * sw[i2];
                  v[64 + c0 + e + i2] = y * cv[i2] + x * sw[i2];
                }
              }
              store_bf16x16(dst + c0, v + c0, prm.wide);
              store_bf16x16(dst + 64 + c0, v + 64 + c0, prm.wide);
            }
          }
        } else {
          const int n0 = tile_n * kPairTile + side * 128;     // this thread's columns: n0 .. n0 + 127
          if (m < prm.M) {
#pragma unroll
            for (int c0 = 0; c0 < 128; c0 += 32) {
              if (n0 + c0 >= prm.N) break;
              if (EPI == PAIR_EPI_ADD_F32) {
                float* o = (float*)prm.out + (size_t)m * prm.ldo + n0 + c0;
                if (n0 + c0 + 32 <= prm.N && prm.wide) {
                  float old[32];
#pragma unroll
                  for (int j = 0; j < 32; j += 8)
                    asm volatile("ld.global.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                                 : "=f"(old[j]), "=f"(old[j + 1]), "=f"(old[j + 2]), "=f"(old[j + 3]), "=f"(old[j + 4]),
                                   "=f"(old[j + 5]), "=f"(old[j + 6]), "=f"(old[j + 7]) : "l"(o + j) : "memory");
#pragma unroll
                  for (int j = 0; j < 32; j += 8)
                    asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(o + j),
                                 "f"(old[j] + v[c0 + j]), "f"(old[j + 1] + v[c0 + j + 1]), "f"(old[j + 2] + v[c0 + j + 2]),
                                 "f"(old[j + 3] + v[c0 + j + 3]), "f"(old[j + 4] + v[c0 + j + 4]),
                                 "f"(old[j + 5] + v[c0 + j + 5]), "f"(old[j + 6] + v[c0 + j + 6]),
                                 "f"(old[j + 7] + v[c0 + j + 7]) : "memory");
                } else if (n0 + c0 + 32 <= prm.N) {
#pragma unroll
                  for (int j = 0; j < 32; j += 4) {
                    const float4 old = *reinterpret_cast<const float4*>(o + j);
                    *reinterpret_cast<float4*>(o + j) = make_float4(old.x + v[c0 + j], old.y + v[c0 + j + 1],
                                                                    old.z + v[c0 + j + 2], old.w + v[c0 + j + 3]);
                  }
                } else {
                  for (int e = 0; e < 32; ++e)
                    if (n0 + c0 + e < prm.N) o[e] += v[c0 + e];
                }
              } else {
                bf16* o = (bf16*)prm.out + (size_t)m * prm.ldo + n0 + c0;
                if (n0 + c0 + 32 <= prm.N) {
                  store_bf16x16(o, v + c0, prm.wide);
                  store_bf16x16(o + 16, v + c0 + 16, prm.wide);
                } else {
                  for (int e = 0; e < 32; ++e)
                    if (n0 + c0 + e < prm.N) o[e] = __float2bfloat16_rn(v[c0 + e]);
                }
              }
            }
          }
        }
      }                                        // the unit's column tiles
      if (EPI == PAIR_EPI_QKV_ROPE && ok) {      // this warp has read the unit's angles for the last time
        __syncwarp();
        if (lane == 0) mbar_arrive(tab_free0 + 8 * quarter);
      }
    }
  }

  const int failed = __syncthreads_or(ok ? 0 : 1);
  if (failed)
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // let copies in flight land
  tc_fence_before();
  cluster_sync();                              // neither block's shared or tensor memory is in use any more
  if (warp == kPairEpilogueWarps) tmem_dealloc_pair(tmem_base, 512);
}

template <int EPI>
static int launch_pair(const CUtensorMap& mx, const CUtensorMap& mw, PairParams prm, cudaStream_t stream) {
  auto kernel = gemm_pair_bf16_kernel<EPI>;
  static int pairs_that_fit[kMaxDevices] = {};
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= kMaxDevices) return EK_ERR_ARG;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = pair_smem(EPI);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  if (pairs_that_fit[device] == 0) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pair_smem(EPI));
    if (e != cudaSuccess) return (int)e;
    prefer_carveout((const void*)kernel, 100);
    // how many pairs the device holds at once (not every SM need have a free neighbour)
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    cfg.numAttrs = 1;
    int clusters = 0;
    e = cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg);
    if (e != cudaSuccess) return (int)e;
    if (clusters < 1) return EK_ERR_ARG;
    pairs_that_fit[device] = clusters;
  }
  // Units of work: the q/k/v form takes a few neighbouring column tiles of a row tile in a row, so that
  // what it fetches per token serves them all, and still leaves about eight units a row tile to deal out
  prm.chunk = 1;
  if (EPI == PAIR_EPI_QKV_ROPE) {
    // rounds of units x (a unit's K blocks + what its fetch of the angles costs, about five K blocks'
    // time), for the chunk sizes that leave at least two units a row tile
    long long best = -1;
    for (int c = 1; c <= 8 && 2 * c <= prm.tiles_n + c - 1; ++c) {
      const long long units = (long long)prm.tiles_m * ((prm.tiles_n + c - 1) / c);
      const long long rounds = (units + pairs_that_fit[device] - 1) / pairs_that_fit[device];
      const long long cost = rounds * ((long long)c * prm.k_blocks + 5);
      if (best < 0 || cost < best) { best = cost; prm.chunk = c; }
    }
  }
  prm.n_chunks = (prm.tiles_n + prm.chunk - 1) / prm.chunk;
  const int n_units = prm.tiles_m * prm.n_chunks;
  prm.n_pairs = n_units < pairs_that_fit[device] ? n_units : pairs_that_fit[device];
  cfg.gridDim = dim3(2 * prm.n_pairs);
  cfg.numAttrs = 2;
  return (int)cudaLaunchKernelEx(&cfg, kernel, mx, mw, prm);
}

}  // namespace ek

// epilogue 0: out[M, N] = x . w^T in bfloat16; 1: out[M, N] (32-bit) += x . w^T; 2: out[M, N / 2] =
// silu(x . wg^T) * (x . wu^T) in bfloat16 with w = [N / 2 gate rows; N / 2 up rows].  K, ldx, ldw
// must be multiples of 8, ldo of 8 (4 for the 32-bit form), the pointers 16-byte aligned.
EK_EXPORT int ek_gemm_pair_bf16(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldw,
                                int ldo, int epilogue, int* status, cudaStream_t stream) {
  using namespace ek;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || !status || epilogue < 0 || epilogue > 2 ||
      ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15) ||
      ldo % (epilogue == PAIR_EPI_ADD_F32 ? 4 : 8) || (epilogue == PAIR_EPI_SWIGLU && (N & 1)))
    return EK_ERR_ARG;
  PairParams prm{};
  prm.out = out; prm.ldo = ldo; prm.M = M; prm.N = N; prm.status = status;
  prm.wide = (((uintptr_t)out & 31) == 0 && ldo % (epilogue == PAIR_EPI_ADD_F32 ? 8 : 16) == 0) ? 1 : 0;
  prm.k_blocks = (K + kTcBK - 1) / kTcBK;
  prm.swiglu_half = N / 2;
  prm.tiles_m = (M + kPairTile - 1) / kPairTile;
  prm.tiles_n = epilogue == PAIR_EPI_SWIGLU ? (N / 2 + kPairRows - 1) / kPairRows : (N + kPairTile - 1) / kPairTile;
  if ((long long)prm.tiles_m * prm.tiles_n > (1ll << 30)) return EK_ERR_ARG;
  CUtensorMap mx, mw;
  int rc;
  if ((rc = tensor_map(x, M, K, ldx, kPairRows, &mx))) return rc;
  if ((rc = tensor_map(w, N, K, ldw, kPairRows, &mw))) return rc;
  if (epilogue == PAIR_EPI_BF16) rc = launch_pair<PAIR_EPI_BF16>(mx, mw, prm, stream);
  else if (epilogue == PAIR_EPI_ADD_F32) rc = launch_pair<PAIR_EPI_ADD_F32>(mx, mw, prm, stream);
  else rc = launch_pair<PAIR_EPI_SWIGLU>(mx, mw, prm, stream);
  return rc;
}

// The q/k/v product of an attention layer whose heads are 128 wide and fully rotated, for many
// rows: qkv = x . w^T, then per head the RMSNorm of q and k (gains may be null), the rotation by
// cos/sin[position] ([P, 64] each), q to `out` [M, (NQ + 2 NKV) * 128] (its k and v columns are
// not written) and, with write_kv, k and v into the pages at the token's place.  Rows whose
// position is negative are skipped.
EK_EXPORT int ek_gemm_pair_qkv_rope(void* out, const void* x, const void* w, int M, int K, int ldx, int ldw,
                                    int ldo, const float* q_gain, const float* k_gain, float qk_eps,
                                    const float* cos_tab, const float* sin_tab, const int* positions,
                                    const int* token_slot, void* k_pages, void* v_pages,
                                    const int* block_table, int table_stride, int n_q_heads, int n_kv_heads,
                                    int write_kv, int* status, cudaStream_t stream) {
  using namespace ek;
  if (M <= 0) return 0;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ldo % 8 || !status || n_q_heads <= 0 || n_kv_heads <= 0 ||
      !positions || !token_slot || !cos_tab || !sin_tab || !k_pages || !v_pages || !block_table ||
      ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15) || ((uintptr_t)cos_tab & 31) ||
      ((uintptr_t)sin_tab & 31) || ((uintptr_t)q_gain & 15) || ((uintptr_t)k_gain & 15) ||
      ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15))
    return EK_ERR_ARG;
  PairParams prm{};
  prm.out = out; prm.ldo = ldo; prm.M = M; prm.status = status;
  prm.wide = (((uintptr_t)out & 31) == 0 && ldo % 16 == 0 && ((uintptr_t)k_pages & 31) == 0 &&
              ((uintptr_t)v_pages & 31) == 0) ? 1 : 0;
  prm.N = (n_q_heads + 2 * n_kv_heads) * 128;
  prm.k_blocks = (K + kTcBK - 1) / kTcBK;
  prm.tiles_m = (M + kPairTile - 1) / kPairTile;
  prm.tiles_n = (prm.N + kPairTile - 1) / kPairTile;
  if ((long long)prm.tiles_m * prm.tiles_n > (1ll << 30)) return EK_ERR_ARG;
  prm.positions = positions; prm.slots = token_slot;
  prm.q_gain = q_gain; prm.k_gain = k_gain; prm.qk_eps = qk_eps;
  prm.cos_tab = cos_tab; prm.sin_tab = sin_tab;
  prm.cache = PagedKV{k_pages, v_pages, block_table, table_stride, n_kv_heads, 128};
  prm.n_q_heads = n_q_heads; prm.write_kv = write_kv;
  CUtensorMap mx, mw;
  int rc;
  if ((rc = tensor_map(x, M, K, ldx, kPairRows, &mx))) return rc;
  if ((rc = tensor_map(w, prm.N, K, ldw, kPairRows, &mw))) return rc;
  return launch_pair<PAIR_EPI_QKV_ROPE>(mx, mw, prm, stream);
}
