// D = P . Q^T on the 5th-generation tensor cores: bfloat16 operands staged in shared memory
// by TMA (cp.async.bulk.tensor, 128-byte swizzle), tcgen05.mma issued by one thread with
// the 32-bit accumulator in tensor memory (TMEM), read back with tcgen05.ld for the
// epilogue.  P [rows_p, K] and Q [rows_q, K] are both K-major (rows contiguous in K).
//
// One block computes one 128 x BN tile of D over a range of K:
//   warp 0, one thread : TMA producer - fills a ring of STAGES (P tile, Q tile) pairs
//   warp 1, one thread : issues 4 tcgen05.mma (K = 16 each) per stage, commits to the
//                        stage's "empty" barrier, and finally to the accumulator barrier
//                        (swapped form: one thread of warp 2 as well; they take the stages in
//                        turn, each with an accumulator of its own)
//   all 4 warps        : epilogue - each warp reads its 32 TMEM lanes (rows of the tile)
// Two uses:
//   * swapped (decode, 1..64 sequences): P = the weight matrix, Q = the activations, so
//     the 128-row side of the MMA is filled with weight rows and the batch is the narrow
//     N side; the tile is out^T and is stored transposed.  The work is bound by streaming
//     the weights, so K is also split over blocks (grid.y).  Up to 8 blocks of a tile form
//     a thread-block cluster: each leaves its partial tile in its own shared memory and sums
//     its share of the tile's columns over all of them, in split order, through distributed
//     shared memory (with at most 8 sequences each block sends its partial sums to the
//     owning block instead, by stores that count their bytes on a barrier of the owner, and
//     only the owner waits - for those bytes, not for the cluster).  More splits than that go through scratch in global memory, and
//     the block that delivers the last partial of a tile adds them in split order.
//   * direct (prompts): P = activations, Q = weights, 128 x 256 tiles.
// Epilogues: bfloat16, 32-bit, or SwiGLU (the tile holds gate rows/columns in its first
// half and the matching up rows/columns in its second half).  The swapped form can also carry
// what would otherwise be small kernels between the products (see TcParams): the row scale of a
// deferred RMSNorm, the residual add with the next norm's gain and sums of squares, and for the
// q/k/v product the per-head norm, the rotation and the cache write.
// The reference calls cuBLAS for these products (engine/ek_model.py:203,209,298,311) and
// has no Blackwell path.  Every barrier wait is bounded: on a timeout the kernel records a
// code in `status`, lets in-flight copies land, frees its TMEM and returns.
#include "tc_common.cuh"

namespace ek {

enum { TC_EPI_BF16 = 0, TC_EPI_F32 = 1, TC_EPI_SWIGLU = 2 };

constexpr int kTcBM = 128;                    // rows of P per tile (TMEM lanes)
constexpr int kTcPushRows = 8;               // sequences whose partial sums are sent, not fetched
constexpr int kTcMaxCluster = 8;              // blocks of a cluster (the portable limit)

// Instruction descriptor: bfloat16 x bfloat16 -> float, both operands K-major, M = 128.
__host__ __device__ constexpr uint32_t tc_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTcBM >> 4) << 24);
}

// silu for a bfloat16 result: the fast exponential and division are good to a few 32-bit ulps
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.f + __expf(-x)); }

struct TcParams {
  void* out;            // [M_out, N_out] row-major, ldo elements between rows
  int ldo;
  int rows_p;           // valid rows of P (tile rows beyond it are not stored)
  int rows_q;           // valid rows of Q
  int k_blocks;         // ceil(K / 64)
  int k_blocks_per_split;
  int swiglu_half;      // SwiGLU: second-half row offset in the weight matrix (I)
  float* partials;      // split-K scratch [tile][split][BN][128]
  unsigned int* tickets;
  int* status;          // 0, or the code of the first wait that timed out
  // A norm deferred to this product (swapped form): the activations are the residual stream
  // times the norm's gain, and each sequence's 1/rms comes from the sums of squares that the
  // product before left per 128-column tile.  The result is scaled by it.
  const float* ss_in;   // [rows_q][ss_tiles], or null
  int ss_tiles;
  float ss_inv_size, eps;
  // The residual add and the next norm's share moved into this product (swapped form, bfloat16
  // result): stream += result in 32-bit; `out` gets stream * next_gain; ss_out[m][tile] gets the
  // tile's sum of stream^2.
  float* stream;        // [rows_q][ld_stream], or null
  int ld_stream;
  const float* next_gain;   // [rows_p]
  float* ss_out;        // [rows_q][gridDim.x]
  // The q/k/v product of an attention layer with heads of 128 (swapped form, bfloat16 result): a
  // 128-row tile is one head, so the per-head RMSNorm of q and k, the rotation by the token's
  // position and the write of k and v into the paged cache are done on the 32-bit sums, with one
  // rounding; q goes to `out`.  Same arithmetic as qk_norm_rope_kv_kernel.
  const int* qkv_positions;   // [rows_q], or null: not this form
  const int* qkv_slots;
  const float* q_gain;        // [128] or null
  const float* k_gain;
  const float* cos_tab;       // [positions][64]
  const float* sin_tab;
  PagedKV cache;
  int n_q_heads;
  int write_kv;
  float qk_eps;
};

// --------------------------------------------------------------------------------- kernel
template <int BN, int EPI, bool SWAP, int STAGES, bool CL>
__global__ void __launch_bounds__(128, (SWAP || BN > 128) ? 2 : 1)
gemm_tc_bf16_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                    const TcParams prm) {
  constexpr uint32_t kBytesP = kTcBM * kTcBK * 2;
  constexpr uint32_t kBytesQ = BN * kTcBK * 2;
  // The swapped form has two MMA-issuing threads with an accumulator each (stages in turn); the
  // second accumulator stands BN columns after the first.
  constexpr bool TWO = SWAP;
  static_assert(!TWO || STAGES % 2 == 0, "two issuing threads need an even number of stages");
  constexpr uint32_t kTmemCols = TWO ? (2 * BN < 32 ? 32 : 2 * BN) : (BN < 32 ? 32 : BN);
  // No static shared memory in this kernel, so the dynamic part starts at the block's first shared
  // byte, which is 1024-byte aligned as the 128-byte swizzle needs (checked below): two blocks of
  // the narrowest swapped form fill an SM's shared memory to the last kilobyte.
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* p_tiles = smem;
  unsigned char* q_tiles = smem + STAGES * kBytesP;
  uint64_t* bars = (uint64_t*)(q_tiles + STAGES * kBytesQ);   // full[STAGES], empty[STAGES], accum, received
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 2);
  int& is_last = *(int*)(tmem_slot + 1);
  float* rstd_s = (float*)(tmem_slot + 4);     // [64] 1/rms of each sequence (a norm deferred to here)
  // Clustered narrowest form with at most 8 sequences: what the other blocks of the cluster send,
  // [split][sequence of mine][weight row] (kTcRecvFloats floats, 16-byte aligned)
  float* recv = rstd_s + 64;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile_p = blockIdx.x;               // 128-row tile of P
  const int tile_q = SWAP ? 0 : blockIdx.z;    // BN-row tile of Q (direct use only)
  const int split = blockIdx.y, n_split = gridDim.y;
  const int kb_begin = split * prm.k_blocks_per_split;
  const int kb_end = min(prm.k_blocks, kb_begin + prm.k_blocks_per_split);
  const int n_iter = kb_end - kb_begin;

  pdl_launch_dependents();
  if (tid == 0) {
    tma_prefetch_map(&map_p);
    tma_prefetch_map(&map_q);
  }
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES),
                 accum_bar = smem_u32(bars + 2 * STAGES), recv_bar = smem_u32(bars + 2 * STAGES + 1);
  // The narrowest clustered form with at most kTcPushRows sequences: every block sends its partial
  // sums of a sequence into the shared memory of the block that owns the sequence, by stores that
  // count their bytes on a barrier of the owner (st.async); the owner waits for the bytes it
  // expects and no block waits for the whole cluster.
  constexpr bool kCanPush = CL && BN == 16;
  const int push_slots = (prm.rows_q + n_split - 1) / n_split;     // sequences a block owns at most
  const bool push = kCanPush && n_split * push_slots <= kTcPushRows;
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(accum_bar, TWO ? 2 : 1);
    mbar_init(recv_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (push) {                                  // the sequences split, split + n_split, ...: 512 bytes from every block each
      const int mine = prm.rows_q > split ? (prm.rows_q - split + n_split - 1) / n_split : 0;
      mbar_expect_tx(recv_bar, (uint32_t)(n_split * mine * kTcBM * 4));
    }
  }
  // (the barrier exists in every block of the cluster before a store from another block reaches it:
  // arrive here, wait just before the first such store)
  if (kCanPush) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  if (warp == 0) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  bool ok = (smem_u32(smem) & 1023u) == 0;       // never seen otherwise; the swizzled tiles would be wrong
  if (!ok && tid == 0) atomicCAS(prm.status, 0, 9);
  int fillings = 0;                              // stage fillings this thread has asked TMA for
  if (tid == 0) {
    // ---------------------------------------------------------------- TMA producer
    int p_row0, p_row1 = 0;
    if (EPI == TC_EPI_SWIGLU && SWAP) {        // weights on the P side: 64 gate rows + 64 up rows
      p_row0 = tile_p * 64;
      p_row1 = prm.swiglu_half + tile_p * 64;
    } else {
      p_row0 = tile_p * kTcBM;
    }
    int q_row0, q_row1 = 0;
    if (EPI == TC_EPI_SWIGLU && !SWAP) {       // weights on the Q side: BN/2 gate + BN/2 up rows
      q_row0 = tile_q * (BN / 2);
      q_row1 = prm.swiglu_half + tile_q * (BN / 2);
    } else {
      q_row0 = tile_q * BN;
    }
    const uint64_t stream_policy = l2_policy_evict_first();
    auto load_p = [&](int it) {
      const int s = it % STAGES;
      const uint32_t full = full0 + 8 * s, pd = smem_u32(p_tiles + s * kBytesP);
      const int k0 = (kb_begin + it) * kTcBK;
      if (SWAP) {                              // the weights are read once: first out of L2
        tma_load_2d_hint(pd, &map_p, k0, p_row0, full, stream_policy);
        if (EPI == TC_EPI_SWIGLU) tma_load_2d_hint(pd + kBytesP / 2, &map_p, k0, p_row1, full, stream_policy);
      } else {
        tma_load_2d(pd, &map_p, k0, p_row0, full);
      }
    };
    auto load_q = [&](int it) {
      const int s = it % STAGES;
      const uint32_t full = full0 + 8 * s, qd = smem_u32(q_tiles + s * kBytesQ);
      const int k0 = (kb_begin + it) * kTcBK;
      tma_load_2d(qd, &map_q, k0, q_row0, full);
      if (EPI == TC_EPI_SWIGLU && !SWAP) tma_load_2d(qd + kBytesQ / 2, &map_q, k0, q_row1, full);
    };
    // The weight operand does not depend on the kernel before this one: the first ring of
    // weight tiles is requested before waiting for that kernel, the activations after.
    const int first = ok ? min(n_iter, STAGES) : 0;
    for (int it = 0; it < first; ++it) {
      mbar_expect_tx(full0 + 8 * (it % STAGES), kBytesP + kBytesQ);
      if (SWAP) load_p(it); else load_q(it);
    }
    pdl_wait();
    for (int it = 0; it < first; ++it) {
      if (SWAP) load_q(it); else load_p(it);
    }
    fillings = first;
    for (int it = first; it < n_iter && ok; ++it) {
      const int s = it % STAGES;
      const uint32_t phase = (it / STAGES) & 1;
      ok = mbar_wait(empty0 + 8 * s, phase ^ 1, prm.status, 1);
      if (!ok) break;
      mbar_expect_tx(full0 + 8 * s, kBytesP + kBytesQ);
      load_p(it);
      load_q(it);
      fillings = it + 1;
    }
  } else if (tid == 32 || (TWO && tid == 64)) {
    // ---------------------------------------------------------------- MMA issuer(s)
    // A stage costs its issuing thread about 600 cycles (the barrier read 220, four MMAs 65 each,
    // the commit 130) whether or not the tile was there already, and with one thread that chain,
    // not the memory, set the pace of a block with many K blocks.  In the swapped form two
    // threads of two warps take the stages in turn, each into its own accumulator (the order of
    // the sum stays fixed); the epilogue adds the two.
    constexpr uint32_t idesc = tc_idesc(BN);
    const int mine = tid == 32 ? 0 : 1, step = TWO ? 2 : 1;
    const uint32_t acc = tmem_base + (uint32_t)(mine * BN);
    for (int it = mine; it < n_iter && ok; it += step) {
      const int s = it % STAGES;
      const uint32_t phase = (it / STAGES) & 1;
      ok = mbar_wait(full0 + 8 * s, phase, prm.status, 2);
      if (!ok) break;
      tc_fence_after();
      const uint64_t da = smem_desc_k_sw128(smem_u32(p_tiles + s * kBytesP));
      const uint64_t db = smem_desc_k_sw128(smem_u32(q_tiles + s * kBytesQ));
#pragma unroll
      for (int k = 0; k < kTcBK / 16; ++k)       // 32 bytes further along K inside the swizzle row
        tc_mma(acc, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (it >= step || k) ? 1u : 0u);
      tc_commit(empty0 + 8 * s);               // the stage is free once these MMAs have read it
    }
    tc_commit(accum_bar);                      // this thread's MMAs done: its accumulator is complete
  }

  // -------------------------------------------------------------------- epilogue (all warps)
  if (tid != 0) pdl_wait();                    // before any global write (thread 0 waited above)
  __syncwarp();
  if (SWAP && prm.ss_in != nullptr) {
    // two threads a sequence, 16 tiles each a round, all loads of a round in flight together; the
    // order of the sum is fixed, so every block gets the same 1/rms
    const int m = tid >> 1, h = tid & 1;
    float ss = 0.f;
    for (int t0 = 0; t0 < prm.ss_tiles; t0 += 32) {
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int t = t0 + 16 * h + i;
        v[i] = (m < prm.rows_q && t < prm.ss_tiles) ? __ldcg(&prm.ss_in[(size_t)m * prm.ss_tiles + t]) : 0.f;
      }
      float part = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) part += v[i];
      const float other = __shfl_xor_sync(0xffffffffu, part, 1);
      ss += h == 0 ? part + other : other + part;
    }
    if (h == 0 && m < prm.rows_q && m < 64) rstd_s[m] = rsqrtf(ss * prm.ss_inv_size + prm.eps);
  }
  // The staged epilogue (swapped form, below): a thread takes 4 neighbouring weight rows of one
  // sequence; a warp covers the tile's rows for one sequence (two with SwiGLU, whose outputs are
  // the 64 gate rows), the block 4 (8) sequences a pass, P passes a batch.  What a batch needs from
  // global memory - the stream and the next norm's gain, or the token's position, angles and cache
  // page - is asked for here for the first batch, while the MMAs still run: behind the cluster
  // barrier these loads (two and three dependent rounds) were the longest part of the epilogue.
  constexpr int R = EPI == TC_EPI_SWIGLU ? 64 : kTcBM;     // output rows of the tile
  constexpr int MPW = 32 / (R / 4);                         // sequences a warp and pass
  constexpr int P = CL ? 2 : 4;                             // passes a batch
  const int step = CL ? n_split : 1, first = CL ? split : 0;
  const int owned = prm.rows_q > first ? (prm.rows_q - first + step - 1) / step : 0;
  const int sub = lane / (R / 4), r0 = 4 * (lane % (R / 4));
  const bool fused_add = EPI == TC_EPI_BF16 && prm.stream != nullptr;
  const bool qkv_form = EPI == TC_EPI_BF16 && prm.qkv_positions != nullptr;
  const bool head_is_q = tile_p < prm.n_q_heads, head_is_k = !head_is_q && tile_p < prm.n_q_heads + prm.cache.heads;
  struct Asked { float4 st, gn, cs, sn; int pos, page; };
  Asked pre[P];
  auto ask = [&](int base) {
#pragma unroll
    for (int ps = 0; ps < P; ++ps) {
      const int idx = base + (ps * 4 + warp) * MPW + sub;
      const int m = first + idx * step;
      pre[ps].pos = -1;
      pre[ps].page = 0;
      if (fused_add && idx < owned && tile_p * kTcBM + r0 < prm.rows_p) {
        const int n_out = tile_p * kTcBM + r0;
        pre[ps].st = __ldcg(reinterpret_cast<const float4*>(prm.stream + (size_t)m * prm.ld_stream + n_out));
        pre[ps].gn = *reinterpret_cast<const float4*>(prm.next_gain + n_out);
      }
      if (qkv_form && idx < owned) {
        const int pos = prm.qkv_positions[m];
        pre[ps].pos = pos;
        if (pos >= 0 && (head_is_q || head_is_k)) {
          // dimension d pairs with d + 64: 16 lanes further on, same place in the lane
          pre[ps].cs = *reinterpret_cast<const float4*>(prm.cos_tab + (size_t)pos * 64 + (r0 & 63));
          pre[ps].sn = *reinterpret_cast<const float4*>(prm.sin_tab + (size_t)pos * 64 + (r0 & 63));
        }
        if (pos >= 0 && !head_is_q && prm.write_kv)
          pre[ps].page = prm.cache.block_table[(size_t)prm.qkv_slots[m] * prm.cache.table_stride + pos / EK_PAGE];
      }
    }
  };
  if (SWAP && (CL || n_split == 1)) ask(0);
  bool acc_ok = n_iter > 0 ? mbar_wait(accum_bar, 0, prm.status, 3) : true;
  tc_fence_after();
  // a failure anywhere in the block is everybody's failure
  const int failed = __syncthreads_or((ok && acc_ok) ? 0 : 1);

  const int row = warp * 32 + lane;            // row of the tile = TMEM lane
  const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
  const int tile_linear = SWAP ? tile_p : (tile_q * gridDim.x + tile_p);
  auto acc_ld16 = [&](uint32_t col, float* v) {     // 16 columns of the sum, this thread's row
    tmem_ld16(lane_addr + col, v);
    if (TWO && n_iter > 1) {                   // (with one K block the second accumulator was never written)
      float w[16];
      tmem_ld16(lane_addr + BN + col, w);
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] += w[i];
    }
  };

  if (SWAP && (CL || n_split == 1)) {
    // The tile goes to shared memory as [sequence][weight row] (the operand tiles are dead), and
    // from there each output is put together: the sum over the blocks of the cluster in split
    // order, SwiGLU of a gate row and its up row 64 further on, one rounding, one store.  A
    // block takes the sequences split, split + n_split, ...  Every block of a cluster passes
    // the barriers whatever happened to it, so that none waits for one that gave up.
    // With at most kTcPushRows sequences (narrowest clustered form) a block does not wait to be
    // read: it sends each sequence's partial sums (16 bytes a store) into the shared memory of the
    // block that owns the sequence (a buffer beside the ring - the owner may still be
    // multiplying), and after ONE cluster barrier every block has all it needs at home.
    float* red = (float*)smem;
    constexpr int NS = CL ? kTcMaxCluster : 1;
    const int slots = push_slots;
    if (kCanPush) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (!failed) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN && c0 < prm.rows_q; c0 += 16) {
        float v[16];
        if (n_iter > 0) {
          acc_ld16(c0, v);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) red[(c0 + i) * kTcBM + row] = v[i];
      }
    }
    if (push) {
      __syncthreads();
      if (!failed) {
        for (int f = tid; f < prm.rows_q * (kTcBM / 4); f += 128) {
          const int m = f / (kTcBM / 4), c = 4 * (f % (kTcBM / 4));
          st_async_f32x4(&recv[(split * slots + m / n_split) * kTcBM + c], (unsigned)(m % n_split),
                         *reinterpret_cast<const float4*>(&red[m * kTcBM + c]), recv_bar);
        }
      }
      // what this block owns has arrived when its barrier has counted the bytes (a block that gave
      // up sends nothing: the others' waits run out and say so)
      if (!mbar_wait(recv_bar, 0, prm.status, 5) && tid == 0) atomicCAS(prm.status, 0, 5);
    } else if (CL) {
      cluster_sync();
    } else {
      __syncthreads();
    }
    if (!failed) {
      // One 16-byte load a block of the cluster and thread; all loads of a batch are issued before
      // the first sum.
      const bool wide_ok = (prm.ldo & 3) == 0 && ((uintptr_t)prm.out & 15) == 0;
      auto fetch4 = [&](int m, int idx, int col, int sp) {   // 4 weight rows from `col` of split sp's tile
        if (push) return *reinterpret_cast<const float4*>(&recv[(sp * slots + idx) * kTcBM + col]);
        const float* p = &red[m * kTcBM + col];
        return CL ? ld_cluster_f32x4(p, (unsigned)sp) : *reinterpret_cast<const float4*>(p);
      };
#pragma unroll 1
      for (int base = 0; base < owned; base += P * 4 * MPW) {
        float4 part[P][NS], part_up[P][NS];
        if (base > 0) ask(base);                 // (the first batch was asked for before the barrier)
#pragma unroll
        for (int ps = 0; ps < P; ++ps) {
          const int idx = base + (ps * 4 + warp) * MPW + sub;
          const int m = first + idx * step;
#pragma unroll
          for (int sp = 0; sp < NS; ++sp) {
            const bool live = idx < owned && sp < n_split;
            part[ps][sp] = live ? fetch4(m, idx, r0, sp) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (EPI == TC_EPI_SWIGLU)
              part_up[ps][sp] = live ? fetch4(m, idx, r0 + 64, sp) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
#pragma unroll
        for (int ps = 0; ps < P; ++ps) {
          const int idx = base + (ps * 4 + warp) * MPW + sub;
          const int m = first + idx * step;
          float4 acc = part[ps][0];
          float4 up = EPI == TC_EPI_SWIGLU ? part_up[ps][0] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int sp = 1; sp < NS; ++sp) {
            if (sp < n_split) {
              acc.x += part[ps][sp].x; acc.y += part[ps][sp].y;
              acc.z += part[ps][sp].z; acc.w += part[ps][sp].w;
              if (EPI == TC_EPI_SWIGLU) {
                up.x += part_up[ps][sp].x; up.y += part_up[ps][sp].y;
                up.z += part_up[ps][sp].z; up.w += part_up[ps][sp].w;
              }
            }
          }
          if (prm.ss_in != nullptr && idx < owned) {
            const float rs = rstd_s[m];
            acc.x *= rs; acc.y *= rs; acc.z *= rs; acc.w *= rs;
            up.x *= rs; up.y *= rs; up.z *= rs; up.w *= rs;
          }
          int n_out, n_limit;
          if (EPI == TC_EPI_SWIGLU) {
            n_out = tile_p * 64 + r0;
            n_limit = prm.swiglu_half;
            acc.x = silu_fast(acc.x) * up.x; acc.y = silu_fast(acc.y) * up.y;
            acc.z = silu_fast(acc.z) * up.z; acc.w = silu_fast(acc.w) * up.w;
          } else {
            n_out = tile_p * kTcBM + r0;
            n_limit = prm.rows_p;
          }
          if (qkv_form) {
            // head = tile; everything below is uniform over the warp except the lane's 4 dimensions
            const int head = tile_p, n_kv = prm.cache.heads;
            const int pos = pre[ps].pos;
            const bool is_q = head_is_q, is_k = head_is_k;
            if (pos >= 0 && (is_q || prm.write_kv) && head < prm.n_q_heads + 2 * n_kv) {
              float y[4] = {acc.x, acc.y, acc.z, acc.w};
              if (is_q || is_k) {
                const float* gain = is_q ? prm.q_gain : prm.k_gain;
                if (gain != nullptr) {
                  const float ss = warp_sum(y[0] * y[0] + y[1] * y[1] + y[2] * y[2] + y[3] * y[3]);
                  const float rstd = rsqrtf(ss / 128.f + prm.qk_eps);
                  const float4 g4 = *reinterpret_cast<const float4*>(gain + r0);
                  y[0] = y[0] * rstd * g4.x; y[1] = y[1] * rstd * g4.y;
                  y[2] = y[2] * rstd * g4.z; y[3] = y[3] * rstd * g4.w;
                }
                const float4 cs = pre[ps].cs, sn = pre[ps].sn;
                const float c[4] = {cs.x, cs.y, cs.z, cs.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float partner = __shfl_xor_sync(0xffffffffu, y[i], 16);
                  y[i] = lane < 16 ? y[i] * c[i] - partner * sv[i] : y[i] * c[i] + partner * sv[i];
                }
              }
              bf16* dst;
              if (is_q) {
                dst = (bf16*)prm.out + (size_t)m * prm.ldo + n_out;
              } else {
                const int page = pre[ps].page;
                const int kv_head = is_k ? head - prm.n_q_heads : head - prm.n_q_heads - n_kv;
                dst = (bf16*)(is_k ? prm.cache.k : prm.cache.v) + page_offset(prm.cache, page, kv_head, pos) + r0;
              }
              __nv_bfloat162 lo = __floats2bfloat162_rn(y[0], y[1]), hi = __floats2bfloat162_rn(y[2], y[3]);
              *reinterpret_cast<uint2*>(dst) =
                  make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            }
          } else if (fused_add) {
            // rows_p and the strides are multiples of 4 here (checked by the launcher)
            float ssq = 0.f;
            if (idx < owned && n_out < n_limit) {
              float* sp = prm.stream + (size_t)m * prm.ld_stream + n_out;
              float4 st = pre[ps].st;
              st.x += acc.x; st.y += acc.y; st.z += acc.z; st.w += acc.w;
              *reinterpret_cast<float4*>(sp) = st;
              ssq = st.x * st.x + st.y * st.y + st.z * st.z + st.w * st.w;
              __nv_bfloat162 lo = __floats2bfloat162_rn(st.x * pre[ps].gn.x, st.y * pre[ps].gn.y);
              __nv_bfloat162 hi = __floats2bfloat162_rn(st.z * pre[ps].gn.z, st.w * pre[ps].gn.w);
              *reinterpret_cast<uint2*>((bf16*)prm.out + (size_t)m * prm.ldo + n_out) =
                  make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            }
            ssq = warp_sum(ssq);                 // a warp holds one sequence's 128 columns
            if (lane == 0 && idx < owned) prm.ss_out[(size_t)m * gridDim.x + tile_p] = ssq;
          } else if (idx < owned && n_out < n_limit) {
            const float v[4] = {acc.x, acc.y, acc.z, acc.w};
            if (EPI == TC_EPI_F32) {
              float* o = (float*)prm.out + (size_t)m * prm.ldo + n_out;
              if (n_out + 4 <= n_limit && wide_ok) {
                *reinterpret_cast<float4*>(o) = acc;
              } else {
                for (int i = 0; i < 4 && n_out + i < n_limit; ++i) o[i] = v[i];
              }
            } else {
              bf16* o = (bf16*)prm.out + (size_t)m * prm.ldo + n_out;
              if (n_out + 4 <= n_limit && wide_ok) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
                *reinterpret_cast<uint2*>(o) = make_uint2(*reinterpret_cast<uint32_t*>(&lo),
                                                          *reinterpret_cast<uint32_t*>(&hi));
              } else {
                for (int i = 0; i < 4 && n_out + i < n_limit; ++i) o[i] = __float2bfloat16_rn(v[i]);
              }
            }
          }
        }
      }
    } else {
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    if (CL && !push) cluster_sync();           // nobody leaves while its partial may be read
  } else if (!failed) {
    if (n_split > 1) {
      // partial tile -> scratch [tile][split][BN][128] (coalesced over rows)
      float* mine = prm.partials + ((size_t)tile_linear * n_split + split) * BN * kTcBM;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        float v[16];
        if (n_iter > 0) {
          acc_ld16(c0, v);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) mine[(size_t)(c0 + i) * kTcBM + row] = v[i];
      }
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const unsigned int ticket = atomicAdd(&prm.tickets[tile_linear], 1u);
        is_last = ticket == (unsigned int)(n_split - 1);
        if (is_last) prm.tickets[tile_linear] = 0;
      }
      __syncthreads();
    }
    if (n_split == 1 || is_last) {
      if (n_split > 1) __threadfence();
      const float* all = prm.partials + (size_t)tile_linear * n_split * BN * kTcBM;
      float* xch = (float*)smem;               // SwiGLU exchange buffer (operand tiles are dead)
      constexpr int kCols = (EPI == TC_EPI_SWIGLU && !SWAP) ? BN / 2 : BN;
#pragma unroll 1
      for (int c0 = 0; c0 < kCols; c0 += 16) {
        float v[16], u[16];
        auto fetch = [&](int col, float dst[16]) {
          if (n_split == 1) {
            acc_ld16(col, dst);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) dst[i] = 0.f;
            for (int sp = 0; sp < n_split; ++sp)
#pragma unroll
              for (int i = 0; i < 16; ++i)
                dst[i] += __ldcg(&all[((size_t)sp * BN + col + i) * kTcBM + row]);
          }
        };
        fetch(c0, v);
        if (EPI == TC_EPI_SWIGLU && !SWAP) {
          fetch(c0 + BN / 2, u);               // the matching up columns
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = silu_fast(v[i]) * u[i];
        }
        if (EPI == TC_EPI_SWIGLU && SWAP) {
          // rows 64..127 hold the up rows of the gate rows 0..63: pass them through shared memory
          __syncthreads();
          if (row >= 64) {
#pragma unroll
            for (int i = 0; i < 16; ++i) xch[(row - 64) * 16 + i] = v[i];
          }
          __syncthreads();
          if (row < 64) {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = silu_fast(v[i]) * xch[row * 16 + i];
          }
        }
        if (SWAP) {
          // tile row = output column (weight row), tile column = output row (sequence)
          int n_out;
          bool row_ok;
          if (EPI == TC_EPI_SWIGLU) {
            n_out = tile_p * 64 + row;
            row_ok = row < 64 && n_out < prm.swiglu_half;
          } else {
            n_out = tile_p * kTcBM + row;
            row_ok = n_out < prm.rows_p;
          }
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int m = c0 + i;
              if (m < prm.rows_q) {
                if (EPI == TC_EPI_F32) ((float*)prm.out)[(size_t)m * prm.ldo + n_out] = v[i];
                else ((bf16*)prm.out)[(size_t)m * prm.ldo + n_out] = __float2bfloat16_rn(v[i]);
              }
            }
          }
        } else {
          const int m = tile_p * kTcBM + row;
          const int n0 = tile_q * kCols + c0;
          const int n_limit = EPI == TC_EPI_SWIGLU ? prm.swiglu_half : prm.rows_q;
          if (m < prm.rows_p) {
            if (EPI == TC_EPI_F32) {
              float* o = (float*)prm.out + (size_t)m * prm.ldo + n0;
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (n0 + i < n_limit) o[i] = v[i];
            } else {
              bf16* o = (bf16*)prm.out + (size_t)m * prm.ldo + n0;
              if (n0 + 16 <= n_limit && (prm.ldo % 8) == 0) {
                uint32_t w[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                  w[i] = *reinterpret_cast<uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(o) = make_uint4(w[0], w[1], w[2], w[3]);
                *reinterpret_cast<uint4*>(o + 8) = make_uint4(w[4], w[5], w[6], w[7]);
              } else {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                  if (n0 + i < n_limit) o[i] = __float2bfloat16_rn(v[i]);
              }
            }
          }
        }
      }
    }
  } else {
    // let copies that are still in flight land before the shared memory is given up
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }

  // No copy of this block may still be on its way when the block exits: a bulk copy that lands in
  // the shared memory of a block that is gone, and completes a barrier there, is a fault (an
  // "unspecified launch failure"), not a wrong number.  On the ordinary path every filling has
  // been waited for by the thread that multiplied it (each issuing thread sees every filling of
  // its stages: the stage count is even).  A block in which a wait ran out has skipped such
  // waits, so there the producer waits (bounded) for the last filling of every stage it asked
  // for before the block goes.  (Looking at the barriers on every exit was measured: 6 reads of
  // ~220 cycles at the end of each of a step's 145 products, 5 % of a decode step.)
  if (failed && tid == 0) {
    for (int it = fillings > STAGES ? fillings - STAGES : 0; it < fillings; ++it)
      if (!mbar_wait(full0 + 8 * (it % STAGES), (it / STAGES) & 1, prm.status, 4)) break;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

// A bounded wait that must run out: one thread waits for a barrier that nothing completes, for
// `limit` rounds, records `code` in `status` and returns.  For the host-side test of the path from
// a timed-out wait to the error the caller sees; the kernel ends by itself after `limit` rounds.
__global__ void wait_that_runs_out_kernel(int* status, int code, unsigned limit) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_wait_limit(smem_u32(&bar), 0, status, code, limit);
  }
}

// Stages of the swapped form's operand ring: what two blocks an SM can hold, and an even number.
// Its two MMA-issuing threads take the stages in turn, and a thread has to see every filling of
// a stage it waits for: an mbarrier's phase is known by its parity alone, so a thread that saw
// only every other filling would take "the filling before is not there yet" for "mine is
// complete" (with 5 stages that happened, rarely, and broke the barrier protocol).
constexpr int swap_stages(int bn) { return bn <= 16 ? 6 : 4; }

template <int BN, int EPI, bool SWAP, bool CL = false>
static int launch_tc(const CUtensorMap& mp, const CUtensorMap& mq, const TcParams& prm, dim3 grid,
                     cudaStream_t stream) {
  // swapped: two blocks an SM, stages as swap_stages says (a stage is 16 KB of weights and BN rows
  // of activations); direct with 256-wide tiles: two blocks an SM of two 48 KB
  // stages each, so that one block's epilogue runs under the other's MMAs
  constexpr int STAGES = SWAP ? swap_stages(BN) : (BN <= 128 ? 6 : 2);
  // ring, barriers, TMEM slot + flag, 64 row scales, and the receive buffer of the clustered
  // narrowest form; 2 x (this + 1 KB the system keeps) fits an SM's 228 KB
  constexpr size_t smem = (size_t)STAGES * (kTcBM * kTcBK * 2 + BN * kTcBK * 2) + (2 * STAGES + 2) * 8 + 16 +
                          64 * 4 + ((CL && BN == 16) ? kTcPushRows * kTcBM * 4 : 0);
  static_assert(!SWAP || 2 * (smem + 1024) <= 228 * 1024, "two blocks an SM");
  auto kernel = gemm_tc_bf16_kernel<BN, EPI, SWAP, STAGES, CL>;
  static bool configured[kMaxDevices] = {};     // the attribute is per device and sticks
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= kMaxDevices) return EK_ERR_ARG;
  if (!configured[device]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured[device] = true;
  }
  prefer_carveout((const void*)kernel, 100);   // the operand ring wants all the shared memory
  if (CL) return (int)launch_pdl_cluster(kernel, grid, dim3(128), smem, stream, (int)grid.y, mp, mq, prm);
  return (int)launch_pdl(kernel, grid, dim3(128), smem, stream, mp, mq, prm);
}

}  // namespace ek

// out[M, N] = x[M, K] . w[N, K]^T  (epilogue 0/1) or out[M, N/2] = silu(x.wg^T) * (x.wu^T) with w =
// [gate rows; up rows] (epilogue 2).  swap != 0: weights fill the 128-row MMA side (for
// 1..64 rows of x); k_split blocks share a tile's K: as a cluster if `cluster` != 0 and k_split is
// at most 8, else through `partials` (at least tiles * k_split * bn * 128 floats) and zeroed
// `tickets` (at least `tiles`).
// K, ldx, ldw must be multiples of 8; `status` is one int on the device.
static int gemm_tc_run(const ek::TcParams& extras, void* out, const void* x, const void* w, int M, int N,
                       int K, int ldx, int ldw, int ldo, int epilogue, int swap, int k_split, int cluster,
                       float* partials, unsigned int* tickets, long long partial_floats, int n_tickets,
                       const float* ss_in, int ss_tiles, int norm_size, float eps, float* residual,
                       int ld_residual, const float* next_gain, float* ss_out, int* status,
                       cudaStream_t stream) {
  using namespace ek;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || !status || epilogue < 0 || epilogue > 2 ||
      (epilogue == TC_EPI_SWIGLU && (N & 1)) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
    return EK_ERR_ARG;
  const int k_blocks = (K + kTcBK - 1) / kTcBK;
  TcParams prm = extras;
  prm.out = out; prm.ldo = ldo; prm.k_blocks = k_blocks; prm.status = status;
  prm.partials = partials; prm.tickets = tickets;
  prm.swiglu_half = N / 2;
  prm.ss_in = ss_in; prm.ss_tiles = ss_tiles; prm.eps = eps;
  prm.ss_inv_size = norm_size > 0 ? 1.f / (float)norm_size : 0.f;
  prm.stream = residual; prm.ld_stream = ld_residual; prm.next_gain = next_gain; prm.ss_out = ss_out;
  if (ss_in && (!swap || ss_tiles <= 0 || norm_size <= 0)) return EK_ERR_ARG;
  if (residual && (!swap || epilogue != TC_EPI_BF16 || !next_gain || !ss_out || N % 4 || ldo % 4 ||
                   ld_residual % 4 || ((uintptr_t)residual & 15) || ((uintptr_t)next_gain & 15) ||
                   ((uintptr_t)out & 7)))
    return EK_ERR_ARG;
  if (k_split < 1) k_split = 1;
  if (k_split > k_blocks) k_split = k_blocks;
  CUtensorMap mp, mq;
  int rc;
  if (swap) {
    if (M > 64) return EK_ERR_ARG;
    const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    const bool sw = epilogue == TC_EPI_SWIGLU;
    const int tiles = sw ? (N / 2 + 63) / 64 : (N + kTcBM - 1) / kTcBM;
    prm.k_blocks_per_split = (k_blocks + k_split - 1) / k_split;
    k_split = (k_blocks + prm.k_blocks_per_split - 1) / prm.k_blocks_per_split;
    const bool clustered = cluster && k_split > 1 && k_split <= kTcMaxCluster;
    if (k_split > 1 && !clustered && (ss_in || residual || prm.qkv_positions || !partials || !tickets || tiles > n_tickets ||
                                      (long long)tiles * k_split * bn * kTcBM > partial_floats)) {
      k_split = 1;                             // (the deferred-norm forms have no scratch path)
      prm.k_blocks_per_split = k_blocks;
    }
    prm.rows_p = N; prm.rows_q = M;
    if ((rc = tensor_map(w, N, K, ldw, sw ? 64 : kTcBM, &mp))) return rc;
    if ((rc = tensor_map(x, M, K, ldx, bn, &mq))) return rc;
    dim3 grid(tiles, k_split, 1);
#define EK_SWAP(BN)                                                                              \
  if (bn == BN && clustered) {                                                                   \
    if (epilogue == TC_EPI_BF16) return launch_tc<BN, TC_EPI_BF16, true, true>(mp, mq, prm, grid, stream); \
    if (epilogue == TC_EPI_F32) return launch_tc<BN, TC_EPI_F32, true, true>(mp, mq, prm, grid, stream);   \
    return launch_tc<BN, TC_EPI_SWIGLU, true, true>(mp, mq, prm, grid, stream);                  \
  }                                                                                              \
  if (bn == BN) {                                                                                \
    if (epilogue == TC_EPI_BF16) return launch_tc<BN, TC_EPI_BF16, true>(mp, mq, prm, grid, stream); \
    if (epilogue == TC_EPI_F32) return launch_tc<BN, TC_EPI_F32, true>(mp, mq, prm, grid, stream);   \
    return launch_tc<BN, TC_EPI_SWIGLU, true>(mp, mq, prm, grid, stream);                        \
  }
    EK_SWAP(16) EK_SWAP(32) EK_SWAP(64)
#undef EK_SWAP
    return EK_ERR_ARG;
  }
  // direct: P = x (128-row tiles), Q = w (BN-row tiles); no K split
  prm.k_blocks_per_split = k_blocks;
  prm.rows_p = M; prm.rows_q = N;
  const bool sw = epilogue == TC_EPI_SWIGLU;
  constexpr int BN = 256;
  const int tiles_q = sw ? (N / 2 + BN / 2 - 1) / (BN / 2) : (N + BN - 1) / BN;
  if (tiles_q > 65535) return EK_ERR_ARG;
  if ((rc = tensor_map(x, M, K, ldx, kTcBM, &mp))) return rc;
  if ((rc = tensor_map(w, N, K, ldw, sw ? BN / 2 : BN, &mq))) return rc;
  dim3 grid((M + kTcBM - 1) / kTcBM, 1, tiles_q);
  if (epilogue == TC_EPI_BF16) return launch_tc<BN, TC_EPI_BF16, false>(mp, mq, prm, grid, stream);
  if (epilogue == TC_EPI_F32) return launch_tc<BN, TC_EPI_F32, false>(mp, mq, prm, grid, stream);
  return launch_tc<BN, TC_EPI_SWIGLU, false>(mp, mq, prm, grid, stream);
}

EK_EXPORT int ek_gemm_tc_bf16(void* out, const void* x, const void* w, int M, int N, int K, int ldx,
                              int ldw, int ldo, int epilogue, int swap, int k_split, int cluster,
                              float* partials, unsigned int* tickets, long long partial_floats,
                              int n_tickets, const float* ss_in, int ss_tiles, int norm_size, float eps,
                              float* residual, int ld_residual, const float* next_gain, float* ss_out,
                              int* status, cudaStream_t stream) {
  return gemm_tc_run(ek::TcParams{}, out, x, w, M, N, K, ldx, ldw, ldo, epilogue, swap, k_split, cluster,
                     partials, tickets, partial_floats, n_tickets, ss_in, ss_tiles, norm_size, eps,
                     residual, ld_residual, next_gain, ss_out, status, stream);
}

// The q/k/v product of an attention layer whose heads are 128 wide and fully rotated, for at most
// 64 rows: qkv = x . w^T (optionally with the row scale of a deferred norm), then per head the
// RMSNorm of q and k (gains may be null), the rotation by cos/sin[position] ([P, 64] each), q to
// `out` [M, (NQ + 2 NKV) * 128] and, with write_kv, k and v into the pages at the token's place.
// Up to 8 K splits as a cluster.
EK_EXPORT int ek_gemm_tc_qkv_rope(void* out, const void* x, const void* w, int M, int K, int ldx, int ldw,
                                  int ldo, int k_split, const float* ss_in, int ss_tiles, int norm_size,
                                  float eps, const float* q_gain, const float* k_gain, float qk_eps,
                                  const float* cos_tab, const float* sin_tab, const int* positions,
                                  const int* token_slot, void* k_pages, void* v_pages,
                                  const int* block_table, int table_stride, int n_q_heads,
                                  int n_kv_heads, int write_kv, int* status, cudaStream_t stream) {
  using namespace ek;
  if (M <= 0) return 0;
  if (M > 64 || n_q_heads <= 0 || n_kv_heads <= 0 || !positions || !token_slot || !cos_tab || !sin_tab ||
      !k_pages || !v_pages || !block_table || ldo % 4 || ((uintptr_t)out & 7) ||
      ((uintptr_t)cos_tab & 15) || ((uintptr_t)sin_tab & 15) || ((uintptr_t)q_gain & 15) ||
      ((uintptr_t)k_gain & 15) || ((uintptr_t)k_pages & 7) || ((uintptr_t)v_pages & 7))
    return EK_ERR_ARG;
  TcParams extras{};
  extras.qkv_positions = positions;
  extras.qkv_slots = token_slot;
  extras.q_gain = q_gain;
  extras.k_gain = k_gain;
  extras.cos_tab = cos_tab;
  extras.sin_tab = sin_tab;
  extras.cache = PagedKV{k_pages, v_pages, block_table, table_stride, n_kv_heads, kTcBM};
  extras.n_q_heads = n_q_heads;
  extras.write_kv = write_kv;
  extras.qk_eps = qk_eps;
  const int N = (n_q_heads + 2 * n_kv_heads) * kTcBM;
  if (k_split > kTcMaxCluster) k_split = kTcMaxCluster;
  return gemm_tc_run(extras, out, x, w, M, N, K, ldx, ldw, ldo, TC_EPI_BF16, 1, k_split, 1, nullptr,
                     nullptr, 0, 0, ss_in, ss_tiles, norm_size, eps, nullptr, 0, nullptr, nullptr, status,
                     stream);
}

// Launches one thread that waits `limit` rounds (at most 1,000,000, a fraction of a second) for a
// barrier that never completes and then records `code` in `status`.  Nothing else is touched.
EK_EXPORT int ek_tc_wait_that_runs_out(int* status, int code, unsigned limit, cudaStream_t stream) {
  if (!status || code <= 0 || limit == 0 || limit > 1000000u) return EK_ERR_ARG;
  ek::wait_that_runs_out_kernel<<<1, 32, 0, stream>>>(status, code, limit);
  EK_RETURN_LAUNCH_STATUS();
}
