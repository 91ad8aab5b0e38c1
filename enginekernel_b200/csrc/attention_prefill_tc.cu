// Causal prompt attention on the 5th-generation tensor cores (head sizes 64 and 128).
//
// A block owns 128 rows - (token, query head of one GQA group) pairs of consecutive new
// tokens of one sequence - and one KV head, like the mma.sync kernel in
// attention_prefill_bf16.cu, and walks the sequence's cache pages (64 keys each):
//   S  = Q . K^T      tcgen05.mma, Q and the K page in shared memory (K by TMA), S in TMEM,
//                     two S buffers so that page t+1 is scored while page t is in softmax
//   P  = softmax step  4 warps, a thread a row (warp w reaches TMEM lanes 32 w ...): the 64
//                      scores come into registers by tcgen05.ld, and P, rounded to bfloat16,
//                      goes back into the first 32 columns of the S buffer it came from
//                      (tcgen05.st, two values a column); no thread needs another's numbers
//   O += P . V        tcgen05.mma with P read from TMEM, accumulating in TMEM; the V page arrives
//                      by TMA and is used as it lies (rows = keys, i.e. an MN-major operand)
// The scores of page t+2 overwrite an S buffer only after the P.V of page t, which reads its P
// from there, is done: the S issuer waits for that page's pv_done barrier.
// The running maximum is lazy: exponentials are taken against a reference that is raised (and O
// and the running sum rescaled, by tcgen05.ld/st of the row) only when a page's maximum exceeds
// it by more than 2^8, which keeps every probability finite in bfloat16 and skips the rescale
// of almost every page.  O is divided by the sum once, at the end.
// Warp 4 (one thread) is the TMA producer, warps 5 and 6 (one thread each) issue the S and the
// P.V MMAs.  Q comes by TMA as well: the rows (token, head of the group) are a box of a tensor map
// that sees the query rows as [tokens][heads][head size].  A block's fixed costs count here (half
// the time of a 2,048-token prompt went to them when Q was fetched with plain loads and all
// setup stood behind the wait for the kernel ahead), so everything that does not read that
// kernel's results - tile search, barriers, the TMEM allocation - is done before the wait.  Shared memory
// holds Q, three stages of K (the scores of page t+1 need their K two softmax steps ahead of
// time, or the softmax warps wait for it) and two of V - 112 KB at head size 128 - and TMEM 256
// columns (S, S, O): two blocks an SM.  Every wait is bounded and reports through `status`.
// Formula and rounding points as in the mma.sync kernel (scores and softmax in 32-bit, P in
// bfloat16 before P.V; engine/ek_kernels.py:166-221 is the reference's Triton counterpart).
#include "tc_common.cuh"

namespace ek {

constexpr int kFaRows = 128;
constexpr int kFaKeys = EK_PAGE;             // 64
constexpr int kFaThreads = 224;              // 4 softmax warps, a producer warp, two MMA warps
constexpr int kFaKStages = 3;                // K pages in flight: two pages of lookahead for the scores
constexpr int kFaVStages = 2;
// mbarriers: K full / empty per K stage, V full / empty per V stage, then per S buffer (2):
// scores complete, P written, P.V done; and Q landed
constexpr int kBarKFull = 0, kBarKEmpty = kBarKFull + kFaKStages, kBarVFull = kBarKEmpty + kFaKStages,
              kBarVEmpty = kBarVFull + kFaVStages, kBarSFull = kBarVEmpty + kFaVStages,
              kBarPFull = kBarSFull + 2, kBarPvDone = kBarPFull + 2, kBarQFull = kBarPvDone + 2,
              kFaBars = kBarQFull + 1;

// Two 32-bit values at once (sm_100's packed single-precision pipe): the softmax warps are short
// of issue slots, and the scale-and-shift before each exponential and the running sums are half
// as many instructions this way, with the same rounding as their scalar forms.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  uint64_t ra, rb, rc, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  uint64_t ra, rb, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}

template <int D>
__global__ void __launch_bounds__(kFaThreads, 2)
attention_prefill_tc_kernel(bf16* __restrict__ out, const __grid_constant__ CUtensorMap map_q,
                            const int4* __restrict__ tiles,
                            const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* block_table,
                            int table_stride, int n_kv_heads, int n_q_heads, float scale_log2,
                            int window, int tok_per_tile, int* status) {
  constexpr int DB = D / 64;                       // 64-wide blocks of the head dimension
  constexpr uint32_t kSub = kFaKeys * 128;         // one [64 x 64] bfloat16 sub-tile: 8 KB
  constexpr uint32_t kTmemCols = 256;
  constexpr uint32_t kColS = 0, kColO = 128;        // S buffers at 0 and 64, O at 128
  // No static shared memory in this kernel, so the dynamic part starts at the block's first
  // shared byte, which is 1024-byte aligned as the 128-byte swizzle needs; the kernel checks it.
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* q_s = smem;                                   // DB x [128 x 64]
  unsigned char* k_s = q_s + DB * 2 * kSub;                    // K stages x DB x [64 x 64]
  unsigned char* v_s = k_s + kFaKStages * DB * kSub;           // V stages x DB x [64 x 64]
  uint64_t* bars = (uint64_t*)(v_s + kFaVStages * DB * kSub);
  uint32_t* tmem_slot = (uint32_t*)(bars + kFaBars);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kv_head = blockIdx.x;             // heads fastest: blocks start longest key range first
  const int group = n_q_heads / n_kv_heads;

  pdl_launch_dependents();
  // The tile's tokens, position and slot come from a table made once per step (sequence bounds,
  // positions and slots were uploaded before the step's first kernel, and the table is made
  // before its first attention kernel): one 16-byte load instead of a search through the
  // sequences and two more dependent loads in every block of every layer.
  const int4 tile = __ldg(&tiles[blockIdx.y]);     // first token, tokens, position of the first, slot
  const int t_first = tile.x, n_tok = tile.y;
  if (n_tok <= 0) return;                          // the table is padded to the grid's size
  if (tid == 128) {
    tma_prefetch_map(&map_q);
    tma_prefetch_map(&map_k);
    tma_prefetch_map(&map_v);
  }
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };
  if (tid == 0) {
    for (int i = 0; i < kFaBars; ++i) mbar_init(bar(i), (i == kBarPFull || i == kBarPFull + 1) ? 4 : 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int n_rows = n_tok * group;
  const bool misplaced = (smem_u32(smem) & 1023u) != 0;   // never seen; the swizzled tiles would be wrong
  const int pos0 = misplaced ? -1 : tile.z;
  if (pos0 < 0) {                                  // rows of a finished sequence: zeros
    if (misplaced && tid == 0) atomicCAS(status, 0, 19);
    if (!misplaced) {
      pdl_wait();                                  // the rows may still be read by a kernel ahead
      for (int i = tid; i < n_rows * D; i += kFaThreads) {
        const int r = i / D, d = i % D;
        out[((size_t)(t_first + r / group) * n_q_heads + kv_head * group + r % group) * D + d] =
            __float2bfloat16_rn(0.f);
      }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) tmem_dealloc(tmem_base, kTmemCols);
    return;
  }
  const int* table = block_table + (size_t)tile.w * table_stride;
  const int hi_tile = pos0 + n_tok - 1;
  const int lo_tile = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int kt_lo = lo_tile / kFaKeys, kt_hi = hi_tile / kFaKeys;
  const int n_iter = kt_hi - kt_lo + 1;
  pdl_wait();                                      // Q and the newest keys and values: the kernel ahead

  bool ok = true;
  if (tid == 128) {
    // ------------------------------------------------------------------- TMA producer
    // Rows of Q past this tile's tokens are the next sequence's or zeros (past the last token);
    // they make rows of S and O that nobody stores.
    mbar_expect_tx(bar(kBarQFull), DB * 2 * kSub);
#pragma unroll
    for (int j = 0; j < DB; ++j)
      tma_load_3d(smem_u32(q_s + j * 2 * kSub), &map_q, 64 * j, kv_head * group, t_first, bar(kBarQFull));
    for (int it = 0; it < n_iter; ++it) {
      const int ks = it % kFaKStages, vs = it % kFaVStages;
      const uint32_t k_phase = (it / kFaKStages) & 1, v_phase = (it / kFaVStages) & 1;
      const int row = (table[kt_lo + it] * n_kv_heads + kv_head) * kFaKeys;
      ok = mbar_wait(bar(kBarKEmpty + ks), k_phase ^ 1, status, 11);
      if (!ok) break;
      mbar_expect_tx(bar(kBarKFull + ks), DB * kSub);
#pragma unroll
      for (int j = 0; j < DB; ++j)
        tma_load_2d(smem_u32(k_s + (ks * DB + j) * kSub), &map_k, 64 * j, row, bar(kBarKFull + ks));
      ok = mbar_wait(bar(kBarVEmpty + vs), v_phase ^ 1, status, 12);
      if (!ok) break;
      mbar_expect_tx(bar(kBarVFull + vs), DB * kSub);
#pragma unroll
      for (int j = 0; j < DB; ++j)
        tma_load_2d(smem_u32(v_s + (vs * DB + j) * kSub), &map_v, 64 * j, row, bar(kBarVFull + vs));
    }
  } else if (tid == 160) {
    // ------------------------------------------------------------------- issuer of S = Q.K^T
    // Its own thread: every wait and commit costs this thread a few hundred cycles, and one
    // thread issuing both kinds of MMA spent 2,000 cycles a page, more than the softmax needs.
    constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kFaKeys >> 3) << 17) |
                                 ((uint32_t)(kFaRows >> 4) << 24);
    ok = mbar_wait(bar(kBarQFull), 0, status, 20);
    for (int it = 0; it < n_iter && ok; ++it) {
      const int s = it & 1;
      const int ks = it % kFaKStages;
      ok = mbar_wait(bar(kBarKFull + ks), (it / kFaKStages) & 1, status, 21);
      // S buffer s still holds the P of page it-2 until that page's P.V is done (the other
      // issuer's MMAs are not ordered against this one's)
      if (ok && it >= 2) ok = mbar_wait(bar(kBarPvDone + s), ((it - 2) >> 1) & 1, status, 22);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int j = 0; j < DB; ++j) {
        const uint64_t dq = smem_desc_k_sw128(smem_u32(q_s + j * 2 * kSub));
        const uint64_t dk = smem_desc_k_sw128(smem_u32(k_s + (ks * DB + j) * kSub));
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma(tmem_base + kColS + 64 * s, dq + (uint64_t)(2 * k), dk + (uint64_t)(2 * k), idesc_s,
                 (j | k) ? 1u : 0u);
      }
      tc_commit(bar(kBarKEmpty + ks));             // the K stage is free when these are done
      tc_commit(bar(kBarSFull + s));               // S is complete
    }
  } else if (tid == 192) {
    // ------------------------------------------------------------------- issuer of O += P.V
    constexpr uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                  ((uint32_t)(D >> 3) << 17) | ((uint32_t)(kFaRows >> 4) << 24);
    for (int u = 0; u < n_iter; ++u) {
      const int s = u & 1;
      const int vs = u % kFaVStages;
      ok = mbar_wait(bar(kBarPFull + s), (u >> 1) & 1, status, 23);   // P written (O rescaled)
      if (ok) ok = mbar_wait(bar(kBarVFull + vs), (u / kFaVStages) & 1, status, 24);   // V landed
      if (!ok) break;
      tc_fence_after();
      const uint64_t dv = smem_desc_mn_sw128(smem_u32(v_s + vs * DB * kSub), kSub, 1024);
#pragma unroll
      for (int k = 0; k < 4; ++k)                  // 16 keys a step: 8 columns of P,
        tc_mma_ts(tmem_base + kColO, tmem_base + kColS + 64 * s + 8 * k, dv + (uint64_t)(128 * k),
                  idesc_pv, (u | k) ? 1u : 0u);    // 16 rows (2048 bytes) down V
      tc_commit(bar(kBarVEmpty + vs));             // the V stage is free
      tc_commit(bar(kBarPvDone + s));              // O holds pages 0..u
    }
  }

  // ------------------------------------------------------------------------ softmax rows
  constexpr float kLazy = 8.f;                     // raise the reference maximum above 2^8 only
  float m_ref = -INFINITY, l_run = 0.f;            // the reference is in units of log2(e)/scale
  const int r = tid;                               // row = TMEM lane (softmax threads)
  const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
  if (tid < kFaRows) {
    const int pos_r = pos0 + min(r / group, n_tok - 1);
    for (int it = 0; it < n_iter && ok; ++it) {
      const int s = it & 1;
      const uint32_t phase = (it >> 1) & 1;
      const int key0 = (kt_lo + it) * kFaKeys;
      ok = mbar_wait(bar(kBarSFull + s), phase, status, 31);
      if (!ok) break;
      tc_fence_after();
      // Two passes over the 64 scores keep the registers of this thread under the limit that
      // two blocks of 7 warps an SM set: first the maximum (keys 32..63 are only looked at,
      // keys 0..31 stay in registers), then the exponentials of keys 0..31, their P, and the
      // same for keys 32..63, read from TMEM once more.
      const bool full = key0 + kFaKeys - 1 <= pos_r && (window <= 0 || key0 > pos_r - window);
      auto load_half = [&](int h, float* v) {      // scores of keys key0 + 32 h .., masked
        tmem_ld32_nowait(lane_addr + kColS + 64 * s + 32 * h, v);
        tmem_ld_wait();
        if (!full) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = key0 + 32 * h + i;
            const bool seen = key <= pos_r && (window <= 0 || key > pos_r - window);
            v[i] = seen ? v[i] : -INFINITY;
          }
        }
      };
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // of the raw scores
      float sc[32];                                // (the scale is positive)
      load_half(1, sc);
#pragma unroll
      for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], sc[i]);
      load_half(0, sc);
#pragma unroll
      for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], sc[i]);
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
      // tcgen05.ld/st are warp-wide: if any row of the warp raises its reference, the whole warp
      // rescales (rows that keep theirs multiply by 1)
      const bool raise = mx > m_ref + kLazy;       // also the first page with a visible key
      const float alpha = raise ? ex2_approx(m_ref - mx) : 1.f;   // 0 while the reference is -inf
      if (it > 0 && __any_sync(0xffffffffu, raise)) {
        // O holds pages 0..it-1 once their last P.V is done
        const int u = it - 1;
        ok = mbar_wait(bar(kBarPvDone + (u & 1)), (u >> 1) & 1, status, 34);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          float v[32];
          tmem_ld32_nowait(lane_addr + kColO + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] *= alpha;
          tmem_st32(lane_addr + kColO + c, v);
        }
      }
      if (raise) {
        l_run *= alpha;
        m_ref = mx;
      }
      const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
      const float2 scale2 = make_float2(scale_log2, scale_log2), shift2 = make_float2(neg_m, neg_m);
      float2 psum[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      // P over the scores it came from: 32 keys are 16 columns; the first store is under way
      // while the second half is read again and computed
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (h == 1) load_half(1, sc);              // columns 32..63: untouched by the P of keys 0..31
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 a = fma2(make_float2(sc[i], sc[i + 1]), scale2, shift2);
          const float2 p = make_float2(ex2_approx(a.x), ex2_approx(a.y));
          psum[(i >> 1) & 1] = add2(psum[(i >> 1) & 1], p);
          __nv_bfloat162 hh = __floats2bfloat162_rn(p.x, p.y);
          w[i / 2] = *reinterpret_cast<uint32_t*>(&hh);
        }
        tmem_st16(lane_addr + kColS + 64 * s + 16 * h, w);
      }
      l_run += (psum[0].x + psum[0].y) + (psum[1].x + psum[1].y);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarPFull + s));   // P (and any rescale of O) is in place
    }
    if (ok) {                                      // the last P.V
      const int u = n_iter - 1;
      ok = mbar_wait(bar(kBarPvDone + (u & 1)), (u >> 1) & 1, status, 36);
      tc_fence_after();
    }
  }

  const int failed = __syncthreads_or(ok ? 0 : 1);
  if (!failed) {
    if (tid < kFaRows) {                           // whole warps: tcgen05.ld is warp-wide
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const bool wide_out = ((uintptr_t)out & 31) == 0;     // rows of D values are then 32-byte aligned
      const int row = min(r, n_rows - 1);
      bf16* o = out + ((size_t)(t_first + row / group) * n_q_heads + kv_head * group + row % group) * D;
#pragma unroll
      for (int c = 0; c < D; c += 32) {
        float v[32];
        tmem_ld32_nowait(lane_addr + kColO + c, v);
        tmem_ld_wait();
        if (r < n_rows) {
#pragma unroll
          for (int j = 0; j < 32; j += 16) {     // 32 bytes a store: whole sectors of L2, a row a lane
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              __nv_bfloat162 h = __floats2bfloat162_rn(v[j + 2 * i] * inv, v[j + 2 * i + 1] * inv);
              w[i] = *reinterpret_cast<uint32_t*>(&h);
            }
            if (wide_out) {
              asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(o + c + j), "r"(w[0]),
                           "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
            } else {
              *reinterpret_cast<uint4*>(o + c + j) = make_uint4(w[0], w[1], w[2], w[3]);
              *reinterpret_cast<uint4*>(o + c + j + 8) = make_uint4(w[4], w[5], w[6], w[7]);
            }
          }
        }
      }
    }
  } else {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // let copies in flight land
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, kTmemCols);
}

// The table of tiles of a prompt step: entry = (first token, tokens, position of the first token,
// slot), `tok_per_tile` consecutive new tokens of one sequence each.  The sequences are taken by the
// length of their context, longest first, and put into bands of at most `band_tokens` tokens of
// context (at least one sequence a band); the bands stand one after another, and inside a band the
// tiles are listed by their place in their sequence, last places (the longest key ranges) first,
// over the band's sequences.  So the blocks that run together read the keys and values of one band,
// which the caller sizes to stay in L2 (with all sequences interleaved, 16 prompts of 7,936 tokens
// read 520 MB of keys and values a layer over and over from memory: 6.0 ms a layer against 4.2),
// the blocks that run longest start first and the short ones fill the gaps at the end.
// Entries past the last tile have 0 tokens.  One block (a step has at most a few hundred sequences).
constexpr int kFaTileThreads = 1024;         // also the most sequences a step may bring

__global__ void __launch_bounds__(kFaTileThreads)
attention_prefill_tiles_kernel(int4* tiles, int max_tiles, const int* cu_seqlens, const int* positions,
                               const int* token_slot, int n_seqs, int tok_per_tile, int band_tokens) {
  __shared__ int count_s[kFaTileThreads], start_s[kFaTileThreads], len_s[kFaTileThreads],
      context_s[kFaTileThreads];
  __shared__ int by_rank_s[kFaTileThreads];                  // the sequence that stands r-th
  __shared__ int rank_s[kFaTileThreads];                     // where a sequence stands
  __shared__ int band_first_s[kFaTileThreads], band_end_s[kFaTileThreads];   // by rank: its band's ranks [first, end)
  __shared__ int band_at_s[kFaTileThreads];                  // by rank: tiles of the bands before its band
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  if (tid < n_seqs) {
    const int a = cu_seqlens[tid], n = cu_seqlens[tid + 1] - a;
    start_s[tid] = a;
    len_s[tid] = n;
    count_s[tid] = (n + tok_per_tile - 1) / tok_per_tile;
    context_s[tid] = n > 0 ? positions[a] + n : 0;
  }
  __syncthreads();
  if (tid < n_seqs) {
    int rank = 0;                              // longer context first, ties as listed
    for (int c = 0; c < n_seqs; ++c)
      rank += (context_s[c] > context_s[tid] || (context_s[c] == context_s[tid] && c < tid)) ? 1 : 0;
    rank_s[tid] = rank;
    by_rank_s[rank] = tid;
  }
  __syncthreads();
  if (tid == 0) {
    int first = 0, held = 0, at = 0, tiles_in_band = 0;
    for (int r = 0; r <= n_seqs; ++r) {
      const int ctx = r < n_seqs ? context_s[by_rank_s[r]] : 0;
      if (r == n_seqs || (r > first && held + ctx > band_tokens)) {     // the band [first, r) is closed
        for (int q = first; q < r; ++q) {
          band_first_s[q] = first;
          band_end_s[q] = r;
          band_at_s[q] = at;
        }
        at += tiles_in_band;
        first = r;
        held = 0;
        tiles_in_band = 0;
      }
      if (r < n_seqs) {
        held += ctx;
        tiles_in_band += count_s[by_rank_s[r]];
      }
    }
  }
  int most = 0, total = 0;
  for (int b = 0; b < n_seqs; ++b) {
    most = max(most, count_s[b]);
    total += count_s[b];
  }
  __syncthreads();
  // inside its band, tile r of a sequence stands behind every tile with a later place r' > r and
  // behind the tiles with the same place of the band's sequences before it
  for (int p = tid; p < most * n_seqs; p += kFaTileThreads) {
    const int r = p / n_seqs, b = p % n_seqs;
    if (r >= count_s[b]) continue;
    const int mine = rank_s[b];
    int at = band_at_s[mine];
    for (int q = band_first_s[mine]; q < band_end_s[mine]; ++q) {
      const int n = count_s[by_rank_s[q]];
      at += max(0, n - 1 - r) + (q < mine && n > r ? 1 : 0);
    }
    if (at < max_tiles) {
      const int first = start_s[b] + r * tok_per_tile;
      tiles[at] = make_int4(first, min(tok_per_tile, len_s[b] - r * tok_per_tile), positions[first],
                            token_slot[first]);
    }
  }
  for (int i = total + tid; i < max_tiles; i += kFaTileThreads) tiles[i] = make_int4(0, 0, -1, 0);
}

template <int D>
static int launch_fa(bf16* out, const bf16* q, int q_row_stride, const int4* tiles, int n_tiles, int n_tokens,
                     const void* k_pages, const void* v_pages, long long page_rows,
                     const int* block_table, int table_stride, int n_q_heads, int n_kv_heads,
                     float scale, int window, int* status, cudaStream_t stream) {
  const int group = n_q_heads / n_kv_heads;
  const int tok_per_tile = kFaRows / group;
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = tensor_map_heads(q, n_tokens, n_q_heads, D, q_row_stride, group, tok_per_tile, &mq))) return rc;
  if ((rc = tensor_map(k_pages, page_rows, D, D, kFaKeys, &mk))) return rc;
  if ((rc = tensor_map(v_pages, page_rows, D, D, kFaKeys, &mv))) return rc;
  constexpr int DB = D / 64;
  constexpr size_t smem = (size_t)(2 * DB + (kFaKStages + kFaVStages) * DB) * kFaKeys * 128 + kFaBars * 8 + 16;
  auto kernel = attention_prefill_tc_kernel<D>;
  static bool configured[kMaxDevices] = {};
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= kMaxDevices) return EK_ERR_ARG;
  if (!configured[device]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured[device] = true;
  }
  prefer_carveout((const void*)kernel, 100);
  if (n_tiles > 65535) return EK_ERR_ARG;
  dim3 grid(n_kv_heads, n_tiles);
  return (int)launch_pdl(kernel, grid, dim3(kFaThreads), smem, stream, out, mq, tiles, mk, mv, block_table,
                         table_stride, n_kv_heads, n_q_heads, scale * 1.4426950408889634f, window,
                         tok_per_tile, status);
}

}  // namespace ek

// The table of tiles that ek_attention_prefill_tc walks, for one step's sequences: `tiles` holds
// `max_tiles` >= ceil(n_tokens / tok_per_tile) + n_seqs entries of 4 ints; tok_per_tile is
// 128 / (query heads per KV head); band_tokens is the context (tokens) whose keys and values of one
// layer should stay in L2 together.  Made once per step, used by every layer.
EK_EXPORT int ek_attention_prefill_tiles(int* tiles, int max_tiles, const int* cu_seqlens,
                                         const int* positions, const int* token_slot, int n_seqs,
                                         int tok_per_tile, int band_tokens, cudaStream_t stream) {
  using namespace ek;
  if (n_seqs <= 0 || max_tiles <= 0) return 0;
  if (n_seqs > kFaTileThreads || tok_per_tile <= 0 || band_tokens <= 0 || !tiles || ((uintptr_t)tiles & 15))
    return EK_ERR_ARG;
  return (int)launch_pdl(attention_prefill_tiles_kernel, dim3(1), dim3(kFaTileThreads), 0, stream, (int4*)tiles,
                         max_tiles, cu_seqlens, positions, token_slot, n_seqs, tok_per_tile, band_tokens);
}

// head_dim 64 or 128; the group (query heads per KV head) must divide 128; q rows 16-byte
// aligned; n_pages = number of pages in k_pages / v_pages ([pages, kv heads, 64, head_dim]);
// `tiles` / n_tiles: the table ek_attention_prefill_tiles made for this step and group size.
EK_EXPORT int ek_attention_prefill_tc(void* out, const void* q, int q_row_stride, const int* tiles,
                                      int n_tiles, int n_tokens,
                                      const void* k_pages, const void* v_pages, int n_pages,
                                      const int* block_table, int table_stride, int n_q_heads,
                                      int n_kv_heads, int head_dim, float scale, int window,
                                      int* status, cudaStream_t stream) {
  using namespace ek;
  if (n_tokens <= 0 || n_tiles <= 0) return 0;
  if ((head_dim != 64 && head_dim != 128) || n_kv_heads <= 0 || n_q_heads % n_kv_heads ||
      kFaRows % (n_q_heads / n_kv_heads) || q_row_stride % 8 || ((uintptr_t)q & 15) || !status ||
      !(scale > 0.f) || n_pages <= 0 || !tiles || ((uintptr_t)tiles & 15))
    return EK_ERR_ARG;
  const long long page_rows = (long long)n_pages * n_kv_heads * EK_PAGE;
  if (head_dim == 64)
    return launch_fa<64>((bf16*)out, (const bf16*)q, q_row_stride, (const int4*)tiles, n_tiles, n_tokens,
                         k_pages, v_pages, page_rows, block_table, table_stride,
                         n_q_heads, n_kv_heads, scale, window, status, stream);
  return launch_fa<128>((bf16*)out, (const bf16*)q, q_row_stride, (const int4*)tiles, n_tiles, n_tokens,
                        k_pages, v_pages, page_rows, block_table, table_stride,
                        n_q_heads, n_kv_heads, scale, window, status, stream);
}
