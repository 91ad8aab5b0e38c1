// Causal attention for prompts (and any run of several new tokens) in bfloat16, over
// the paged cache: a flash-attention kernel with online softmax, built on
// mma.sync.m16n8k16 with operands staged in shared memory by cp.async.
//
// Work decomposition, chosen for grouped-query attention on a paged cache:
//   * a block owns a tile of consecutive new tokens of ONE sequence and ONE KV head; the
//     128 rows of its score tile are (token, query head of the group) pairs, so a K/V
//     page is fetched once for all heads of the group;
//   * keys and values are read from the cache pages, which already hold this step's
//     tokens, so a prompt cut into pieces, or appended to an earlier part, is the same
//     code: a row at position p sees keys [max(0, p - window + 1), p];
//   * one cache page (64 keys) is one key tile; K and V tiles are double-buffered.
// Tiles are found from cu_seqlens on the device (no host-built schedule).
// The reference's counterpart is a Triton kernel over a padded rectangle, 128x128 tiles,
// probabilities rounded to bfloat16 before P.V as here (engine/ek_kernels.py:166-221),
// or cuDNN's fused attention (engine/ek_model.py:268-278).
#include "common.cuh"

namespace ek {

constexpr int kPfWarps = 8;
constexpr int kPfRows = kPfWarps * 16;       // 128 rows per block
constexpr int kPfKeys = EK_PAGE;             // 64 keys per tile

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t r[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t r[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// grid (tiles upper bound, kv heads).  tok_per_tile = max(1, 128 / group).
template <int DMAX>
__global__ void __launch_bounds__(kPfWarps * 32, 1)
attention_prefill_bf16_kernel(bf16* __restrict__ out, const bf16* __restrict__ q, int q_row_stride,
                              const int* __restrict__ positions, const int* __restrict__ token_slot,
                              const int* __restrict__ cu_seqlens, int n_seqs, PagedKV cache,
                              int n_q_heads, float scale_log2, int window, int tok_per_tile) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int tile_info[3];                 // first token (packed index), tokens, sequence
  const int D = cache.head_dim;
  const int LD = D + 8;                        // padded row length (elements): no bank conflicts
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);            // [128][LD]
  bf16* k_s = q_s + kPfRows * LD;                           // [2][64][LD]
  bf16* v_s = k_s + 2 * kPfKeys * LD;                       // [2][64][LD]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int kv_head = blockIdx.x;             // heads fastest: longest key ranges start first
  const int group = n_q_heads / cache.heads;

  if (tid == 0) {
    int idx = blockIdx.y, found = -1, first = 0, count = 0;
    for (int b = 0; b < n_seqs; ++b) {
      const int n = cu_seqlens[b + 1] - cu_seqlens[b];
      const int tiles = (n + tok_per_tile - 1) / tok_per_tile;
      if (idx < tiles) {
        const int tile = tiles - 1 - idx;      // long key ranges first
        found = b;
        first = cu_seqlens[b] + tile * tok_per_tile;
        count = min(tok_per_tile, n - tile * tok_per_tile);
        break;
      }
      idx -= tiles;
    }
    tile_info[0] = first; tile_info[1] = count; tile_info[2] = found;
  }
  __syncthreads();
  if (tile_info[2] < 0) return;
  const int t_first = tile_info[0], n_tok = tile_info[1];
  const int pos0 = positions[t_first];
  const int n_rows = n_tok * group;            // real rows (<= 128)
  if (pos0 < 0) {                              // rows of a finished sequence: zeros
    for (int i = tid; i < n_rows * D; i += blockDim.x) {
      const int r = i / D, d = i % D;
      out[((size_t)(t_first + r / group) * n_q_heads + kv_head * group + r % group) * D + d] =
          __float2bfloat16_rn(0.f);
    }
    return;
  }
  const int slot = token_slot[t_first];
  const int* table = cache.block_table + (size_t)slot * cache.table_stride;
  const int hi_tile = pos0 + n_tok - 1;
  const int lo_tile = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int kt_lo = lo_tile / kPfKeys, kt_hi = hi_tile / kPfKeys;
  const int chunks = D / 8;                    // 16-byte pieces per row

  // ---- stage Q (rows beyond the real ones are zero) and the first K/V tile ---------------
  for (int i = tid; i < kPfRows * chunks; i += blockDim.x) {
    const int r = i / chunks, c = i % chunks;
    bf16* dst = q_s + r * LD + c * 8;
    if (r < n_rows) {
      const bf16* src = q + (size_t)(t_first + r / group) * q_row_stride +
                        (size_t)(kv_head * group + r % group) * D + c * 8;
      cp_async16(dst, src);
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
  }
  auto load_kv = [&](int kt, int buf) {
    const int page = table[kt];
    const size_t base = ((size_t)page * cache.heads + kv_head) * EK_PAGE * (size_t)D;
    const bf16* ksrc = (const bf16*)cache.k + base;
    const bf16* vsrc = (const bf16*)cache.v + base;
    bf16* kd = k_s + buf * kPfKeys * LD;
    bf16* vd = v_s + buf * kPfKeys * LD;
    for (int i = tid; i < kPfKeys * chunks; i += blockDim.x) {
      const int r = i / chunks, c = i % chunks;
      cp_async16(kd + r * LD + c * 8, ksrc + (size_t)r * D + c * 8);
      cp_async16(vd + r * LD + c * 8, vsrc + (size_t)r * D + c * 8);
    }
  };
  load_kv(kt_lo, 0);
  cp_async_commit();

  // ---- per-thread state --------------------------------------------------------------------
  float o_acc[DMAX / 8][4];
#pragma unroll
  for (int i = 0; i < DMAX / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  // rows of this thread: warp*16 + g and + 8; their positions
  const int row_lo = warp * 16 + g, row_hi = row_lo + 8;
  const int pos_lo = pos0 + row_lo / group, pos_hi = pos0 + row_hi / group;
  const int warp_pos_min = pos0 + (warp * 16) / group;
  const int warp_pos_max = pos0 + min((warp * 16 + 15) / group, n_tok - 1);
  const bool warp_active = warp * 16 < n_rows;

  for (int kt = kt_lo; kt <= kt_hi; ++kt) {
    const int buf = (kt - kt_lo) & 1;
    if (kt + 1 <= kt_hi) load_kv(kt + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();                        // tile kt (and Q) have landed
    __syncthreads();

    const int key0 = kt * kPfKeys;
    // a warp skips tiles none of its rows can see
    const bool tile_visible = warp_active && key0 <= warp_pos_max &&
                              (window <= 0 || key0 + kPfKeys - 1 > warp_pos_min - window);
    if (tile_visible) {
      const bf16* kb = k_s + buf * kPfKeys * LD;
      const bf16* vb = v_s + buf * kPfKeys * LD;
      float s[kPfKeys / 8][4];
#pragma unroll
      for (int j = 0; j < kPfKeys / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < DMAX / 16; ++kk) {
        if (kk * 16 < D) {
          uint32_t a[4];
          ldmatrix_x4(a, q_s + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + kk * 16 +
                             (lane >> 4) * 8);
#pragma unroll
          for (int jp = 0; jp < kPfKeys / 16; ++jp) {
            uint32_t b[4];
            ldmatrix_x4(b, kb + (jp * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + kk * 16 +
                               ((lane >> 3) & 1) * 8);
            mma_16816(s[2 * jp], a, b[0], b[1]);
            mma_16816(s[2 * jp + 1], a, b[2], b[3]);
          }
        }
      }
      // scale and mask.  s[j][e]: row (e < 2 ? lo : hi), key key0 + 8j + 2tq + (e & 1)
      const bool need_mask = key0 + kPfKeys - 1 > warp_pos_min ||
                             (window > 0 && key0 <= warp_pos_max - window);
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < kPfKeys / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[j][e] * scale_log2;
          if (need_mask) {
            const int key = key0 + 8 * j + 2 * tq + (e & 1);
            const int p = e < 2 ? pos_lo : pos_hi;
            if (key > p || (window > 0 && key <= p - window)) v = -INFINITY;
          }
          s[j][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      float alpha[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[r], mx[r]);
        // a row that sees no key of this tile and none before keeps -inf: use 0 to avoid inf - inf
        m_use[r] = m_new == -INFINITY ? 0.f : m_new;
        alpha[r] = exp2f(m_run[r] - m_use[r]);
        m_run[r] = m_new;
      }
      float psum[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < kPfKeys / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = exp2f(s[j][e] - m_use[e >> 1]);
          s[j][e] = p;
          psum[e >> 1] += p;
        }
      l_run[0] = l_run[0] * alpha[0] + psum[0];
      l_run[1] = l_run[1] * alpha[1] + psum[1];
#pragma unroll
      for (int i = 0; i < DMAX / 8; ++i) {
        o_acc[i][0] *= alpha[0]; o_acc[i][1] *= alpha[0];
        o_acc[i][2] *= alpha[1]; o_acc[i][3] *= alpha[1];
      }
      // O += P . V
#pragma unroll
      for (int ks = 0; ks < kPfKeys / 16; ++ks) {
        uint32_t a[4];
        a[0] = pack2(s[2 * ks][0], s[2 * ks][1]);
        a[1] = pack2(s[2 * ks][2], s[2 * ks][3]);
        a[2] = pack2(s[2 * ks + 1][0], s[2 * ks + 1][1]);
        a[3] = pack2(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
        for (int dp = 0; dp < DMAX / 16; ++dp) {
          if (dp * 16 < D) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, vb + (ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LD + dp * 16 +
                                     (lane >> 4) * 8);
            mma_16816(o_acc[2 * dp], a, b[0], b[1]);
            mma_16816(o_acc[2 * dp + 1], a, b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();                           // everyone is done with buffer `buf`
  }
  cp_async_wait<0>();

  // ---- normalise and store --------------------------------------------------------------------
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  const float inv_lo = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f;
  const float inv_hi = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
#pragma unroll
  for (int i = 0; i < DMAX / 8; ++i) {
    const int d = 8 * i + 2 * tq;
    if (d < D) {
      if (row_lo < n_rows) {
        bf16* o = out + ((size_t)(t_first + row_lo / group) * n_q_heads + kv_head * group +
                         row_lo % group) * D + d;
        *reinterpret_cast<uint32_t*>(o) = pack2(o_acc[i][0] * inv_lo, o_acc[i][1] * inv_lo);
      }
      if (row_hi < n_rows) {
        bf16* o = out + ((size_t)(t_first + row_hi / group) * n_q_heads + kv_head * group +
                         row_hi % group) * D + d;
        *reinterpret_cast<uint32_t*>(o) = pack2(o_acc[i][2] * inv_hi, o_acc[i][3] * inv_hi);
      }
    }
  }
}

template <int DMAX>
static int launch_dmax(bf16* out, const bf16* q, int q_row_stride, const int* positions,
                       const int* token_slot, const int* cu_seqlens, int n_seqs, int n_tokens,
                       PagedKV cache, int n_q_heads, float scale, int window, cudaStream_t stream) {
  const int group = n_q_heads / cache.heads;
  const int tok_per_tile = kPfRows / group;
  const int D = cache.head_dim, LD = D + 8;
  const size_t smem = (size_t)(kPfRows + 4 * kPfKeys) * LD * sizeof(bf16);
  cudaError_t e = cudaFuncSetAttribute(attention_prefill_bf16_kernel<DMAX>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  prefer_carveout((const void*)attention_prefill_bf16_kernel<DMAX>, 100);
  const int tiles = (n_tokens + tok_per_tile - 1) / tok_per_tile + n_seqs;   // upper bound
  dim3 grid(cache.heads, tiles);
  if (tiles > 65535) return EK_ERR_ARG;
  attention_prefill_bf16_kernel<DMAX><<<grid, kPfWarps * 32, smem, stream>>>(
      out, q, q_row_stride, positions, token_slot, cu_seqlens, n_seqs, cache, n_q_heads,
      scale * 1.4426950408889634f, window, tok_per_tile);
  EK_RETURN_LAUNCH_STATUS();
}

}  // namespace ek

// head_dim a multiple of 16 up to 256; the group (query heads per KV head) at most 128.
// Tokens of a sequence must stand at consecutive positions in the step.
EK_EXPORT int ek_attention_prefill_bf16(void* out, const void* q, int q_row_stride,
                                        const int* positions, const int* token_slot,
                                        const int* cu_seqlens, int n_seqs, int n_tokens,
                                        const void* k_pages, const void* v_pages,
                                        const int* block_table, int table_stride, int n_q_heads,
                                        int n_kv_heads, int head_dim, float scale, int window,
                                        cudaStream_t stream) {
  using namespace ek;
  if (n_tokens <= 0 || n_seqs <= 0) return 0;
  if (head_dim % 16 || head_dim < 16 || head_dim > 256 || n_kv_heads <= 0 ||
      n_q_heads % n_kv_heads || n_q_heads / n_kv_heads > kPfRows || q_row_stride % 8)
    return EK_ERR_ARG;
  PagedKV cache{(void*)k_pages, (void*)v_pages, block_table, table_stride, n_kv_heads, head_dim};
  if (head_dim <= 64)
    return launch_dmax<64>((bf16*)out, (const bf16*)q, q_row_stride, positions, token_slot,
                           cu_seqlens, n_seqs, n_tokens, cache, n_q_heads, scale, window, stream);
  if (head_dim <= 128)
    return launch_dmax<128>((bf16*)out, (const bf16*)q, q_row_stride, positions, token_slot,
                            cu_seqlens, n_seqs, n_tokens, cache, n_q_heads, scale, window, stream);
  return launch_dmax<256>((bf16*)out, (const bf16*)q, q_row_stride, positions, token_slot,
                          cu_seqlens, n_seqs, n_tokens, cache, n_q_heads, scale, window, stream);
}
