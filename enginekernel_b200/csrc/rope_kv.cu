// Per-head RMSNorm of queries and keys, rotary position encoding, and the write of
// keys and values into the paged cache - one pass over the fused q/k/v rows.
//
// Same work as the reference's _qk_norm_rope_kv_kernel (engine/ek_kernels.py:223-279):
// normalise each head over its dimension, rotate pairs (j, j + rot/2) by the angle of
// the token's position (NeoX pairing, engine/ek_model.py:164-174), leave values
// untouched, store keys and values at the token's place in its sequence's cache.
// Differences: positions and slots come per token (no padded rectangle), the cache is
// paged, and all arithmetic is 32-bit with one rounding at the end.
#include "common.cuh"

namespace ek {

constexpr int kRopeWarps = 4;


template <typename T>
__global__ void qk_norm_rope_kv_kernel(T* qkv, int row_stride,
                                       const float* __restrict__ q_gain,
                                       const float* __restrict__ k_gain,
                                       const float* __restrict__ cos_tab,
                                       const float* __restrict__ sin_tab, int rot_dim,
                                       const int* positions, const int* token_slot,
                                       PagedKV cache,
                                       int n_q_heads, float eps, int write_kv) {
  __shared__ __align__(16) float buf[kRopeWarps][EK_MAX_HEAD_DIM];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y * kRopeWarps + warp;
  const int n_kv = cache.heads, d = cache.head_dim;
  if (head >= n_q_heads + 2 * n_kv) return;
  const int pos = positions[t];
  if (pos < 0) return;                        // a row of a finished sequence
  const bool is_q = head < n_q_heads;
  const bool is_k = !is_q && head < n_q_heads + n_kv;
  if (!is_q && !write_kv) return;

  T* src = qkv + (size_t)t * row_stride + (size_t)head * d;
  T* dst = src;
  if (!is_q) {
    const int slot = token_slot[t];
    const int page = cache.block_table[(size_t)slot * cache.table_stride + pos / EK_PAGE];
    const int kv_head = is_k ? head - n_q_heads : head - n_q_heads - n_kv;
    dst = (T*)(is_k ? cache.k : cache.v) + page_offset(cache, page, kv_head, pos);
  }

  // Four neighbouring dimensions a lane when the sizes allow (head size a multiple of 4 and
  // the rotated half a multiple of 4), else one.
  const bool vec = (d % 4 == 0) && (rot_dim % 8 == 0) && (row_stride % 4 == 0);
  if (!is_q && !is_k) {                       // values: a copy
    if (vec) {
      for (int i = lane * 4; i < d; i += 128) Vec4<T>::store(dst + i, Vec4<T>::load(src + i));
    } else {
      for (int i = lane; i < d; i += 32) dst[i] = src[i];
    }
    return;
  }

  const float* gain = is_q ? q_gain : k_gain;
  float ss = 0.f;
  if (vec) {
    for (int i = lane * 4; i < d; i += 128) {
      const float4 v = Vec4<T>::load(src + i);
      *reinterpret_cast<float4*>(&buf[warp][i]) = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int i = lane; i < d; i += 32) {
      const float v = to_f<T>(src[i]);
      buf[warp][i] = v;
      ss += v * v;
    }
  }
  float rstd = 1.f;
  if (gain) {
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / (float)d + eps);
  }
  __syncwarp();
  const int half = rot_dim >> 1;
  const float* cs = cos_tab + (size_t)pos * half;
  const float* sn = sin_tab + (size_t)pos * half;
  auto rotated = [&](int i) {
    const float g = gain ? gain[i] : 1.f;
    const float x = buf[warp][i] * rstd * g;
    if (i < half) {
      const float partner = buf[warp][i + half] * rstd * (gain ? gain[i + half] : 1.f);
      return x * cs[i] - partner * sn[i];
    }
    if (i < rot_dim) {
      const int j = i - half;
      const float partner = buf[warp][j] * rstd * (gain ? gain[j] : 1.f);
      return x * cs[j] + partner * sn[j];
    }
    return x;
  };
  if (vec) {
    for (int i = lane * 4; i < d; i += 128)
      Vec4<T>::store(dst + i, make_float4(rotated(i), rotated(i + 1), rotated(i + 2), rotated(i + 3)));
  } else {
    for (int i = lane; i < d; i += 32) dst[i] = from_f<T>(rotated(i));
  }
}

template <typename T>
static int launch(void* qkv, int row_stride, const float* q_gain, const float* k_gain,
                  const float* cos_tab, const float* sin_tab, int rot_dim, const int* positions,
                  const int* token_slot, void* k_pages, void* v_pages, const int* block_table,
                  int table_stride, int n_tokens, int n_q_heads, int n_kv_heads, int head_dim,
                  float eps, int write_kv, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (head_dim <= 0 || head_dim > EK_MAX_HEAD_DIM || (head_dim & 1) || rot_dim < 0 ||
      rot_dim > head_dim || (rot_dim & 1) || n_tokens > 2147483647 / 2)
    return EK_ERR_ARG;
  PagedKV cache{k_pages, v_pages, block_table, table_stride, n_kv_heads, head_dim};
  const int heads = n_q_heads + 2 * n_kv_heads;
  dim3 grid(n_tokens, (heads + kRopeWarps - 1) / kRopeWarps);
  return (int)launch_pdl(qk_norm_rope_kv_kernel<T>, grid, dim3(kRopeWarps * 32), 0, stream, (T*)qkv,
                         row_stride, q_gain, k_gain, cos_tab, sin_tab, rot_dim, positions,
                         token_slot, cache, n_q_heads, eps, write_kv);
}

}  // namespace ek

#define EK_INSTANTIATE(SUFFIX, T)                                                              \
  EK_EXPORT int ek_qk_norm_rope_kv_##SUFFIX(                                                    \
      void* qkv, int row_stride, const float* q_gain, const float* k_gain, const float* cos_tab, \
      const float* sin_tab, int rot_dim, const int* positions, const int* token_slot,          \
      void* k_pages, void* v_pages, const int* block_table, int table_stride, int n_tokens,    \
      int n_q_heads, int n_kv_heads, int head_dim, float eps, int write_kv,                    \
      cudaStream_t stream) {                                                                   \
    return ek::launch<T>(qkv, row_stride, q_gain, k_gain, cos_tab, sin_tab, rot_dim, positions, \
                         token_slot, k_pages, v_pages, block_table, table_stride, n_tokens,    \
                         n_q_heads, n_kv_heads, head_dim, eps, write_kv, stream);              \
  }

EK_INSTANTIATE(f32, float)
EK_INSTANTIATE(bf16, ek::bf16)
