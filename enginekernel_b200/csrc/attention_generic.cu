// Attention over the paged cache for any head size, head count and group size, in
// 32-bit or bfloat16 storage with 32-bit arithmetic throughout.  One block per
// (token, query head, key split) walks the keys the token may see:
//     lo = max(0, pos - window + 1) (window <= 0: 0)  ...  pos
// with a running maximum and sum (online softmax) so that no score row is stored.
// It serves whole prompts, chunks and single decoded tokens alike, since each token
// carries its own position and slot; the faster bfloat16 kernels in attention_bf16.cu
// cover the common head sizes, this one covers everything and is the 32-bit path.
//
// Formula: engine/ek_model.py:475-488 (scores q.k * scale in 32-bit, softmax in 32-bit,
// weighted sum of values in 32-bit); query head h reads KV head h / (heads / kv heads).
// Splitting the keys and merging partial (max, sum, accumulator) triples in split order
// is the reference's flash-decoding scheme (engine/ek_kernels.py:534-615, 988-1019).
#include "common.cuh"

namespace ek {

constexpr int kAttnThreads = 128;

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ row, const float* __restrict__ q, int d);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ row,
                                                const float* __restrict__ q, int d) {
  float s = 0.f;
  const float4* r4 = reinterpret_cast<const float4*>(row);
  for (int i = 0; i < d / 4; ++i) {
    const float4 v = r4[i];
    s += v.x * q[4 * i] + v.y * q[4 * i + 1] + v.z * q[4 * i + 2] + v.w * q[4 * i + 3];
  }
  return s;
}

template <>
__device__ __forceinline__ float dot_row<bf16>(const bf16* __restrict__ row,
                                               const float* __restrict__ q, int d) {
  float s = 0.f;
  const uint4* r4 = reinterpret_cast<const uint4*>(row);
  for (int i = 0; i < d / 8; ++i) {
    const uint4 v = r4[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      s += f.x * q[8 * i + 2 * j] + f.y * q[8 * i + 2 * j + 1];
    }
  }
  return s;
}

template <typename T>
__global__ void attention_generic_kernel(T* __restrict__ out, const T* __restrict__ q,
                                         int q_row_stride, const int* __restrict__ positions,
                                         const int* __restrict__ token_slot, PagedKV cache,
                                         int n_q_heads, float scale, int window, int n_splits,
                                         int keys_per_split, float* __restrict__ part_acc,
                                         float* __restrict__ part_ml) {
  __shared__ float q_s[EK_MAX_HEAD_DIM];
  __shared__ float p_s[kAttnThreads];
  __shared__ size_t voff_s[kAttnThreads];
  __shared__ float scratch[33];

  const int t = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x;
  const int d = cache.head_dim;
  const int kv_head = h / (n_q_heads / cache.heads);
  const int pos = positions[t];
  const size_t part_index = ((size_t)t * n_q_heads + h) * n_splits + split;

  int lo = 0, hi = -1;                          // keys [lo, hi]
  if (pos >= 0) {
    lo = window > 0 ? max(0, pos - window + 1) : 0;
    hi = pos;
    if (n_splits > 1) {
      lo = max(lo, split * keys_per_split);
      hi = min(hi, (split + 1) * keys_per_split - 1);
    }
  }

  float acc0 = 0.f, acc1 = 0.f;                 // dims tid and tid + 128
  float m = -INFINITY, l = 0.f;
  if (hi >= lo) {
    const int slot = token_slot[t];
    const int* table = cache.block_table + (size_t)slot * cache.table_stride;
    const T* qrow = q + (size_t)t * q_row_stride + (size_t)h * d;
    for (int i = tid; i < d; i += kAttnThreads) q_s[i] = to_f<T>(qrow[i]) * scale;
    __syncthreads();
    const T* kbase = (const T*)cache.k;
    const T* vbase = (const T*)cache.v;
    for (int start = lo; start <= hi; start += kAttnThreads) {
      const int j = start + tid;
      float s = -INFINITY;
      if (j <= hi) {
        const size_t off = page_offset(cache, table[j / EK_PAGE], kv_head, j);
        voff_s[tid] = off;
        s = dot_row<T>(kbase + off, q_s, d);
      }
      const float m_new = fmaxf(m, block_max(s, scratch));
      const float p = j <= hi ? expf(s - m_new) : 0.f;
      p_s[tid] = p;
      const float alpha = expf(m - m_new);      // m = -inf on the first chunk: 0
      l = l * alpha + block_sum(p, scratch);    // the barriers inside also publish p_s, voff_s
      m = m_new;
      const int n = min(kAttnThreads, hi - start + 1);
      acc0 *= alpha;
      acc1 *= alpha;
      if (tid < d) {
        for (int i = 0; i < n; ++i) acc0 += p_s[i] * to_f<T>(vbase[voff_s[i] + tid]);
      }
      if (tid + kAttnThreads < d) {
        for (int i = 0; i < n; ++i) acc1 += p_s[i] * to_f<T>(vbase[voff_s[i] + tid + kAttnThreads]);
      }
      __syncthreads();                          // before p_s / voff_s are overwritten
    }
  }

  if (n_splits == 1) {
    T* orow = out + ((size_t)t * n_q_heads + h) * d;
    const float inv = l > 0.f ? 1.f / l : 0.f;
    if (tid < d) orow[tid] = from_f<T>(acc0 * inv);
    if (tid + kAttnThreads < d) orow[tid + kAttnThreads] = from_f<T>(acc1 * inv);
  } else {
    float* pa = part_acc + part_index * d;
    if (tid < d) pa[tid] = acc0;
    if (tid + kAttnThreads < d) pa[tid + kAttnThreads] = acc1;
    if (tid == 0) {
      part_ml[2 * part_index] = m;
      part_ml[2 * part_index + 1] = l;
    }
  }
}

// Merge the partial results of the key splits in split order.
template <typename T>
__global__ void attention_combine_kernel(T* __restrict__ out, const float* __restrict__ part_acc,
                                         const float* __restrict__ part_ml, int n_q_heads,
                                         int head_dim, int n_splits) {
  const size_t th = (size_t)blockIdx.x * n_q_heads + blockIdx.y;
  const float* ml = part_ml + 2 * th * n_splits;
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, ml[2 * s]);
  float l = 0.f;
  for (int s = 0; s < n_splits; ++s)
    if (ml[2 * s + 1] > 0.f) l += ml[2 * s + 1] * expf(ml[2 * s] - m);
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int i = threadIdx.x; i < head_dim; i += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < n_splits; ++s)
      if (ml[2 * s + 1] > 0.f) acc += part_acc[(th * n_splits + s) * head_dim + i] * expf(ml[2 * s] - m);
    out[th * head_dim + i] = from_f<T>(acc * inv);
  }
}

template <typename T>
static int launch(void* out, const void* q, int q_row_stride, const int* positions,
                  const int* token_slot, const void* k_pages, const void* v_pages,
                  const int* block_table, int table_stride, int n_tokens, int n_q_heads,
                  int n_kv_heads, int head_dim, float scale, int window, int n_splits,
                  int keys_per_split, float* part_acc, float* part_ml, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (head_dim <= 0 || head_dim > EK_MAX_HEAD_DIM || head_dim % 8 || n_kv_heads <= 0 ||
      n_q_heads % n_kv_heads || n_q_heads > 65535 || n_splits < 1 || n_splits > 65535 ||
      (n_splits > 1 && (!part_acc || !part_ml || keys_per_split <= 0)))
    return EK_ERR_ARG;
  PagedKV cache{(void*)k_pages, (void*)v_pages, block_table, table_stride, n_kv_heads, head_dim};
  dim3 grid(n_tokens, n_q_heads, n_splits);
  attention_generic_kernel<T><<<grid, kAttnThreads, 0, stream>>>(
      (T*)out, (const T*)q, q_row_stride, positions, token_slot, cache, n_q_heads, scale, window,
      n_splits, keys_per_split, part_acc, part_ml);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || n_splits == 1) return (int)e;
  dim3 cgrid(n_tokens, n_q_heads);
  attention_combine_kernel<T><<<cgrid, 64, 0, stream>>>((T*)out, part_acc, part_ml, n_q_heads,
                                                        head_dim, n_splits);
  EK_RETURN_LAUNCH_STATUS();
}

}  // namespace ek

#define EK_INSTANTIATE(SUFFIX, T)                                                              \
  EK_EXPORT int ek_attention_generic_##SUFFIX(                                                  \
      void* out, const void* q, int q_row_stride, const int* positions, const int* token_slot, \
      const void* k_pages, const void* v_pages, const int* block_table, int table_stride,      \
      int n_tokens, int n_q_heads, int n_kv_heads, int head_dim, float scale, int window,      \
      int n_splits, int keys_per_split, float* part_acc, float* part_ml, cudaStream_t stream) { \
    return ek::launch<T>(out, q, q_row_stride, positions, token_slot, k_pages, v_pages,        \
                         block_table, table_stride, n_tokens, n_q_heads, n_kv_heads, head_dim, \
                         scale, window, n_splits, keys_per_split, part_acc, part_ml, stream);  \
  }

EK_INSTANTIATE(f32, float)
EK_INSTANTIATE(bf16, ek::bf16)
