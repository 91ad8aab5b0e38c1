// Embedding lookup, RMSNorm (plain, with the residual add folded in, and on
// gathered rows) and the SwiGLU gate.
//
// The residual stream is held in 32-bit in both precisions; T is the type of the
// normalised activations that feed the matrix products (float or bfloat16).
// Mean of squares, the scaling and the residual sum are computed in 32-bit
// (the reference does the same inside its norm kernels, engine/ek_kernels.py:89-123,
// but stores the stream in bfloat16).
#include "common.cuh"

namespace ek {

template <typename T>
__global__ void embed_kernel(float* __restrict__ resid, const T* __restrict__ table,
                             const int* ids, int hidden, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const T* row = table + (size_t)id * hidden;
  float* out = resid + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = to_f<T>(row[i]);
}

// y = gain * x * rsqrt(mean(x^2) + eps) for each row; x is the 32-bit stream.
// If `add` is given, the stream first becomes stream + add (written back when
// `write_back`).  If `rows` is given, output row i reads stream row rows[i].
template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ y, float* resid, const T* add,
                               const float* __restrict__ gain, const int* rows, float eps, int hidden,
                               int write_back) {
  __shared__ float scratch[33];
  extern __shared__ float row_cache[];          // `hidden` floats
  pdl_launch_dependents();
  pdl_wait();
  const int out_row = blockIdx.x;
  const int src_row = rows ? rows[out_row] : out_row;
  float* r = resid + (size_t)src_row * hidden;
  const T* a = add ? add + (size_t)src_row * hidden : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = r[i];
    if (a) {
      v += to_f<T>(a[i]);
      if (write_back) r[i] = v;
    }
    row_cache[i] = v;
    ss += v * v;
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)hidden + eps);
  T* out = y + (size_t)out_row * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    out[i] = from_f<T>(row_cache[i] * rstd * gain[i]);
}

// stream += add, without a norm (the last feed-forward output when no norm follows)
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ resid, const T* __restrict__ add, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) resid[i] += to_f<T>(add[i]);
}

// out[r, i] = silu(gu[r, i]) * gu[r, inter + i]    (engine/ek_kernels.py:125-143)
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int inter) {
  const size_t r = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= inter) return;
  const float g = to_f<T>(gu[r * 2 * inter + i]);
  const float u = to_f<T>(gu[r * 2 * inter + inter + i]);
  const float s = g / (1.f + expf(-g));
  out[r * inter + i] = from_f<T>(s * u);
}

template <typename T>
static int launch_rmsnorm(void* y, float* resid, const void* add, const float* gain,
                          const int* rows, float eps, int n_rows, int hidden, int write_back,
                          cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden <= 0 || (size_t)hidden * 4 > 200 * 1024) return EK_ERR_ARG;
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(rmsnorm_kernel<T>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  return (int)launch_pdl(rmsnorm_kernel<T>, dim3(n_rows), dim3(threads), smem, stream, (T*)y, resid,
                         (const T*)add, gain, rows, eps, hidden, write_back);
}

}  // namespace ek

using namespace ek;

#define EK_INSTANTIATE(SUFFIX, T)                                                               \
  EK_EXPORT int ek_embed_##SUFFIX(float* resid, const void* table, const int* ids, int n_tokens, \
                                  int hidden, int vocab, cudaStream_t stream) {                 \
    if (n_tokens <= 0) return 0;                                                                \
    return (int)ek::launch_pdl(embed_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, resid,    \
                               (const T*)table, ids, hidden, vocab);                            \
  }                                                                                             \
  EK_EXPORT int ek_rmsnorm_##SUFFIX(void* y, float* resid, const void* add, const float* gain,  \
                                    const int* rows, float eps, int n_rows, int hidden,         \
                                    int write_back, cudaStream_t stream) {                      \
    return launch_rmsnorm<T>(y, resid, add, gain, rows, eps, n_rows, hidden, write_back, stream); \
  }                                                                                             \
  EK_EXPORT int ek_add_residual_##SUFFIX(float* resid, const void* add, long long n,            \
                                         cudaStream_t stream) {                                 \
    if (n <= 0) return 0;                                                                       \
    add_residual_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(resid, (const T*)add, \
                                                                             (size_t)n);        \
    EK_RETURN_LAUNCH_STATUS();                                                                  \
  }                                                                                             \
  EK_EXPORT int ek_silu_mul_##SUFFIX(void* out, const void* gu, int rows, int inter,            \
                                     cudaStream_t stream) {                                     \
    if (rows <= 0 || inter <= 0) return 0;                                                      \
    if (rows > 65535) return EK_ERR_ARG;                                                        \
    dim3 grid((inter + 255) / 256, rows);                                                       \
    silu_mul_kernel<T><<<grid, 256, 0, stream>>>((T*)out, (const T*)gu, inter);                 \
    EK_RETURN_LAUNCH_STATUS();                                                                  \
  }

EK_INSTANTIATE(f32, float)
EK_INSTANTIATE(bf16, ek::bf16)
