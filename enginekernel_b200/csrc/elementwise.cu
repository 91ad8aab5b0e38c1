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

// resid[t] = table[ids[t]] * scale (+ pos_table[positions[t]] if the model has learned positions)
template <typename T>
__global__ void embed_kernel(float* __restrict__ resid, const T* __restrict__ table,
                             const int* ids, int hidden, int vocab, float scale,
                             const T* __restrict__ pos_table, const int* positions, int max_positions) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const T* row = table + (size_t)id * hidden;
  float* out = resid + (size_t)t * hidden;
  const T* prow = nullptr;
  if (pos_table != nullptr) {
    const int p = positions[t];                // rows of finished sequences (negative) get no position
    if (p >= 0) prow = pos_table + (size_t)min(p, max_positions - 1) * hidden;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    out[i] = to_f<T>(row[i]) * scale + (prow ? to_f<T>(prow[i]) : 0.f);
}

__global__ void scale_f32_kernel(float* x, size_t n, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] *= scale;
}


// y = gain * x * rsqrt(mean(x^2) + eps) for each row; x is the 32-bit stream.
// If `add` is given, the stream first becomes stream + add (written back when
// `write_back`).  If `rows` is given, output row i reads stream row rows[i].
// VEC: the row length is a multiple of 4 and rows are accessed four values at a time.
template <typename T, bool VEC>
__global__ void rmsnorm_kernel(T* __restrict__ y, float* resid, const T* add,
                               const float* __restrict__ gain, const int* rows, float eps, int hidden,
                               int write_back) {
  __shared__ float scratch[33];
  extern __shared__ __align__(16) float row_cache[];          // `hidden` floats
  pdl_launch_dependents();
  pdl_wait();
  const int out_row = blockIdx.x;
  const int src_row = rows ? rows[out_row] : out_row;
  float* r = resid + (size_t)src_row * hidden;
  const T* a = add ? add + (size_t)src_row * hidden : nullptr;
  T* out = y + (size_t)out_row * hidden;
  float ss = 0.f;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(r + i);
      if (a) {
        const float4 w = Vec4<T>::load(a + i);
        v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
        if (write_back) *reinterpret_cast<float4*>(r + i) = v;
      }
      *reinterpret_cast<float4*>(row_cache + i) = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = r[i];
      if (a) {
        v += to_f<T>(a[i]);
        if (write_back) r[i] = v;
      }
      row_cache[i] = v;
      ss += v * v;
    }
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)hidden + eps);
  if (VEC) {
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row_cache + i);
      const float4 g = *reinterpret_cast<const float4*>(gain + i);
      Vec4<T>::store(out + i, make_float4(v.x * rstd * g.x, v.y * rstd * g.y, v.z * rstd * g.z,
                                          v.w * rstd * g.w));
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      out[i] = from_f<T>(row_cache[i] * rstd * gain[i]);
  }
}

// The same for rows of at most 4,096 values in steps of 4: 128 threads a row, the row held in
// registers (NV loads of 16 bytes a thread at most, all issued before the first use), no row in
// shared memory - so that an SM keeps more rows in flight, which is what a kernel that only moves
// memory needs.  Same arithmetic; the sum of squares is taken in another order.
constexpr int kNormRegThreads = 128, kNormRegVecs = 8;
template <typename T, int NV>
__global__ void __launch_bounds__(kNormRegThreads, NV <= 6 ? 8 : 5)
rmsnorm_reg_kernel(T* __restrict__ y, float* resid, const T* add, const float* __restrict__ gain,
                   const int* rows, float eps, int hidden, int write_back) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int out_row = blockIdx.x;
  const int src_row = rows ? rows[out_row] : out_row;
  float* r = resid + (size_t)src_row * hidden;
  const T* a = add ? add + (size_t)src_row * hidden : nullptr;
  T* out = y + (size_t)out_row * hidden;
  float4 v[NV], w[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = (threadIdx.x + j * kNormRegThreads) * 4;
    v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    w[j] = v[j];
    if (i < hidden) {
      v[j] = *reinterpret_cast<const float4*>(r + i);
      if (a) w[j] = Vec4<T>::load(a + i);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = (threadIdx.x + j * kNormRegThreads) * 4;
    if (a) {
      v[j].x += w[j].x; v[j].y += w[j].y; v[j].z += w[j].z; v[j].w += w[j].w;
      if (write_back && i < hidden) *reinterpret_cast<float4*>(r + i) = v[j];
    }
    ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)hidden + eps);
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = (threadIdx.x + j * kNormRegThreads) * 4;
    if (i < hidden) {
      const float4 g = *reinterpret_cast<const float4*>(gain + i);
      Vec4<T>::store(out + i, make_float4(v[j].x * rstd * g.x, v[j].y * rstd * g.y, v[j].z * rstd * g.z,
                                          v[j].w * rstd * g.w));
    }
  }
}

// stream += add, without a norm (the last feed-forward output when no norm follows)
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ resid, const T* __restrict__ add, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) resid[i] += to_f<T>(add[i]);
}

// out[r, i] = silu(gu[r, i]) * gu[r, inter + i]    (engine/ek_kernels.py:125-143)
// VEC: inter is a multiple of 4; a thread handles four neighbours.  A 16-bit result takes the
// fast exponential and division (a few 32-bit ulps, far below its own rounding); a 32-bit
// result the exact ones.
template <typename T>
__device__ __forceinline__ float silu_of(float g) {
  if (sizeof(T) == 2) return __fdividef(g, 1.f + __expf(-g));
  return g / (1.f + expf(-g));
}

template <typename T, bool VEC>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int inter) {
  const size_t r = blockIdx.y;
  const T* g_row = gu + r * 2 * inter;
  T* o_row = out + r * inter;
  if (VEC) {
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= inter) return;
    const float4 g = Vec4<T>::load(g_row + i), u = Vec4<T>::load(g_row + inter + i);
    Vec4<T>::store(o_row + i, make_float4(silu_of<T>(g.x) * u.x, silu_of<T>(g.y) * u.y,
                                          silu_of<T>(g.z) * u.z, silu_of<T>(g.w) * u.w));
  } else {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= inter) return;
    const float g = to_f<T>(g_row[i]), u = to_f<T>(g_row[inter + i]);
    o_row[i] = from_f<T>(silu_of<T>(g) * u);
  }
}

// The same for bfloat16 rows whose halves start on 16-byte boundaries: eight neighbours a thread.
__global__ void silu_mul_wide_kernel(bf16* __restrict__ out, const bf16* __restrict__ gu, int inter) {
  const size_t r = blockIdx.y;
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= inter) return;
  const bf16* g_row = gu + r * 2 * inter;
  const uint4 g = *reinterpret_cast<const uint4*>(g_row + i);
  const uint4 u = *reinterpret_cast<const uint4*>(g_row + inter + i);
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 a = __bfloat1622float2(g2[j]), b = __bfloat1622float2(u2[j]);
    __nv_bfloat162 h = __floats2bfloat162_rn(silu_of<bf16>(a.x) * b.x, silu_of<bf16>(a.y) * b.y);
    w[j] = *reinterpret_cast<uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(out + r * inter + i) = make_uint4(w[0], w[1], w[2], w[3]);
}

template <typename T>
static int launch_rmsnorm(void* y, float* resid, const void* add, const float* gain,
                          const int* rows, float eps, int n_rows, int hidden, int write_back,
                          cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden <= 0 || (size_t)hidden * 4 > 200 * 1024) return EK_ERR_ARG;
  const size_t smem = (size_t)hidden * sizeof(float);
  const bool vec = hidden % 4 == 0 && ((uintptr_t)y % 8) == 0 && ((uintptr_t)add % 8) == 0;
  if (vec && hidden <= kNormRegThreads * kNormRegVecs * 4 && ((uintptr_t)resid % 16) == 0 &&
      ((uintptr_t)gain % 16) == 0)
  {
    const int nv = (hidden / 4 + kNormRegThreads - 1) / kNormRegThreads;
    auto reg_kernel = nv <= 2 ? rmsnorm_reg_kernel<T, 2> : nv <= 4 ? rmsnorm_reg_kernel<T, 4>
                    : nv <= 6 ? rmsnorm_reg_kernel<T, 6> : rmsnorm_reg_kernel<T, 8>;
    return (int)launch_pdl(reg_kernel, dim3(n_rows), dim3(kNormRegThreads), 0, stream, (T*)y, resid,
                           (const T*)add, gain, rows, eps, hidden, write_back);
  }
  auto kernel = vec ? rmsnorm_kernel<T, true> : rmsnorm_kernel<T, false>;
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int per_thread = vec ? 4 : 1;
  int threads = hidden / per_thread >= 512 ? 512 : (hidden / per_thread >= 256 ? 256 : 128);
  return (int)launch_pdl(kernel, dim3(n_rows), dim3(threads), smem, stream, (T*)y, resid,
                         (const T*)add, gain, rows, eps, hidden, write_back);
}

template <typename T>
static int launch_silu_mul(void* out, const void* gu, int rows, int inter, cudaStream_t stream) {
  if (rows <= 0 || inter <= 0) return 0;
  if (rows > 65535) return EK_ERR_ARG;
  if (sizeof(T) == 2 && inter % 8 == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)gu % 16) == 0) {
    dim3 wide((inter / 8 + 255) / 256, rows);
    silu_mul_wide_kernel<<<wide, 256, 0, stream>>>((bf16*)out, (const bf16*)gu, inter);
    EK_RETURN_LAUNCH_STATUS();
  }
  const bool vec = inter % 4 == 0 && ((uintptr_t)out % 8) == 0 && ((uintptr_t)gu % 8) == 0;
  const int per_thread = vec ? 4 : 1;
  dim3 grid((inter / per_thread + 255) / 256 + (inter % per_thread ? 1 : 0), rows);
  if (vec) silu_mul_kernel<T, true><<<grid, 256, 0, stream>>>((T*)out, (const T*)gu, inter);
  else silu_mul_kernel<T, false><<<grid, 256, 0, stream>>>((T*)out, (const T*)gu, inter);
  EK_RETURN_LAUNCH_STATUS();
}

}  // namespace ek

using namespace ek;

#define EK_INSTANTIATE(SUFFIX, T)                                                               \
  EK_EXPORT int ek_embed_##SUFFIX(float* resid, const void* table, const int* ids, int n_tokens, \
                                  int hidden, int vocab, float scale, const void* pos_table,    \
                                  const int* positions, int max_positions, cudaStream_t stream) { \
    if (n_tokens <= 0) return 0;                                                                \
    if (pos_table && (!positions || max_positions <= 0)) return EK_ERR_ARG;                     \
    /* A plain launch, on purpose: the first kernel of a step starts only when everything   */ \
    /* before it on the stream has finished and is visible.  The kernels behind it may then */ \
    /* read per-step state (positions, slots) before their own griddepcontrol.wait even     */ \
    /* when the step before was not a graph launch of its own (eager decode).               */ \
    embed_kernel<T><<<dim3(n_tokens), dim3(256), 0, stream>>>(resid, (const T*)table, ids,     \
                                                               hidden, vocab, scale,            \
                                                               (const T*)pos_table, positions,  \
                                                               max_positions);                  \
    EK_RETURN_LAUNCH_STATUS();                                                                  \
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
    return launch_silu_mul<T>(out, gu, rows, inter, stream);                                    \
  }

EK_INSTANTIATE(f32, float)
EK_INSTANTIATE(bf16, ek::bf16)

// x[i] *= scale for n 32-bit values (logits of a model with a logit multiplier)
EK_EXPORT int ek_scale_f32(float* x, long long n, float scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  return (int)ek::launch_pdl(ek::scale_f32_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x,
                             (size_t)n, scale);
}
