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


// Wide form for 16-bit rows whose head size is 64, 128 or 256 and fully rotated: a block takes
// every head of one token, D/8 lanes a head.  A lane holds 4 neighbouring dimensions of the head's
// first half and the 4 they turn with in the second half (two 8-byte loads, each a full 128-byte
// line over the head's lanes), so the rotation needs no exchange between lanes; only the sum of
// squares of the head norm goes through shuffles.  The kernel is bound by instruction issue, not by
// memory (with the arithmetic taken out it runs at the copy bandwidth), so the gain and the angle
// are multiplied once per token and lane - four products per pair of dimensions, for q and for k -
// and a head costs a lane two multiply-adds and one multiply per value:
//     y_lo = rstd * (x_lo * (g_lo cos) - x_hi * (g_hi sin)),   y_hi = rstd * (x_hi * (g_hi cos) + x_lo * (g_lo sin))
// which is gain * x * rstd rotated, with the 32-bit products taken in another order.  All loads of
// a token are issued before the first use.
constexpr int kWideThreads = 256;
constexpr int kWidePasses = 4;

template <int D>
__global__ void __launch_bounds__(kWideThreads, 4)
qk_norm_rope_kv_wide_kernel(bf16* qkv, int row_stride, const float* __restrict__ q_gain,
                            const float* __restrict__ k_gain, const float* __restrict__ cos_tab,
                            const float* __restrict__ sin_tab, const int* positions,
                            const int* token_slot, PagedKV cache, int n_q_heads, float eps,
                            int write_kv) {
  constexpr int LPH = D / 8;                       // lanes a head
  constexpr int HPP = kWideThreads / LPH;          // heads a pass
  constexpr int half = D / 2;
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int n_kv = cache.heads;
  const int n_heads = write_kv ? n_q_heads + 2 * n_kv : n_q_heads;
  const int lih = threadIdx.x % LPH;               // lane in head
  const int head0 = threadIdx.x / LPH;
  const int d0 = 4 * lih;                          // this lane's dimensions: d0.. and half + d0..
  bf16* row = qkv + (size_t)t * row_stride;
  // the first heads are asked for before the position is known: one round trip less in the chain
  uint2 raw_lo[kWidePasses], raw_hi[kWidePasses];
  auto load_heads = [&](int base) {
#pragma unroll
    for (int p = 0; p < kWidePasses; ++p) {
      const int head = base + p * HPP + head0;
      if (head < n_heads) {
        raw_lo[p] = *reinterpret_cast<const uint2*>(row + (size_t)head * D + d0);
        raw_hi[p] = *reinterpret_cast<const uint2*>(row + (size_t)head * D + half + d0);
      }
    }
  };
  load_heads(0);
  const int pos = positions[t];
  if (pos < 0) return;
  // the lanes of this head within the warp: heads of one warp may take different branches
  const unsigned seg = LPH == 32 ? 0xffffffffu
                                 : ((1u << (LPH & 31)) - 1u) << ((threadIdx.x & 31) / LPH * LPH);
  size_t page_base = 0;
  if (write_kv) {
    const int page = cache.block_table[(size_t)token_slot[t] * cache.table_stride + pos / EK_PAGE];
    page_base = page_offset(cache, page, 0, pos);
  }
  // gain x angle, once per token and lane, for the query heads (most of a token's heads); a key
  // head takes its own four products when it comes
  float cs[4], sn[4];
  {
    const float4 c4 = *reinterpret_cast<const float4*>(cos_tab + (size_t)pos * half + d0);
    const float4 s4 = *reinterpret_cast<const float4*>(sin_tab + (size_t)pos * half + d0);
    cs[0] = c4.x; cs[1] = c4.y; cs[2] = c4.z; cs[3] = c4.w;
    sn[0] = s4.x; sn[1] = s4.y; sn[2] = s4.z; sn[3] = s4.w;
  }
  auto products = [&](const float* gain, float* lc, float* hs, float* hc, float* ls) {
    float gl[4] = {1.f, 1.f, 1.f, 1.f}, gh[4] = {1.f, 1.f, 1.f, 1.f};
    if (gain) {
      const float4 l4 = *reinterpret_cast<const float4*>(gain + d0);
      const float4 h4 = *reinterpret_cast<const float4*>(gain + half + d0);
      gl[0] = l4.x; gl[1] = l4.y; gl[2] = l4.z; gl[3] = l4.w;
      gh[0] = h4.x; gh[1] = h4.y; gh[2] = h4.z; gh[3] = h4.w;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lc[i] = gl[i] * cs[i];
      hs[i] = gh[i] * sn[i];
      hc[i] = gh[i] * cs[i];
      ls[i] = gl[i] * sn[i];
    }
  };
  float q_lc[4], q_hs[4], q_hc[4], q_ls[4];
  products(q_gain, q_lc, q_hs, q_hc, q_ls);
  const bool q_norm = q_gain != nullptr, k_norm = k_gain != nullptr;
  for (int base = 0; base < n_heads; base += HPP * kWidePasses) {
    if (base > 0) load_heads(base);
#pragma unroll
    for (int p = 0; p < kWidePasses; ++p) {
      const int head = base + p * HPP + head0;
      // shuffles below are among the D/8 lanes of a head, which are all in or all out
      if (head >= n_heads) continue;
      const bool is_q = head < n_q_heads;
      const bool is_k = !is_q && head < n_q_heads + n_kv;
      bf16* dst = row + (size_t)head * D + d0;
      if (!is_q) {
        const int kv_head = is_k ? head - n_q_heads : head - n_q_heads - n_kv;
        dst = (bf16*)(is_k ? cache.k : cache.v) + page_base + (size_t)kv_head * EK_PAGE * D + d0;
      }
      if (!is_q && !is_k) {
        *reinterpret_cast<uint2*>(dst) = raw_lo[p];
        *reinterpret_cast<uint2*>(dst + half) = raw_hi[p];
        continue;
      }
      float lo[4], hi[4];
      {
        const __nv_bfloat162* l2 = reinterpret_cast<const __nv_bfloat162*>(&raw_lo[p]);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw_hi[p]);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float2 f = __bfloat1622float2(l2[i]), g = __bfloat1622float2(h2[i]);
          lo[2 * i] = f.x; lo[2 * i + 1] = f.y;
          hi[2 * i] = g.x; hi[2 * i + 1] = g.y;
        }
      }
      float rstd = 1.f;
      if (is_q ? q_norm : k_norm) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) ss += lo[i] * lo[i] + hi[i] * hi[i];
#pragma unroll
        for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(seg, ss, o, LPH);
        rstd = rsqrtf(ss / (float)D + eps);
      }
      float ylo[4], yhi[4];
      if (is_q) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ylo[i] = (lo[i] * q_lc[i] - hi[i] * q_hs[i]) * rstd;
          yhi[i] = (hi[i] * q_hc[i] + lo[i] * q_ls[i]) * rstd;
        }
      } else {
        float k_lc[4], k_hs[4], k_hc[4], k_ls[4];
        products(k_gain, k_lc, k_hs, k_hc, k_ls);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ylo[i] = (lo[i] * k_lc[i] - hi[i] * k_hs[i]) * rstd;
          yhi[i] = (hi[i] * k_hc[i] + lo[i] * k_ls[i]) * rstd;
        }
      }
      __nv_bfloat162 l0 = __floats2bfloat162_rn(ylo[0], ylo[1]), l1 = __floats2bfloat162_rn(ylo[2], ylo[3]);
      __nv_bfloat162 h0 = __floats2bfloat162_rn(yhi[0], yhi[1]), h1 = __floats2bfloat162_rn(yhi[2], yhi[3]);
      *reinterpret_cast<uint2*>(dst) =
          make_uint2(*reinterpret_cast<uint32_t*>(&l0), *reinterpret_cast<uint32_t*>(&l1));
      *reinterpret_cast<uint2*>(dst + half) =
          make_uint2(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1));
    }
  }
}

template <int D>
static int launch_wide(bf16* qkv, int row_stride, const float* q_gain, const float* k_gain,
                       const float* cos_tab, const float* sin_tab, const int* positions,
                       const int* token_slot, PagedKV cache, int n_tokens, int n_q_heads, float eps,
                       int write_kv, cudaStream_t stream) {
  return (int)launch_pdl(qk_norm_rope_kv_wide_kernel<D>, dim3(n_tokens), dim3(kWideThreads), 0, stream,
                         qkv, row_stride, q_gain, k_gain, cos_tab, sin_tab, positions, token_slot, cache,
                         n_q_heads, eps, write_kv);
}

// The wide form needs 16-byte rows and tables; one token a block pays once there are enough
// tokens to fill the machine.
template <typename T>
static bool wide_takes(const void*, int, const float*, const float*, const float*, const float*, int,
                       const void*, const void*, int, int) {
  return false;
}
template <>
bool wide_takes<bf16>(const void* qkv, int row_stride, const float* q_gain, const float* k_gain,
                      const float* cos_tab, const float* sin_tab, int rot_dim, const void* k_pages,
                      const void* v_pages, int n_tokens, int head_dim) {
  auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  return (head_dim == 64 || head_dim == 128 || head_dim == 256) && rot_dim == head_dim &&
         n_tokens >= 128 && row_stride % 8 == 0 && aligned(qkv) && aligned(q_gain) && aligned(k_gain) &&
         aligned(cos_tab) && aligned(sin_tab) && aligned(k_pages) && aligned(v_pages);
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
  if (wide_takes<T>(qkv, row_stride, q_gain, k_gain, cos_tab, sin_tab, rot_dim, k_pages, v_pages,
                    n_tokens, head_dim)) {
    bf16* rows = (bf16*)qkv;
    if (head_dim == 64)
      return launch_wide<64>(rows, row_stride, q_gain, k_gain, cos_tab, sin_tab, positions, token_slot,
                             cache, n_tokens, n_q_heads, eps, write_kv, stream);
    if (head_dim == 128)
      return launch_wide<128>(rows, row_stride, q_gain, k_gain, cos_tab, sin_tab, positions, token_slot,
                              cache, n_tokens, n_q_heads, eps, write_kv, stream);
    return launch_wide<256>(rows, row_stride, q_gain, k_gain, cos_tab, sin_tab, positions, token_slot,
                            cache, n_tokens, n_q_heads, eps, write_kv, stream);
  }
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
