// Decode attention in bfloat16: one new token per sequence against its paged cache.
//
// The work is bound by reading the sequence's keys and values once from HBM, so the
// kernel is a register-streaming design with no shared-memory staging of K or V:
//   * the G query heads that share a KV head are the 16 rows of mma.sync.m16n8k16
//     (G padded to 16), so every K/V byte is read once for the whole group;
//   * S = Q.K^T: a key row is the "n" operand.  Within each 32-wide slice of the head
//     dimension the contraction index is permuted identically for Q and K, which lets a
//     thread fetch 8 consecutive values of one key row with one 16-byte load;
//   * O = P.V: P comes straight from the S accumulators (rounded to bfloat16); V rows are
//     fetched with 16-byte loads and turned into the "k-major" operand with
//     movmatrix.trans, which leaves each thread 8 consecutive output dimensions;
//   * the 4 warps of a block take alternate 16-key units of the block's key range with
//     their own running (max, sum, accumulator) and merge them in shared memory; blocks
//     split long sequences (grid.z) into partials that a combine kernel merges in order.
// The reference's counterpart is the Triton split-K flash-decoding kernel with the group
// padded to 16 rows and tiles staged through shared memory (engine/ek_kernels.py:534-615,
// combine 988-1019; split planning 1355-1381).  Softmax is computed in 32-bit.
#include "common.cuh"

namespace ek {

constexpr int kDecWarps = 4;
constexpr int kUnit = 16;                    // keys per warp iteration

__device__ __forceinline__ uint4 ldg16(const void* p) {
  uint4 v;
  // not .nc: the newest key and value were written by the kernel just before this one
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mma16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t reg_of(const uint4& v, int i) {
  return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// grid (tokens, kv_heads * row_blocks, splits); DCH = head_dim / 32
template <int DCH>
__global__ void __launch_bounds__(kDecWarps * 32)
attention_decode_bf16_kernel(bf16* __restrict__ out, const bf16* q, int q_row_stride,
                             const int* positions, const int* token_slot,
                             PagedKV cache, int n_q_heads, int row_blocks, float scale_log2,
                             int window, int n_splits, int keys_per_split,
                             float* __restrict__ part_acc, float* __restrict__ part_ml) {
  constexpr int D = DCH * 32;
  extern __shared__ float smem[];              // [warps][16][D] accumulators, then [warps][16][2]
  float* o_s = smem;
  float* ml_s = smem + kDecWarps * 16 * D;
  pdl_launch_dependents();
  pdl_wait();

  const int t = blockIdx.x;
  const int kv_head = blockIdx.y / row_blocks, rb = blockIdx.y % row_blocks;
  const int split = blockIdx.z;
  const int group = n_q_heads / cache.heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int pos = positions[t];
  const int head0 = kv_head * group + rb * 16;             // query head of row 0
  const int rows = min(16, group - rb * 16);               // real rows of this block

  int lo = 0, hi = -1;
  if (pos >= 0) {
    lo = window > 0 ? max(0, pos - window + 1) : 0;
    hi = pos;
    if (n_splits > 1) {
      if (keys_per_split > 0) {                // fixed cut of the key axis
        lo = max(lo, split * keys_per_split);
        hi = min(hi, (split + 1) * keys_per_split - 1);
      } else {                                 // cut this token's visible keys evenly
        const int first = lo & ~(kUnit - 1);
        const int per = max(kUnit, (((hi - first + n_splits) / n_splits) + kUnit - 1) & ~(kUnit - 1));
        lo = max(lo, first + split * per);
        hi = min(hi, first + (split + 1) * per - 1);
      }
    }
  }

  float acc[DCH][4][4];
#pragma unroll
  for (int c = 0; c < DCH; ++c)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[c][i][0] = acc[c][i][1] = acc[c][i][2] = acc[c][i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // rows g and g + 8

  if (hi >= lo) {
    // Q fragments: row g and g + 8, 8 consecutive dims at 32c + 8 tq
    uint4 q_lo[DCH], q_hi[DCH];
    const bf16* qrow = q + (size_t)t * q_row_stride + (size_t)head0 * D;
#pragma unroll
    for (int c = 0; c < DCH; ++c) {
      q_lo[c] = g < rows ? *reinterpret_cast<const uint4*>(qrow + (size_t)g * D + 32 * c + 8 * tq)
                         : make_uint4(0, 0, 0, 0);
      q_hi[c] = g + 8 < rows
                    ? *reinterpret_cast<const uint4*>(qrow + (size_t)(g + 8) * D + 32 * c + 8 * tq)
                    : make_uint4(0, 0, 0, 0);
    }
    const int slot = token_slot[t];
    const int* table = cache.block_table + (size_t)slot * cache.table_stride;
    const bf16* kbase = (const bf16*)cache.k;
    const bf16* vbase = (const bf16*)cache.v;

    const int u_first = lo / kUnit, u_last = hi / kUnit;
    for (int u = u_first + warp; u <= u_last; u += kDecWarps) {
      const int key0 = u * kUnit;
      const int page = table[key0 / EK_PAGE];
      const size_t row0 = ((size_t)page * cache.heads + kv_head) * EK_PAGE + (key0 & (EK_PAGE - 1));
      // this lane's rows: keys key0 + g and key0 + 8 + g, dims 32c + 8 tq .. + 7
      const bf16* kp = kbase + (row0 + g) * D + 8 * tq;
      const bf16* vp = vbase + (row0 + g) * D + 8 * tq;
      uint4 kr[2][DCH], vr[2][DCH];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int c = 0; c < DCH; ++c) kr[j][c] = ldg16(kp + (size_t)j * 8 * D + 32 * c);
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int c = 0; c < DCH; ++c) vr[j][c] = ldg16(vp + (size_t)j * 8 * D + 32 * c);

      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int c = 0; c < DCH; ++c) {
          mma16816(s[j], q_lo[c].x, q_hi[c].x, q_lo[c].y, q_hi[c].y, kr[j][c].x, kr[j][c].y);
          mma16816(s[j], q_lo[c].z, q_hi[c].z, q_lo[c].w, q_hi[c].w, kr[j][c].z, kr[j][c].w);
        }
      }
      // scale, mask, running softmax.  s[j][0..1]: row g, keys key0 + 8j + 2tq + {0,1};
      // s[j][2..3]: row g + 8, same keys.
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key0 + 8 * j + 2 * tq + (e & 1);
          const float v = (key >= lo && key <= hi) ? s[j][e] * scale_log2 : -INFINITY;
          s[j][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      float alpha[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[r], mx[r]);          // finite: the unit has a visible key
        alpha[r] = exp2f(m_run[r] - m_new);
        m_run[r] = m_new;
      }
      float psum[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = exp2f(s[j][e] - m_run[e >> 1]);
          s[j][e] = p;
          psum[e >> 1] += p;
        }
      l_run[0] = l_run[0] * alpha[0] + psum[0];
      l_run[1] = l_run[1] * alpha[1] + psum[1];
      const uint32_t p0 = pack_bf16(s[0][0], s[0][1]), p1 = pack_bf16(s[0][2], s[0][3]);
      const uint32_t p2 = pack_bf16(s[1][0], s[1][1]), p3 = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
      for (int c = 0; c < DCH; ++c)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[c][i][0] *= alpha[0]; acc[c][i][1] *= alpha[0];
          acc[c][i][2] *= alpha[1]; acc[c][i][3] *= alpha[1];
          const uint32_t b0 = movmatrix_trans(reg_of(vr[0][c], i));
          const uint32_t b1 = movmatrix_trans(reg_of(vr[1][c], i));
          mma16816(acc[c][i], p0, p1, p2, p3, b0, b1);
        }
    }
  }

  // per-warp results -> shared memory.  acc[c][i][e]: row g (e<2) or g+8, dim 32c + 8tq + 2i + (e&1)
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int c = 0; c < DCH; ++c)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float* o_lo = o_s + ((size_t)warp * 16 + g) * D + 32 * c + 8 * tq + 2 * i;
      float* o_hi = o_s + ((size_t)warp * 16 + g + 8) * D + 32 * c + 8 * tq + 2 * i;
      *reinterpret_cast<float2*>(o_lo) = make_float2(acc[c][i][0], acc[c][i][1]);
      *reinterpret_cast<float2*>(o_hi) = make_float2(acc[c][i][2], acc[c][i][3]);
    }
  if (tq == 0) {
    ml_s[(warp * 16 + g) * 2] = m_run[0];
    ml_s[(warp * 16 + g) * 2 + 1] = l_run[0];
    ml_s[(warp * 16 + g + 8) * 2] = m_run[1];
    ml_s[(warp * 16 + g + 8) * 2 + 1] = l_run[1];
  }
  __syncthreads();

  // merge the warps in warp order; thread handles (row, dim) pairs
  for (int idx = threadIdx.x; idx < rows * D; idx += kDecWarps * 32) {
    const int r = idx / D, d = idx % D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) m = fmaxf(m, ml_s[(w * 16 + r) * 2]);
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float lw = ml_s[(w * 16 + r) * 2 + 1];
      if (lw > 0.f) {
        const float f = exp2f(ml_s[(w * 16 + r) * 2] - m);
        l += lw * f;
        o += o_s[((size_t)w * 16 + r) * D + d] * f;
      }
    }
    const int head = head0 + r;
    if (n_splits == 1) {
      out[((size_t)t * n_q_heads + head) * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    } else {
      const size_t pi = ((size_t)t * n_q_heads + head) * n_splits + split;
      part_acc[pi * D + d] = o;
      if (d == 0) {
        part_ml[2 * pi] = m;                   // in units of log2 (scores were scaled by log2 e)
        part_ml[2 * pi + 1] = l;
      }
    }
  }
}

// Merge split partials in split order (running maxima are in log2 units).
__global__ void attention_decode_combine_kernel(bf16* __restrict__ out,
                                                const float* part_acc,
                                                const float* part_ml, int n_q_heads,
                                                int head_dim, int n_splits) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t th = (size_t)blockIdx.x * n_q_heads + blockIdx.y;
  const float* ml = part_ml + 2 * th * n_splits;
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, ml[2 * s]);
  float l = 0.f;
  for (int s = 0; s < n_splits; ++s)
    if (ml[2 * s + 1] > 0.f) l += ml[2 * s + 1] * exp2f(ml[2 * s] - m);
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int i = threadIdx.x; i < head_dim; i += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < n_splits; ++s)
      if (ml[2 * s + 1] > 0.f)
        acc += part_acc[(th * n_splits + s) * head_dim + i] * exp2f(ml[2 * s] - m);
    out[th * head_dim + i] = __float2bfloat16_rn(acc * inv);
  }
}

template <int DCH>
static int launch_dch(bf16* out, const bf16* q, int q_row_stride, const int* positions,
                      const int* token_slot, PagedKV cache, int n_tokens, int n_q_heads,
                      float scale, int window, int n_splits, int keys_per_split, float* part_acc,
                      float* part_ml, cudaStream_t stream) {
  constexpr int D = DCH * 32;
  const int group = n_q_heads / cache.heads;
  const int row_blocks = (group + 15) / 16;
  const size_t smem = (size_t)kDecWarps * 16 * (D + 2) * sizeof(float);
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_bf16_kernel<DCH>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(n_tokens, cache.heads * row_blocks, n_splits);
  // three blocks an SM (two for the largest head sizes) need this much shared memory; the rest
  // stays L1, which the K/V stream needs for its loads in flight
  const int blocks_per_sm = DCH <= 4 ? 3 : 2;
  const int percent = (int)((blocks_per_sm * (smem + 1024) * 100 + 228 * 1024 - 1) / (228 * 1024));
  prefer_carveout((const void*)attention_decode_bf16_kernel<DCH>, percent < 50 ? 50 : percent);
  cudaError_t e = launch_pdl(attention_decode_bf16_kernel<DCH>, grid, dim3(kDecWarps * 32), smem,
                             stream, out, q, q_row_stride, positions, token_slot, cache, n_q_heads,
                             row_blocks, scale * 1.4426950408889634f, window, n_splits,
                             keys_per_split, part_acc, part_ml);
  if (e != cudaSuccess || n_splits == 1) return (int)e;
  dim3 cgrid(n_tokens, n_q_heads);
  return (int)launch_pdl(attention_decode_combine_kernel, cgrid, dim3(64), 0, stream, out,
                         (const float*)part_acc, (const float*)part_ml, n_q_heads, D, n_splits);
}

}  // namespace ek

// head_dim must be a multiple of 32 (up to 256); keys_per_split a multiple of 16, or 0 to cut
// each token's visible keys into n_splits equal parts.
EK_EXPORT int ek_attention_decode_bf16(void* out, const void* q, int q_row_stride,
                                       const int* positions, const int* token_slot,
                                       const void* k_pages, const void* v_pages,
                                       const int* block_table, int table_stride, int n_tokens,
                                       int n_q_heads, int n_kv_heads, int head_dim, float scale,
                                       int window, int n_splits, int keys_per_split,
                                       float* part_acc, float* part_ml, cudaStream_t stream) {
  using namespace ek;
  if (n_tokens <= 0) return 0;
  if (head_dim % 32 || head_dim < 32 || head_dim > 256 || n_kv_heads <= 0 ||
      n_q_heads % n_kv_heads || n_splits < 1 || n_splits > 65535 || q_row_stride % 8 ||
      (n_splits > 1 && (!part_acc || !part_ml || keys_per_split < 0 || keys_per_split % kUnit)))
    return EK_ERR_ARG;
  PagedKV cache{(void*)k_pages, (void*)v_pages, block_table, table_stride, n_kv_heads, head_dim};
#define EK_CASE(DCH)                                                                              \
  case DCH:                                                                                       \
    return launch_dch<DCH>((bf16*)out, (const bf16*)q, q_row_stride, positions, token_slot, cache, \
                           n_tokens, n_q_heads, scale, window, n_splits, keys_per_split, part_acc, \
                           part_ml, stream);
  switch (head_dim / 32) {
    EK_CASE(1) EK_CASE(2) EK_CASE(3) EK_CASE(4) EK_CASE(5) EK_CASE(6) EK_CASE(7) EK_CASE(8)
  }
#undef EK_CASE
  return EK_ERR_ARG;
}

// ---------------------------------------------------------------------------------------
// The allocation-free variant (declared and described in attention_decode_noalloc.h).
// ---------------------------------------------------------------------------------------
#include <stdio.h>

#include "attention_decode_noalloc.h"

namespace ek {

// Partial accumulators and (max, sum) pairs of the key splits.  In host code this name is
// only a handle for cudaGetSymbolAddress, never a pointer a kernel may be given.
static __device__ __align__(256) float noalloc_scratch[EK_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
static float* noalloc_scratch_address[kMaxDevices];     // per device, filled on first use

// Device address of the array on the current device; looked up once per device.
static int noalloc_scratch_pointer(float** ptr) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= kMaxDevices) return EK_ERR_ARG;
  if (noalloc_scratch_address[device] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    noalloc_scratch_address[device] = p;
  }
  *ptr = noalloc_scratch_address[device];
  return 0;
}

}  // namespace ek

EK_EXPORT int ek_attention_decode_bf16_noalloc(void* out, const void* q, int q_row_stride,
                                               const int* positions, const int* token_slot,
                                               const void* k_pages, const void* v_pages,
                                               const int* block_table, int table_stride,
                                               int n_tokens, int n_q_heads, int n_kv_heads,
                                               int head_dim, float scale, int window, int n_splits,
                                               int keys_per_split, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  float* part_acc = nullptr;
  float* part_ml = nullptr;
  if (n_splits > 1) {
    if (n_q_heads <= 0 || head_dim <= 0) return EK_ERR_ARG;
    const unsigned long long cells = (unsigned long long)n_tokens * (unsigned long long)n_q_heads *
                                     (unsigned long long)n_splits;
    const unsigned long long need = cells * (unsigned long long)(head_dim + 2);
    if (need > (unsigned long long)EK_NOALLOC_SCRATCH_FLOATS) {
      fprintf(stderr,
              "ek_attention_decode_bf16_noalloc: this call needs %llu scratch values, the fixed "
              "array holds %d; nothing was launched\n", need, EK_NOALLOC_SCRATCH_FLOATS);
      return EK_NOALLOC_TOO_LARGE;
    }
    float* base = nullptr;
    const int status = ek::noalloc_scratch_pointer(&base);
    if (status != 0) return status;
    part_acc = base;                                         // [cells][head_dim]
    part_ml = base + cells * (unsigned long long)head_dim;   // [cells][2]
  }
  return ek_attention_decode_bf16(out, q, q_row_stride, positions, token_slot, k_pages, v_pages,
                                  block_table, table_stride, n_tokens, n_q_heads, n_kv_heads,
                                  head_dim, scale, window, n_splits, keys_per_split, part_acc,
                                  part_ml, stream);
}
