// Weight-streaming product for decode: out[M,N] = x[M,K] . W[N,K]^T with few rows
// (M <= 64 sequences) in bfloat16 and 32-bit accumulation.  The step is bound by
// reading W once from HBM, so the kernel is built around that stream:
//   * the weights are the 16-row operand of mma.sync.m16n8k16 and go from global
//     memory straight into registers with 16-byte loads - within a 32-wide slice of K
//     the contraction index is permuted identically for both operands, which lets each
//     thread fetch eight consecutive weights of one row (no shared-memory staging);
//   * the batch is the 8-column operand (M padded to a multiple of 8 in registers);
//   * the warps of a block split K between them in interleaved 32-element slices and
//     add their partial tiles in shared memory in warp order (no atomics, so results
//     are the same from run to run).
// The reference does this with Triton kernels that pad the batch to 16 rows
// (engine/ek_kernels.py:281-308 `_gemv_kernel`, 413-445 split-K parts,
// 375-411 SwiGLU epilogue); the epilogues here are: store bfloat16, store 32-bit
// (logits), and SwiGLU, where one 16-row tile holds 8 gate rows and the 8 matching up
// rows so that silu(gate) * up is formed in registers and the [M, 2I] intermediate is
// never written.
#include "common.cuh"

namespace ek {

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2 };

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_cached(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_bf16(float c[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Tile `blockIdx.x` covers weight rows  lo = tile * lo_step + g  and  hi = lo + hi_offset
// for g = 0..7  (plain: lo_step 16, hi_offset 8; SwiGLU: lo_step 8, hi_offset I).
template <int NT, int EPI>
__global__ void gemv_bf16_kernel(void* __restrict__ out, const bf16* __restrict__ x,
                                 const bf16* __restrict__ W, int M, int n_lo_rows, int K, int ldx,
                                 int ldw, int ldo, int lo_step, int hi_offset) {
  extern __shared__ float red[];               // [warps][NT][32][4]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int row_lo = blockIdx.x * lo_step + g;
  // EPI_BF16/F32: n_lo_rows = N and both halves are checked against it.
  const bool lo_ok = row_lo < n_lo_rows;
  const bool hi_ok = (EPI == EPI_SWIGLU) ? lo_ok : (row_lo + hi_offset < n_lo_rows);
  const bf16* w_lo = W + (size_t)(lo_ok ? row_lo : 0) * ldw;
  const bf16* w_hi = W + (size_t)(hi_ok ? row_lo + hi_offset : 0) * ldw;

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  const int n_chunks = (K + 31) >> 5;
#pragma unroll 4
  for (int c = warp; c < n_chunks; c += warps) {
    const int k = (c << 5) + (t << 3);
    uint4 a_lo = make_uint4(0, 0, 0, 0), a_hi = make_uint4(0, 0, 0, 0);
    const bool k_ok = k < K;                   // K is a multiple of 8
    if (k_ok) {
      a_lo = ldg_stream(w_lo + k);
      a_hi = ldg_stream(w_hi + k);
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int m = 8 * j + g;
      uint4 b = make_uint4(0, 0, 0, 0);
      if (k_ok && m < M) b = ldg_cached(x + (size_t)m * ldx + k);
      mma_bf16(acc[j], a_lo.x, a_hi.x, a_lo.y, a_hi.y, b.x, b.y);
      mma_bf16(acc[j], a_lo.z, a_hi.z, a_lo.w, a_hi.w, b.z, b.w);
    }
  }

  // partial tiles -> shared memory, summed in warp order by the first NT warps
#pragma unroll
  for (int j = 0; j < NT; ++j)
    *reinterpret_cast<float4*>(&red[((warp * NT + j) * 32 + lane) * 4]) =
        make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
  __syncthreads();
  for (int j = warp; j < NT; j += warps) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int w = 0; w < warps; ++w) {
      const float4 p = *reinterpret_cast<const float4*>(&red[((w * NT + j) * 32 + lane) * 4]);
      s.x += p.x; s.y += p.y; s.z += p.z; s.w += p.w;
    }
    // s.x, s.y: row lo, batch columns 8j+2t, 8j+2t+1;  s.z, s.w: row hi, same columns
    const int m0 = 8 * j + 2 * t;
    if (EPI == EPI_SWIGLU) {
      if (lo_ok) {
        bf16* o = (bf16*)out;
        if (m0 < M) o[(size_t)m0 * ldo + row_lo] = __float2bfloat16_rn(s.x / (1.f + expf(-s.x)) * s.z);
        if (m0 + 1 < M)
          o[(size_t)(m0 + 1) * ldo + row_lo] = __float2bfloat16_rn(s.y / (1.f + expf(-s.y)) * s.w);
      }
    } else if (EPI == EPI_F32) {
      float* o = (float*)out;
      if (lo_ok) {
        if (m0 < M) o[(size_t)m0 * ldo + row_lo] = s.x;
        if (m0 + 1 < M) o[(size_t)(m0 + 1) * ldo + row_lo] = s.y;
      }
      if (hi_ok) {
        if (m0 < M) o[(size_t)m0 * ldo + row_lo + hi_offset] = s.z;
        if (m0 + 1 < M) o[(size_t)(m0 + 1) * ldo + row_lo + hi_offset] = s.w;
      }
    } else {
      bf16* o = (bf16*)out;
      if (lo_ok) {
        if (m0 < M) o[(size_t)m0 * ldo + row_lo] = __float2bfloat16_rn(s.x);
        if (m0 + 1 < M) o[(size_t)(m0 + 1) * ldo + row_lo] = __float2bfloat16_rn(s.y);
      }
      if (hi_ok) {
        if (m0 < M) o[(size_t)m0 * ldo + row_lo + hi_offset] = __float2bfloat16_rn(s.z);
        if (m0 + 1 < M) o[(size_t)(m0 + 1) * ldo + row_lo + hi_offset] = __float2bfloat16_rn(s.w);
      }
    }
  }
}

template <int NT, int EPI>
static int launch_nt(void* out, const void* x, const void* W, int M, int N, int K, int ldx, int ldw,
                     int ldo, int warps, cudaStream_t stream) {
  int tiles, lo_step, hi_offset, n_lo_rows;
  if (EPI == EPI_SWIGLU) {                     // N = 2 * I rows: gate rows then up rows
    const int inter = N / 2;
    tiles = (inter + 7) / 8; lo_step = 8; hi_offset = inter; n_lo_rows = inter;
  } else {
    tiles = (N + 15) / 16; lo_step = 16; hi_offset = 8; n_lo_rows = N;
  }
  const size_t smem = (size_t)warps * NT * 32 * 4 * sizeof(float);
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(gemv_bf16_kernel<NT, EPI>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  gemv_bf16_kernel<NT, EPI><<<tiles, warps * 32, smem, stream>>>(
      out, (const bf16*)x, (const bf16*)W, M, n_lo_rows, K, ldx, ldw, ldo, lo_step, hi_offset);
  EK_RETURN_LAUNCH_STATUS();
}

template <int EPI>
static int launch(void* out, const void* x, const void* W, int M, int N, int K, int ldx, int ldw,
                  int ldo, int warps, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || K % 8 || ldx % 8 || ldw % 8 || warps < 1 || warps > 32 ||
      (EPI == EPI_SWIGLU && (N & 1)))
    return EK_ERR_ARG;
  if (warps > 16) warps = 16;              // 8 batch tiles need 96 registers a thread
  if (M <= 8) return launch_nt<1, EPI>(out, x, W, M, N, K, ldx, ldw, ldo, warps, stream);
  if (M <= 16) return launch_nt<2, EPI>(out, x, W, M, N, K, ldx, ldw, ldo, warps, stream);
  if (M <= 32) return launch_nt<4, EPI>(out, x, W, M, N, K, ldx, ldw, ldo, warps, stream);
  return launch_nt<8, EPI>(out, x, W, M, N, K, ldx, ldw, ldo, warps, stream);
}

}  // namespace ek

// epilogue: 0 bfloat16 out [M,N]; 1 float out [M,N]; 2 SwiGLU, bfloat16 out [M,N/2]
EK_EXPORT int ek_gemv_bf16(void* out, const void* x, const void* W, int M, int N, int K, int ldx,
                           int ldw, int ldo, int epilogue, int warps, cudaStream_t stream) {
  switch (epilogue) {
    case ek::EPI_BF16: return ek::launch<ek::EPI_BF16>(out, x, W, M, N, K, ldx, ldw, ldo, warps, stream);
    case ek::EPI_F32: return ek::launch<ek::EPI_F32>(out, x, W, M, N, K, ldx, ldw, ldo, warps, stream);
    case ek::EPI_SWIGLU: return ek::launch<ek::EPI_SWIGLU>(out, x, W, M, N, K, ldx, ldw, ldo, warps, stream);
  }
  return EK_ERR_ARG;
}
