// Weight-streaming product for decode: out[M,N] = x[M,K] . W[N,K]^T with few rows
// (M <= 64 sequences) in bfloat16 and 32-bit accumulation.  The step is bound by
// reading W once from HBM, so the kernel is built around that stream:
//   * the weights are the 16-row operand of mma.sync.m16n8k16 and go from global
//     memory straight into registers with 16-byte loads - within a 32-wide slice of K
//     the contraction index is permuted identically for both operands, which lets each
//     thread fetch eight consecutive weights of one row (no shared-memory staging);
//   * the batch is the 8-column operand (M padded to a multiple of 8 in registers);
//   * K is split three ways to put enough bytes in flight on 148 SMs whatever N is: over
//     blocks (grid.y), over the warps of a block, and each warp issues the loads of
//     several slices before it uses the first;
//   * partial tiles are summed in a fixed order - warps in shared memory, blocks through
//     a scratch buffer where the block that arrives last (an atomic ticket, no waiting)
//     adds the others' partials in split order - so results are the same from run to run.
// The reference does this with Triton kernels that pad the batch to 16 rows
// (engine/ek_kernels.py:281-308 `_gemv_kernel`, 413-445 split-K parts summed by the
// consumer 447-470, 375-411 SwiGLU epilogue); the epilogues here are: store bfloat16,
// store 32-bit (logits), and SwiGLU, where one 16-row tile holds 8 gate rows and the 8
// matching up rows so that silu(gate) * up is formed in registers and the [M, 2I]
// intermediate is never written.
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
  // activations were written by the kernel before this one: an ordinary (coherent) load
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
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

template <int EPI>
__device__ __forceinline__ void store_tile(void* out, float4 s, int M, int m0, int ldo, int row_lo,
                                           int hi_offset, bool lo_ok, bool hi_ok) {
  // s.x, s.y: weight row lo, batch columns m0, m0+1;  s.z, s.w: weight row hi, same columns
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

// A tile is 16 weight rows:  lo = tile * lo_step + g  and  hi = lo + hi_offset  for g = 0..7
// (plain: lo_step 16, hi_offset 8; SwiGLU: lo_step 8, hi_offset I).  The work is the list of
// (tile, 32-wide slice of K) units in tile-major order; block b owns the contiguous run
// [b * units_per_block, (b+1) * units_per_block) of it, so every block streams the same
// number of bytes whatever N and K are.  A run covers at most one tile from its middle (its
// first, "head" segment), whole tiles, and at most one tile it does not finish ("tail").
// Whole tiles are stored directly; head and tail partials go to the block's two scratch slots
// and the last block to deliver a tile's partial adds them in block order (= K order).
template <int NT, int EPI>
__global__ void gemv_bf16_kernel(void* __restrict__ out, const bf16* x,
                                 const bf16* __restrict__ W, int M, int n_lo_rows, int K, int ldx,
                                 int ldw, int ldo, int lo_step, int hi_offset, int n_tiles,
                                 int units_per_block, float* __restrict__ partials,
                                 unsigned int* __restrict__ tickets) {
  constexpr int UNR = NT <= 2 ? 4 : (NT == 4 ? 2 : 1);   // slices whose loads are issued together
  extern __shared__ float red[];               // [warps][NT][32][4]
  __shared__ int is_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n_chunks = (K + 31) >> 5;
  const long long total = (long long)n_tiles * n_chunks;
  const long long u_begin = (long long)blockIdx.x * units_per_block;
  const long long u_end = min(total, u_begin + units_per_block);
  pdl_launch_dependents();

  pdl_wait();

  for (long long u = u_begin; u < u_end;) {
    const int tile = (int)(u / n_chunks);
    const int c_begin = (int)(u - (long long)tile * n_chunks);
    const int c_end = (int)min((long long)n_chunks, c_begin + (u_end - u));
    const int row_lo = tile * lo_step + g;
    // EPI_BF16/F32: n_lo_rows = N and both halves are checked against it.
    const bool lo_ok = row_lo < n_lo_rows;
    const bool hi_ok = (EPI == EPI_SWIGLU) ? lo_ok : (row_lo + hi_offset < n_lo_rows);
    const bf16* w_lo = W + (size_t)(lo_ok ? row_lo : 0) * ldw;
    const bf16* w_hi = W + (size_t)(hi_ok ? row_lo + hi_offset : 0) * ldw;

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    for (int c = c_begin + warp * UNR; c < c_end; c += warps * UNR) {
      uint4 a_lo[UNR], a_hi[UNR], b[UNR][NT];
#pragma unroll
      for (int i = 0; i < UNR; ++i) {
        const int k = ((c + i) << 5) + (t << 3);
        const bool ok = (c + i) < c_end && k < K;        // K is a multiple of 8
        a_lo[i] = ok ? ldg_stream(w_lo + k) : make_uint4(0, 0, 0, 0);
        a_hi[i] = ok ? ldg_stream(w_hi + k) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const int m = 8 * j + g;
          b[i][j] = (ok && m < M) ? ldg_cached(x + (size_t)m * ldx + k) : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int i = 0; i < UNR; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          mma_bf16(acc[j], a_lo[i].x, a_hi[i].x, a_lo[i].y, a_hi[i].y, b[i][j].x, b[i][j].y);
          mma_bf16(acc[j], a_lo[i].z, a_hi[i].z, a_lo[i].w, a_hi[i].w, b[i][j].z, b[i][j].w);
        }
    }

    // warps -> shared memory, summed in warp order by the first NT warps
    const bool whole = c_begin == 0 && c_end == n_chunks;
    // head segments (the tile was begun by an earlier block) use slot 0, tail segments slot 1
    float* my_slot = partials + ((size_t)blockIdx.x * 2 + (c_begin == 0 ? 1 : 0)) * NT * 128;
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
      if (whole) {
        store_tile<EPI>(out, s, M, 8 * j + 2 * t, ldo, row_lo, hi_offset, lo_ok, hi_ok);
      } else {
        *reinterpret_cast<float4*>(&my_slot[(j * 32 + lane) * 4]) = s;
      }
    }
    if (!whole) {
      // the block that delivers the tile's last partial adds all of them in block order
      const long long t_begin = (long long)tile * n_chunks;
      const int first_block = (int)(t_begin / units_per_block);
      const int last_block = (int)((t_begin + n_chunks - 1) / units_per_block);
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        const unsigned int ticket = atomicAdd(&tickets[tile], 1u);
        is_last = ticket == (unsigned int)(last_block - first_block);
        if (is_last) tickets[tile] = 0;        // ready for the next launch
      }
      __syncthreads();
      if (is_last) {
        __threadfence();
        for (int j = warp; j < NT; j += warps) {
          float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int b = first_block; b <= last_block; ++b) {
            // block b's segment of this tile starts at chunk 0 only if b's run starts at or
            // before the tile's first unit
            const bool starts_tile = (long long)b * units_per_block <= t_begin;
            const float4 p = __ldcg(reinterpret_cast<const float4*>(
                &partials[(((size_t)b * 2 + (starts_tile ? 1 : 0)) * NT + j) * 128 + lane * 4]));
            s.x += p.x; s.y += p.y; s.z += p.z; s.w += p.w;
          }
          store_tile<EPI>(out, s, M, 8 * j + 2 * t, ldo, row_lo, hi_offset, lo_ok, hi_ok);
        }
      }
    }
    __syncthreads();                           // `red` and `is_last` are reused
    u += c_end - c_begin;
  }
}

template <int NT, int EPI>
static int launch_nt(void* out, const void* x, const void* W, int M, int N, int K, int ldx, int ldw,
                     int ldo, int warps, int n_blocks, float* partials, unsigned int* tickets,
                     long long partial_floats, int n_tickets, cudaStream_t stream) {
  int tiles, lo_step, hi_offset, n_lo_rows;
  if (EPI == EPI_SWIGLU) {                     // N = 2 * I rows: gate rows then up rows
    const int inter = N / 2;
    tiles = (inter + 7) / 8; lo_step = 8; hi_offset = inter; n_lo_rows = inter;
  } else {
    tiles = (N + 15) / 16; lo_step = 16; hi_offset = 8; n_lo_rows = N;
  }
  const int n_chunks = (K + 31) / 32;
  const long long total = (long long)tiles * n_chunks;
  if (n_blocks > total) n_blocks = (int)total;
  long long per_block = (total + n_blocks - 1) / n_blocks;
  const bool can_share = partials && tickets && tiles <= n_tickets &&
                         (long long)n_blocks * 2 * NT * 128 <= partial_floats;
  if (!can_share || per_block % n_chunks == 0) {
    // whole tiles only: no tile is shared between blocks
    per_block = (per_block + n_chunks - 1) / n_chunks * n_chunks;
  }
  if (per_block > 2147483647LL) return EK_ERR_ARG;
  n_blocks = (int)((total + per_block - 1) / per_block);
  const size_t smem = (size_t)warps * NT * 32 * 4 * sizeof(float);
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(gemv_bf16_kernel<NT, EPI>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)launch_pdl(gemv_bf16_kernel<NT, EPI>, dim3(n_blocks), dim3(warps * 32), smem, stream,
                         out, (const bf16*)x, (const bf16*)W, M, n_lo_rows, K, ldx, ldw, ldo, lo_step,
                         hi_offset, tiles, (int)per_block, partials, tickets);
}

template <int EPI>
static int launch(void* out, const void* x, const void* W, int M, int N, int K, int ldx, int ldw,
                  int ldo, int warps, int n_blocks, float* partials, unsigned int* tickets,
                  long long partial_floats, int n_tickets, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || K % 8 || ldx % 8 || ldw % 8 || warps < 1 || warps > 32 || n_blocks < 1 ||
      (EPI == EPI_SWIGLU && (N & 1)))
    return EK_ERR_ARG;
  if (warps > 16) warps = 16;              // 8 batch tiles need up to 128 registers a thread
#define EK_GO(NT) \
  return launch_nt<NT, EPI>(out, x, W, M, N, K, ldx, ldw, ldo, warps, n_blocks, partials, tickets, \
                            partial_floats, n_tickets, stream)
  if (M <= 8) EK_GO(1);
  if (M <= 16) EK_GO(2);
  if (M <= 32) EK_GO(4);
  EK_GO(8);
#undef EK_GO
}

}  // namespace ek

// epilogue: 0 bfloat16 out [M,N]; 1 float out [M,N]; 2 SwiGLU, bfloat16 out [M,N/2].
// The (tile, K slice) work list is cut evenly over `n_blocks` blocks.  Tiles shared between
// blocks need `partials` (partial_floats 32-bit values, at least n_blocks * 2 * ceil8(M) * 16)
// and `tickets` (n_tickets >= number of 16-row tiles, unsigned ints, zero before the first
// launch; every launch leaves them zero).  Without them every block gets whole tiles.
EK_EXPORT int ek_gemv_bf16(void* out, const void* x, const void* W, int M, int N, int K, int ldx,
                           int ldw, int ldo, int epilogue, int warps, int n_blocks, float* partials,
                           unsigned int* tickets, long long partial_floats, int n_tickets,
                           cudaStream_t stream) {
  switch (epilogue) {
    case ek::EPI_BF16:
      return ek::launch<ek::EPI_BF16>(out, x, W, M, N, K, ldx, ldw, ldo, warps, n_blocks, partials,
                                      tickets, partial_floats, n_tickets, stream);
    case ek::EPI_F32:
      return ek::launch<ek::EPI_F32>(out, x, W, M, N, K, ldx, ldw, ldo, warps, n_blocks, partials,
                                     tickets, partial_floats, n_tickets, stream);
    case ek::EPI_SWIGLU:
      return ek::launch<ek::EPI_SWIGLU>(out, x, W, M, N, K, ldx, ldw, ldo, warps, n_blocks, partials,
                                        tickets, partial_floats, n_tickets, stream);
  }
  return EK_ERR_ARG;
}
