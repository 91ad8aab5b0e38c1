// Decode attention in bfloat16 with the cache pages streamed by TMA (head sizes 64 and 128,
// up to 16 query heads a KV head).
//
// One new token per sequence against its paged cache; the work is reading the sequence's keys
// and values once.  A block owns (token, KV head, split): a whole number of cache pages (64 keys
// each) of that head.
//   * warp 4, one thread: the producer.  A page's K and V tiles (64 x head_dim each) come by
//     cp.async.bulk.tensor into a ring of shared-memory stages, 128-byte swizzled, each stage
//     signalled by an mbarrier.  Old pages do not depend on the kernel before this one (only
//     the newest key and value do), so their copies are issued BEFORE the programmatic-launch
//     wait: the cache stream runs while the q/k/v product and the position encoding finish.
//   * warps 0-3: each takes 16 keys of a page.  The G query heads of the group are the 16 rows
//     of mma.sync.m16n8k16 (padded), K fragments come by ldmatrix, V fragments by
//     ldmatrix.trans, softmax is online in 32-bit in units of log2, P is rounded to bfloat16
//     before P.V - the same arithmetic as the register-streaming kernel in
//     attention_decode_bf16.cu, which remains for the other head sizes.
//   * the warps merge in shared memory; the splits of one (token, KV head) are a thread-block
//     cluster.  The (head, dimension) pairs are dealt to its blocks in equal runs; a block sends
//     its partial result for a pair, with its maximum and sum, into the shared memory of the
//     block that owns the pair (st.shared::cluster, into a buffer beside the ring, since the
//     owner may still be reading pages), and after one cluster barrier every block merges what
//     it was sent, in split order, and stores its run: no partials in global memory, no second
//     kernel, and no block has to outlive another's reads.
// The reference's counterpart is its Triton split-K flash-decoding kernel and combine kernel
// (engine/ek_kernels.py:534-615, 988-1019).  Every barrier wait is bounded and reports through
// `status`; every block of a cluster reaches the cluster barrier whatever happened to it.
#include "tc_common.cuh"

namespace ek {

constexpr int kDtWarps = 4;                  // consumer warps
constexpr int kDtThreads = (kDtWarps + 1) * 32;
constexpr int kDtPortableSplits = 8;         // blocks of a cluster: the portable limit
constexpr int kDtMaxSplits = 16;             // and the limit with the attribute for larger ones
// floats a block can be sent by its cluster: every (head, dimension) pair once (dealt in runs of
// ceil(pairs / splits), so up to one more a split), and (max, sum) of 16 heads from 16 splits
template <int D>
constexpr int kDtRecvO = 16 * D + kDtMaxSplits;
constexpr int kDtRecvMl = kDtMaxSplits * 16 * 2;

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                              uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
__device__ __forceinline__ void mma_bf16_16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// grid (splits, kv heads, tokens); cluster (splits, 1, 1) when splits > 1
template <int D, int STAGES>
__global__ void __launch_bounds__(kDtThreads)
attention_decode_tma_kernel(bf16* __restrict__ out, const bf16* q, int q_row_stride,
                            const int* positions, const int* token_slot,
                            const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* block_table,
                            int table_stride, int n_kv_heads, int n_q_heads, float scale_log2,
                            int window, int* status) {
  constexpr int DB = D / 64;                       // 64-wide (128-byte) blocks of the head dimension
  constexpr uint32_t kSub = EK_PAGE * 128;         // one [64 keys x 64 dims] sub-tile: 8 KB
  constexpr uint32_t kStage = 2 * DB * kSub;       // K tile + V tile
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * kStage);        // full[STAGES], empty[STAGES]
  // after the last page the ring is dead and holds, from its start: the warps' accumulators
  // [4][16][OS] and their (max, sum) [4][16][2].
  // A row of the accumulators is OS = D + 8 floats long, so that the rows a warp stores at once
  // (one per group of four lanes) lie on different banks.
  constexpr int OS = D + 8;
  float* o_s = (float*)smem;
  float* ml_s = o_s + kDtWarps * 16 * OS;
  static_assert((size_t)(kDtWarps * 16 * (OS + 2)) * 4 <= (size_t)STAGES * kStage,
                "merge buffers must fit the ring");
  // what the other blocks of the cluster send: [split][run] results, [split][head][2] (max, sum)
  float* recv_o = (float*)(bars + 2 * STAGES);
  float* recv_ml = recv_o + kDtRecvO<D>;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int split = blockIdx.x, n_splits = gridDim.x;
  const int kv_head = blockIdx.y, t = blockIdx.z;
  const int group = n_q_heads / n_kv_heads;
  const int head0 = kv_head * group;

  pdl_launch_dependents();
  if (tid == kDtWarps * 32) {
    tma_prefetch_map(&map_k);
    tma_prefetch_map(&map_v);
  }
  // Read before the wait: positions, slots and block tables must have been written by work that
  // a plain (not programmatic) launch separates from this kernel.  A step's first kernel, the
  // embedding lookup, is such a launch, so the state advance of the step before is complete and
  // visible here, in a captured graph and in eager decoding alike.
  const int pos = positions[t];
  int lo = 0, hi = -1, pg_first = 0, pg_last = -1;
  if (pos >= 0) {
    lo = window > 0 ? max(0, pos - window + 1) : 0;
    hi = pos;
    const int pg_lo = lo / EK_PAGE, pg_hi = hi / EK_PAGE;
    const int per = (pg_hi - pg_lo + n_splits) / n_splits;     // pages a split, rounded up
    pg_first = pg_lo + split * per;
    pg_last = min(pg_hi, pg_first + per - 1);
  }
  const int n_pages = pg_last - pg_first + 1;                  // <= 0: nothing for this split
  const int new_page = pos >= 0 ? pos / EK_PAGE : -1;          // holds the key written just now

  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), kDtWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  bool ok = true;
  float acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // rows g and g + 8

  if (tid == kDtWarps * 32) {
    // ------------------------------------------------------------------- TMA producer
    const int* table = block_table + (size_t)(pos >= 0 ? token_slot[t] : 0) * table_stride;
    bool waited = false;
    const uint64_t stream_policy = l2_policy_evict_first();   // a page is read once a step
    for (int i = 0; i < n_pages; ++i) {
      const int s = i % STAGES;
      const int pg = pg_first + i;
      if (i >= STAGES) {
        ok = mbar_wait(empty(s), ((i / STAGES) & 1) ^ 1, status, 41);
        if (!ok) break;
      }
      if (pg == new_page && !waited) {           // this page was written to by the kernel before
        pdl_wait();
        waited = true;
      }
      const int row = (table[pg] * n_kv_heads + kv_head) * EK_PAGE;
      const uint32_t dst = smem_u32(smem + s * kStage);
      mbar_expect_tx(full(s), kStage);
#pragma unroll
      for (int j = 0; j < DB; ++j) {
        tma_load_2d_hint(dst + j * kSub, &map_k, 64 * j, row, full(s), stream_policy);
        tma_load_2d_hint(dst + (DB + j) * kSub, &map_v, 64 * j, row, full(s), stream_policy);
      }
    }
  } else if (warp < kDtWarps) {
    // ------------------------------------------------------------------- consumers
    pdl_wait();                                  // the queries come from the kernel before
    if (n_pages > 0) {
      // Q fragments of m16n8k16 for every 16-wide step of the head dimension: rows g and g + 8
      uint32_t qa[D / 16][4];
      const bf16* qrow = q + (size_t)t * q_row_stride + (size_t)head0 * D;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int d0 = 16 * ks + 2 * tq;
        qa[ks][0] = g < group ? *reinterpret_cast<const uint32_t*>(qrow + (size_t)g * D + d0) : 0u;
        qa[ks][1] = g + 8 < group ? *reinterpret_cast<const uint32_t*>(qrow + (size_t)(g + 8) * D + d0) : 0u;
        qa[ks][2] = g < group ? *reinterpret_cast<const uint32_t*>(qrow + (size_t)g * D + d0 + 8) : 0u;
        qa[ks][3] = g + 8 < group ? *reinterpret_cast<const uint32_t*>(qrow + (size_t)(g + 8) * D + d0 + 8) : 0u;
      }
      // this lane's row and 16-byte column inside a [64 x 64] sub-tile for the two ldmatrix forms
      const int k_row = 16 * warp + (lane & 7) + 8 * (lane >> 4), k_half = (lane >> 3) & 1;
      const int v_row = 16 * warp + (lane & 7) + 8 * ((lane >> 3) & 1), v_half = lane >> 4;
      for (int i = 0; i < n_pages; ++i) {
        const int s = i % STAGES;
        ok = mbar_wait(full(s), (i / STAGES) & 1, status, 42);
        if (!ok) break;
        const int key0 = (pg_first + i) * EK_PAGE + 16 * warp;
        if (key0 <= hi && key0 + 15 >= lo) {     // else none of this warp's 16 keys is visible
          const uint32_t k_s = smem_u32(smem + s * kStage), v_s = k_s + DB * kSub;
          float sc[2][4];
          sc[0][0] = sc[0][1] = sc[0][2] = sc[0][3] = 0.f;
          sc[1][0] = sc[1][1] = sc[1][2] = sc[1][3] = 0.f;
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const int chunk = 2 * ks + k_half;               // 16-byte column of the head dimension
            uint32_t b0, b1, b2, b3;
            ldsm_x4(k_s + (chunk >> 3) * kSub + k_row * 128 + (((chunk & 7) ^ (k_row & 7)) << 4), b0, b1,
                    b2, b3);
            mma_bf16_16816(sc[0], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
            mma_bf16_16816(sc[1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
          }
          // sc[j][0..1]: row g, keys key0 + 8j + 2tq + {0,1}; sc[j][2..3]: row g + 8, same keys
          float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
          for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int key = key0 + 8 * j + 2 * tq + (e & 1);
              const float v = (key >= lo && key <= hi) ? sc[j][e] * scale_log2 : -INFINITY;
              sc[j][e] = v;
              mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
          float alpha[2];
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);      // finite: a key of the unit is visible
            alpha[r] = exp2f(m_run[r] - m_new);
            m_run[r] = m_new;
          }
          float psum[2] = {0.f, 0.f};
#pragma unroll
          for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float p = exp2f(sc[j][e] - m_run[e >> 1]);
              sc[j][e] = p;
              psum[e >> 1] += p;
            }
          l_run[0] = l_run[0] * alpha[0] + psum[0];
          l_run[1] = l_run[1] * alpha[1] + psum[1];
          const uint32_t p0 = pack2_bf16(sc[0][0], sc[0][1]), p1 = pack2_bf16(sc[0][2], sc[0][3]);
          const uint32_t p2 = pack2_bf16(sc[1][0], sc[1][1]), p3 = pack2_bf16(sc[1][2], sc[1][3]);
#pragma unroll
          for (int x = 0; x < D / 16; ++x) {
            const int chunk = 2 * x + v_half;
            uint32_t b0, b1, b2, b3;
            ldsm_x4_trans(v_s + (chunk >> 3) * kSub + v_row * 128 + (((chunk & 7) ^ (v_row & 7)) << 4), b0,
                          b1, b2, b3);
            float* a0 = acc[2 * x];
            float* a1 = acc[2 * x + 1];
            a0[0] *= alpha[0]; a0[1] *= alpha[0]; a0[2] *= alpha[1]; a0[3] *= alpha[1];
            a1[0] *= alpha[0]; a1[1] *= alpha[0]; a1[2] *= alpha[1]; a1[3] *= alpha[1];
            mma_bf16_16816(a0, p0, p1, p2, p3, b0, b1);
            mma_bf16_16816(a1, p0, p1, p2, p3, b2, b3);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty(s));
      }
    }
  }

  // ------------------------------------------------------------ the warps' results, merged
  const int failed = __syncthreads_or(ok ? 0 : 1);  // every page consumed: the ring is dead
  if (!failed && warp < kDtWarps) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    // acc[n][e]: row g (e < 2) or g + 8, dimension 8n + 2tq + (e & 1); only the group's rows
    // are real (the others pad the MMA's 16) and only those are stored and merged
    if (g < group) {
#pragma unroll
      for (int n = 0; n < D / 8; ++n)
        *reinterpret_cast<float2*>(o_s + ((size_t)warp * 16 + g) * OS + 8 * n + 2 * tq) =
            make_float2(acc[n][0], acc[n][1]);
      if (tq == 0) {
        ml_s[(warp * 16 + g) * 2] = m_run[0];
        ml_s[(warp * 16 + g) * 2 + 1] = l_run[0];
      }
    }
    if (g + 8 < group) {
#pragma unroll
      for (int n = 0; n < D / 8; ++n)
        *reinterpret_cast<float2*>(o_s + ((size_t)warp * 16 + g + 8) * OS + 8 * n + 2 * tq) =
            make_float2(acc[n][2], acc[n][3]);
      if (tq == 0) {
        ml_s[(warp * 16 + g + 8) * 2] = m_run[1];
        ml_s[(warp * 16 + g + 8) * 2 + 1] = l_run[1];
      }
    }
  }
  __syncthreads();
  const int pairs = group * D;
  const int run = (pairs + n_splits - 1) / n_splits;            // pairs a block of the cluster owns
  if (!failed) {
    // in warp order; a thread takes (row, dimension) pairs
    for (int idx = tid; idx < pairs; idx += kDtThreads) {
      const int r = idx / D, d = idx % D;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < kDtWarps; ++w) m = fmaxf(m, ml_s[(w * 16 + r) * 2]);
      float l = 0.f, o = 0.f;
#pragma unroll
      for (int w = 0; w < kDtWarps; ++w) {
        const float lw = ml_s[(w * 16 + r) * 2 + 1];
        if (lw > 0.f) {
          const float f = exp2f(ml_s[(w * 16 + r) * 2] - m);
          l += lw * f;
          o += o_s[((size_t)w * 16 + r) * OS + d] * f;
        }
      }
      if (n_splits == 1) {
        out[((size_t)t * n_q_heads + head0 + r) * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
      } else {
        const int owner = idx / run;
        st_cluster_f32(&recv_o[split * run + (idx - owner * run)], (unsigned)owner, o);
        if (d == 0) {                            // every block needs this head's maximum and sum
          for (int sp = 0; sp < n_splits; ++sp) {
            st_cluster_f32(&recv_ml[(split * 16 + r) * 2], (unsigned)sp, m);
            st_cluster_f32(&recv_ml[(split * 16 + r) * 2 + 1], (unsigned)sp, l);
          }
        }
      }
    }
  } else {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);     // let copies in flight land
  }
  if (n_splits == 1) return;

  // ------------------------------------------------------------ the splits, merged in order
  cluster_sync();                                // (every block gets here, whatever happened to it)
  if (!failed) {
    for (int slot = tid; slot < run && split * run + slot < pairs; slot += kDtThreads) {
      const int idx = split * run + slot;
      const int r = idx / D;
      float m = -INFINITY;
      for (int sp = 0; sp < n_splits; ++sp) m = fmaxf(m, recv_ml[(sp * 16 + r) * 2]);
      float l = 0.f, o = 0.f;
      for (int sp = 0; sp < n_splits; ++sp) {
        const float ls = recv_ml[(sp * 16 + r) * 2 + 1];
        if (ls > 0.f) {
          const float f = exp2f(recv_ml[(sp * 16 + r) * 2] - m);
          l += ls * f;
          o += recv_o[sp * run + slot] * f;
        }
      }
      out[((size_t)t * n_q_heads + head0) * D + idx] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
  }
}

// DEEP: a ring twice as deep (192 KB, one block an SM) for launches that leave SMs empty anyway, so
// that more of a block's pages are on their way before the wait returns.
template <int D, bool DEEP, bool QUERY = false>
static int launch_dt(bf16* out, const bf16* q, int q_row_stride, const int* positions,
                     const int* token_slot, const void* k_pages, const void* v_pages,
                     long long page_rows, const int* block_table, int table_stride, int n_tokens,
                     int n_q_heads, int n_kv_heads, float scale, int window, int n_splits, int* status,
                     cudaStream_t stream) {
  constexpr int STAGES = (D == 128 ? 3 : 6) * (DEEP ? 2 : 1);
  constexpr int DB = D / 64;
  constexpr size_t smem = 1024 + (size_t)STAGES * 2 * DB * EK_PAGE * 128 + 2 * STAGES * 8 +
                          (size_t)(kDtRecvO<D> + kDtRecvMl) * 4;
  CUtensorMap mk, mv;
  int rc;
  if (!QUERY) {
    if ((rc = tensor_map(k_pages, page_rows, D, D, EK_PAGE, &mk))) return rc;
    if ((rc = tensor_map(v_pages, page_rows, D, D, EK_PAGE, &mv))) return rc;
  }
  auto kernel = attention_decode_tma_kernel<D, STAGES>;
  static bool configured[kMaxDevices] = {};
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= kMaxDevices) return EK_ERR_ARG;
  if (!configured[device]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    if (!DEEP) {                                 // clusters of 9 to 16 blocks (two blocks an SM only)
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
      if (e != cudaSuccess) return (int)e;
    }
    configured[device] = true;
  }
  prefer_carveout((const void*)kernel, 100);
  dim3 grid(n_splits, n_kv_heads, n_tokens);
  if (QUERY) {                                   // can a cluster of 16 of these blocks run at all?
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kDtMaxSplits, 1, 1);
    cfg.blockDim = dim3(kDtThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kDtMaxSplits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    e = cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg);
    if (e != cudaSuccess) { cudaGetLastError(); return 0; }
    return clusters;
  }
  if (n_splits > 1)
    return (int)launch_pdl_cluster_x(kernel, grid, dim3(kDtThreads), smem, stream, n_splits, out, q,
                                     q_row_stride, positions, token_slot, mk, mv, block_table,
                                     table_stride, n_kv_heads, n_q_heads,
                                     scale * 1.4426950408889634f, window, status);
  return (int)launch_pdl(kernel, grid, dim3(kDtThreads), smem, stream, out, q, q_row_stride, positions,
                         token_slot, mk, mv, block_table, table_stride, n_kv_heads, n_q_heads,
                         scale * 1.4426950408889634f, window, status);
}

}  // namespace ek

// How many blocks may share a token on this device: 16 if clusters of that size can be
// scheduled for this head size, else 8 (0: the head size has no such kernel).
EK_EXPORT int ek_attention_decode_tma_max_splits(int head_dim) {
  using namespace ek;
  int clusters = 0;
  if (head_dim == 64)
    clusters = launch_dt<64, false, true>(nullptr, nullptr, 0, nullptr, nullptr, &clusters, &clusters, 64,
                                          nullptr, 0, 1, 1, 1, 1.f, 0, 1, nullptr, nullptr);
  else if (head_dim == 128)
    clusters = launch_dt<128, false, true>(nullptr, nullptr, 0, nullptr, nullptr, &clusters, &clusters, 64,
                                           nullptr, 0, 1, 1, 1, 1.f, 0, 1, nullptr, nullptr);
  else
    return 0;
  return clusters >= 1 ? kDtMaxSplits : kDtPortableSplits;
}

// head_dim 64 or 128; at most 16 query heads a KV head; 1 to 16 splits (each takes whole pages of
// the token's visible range); q rows 4-byte aligned; n_pages = pages in k_pages / v_pages
// ([pages, kv heads, 64, head_dim]); `status` is one int on the device.
EK_EXPORT int ek_attention_decode_tma(void* out, const void* q, int q_row_stride,
                                      const int* positions, const int* token_slot,
                                      const void* k_pages, const void* v_pages, int n_pages,
                                      const int* block_table, int table_stride, int n_tokens,
                                      int n_q_heads, int n_kv_heads, int head_dim, float scale,
                                      int window, int n_splits, int* status, cudaStream_t stream) {
  using namespace ek;
  if (n_tokens <= 0) return 0;
  if ((head_dim != 64 && head_dim != 128) || n_kv_heads <= 0 || n_q_heads % n_kv_heads ||
      n_q_heads / n_kv_heads > 16 || n_splits < 1 || n_splits > kDtMaxSplits || q_row_stride % 2 ||
      ((uintptr_t)q & 3) || !status || n_kv_heads > 65535 || n_tokens > 65535 || n_pages <= 0)
    return EK_ERR_ARG;
  const long long page_rows = (long long)n_pages * n_kv_heads * EK_PAGE;
  // one block an SM at most, and a cluster of the portable size (a deep ring is one block an SM)
  const bool deep = (long long)n_tokens * n_kv_heads * n_splits <= sm_count() && n_splits <= kDtPortableSplits;
#define EK_DT(D_, DEEP_)                                                                          \
  return launch_dt<D_, DEEP_>((bf16*)out, (const bf16*)q, q_row_stride, positions, token_slot,     \
                              k_pages, v_pages, page_rows, block_table, table_stride, n_tokens,   \
                              n_q_heads, n_kv_heads, scale, window, n_splits, status, stream)
  if (head_dim == 64) {
    if (deep) EK_DT(64, true);
    EK_DT(64, false);
  }
  if (deep) EK_DT(128, true);
  EK_DT(128, false);
#undef EK_DT
}
