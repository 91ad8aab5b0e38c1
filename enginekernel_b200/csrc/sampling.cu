// Picking the next token from 32-bit logits, and advancing the per-sequence decode
// state on the device so that a captured decode step needs no host round trip.
//
// Greedy is arg-max with ties to the lowest index, as torch.argmax in the reference
// (engine/ek_model.py:490-493).  Temperature and top-k sampling (not in the reference,
// which is greedy only) use the Gumbel-max rule: argmax_i(logit_i / T - log(-log u_i))
// over the k largest logits, with u_i from Philox-4x32-10 keyed by (seed) and counted by
// (vocabulary index / 4, draw number, sequence stream), so a draw depends on nothing
// else in the batch.  The state advance mirrors the reference's captured step body
// (engine/engine.py:284-292) with per-sequence positions and stop conditions added.
#include "common.cuh"

namespace ek {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              uint32_t k0, uint32_t k1, uint32_t out[4]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

__device__ __forceinline__ uint32_t order_key(float v) {   // larger float -> larger key
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct Best { float score; int index; };

__device__ __forceinline__ Best better(Best a, Best b) {
  if (b.score > a.score || (b.score == a.score && b.index < a.index)) return b;
  return a;
}

__device__ Best block_best(Best v, Best* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, v.score, o), __shfl_xor_sync(0xffffffffu, v.index, o)};
    v = better(v, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    Best t = lane < nw ? scratch[lane] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best other{__shfl_xor_sync(0xffffffffu, t.score, o), __shfl_xor_sync(0xffffffffu, t.index, o)};
      t = better(t, other);
    }
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// One block per row.  `active` (optional): rows whose entry is negative are skipped.
// `dyn` (optional, 4 ints on the device: temperature bits, top_k, seed low, seed high)
// replaces the by-value settings, so that a captured launch follows later changes.
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(int* __restrict__ out_token, const float* logits, long long row_stride, int vocab,
              float temperature, int top_k, unsigned long long seed, const int* streams,
              const int* draws, const int* active, const int* dyn) {
  __shared__ Best scratch[33];
  __shared__ unsigned int hist[256];
  __shared__ unsigned int sel_prefix, sel_remaining;
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x;
  if (active && active[row] < 0) return;
  if (dyn) {
    temperature = __int_as_float(dyn[0]);
    top_k = dyn[1];
    seed = (unsigned long long)(uint32_t)dyn[2] | ((unsigned long long)(uint32_t)dyn[3] << 32);
  }
  const float* x = logits + (size_t)row * row_stride;

  uint32_t threshold_key = 0;                    // keep logits whose key >= this
  if (temperature > 0.f && top_k > 0 && top_k < vocab) {
    // radix select of the top_k-th largest key, 8 bits at a time from the top
    if (tid == 0) { sel_prefix = 0; sel_remaining = (unsigned)top_k; }
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int i = tid; i < 256; i += blockDim.x) hist[i] = 0;
      __syncthreads();
      const uint32_t prefix = sel_prefix;
      const uint32_t mask = shift == 24 ? 0u : (0xFFFFFFFFu << (shift + 8));
      for (int i = tid; i < vocab; i += blockDim.x) {
        const uint32_t k = order_key(x[i]);
        if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        unsigned int need = sel_remaining;
        int bin = 255;
        for (; bin > 0; --bin) {
          if (hist[bin] >= need) break;
          need -= hist[bin];
        }
        sel_prefix = prefix | ((uint32_t)bin << shift);
        sel_remaining = need;
      }
      __syncthreads();
    }
    threshold_key = sel_prefix;
  }

  Best best{-INFINITY, 0x7fffffff};
  if (temperature > 0.f) {
    const float inv_t = 1.f / temperature;
    const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    const uint32_t stream = streams ? (uint32_t)streams[row] : (uint32_t)row;
    const uint32_t draw = draws ? (uint32_t)draws[row] : 0u;
    for (int g = tid; 4 * g < vocab; g += blockDim.x) {
      uint32_t w[4];
      philox4x32_10((uint32_t)g, draw, stream, 0u, k0, k1, w);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = 4 * g + j;
        if (i >= vocab) break;
        const float v = x[i];
        if (order_key(v) < threshold_key || !(v == v)) continue;
        const float u = ((float)(w[j] >> 9) + 0.5f) * (1.0f / 8388608.0f);
        const float score = v * inv_t - logf(-logf(u));
        best = better(best, Best{score, i});
      }
    }
  } else {
    for (int i = tid; i < vocab; i += blockDim.x) {
      const float v = x[i];
      if (v == v) best = better(best, Best{v, i});
    }
  }
  best = block_best(best, scratch);
  if (tid == 0) out_token[row] = best.index == 0x7fffffff ? 0 : best.index;
}

// Wide rows without top-k: the vocabulary is cut into `segments` pieces, one block each,
// whose best (score, index) pairs a second small kernel merges.  Maximum and tie rule are
// associative, so the result equals the one-block kernel's.
__global__ void __launch_bounds__(256)
sample_partial_kernel(float* __restrict__ part_score, int* __restrict__ part_index,
                      const float* logits, long long row_stride, int vocab, int segments,
                      float temperature, unsigned long long seed, const int* streams,
                      const int* draws, const int* active, const int* dyn) {
  __shared__ Best scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, seg = blockIdx.y, tid = threadIdx.x;
  if (active && active[row] < 0) return;
  if (dyn) {
    temperature = __int_as_float(dyn[0]);
    seed = (unsigned long long)(uint32_t)dyn[2] | ((unsigned long long)(uint32_t)dyn[3] << 32);
  }
  const float* x = logits + (size_t)row * row_stride;
  // segments are whole groups of 4 entries, so a Philox block never straddles two of them
  const int groups = (vocab + 3) / 4;
  const int per = (groups + segments - 1) / segments;
  const int g_begin = seg * per, g_end = min(groups, g_begin + per);
  Best best{-INFINITY, 0x7fffffff};
  if (temperature > 0.f) {
    const float inv_t = 1.f / temperature;
    const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    const uint32_t stream = streams ? (uint32_t)streams[row] : (uint32_t)row;
    const uint32_t draw = draws ? (uint32_t)draws[row] : 0u;
    for (int g = g_begin + tid; g < g_end; g += blockDim.x) {
      uint32_t w[4];
      philox4x32_10((uint32_t)g, draw, stream, 0u, k0, k1, w);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = 4 * g + j;
        if (i >= vocab) break;
        const float v = x[i];
        if (!(v == v)) continue;
        const float u = ((float)(w[j] >> 9) + 0.5f) * (1.0f / 8388608.0f);
        best = better(best, Best{v * inv_t - logf(-logf(u)), i});
      }
    }
  } else {
    for (int g = g_begin + tid; g < g_end; g += blockDim.x) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = 4 * g + j;
        if (i >= vocab) break;
        const float v = x[i];
        if (v == v) best = better(best, Best{v, i});
      }
    }
  }
  best = block_best(best, scratch);
  if (tid == 0) {
    part_score[(size_t)row * segments + seg] = best.score;
    part_index[(size_t)row * segments + seg] = best.index;
  }
}

__global__ void sample_final_kernel(int* __restrict__ out_token, const float* part_score,
                                    const int* part_index, int segments, const int* active) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  if (active && active[row] < 0) return;
  Best best{-INFINITY, 0x7fffffff};
  for (int s = threadIdx.x; s < segments; s += 32)
    best = better(best, Best{part_score[(size_t)row * segments + s], part_index[(size_t)row * segments + s]});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, best.score, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
    best = better(best, other);
  }
  if (threadIdx.x == 0) out_token[row] = best.index == 0x7fffffff ? 0 : best.index;
}

// The one-block kernel with a row spread over the 8 blocks of a thread-block cluster (wide
// vocabularies with top-k): every block counts the radix digits of its piece of the row, the
// blocks read one another's 256 counters through distributed shared memory and each takes the
// same decision, four times; then each samples its piece above the threshold and block 0 takes
// the best of the eight.  Same keys, same threshold, same noise (keyed by vocabulary index) and
// same tie rules as `sample_kernel`, so the token is the same.
constexpr int kTopkSegments = 8;

__device__ __forceinline__ unsigned int ld_cluster_u32(const unsigned int* own, unsigned rank) {
  unsigned a = (unsigned)__cvta_generic_to_shared(own), r, v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(r) : "memory");
  return v;
}

__global__ void __launch_bounds__(256)
sample_topk_cluster_kernel(int* __restrict__ out_token, const float* logits, long long row_stride,
                           int vocab, float temperature, int top_k, unsigned long long seed,
                           const int* streams, const int* draws, const int* active, const int* dyn) {
  __shared__ Best scratch[33];
  __shared__ unsigned int hist[256];
  __shared__ unsigned int warp_total[8];
  __shared__ unsigned int sel[2];                // digit chosen, keys still wanted below it
  __shared__ float mine_score;
  __shared__ int mine_index;
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, seg = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (active && active[row] < 0) return;         // the whole cluster (same row) leaves together
  if (dyn) {
    temperature = __int_as_float(dyn[0]);
    top_k = dyn[1];
    seed = (unsigned long long)(uint32_t)dyn[2] | ((unsigned long long)(uint32_t)dyn[3] << 32);
  }
  const float* x = logits + (size_t)row * row_stride;
  // pieces are whole groups of 4 entries, so a Philox block never straddles two of them
  const int groups = (vocab + 3) / 4;
  const int per = (groups + kTopkSegments - 1) / kTopkSegments;
  const int g_begin = min(groups, seg * per), g_end = min(groups, g_begin + per);
  const int i_begin = 4 * g_begin, i_end = min(vocab, 4 * g_end);

  uint32_t threshold_key = 0;                    // keep logits whose key >= this
  if (temperature > 0.f && top_k > 0 && top_k < vocab) {
    uint32_t prefix = 0, remaining = (uint32_t)top_k;
    for (int shift = 24; shift >= 0; shift -= 8) {
      hist[tid] = 0;
      __syncthreads();
      const uint32_t mask = shift == 24 ? 0u : (0xFFFFFFFFu << (shift + 8));
      for (int i = i_begin + tid; i < i_end; i += 256) {
        const uint32_t k = order_key(x[i]);
        if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1u);
      }
      cluster_sync();
      // thread t looks after digit 255 - t: keys of the whole row with that digit, and with
      // that digit or a larger one
      unsigned int v = 0;
#pragma unroll
      for (int r = 0; r < kTopkSegments; ++r) v += ld_cluster_u32(&hist[255 - tid], (unsigned)r);
      unsigned int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      if (lane == 31) warp_total[warp] = incl;
      __syncthreads();
      for (int w = 0; w < warp; ++w) incl += warp_total[w];
      const unsigned int excl = incl - v;
      // the largest digit whose count reaches what is still wanted; digit 0 if none does
      if (excl < remaining && (incl >= remaining || tid == 255)) {
        sel[0] = 255u - (unsigned)tid;
        sel[1] = remaining - excl;
      }
      __syncthreads();
      prefix |= sel[0] << shift;
      remaining = sel[1];
      cluster_sync();                            // the counters are zeroed again only after all have read them
    }
    threshold_key = prefix;
  }

  Best best{-INFINITY, 0x7fffffff};
  if (temperature > 0.f) {
    const float inv_t = 1.f / temperature;
    const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    const uint32_t stream = streams ? (uint32_t)streams[row] : (uint32_t)row;
    const uint32_t draw = draws ? (uint32_t)draws[row] : 0u;
    for (int g = g_begin + tid; g < g_end; g += 256) {
      uint32_t w[4];
      philox4x32_10((uint32_t)g, draw, stream, 0u, k0, k1, w);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = 4 * g + j;
        if (i >= vocab) break;
        const float v = x[i];
        if (order_key(v) < threshold_key || !(v == v)) continue;
        const float u = ((float)(w[j] >> 9) + 0.5f) * (1.0f / 8388608.0f);
        best = better(best, Best{v * inv_t - logf(-logf(u)), i});
      }
    }
  } else {
    for (int i = i_begin + tid; i < i_end; i += 256) {
      const float v = x[i];
      if (v == v) best = better(best, Best{v, i});
    }
  }
  best = block_best(best, scratch);
  if (tid == 0) {
    mine_score = best.score;
    mine_index = best.index;
  }
  cluster_sync();
  if (seg == 0 && tid < 32) {
    Best b{-INFINITY, 0x7fffffff};
    if (tid < kTopkSegments) {
      b.score = ld_cluster_f32(&mine_score, (unsigned)tid);
      b.index = (int)ld_cluster_u32(reinterpret_cast<const unsigned int*>(&mine_index), (unsigned)tid);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best other{__shfl_xor_sync(0xffffffffu, b.score, o), __shfl_xor_sync(0xffffffffu, b.index, o)};
      b = better(b, other);
    }
    if (tid == 0) out_token[row] = b.index == 0x7fffffff ? 0 : b.index;
  }
  cluster_sync();                                // nobody leaves while its result may be read
}

// After sampling: record the token, count the draw, decide whether the sequence goes on.
// A row whose position is negative is finished: it emits -1 and nothing of it changes.
__global__ void decode_advance_kernel(const int* sampled, int* token_ids, int* positions,
                                      int* draws, int* remaining, int* out_tokens,
                                      int* step_index, const int* __restrict__ stop_ids,
                                      int n_stop, int batch, int max_steps) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = threadIdx.x;
  const int step = *step_index;
  if (b < batch) {
    int emitted = -1;
    if (positions[b] >= 0) {
      const int tok = sampled[b];
      emitted = tok;
      draws[b] += 1;
      const int left = remaining[b] - 1;
      remaining[b] = left;
      bool stop = left <= 0;
      for (int i = 0; i < n_stop; ++i) stop |= (stop_ids[i] == tok);
      if (stop) {
        positions[b] = -1;
      } else {
        token_ids[b] = tok;
        positions[b] += 1;
      }
    }
    if (step < max_steps) out_tokens[(size_t)step * batch + b] = emitted;
  }
  __syncthreads();
  if (b == 0) *step_index = step + 1;
}

}  // namespace ek

EK_EXPORT int ek_sample(int* out_token, const float* logits, long long row_stride, int rows, int vocab,
                        float temperature, int top_k, unsigned long long seed, const int* streams,
                        const int* draws, const int* active, const int* dyn, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || temperature < 0.f || top_k < 0) return EK_ERR_ARG;
  return (int)ek::launch_pdl(ek::sample_kernel, dim3(rows), dim3(ek::kSampleThreads), 0, stream,
                             out_token, logits, row_stride, vocab, temperature, top_k, seed, streams,
                             draws, active, dyn);
}

// One launch, 8 blocks a row as a cluster; all of `ek_sample`'s modes, the same tokens.
EK_EXPORT int ek_sample_cluster(int* out_token, const float* logits, long long row_stride, int rows,
                                int vocab, float temperature, int top_k, unsigned long long seed,
                                const int* streams, const int* draws, const int* active,
                                const int* dyn, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || temperature < 0.f || top_k < 0 || rows > 2147483647) return EK_ERR_ARG;
  return (int)ek::launch_pdl_cluster(ek::sample_topk_cluster_kernel, dim3(rows, ek::kTopkSegments),
                                     dim3(256), 0, stream, ek::kTopkSegments, out_token, logits,
                                     row_stride, vocab, temperature, top_k, seed, streams, draws, active,
                                     dyn);
}

// Two launches over `segments` pieces of the vocabulary; top-k is not offered here.
// part_score / part_index: rows * segments values each.
EK_EXPORT int ek_sample_wide(int* out_token, const float* logits, long long row_stride, int rows,
                             int vocab, float temperature, unsigned long long seed,
                             const int* streams, const int* draws, const int* active,
                             const int* dyn, float* part_score, int* part_index, int segments,
                             cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || temperature < 0.f || segments < 1 || segments > 1024 || !part_score ||
      !part_index || rows > 65535)
    return EK_ERR_ARG;
  dim3 grid(rows, segments);
  cudaError_t e = ek::launch_pdl(ek::sample_partial_kernel, grid, dim3(256), 0, stream, part_score,
                                 part_index, logits, row_stride, vocab, segments, temperature, seed,
                                 streams, draws, active, dyn);
  if (e != cudaSuccess) return (int)e;
  return (int)ek::launch_pdl(ek::sample_final_kernel, dim3(rows), dim3(32), 0, stream, out_token,
                             (const float*)part_score, (const int*)part_index, segments, active);
}

EK_EXPORT int ek_decode_advance(const int* sampled, int* token_ids, int* positions, int* draws,
                                int* remaining, int* out_tokens, int* step_index,
                                const int* stop_ids, int n_stop, int batch, int max_steps,
                                cudaStream_t stream) {
  if (batch <= 0) return 0;
  if (batch > 1024) return EK_ERR_ARG;
  const int threads = ((batch + 31) / 32) * 32;
  return (int)ek::launch_pdl(ek::decode_advance_kernel, dim3(1), dim3(threads), 0, stream, sampled,
                             token_ids, positions, draws, remaining, out_tokens, step_index,
                             stop_ids, n_stop, batch, max_steps);
}
