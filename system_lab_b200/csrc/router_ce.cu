// Fused router (score function + bias + top-k + normalisation in one pass, one warp per token) and the
// softmax cross-entropy forward+backward that turns a chunk of logits into its gradient in place.
//
// Reference analogues: fused router with aux score (notes/2026-04/2026-04-25_gptoss_22_*:118-127),
// fused cross entropy (notes/2026-04/2026-04-19_gptoss_01_mlperf_best_e2e_run.md:85).
#include "common.cuh"

namespace slab {

constexpr int ROUTER_MAX_PER_LANE = 16;   // up to 512 experts

// logits: [T, E] fp32.  score: 0 softmax, 1 sigmoid.  bias (optional, [E]) only affects selection.
// Outputs: weights [T, K] fp32 (normalised over the selected experts if norm, times scaling), idx [T, K].
__global__ void router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                   float* __restrict__ weights, int* __restrict__ idx, int T, int E, int K,
                                   int score, int norm, float scaling) {
  const int warps = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int t = blockIdx.x * warps + (threadIdx.x >> 5); t < T; t += gridDim.x * warps) {
    float s[ROUTER_MAX_PER_LANE], sel[ROUTER_MAX_PER_LANE];
    const float* row = logits + (size_t)t * E;
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
      int e = lane + i * 32;
      s[i] = e < E ? row[e] : -INFINITY;
      mx = fmaxf(mx, s[i]);
    }
    if (score == 0) {
      mx = warp_max(mx);
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
        int e = lane + i * 32;
        s[i] = e < E ? __expf(s[i] - mx) : 0.f;
        sum += s[i];
      }
      sum = warp_sum(sum);
      const float inv = 1.f / sum;
#pragma unroll
      for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) s[i] *= inv;
    } else {
#pragma unroll
      for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
        int e = lane + i * 32;
        s[i] = e < E ? 1.f / (1.f + __expf(-s[i])) : 0.f;
      }
    }
#pragma unroll
    for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
      int e = lane + i * 32;
      sel[i] = e < E ? (s[i] + (bias ? bias[e] : 0.f)) : -INFINITY;
    }
    float wsum = 0.f;
    float my_w = 0.f;     // lane k keeps the k-th selection
    int my_i = 0;
    for (int k = 0; k < K; ++k) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
        int e = lane + i * 32;
        if (sel[i] > best) { best = sel[i]; bi = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        float ob = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      // owner lane publishes the (unbiased) score and retires the expert
      float sc = 0.f;
#pragma unroll
      for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
        if (lane + i * 32 == bi) { sc = s[i]; sel[i] = -INFINITY; }
      }
      sc = __shfl_sync(0xffffffffu, sc, bi & 31);
      wsum += sc;
      if (lane == k) { my_w = sc; my_i = bi; }
    }
    if (lane < K) {
      float w = norm ? my_w / (wsum + 1e-20f) : my_w;
      weights[(size_t)t * K + lane] = w * scaling;
      idx[(size_t)t * K + lane] = my_i;
    }
  }
}

// ---------------------------------------------------------------- fused router with load statistics + aux loss
// Scores of one token (softmax or sigmoid of its fp32 logits), spread over the warp: lane l holds experts
// l, l + 32, ...
__device__ __forceinline__ void router_scores(const float* __restrict__ row, int E, int score, int lane,
                                              float (&s)[ROUTER_MAX_PER_LANE]) {
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
    const int e = lane + i * 32;
    s[i] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, s[i]);
  }
  if (score == 0) {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
      const int e = lane + i * 32;
      s[i] = e < E ? __expf(s[i] - mx) : 0.f;
      sum += s[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) s[i] *= inv;
  } else {
#pragma unroll
    for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
      const int e = lane + i * 32;
      s[i] = e < E ? 1.f / (1.f + __expf(-s[i])) : 0.f;
    }
  }
}

constexpr float ROUTER_FIX = 1099511627776.f;      // 2^40: scores in [0, 1] as fixed point, exact integer sums

// Same selection as router_topk_kernel, plus in the same pass the statistics the load-balancing loss needs:
//   counts[e]  = pairs routed to expert e               (int)
//   p_fix[e]   = sum over tokens of score[t, e] * 2^40  (unsigned 64-bit fixed point: the sum does not depend on
//                the order in which blocks arrive, so the loss is reproducible bit for bit)
// and the loss itself, written by the last block to finish:
//   aux = aux_coeff * E * sum_e (counts[e] / (T K)) * (p_sum[e] / T)
// counts, p_fix and ticket must be zero on entry.
__global__ void __launch_bounds__(256)
router_fused_fwd_kernel(const float* __restrict__ logits, const float* __restrict__ bias, float* __restrict__ weights,
                        int* __restrict__ idx, int T, int E, int K, int score, int norm, float scaling,
                        int* __restrict__ counts, unsigned long long* __restrict__ p_fix, int* __restrict__ ticket,
                        float aux_coeff, float* __restrict__ aux_out) {
  __shared__ unsigned long long p_s[32 * ROUTER_MAX_PER_LANE];
  __shared__ int c_s[32 * ROUTER_MAX_PER_LANE];
  __shared__ float red[8];
  __shared__ int last;
  for (int e = threadIdx.x; e < E; e += blockDim.x) { p_s[e] = 0ull; c_s[e] = 0; }
  __syncthreads();
  const int warps = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  unsigned long long pacc[ROUTER_MAX_PER_LANE];     // this lane's experts, summed over the warp's tokens
#pragma unroll
  for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) pacc[i] = 0ull;
  for (int t = blockIdx.x * warps + (threadIdx.x >> 5); t < T; t += gridDim.x * warps) {
    float s[ROUTER_MAX_PER_LANE], sel[ROUTER_MAX_PER_LANE];
    router_scores(logits + (size_t)t * E, E, score, lane, s);
#pragma unroll
    for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
      const int e = lane + i * 32;
      sel[i] = e < E ? (s[i] + (bias ? bias[e] : 0.f)) : -INFINITY;
      pacc[i] += (unsigned long long)(s[i] * ROUTER_FIX);      // padding lanes hold score 0
    }
    float wsum = 0.f, my_w = 0.f;
    int my_i = 0;
    for (int k = 0; k < K; ++k) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
        const int e = lane + i * 32;
        if (sel[i] > best) { best = sel[i]; bi = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      float sc = 0.f;
#pragma unroll
      for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
        if (lane + i * 32 == bi) { sc = s[i]; sel[i] = -INFINITY; }
      }
      sc = __shfl_sync(0xffffffffu, sc, bi & 31);
      wsum += sc;
      if (lane == k) { my_w = sc; my_i = bi; }
    }
    if (lane < K) {
      const float w = norm ? my_w / (wsum + 1e-20f) : my_w;
      weights[(size_t)t * K + lane] = w * scaling;
      idx[(size_t)t * K + lane] = my_i;
      if (my_i >= 0 && my_i < E) atomicAdd(&c_s[my_i], 1);
    }
  }
#pragma unroll
  for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
    const int e = lane + i * 32;
    if (e < E && pacc[i]) atomicAdd(&p_s[e], pacc[i]);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    if (c_s[e]) atomicAdd(&counts[e], c_s[e]);
    if (p_s[e]) atomicAdd(&p_fix[e], p_s[e]);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = (atomicAdd(ticket, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (!last) return;
  __threadfence();
  float acc = 0.f;                                  // fixed order: thread i sums experts i, i + 256, ...
  for (int e = threadIdx.x; e < E && T > 0; e += blockDim.x) {
    const float f = (float)__ldcg(&counts[e]) / ((float)T * (float)K);
    const float pm = (float)((double)__ldcg(&p_fix[e]) / (double)ROUTER_FIX) / (float)T;
    acc += f * pm;
  }
  acc = warp_sum(acc);
  if (lane == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < warps; ++w) tot += red[w];
    *aux_out = aux_coeff * (float)E * tot;
  }
}

// Gradient of the fused router with respect to the logits, one warp per token: the scores are recomputed from
// the logits (cheaper than storing [T, E] of them), then
//   G[e]      = g_aux * aux_coeff * E * counts[e] / (T^2 K)                      (dense: the load-balancing loss)
//             + for the selected experts, the gate-weight path: with W = sum of the selected scores,
//               norm:  (scaling / W) * (gw[k] - sum_j gw[j] * s_j / W),   else  scaling * gw[k]
//   softmax:  dlogit[e] = s[e] * (G[e] - sum_j s[j] G[j]);     sigmoid:  dlogit[e] = G[e] * s[e] * (1 - s[e]).
// counts / g_aux may be null (no auxiliary loss).
__global__ void __launch_bounds__(256)
router_fused_bwd_kernel(const float* __restrict__ logits, const int* __restrict__ idx, const float* __restrict__ gw,
                        const int* __restrict__ counts, const float* __restrict__ g_aux, float aux_coeff,
                        float* __restrict__ dlogits, int T, int E, int K, int score, int norm, float scaling) {
  const int warps = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const float ga = (g_aux && counts) ? *g_aux * aux_coeff * (float)E / ((float)T * (float)T * (float)K) : 0.f;
  for (int t = blockIdx.x * warps + (threadIdx.x >> 5); t < T; t += gridDim.x * warps) {
    float s[ROUTER_MAX_PER_LANE], G[ROUTER_MAX_PER_LANE];
    router_scores(logits + (size_t)t * E, E, score, lane, s);
#pragma unroll
    for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
      const int e = lane + i * 32;
      G[i] = (ga != 0.f && e < E) ? ga * (float)counts[e] : 0.f;
    }
    // lane k < K holds selection k
    const int my_i = lane < K ? idx[(size_t)t * K + lane] : -1;
    const float my_g = lane < K ? gw[(size_t)t * K + lane] : 0.f;
    float my_s = 0.f;
    for (int k = 0; k < K; ++k) {
      const int e = __shfl_sync(0xffffffffu, my_i, k);
      float sc = 0.f;
#pragma unroll
      for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i)
        if (lane + i * 32 == e) sc = s[i];
      sc = __shfl_sync(0xffffffffu, sc, e & 31);
      if (lane == k) my_s = sc;
    }
    const float W = warp_sum(my_s) + 1e-20f;
    const float gdot = warp_sum(my_g * my_s) / W;          // sum_j gw[j] * s_j / W
    const float my_G = lane < K ? (norm ? (scaling / W) * (my_g - gdot) : scaling * my_g) : 0.f;
    for (int k = 0; k < K; ++k) {
      const int e = __shfl_sync(0xffffffffu, my_i, k);
      const float add = __shfl_sync(0xffffffffu, my_G, k);
#pragma unroll
      for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i)
        if (lane + i * 32 == e) G[i] += add;
    }
    float* out = dlogits + (size_t)t * E;
    if (score == 0) {
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) dot += s[i] * G[i];
      dot = warp_sum(dot);
#pragma unroll
      for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
        const int e = lane + i * 32;
        if (e < E) out[e] = s[i] * (G[i] - dot);
      }
    } else {
#pragma unroll
      for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
        const int e = lane + i * 32;
        if (e < E) out[e] = G[i] * s[i] * (1.f - s[i]);
      }
    }
  }
}

// One block per row: loss_row = logsumexp(logits) - logits[target]; logits <- (softmax - onehot) * gscale.
// `loss_sum` accumulates sum of row losses (fp32 atomics).  V % 8 == 0.
__global__ void __launch_bounds__(512)
ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const long* __restrict__ targets, float* __restrict__ loss_sum,
                  int rows, int V, float gscale) {
  __shared__ float red[32];
  __shared__ float bc[2];
  const int nvec = V >> 3;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    bf16x8* row = reinterpret_cast<bf16x8*>(logits + (size_t)r * V);
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      float f[8];
      unpack8(row[c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmaxf(mx, f[j]);
    }
    mx = warp_max(mx);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : -INFINITY;
      t = warp_max(t);
      if (threadIdx.x == 0) bc[0] = t;
    }
    __syncthreads();
    mx = bc[0];
    float sum = 0.f;
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      float f[8];
      unpack8(row[c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += __expf(f[j] - mx);
    }
    sum = warp_sum(sum);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
      t = warp_sum(t);
      if (threadIdx.x == 0) bc[1] = t;
    }
    __syncthreads();
    sum = bc[1];
    const long tgt = targets[r];
    if (threadIdx.x == 0) {
      float lt = __bfloat162float(logits[(size_t)r * V + tgt]);
      atomicAdd(loss_sum, logf(sum) + mx - lt);
    }
    __syncthreads();        // the target logit is read before anyone overwrites it
    const float inv = gscale / sum;
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      float f[8];
      unpack8(row[c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f[j] = __expf(f[j] - mx) * inv;
        if ((long)c * 8 + j == tgt) f[j] -= gscale;
      }
      row[c] = pack8(f);
    }
  }
}

}  // namespace slab

using namespace slab;

extern "C" int slab_router_topk(const float* logits, const float* bias, float* weights, int* idx, int T, int E,
                                int K, int score, int norm, float scaling, cudaStream_t st) {
  if (E > 32 * ROUTER_MAX_PER_LANE || K > 32 || K > E) return -100;
  if (T == 0) return 0;
  int blocks = (T + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  router_topk_kernel<<<blocks, 256, 0, st>>>(logits, bias, weights, idx, T, E, K, score, norm, scaling);
  return (int)cudaGetLastError();
}

// Router forward with load statistics and the load-balancing loss in one launch.  stats: int32 [3 * E + 2], zero on
// entry, laid out as counts [E] | p_fix [E] as unsigned 64-bit (2 ints each, 8-byte aligned because E is rounded to
// even by the caller's layout: offset (E + E % 2) ints) | ticket.  aux_out: fp32 [1].
extern "C" int slab_router_fused_fwd(const float* logits, const float* bias, float* weights, int* idx, int T, int E,
                                     int K, int score, int norm, float scaling, int* stats, float aux_coeff,
                                     float* aux_out, cudaStream_t st) {
  if (E > 32 * ROUTER_MAX_PER_LANE || K > 32 || K > E) return -100;
  if ((uintptr_t)stats & 7) return -101;
  int blocks = (T + 7) / 8;
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  const int e2 = E + (E & 1);
  router_fused_fwd_kernel<<<blocks, 256, 0, st>>>(logits, bias, weights, idx, T, E, K, score, norm, scaling, stats,
                                                  reinterpret_cast<unsigned long long*>(stats + e2), stats + e2 + 2 * E,
                                                  aux_coeff, aux_out);
  return (int)cudaGetLastError();
}

extern "C" int slab_router_fused_bwd(const float* logits, const int* idx, const float* gw, const int* counts,
                                     const float* g_aux, float aux_coeff, float* dlogits, int T, int E, int K,
                                     int score, int norm, float scaling, cudaStream_t st) {
  if (E > 32 * ROUTER_MAX_PER_LANE || K > 32 || K > E) return -100;
  if (T == 0) return 0;
  int blocks = (T + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  router_fused_bwd_kernel<<<blocks, 256, 0, st>>>(logits, idx, gw, counts, g_aux, aux_coeff, dlogits, T, E, K, score,
                                                  norm, scaling);
  return (int)cudaGetLastError();
}

extern "C" int slab_ce_fwd_bwd(void* logits, const long* targets, float* loss_sum, int rows, int V, float gscale,
                               cudaStream_t st) {
  if (V % 8) return -100;
  if (rows == 0) return 0;
  int grid = rows < 148 * 4 ? rows : 148 * 4;
  ce_fwd_bwd_kernel<<<grid, 512, 0, st>>>((__nv_bfloat16*)logits, targets, loss_sum, rows, V, gscale);
  return (int)cudaGetLastError();
}
