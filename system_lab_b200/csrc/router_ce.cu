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

extern "C" int slab_ce_fwd_bwd(void* logits, const long* targets, float* loss_sum, int rows, int V, float gscale,
                               cudaStream_t st) {
  if (V % 8) return -100;
  if (rows == 0) return 0;
  int grid = rows < 148 * 4 ? rows : 148 * 4;
  ce_fwd_bwd_kernel<<<grid, 512, 0, st>>>((__nv_bfloat16*)logits, targets, loss_sum, rows, V, gscale);
  return (int)cudaGetLastError();
}
