// Bandwidth-bound fused ops: RMSNorm (+residual) fwd/bwd, SwiGLU(*probs) fwd/bwd without the
// concatenated gradient, RoPE, 1x128 / 128x128 fp8 quantisation, squared L2 norm and the flat AdamW
// step.  All activations are bf16, all arithmetic is fp32, every access is a 16-byte vector.
//
// Reference analogues: Triton RMSNorm with fp32 row partials for dgamma
// (notes/2026-04/2026-04-20_gptoss_02_triton_rmsnorm_optimization.md:47-62), fused residual+RMSNorm
// (notes/2026-04/2026-04-24_gptoss_17_fused_residual_rmsnorm_impl.md:43-83), SwiGLU*probs forward and
// no-cat backward (notes/2026-04/2026-04-25_gptoss_23_swiglu_nocat_triton_verify.md:92-113).
#include <cstdio>

#include "common.cuh"
#include "slab_noalloc.h"

namespace slab {

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

constexpr int NORM_THREADS = 256;
constexpr int NORM_WARPS = NORM_THREADS / 32;
constexpr int NORM_MAX_H = 16384;            // 8 warps x 32 lanes x 8 chunks x 8 elements
constexpr int NORM_GROUP = 8;                // blocks per first-level group of the gain-gradient reduction
constexpr int NORM_MAX_GRID = 296;           // two resident blocks on each of 148 SMs
constexpr int NORM_MAX_GROUPS = (NORM_MAX_GRID + NORM_GROUP - 1) / NORM_GROUP;
constexpr int NORM_COUNTERS = NORM_MAX_GROUPS + 1;   // one ticket counter per group + one for the groups

// Thread mapping shared by the forward and the backward: RW warps cooperate on one row (RW in {1, 2, 4, 8}), so a
// 256-thread block works on RPB = 8 / RW rows at a time; thread `li` of a row (0 .. 32 * RW) owns the 16-byte
// chunks li, li + 32 * RW, ... (CH of them).  A whole row is in flight per warp group, so the row sums need one
// warp shuffle reduction plus, for RW > 1, one exchange through shared memory (double buffered by iteration
// parity: one __syncthreads per row).
__device__ __forceinline__ float row_sum(float v, float (*red)[NORM_WARPS], int it, int warp, int rw, int rg) {
  v = warp_sum(v);
  if (rw == 1) return v;
  if ((threadIdx.x & 31) == 0) red[it & 1][warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int k = 0; k < rw; ++k) t += red[it & 1][rg * rw + k];
  return t;
}

// y = (x [+ res]) * rstd * w ; optionally writes xpr = x + res and rstd.
template <bool RESIDUAL, int RW, int CH>
__global__ void __launch_bounds__(NORM_THREADS, CH <= 4 ? 2 : 1)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ xpr, float* __restrict__ rstd_out, int rows, int H, float eps) {
  __shared__ float red[2][NORM_WARPS];
  constexpr int RPB = NORM_WARPS / RW;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rg = warp / RW;
  const int li = (warp % RW) * 32 + lane;
  const int nvec = H >> 3;
  bf16x8 wv[CH];
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const int c = li + i * 32 * RW;
    if (c < nvec) wv[i] = reinterpret_cast<const bf16x8*>(w)[c];
  }
  int it = 0;
  for (long r0 = (long)blockIdx.x * RPB; r0 < rows; r0 += (long)gridDim.x * RPB, ++it) {
    const long r = r0 + rg;
    const bool active = r < rows;
    float vals[CH][8];
    float ss = 0.f;
    if (active) {
      const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)r * H);
      const bf16x8* rr = RESIDUAL ? reinterpret_cast<const bf16x8*>(res + (size_t)r * H) : nullptr;
      bf16x8 xv[CH], rv[CH];
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int c = li + i * 32 * RW;
        if (c < nvec) {
          xv[i] = xr[c];
          if (RESIDUAL) rv[i] = rr[c];
        }
      }
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int c = li + i * 32 * RW;
        if (c < nvec) {
          unpack8(xv[i], vals[i]);
          if (RESIDUAL) {
            float e[8];
            unpack8(rv[i], e);
#pragma unroll
            for (int j = 0; j < 8; ++j) vals[i][j] += e[j];
            // the normalised value is computed from the fp32 sum; the stored sum is its bf16 rounding
            reinterpret_cast<bf16x8*>(xpr + (size_t)r * H)[c] = pack8(vals[i]);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
        }
      }
    }
    ss = row_sum(ss, red, it, warp, RW, rg);
    if (active) {
      const float rstd = rsqrtf(ss / H + eps);
      if (li == 0 && rstd_out) rstd_out[r] = rstd;
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int c = li + i * 32 * RW;
        if (c < nvec) {
          float wf[8], o[8];
          unpack8(wv[i], wf);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * rstd * wf[j];
          reinterpret_cast<bf16x8*>(y + (size_t)r * H)[c] = pack8(o);
        }
      }
    }
  }
}

// dx = rstd * (g*w) - x * rstd^3 * mean(g*w*x) [+ gres] ;  dw = sum_r g * x * rstd, finished inside this launch:
// every block leaves its fp32 partial in `scratch` (row blockIdx.x), the last block of each group of NORM_GROUP
// blocks to arrive sums the group's rows into row gridDim.x + group, and the last group to arrive sums those into
// the bf16 result -- a fixed summation order, so the result does not depend on which block arrives when.
// `scratch`: fp32 [gridDim.x + groups, H], contents irrelevant on entry.  `counters`: int [NORM_COUNTERS], all zero
// on entry and all zero again when the kernel ends.
template <bool ADD_RES, int RW, int CH>
__global__ void __launch_bounds__(NORM_THREADS, CH <= 4 ? 2 : 1)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ gres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ scratch, int* __restrict__ counters, __nv_bfloat16* __restrict__ dw_out,
                   int rows, int H) {
  __shared__ float red[2][NORM_WARPS];
  __shared__ float dw_s[RW == NORM_WARPS ? 8 : 32 * RW * CH * 8];   // block partial when several rows run side by side
  __shared__ int last_flag;
  constexpr int RPB = NORM_WARPS / RW;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rg = warp / RW;
  const int li = (warp % RW) * 32 + lane;
  const int nvec = H >> 3;
  const bf16x8* wp = reinterpret_cast<const bf16x8*>(w);   // re-read per row: a few KB that stay in L1
  float dw[CH][8];
#pragma unroll
  for (int i = 0; i < CH; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[i][j] = 0.f;
  }
  int it = 0;
  for (long r0 = (long)blockIdx.x * RPB; r0 < rows; r0 += (long)gridDim.x * RPB, ++it) {
    const long r = r0 + rg;
    const bool active = r < rows;
    bf16x8 xv[CH], gv[CH], ev[CH];
    float rstd = 0.f, dot = 0.f;
    if (active) {
      rstd = rstd_in[r];
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int c = li + i * 32 * RW;
        if (c < nvec) {
          xv[i] = reinterpret_cast<const bf16x8*>(x + (size_t)r * H)[c];
          gv[i] = reinterpret_cast<const bf16x8*>(g + (size_t)r * H)[c];
          if (ADD_RES) ev[i] = reinterpret_cast<const bf16x8*>(gres + (size_t)r * H)[c];
        }
      }
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int c = li + i * 32 * RW;
        if (c < nvec) {
          float xf[8], gf[8], wf[8];
          unpack8(xv[i], xf);
          unpack8(gv[i], gf);
          unpack8(wp[c], wf);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            dw[i][j] += gf[j] * xf[j] * rstd;
            dot += gf[j] * wf[j] * xf[j];
          }
        }
      }
    }
    dot = row_sum(dot, red, it, warp, RW, rg);
    if (active) {
      const float coef = dot * rstd * rstd * rstd / H;
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int c = li + i * 32 * RW;
        if (c < nvec) {
          float xf[8], gf[8], wf[8], o[8];
          unpack8(xv[i], xf);
          unpack8(gv[i], gf);
          unpack8(wp[c], wf);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = gf[j] * wf[j] * rstd - xf[j] * coef;
          if (ADD_RES) {
            float e[8];
            unpack8(ev[i], e);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] += e[j];
          }
          reinterpret_cast<bf16x8*>(dx + (size_t)r * H)[c] = pack8(o);
        }
      }
    }
  }
  // ---- this block's partial -> scratch row blockIdx.x
  float* my_row = scratch + (size_t)blockIdx.x * H;
  if (RPB == 1) {
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int c = li + i * 32 * RW;
      if (c < nvec) {
        *reinterpret_cast<float4*>(my_row + c * 8) = make_float4(dw[i][0], dw[i][1], dw[i][2], dw[i][3]);
        *reinterpret_cast<float4*>(my_row + c * 8 + 4) = make_float4(dw[i][4], dw[i][5], dw[i][6], dw[i][7]);
      }
    }
  } else {
    for (int sgrp = 0; sgrp < RPB; ++sgrp) {      // the row slots add their registers in turn (fixed order)
      __syncthreads();
      if (rg == sgrp) {
#pragma unroll
        for (int i = 0; i < CH; ++i) {
          const int c = li + i * 32 * RW;
          if (c < nvec) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (sgrp == 0) dw_s[c * 8 + j] = dw[i][j];
              else dw_s[c * 8 + j] += dw[i][j];
            }
          }
        }
      }
    }
    __syncthreads();
    for (int c4 = threadIdx.x; c4 < (H >> 2); c4 += NORM_THREADS)
      reinterpret_cast<float4*>(my_row)[c4] = reinterpret_cast<const float4*>(dw_s)[c4];
  }
  // ---- two-level reduction by the last arrivers
  const int grid = gridDim.x;
  const int n_groups = (grid + NORM_GROUP - 1) / NORM_GROUP;
  const int grp = blockIdx.x / NORM_GROUP;
  const int grp_first = grp * NORM_GROUP;
  const int grp_size = min(NORM_GROUP, grid - grp_first);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last_flag = (atomicAdd(&counters[grp], 1) == grp_size - 1);
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  float* grp_row = scratch + (size_t)(grid + grp) * H;
  for (int c4 = threadIdx.x; c4 < (H >> 2); c4 += NORM_THREADS) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < grp_size; ++k) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(scratch + (size_t)(grp_first + k) * H) + c4);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<float4*>(grp_row)[c4] = acc;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    counters[grp] = 0;                            // ready for the next launch
    last_flag = (atomicAdd(&counters[NORM_MAX_GROUPS], 1) == n_groups - 1);
  }
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  for (int c4 = threadIdx.x; c4 < (H >> 2); c4 += NORM_THREADS) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < n_groups; ++k) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(scratch + (size_t)(grid + k) * H) + c4);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(dw_out + c4 * 4);
    o[0] = __floats2bfloat162_rn(acc.x, acc.y);
    o[1] = __floats2bfloat162_rn(acc.z, acc.w);
  }
  if (threadIdx.x == 0) counters[NORM_MAX_GROUPS] = 0;
}

// ------------------------------------------------------------------ SwiGLU (* probs)
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// `rows_dev` (optional): device-side count of rows in use; rows beyond it are skipped (capacity-sized
// expert buffers are mostly empty).
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ probs,
                                  __nv_bfloat16* __restrict__ out, long rows, int F, const int* __restrict__ rows_dev) {
  if (rows_dev && *rows_dev < rows) rows = *rows_dev;
  const int fv = F >> 3;
  const long total = rows * fv;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    long r = i / fv;
    int c = int(i - r * fv);
    float g[8], u[8], o[8];
    const bf16x8* row = reinterpret_cast<const bf16x8*>(gu + r * 2 * F);
    unpack8(row[c], g);
    unpack8(row[fv + c], u);
    const float p = probs ? probs[r] : 1.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] * sigmoidf_(g[j]) * u[j] * p;
    reinterpret_cast<bf16x8*>(out + r * F)[c] = pack8(o);
  }
}

// One warp per row: writes d_gate | d_up into the two halves of dgu and the row sum d_probs.
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ gu,
                                  const float* __restrict__ probs, __nv_bfloat16* __restrict__ dgu,
                                  float* __restrict__ dprobs, long rows, int F, const int* __restrict__ rows_dev) {
  if (rows_dev && *rows_dev < rows) rows = *rows_dev;
  const int fv = F >> 3;
  const int warps = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long r = blockIdx.x * (long)warps + (threadIdx.x >> 5); r < rows; r += (long)gridDim.x * warps) {
    const bf16x8* grow = reinterpret_cast<const bf16x8*>(gu + r * 2 * F);
    const bf16x8* drow = reinterpret_cast<const bf16x8*>(dout + r * F);
    bf16x8* orow = reinterpret_cast<bf16x8*>(dgu + r * 2 * F);
    const float p = probs ? probs[r] : 1.f;
    float dp = 0.f;
    for (int c = lane; c < fv; c += 32) {
      float g[8], u[8], d[8], dg[8], du[8];
      unpack8(grow[c], g);
      unpack8(grow[fv + c], u);
      unpack8(drow[c], d);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float s = sigmoidf_(g[j]);
        float act = g[j] * s;
        dp += d[j] * act * u[j];
        float dpd = d[j] * p;
        du[j] = dpd * act;
        dg[j] = dpd * u[j] * s * (1.f + g[j] * (1.f - s));
      }
      orow[c] = pack8(dg);
      orow[fv + c] = pack8(du);
    }
    if (dprobs) {
      dp = warp_sum(dp);
      if (lane == 0) dprobs[r] = dp;
    }
  }
}

// ------------------------------------------------------------------ RoPE (half-split)
// x: rows of `Hh` heads x D, `row_stride` elements apart (a packed qkv buffer rotates only its first Hh
// heads); cos/sin: [S, D/2] fp32; sign = +1 forward, -1 backward.  y may alias x (in place).
__global__ void rope_kernel(const __nv_bfloat16* x, const float* __restrict__ cs, const float* __restrict__ sn,
                            __nv_bfloat16* y, long n_tok, int S, int Hh, int D, long row_stride_x,
                            long row_stride_y, float sign) {
  const int d2 = D >> 1;
  const int vec_per_half = d2 >> 3;          // vec8 chunks per half head
  const long per_tok = (long)Hh * vec_per_half;
  const long total = n_tok * per_tok;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    long tok = i / per_tok;
    int rem = int(i - tok * per_tok);
    int head = rem / vec_per_half, c = rem - head * vec_per_half;
    int s = int(tok % S);
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + tok * row_stride_x + (long)head * D);
    float a[8], b[8], co[8], si[8], oa[8], ob[8];
    unpack8(xr[c], a);
    unpack8(xr[vec_per_half + c], b);
    const float4* cp = reinterpret_cast<const float4*>(cs + (size_t)s * d2 + c * 8);
    const float4* sp = reinterpret_cast<const float4*>(sn + (size_t)s * d2 + c * 8);
    float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    co[0] = c0.x; co[1] = c0.y; co[2] = c0.z; co[3] = c0.w; co[4] = c1.x; co[5] = c1.y; co[6] = c1.z; co[7] = c1.w;
    si[0] = s0.x; si[1] = s0.y; si[2] = s0.z; si[3] = s0.w; si[4] = s1.x; si[5] = s1.y; si[6] = s1.z; si[7] = s1.w;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float sj = si[j] * sign;
      oa[j] = a[j] * co[j] - b[j] * sj;
      ob[j] = b[j] * co[j] + a[j] * sj;
    }
    bf16x8* yr = reinterpret_cast<bf16x8*>(y + tok * row_stride_y + (long)head * D);
    yr[c] = pack8(oa);
    yr[vec_per_half + c] = pack8(ob);
  }
}

// ------------------------------------------------------------------ fp8 block quantisation
// 1x128: one warp per (row, 128-column block): 4 elements per lane.
__global__ void quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, __nv_fp8_e4m3* __restrict__ q,
                                   float* __restrict__ scale, long rows, int H) {
  const int nb = H >> 7;
  const int warps = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const long total = rows * nb;
  for (long w = blockIdx.x * (long)warps + (threadIdx.x >> 5); w < total; w += (long)gridDim.x * warps) {
    long r = w / nb;
    int b = int(w - r * nb);
    const __nv_bfloat162* src = reinterpret_cast<const __nv_bfloat162*>(x + r * H + b * 128 + lane * 4);
    float2 v0 = __bfloat1622float2(src[0]), v1 = __bfloat1622float2(src[1]);
    float amax = fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v1.x), fabsf(v1.y)));
    amax = fmaxf(warp_max(amax), 1e-12f);
    const float sc = amax / 448.f;
    const float inv = 448.f / amax;
    __nv_fp8_e4m3 o[4] = {__nv_fp8_e4m3(v0.x * inv), __nv_fp8_e4m3(v0.y * inv), __nv_fp8_e4m3(v1.x * inv),
                          __nv_fp8_e4m3(v1.y * inv)};
    *reinterpret_cast<uint32_t*>(q + r * H + b * 128 + lane * 4) = *reinterpret_cast<uint32_t*>(o);
    if (lane == 0) scale[r * nb + b] = sc;
  }
}

// Row-wise: one scale per row (activations: per token; weights viewed as [E*N, K]: per output channel).
// One warp per row, two passes over the row (the second pass hits L1/L2).
__global__ void quant_rowwise_kernel(const __nv_bfloat16* __restrict__ x, __nv_fp8_e4m3* __restrict__ q,
                                     float* __restrict__ scale, long rows, int H) {
  const int warps = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (long r = blockIdx.x * (long)warps + (threadIdx.x >> 5); r < rows; r += (long)gridDim.x * warps) {
    const bf16x8* src = reinterpret_cast<const bf16x8*>(x + r * H);
    float amax = 0.f;
    for (int c = lane; c < nvec; c += 32) {
      float v[8];
      unpack8(src[c], v);
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    }
    amax = fmaxf(warp_max(amax), 1e-12f);
    const float inv = 448.f / amax;
    uint2* dst = reinterpret_cast<uint2*>(q + r * H);
    for (int c = lane; c < nvec; c += 32) {
      float v[8];
      unpack8(src[c], v);
      __nv_fp8_e4m3 o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = __nv_fp8_e4m3(v[j] * inv);
      dst[c] = *reinterpret_cast<uint2*>(o);
    }
    if (lane == 0) scale[r] = amax / 448.f;
  }
}

// 128x128: one block (256 threads) per weight block.
__global__ void __launch_bounds__(256)
quant_128x128_kernel(const __nv_bfloat16* __restrict__ w, __nv_fp8_e4m3* __restrict__ q, float* __restrict__ scale,
                     int N, int K) {
  __shared__ float red[32];
  const int kb = blockIdx.x, nb = blockIdx.y;
  const long mat = blockIdx.z;
  const __nv_bfloat16* base = w + mat * (long)N * K + (long)nb * 128 * K + kb * 128;
  float vals[8][8];
  float amax = 0.f;
  // 128 rows x 16 vec8 = 2048 vec8 chunks, 8 per thread
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int idx = threadIdx.x + i * 256;
    int r = idx >> 4, c = idx & 15;
    unpack8(*reinterpret_cast<const bf16x8*>(base + (long)r * K + c * 8), vals[i]);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(vals[i][j]));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  amax = fmaxf(amax, 1e-12f);
  const float inv = 448.f / amax;
  if (threadIdx.x == 0) scale[mat * (long)(N / 128) * (K / 128) + (long)nb * (K / 128) + kb] = amax / 448.f;
  __nv_fp8_e4m3* qb = q + mat * (long)N * K + (long)nb * 128 * K + kb * 128;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int idx = threadIdx.x + i * 256;
    int r = idx >> 4, c = idx & 15;
    __nv_fp8_e4m3 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __nv_fp8_e4m3(vals[i][j] * inv);
    *reinterpret_cast<uint2*>(qb + (long)r * K + c * 8) = *reinterpret_cast<uint2*>(o);
  }
}

// ------------------------------------------------------------------ squared L2 norm (fp32 input)
template <typename G>
__global__ void sumsq_kernel(const G* __restrict__ g, long n, float scale, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  const long nv = n >> 2;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nv; i += (long)gridDim.x * blockDim.x) {
    if (sizeof(G) == 4) {
      float4 v = reinterpret_cast<const float4*>(g)[i];
      s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    } else {
      const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(g) + 2 * i;
      float2 a = __bfloat1622float2(gp[0]), b = __bfloat1622float2(gp[1]);
      s += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long i = nv << 2; i < n; ++i) {
      float v = float(g[i]);
      s += v * v;
    }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s * scale);
}

// ------------------------------------------------------------------ flat AdamW
// One thread handles 4 consecutive elements; a 128-element block (one fp8 scale) is one warp.
// P: master/weight dtype (float or bf16).  State kinds: 0 fp32, 1 bf16, 2 fp8 (e4m3 + per-128 fp32
// scale; v is stored as sqrt(v)).  `coef` is the clip coefficient on the device (no host sync).
struct AdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2;
  long decay_end;      // elements [0, decay_end) of the shard get weight decay, the rest (norm gains: 1-D parameters,
                       // packed at the tail of a flat group on 128-element boundaries) do not
};

// 16 consecutive elements per thread (16-byte accesses for every storage type); the 8 threads that share a
// 128-element scale block are neighbouring lanes.  If `sq_out` is given the kernel also adds sum(g^2) of the
// raw gradient to it (the global-norm accumulation of the optimizer-in-backward mode).
template <typename T>
__device__ __forceinline__ void load16(const T* base, long i, float (&f)[16]);
template <>
__device__ __forceinline__ void load16<float>(const float* base, long i, float (&f)[16]) {
  const float4* p = reinterpret_cast<const float4*>(base) + 4 * i;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float4 t = p[k];
    f[4 * k] = t.x; f[4 * k + 1] = t.y; f[4 * k + 2] = t.z; f[4 * k + 3] = t.w;
  }
}
template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* base, long i, float (&f)[16]) {
  const bf16x8* p = reinterpret_cast<const bf16x8*>(base) + 2 * i;
  float a[8], b[8];
  unpack8(p[0], a);
  unpack8(p[1], b);
#pragma unroll
  for (int k = 0; k < 8; ++k) { f[k] = a[k]; f[8 + k] = b[k]; }
}
template <typename T>
__device__ __forceinline__ void store16(T* base, long i, const float (&f)[16]);
template <>
__device__ __forceinline__ void store16<float>(float* base, long i, const float (&f)[16]) {
  float4* p = reinterpret_cast<float4*>(base) + 4 * i;
#pragma unroll
  for (int k = 0; k < 4; ++k) p[k] = make_float4(f[4 * k], f[4 * k + 1], f[4 * k + 2], f[4 * k + 3]);
}
template <>
__device__ __forceinline__ void store16<__nv_bfloat16>(__nv_bfloat16* base, long i, const float (&f)[16]) {
  bf16x8* p = reinterpret_cast<bf16x8*>(base) + 2 * i;
  float a[8], b[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) { a[k] = f[k]; b[k] = f[8 + k]; }
  p[0] = pack8(a);
  p[1] = pack8(b);
}

template <typename P, int KIND, typename G>
__global__ void __launch_bounds__(256)
adamw_kernel(P* __restrict__ p, const G* __restrict__ g, void* __restrict__ m_raw, void* __restrict__ v_raw,
             float* __restrict__ m_scale, float* __restrict__ v_scale, __nv_bfloat16* __restrict__ out_bf16,
             const float* __restrict__ coef, float* __restrict__ sq_out, long q_begin, long nq, AdamArgs a) {
  // One launch covers the 16-element items [q_begin, nq); q_begin is a multiple of 32.
  __shared__ float red[32];
  const float c = coef ? *coef : 1.f;
  float sq = 0.f;
  // warp-uniform trip count: lanes past the end idle through the body so the block-scale shuffles stay full-warp
  for (long i0 = q_begin + blockIdx.x * (long)blockDim.x + (threadIdx.x & ~31); i0 < nq;
       i0 += (long)gridDim.x * blockDim.x) {
    const long i = i0 + (threadIdx.x & 31);
    const bool act = i < nq;
    if (!act && KIND != 2) continue;
    if (!act) {                                  // nq is a multiple of 8, so whole 8-lane groups are idle together
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {
        __shfl_xor_sync(0xffffffffu, 0.f, o);
        __shfl_xor_sync(0xffffffffu, 0.f, o);
      }
      continue;
    }
    const long e0 = i << 4;
    const float decay = e0 < a.decay_end ? 1.f - a.lr * a.wd : 1.f;
    float gv[16], mv[16], vv[16], pv[16];
    load16<G>(g, i, gv);
    load16<P>(p, i, pv);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      sq += gv[j] * gv[j];
      gv[j] *= c;
    }
    if (KIND == 0) {
      load16<float>(reinterpret_cast<const float*>(m_raw), i, mv);
      load16<float>(reinterpret_cast<const float*>(v_raw), i, vv);
    } else if (KIND == 1) {
      load16<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(m_raw), i, mv);
      load16<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(v_raw), i, vv);
#pragma unroll
      for (int j = 0; j < 16; ++j) vv[j] *= vv[j];
    } else {
      const float ms = m_scale[e0 >> 7], vs = v_scale[e0 >> 7];
      uint4 mq = reinterpret_cast<const uint4*>(m_raw)[i], vq = reinterpret_cast<const uint4*>(v_raw)[i];
      const __nv_fp8_e4m3* m8 = reinterpret_cast<const __nv_fp8_e4m3*>(&mq);
      const __nv_fp8_e4m3* v8 = reinterpret_cast<const __nv_fp8_e4m3*>(&vq);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        mv[j] = float(m8[j]) * ms;
        float sv = float(v8[j]) * vs;
        vv[j] = sv * sv;
      }
    }
    float m_amax = 0.f, v_amax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      mv[j] = a.beta1 * mv[j] + (1.f - a.beta1) * gv[j];
      vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gv[j] * gv[j];
      const float denom = sqrtf(vv[j] / a.bc2) + a.eps;
      pv[j] = pv[j] * decay - a.lr * (mv[j] / a.bc1) / denom;
      if (KIND != 0) vv[j] = sqrtf(vv[j]);        // stored in the sqrt domain
      m_amax = fmaxf(m_amax, fabsf(mv[j]));
      v_amax = fmaxf(v_amax, vv[j]);
    }
    store16<P>(p, i, pv);
    if (out_bf16) store16<__nv_bfloat16>(out_bf16, i, pv);
    if (KIND == 0) {
      store16<float>(reinterpret_cast<float*>(m_raw), i, mv);
      store16<float>(reinterpret_cast<float*>(v_raw), i, vv);
    } else if (KIND == 1) {
      store16<__nv_bfloat16>(reinterpret_cast<__nv_bfloat16*>(m_raw), i, mv);
      store16<__nv_bfloat16>(reinterpret_cast<__nv_bfloat16*>(v_raw), i, vv);
    } else {
      // 8 neighbouring lanes cover one 128-element scale block
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {
        m_amax = fmaxf(m_amax, __shfl_xor_sync(0xffffffffu, m_amax, o));
        v_amax = fmaxf(v_amax, __shfl_xor_sync(0xffffffffu, v_amax, o));
      }
      m_amax = fmaxf(m_amax, 1e-30f);
      v_amax = fmaxf(v_amax, 1e-30f);
      const float mi = 448.f / m_amax, vi = 448.f / v_amax;
      uint4 mo, vo;
      __nv_fp8_e4m3* m8 = reinterpret_cast<__nv_fp8_e4m3*>(&mo);
      __nv_fp8_e4m3* v8 = reinterpret_cast<__nv_fp8_e4m3*>(&vo);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        m8[j] = __nv_fp8_e4m3(mv[j] * mi);
        v8[j] = __nv_fp8_e4m3(vv[j] * vi);
      }
      reinterpret_cast<uint4*>(m_raw)[i] = mo;
      reinterpret_cast<uint4*>(v_raw)[i] = vo;
      if ((threadIdx.x & 7) == 0) {
        m_scale[e0 >> 7] = m_amax / 448.f;
        v_scale[e0 >> 7] = v_amax / 448.f;
      }
    }
  }
  if (sq_out) {
    sq = block_sum(sq, red);
    if (threadIdx.x == 0) atomicAdd(sq_out, sq);
  }
}

static inline int sm_count_cached() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 148;
  }
  return sms;
}

static inline int grid_for(long work_items, int threads, int per_sm = 8) {
  const int sms = sm_count_cached();
  long blocks = (work_items + threads - 1) / threads;
  long cap = (long)sms * per_sm;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace slab

using namespace slab;

// Warps per row and chunks per thread for a hidden size (see the thread mapping above): at most 4 chunks per
// thread up to H = 8192, 8 beyond.
static void norm_shape(int H, int* rw, int* ch) {
  const int nvec = H / 8;
  int r = 1;
  while (r < NORM_WARPS && nvec > 32 * r * 4) r *= 2;
  int per = (nvec + 32 * r - 1) / (32 * r);
  int c = 1;
  while (c < per) c *= 2;
  *rw = r;
  *ch = c;
}

static int norm_grid(int rows, int rw, int ch, int max_grid) {
  const int rpb = NORM_WARPS / rw;
  long want = ((long)rows + rpb - 1) / rpb;
  int cap = sm_count_cached() * (ch <= 4 ? 2 : 1);
  if (cap > NORM_MAX_GRID) cap = NORM_MAX_GRID;
  if (cap > max_grid) cap = sm_count_cached() <= max_grid ? sm_count_cached() : max_grid;   // whole waves where possible
  if (want < 1) want = 1;
  return (int)(want < cap ? want : cap);
}

#define SLAB_NORM_DISPATCH(LAUNCH)                     \
  do {                                                 \
    if (rw == 1 && ch == 1) LAUNCH(1, 1);              \
    else if (rw == 1 && ch == 2) LAUNCH(1, 2);         \
    else if (rw == 1 && ch == 4) LAUNCH(1, 4);         \
    else if (rw == 2) LAUNCH(2, 4);                    \
    else if (rw == 4) LAUNCH(4, 4);                    \
    else if (ch <= 4) LAUNCH(8, 4);                    \
    else LAUNCH(8, 8);                                 \
  } while (0)

extern "C" int slab_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* xpr, float* rstd,
                                int rows, int H, float eps, cudaStream_t st) {
  if (H % 8 || H > NORM_MAX_H) return -100;
  if (rows < 1) return 0;
  int rw, ch;
  norm_shape(H, &rw, &ch);
  const int grid = norm_grid(rows, rw, ch, NORM_MAX_GRID);
#define SLAB_FWD(RW, CH)                                                                                             \
  do {                                                                                                               \
    if (res)                                                                                                         \
      rmsnorm_fwd_kernel<true, RW, CH><<<grid, NORM_THREADS, 0, st>>>(                                               \
          (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w, (__nv_bfloat16*)y,            \
          (__nv_bfloat16*)xpr, rstd, rows, H, eps);                                                                  \
    else                                                                                                             \
      rmsnorm_fwd_kernel<false, RW, CH><<<grid, NORM_THREADS, 0, st>>>(                                              \
          (const __nv_bfloat16*)x, nullptr, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, nullptr, rstd, rows, H, eps); \
  } while (0)
  SLAB_NORM_DISPATCH(SLAB_FWD);
#undef SLAB_FWD
  return (int)cudaGetLastError();
}

// Rows of fp32 [*, H] scratch and ints of zeroed counters a backward call needs, whatever its row count.
extern "C" int slab_rmsnorm_bwd_blocks(int rows) { (void)rows; return NORM_MAX_GRID + NORM_MAX_GROUPS; }
extern "C" int slab_rmsnorm_bwd_counters() { return NORM_COUNTERS; }

static int launch_rmsnorm_bwd(const void* g, const void* x, const void* w, const float* rstd, const void* gres,
                              void* dx, float* scratch, int* counters, void* dw, int rows, int H, int max_rows,
                              cudaStream_t st) {
  int rw, ch;
  norm_shape(H, &rw, &ch);
  // scratch rows in use: grid + ceil(grid / NORM_GROUP) <= max_rows
  int max_grid = max_rows * NORM_GROUP / (NORM_GROUP + 1);
  while (max_grid > 1 && max_grid + (max_grid + NORM_GROUP - 1) / NORM_GROUP > max_rows) --max_grid;
  const int grid = norm_grid(rows < 1 ? 1 : rows, rw, ch, max_grid);
#define SLAB_BWD(RW, CH)                                                                                            \
  do {                                                                                                              \
    if (gres)                                                                                                       \
      rmsnorm_bwd_kernel<true, RW, CH><<<grid, NORM_THREADS, 0, st>>>(                                              \
          (const __nv_bfloat16*)g, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd,                          \
          (const __nv_bfloat16*)gres, (__nv_bfloat16*)dx, scratch, counters, (__nv_bfloat16*)dw, rows, H);          \
    else                                                                                                            \
      rmsnorm_bwd_kernel<false, RW, CH><<<grid, NORM_THREADS, 0, st>>>(                                             \
          (const __nv_bfloat16*)g, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, nullptr,                 \
          (__nv_bfloat16*)dx, scratch, counters, (__nv_bfloat16*)dw, rows, H);                                      \
  } while (0)
  SLAB_NORM_DISPATCH(SLAB_BWD);
#undef SLAB_BWD
  return (int)cudaGetLastError();
}

// dw_partial: fp32 [slab_rmsnorm_bwd_blocks(rows), H] scratch owned by the caller (contents irrelevant);
// counters: int [slab_rmsnorm_bwd_counters()], zero before the first call (every call leaves them zero).  Calls that
// share scratch or counters must not overlap on the GPU.  rows == 0 writes dw = 0.
extern "C" int slab_rmsnorm_bwd(const void* g, const void* x, const void* w, const float* rstd, const void* gres,
                                void* dx, float* dw_partial, int* counters, void* dw, int rows, int H,
                                cudaStream_t st) {
  if (H % 8 || H > NORM_MAX_H) return -100;
  return launch_rmsnorm_bwd(g, x, w, rstd, gres, dx, dw_partial, counters, dw, rows, H,
                            NORM_MAX_GRID + NORM_MAX_GROUPS, st);
}

extern "C" int slab_swiglu_fwd(const void* gu, const float* probs, void* out, long rows, int F, const int* rows_dev,
                               cudaStream_t st) {
  if (F % 8) return -100;
  if (rows == 0) return 0;
  swiglu_fwd_kernel<<<grid_for(rows * (F / 8), 256), 256, 0, st>>>((const __nv_bfloat16*)gu, probs,
                                                                    (__nv_bfloat16*)out, rows, F, rows_dev);
  return (int)cudaGetLastError();
}

extern "C" int slab_swiglu_bwd(const void* dout, const void* gu, const float* probs, void* dgu, float* dprobs,
                               long rows, int F, const int* rows_dev, cudaStream_t st) {
  if (F % 8) return -100;
  if (rows == 0) return 0;
  swiglu_bwd_kernel<<<grid_for(rows * 32, 256), 256, 0, st>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)gu,
                                                               probs, (__nv_bfloat16*)dgu, dprobs, rows, F, rows_dev);
  return (int)cudaGetLastError();
}

// n_tok = B*S tokens, each with Hh heads of D starting at x + tok*row_stride_x (strides in elements).
extern "C" int slab_rope(const void* x, const float* cs, const float* sn, void* y, long n_tok, int S, int Hh, int D,
                         long row_stride_x, long row_stride_y, float sign, cudaStream_t st) {
  if (D % 16 || row_stride_x % 8 || row_stride_y % 8) return -100;
  if (n_tok == 0) return 0;
  rope_kernel<<<grid_for(n_tok * Hh * (D / 16), 256), 256, 0, st>>>((const __nv_bfloat16*)x, cs, sn, (__nv_bfloat16*)y,
                                                                     n_tok, S, Hh, D, row_stride_x, row_stride_y, sign);
  return (int)cudaGetLastError();
}

extern "C" int slab_quant_1x128(const void* x, void* q, float* scale, long rows, int H, cudaStream_t st) {
  if (H % 128) return -100;
  if (rows == 0) return 0;
  quant_1x128_kernel<<<grid_for(rows * (H / 128) * 32, 256), 256, 0, st>>>((const __nv_bfloat16*)x,
                                                                            (__nv_fp8_e4m3*)q, scale, rows, H);
  return (int)cudaGetLastError();
}

extern "C" int slab_quant_rowwise(const void* x, void* q, float* scale, long rows, int H, cudaStream_t st) {
  if (H % 8) return -100;
  if (rows == 0) return 0;
  quant_rowwise_kernel<<<grid_for(rows * 32, 256), 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_fp8_e4m3*)q, scale,
                                                                 rows, H);
  return (int)cudaGetLastError();
}

extern "C" int slab_quant_128x128(const void* w, void* q, float* scale, int mats, int N, int K, cudaStream_t st) {
  if (N % 128 || K % 128) return -100;
  dim3 grid(K / 128, N / 128, mats);
  quant_128x128_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)w, (__nv_fp8_e4m3*)q, scale, N, K);
  return (int)cudaGetLastError();
}

// out += scale * sum(g^2); g is fp32 (g_is_bf16 == 0) or bf16.
extern "C" int slab_sumsq(const void* g, int g_is_bf16, long n, float scale, float* out, cudaStream_t st) {
  if (n == 0) return 0;
  if (g_is_bf16)
    sumsq_kernel<__nv_bfloat16><<<grid_for(n / 4 + 1, 256, 4), 256, 0, st>>>((const __nv_bfloat16*)g, n, scale, out);
  else
    sumsq_kernel<float><<<grid_for(n / 4 + 1, 256, 4), 256, 0, st>>>((const float*)g, n, scale, out);
  return (int)cudaGetLastError();
}

// p_is_bf16: weights updated in place are bf16 (no fp32 master); g_is_bf16: gradient dtype;
// state_kind: 0 fp32, 1 bf16, 2 fp8.  n must be a multiple of 128.
// A background update (ctas_per_sm > 0) is cut into launches of this many elements.  The kernel is a grid-stride
// loop whose blocks stay resident until the launch ends, and two of them hold most of an SM's registers: a kernel
// of the compute stream with large blocks (a GEMM, attention) cannot be placed beside them and waits for the launch
// to end.  With pieces of a few hundred microseconds that wait is bounded by one piece instead of the whole update.
static long g_adamw_background_piece = 1L << 25;          // elements, a multiple of 512; 0 = one launch
extern "C" int slab_set_adamw_background_piece(long elements) {
  if (elements < 0 || elements % 512) return -100;
  g_adamw_background_piece = elements;
  return 0;
}

template <typename P, typename G>
static void launch_adamw(void* p, const void* g, void* m, void* v, float* m_scale, float* v_scale, void* out_bf16,
                         const float* coef, float* sq_out, long n, int state_kind, AdamArgs a, int ctas_per_sm,
                         cudaStream_t st) {
  const bool background = ctas_per_sm > 0 && ctas_per_sm < 8;
  const long nq = n >> 4;
  const long piece = background && g_adamw_background_piece > 0 ? (g_adamw_background_piece >> 4) : nq;
  for (long q0 = 0; q0 < nq; q0 += piece) {
    const long q1 = q0 + piece < nq ? q0 + piece : nq;
    const int grid = grid_for(q1 - q0, 256, background ? ctas_per_sm : 8);
    if (state_kind == 0)
      adamw_kernel<P, 0, G><<<grid, 256, 0, st>>>((P*)p, (const G*)g, m, v, m_scale, v_scale, (__nv_bfloat16*)out_bf16, coef, sq_out, q0, q1, a);
    else if (state_kind == 1)
      adamw_kernel<P, 1, G><<<grid, 256, 0, st>>>((P*)p, (const G*)g, m, v, m_scale, v_scale, (__nv_bfloat16*)out_bf16, coef, sq_out, q0, q1, a);
    else
      adamw_kernel<P, 2, G><<<grid, 256, 0, st>>>((P*)p, (const G*)g, m, v, m_scale, v_scale, (__nv_bfloat16*)out_bf16, coef, sq_out, q0, q1, a);
  }
}

extern "C" long slab_adamw_background_piece() { return g_adamw_background_piece; }

extern "C" int slab_adamw(void* p, int p_is_bf16, const void* g, int g_is_bf16, void* m, void* v, float* m_scale,
                          float* v_scale, void* out_bf16, const float* coef, float* sq_out, long n, int state_kind,
                          float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                          long decay_end, int ctas_per_sm, cudaStream_t st) {
  // ctas_per_sm bounds the resident footprint of this grid-stride kernel.  A kernel that fills every thread slot
  // of every SM (8 x 256) keeps CTAs of kernels launched later on other streams from being scheduled until it
  // exits; an update that runs beside the backward pass asks for 2-3 and leaves the rest to the compute stream.
  if (n % 128) return -100;
  if (n == 0) return 0;
  if (decay_end % 128) return -101;
  AdamArgs a{lr, beta1, beta2, eps, wd, bc1, bc2, decay_end};
  if (p_is_bf16) {
    if (g_is_bf16) launch_adamw<__nv_bfloat16, __nv_bfloat16>(p, g, m, v, m_scale, v_scale, out_bf16, coef, sq_out, n, state_kind, a, ctas_per_sm, st);
    else launch_adamw<__nv_bfloat16, float>(p, g, m, v, m_scale, v_scale, out_bf16, coef, sq_out, n, state_kind, a, ctas_per_sm, st);
  } else {
    if (g_is_bf16) launch_adamw<float, __nv_bfloat16>(p, g, m, v, m_scale, v_scale, out_bf16, coef, sq_out, n, state_kind, a, ctas_per_sm, st);
    else launch_adamw<float, float>(p, g, m, v, m_scale, v_scale, out_bf16, coef, sq_out, n, state_kind, a, ctas_per_sm, st);
  }
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ allocation-free RMSNorm backward
// Scratch for the gain-gradient partials and the ticket counters of the in-kernel reduction live in the module
// image (see slab_noalloc.h).  The counters start at zero (static storage) and every launch leaves them at zero.
static_assert(SLAB_NOALLOC_MAX_BLOCKS >= 148 + (148 + NORM_GROUP - 1) / NORM_GROUP,
              "the built-in scratch must hold one partial row per SM plus the group rows");
static __device__ __align__(256) float g_noalloc_dw_partial[SLAB_NOALLOC_MAX_BLOCKS * SLAB_NOALLOC_MAX_H];
static __device__ __align__(256) int g_noalloc_counters[NORM_COUNTERS];

// In host code `g_noalloc_dw_partial` / `g_noalloc_counters` are only handles for the symbols, never device
// addresses: the addresses are looked up once per device and cached here.
constexpr int NOALLOC_MAX_DEVICES = 64;
static float* g_noalloc_scratch_addr[NOALLOC_MAX_DEVICES] = {nullptr};
static int* g_noalloc_counter_addr[NOALLOC_MAX_DEVICES] = {nullptr};

extern "C" int slab_rmsnorm_bwd_noalloc(const void* g, const void* x, const void* w, const float* rstd,
                                        const void* gres, void* dx, void* dw, int rows, int H, cudaStream_t st) {
  if (H % 8) return SLAB_NOALLOC_ERR_SHAPE;
  if (H > SLAB_NOALLOC_MAX_H) {
    fprintf(stderr,
            "slab_rmsnorm_bwd_noalloc: hidden size %d exceeds the built-in scratch (max %d); call "
            "slab_rmsnorm_bwd with caller-provided scratch instead\n",
            H, SLAB_NOALLOC_MAX_H);
    return SLAB_NOALLOC_ERR_TOO_LARGE;
  }
  int dev = 0;
  SLAB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return SLAB_NOALLOC_ERR_DEVICE;
  if (g_noalloc_scratch_addr[dev] == nullptr || g_noalloc_counter_addr[dev] == nullptr) {
    // first call on this device (it is the current one): resolve the symbols' device addresses
    float* addr = nullptr;
    int* caddr = nullptr;
    SLAB_CUDA_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&addr), g_noalloc_dw_partial));
    SLAB_CUDA_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&caddr), g_noalloc_counters));
    g_noalloc_counter_addr[dev] = caddr;
    g_noalloc_scratch_addr[dev] = addr;
  }
  // rows <= 0: one block runs, finds no rows and writes dw = 0, exactly as slab_rmsnorm_bwd does
  return launch_rmsnorm_bwd(g, x, w, rstd, gres, dx, g_noalloc_scratch_addr[dev], g_noalloc_counter_addr[dev], dw,
                            rows < 0 ? 0 : rows, H, SLAB_NOALLOC_MAX_BLOCKS, st);
}
