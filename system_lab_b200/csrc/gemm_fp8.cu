// Block-scaled fp8 (e4m3) grouped expert GEMM, forward:  C[r, n] = sum_k A[r, k] * B[e, n, k]  with
//   A: [R, K] e4m3, scales sa [R, K/128] fp32 (1x128 blocks along K, as written by the fused dispatch or the
//      quantising SwiGLU), B: [E, N, K] e4m3, scales sb [E, N/128, K/128] fp32 (128x128 blocks), C bf16.
//
// tcgen05.mma kind::f8f6f4 (128x128x32 per instruction) accumulates one 128-wide K block into a TMEM buffer;
// because the scale changes every K block the partial sum is promoted outside the tensor core: the four
// epilogue warps read the 128x128 fp32 partial with tcgen05.ld, multiply by sa[row, kb] * sb[e, nb, kb] and
// add into register accumulators while the MMA warp already fills the next TMEM buffer (4 buffers of 128
// columns).  Operands arrive by TMA (128-byte swizzle: one 128-element fp8 row per swizzle row), 6 stages,
// no cluster multicast.  The output goes through swizzled shared staging and a TMA store.
//
// Reference analogues: the fused fp8 grouped GEMM with dequantising epilogue (`acc *= sa*sb`,
// summary/fp8_expert_gemm_optimization.md:84-116) and the blockwise recipe that was the slowest variant there
// (notes/2026-04/2026-04-21_gptoss_10_moe_fp8_grouped_gemm_diagnosis.md:74-85).
#include "common.cuh"
#include "tma_host.cuh"

namespace slab {

constexpr int F8_BM = 128, F8_BN = 128, F8_BK = 128, F8_UK = 32, F8_STAGES = 6, F8_TBUF = 4;
constexpr int F8_THREADS = 320;          // TMA warp, MMA warp, 2 x 4 epilogue warps (each group owns 64 columns)
constexpr int F8_CTRL = 3072, F8_PREFIX_OFF = 256;
constexpr int F8_A_BYTES = F8_BM * F8_BK, F8_B_BYTES = F8_BN * F8_BK, F8_STAGE = F8_A_BYTES + F8_B_BYTES;
constexpr int F8_STORE_OFF = F8_CTRL + F8_STAGES * F8_STAGE;
constexpr int F8_STORE_BYTES = F8_BM * 64 * 2;
constexpr int F8_SMEM = F8_STORE_OFF + 2 * F8_STORE_BYTES;
static_assert(F8_SMEM <= 232448, "shared memory budget");

struct Fp8Params {
  const int* seg_offsets;
  const int* seg_counts;
  const float* sa;       // [R, K/128]
  const float* sb;       // [E, N/128, K/128]
  int E, R, N, K;
  int* status;
};

__device__ __forceinline__ int f8_seg_rows(const Fp8Params& p, int e) {
  const int off = p.seg_offsets[e], cnt = p.seg_counts[e];
  if (off < 0 || off >= p.R || cnt <= 0) return 0;
  return cnt < p.R - off ? cnt : p.R - off;
}

struct F8Tile {
  int e, m_idx, n_idx, row0;
};

__device__ __forceinline__ bool f8_get_tile(int t, const int* prefix, const Fp8Params& p, F8Tile& ti) {
  if (t >= prefix[p.E]) return false;
  int lo = 0, hi = p.E;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (prefix[mid] <= t) lo = mid; else hi = mid;
  }
  const int local = t - prefix[lo];
  const int m_tiles = (f8_seg_rows(p, lo) + F8_BM - 1) / F8_BM;
  ti.e = lo;
  ti.m_idx = local % m_tiles;
  ti.n_idx = local / m_tiles;
  ti.row0 = p.seg_offsets[lo] + ti.m_idx * F8_BM;
  return true;
}

__global__ void __launch_bounds__(F8_THREADS, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_c, const Fp8Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ST_BAD_INDEX);
    return;
  }
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty_bar = full_bar + F8_STAGES;
  uint64_t* tfull_bar = empty_bar + F8_STAGES;
  uint64_t* tempty_bar = tfull_bar + F8_TBUF;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + F8_TBUF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* prefix = reinterpret_cast<int*>(smem + F8_PREFIX_OFF);
  uint8_t* ring = smem + F8_CTRL;
  uint8_t* store_buf = smem + F8_STORE_OFF;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (p.N + F8_BN - 1) / F8_BN;
  const int kblocks = p.K / F8_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < F8_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < F8_TBUF; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 8); }
    *abort_flag = 0;
    fence_mbar_init();
    int acc = 0;
    for (int e = 0; e < p.E; ++e) {
      prefix[e] = acc;
      acc += ((f8_seg_rows(p, e) + F8_BM - 1) / F8_BM) * n_tiles;
    }
    prefix[p.E] = acc;
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_c);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, F8_TBUF * F8_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {                                   // ---------------- TMA producer
      int s = 0;
      uint32_t ph = 0;
      F8Tile ti;
      bool ok = true;
      for (int t = blockIdx.x; ok && f8_get_tile(t, prefix, p, ti); t += gridDim.x) {
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* a_dst = ring + s * F8_STAGE;
          mbar_arrive_expect_tx(&full_bar[s], F8_STAGE);
          tma_load_2d(a_dst, &tmap_a, &full_bar[s], kb * F8_BK, ti.row0);
          tma_load_2d(a_dst + F8_A_BYTES, &tmap_b, &full_bar[s], kb * F8_BK, ti.e * p.N + ti.n_idx * F8_BN);
          if (++s == F8_STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {                                   // ---------------- MMA issuer: one TMEM buffer per K block
      constexpr uint32_t idesc = make_idesc(0, 0, 0, 0, F8_BM, F8_BN);     // e4m3 x e4m3, K-major both
      int s = 0;
      uint32_t ph = 0;
      uint32_t it = 0;                                 // K blocks issued so far (selects the TMEM buffer)
      F8Tile ti;
      bool ok = true;
      for (int t = blockIdx.x; ok && f8_get_tile(t, prefix, p, ti); t += gridDim.x) {
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t buf = it % F8_TBUF;
          if (!mbar_wait(&tempty_bar[buf], ((it / F8_TBUF) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(ring + s * F8_STAGE);
          const uint32_t b_addr = a_addr + F8_A_BYTES;
#pragma unroll
          for (int k4 = 0; k4 < F8_BK / F8_UK; ++k4) {
            const uint64_t adesc = make_smem_desc(a_addr + k4 * 32, 16, 1024, 2);
            const uint64_t bdesc = make_smem_desc(b_addr + k4 * 32, 16, 1024, 2);
            umma_f8(tmem_base + buf * F8_BN, adesc, bdesc, idesc, k4 != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);
          umma_commit(&tfull_bar[buf]);
          if (++s == F8_STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else {
    // ---------------- epilogue warps: promote every K block with its scales, then store the tile.
    // Two groups of four warps; group `half` owns output columns [64*half, 64*half + 64) of the tile.
    const int lg = warp & 3;
    const int half = (warp - 2) >> 2;
    const bool store_thread = ((warp == 2 || warp == 6) && lane == 0);
    const int r_in_tile = lg * 32 + lane;
    const int nb_total = p.N / 128;
    uint8_t* sbuf = store_buf + half * F8_STORE_BYTES;
    uint32_t it = 0;
    F8Tile ti;
    bool ok = true;
    for (int t = blockIdx.x; ok && f8_get_tile(t, prefix, p, ti); t += gridDim.x) {
      float acc[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) acc[i] = 0.f;
      const int row = ti.row0 + r_in_tile;
      const float* sa_row = p.sa + (size_t)(row < p.R ? row : 0) * kblocks;
      const float* sb_row = p.sb + ((size_t)ti.e * nb_total + ti.n_idx) * kblocks;
      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        const uint32_t buf = it % F8_TBUF;
        const float sc = (row < p.R ? __ldg(sa_row + kb) : 0.f) * __ldg(sb_row + kb);
        if (!mbar_wait(&tfull_bar[buf], (it / F8_TBUF) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (uint32_t(lg * 32) << 16) + buf * F8_BN + half * 64;
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(taddr, v0);
        tmem_ld_32x32(taddr + 32, v1);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[buf]);     // the MMA warp may refill this buffer during the FMAs
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          acc[i] = fmaf(__uint_as_float(v0[i]), sc, acc[i]);
          acc[32 + i] = fmaf(__uint_as_float(v1[i]), sc, acc[32 + i]);
        }
      }
      if (!ok) break;
      // this group's 64 columns: swizzled staging (one buffer per group) -> TMA store
      if (store_thread) tma_store_wait_read<0>();
      if (half == 0) asm volatile("bar.sync 1, 128;" ::: "memory"); else asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = acc[g * 8 + i];
        *reinterpret_cast<bf16x8*>(sbuf + r_in_tile * 128 + ((g ^ (r_in_tile & 7)) << 4)) = pack8(f);
      }
      fence_proxy_async();
      if (half == 0) asm volatile("bar.sync 1, 128;" ::: "memory"); else asm volatile("bar.sync 2, 128;" ::: "memory");
      if (store_thread) {
        tma_store_2d(&tmap_c, sbuf, ti.n_idx * F8_BN + half * 64, ti.row0);
        tma_store_commit();
      }
    }
    if (store_thread) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 100000) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, F8_TBUF * F8_BN);
  }
}


// ------------------------------------------------------------------------------------------------------------
// Row-scaled fp8 forward:  C[r, n] = sa[r] * sb[e, n] * sum_k A[r, k] * B[e, n, k]
//   one scale per activation row and one per output channel of every expert.  The scales do not depend on k,
//   so the whole K loop accumulates inside TMEM at the fp8 tensor rate and the scales are applied once in the
//   epilogue.  128x256 tiles (a 128x128 tile would need the full 128 B/clk of shared-memory bandwidth at the
//   fp8 rate), 4 stages of 48 KB, two 256-column TMEM accumulators, two groups of four epilogue warps that each
//   own 128 output columns and stream them through a 16 KB swizzled staging buffer to TMA stores.
constexpr int R8_BM = 128, R8_BN = 256, R8_BK = 128, R8_STAGES = 4, R8_TBUF = 2;
constexpr int R8_A_BYTES = R8_BM * R8_BK, R8_B_BYTES = R8_BN * R8_BK, R8_STAGE = R8_A_BYTES + R8_B_BYTES;
constexpr int R8_STORE_OFF = F8_CTRL + R8_STAGES * R8_STAGE;
constexpr int R8_SMEM = R8_STORE_OFF + 2 * F8_STORE_BYTES;
static_assert(R8_SMEM <= 232448, "shared memory budget");

struct R8Params {
  const int* seg_offsets;
  const int* seg_counts;
  const float* sa;       // [R]
  const float* sb;       // [E, N]
  int E, R, N, K;
  int* status;
};

__global__ void __launch_bounds__(F8_THREADS, 1)
grouped_gemm_fp8_rowwise_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                                const __grid_constant__ CUtensorMap tmap_c, const R8Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ST_BAD_INDEX);
    return;
  }
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty_bar = full_bar + R8_STAGES;
  uint64_t* tfull_bar = empty_bar + R8_STAGES;
  uint64_t* tempty_bar = tfull_bar + R8_TBUF;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + R8_TBUF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* prefix = reinterpret_cast<int*>(smem + F8_PREFIX_OFF);
  uint8_t* ring = smem + F8_CTRL;
  uint8_t* store_buf = smem + R8_STORE_OFF;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (p.N + R8_BN - 1) / R8_BN;
  const int kblocks = p.K / R8_BK;
  const Fp8Params seg{p.seg_offsets, p.seg_counts, nullptr, nullptr, p.E, p.R, p.N, p.K, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < R8_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < R8_TBUF; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 8); }
    *abort_flag = 0;
    fence_mbar_init();
    int acc = 0;
    for (int e = 0; e < p.E; ++e) {
      prefix[e] = acc;
      acc += ((f8_seg_rows(seg, e) + R8_BM - 1) / R8_BM) * n_tiles;
    }
    prefix[p.E] = acc;
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_c);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, R8_TBUF * R8_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // f8_get_tile only needs the per-expert M-tile count and the tile prefix, both independent of the tile width
  if (warp == 0) {
    if (lane == 0) {                                   // ---------------- TMA producer
      int s = 0;
      uint32_t ph = 0;
      F8Tile ti;
      bool ok = true;
      for (int t = blockIdx.x; ok && f8_get_tile(t, prefix, seg, ti); t += gridDim.x) {
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* a_dst = ring + s * R8_STAGE;
          mbar_arrive_expect_tx(&full_bar[s], R8_STAGE);
          tma_load_2d(a_dst, &tmap_a, &full_bar[s], kb * R8_BK, ti.row0);
          tma_load_2d(a_dst + R8_A_BYTES, &tmap_b, &full_bar[s], kb * R8_BK, ti.e * p.N + ti.n_idx * R8_BN);
          if (++s == R8_STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {                                   // ---------------- MMA issuer: one TMEM buffer per tile
      constexpr uint32_t idesc = make_idesc(0, 0, 0, 0, R8_BM, R8_BN);
      int s = 0;
      uint32_t ph = 0, tit = 0;
      F8Tile ti;
      bool ok = true;
      for (int t = blockIdx.x; ok && f8_get_tile(t, prefix, seg, ti); t += gridDim.x, ++tit) {
        const uint32_t buf = tit & 1;
        if (!mbar_wait(&tempty_bar[buf], ((tit >> 1) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(ring + s * R8_STAGE);
          const uint32_t b_addr = a_addr + R8_A_BYTES;
#pragma unroll
          for (int k4 = 0; k4 < R8_BK / F8_UK; ++k4) {
            const uint64_t adesc = make_smem_desc(a_addr + k4 * 32, 16, 1024, 2);
            const uint64_t bdesc = make_smem_desc(b_addr + k4 * 32, 16, 1024, 2);
            umma_f8(tmem_base + buf * R8_BN, adesc, bdesc, idesc, (kb | k4) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);
          if (++s == R8_STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&tfull_bar[buf]);
      }
    }
  } else {
    // ---------------- epilogue: group `half` owns columns [128*half, 128*half + 128) in two 64-column passes
    const int lg = warp & 3;
    const int half = (warp - 2) >> 2;
    const bool store_thread = ((warp == 2 || warp == 6) && lane == 0);
    const int r_in_tile = lg * 32 + lane;
    uint8_t* sbuf = store_buf + half * F8_STORE_BYTES;
    uint32_t tit = 0;
    F8Tile ti;
    for (int t = blockIdx.x; f8_get_tile(t, prefix, seg, ti); t += gridDim.x, ++tit) {
      const uint32_t buf = tit & 1;
      const int row = ti.row0 + r_in_tile;
      const float sa_r = row < p.R ? __ldg(p.sa + row) : 0.f;
      if (!mbar_wait(&tfull_bar[buf], (tit >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int col0 = half * 128 + c * 64;
        const int ncol = ti.n_idx * R8_BN + col0;
        const uint32_t taddr = tmem_base + (uint32_t(lg * 32) << 16) + buf * R8_BN + col0;
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(taddr, v0);
        tmem_ld_32x32(taddr + 32, v1);
        tmem_ld_wait();
        if (c == 1) {                                    // accumulator fully read: hand the buffer back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[buf]);
        }
        if (store_thread) tma_store_wait_read<0>();
        if (half == 0) asm volatile("bar.sync 1, 128;" ::: "memory"); else asm volatile("bar.sync 2, 128;" ::: "memory");
        const float* sbp = p.sb + (size_t)ti.e * p.N + ncol;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0;
          if (ncol + g * 8 + 8 <= p.N) {
            s0 = __ldg(reinterpret_cast<const float4*>(sbp + g * 8));
            s1 = __ldg(reinterpret_cast<const float4*>(sbp + g * 8 + 4));
          }
          const uint32_t* v = g < 4 ? v0 + g * 8 : v1 + (g - 4) * 8;
          float f[8];
          f[0] = __uint_as_float(v[0]) * sa_r * s0.x;
          f[1] = __uint_as_float(v[1]) * sa_r * s0.y;
          f[2] = __uint_as_float(v[2]) * sa_r * s0.z;
          f[3] = __uint_as_float(v[3]) * sa_r * s0.w;
          f[4] = __uint_as_float(v[4]) * sa_r * s1.x;
          f[5] = __uint_as_float(v[5]) * sa_r * s1.y;
          f[6] = __uint_as_float(v[6]) * sa_r * s1.z;
          f[7] = __uint_as_float(v[7]) * sa_r * s1.w;
          *reinterpret_cast<bf16x8*>(sbuf + r_in_tile * 128 + ((g ^ (r_in_tile & 7)) << 4)) = pack8(f);
        }
        fence_proxy_async();
        if (half == 0) asm volatile("bar.sync 1, 128;" ::: "memory"); else asm volatile("bar.sync 2, 128;" ::: "memory");
        if (store_thread && ncol < p.N) {
          tma_store_2d(&tmap_c, sbuf, ncol, ti.row0);
          tma_store_commit();
        }
      }
    }
    if (store_thread) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 100000) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, R8_TBUF * R8_BN);
  }
}

}  // namespace slab

// ---------------------------------------------------------------- host side (tensor maps: tma_host.cuh)
// Forward only.  Requires K % 128 == 0, N % 128 == 0, E <= 512; expert segments start on multiples of 128 rows.
extern "C" int slab_grouped_gemm_fp8(const void* A, const float* sa, const void* B, const float* sb, void* C,
                                     const int* seg_offsets, const int* seg_counts, int E, int R, int N, int K,
                                     int max_ctas, int* status, cudaStream_t stream) {
  using namespace slab;
  if (E > 512 || K % 128 || N % 128) return -100;
  Fp8Params p{seg_offsets, seg_counts, sa, sb, E, R, N, K, status};
  CUtensorMap ma, mb, mc;
  int rc;
  if ((rc = tma_make_map_2d(&ma, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, R, K, K, F8_BM, F8_BK))) return rc;
  if ((rc = tma_make_map_2d(&mb, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)E * N, K, K, F8_BN, F8_BK))) return rc;
  if ((rc = tma_make_map_2d(&mc, C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, N, N, F8_BM, 64))) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    SLAB_CUDA_CHECK(cudaFuncSetAttribute(grouped_gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM));
    attr_set = true;
  }
  int dev = 0, grid = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&grid, cudaDevAttrMultiProcessorCount, dev);
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  grouped_gemm_fp8_kernel<<<grid, F8_THREADS, F8_SMEM, stream>>>(ma, mb, mc, p);
  return (int)cudaGetLastError();
}

// Row-scaled forward: sa [R], sb [E, N].  Requires K % 128 == 0, N % 64 == 0, E <= 512.
extern "C" int slab_grouped_gemm_fp8_rowwise(const void* A, const float* sa, const void* B, const float* sb, void* C,
                                             const int* seg_offsets, const int* seg_counts, int E, int R, int N,
                                             int K, int max_ctas, int* status, cudaStream_t stream) {
  using namespace slab;
  if (E > 512 || K % 128 || N % 64) return -100;
  R8Params p{seg_offsets, seg_counts, sa, sb, E, R, N, K, status};
  CUtensorMap ma, mb, mc;
  int rc;
  if ((rc = tma_make_map_2d(&ma, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, R, K, K, R8_BM, R8_BK))) return rc;
  if ((rc = tma_make_map_2d(&mb, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)E * N, K, K, R8_BN, R8_BK))) return rc;
  if ((rc = tma_make_map_2d(&mc, C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, N, N, R8_BM, 64))) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    SLAB_CUDA_CHECK(cudaFuncSetAttribute(grouped_gemm_fp8_rowwise_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         R8_SMEM));
    attr_set = true;
  }
  int dev = 0, grid = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&grid, cudaDevAttrMultiProcessorCount, dev);
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  grouped_gemm_fp8_rowwise_kernel<<<grid, F8_THREADS, R8_SMEM, stream>>>(ma, mb, mc, p);
  return (int)cudaGetLastError();
}
