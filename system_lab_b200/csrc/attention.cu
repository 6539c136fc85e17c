// Causal attention for sm_100a, forward and (further down) backward.
// Forward: S = Q K^T and O = P V on tcgen05 with TMEM accumulators, operands staged by TMA (no cluster multicast),
// online softmax in registers.  GQA, optional sliding window, head dim 64 or 128.
//
// One CTA owns 128 query rows of one (batch, head) and walks the key/value tiles its rows may see.  Roles
// (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (owns the TMEM allocation), warps 2..5 = softmax (thread
// r owns query row r: the 32x32b TMEM load hands each thread one accumulator row, so row max / row sum need no
// shuffles).  Per key tile t:
//   MMA      S[t & 1] = Q K_t^T               (issued one tile ahead, so it overlaps the softmax of tile t - 1)
//   softmax  two passes over S in TMEM (max, then exp2 -> P as bf16 into swizzled shared memory); in between it
//            drains the previous tile's P V product from TMEM into its register accumulator and rescales it
//   MMA      Otile = P V_t                    (fresh accumulator every tile; the running sum lives in registers)
// The last step adds the final product, divides by the row sum and writes the output row and its log-sum-exp.
//
// Operand layouts (all 128-byte swizzle, the forms the grouped GEMM uses): Q and K tiles are K-major ([rows][64
// columns] boxes); P is written by the softmax threads in the same K-major form the TMA would produce; V is the
// MN-major operand ([64 key rows][64 columns] boxes, as the dgrad GEMM loads its weights).
// All waits are bounded (common.cuh): a wait that runs out sets the status word and the CTA unwinds.
//
// Reference analogue: the FMHA kernels of the measured runs (aiter / CK-tile hd64 GQA with a 128-token window on
// alternate layers, notes/2026-04/2026-04-21_gptoss_13_*:19-105; cuDNN flash attention in the B200 trace,
// docs/b200-vs-mi355x-ep8-gbs16-trace.html:433).
#include "common.cuh"
#include "tma_host.cuh"

namespace slab {

constexpr int AT_BM = 128;          // query rows per CTA
constexpr int AT_BN = 128;          // key rows per tile
constexpr int AT_THREADS = 192;
constexpr int AT_TMEM_COLS = 512;   // S: 2 x 128 columns, product tile: D columns at 256

enum : int {
  ST_ATTN_Q = 20,        // waited for the query tile
  ST_ATTN_KV_FULL = 21,  // MMA waited for a key/value stage
  ST_ATTN_KV_EMPTY = 22, // producer waited for a free stage
  ST_ATTN_S = 23,        // softmax waited for Q K^T
  ST_ATTN_P = 24,        // MMA waited for the probabilities
  ST_ATTN_PV = 25,       // softmax waited for P V
};

struct AttnParams {
  __nv_bfloat16* O;     // [B, S, Hq, D] contiguous
  float* lse;           // [B, Hq, S] natural-log log-sum-exp of the scaled scores
  int B, S, Hq, Hkv;
  int window;           // 0: full causal; w > 0: key j visible to query i iff i - w < j <= i
  float scale_log2;     // softmax scale * log2(e)
  int* status;
};

template <int D>
struct AttnSmem {
  static constexpr int CTRL_BYTES = 1024;
  static constexpr int Q_BYTES = AT_BM * D * 2;
  static constexpr int K_BYTES = AT_BN * D * 2;
  static constexpr int V_BYTES = AT_BN * D * 2;
  static constexpr int STAGE_BYTES = K_BYTES + V_BYTES;
  static constexpr int P_BYTES = AT_BM * AT_BN * 2;
  static constexpr int Q_OFFSET = CTRL_BYTES;
  static constexpr int KV_OFFSET = Q_OFFSET + Q_BYTES;
  static constexpr int P_OFFSET = KV_OFFSET + 2 * STAGE_BYTES;
  static constexpr int TOTAL = P_OFFSET + P_BYTES;
};
static_assert(AttnSmem<128>::TOTAL <= 232448, "shared memory budget");

template <int D>
__global__ void __launch_bounds__(AT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  using L = AttnSmem<D>;
  constexpr int DB = D / 64;                   // 64-column boxes per row
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ST_BAD_INDEX);
    return;
  }
  uint64_t* q_full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* kv_full = q_full + 1;              // [2]
  uint64_t* kv_empty = kv_full + 2;            // [2]
  uint64_t* s_full = kv_empty + 2;             // [2]
  uint64_t* p_ready = s_full + 2;
  uint64_t* pv_done = p_ready + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* q_s = smem + L::Q_OFFSET;
  uint8_t* kv_s = smem + L::KV_OFFSET;
  uint8_t* p_s = smem + L::P_OFFSET;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_q_tiles = p.S / AT_BM;
  const int qi = n_q_tiles - 1 - (int)blockIdx.x;          // longest rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qi * AT_BM;
  const int j_hi = qi;                                     // diagonal tile
  int j_lo = 0;
  if (p.window > 0) {
    const int lo = q0 - p.window + 1;                      // first key the tile's first row may see
    j_lo = lo > 0 ? lo / AT_BN : 0;
  }
  const int n_tiles = j_hi - j_lo + 1;
  const int row_base = b * p.S;                            // row of (b, 0) in the [B*S, heads*D] views

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
      mbar_init(&s_full[s], 1);
    }
    mbar_init(p_ready, 4);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, AT_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int jb = 0; jb < DB; ++jb)
        tma_load_2d(q_s + jb * 16384, &tmap_q, q_full, h * D + jb * 64, row_base + q0);
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t & 1;
        if (!mbar_wait(&kv_empty[s], ((t >> 1) & 1) ^ 1, abort_flag, p.status, ST_ATTN_KV_EMPTY)) break;
        uint8_t* k_dst = kv_s + s * L::STAGE_BYTES;
        uint8_t* v_dst = k_dst + L::K_BYTES;
        const int kv0 = (j_lo + t) * AT_BN;
        mbar_arrive_expect_tx(&kv_full[s], L::STAGE_BYTES);
#pragma unroll
        for (int jb = 0; jb < DB; ++jb)
          tma_load_2d(k_dst + jb * 16384, &tmap_k, &kv_full[s], hk * D + jb * 64, row_base + kv0);
        // V: [key half][64-column box][64 key rows][128 bytes]
#pragma unroll
        for (int kh = 0; kh < 2; ++kh)
#pragma unroll
          for (int jn = 0; jn < DB; ++jn)
            tma_load_2d(v_dst + (kh * DB + jn) * 8192, &tmap_v, &kv_full[s], hk * D + jn * 64,
                        row_base + kv0 + kh * 64);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(1, 1, 0, 0, AT_BM, AT_BN);
      constexpr uint32_t idesc_pv = make_idesc(1, 1, 0, 1, AT_BM, D);
      const uint32_t q_addr = smem_u32(q_s);
      const uint32_t p_addr = smem_u32(p_s);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, ST_ATTN_Q);
      auto issue_qk = [&](int t) -> bool {
        const int s = t & 1;
        if (!mbar_wait(&kv_full[s], (t >> 1) & 1, abort_flag, p.status, ST_ATTN_KV_FULL)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(kv_s + s * L::STAGE_BYTES);
        const uint32_t d_tmem = tmem_base + s * AT_BN;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const int jb = kk >> 2, k4 = kk & 3;
          const uint64_t adesc = make_smem_desc(q_addr + jb * 16384 + k4 * 32, 16, 1024, 2);
          const uint64_t bdesc = make_smem_desc(k_addr + jb * 16384 + k4 * 32, 16, 1024, 2);
          umma_f16(d_tmem, adesc, bdesc, idesc_qk, kk != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[s]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int t = 0; ok && t < n_tiles; ++t) {
        if (t + 1 < n_tiles && !issue_qk(t + 1)) break;
        if (!mbar_wait(p_ready, t & 1, abort_flag, p.status, ST_ATTN_P)) break;
        tc_fence_after();
        const int s = t & 1;
        const uint32_t v_addr = smem_u32(kv_s + s * L::STAGE_BYTES + L::K_BYTES);
        const uint32_t d_tmem = tmem_base + 2 * AT_BN;
#pragma unroll
        for (int kk = 0; kk < AT_BN / 16; ++kk) {
          const int half = kk >> 2, k4 = kk & 3;
          const uint64_t adesc = make_smem_desc(p_addr + half * 16384 + k4 * 32, 16, 1024, 2);
          const uint64_t bdesc = make_smem_desc(v_addr + half * (DB * 8192) + k4 * 2048, 8192, 1024, 2);
          umma_f16(d_tmem, adesc, bdesc, idesc_pv, kk != 0 ? 1u : 0u);
        }
        umma_commit(&kv_empty[s]);             // the stage is free once these MMAs have read it
        umma_commit(pv_done);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax (warps 2..5), one query row per thread
    const int lg = warp & 3;                   // TMEM lane group this warp may read
    const int r = lg * 32 + lane;
    const int q_idx = q0 + r;
    const uint32_t lane_addr = tmem_base + (uint32_t(lg * 32) << 16);
    float m = -INFINITY, l = 0.f;
    float acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) acc[i] = 0.f;
    bool ok = true;
    for (int t = 0; t < n_tiles; ++t) {
      const int j = j_lo + t;
      const int kv0 = j * AT_BN;
      const bool masked_tile = (j == j_hi) || (p.window > 0);
      // keys [k_first, k_last] of this tile are visible to this row
      const int k_last = q_idx - kv0;                                    // >= 127 off the diagonal
      const int k_first = p.window > 0 ? q_idx - p.window + 1 - kv0 : -1;
      if (!mbar_wait(&s_full[t & 1], (t >> 1) & 1, abort_flag, p.status, ST_ATTN_S)) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = lane_addr + (t & 1) * AT_BN;
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < AT_BN; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(s_addr + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float sv = __uint_as_float(v[i]);
          const bool vis = !masked_tile || (c + i <= k_last && c + i >= k_first);
          mx = fmaxf(mx, vis ? sv : -INFINITY);
        }
      }
      const float m_new = fmaxf(m, mx * p.scale_log2);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;            // a row with nothing visible so far
      const float alpha = exp2f(m - m_use);
      // previous tile's P V: add, then bring the running sums to the new maximum
      if (t > 0) {
        if (!mbar_wait(pv_done, (t - 1) & 1, abort_flag, p.status, ST_ATTN_PV)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32(lane_addr + 2 * AT_BN + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c + i] += __uint_as_float(v[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < D; ++i) acc[i] *= alpha;
      l *= alpha;
      // second pass: probabilities as bf16 into the K-major swizzled tile the P V MMA reads
      float sum = 0.f;
#pragma unroll 1
      for (int c = 0; c < AT_BN; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(s_addr + c, v);
        tmem_ld_wait();
        uint8_t* blk = p_s + (c >> 6) * 16384 + r * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int col = c + g * 8 + i;
            const bool vis = !masked_tile || (col <= k_last && col >= k_first);
            const float pv = vis ? exp2f(__uint_as_float(v[g * 8 + i]) * p.scale_log2 - m_use) : 0.f;
            f[i] = pv;
            sum += pv;
          }
          const int g64 = ((c & 32) >> 3) + g;                           // 16-byte chunk inside the 128-byte row
          *reinterpret_cast<bf16x8*>(blk + ((g64 ^ (r & 7)) << 4)) = pack8(f);
        }
      }
      l += sum;
      m = m_new;
      fence_proxy_async();                     // the MMA reads P through the async proxy
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    if (ok && mbar_wait(pv_done, (n_tiles - 1) & 1, abort_flag, p.status, ST_ATTN_PV)) {
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < D; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(lane_addr + 2 * AT_BN + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[c + i] += __uint_as_float(v[i]);
      }
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* o_row = p.O + ((size_t)(row_base + q_idx) * p.Hq + h) * D;
#pragma unroll
      for (int g = 0; g < D / 8; ++g) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = acc[g * 8 + i] * inv;
        *reinterpret_cast<bf16x8*>(o_row + g * 8) = pack8(f);
      }
      p.lse[((size_t)b * p.Hq + h) * p.S + q_idx] = (l > 0.f) ? m * 0.6931471805599453f + logf(l) : -INFINITY;
    }
    tc_fence_before();
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 100000) __nanosleep(1000);   // let copies in flight land
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, AT_TMEM_COLS);
  }
}

// ================================================================ backward
// One CTA owns 128 key/value rows of one (batch, kv head) and walks the query tiles that can see them, for every
// query head of the group.  Per query tile (five GEMMs, FlashAttention-2 order):
//   MMA      S = Q K^T  and  dP = dO V^T                         (TMEM columns [0,128) and [128,256))
//   softmax  P = exp2(S * scale_log2 - lse2),  dS = P * (dP - delta) * scale   -> bf16 tiles in shared memory
//   MMA      dV += P^T dO,  dK += dS^T Q  (accumulate over all query tiles and heads of the group, TMEM columns
//            [256, 256+D) and [256+D, 256+2D)),  dQ = dS K  (fresh, into the columns S occupied)
//   softmax  drains dQ and adds it to the fp32 dQ buffer with global atomics (other CTAs add their key tiles)
// At the end the softmax threads (thread = key row) write dK and dV.  The pipeline is serial per query tile (one
// stage of Q / dO, one S region): a first version for correctness, not yet for speed.
// Operand forms: every tile is loaded K-major ([128 rows][64 columns] boxes).  The GEMMs that reduce over rows
// (P^T dO, dS^T Q, dS K's B operand) read the same bytes through MN-major descriptors: a 128-byte row of a box is
// 64 consecutive MN elements of one reduction index, 8 rows form a swizzle atom (stride 1024), the next 64 MN
// elements are the next box (leading-dimension stride 16384).
enum : int {
  ST_ATTNB_KV = 30, ST_ATTNB_QDO_FULL = 31, ST_ATTNB_QDO_EMPTY = 32, ST_ATTNB_SDP = 33, ST_ATTNB_PDS = 34,
  ST_ATTNB_MMA2 = 35, ST_ATTNB_DQ = 36,
};

struct AttnBwdParams {
  const float* lse;     // [B, Hq, S] natural log
  const float* delta;   // [B, Hq, S] rowsum(dO * O)
  float* dq_acc;        // [B, S, Hq, D] fp32, zero-initialised by the caller
  __nv_bfloat16* dK;    // [B, S, Hkv, D]
  __nv_bfloat16* dV;    // [B, S, Hkv, D]
  int B, S, Hq, Hkv;
  int window;
  float scale;          // softmax scale
  float scale_log2;     // scale * log2(e)
  int* status;
};

template <int D>
struct AttnBwdSmem {
  static constexpr int CTRL_BYTES = 1024;
  static constexpr int TILE_BYTES = 128 * D * 2;          // K, V, Q, dO tiles
  static constexpr int PS_BYTES = 128 * 128 * 2;          // P, dS tiles
  static constexpr int K_OFFSET = CTRL_BYTES;
  static constexpr int V_OFFSET = K_OFFSET + TILE_BYTES;
  static constexpr int Q_OFFSET = V_OFFSET + TILE_BYTES;
  static constexpr int DO_OFFSET = Q_OFFSET + TILE_BYTES;
  static constexpr int P_OFFSET = DO_OFFSET + TILE_BYTES;
  static constexpr int DS_OFFSET = P_OFFSET + PS_BYTES;
  static constexpr int TOTAL = DS_OFFSET + PS_BYTES;
};
static_assert(AttnBwdSmem<128>::TOTAL <= 232448, "shared memory budget");

template <int D>
__global__ void __launch_bounds__(AT_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                const AttnBwdParams p) {
  using L = AttnBwdSmem<D>;
  constexpr int DB = D / 64;
  constexpr int COL_DP = 128, COL_DV = 256, COL_DK = 256 + D;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ST_BAD_INDEX);
    return;
  }
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* qdo_full = kv_full + 1;
  uint64_t* qdo_empty = qdo_full + 1;
  uint64_t* sdp_full = qdo_empty + 1;
  uint64_t* pds_ready = sdp_full + 1;
  uint64_t* mma2_done = pds_ready + 1;
  uint64_t* dq_drained = mma2_done + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dq_drained + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* k_s = smem + L::K_OFFSET;
  uint8_t* v_s = smem + L::V_OFFSET;
  uint8_t* q_s = smem + L::Q_OFFSET;
  uint8_t* do_s = smem + L::DO_OFFSET;
  uint8_t* p_s = smem + L::P_OFFSET;
  uint8_t* ds_s = smem + L::DS_OFFSET;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = p.S / AT_BM;
  const int j = blockIdx.x;                                // key tile (small j = most query tiles: scheduled first)
  const int hk = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int kv0 = j * AT_BN;
  const int i_lo = j;
  int i_hi = n_tiles - 1;
  if (p.window > 0) {
    const int last_q = kv0 + AT_BN - 1 + p.window - 1;     // last query row that sees the tile's last key
    i_hi = min(i_hi, last_q / AT_BM);
  }
  const int per_head = i_hi - i_lo + 1;
  const int n_it = G * per_head;
  const int row_base = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(qdo_full, 1);
    mbar_init(qdo_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_ready, 4);
    mbar_init(mma2_done, 1);
    mbar_init(dq_drained, 4);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    prefetch_tmap(&tmap_do);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, AT_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 2 * L::TILE_BYTES);
#pragma unroll
      for (int jb = 0; jb < DB; ++jb) {
        tma_load_2d(k_s + jb * 16384, &tmap_k, kv_full, hk * D + jb * 64, row_base + kv0);
        tma_load_2d(v_s + jb * 16384, &tmap_v, kv_full, hk * D + jb * 64, row_base + kv0);
      }
      for (int it = 0; it < n_it; ++it) {
        const int h = hk * G + it / per_head;
        const int q0 = (i_lo + it % per_head) * AT_BM;
        if (!mbar_wait(qdo_empty, (it & 1) ^ 1, abort_flag, p.status, ST_ATTNB_QDO_EMPTY)) break;
        mbar_arrive_expect_tx(qdo_full, 2 * L::TILE_BYTES);
#pragma unroll
        for (int jb = 0; jb < DB; ++jb) {
          tma_load_2d(q_s + jb * 16384, &tmap_q, qdo_full, h * D + jb * 64, row_base + q0);
          tma_load_2d(do_s + jb * 16384, &tmap_do, qdo_full, h * D + jb * 64, row_base + q0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_kk = make_idesc(1, 1, 0, 0, 128, 128);     // S, dP: both operands K-major
      constexpr uint32_t idesc_mm = make_idesc(1, 1, 1, 1, 128, D);       // dV, dK: both operands MN-major views
      constexpr uint32_t idesc_km = make_idesc(1, 1, 0, 1, 128, D);       // dQ: dS K-major, K tile as MN-major view
      const uint32_t k_addr = smem_u32(k_s), v_addr = smem_u32(v_s), q_addr = smem_u32(q_s), do_addr = smem_u32(do_s);
      const uint32_t p_addr = smem_u32(p_s), ds_addr = smem_u32(ds_s);
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, ST_ATTNB_KV);
      for (int it = 0; ok && it < n_it; ++it) {
        const uint32_t ph = it & 1;
        if (!mbar_wait(qdo_full, ph, abort_flag, p.status, ST_ATTNB_QDO_FULL)) break;
        if (it > 0 && !mbar_wait(dq_drained, (it - 1) & 1, abort_flag, p.status, ST_ATTNB_DQ)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const int jb = kk >> 2, k4 = kk & 3;
          const uint32_t off = jb * 16384 + k4 * 32;
          umma_f16(tmem_base, make_smem_desc(q_addr + off, 16, 1024, 2), make_smem_desc(k_addr + off, 16, 1024, 2),
                   idesc_kk, kk != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const int jb = kk >> 2, k4 = kk & 3;
          const uint32_t off = jb * 16384 + k4 * 32;
          umma_f16(tmem_base + COL_DP, make_smem_desc(do_addr + off, 16, 1024, 2),
                   make_smem_desc(v_addr + off, 16, 1024, 2), idesc_kk, kk != 0 ? 1u : 0u);
        }
        umma_commit(sdp_full);
        if (!mbar_wait(pds_ready, ph, abort_flag, p.status, ST_ATTNB_PDS)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 128 / 16; ++kk) {          // reduce over the 128 query rows, 16 at a time
          const uint32_t acc = (it > 0 || kk > 0) ? 1u : 0u;
          umma_f16(tmem_base + COL_DV, make_smem_desc(p_addr + kk * 2048, 16384, 1024, 2),
                   make_smem_desc(do_addr + kk * 2048, 16384, 1024, 2), idesc_mm, acc);
          umma_f16(tmem_base + COL_DK, make_smem_desc(ds_addr + kk * 2048, 16384, 1024, 2),
                   make_smem_desc(q_addr + kk * 2048, 16384, 1024, 2), idesc_mm, acc);
        }
#pragma unroll
        for (int kk = 0; kk < 128 / 16; ++kk) {          // dQ = dS K: reduce over the 128 key rows
          const int half = kk >> 2, k4 = kk & 3;
          umma_f16(tmem_base, make_smem_desc(ds_addr + half * 16384 + k4 * 32, 16, 1024, 2),
                   make_smem_desc(k_addr + kk * 2048, 16384, 1024, 2), idesc_km, kk != 0 ? 1u : 0u);
        }
        umma_commit(qdo_empty);                            // Q / dO (and P / dS) may be overwritten
        umma_commit(mma2_done);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / dS / drains (warps 2..5)
    const int lg = warp & 3;
    const int r = lg * 32 + lane;                          // query row inside the tile; key row for the final drain
    const uint32_t lane_addr = tmem_base + (uint32_t(lg * 32) << 16);
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int h = hk * G + it / per_head;
      const int i = i_lo + it % per_head;
      const int q_idx = i * AT_BM + r;
      const uint32_t ph = it & 1;
      const size_t stat = ((size_t)b * p.Hq + h) * p.S + q_idx;
      const float lse2 = p.lse[stat] * 1.4426950408889634f;
      const float delta = p.delta[stat];
      const bool masked_tile = (i == j) || (p.window > 0);
      const int k_last = q_idx - kv0;
      const int k_first = p.window > 0 ? q_idx - p.window + 1 - kv0 : -1;
      if (!mbar_wait(sdp_full, ph, abort_flag, p.status, ST_ATTNB_SDP)) { ok = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < AT_BN; c += 32) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(lane_addr + c, sv);
        tmem_ld_32x32(lane_addr + COL_DP + c, dv);
        tmem_ld_wait();
        uint8_t* p_row = p_s + (c >> 6) * 16384 + r * 128;
        uint8_t* ds_row = ds_s + (c >> 6) * 16384 + r * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float pf[8], df[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int col = c + g * 8 + e;
            const bool vis = !masked_tile || (col <= k_last && col >= k_first);
            const float pv = vis ? exp2f(__uint_as_float(sv[g * 8 + e]) * p.scale_log2 - lse2) : 0.f;
            pf[e] = pv;
            df[e] = pv * (__uint_as_float(dv[g * 8 + e]) - delta) * p.scale;
          }
          const int g64 = ((c & 32) >> 3) + g;
          const int sw = (g64 ^ (r & 7)) << 4;
          *reinterpret_cast<bf16x8*>(p_row + sw) = pack8(pf);
          *reinterpret_cast<bf16x8*>(ds_row + sw) = pack8(df);
        }
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_ready);
      // dQ of this (query tile, key tile) pair: add into the fp32 buffer other key tiles add to as well
      if (!mbar_wait(mma2_done, ph, abort_flag, p.status, ST_ATTNB_MMA2)) { ok = false; break; }
      tc_fence_after();
      float* dq_row = p.dq_acc + ((size_t)(row_base + q_idx) * p.Hq + h) * D;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(lane_addr + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) atomicAdd(dq_row + c + e, __uint_as_float(v[e]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_drained);
    }
    if (ok && n_it > 0) {
      // every MMA has completed (the last mma2_done was waited for): thread r owns key row kv0 + r of dK and dV
      tc_fence_after();
      const size_t out_row = ((size_t)(row_base + kv0 + r) * p.Hkv + hk) * D;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t vv[32], kk[32];
        tmem_ld_32x32(lane_addr + COL_DV + c, vv);
        tmem_ld_32x32(lane_addr + COL_DK + c, kk);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float fv[8], fk[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            fv[e] = __uint_as_float(vv[g * 8 + e]);
            fk[e] = __uint_as_float(kk[g * 8 + e]);
          }
          *reinterpret_cast<bf16x8*>(p.dV + out_row + c + g * 8) = pack8(fv);
          *reinterpret_cast<bf16x8*>(p.dK + out_row + c + g * 8) = pack8(fk);
        }
      }
    }
    tc_fence_before();
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 100000) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, AT_TMEM_COLS);
  }
}

// ---------------------------------------------------------------- host side (tensor maps: tma_host.cuh)
// bf16 view [rows, cols] whose rows are `row_stride` elements apart (a column slice of a packed qkv tensor).
static int attn_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                    uint32_t box_rows) {
  return tma_make_map_2d(m, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, cols, row_stride, box_rows, 64);
}

template <int D>
static int launch_attn_fwd(const void* q, const void* k, const void* v, const AttnParams& p, long q_stride,
                           long k_stride, long v_stride, cudaStream_t stream) {
  CUtensorMap mq, mk, mv;
  int rc;
  const uint64_t rows = (uint64_t)p.B * p.S;
  if ((rc = attn_map(&mq, q, rows, (uint64_t)p.Hq * D, q_stride, AT_BM))) return rc;
  if ((rc = attn_map(&mk, k, rows, (uint64_t)p.Hkv * D, k_stride, AT_BN))) return rc;
  if ((rc = attn_map(&mv, v, rows, (uint64_t)p.Hkv * D, v_stride, 64))) return rc;
  // more than half of an SM's shared memory, so two CTAs (each wanting all 512 TMEM columns) never share an SM
  const int smem = AttnSmem<D>::TOTAL > 120 * 1024 ? AttnSmem<D>::TOTAL : 120 * 1024;
  SLAB_CUDA_CHECK(cudaFuncSetAttribute(attn_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid(p.S / AT_BM, p.Hq, p.B);
  attn_fwd_kernel<D><<<grid, AT_THREADS, smem, stream>>>(mq, mk, mv, p);
  return static_cast<int>(cudaGetLastError());
}


template <int D>
static int launch_attn_bwd(const void* q, const void* k, const void* v, const void* dout, const AttnBwdParams& p,
                           long q_stride, long k_stride, long v_stride, cudaStream_t stream) {
  CUtensorMap mq, mk, mv, mdo;
  int rc;
  const uint64_t rows = (uint64_t)p.B * p.S;
  if ((rc = attn_map(&mq, q, rows, (uint64_t)p.Hq * D, q_stride, 128))) return rc;
  if ((rc = attn_map(&mk, k, rows, (uint64_t)p.Hkv * D, k_stride, 128))) return rc;
  if ((rc = attn_map(&mv, v, rows, (uint64_t)p.Hkv * D, v_stride, 128))) return rc;
  if ((rc = attn_map(&mdo, dout, rows, (uint64_t)p.Hq * D, (uint64_t)p.Hq * D, 128))) return rc;
  const int smem = AttnBwdSmem<D>::TOTAL > 120 * 1024 ? AttnBwdSmem<D>::TOTAL : 120 * 1024;
  SLAB_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid(p.S / AT_BN, p.Hkv, p.B);
  attn_bwd_kernel<D><<<grid, AT_THREADS, smem, stream>>>(mq, mk, mv, mdo, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace slab

// q, k, v: bf16 [B, S, heads, D] views with contiguous heads*D and the given row strides (elements between
// consecutive tokens); o: [B, S, Hq, D] contiguous; lse: [B, Hq, S] fp32.
// Limits: D in {64, 128}; S a multiple of 128; Hq a multiple of Hkv; bases 16-byte aligned, strides multiples of 8.
extern "C" int slab_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int Hq,
                             int Hkv, int D, long q_stride, long k_stride, long v_stride, int window, float scale,
                             int* status, cudaStream_t stream) {
  using namespace slab;
  if (B <= 0 || S <= 0 || S % AT_BM || Hq <= 0 || Hkv <= 0 || Hq % Hkv || (D != 64 && D != 128)) return -10;
  if ((q_stride | k_stride | v_stride) & 7) return -11;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o) & 15) return -12;
  AttnParams p;
  p.O = reinterpret_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  return D == 64 ? launch_attn_fwd<64>(q, k, v, p, q_stride, k_stride, v_stride, stream)
                 : launch_attn_fwd<128>(q, k, v, p, q_stride, k_stride, v_stride, stream);
}

// Backward of the same attention.  q, k, v as in the forward; dout: [B, S, Hq, D] contiguous bf16; lse: the forward's
// [B, Hq, S]; delta: [B, Hq, S] fp32 = rowsum(dout * out); dq_acc: [B, S, Hq, D] fp32, zeroed by the caller (key
// tiles add into it); dk, dv: [B, S, Hkv, D] contiguous bf16.  Same limits as the forward.
extern "C" int slab_attn_bwd(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                             const float* delta, float* dq_acc, void* dk, void* dv, int B, int S, int Hq, int Hkv,
                             int D, long q_stride, long k_stride, long v_stride, int window, float scale, int* status,
                             cudaStream_t stream) {
  using namespace slab;
  if (B <= 0 || S <= 0 || S % AT_BM || Hq <= 0 || Hkv <= 0 || Hq % Hkv || (D != 64 && D != 128)) return -10;
  if ((q_stride | k_stride | v_stride) & 7) return -11;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)dout | (uintptr_t)dk | (uintptr_t)dv |
       (uintptr_t)dq_acc) & 15) return -12;
  AttnBwdParams p;
  p.lse = lse;
  p.delta = delta;
  p.dq_acc = dq_acc;
  p.dK = reinterpret_cast<__nv_bfloat16*>(dk);
  p.dV = reinterpret_cast<__nv_bfloat16*>(dv);
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.window = window;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  return D == 64 ? launch_attn_bwd<64>(q, k, v, dout, p, q_stride, k_stride, v_stride, stream)
                 : launch_attn_bwd<128>(q, k, v, dout, p, q_stride, k_stride, v_stride, stream);
}
