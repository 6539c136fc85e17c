// Causal attention forward for sm_100a: S = Q K^T and O = P V on tcgen05 with TMEM accumulators, operands staged by
// TMA (no cluster multicast), online softmax in registers.  GQA, optional sliding window, head dim 64 or 128.
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

// ---------------------------------------------------------------- host side
typedef CUresult (*AttnEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static AttnEncodeFn attn_encode() {
  static AttnEncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<AttnEncodeFn>(ptr);
  }
  return fn;
}

// bf16 view [rows, cols] whose rows are `row_stride` elements apart (a column slice of a packed qkv tensor).
static int attn_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                    uint32_t box_rows) {
  AttnEncodeFn enc = attn_encode();
  if (!enc) return -1;
  static thread_local bool ctx_ready = false;
  if (!ctx_ready) {
    cudaFree(0);
    ctx_ready = true;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2 - (int)r;
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
