// Dropless grouped expert GEMM for sm_100a: tcgen05.mma with TMEM accumulators, operands staged by
// TMA (no cluster multicast), persistent warp-specialised CTAs.
//
// Roles per CTA (192 threads): warp 0 = TMA producer (one lane), warp 1 = MMA issuer (one lane, also
// owns the TMEM allocation), warps 2..5 = epilogue (each drains its 32 TMEM lanes to global memory).
// Two TMEM accumulators (2 x BN fp32 columns) let the epilogue of tile i overlap the main loop of
// tile i+1.  All waits are bounded (see common.cuh).
//
// Three modes share one kernel; rows are grouped by expert, every segment starts at a multiple of 128
// rows and padding rows are zero (the dispatch kernels guarantee both):
//   FWD    C[r, n]   = sum_k A[r, k]  * B[e, n, k]      A: acts  [R, K]   B: weights [E, N, K]
//   DGRAD  C[r, k]   = sum_n A[r, n]  * B[e, n, k]      A: dY    [R, N]   B: weights [E, N, K] (MN-major operand)
//   WGRAD  C[e, n, k]= sum_r A[r, n]  * B[r, k]         A: dY    [R, N]   B: acts    [R, K]   (both MN-major,
//                                                       reduction length = rows of expert e)
// Reference analogue: the hand written MFMA grouped GEMM (128x128x32 tiles, double buffered LDS,
// notes/2026-04/2026-04-10-mfma-gemm-optimization.md:35-109) and the variable-K wgrad kernel of
// notes/2026-04/2026-04-21_gptoss_10_moe_fp8_grouped_gemm_diagnosis.md:64-85.
#include "common.cuh"
#include "tma_host.cuh"

namespace slab {

constexpr int BM = 128;
constexpr int BK = 64;            // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;

enum { MODE_FWD = 0, MODE_DGRAD = 1, MODE_WGRAD = 2 };

struct GemmParams {
  const int* seg_offsets;   // [E] first row of each expert segment (multiple of 128)
  const int* seg_counts;    // [E] valid rows
  int E;
  int R;                    // rows of the row-grouped operands
  int N;                    // weights' N
  int K;                    // weights' K
  __nv_bfloat16* C;
  int accumulate;           // WGRAD: add into C instead of overwriting
  int* status;
  // push epilogue (FWD / DGRAD): every output row goes straight to the rank its token came from
  const int* origin;        // [R] (source rank << 24) | pair index, written by the senders' scatter
  uint8_t* peer[16];        // base of every rank's symmetric workspace
  long comb_off;            // byte offset of the pair-major [pairs][out_cols] bf16 region in a workspace
  long flag_off;            // byte offset of the int[world] push flags in a workspace
  int world, me, epoch;
  int pairs;                // rows of the pair-major region (a row origin outside it is reported, not written)
  int* counter;             // CTAs that finished pushing (reset by the last one)
  // per-(source, expert) arrival flags of the row operand A (FWD / DGRAD): the rows of expert e were written by
  // `ready_world` sources, source s releases ready[s * E + e] = ready_epoch when its rows of e are complete
  const int* ready;
  int ready_world, ready_epoch;
  unsigned long long ready_limit_ns;
  // fused all-gather of the weight operand's flat buffer (GATHER, forward only): a seventh warp in every CTA pulls
  // this CTA's share of every piece of [0, g_bytes) of the flat parameter buffer from the ranks' staged shards
  // (plain 16-byte peer loads) and counts the piece; the TMA producer loads a weight tile only after the pieces
  // that cover it are complete.  Pieces are visited starting at the multiplied weight, so the GEMM's first tiles
  // wait for a few hundred KB, and the rest of the buffer (the layer's other matrices) arrives while it runs.
  const uint8_t* g_src[16];   // every rank's staging slot (this call's slot), peer pointers
  uint8_t* g_dst;             // local flat buffer
  long g_bytes, g_shard_bytes, g_piece_bytes, g_w_off;
  int g_pieces, g_first_piece, g_target;
  int* g_piece_count;         // [g_pieces] monotonic: a complete piece holds g_target
  const int* g_ready;         // [world] staged flags of this slot (epoch valued), set by the peers' stage kernels
  int* g_ack[16];             // every rank's ack word for (slot, me): released when this rank has read the slot
  int g_world, g_epoch;
  int* g_done;                // CTAs that finished gathering (reset by the last one)
};

// Shared memory map (exactly the 227 KB a CTA may have): [0, 3072) barriers, TMEM slot, abort flag and the
// tile prefix table; then the operand ring; then two 16 KB staging buffers for the TMA store of the output.
template <int BN>
struct SmemLayout {
  static constexpr int CTRL_BYTES = 3072;
  static constexpr int PREFIX_OFFSET = 256;                   // ints: up to 512 experts + 1
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int RING_OFFSET = CTRL_BYTES;
  static constexpr int STORE_OFFSET = RING_OFFSET + STAGES * STAGE_BYTES;
  static constexpr int STORE_BYTES = BM * 64 * 2;             // 128 rows x 64 bf16 columns
  static constexpr int TOTAL = STORE_OFFSET + 2 * STORE_BYTES;
};
static_assert(SmemLayout<256>::TOTAL <= 232448 && SmemLayout<128>::TOTAL <= 232448, "shared memory budget");

// Tile walk: experts in order; inside an expert the M index runs fastest so CTAs that run at the same
// time share the expert's weight tile in L2.
struct TileInfo {
  int e, m_idx, n_idx, row0, ksteps;
};

// Rows of expert e that lie inside the operand (a corrupt plan must not turn into a runaway tile walk).
__device__ __forceinline__ int seg_rows(const GemmParams& p, int e) {
  const int off = p.seg_offsets[e], cnt = p.seg_counts[e];
  if (off < 0 || off >= p.R || cnt <= 0) return 0;
  return cnt < p.R - off ? cnt : p.R - off;
}

template <int MODE, int BN>
__device__ __forceinline__ bool get_tile(int t, const int* prefix, const GemmParams& p, int n_tiles, TileInfo& ti) {
  int E = p.E;
  if (t >= prefix[E]) return false;
  int lo = 0, hi = E;            // largest e with prefix[e] <= t
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (prefix[mid] <= t) lo = mid; else hi = mid;
  }
  int e = lo;
  int local = t - prefix[e];
  ti.e = e;
  if (MODE == MODE_WGRAD) {
    int m_tiles = (p.N + BM - 1) / BM;        // output rows = weights' N (a partial last tile when N % 128 == 64)
    ti.m_idx = local % m_tiles;
    ti.n_idx = local / m_tiles;
    ti.row0 = p.seg_offsets[e];
    ti.ksteps = (seg_rows(p, e) + BK - 1) / BK;
  } else {
    int m_tiles = (seg_rows(p, e) + BM - 1) / BM;
    ti.m_idx = local % m_tiles;
    ti.n_idx = local / m_tiles;
    ti.row0 = p.seg_offsets[e] + ti.m_idx * BM;
    ti.ksteps = ((MODE == MODE_FWD) ? p.K : p.N) / BK;
  }
  return true;
}

// PUSH (FWD / DGRAD only): the epilogue does not store the tile to C.  Each staged 128x64 chunk is written row
// by row (128 contiguous bytes per row) into the `comb` region of the rank that owns the row's token, at the
// row's pair index, over NVLink with plain peer stores: the transfer of tile i overlaps the MMAs of tile i+1.
// When the last CTA has fenced its stores it releases this rank's push flag on every peer; the token owners
// wait for all flags and reduce their K rows locally (moe_combine_kernel<., true>).
template <int MODE, int BN, bool PUSH = false, bool GATHER = false>
__global__ void __launch_bounds__(GATHER ? GEMM_THREADS + 32 : GEMM_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
  using L = SmemLayout<BN>;
  constexpr int STAGES = L::STAGES;
  constexpr bool A_MN = (MODE == MODE_WGRAD);
  constexpr bool B_MN = (MODE != MODE_FWD);
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {                 // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ST_BAD_INDEX);
    return;
  }
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* prefix = reinterpret_cast<int*>(smem + L::PREFIX_OFFSET);
  uint8_t* ring = smem + L::RING_OFFSET;
  uint8_t* store_buf = smem + L::STORE_OFFSET;
  int* origin_s = reinterpret_cast<int*>(smem + 2048);   // PUSH: 2 x 128 row origins (needs E <= 256: prefix ends < 2048)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // output tiles per expert along the non-grouped axis
  const int out_cols = (MODE == MODE_FWD) ? p.N : p.K;
  const int n_tiles = (out_cols + BN - 1) / BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
    int acc = 0;
    for (int e = 0; e < p.E; ++e) {
      prefix[e] = acc;
      int per = (MODE == MODE_WGRAD) ? ((p.N + BM - 1) / BM) : ((seg_rows(p, e) + BM - 1) / BM);
      acc += per * n_tiles;
    }
    prefix[p.E] = acc;
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_c);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // Lane 0 issues the copies.  When the row operand arrives from other GPUs expert by expert (`ready`), the whole
    // warp first polls the flags of the tile's expert, one source per lane: the GEMM starts on an expert as soon as
    // every source has delivered it, while rows of later experts are still in flight.  The rows were written by
    // peers' generic-proxy stores; the proxy fence orders the TMA (async proxy) reads after the acquire.
    int s = 0;
    uint32_t ph = 0;
    int last_e = -1;
    TileInfo ti;
    bool ok = true;
    for (int t = blockIdx.x; ok && get_tile<MODE, BN>(t, prefix, p, n_tiles, ti); t += gridDim.x) {
      if (MODE != MODE_WGRAD && p.ready != nullptr && ti.e != last_e) {
        bool mine = true;
        if (lane < p.ready_world)
          mine = wait_flag_ge(p.ready + lane * p.E + ti.e, p.ready_epoch, p.status, p.ready_limit_ns);
        ok = __all_sync(0xffffffffu, mine);
        if (!ok) {
          if (lane == 0) *abort_flag = 1;
          break;
        }
        asm volatile("fence.proxy.async.global;" ::: "memory");
        last_e = ti.e;
      }
      if (GATHER && MODE == MODE_FWD) {
        // the weight tile's bytes inside the flat buffer -> the pieces that cover them, one piece per lane
        const long t0 = p.g_w_off + ((long)ti.e * p.N + (long)ti.n_idx * BN) * p.K * 2;
        long t1 = t0 + (long)BN * p.K * 2;
        const long w_end = p.g_w_off + (long)p.E * p.N * p.K * 2;
        if (t1 > w_end) t1 = w_end;
        const int p0 = (int)(t0 / p.g_piece_bytes), p1 = (int)((t1 - 1) / p.g_piece_bytes);
        bool mine = true;
        for (int q = p0 + lane; q <= p1 && mine; q += 32) {
          if (q < p.g_pieces) mine = wait_count_ge(p.g_piece_count + q, p.g_target, p.status, p.ready_limit_ns);
        }
        ok = __all_sync(0xffffffffu, mine);
        if (!ok) {
          if (lane == 0) *abort_flag = 1;
          break;
        }
        asm volatile("fence.proxy.async.global;" ::: "memory");
      }
      if (lane == 0) {
        for (int ks = 0; ks < ti.ksteps; ++ks) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* a_dst = ring + s * L::STAGE_BYTES;
          uint8_t* b_dst = a_dst + L::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], L::STAGE_BYTES);
          if (MODE == MODE_FWD) {
            tma_load_2d(a_dst, &tmap_a, &full_bar[s], ks * BK, ti.row0);
            tma_load_2d(b_dst, &tmap_b, &full_bar[s], ks * BK, ti.e * p.N + ti.n_idx * BN);
          } else if (MODE == MODE_DGRAD) {
            tma_load_2d(a_dst, &tmap_a, &full_bar[s], ks * BK, ti.row0);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_dst + j * 8192, &tmap_b, &full_bar[s], ti.n_idx * BN + j * 64, ti.e * p.N + ks * BK);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(a_dst + j * 8192, &tmap_a, &full_bar[s], ti.m_idx * BM + j * 64, ti.row0 + ks * BK);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_dst + j * 8192, &tmap_b, &full_bar[s], ti.n_idx * BN + j * 64, ti.row0 + ks * BK);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0, BM, BN);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      TileInfo ti;
      bool ok = true;
      for (int t = blockIdx.x; ok && get_tile<MODE, BN>(t, prefix, p, n_tiles, ti); t += gridDim.x) {
        if (ti.ksteps == 0) continue;
        const int buf = it & 1;
        if (!mbar_wait(&tempty_bar[buf], ((it >> 1) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int ks = 0; ks < ti.ksteps; ++ks) {
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(ring + s * L::STAGE_BYTES);
          const uint32_t b_addr = a_addr + L::A_BYTES;
#pragma unroll
          for (int k4 = 0; k4 < BK / UMMA_K; ++k4) {
            // K-major: 32 bytes per UMMA_K inside the 128-byte swizzle row; MN-major: 16 k-rows of 128 bytes
            const uint64_t adesc = A_MN ? make_smem_desc(a_addr + k4 * 2048, 8192, 1024, 2)
                                        : make_smem_desc(a_addr + k4 * 32, 16, 1024, 2);
            const uint64_t bdesc = B_MN ? make_smem_desc(b_addr + k4 * 2048, 8192, 1024, 2)
                                        : make_smem_desc(b_addr + k4 * 32, 16, 1024, 2);
            umma_f16(d_tmem, adesc, bdesc, idesc, (ks | k4) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);          // frees the stage when these MMAs have read it
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[buf]);           // accumulator complete
        ++it;
      }
    }
  } else if (GATHER && warp == 6) {
    // ------------------------------------------------------------ gather warp (see GemmParams)
    bool good = true;
    if (lane < p.g_world) good = wait_flag_ge(p.g_ready + lane, p.g_epoch, p.status, p.ready_limit_ns);
    good = __all_sync(0xffffffffu, good);
    // One warp per CTA moves this CTA's share of a piece in units of 512 bytes (32 lanes x 16 bytes), GU units at a
    // time: all GU peer loads of a lane are issued before the first store, so a lane keeps GU x 16 bytes in flight
    // over NVLink instead of one load per round trip.
    constexpr int GU = 16;
    const long unit = 512;
    for (int i = 0; i < p.g_pieces; ++i) {
      const int piece = (p.g_first_piece + i) % p.g_pieces;
      const long lo = (long)piece * p.g_piece_bytes;
      long hi = lo + p.g_piece_bytes;
      if (hi > p.g_bytes) hi = p.g_bytes;
      if (good) {
        const long step = (long)gridDim.x * unit;
        for (long u0 = lo + (long)blockIdx.x * unit; u0 < hi; u0 += GU * step) {
          uint4 v[GU];
#pragma unroll
          for (int q = 0; q < GU; ++q) {
            const long o = u0 + q * step + lane * 16;
            if (o < hi) {
              const int r = (int)(o / p.g_shard_bytes);
              v[q] = *reinterpret_cast<const uint4*>(p.g_src[r] + (o - (long)r * p.g_shard_bytes));
            }
          }
#pragma unroll
          for (int q = 0; q < GU; ++q) {
            const long o = u0 + q * step + lane * 16;
            if (o < hi) *reinterpret_cast<uint4*>(p.g_dst + o) = v[q];
          }
        }
      }
      __threadfence();                                      // this warp's stores before the count (device scope)
      __syncwarp();
      if (lane == 0) atomicAdd(p.g_piece_count + piece, 1); // counted even after a timeout: waiters never hang on us
    }
    // the slot has been read by this CTA; the last CTA tells every peer it may reuse it
    __syncwarp();
    if (lane == 0) {
      const int ticket = atomicAdd(p.g_done, 1);
      if (ticket == (int)gridDim.x - 1) {
        *p.g_done = 0;
        __threadfence_system();
        for (int r = 0; r < p.g_world; ++r) st_release_sys(p.g_ack[r], p.g_epoch);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    // TMEM -> registers -> bf16 -> swizzled shared staging (64 columns at a time, two buffers) -> TMA store.
    // Rows/columns outside the output tensor are clipped by the TMA unit.  The accumulate variant of wgrad
    // (beta = 1) reads and writes global memory directly instead.
    const int lg = warp & 3;                    // TMEM lane group this warp may read
    const bool store_thread = (warp == 2 && lane == 0);
    const int r_in_tile = lg * 32 + lane;
    int it = 0;
    int chunk_ctr = 0;                          // staging buffer toggles per 64-column chunk
    int tile_ctr = 0;
    TileInfo ti;
    for (int t = blockIdx.x; get_tile<MODE, BN>(t, prefix, p, n_tiles, ti); t += gridDim.x) {
      const int col0 = ti.n_idx * BN;
      const int tile_row = (MODE == MODE_WGRAD) ? (ti.e * p.N + ti.m_idx * BM) : ti.row0;
      // wgrad tiles that accumulate (beta = 1), or that hang over the end of an expert's N rows (the 2-D output map
      // cannot clip at an expert boundary), go through guarded global loads / stores instead of the TMA store
      const bool partial = (MODE == MODE_WGRAD) && (ti.m_idx * BM + BM > p.N);
      const bool direct = (MODE == MODE_WGRAD) && (p.accumulate || partial);
      __nv_bfloat16* c_row = p.C + (size_t)(tile_row + r_in_tile) * out_cols;
      const bool row_ok = (MODE == MODE_WGRAD) ? (ti.m_idx * BM + r_in_tile < p.N) : (tile_row + r_in_tile < p.R);
      const bool empty = (ti.ksteps == 0);      // expert without rows (wgrad): the gradient is zero
      if (empty && direct && p.accumulate) continue;
      int* org_tile = origin_s + (tile_ctr & 1) * BM;
      if (PUSH) {
        // padding rows of the segment have no owner; the table is double buffered because a warp may start the
        // next tile while another still pushes the last chunk of this one
        const int valid = seg_rows(p, ti.e) - ti.m_idx * BM;
        org_tile[r_in_tile] = (r_in_tile < valid && row_ok) ? p.origin[tile_row + r_in_tile] : -1;
        ++tile_ctr;
      }
      int buf = 0;
      if (!empty) {
        buf = it & 1;
        if (!mbar_wait(&tfull_bar[buf], (it >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) break;
        tc_fence_after();
      }
      const uint32_t taddr = tmem_base + (uint32_t(lg * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 64) {
        uint32_t v[64];
        if (!empty) {
          uint32_t lo[32], hi[32];
          tmem_ld_32x32(taddr + c, lo);
          tmem_ld_32x32(taddr + c + 32, hi);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) { v[i] = lo[i]; v[32 + i] = hi[i]; }
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i) v[i] = 0u;
        }
        if (direct) {
          if (row_ok) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const int col = col0 + c + g * 8;
              if (col < out_cols) {
                float f[8], o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[g * 8 + i]);
                bf16x8* dst = reinterpret_cast<bf16x8*>(c_row + col);
                if (p.accumulate) {
                  unpack8(*dst, o);
#pragma unroll
                  for (int i = 0; i < 8; ++i) f[i] += o[i];
                }
                *dst = pack8(f);
              }
            }
          }
          continue;
        }
        uint8_t* sb = store_buf + (chunk_ctr & 1) * L::STORE_BYTES;
        // the TMA store that last read this buffer (two chunks ago) must have finished reading it
        if (!PUSH && store_thread) tma_store_wait_read<1>();
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[g * 8 + i]);
          // 128-byte swizzle: 16-byte chunk g of row r lives at chunk (g ^ (r & 7))
          *reinterpret_cast<bf16x8*>(sb + r_in_tile * 128 + ((g ^ (r_in_tile & 7)) << 4)) = pack8(f);
        }
        if (!PUSH) fence_proxy_async();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (PUSH) {
          // 1024 16-byte vectors per chunk, 8 per thread; 8 consecutive lanes write one row's 128 bytes
          const int et = threadIdx.x - 64;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int idx = q * 128 + et;
            const int row = idx >> 3, seg = idx & 7;
            const int org = org_tile[row];
            const int col = col0 + c + seg * 8;
            if (org >= 0 && col < out_cols) {
              const int src = org >> 24, pair = org & 0xFFFFFF;
              if (src >= p.world || pair >= p.pairs) {         // corrupt table: report, never write
                atomicCAS(p.status, 0, ST_BAD_INDEX);
                continue;
              }
              const uint4 val = *reinterpret_cast<const uint4*>(sb + row * 128 + ((seg ^ (row & 7)) << 4));
              uint8_t* dst = p.peer[src] + p.comb_off + ((size_t)pair * out_cols + col) * 2;
              *reinterpret_cast<uint4*>(dst) = val;
            }
          }
        } else if (store_thread) {
          if (col0 + c < out_cols) tma_store_2d(&tmap_c, sb, col0 + c, tile_row);   // a chunk past the last column has nothing to store
          tma_store_commit();
        }
        ++chunk_ctr;
      }
      if (!empty) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[buf]);
        ++it;
      }
    }
    if (PUSH) {
      // completion: every thread fences its peer stores, the last CTA releases this rank's flag on every peer
      __threadfence_system();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (store_thread) {
        const int ticket = atomicAdd(p.counter, 1);
        if (ticket == (int)gridDim.x - 1) {
          *p.counter = 0;
          __threadfence_system();
          for (int r = 0; r < p.world; ++r)
            st_release_sys(reinterpret_cast<int*>(p.peer[r] + p.flag_off) + p.me, p.epoch);
        }
      }
    } else if (store_thread) {
      tma_store_wait<0>();                      // all output written before the CTA retires
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // give copies that are still in flight time to land before shared memory is handed on
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 100000) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ---------------------------------------------------------------- host side (tensor maps: tma_host.cuh)
template <int MODE, int BN, bool PUSH = false, bool GATHER = false>
static int launch(const void* A, const void* B, const GemmParams& p, int grid, cudaStream_t stream) {
  using L = SmemLayout<BN>;
  CUtensorMap ma, mb;
  int rc;
  if (MODE == MODE_FWD) {
    if ((rc = tma_make_map_bf16(&ma, A, p.R, p.K, BM, BK))) return rc;
    if ((rc = tma_make_map_bf16(&mb, B, (uint64_t)p.E * p.N, p.K, BN, BK))) return rc;
  } else if (MODE == MODE_DGRAD) {
    if ((rc = tma_make_map_bf16(&ma, A, p.R, p.N, BM, BK))) return rc;
    if ((rc = tma_make_map_bf16(&mb, B, (uint64_t)p.E * p.N, p.K, BK, 64))) return rc;
  } else {
    if ((rc = tma_make_map_bf16(&ma, A, p.R, p.N, BK, 64))) return rc;
    if ((rc = tma_make_map_bf16(&mb, B, p.R, p.K, BK, 64))) return rc;
  }
  CUtensorMap mc;
  if (PUSH) {
    mc = ma;                                  // the push epilogue stores with plain peer writes: no output map
  } else if (MODE == MODE_WGRAD) {
    if ((rc = tma_make_map_bf16(&mc, p.C, (uint64_t)p.E * p.N, p.K, BM, 64))) return rc;
  } else {
    if ((rc = tma_make_map_bf16(&mc, p.C, p.R, (MODE == MODE_FWD) ? p.N : p.K, BM, 64))) return rc;
  }
  static bool attr_set = false;
  auto kern = grouped_gemm_kernel<MODE, BN, PUSH, GATHER>;
  if (!attr_set) {
    SLAB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    attr_set = true;
  }
  kern<<<grid, GATHER ? GEMM_THREADS + 32 : GEMM_THREADS, L::TOTAL, stream>>>(ma, mb, mc, p);
  return (int)cudaGetLastError();
}

}  // namespace slab

// mode: 0 fwd, 1 dgrad, 2 wgrad.  Shapes: see the header comment.  Requires K % 64 == 0, N % 64 == 0
// (wgrad: a last partial row tile is written with guarded stores), at most 512 experts.  `status` is a device int
// the kernel sets on a
// bounded-wait timeout (0 = ok).  Returns a CUDA/driver error code (0 = launched).
// `ready` (optional, modes 0 and 1): per-(source, expert) arrival flags of the row operand, int [ready_world][E] in
// this GPU's memory; the kernel waits (bounded) for all `ready_world` flags of an expert to reach `ready_epoch`
// before it loads that expert's first row tile.  Null: the operand is complete when the kernel starts.
extern "C" unsigned long long slab_moe_wait_limit_ns();

extern "C" int slab_grouped_gemm_bf16(int mode, const void* A, const void* B, void* C, const int* seg_offsets,
                                      const int* seg_counts, int E, int R, int N, int K, int accumulate,
                                      int block_n, int max_ctas, const int* ready, int ready_world, int ready_epoch,
                                      int* status, cudaStream_t stream) {
  using namespace slab;
  if (E > 512 || K % 64 || N % 64) return -100;
  if (ready && (ready_world < 1 || ready_world > 32 || mode == MODE_WGRAD)) return -102;
  GemmParams p{seg_offsets, seg_counts, E, R, N, K, static_cast<__nv_bfloat16*>(C), accumulate, status};
  p.ready = ready;
  p.ready_world = ready_world;
  p.ready_epoch = ready_epoch;
  p.ready_limit_ns = slab_moe_wait_limit_ns();
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  const bool wide = block_n != 128;
  switch (mode) {
    case MODE_FWD:
      return wide ? launch<MODE_FWD, 256>(A, B, p, grid, stream) : launch<MODE_FWD, 128>(A, B, p, grid, stream);
    case MODE_DGRAD:
      return wide ? launch<MODE_DGRAD, 256>(A, B, p, grid, stream) : launch<MODE_DGRAD, 128>(A, B, p, grid, stream);
    case MODE_WGRAD:
      return wide ? launch<MODE_WGRAD, 256>(A, B, p, grid, stream) : launch<MODE_WGRAD, 128>(A, B, p, grid, stream);
  }
  return -101;
}

// Forward (mode 0) or dgrad (mode 1) whose result rows are pushed to the ranks that own the rows' tokens instead
// of being stored locally.  `origin[r]` = (source rank << 24) | pair index for every valid row, `peer_ptrs` the
// workspace base of every rank, `comb_off` / `flag_off` byte offsets inside a workspace of the pair-major
// [pairs][out_cols] bf16 region and of the int[world] push flags.  `counter` is a zero-initialised device int.
// The caller's matching reduction waits for `epoch` on all flags.  At most 256 experts per rank.
extern "C" int slab_grouped_gemm_bf16_push(int mode, const void* A, const void* B, const int* seg_offsets,
                                           const int* seg_counts, int E, int R, int N, int K, int block_n,
                                           int max_ctas, const int* origin, const long* peer_ptrs, long comb_off,
                                           long flag_off, int world, int me, int epoch, int pairs, int* counter,
                                           int* status, cudaStream_t stream) {
  using namespace slab;
  if (E > 256 || K % 64 || N % 64 || world > 16 || world < 1 || me < 0 || me >= world) return -100;
  if (mode != MODE_FWD && mode != MODE_DGRAD) return -101;
  GemmParams p{seg_offsets, seg_counts, E, R, N, K, nullptr, 0, status};
  p.ready = nullptr;
  p.origin = origin;
  for (int i = 0; i < 16; ++i) p.peer[i] = i < world ? reinterpret_cast<uint8_t*>(peer_ptrs[i]) : nullptr;
  p.comb_off = comb_off;
  p.flag_off = flag_off;
  p.world = world;
  p.me = me;
  p.epoch = epoch;
  p.pairs = pairs;
  p.counter = counter;
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  const bool wide = block_n != 128;
  if (mode == MODE_FWD)
    return wide ? launch<MODE_FWD, 256, true>(A, B, p, grid, stream) : launch<MODE_FWD, 128, true>(A, B, p, grid, stream);
  return wide ? launch<MODE_DGRAD, 256, true>(A, B, p, grid, stream) : launch<MODE_DGRAD, 128, true>(A, B, p, grid, stream);
}

// Dense forward GEMM C[R, N] = A[R, K] * W[N, K]^T fused with the all-gather of the flat parameter buffer W lives
// in (FSDP): every rank has staged its shard of the buffer in its symmetric slot (slab_fsdp_stage); this kernel
// pulls bytes [0, gather_bytes) of the buffer from the ranks' slots into `flat` while it multiplies, loading a
// weight tile as soon as the pieces that cover it have arrived, and acknowledges the slot to every peer at the end.
//   W = flat + w_off_bytes; shard_bytes = bytes of the buffer every rank stages (multiple of 256);
//   layout = {ready_flags, ack_flags, slots, slot_bytes} byte offsets inside a workspace (fsdp_comm.cu);
//   piece_count: int [ceil(gather_bytes / piece_bytes)], zero before the first call, never reset: call number c
//   (1-based, every call with the same SM count) passes target = c * number of SMs;  done_counter: zeroed int.
//   seg_offsets / seg_counts: device ints {0} and {R} (the single segment of a dense GEMM).
extern "C" int slab_dense_gemm_gather(const void* A, void* C, const int* seg_offsets, const int* seg_counts, int R,
                                      int N, int K, int block_n, void* flat,
                                      long w_off_bytes, long gather_bytes, long shard_bytes, long piece_bytes,
                                      const long* peer_ptrs, const long* layout, int world, int me, int slot,
                                      int epoch, int* piece_count, int call_index, int* done_counter, int* status,
                                      cudaStream_t stream) {
  using namespace slab;
  if (K % 64 || N % 64 || world < 1 || world > 16 || me < 0 || me >= world) return -100;
  if (gather_bytes % 512 || shard_bytes % 256 || piece_bytes % 512 || piece_bytes <= 0 || w_off_bytes % 256) return -101;
  if (gather_bytes > shard_bytes * world || w_off_bytes + (long)N * K * 2 > gather_bytes) return -102;
  GemmParams p{};
  p.seg_offsets = seg_offsets;
  p.seg_counts = seg_counts;
  p.E = 1;
  p.R = R;
  p.N = N;
  p.K = K;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.status = status;
  p.ready_limit_ns = slab_moe_wait_limit_ns();
  const long ready_off = layout[0], ack_off = layout[1], slots_off = layout[2], slot_bytes = layout[3];
  for (int r = 0; r < 16; ++r) {
    p.g_src[r] = r < world ? reinterpret_cast<const uint8_t*>(peer_ptrs[r]) + slots_off + (long)slot * slot_bytes : nullptr;
    p.g_ack[r] = r < world ? reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(peer_ptrs[r]) + ack_off) + slot * 16 + me
                           : nullptr;
  }
  p.g_dst = static_cast<uint8_t*>(flat);
  p.g_bytes = gather_bytes;
  p.g_shard_bytes = shard_bytes;
  p.g_piece_bytes = piece_bytes;
  p.g_w_off = w_off_bytes;
  p.g_pieces = (int)((gather_bytes + piece_bytes - 1) / piece_bytes);
  p.g_first_piece = (int)(w_off_bytes / piece_bytes);
  p.g_piece_count = piece_count;
  p.g_ready = reinterpret_cast<const int*>(reinterpret_cast<const uint8_t*>(peer_ptrs[me]) + ready_off) + slot * 16;
  p.g_world = world;
  p.g_epoch = epoch;
  p.g_done = done_counter;
  const int grid = sm_count();
  p.g_target = call_index * grid;
  const void* B = static_cast<const uint8_t*>(flat) + w_off_bytes;
  return block_n != 128 ? launch<MODE_FWD, 256, false, true>(A, B, p, grid, stream)
                        : launch<MODE_FWD, 128, false, true>(A, B, p, grid, stream);
}
