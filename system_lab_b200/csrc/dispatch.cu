// Fused expert-parallel dispatch / combine over NVLink peer memory.
//
// Every rank owns a symmetric workspace; kernels take a table of the peers' base pointers and address
// each region by the same byte offset on every rank.  Rows travel exactly once:
//
//   count   : per-block histograms of (token, k) pairs by global expert (deterministic, no atomics)
//   publish : reduce the histograms, store this rank's counts into every peer's count matrix, release a
//             per-source flag (epoch valued, system scope)
//   plan    : wait for all sources' flags, derive from the full [world, E] matrix (a) this rank's expert
//             segments (offsets aligned to `pad`, valid counts) and (b) for every global expert the row in
//             the owner's buffer where this rank's rows start -- so senders write straight into the final
//             expert-major layout and the grouped GEMM needs no second permute
//   slots   : stable rank of every pair inside its expert -> pair_loc[pair] = (owner rank, row)
//   scatter : one warp per token: read the row once, store it (bf16, or 1x128 block-scaled e4m3 + fp32
//             scales) into each of its K destination rows with 16-byte peer stores, store the gate
//             probability beside it; zero this rank's own padding rows; last block releases "data ready"
//   wait    : receiver waits for every source's "data ready" flag
//   combine : one warp per token pulls its K expert-output rows from the owners with 16-byte peer loads,
//             reduces in fp32 (optionally gate weighted) and writes bf16 -- un-permute, top-k reduction and
//             the transfer are one pass
//
// No kernel both sets and waits on flags of the same epoch, so several ranks can be emulated by
// launching each phase for all of them in turn on one GPU.  All waits are bounded (common.cuh).
//
// Reference analogues: pack/sort + multi-workgroup scatter into a [src][expert][slot] IPC buffer with
// per-(src, expert) ready flags (notes/2026-04/2026-04-10_monolithmoe_layout_c_pack_optimization.md:98-137,
// notes/2026-04/2026-04-14_data_layout_analysis.md:322-330,630-652) and the fp32 gather-combine phase
// (notes/2026-04/2026-04-14_data_layout_analysis.md:534-605).
#include "common.cuh"

namespace slab {

constexpr int PAIRS_PER_BLOCK = 1024;
constexpr int COUNT_THREADS = 256;
constexpr int MAX_EXPERTS = 512;
constexpr int MAX_WORLD = 16;

// Byte offsets of the regions inside every rank's symmetric workspace.
struct WsLayout {
  long counts_all;     // int  [world][E]      counts written by each source
  long counts_flag;    // int  [world]         epoch flags for counts_all
  long data_flag;      // int  [world]         epoch flags: source finished writing rows
  long out_flag;       // int  [world]         epoch flags: owner finished its expert outputs
  long rows;           // recv rows  [cap][H] bf16 (or e4m3)
  long row_scales;     // float [cap][H/128]   (fp8 payload only)
  long scalars;        // float [cap]          per-row scalar travelling with the row (gate prob)
  long out_rows;       // bf16 [cap][H]        expert outputs, pulled by combine
  long out_scalars;    // float [cap]          per-row scalar pulled by combine_scalars
  long origin;         // int   [cap]          (source rank << 24) | pair index of every received row; < 0: not kept
  long comb;           // bf16  [T*K][H]       pair-major rows pushed back by the owners' GEMM epilogues
  long push_flag;      // int   [world]        epoch flags: owner finished pushing its rows
  long eflag;          // int   [world][E_local] epoch flags: source s finished writing its rows of local expert j
};

struct PeerTable {
  uint8_t* base[MAX_WORLD];
};

// ---------------------------------------------------------------- count
__global__ void __launch_bounds__(COUNT_THREADS)
moe_count_kernel(const int* __restrict__ topk_idx, int n_pairs, int E, int* __restrict__ block_hist, int* status) {
  __shared__ int hist[MAX_EXPERTS];
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int base = blockIdx.x * PAIRS_PER_BLOCK;
  for (int i = threadIdx.x; i < PAIRS_PER_BLOCK; i += blockDim.x) {
    int p = base + i;
    if (p < n_pairs) {
      const int e = topk_idx[p];
      if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
      else atomicCAS(status, 0, ST_BAD_INDEX);       // an id outside [0, E): reported, never used as an index
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) block_hist[blockIdx.x * E + e] = hist[e];
}

// ---------------------------------------------------------------- publish (one block)
// block_hist -> block_base (exclusive prefix over blocks), send_counts; store counts to every peer.
__global__ void moe_publish_kernel(int* __restrict__ block_hist, int n_blocks, int E, int* __restrict__ send_counts,
                                   PeerTable peers, WsLayout ws, int world, int me, int epoch) {
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int acc = 0;
    for (int b = 0; b < n_blocks; ++b) {
      int c = block_hist[b * E + e];
      block_hist[b * E + e] = acc;          // becomes block_base
      acc += c;
    }
    send_counts[e] = acc;
    for (int d = 0; d < world; ++d) {
      int* dst = reinterpret_cast<int*>(peers.base[d] + ws.counts_all) + me * E + e;
      *dst = acc;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) {
    int* flag = reinterpret_cast<int*>(peers.base[threadIdx.x] + ws.counts_flag) + me;
    st_release_sys(flag, epoch);
  }
}

// ---------------------------------------------------------------- plan (one block)
// Outputs (local memory): expert_offsets[E_local], expert_counts[E_local], send_base[E], meta[0] = rows used.
//
// For the expert-ordered scatter it also derives, from this rank's own counts:
//   send_prefix[e]  = pairs this rank routes to experts < e (position of expert e's run in `perm`)
//   item_prefix[oi] = work items (chunks of SCATTER_CHUNK rows) before position oi of the send order.  The send order
//                     walks the local expert index j outermost and the destination rank innermost, starting at the
//                     right-hand neighbour ((me + 1 + ph) % world): every rank is writing a different peer at any
//                     moment, and local expert j of every rank is complete after (j + 1) / E_local of the exchange.
constexpr int SCATTER_CHUNK = 16;          // rows per work item; at most 32 (one lane per row in places)

__device__ __forceinline__ int send_order_expert(int oi, int world, int me, int e_local) {
  const int j = oi / world, ph = oi % world;
  return ((me + 1 + ph) % world) * e_local + j;
}

// exclusive prefix sum over blockDim.x values (blockDim.x <= 1024); `tmp` holds 33 ints
__device__ __forceinline__ int block_exclusive_scan(int v, int* tmp, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();
  if (lane == 31) tmp[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = lane < (int)((blockDim.x + 31) >> 5) ? tmp[lane] : 0;
    int winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += n;
    }
    tmp[lane] = winc - w;
    if (lane == 31) tmp[32] = winc;
  }
  __syncthreads();
  *total = tmp[32];
  return tmp[warp] + inc - v;
}

__global__ void moe_plan_kernel(PeerTable peers, WsLayout ws, int world, int me, int E, int pad, int capacity,
                                int epoch, int* __restrict__ expert_offsets, int* __restrict__ expert_counts,
                                int* __restrict__ send_base, int* __restrict__ meta, int* status,
                                unsigned long long limit_ns, const int* __restrict__ send_counts,
                                int* __restrict__ send_prefix, int* __restrict__ item_prefix) {
  __shared__ int total[MAX_EXPERTS];      // rows of expert e over all sources
  __shared__ int before[MAX_EXPERTS];     // rows of expert e from sources < me
  __shared__ int seg_off[MAX_EXPERTS];    // aligned offset of expert e inside its owner's buffer
  __shared__ int ok;
  __shared__ int max_rows;                // most rows (with alignment padding) any rank receives
  __shared__ int scan_tmp[33];
  const int e_local = E / world;
  if (threadIdx.x == 0) { ok = 1; max_rows = 0; }
  __syncthreads();
  if (threadIdx.x < world) {
    const int* flag = reinterpret_cast<const int*>(peers.base[me] + ws.counts_flag) + threadIdx.x;
    if (!wait_flag_ge(flag, epoch, status, limit_ns)) ok = 0;
  }
  __syncthreads();
  if (!ok) {
    // fail safe: an empty plan (no rows anywhere), so every later kernel of this layer does nothing
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      send_base[e] = -(1 << 30);
      if (e < e_local) { expert_offsets[e] = 0; expert_counts[e] = 0; }
    }
    if (send_prefix)
      for (int e = threadIdx.x; e <= E; e += blockDim.x) { send_prefix[e] = 0; item_prefix[e] = 0; }
    if (threadIdx.x == 0) { meta[0] = 0; meta[1] = 0; }
    return;
  }
  if (send_prefix) {                      // blockDim.x >= E (512 threads, E <= 512)
    int tot;
    const int e = threadIdx.x;
    const int c_nat = e < E ? send_counts[e] : 0;
    const int pre = block_exclusive_scan(c_nat, scan_tmp, &tot);
    if (e < E) send_prefix[e] = pre;
    if (e == 0) send_prefix[E] = tot;
    const int c_ord = e < E ? send_counts[send_order_expert(e, world, me, e_local)] : 0;
    const int ipre = block_exclusive_scan((c_ord + SCATTER_CHUNK - 1) / SCATTER_CHUNK, scan_tmp, &tot);
    if (e < E) item_prefix[e] = ipre;
    if (e == 0) item_prefix[E] = tot;
  }
  const int* call = reinterpret_cast<const int*>(peers.base[me] + ws.counts_all);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0, b = 0;
    for (int s = 0; s < world; ++s) {
      int c = ld_acquire_sys(call + s * E + e);
      if (s < me) b += c;
      t += c;
    }
    total[e] = t;
    before[e] = b;
  }
  __syncthreads();
  if (threadIdx.x < world) {             // one thread per owner rank: aligned prefix over its experts
    int d = threadIdx.x, acc = 0;
    for (int j = 0; j < e_local; ++j) {
      int e = d * e_local + j;
      seg_off[e] = acc;
      acc += (total[e] + pad - 1) / pad * pad;
    }
    if (acc > capacity) atomicCAS(status, 0, ST_CAPACITY);
    if (d == me) meta[0] = acc;
    atomicMax(&max_rows, acc);
  }
  __syncthreads();
  // the same number on every rank (all of them see all counts): lets the ranks take the same decision about anything
  // that depends on whether every rank's rows fit a fixed-size buffer, without talking to each other
  if (threadIdx.x == 0) meta[1] = max_rows;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    send_base[e] = seg_off[e] + before[e];
    if (e / e_local == me) {
      expert_offsets[e - me * e_local] = seg_off[e];
      expert_counts[e - me * e_local] = total[e];
    }
  }
}

// ---------------------------------------------------------------- slots
// pair_loc[p] = (owner << 24) | row   (row < 2^24).  Stable: pairs of one expert keep their pair order.
__global__ void __launch_bounds__(COUNT_THREADS)
moe_slots_kernel(const int* __restrict__ topk_idx, int n_pairs, int E, int world, const int* __restrict__ block_base,
                 const int* __restrict__ send_base, int capacity, int* __restrict__ pair_loc, int* status,
                 const int* __restrict__ send_prefix, int* __restrict__ perm) {
  __shared__ int run[MAX_EXPERTS];                 // pairs of e seen so far in this block
  __shared__ int warp_hist[COUNT_THREADS / 32][MAX_EXPERTS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e_local = E / world;
  for (int e = threadIdx.x; e < E; e += blockDim.x) run[e] = block_base[blockIdx.x * E + e];
  const int base = blockIdx.x * PAIRS_PER_BLOCK;
  for (int chunk = 0; chunk < PAIRS_PER_BLOCK; chunk += COUNT_THREADS) {
    for (int i = threadIdx.x; i < (COUNT_THREADS / 32) * E; i += blockDim.x) (&warp_hist[0][0])[(i / E) * MAX_EXPERTS + i % E] = 0;
    __syncthreads();
    const int p = base + chunk + threadIdx.x;
    const bool valid = p < n_pairs;
    int e = valid ? topk_idx[p] : -1 - lane;        // distinct dummies never match
    const bool bad = valid && (e < 0 || e >= E);    // counted by nobody (moe_count_kernel skipped it too)
    if (bad) e = -64 - lane;
    const bool valid_e = valid && !bad;
    const unsigned peers_mask = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(peers_mask & ((1u << lane) - 1));
    if (valid_e && rank_in_warp == 0) warp_hist[warp][e] = __popc(peers_mask);
    __syncthreads();
    if (bad) {
      pair_loc[p] = -1;
      atomicCAS(status, 0, ST_BAD_INDEX);
    }
    if (valid_e) {
      int off = run[e] + rank_in_warp;
      for (int w = 0; w < warp; ++w) off += warp_hist[w][e];
      if (perm) perm[send_prefix[e] + off] = p;      // pairs grouped by expert, in pair order inside an expert
      const int row = send_base[e] + off;
      if (row >= capacity || row < 0) {
        if (row >= capacity) atomicCAS(status, 0, ST_CAPACITY);
        pair_loc[p] = -1;
      } else {
        pair_loc[p] = ((e / e_local) << 24) | row;
      }
    }
    __syncthreads();
    for (int ee = threadIdx.x; ee < E; ee += blockDim.x) {
      int add = 0;
      for (int w = 0; w < COUNT_THREADS / 32; ++w) add += warp_hist[w][ee];
      run[ee] += add;
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------- scatter
// FP8 = false: rows are copied as bf16.  FP8 = true: each 128-column block is scaled to e4m3 with an fp32
// scale (amax / 448) written to row_scales.  `scale_in` (optional, per pair) multiplies the row first
// (backward of a gate-weighted combine).
template <bool FP8, int VPL>
__global__ void __launch_bounds__(256)
moe_scatter_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ pair_scalar,
                   const float* __restrict__ scale_in, const int* __restrict__ pair_loc, int T, int K, int H,
                   PeerTable peers, WsLayout ws, int world, int me, int epoch,
                   const int* __restrict__ expert_offsets, const int* __restrict__ expert_counts, int e_local, int pad,
                   int* __restrict__ done_counter) {
  const int warps_per_block = blockDim.x >> 5;
  const int gwarp = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int n_warps = gridDim.x * warps_per_block;
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (int t = gwarp; t < T; t += n_warps) {
    // the token's row is read once into registers (VPL 16-byte chunks per lane) and stored K times
    const bf16x8* src = reinterpret_cast<const bf16x8*>(x + (size_t)t * H);
    bf16x8 regs[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) regs[i] = src[c];
    }
    for (int k = 0; k < K; ++k) {
      const int loc = pair_loc[t * K + k];
      if (loc < 0) continue;
      const int d = loc >> 24, row = loc & 0xFFFFFF;
      uint8_t* pb = peers.base[d];
      const float sc = scale_in ? scale_in[t * K + k] : 1.f;
      if (!FP8) {
        bf16x8* dst = reinterpret_cast<bf16x8*>(pb + ws.rows) + (size_t)row * nvec;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
          const int c = lane + 32 * i;
          if (c < nvec) {
            bf16x8 v = regs[i];
            if (scale_in) {
              float f[8];
              unpack8(v, f);
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] *= sc;
              v = pack8(f);
            }
            dst[c] = v;
          }
        }
      } else {
        uint2* dst = reinterpret_cast<uint2*>(pb + ws.rows) + (size_t)row * nvec;
        float* sdst = reinterpret_cast<float*>(pb + ws.row_scales) + (size_t)row * (H >> 7);
        // a 128-column block is 16 consecutive vec8 chunks = 16 consecutive lanes
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
          const int c = lane + 32 * i;
          float f[8];
          float amax = 0.f;
          if (c < nvec) {
            unpack8(regs[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              f[j] *= sc;
              amax = fmaxf(amax, fabsf(f[j]));
            }
          }
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
          amax = fmaxf(amax, 1e-12f);
          if (c < nvec) {
            const float inv = 448.f / amax;
            __nv_fp8_e4m3 q[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) q[j] = __nv_fp8_e4m3(f[j] * inv);
            dst[c] = *reinterpret_cast<uint2*>(q);
            if ((lane & 15) == 0) sdst[c >> 4] = amax / 448.f;
          }
        }
      }
      if (pair_scalar && lane == 0)
        reinterpret_cast<float*>(pb + ws.scalars)[row] = pair_scalar[t * K + k];
      if (ws.origin >= 0 && lane == 0)           // lets the owner's GEMM epilogue push this row's result straight back
        reinterpret_cast<int*>(pb + ws.origin)[row] = (me << 24) | (t * K + k);
    }
  }
  // zero this rank's own alignment padding rows (and their scalars): rows [count, roundup(count, pad))
  {
    uint8_t* mine = peers.base[me];
    const int row_bytes = FP8 ? H : 2 * H;
    for (int j = 0; j < e_local; ++j) {
      const int cnt = expert_counts[j];
      const int first = expert_offsets[j] + cnt;
      const int n_pad = (cnt + pad - 1) / pad * pad - cnt;
      for (int r = gwarp; r < n_pad; r += n_warps) {
        uint4* dst = reinterpret_cast<uint4*>(mine + ws.rows + (size_t)(first + r) * row_bytes);
        for (int c = lane; c < row_bytes / 16; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
        if (FP8) {
          float* sd = reinterpret_cast<float*>(mine + ws.row_scales) + (size_t)(first + r) * (H >> 7);
          for (int c = lane; c < (H >> 7); c += 32) sd[c] = 0.f;
        }
        if (lane == 0) reinterpret_cast<float*>(mine + ws.scalars)[first + r] = 0.f;
      }
    }
  }
  // completion: every block fences its peer stores; the last block releases the per-source flag everywhere
  __threadfence_system();
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) {
    int ticket = atomicAdd(done_counter, 1);
    is_last = (ticket == (int)gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    __threadfence_system();
    if (threadIdx.x < world) {
      int* flag = reinterpret_cast<int*>(peers.base[threadIdx.x] + ws.data_flag) + me;
      st_release_sys(flag, epoch);
    }
    if (threadIdx.x == 0) *done_counter = 0;
  }
}

// ---------------------------------------------------------------- scatter, expert by expert
// Same row movement as moe_scatter_kernel, but in the send order of the plan (item_prefix): a work item is a chunk
// of SCATTER_CHUNK consecutive rows of one destination expert, a thread block takes items in ascending order and
// its warps copy one row each.  The block that completes the last chunk of expert e releases
// eflag[me][local index of e] on e's owner, so the owner's expert GEMM can start on an expert as soon as every
// source has delivered that expert's rows (reference: expert_ready[src][e] of the Layout-C receive buffer,
// notes/2026-04/2026-04-14_data_layout_analysis.md:322-367), instead of after the whole exchange.
// `part`: 0 = every destination, 1 = other ranks only, 2 = this rank only (the two halves can be launched
// separately, e.g. the local half first and the remote half beside the expert GEMM).
// `chunk_done`: int [E], zero on entry, zero again on exit.
//
// BULK (bf16 payload only): a warp stages a row in shared memory, 4 KB at a time in two alternating buffers, and lane 0
// sends each piece with one bulk store (cp.async.bulk, shared -> global).  The copy engine of the SM then writes the
// peer's memory in large requests while the warp already loads the next piece; with per-lane 16-byte stores the
// same warp issues 256 store instructions per 4 KB.  A chunk is complete when every warp's bulk groups are.
constexpr int SCATTER_SEG_VEC = 256;                     // 16-byte vectors per staged piece (4 KB)
constexpr int SCATTER_SEG_BYTES = SCATTER_SEG_VEC * 16;
constexpr int SCATTER_BULK_SMEM = 8 * 2 * SCATTER_SEG_BYTES;      // 8 warps x 2 buffers

template <bool FP8, int VPL, bool BULK>
__global__ void __launch_bounds__(256)
moe_scatter_sorted_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ pair_scalar,
                          const float* __restrict__ scale_in, const int* __restrict__ pair_loc,
                          const int* __restrict__ perm, const int* __restrict__ send_counts,
                          const int* __restrict__ send_prefix, const int* __restrict__ item_prefix, int T, int K,
                          int H, int E, PeerTable peers, WsLayout ws, int world, int me, int epoch,
                          const int* __restrict__ expert_offsets, const int* __restrict__ expert_counts, int e_local,
                          int pad, int* __restrict__ chunk_done, int part) {
  __shared__ int ip[MAX_EXPERTS + 1];
  extern __shared__ __align__(128) uint8_t scatter_smem[];        // BULK: SCATTER_BULK_SMEM bytes, else none
  int seg_parity = 0;
  for (int i = threadIdx.x; i <= E; i += blockDim.x) ip[i] = item_prefix[i];
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5;
  const int gwarp = blockIdx.x * warps_per_block + warp;
  const int n_warps = gridDim.x * warps_per_block;
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  // (source, expert) pairs without rows: nothing will ever complete them, so they are released up front
  if (blockIdx.x == 0) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      const int d = e / e_local;
      const bool mine = part == 0 || (part == 1 ? d != me : d == me);
      if (mine && send_counts[e] == 0)
        st_release_sys(reinterpret_cast<int*>(peers.base[d] + ws.eflag) + me * e_local + (e - d * e_local), epoch);
    }
  }
  // zero this rank's own alignment padding rows (and their scalars): rows [count, roundup(count, pad))
  if (part != 1) {
    uint8_t* mine = peers.base[me];
    const int row_bytes = FP8 ? H : 2 * H;
    for (int j = 0; j < e_local; ++j) {
      const int cnt = expert_counts[j];
      const int first = expert_offsets[j] + cnt;
      const int n_pad = (cnt + pad - 1) / pad * pad - cnt;
      for (int r = gwarp; r < n_pad; r += n_warps) {
        uint4* dst = reinterpret_cast<uint4*>(mine + ws.rows + (size_t)(first + r) * row_bytes);
        for (int c = lane; c < row_bytes / 16; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
        if (FP8) {
          float* sd = reinterpret_cast<float*>(mine + ws.row_scales) + (size_t)(first + r) * (H >> 7);
          for (int c = lane; c < (H >> 7); c += 32) sd[c] = 0.f;
        }
        if (lane == 0) reinterpret_cast<float*>(mine + ws.scalars)[first + r] = 0.f;
      }
    }
  }
  __syncthreads();
  const int total_items = ip[E];
  for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
    int lo = 0, hi = E;                      // largest position oi with ip[oi] <= item
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (ip[mid] <= item) lo = mid; else hi = mid;
    }
    const int oi = lo;
    const int e = send_order_expert(oi, world, me, e_local);
    const int d = e / e_local;
    if ((part == 1 && d == me) || (part == 2 && d != me)) continue;
    const int cnt = send_counts[e];
    const int n_chunks = (cnt + SCATTER_CHUNK - 1) / SCATTER_CHUNK;
    const int r0 = (item - ip[oi]) * SCATTER_CHUNK;
    const int r1 = min(cnt, r0 + SCATTER_CHUNK);
    uint8_t* pb = peers.base[d];
    // lane l fetches the pair, the slot and the scale of the l-th row this warp will copy, so the chain of
    // dependent index loads (perm -> pair_loc -> row) is paid once per chunk and not once per row
    int p_l = 0, loc_l = -1;
    float sc_l = 1.f;
    {
      const int i_l = r0 + warp + warps_per_block * lane;
      if (i_l < r1) {
        p_l = perm[send_prefix[e] + i_l];
        loc_l = pair_loc[p_l];
        if (scale_in) sc_l = scale_in[p_l];
      }
    }
    int it = 0;
    for (int i = r0 + warp; i < r1; i += warps_per_block, ++it) {
      const int p = __shfl_sync(0xffffffffu, p_l, it);
      const int loc = __shfl_sync(0xffffffffu, loc_l, it);
      const float sc = __shfl_sync(0xffffffffu, sc_l, it);
      if (loc < 0 || (loc >> 24) != d) continue;         // dropped pair, or a corrupt table: never written
      const int row = loc & 0xFFFFFF;
      const int t = p / K;
      const bf16x8* src = reinterpret_cast<const bf16x8*>(x + (size_t)t * H);
      if (BULK && !FP8) {
        uint8_t* dst_row = pb + ws.rows + (size_t)row * nvec * 16;
        for (int s0 = 0; s0 < nvec; s0 += SCATTER_SEG_VEC) {
          const int nv = min(SCATTER_SEG_VEC, nvec - s0);
          bf16x8* buf = reinterpret_cast<bf16x8*>(scatter_smem + (size_t)(warp * 2 + seg_parity) * SCATTER_SEG_BYTES);
          seg_parity ^= 1;
          bf16x8 regs[SCATTER_SEG_VEC / 32];
#pragma unroll
          for (int q = 0; q < SCATTER_SEG_VEC / 32; ++q) {
            const int c = lane + 32 * q;
            if (c < nv) regs[q] = src[s0 + c];
          }
          // the piece sent two pieces ago from this buffer must have been read out of shared memory
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
#pragma unroll
          for (int q = 0; q < SCATTER_SEG_VEC / 32; ++q) {
            const int c = lane + 32 * q;
            if (c < nv) {
              bf16x8 v = regs[q];
              if (scale_in) {
                float f[8];
                unpack8(v, f);
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) f[jj] *= sc;
                v = pack8(f);
              }
              buf[c] = v;
            }
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            bulk_store(dst_row + (size_t)s0 * 16, buf, (uint32_t)nv * 16);
            tma_store_commit();
          }
        }
      } else if (!FP8) {
        bf16x8* dst = reinterpret_cast<bf16x8*>(pb + ws.rows) + (size_t)row * nvec;
        bf16x8 regs[VPL];
#pragma unroll
        for (int q = 0; q < VPL; ++q) {
          const int c = lane + 32 * q;
          if (c < nvec) regs[q] = src[c];
        }
#pragma unroll
        for (int q = 0; q < VPL; ++q) {
          const int c = lane + 32 * q;
          if (c < nvec) {
            bf16x8 v = regs[q];
            if (scale_in) {
              float f[8];
              unpack8(v, f);
#pragma unroll
              for (int jj = 0; jj < 8; ++jj) f[jj] *= sc;
              v = pack8(f);
            }
            dst[c] = v;
          }
        }
      } else {
        uint2* dst = reinterpret_cast<uint2*>(pb + ws.rows) + (size_t)row * nvec;
        float* sdst = reinterpret_cast<float*>(pb + ws.row_scales) + (size_t)row * (H >> 7);
#pragma unroll
        for (int q = 0; q < VPL; ++q) {
          const int c = lane + 32 * q;
          float f[8];
          float amax = 0.f;
          if (c < nvec) {
            unpack8(src[c], f);
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              f[jj] *= sc;
              amax = fmaxf(amax, fabsf(f[jj]));
            }
          }
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
          amax = fmaxf(amax, 1e-12f);
          if (c < nvec) {
            const float inv = 448.f / amax;
            __nv_fp8_e4m3 qv[8];
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) qv[jj] = __nv_fp8_e4m3(f[jj] * inv);
            dst[c] = *reinterpret_cast<uint2*>(qv);
            if ((lane & 15) == 0) sdst[c >> 4] = amax / 448.f;
          }
        }
      }
    }
    // the chunk's per-row scalars and origins: one lane per row, so that rows in consecutive slots (the usual case:
    // slots are handed out in pair order) leave as one 64-byte store instead of sixteen 4-byte ones
    if (warp == 0 && (pair_scalar || ws.origin >= 0)) {
      const int i = r0 + lane;
      if (i < r1) {
        const int pp = perm[send_prefix[e] + i];
        const int ll = pair_loc[pp];
        if (ll >= 0 && (ll >> 24) == d) {
          const int rr = ll & 0xFFFFFF;
          if (pair_scalar) reinterpret_cast<float*>(pb + ws.scalars)[rr] = pair_scalar[pp];
          if (ws.origin >= 0) reinterpret_cast<int*>(pb + ws.origin)[rr] = (me << 24) | pp;
        }
      }
    }
    // chunk complete: the barrier orders every thread's peer stores before thread 0, whose system-scope fence
    // (cumulative) publishes them ahead of the chunk count; the block that counts the expert's last chunk fences
    // again (acquiring the other blocks' chunks) and releases the flag
    if (BULK && !FP8 && lane == 0) {
      tma_store_wait<0>();                   // this warp's bulk stores have been written, not only read out
      __threadfence_system();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      const int done = atomicAdd(&chunk_done[e], 1);
      if (done == n_chunks - 1) {
        chunk_done[e] = 0;
        __threadfence_system();
        st_release_sys(reinterpret_cast<int*>(pb + ws.eflag) + me * e_local + (e - d * e_local), epoch);
      }
    }
  }
}

// Wait until every source has released every local expert (the consumer-side counterpart of the expert-ordered
// scatter when no kernel downstream does the waiting itself).
__global__ void moe_wait_eflags_kernel(PeerTable peers, long eflag_offset, int n_flags, int me, int epoch, int* status,
                                       unsigned long long limit_ns) {
  const int* flags = reinterpret_cast<const int*>(peers.base[me] + eflag_offset);
  for (int i = threadIdx.x; i < n_flags; i += blockDim.x) wait_flag_ge(flags + i, epoch, status, limit_ns);
}

// Rows in use beyond a caller's fixed-size copy of the receive buffer are reported, never silently cut.
__global__ void moe_check_rows_kernel(const int* __restrict__ meta, int limit, int* status, int* rows_seen) {
  if (threadIdx.x == 0) {
    if (rows_seen) atomicMax(rows_seen, meta[0]);             // high-water mark, read by the host between steps
    if (limit > 0 && meta[0] > limit) atomicCAS(status, 0, ST_CAPACITY);
  }
}

// ---------------------------------------------------------------- wait / signal (one small block)
__global__ void moe_wait_flags_kernel(PeerTable peers, long flag_offset, int world, int me, int epoch, int* status,
                                      unsigned long long limit_ns) {
  if (threadIdx.x < world) {
    const int* flag = reinterpret_cast<const int*>(peers.base[me] + flag_offset) + threadIdx.x;
    wait_flag_ge(flag, epoch, status, limit_ns);
  }
}

__global__ void moe_signal_kernel(PeerTable peers, long flag_offset, int world, int me, int epoch) {
  __threadfence_system();
  if (threadIdx.x < world) {
    int* flag = reinterpret_cast<int*>(peers.base[threadIdx.x] + flag_offset) + me;
    st_release_sys(flag, epoch);
  }
}

// ---------------------------------------------------------------- combine (pull)
// y[t] = sum_k w[t,k] * out_rows_of_owner[row(t,k)]   (w == nullptr: plain sum).  One warp per token;
// the K rows are requested before any is consumed so K peer loads are in flight per lane.
// PUSHED: the rows were already written into this rank's pair-major `comb` region by the owners' GEMM epilogues
// (row of pair (t, k) = t*K + k); the kernel waits for the owners' push flags and reduces local memory.
template <int KMAX, bool PUSHED>
__global__ void __launch_bounds__(256)
moe_combine_kernel(__nv_bfloat16* __restrict__ y, const float* __restrict__ weights, const int* __restrict__ pair_loc,
                   int T, int K, int H, PeerTable peers, WsLayout ws, int world, int me, int epoch, int* status,
                   unsigned long long limit_ns) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const int* flag = reinterpret_cast<const int*>(peers.base[me] + (PUSHED ? ws.push_flag : ws.out_flag)) + threadIdx.x;
    if (!wait_flag_ge(flag, epoch, status, limit_ns)) ok = 0;
  }
  __syncthreads();
  const int warps_per_block = blockDim.x >> 5;
  const int gwarp = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int n_warps = gridDim.x * warps_per_block;
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  if (!ok) {                                   // fail safe: defined (zero) output, error already in the status word
    for (int t = gwarp; t < T; t += n_warps)
      for (int c = lane; c < nvec; c += 32) reinterpret_cast<uint4*>(y + (size_t)t * H)[c] = make_uint4(0, 0, 0, 0);
    return;
  }
  for (int t = gwarp; t < T; t += n_warps) {
    const bf16x8* rows[KMAX];
    float w[KMAX];
#pragma unroll
    for (int k = 0; k < KMAX; ++k) {
      rows[k] = nullptr;
      w[k] = 0.f;
      if (k < K) {
        const int loc = pair_loc[t * K + k];
        if (loc >= 0) {
          rows[k] = PUSHED
              ? reinterpret_cast<const bf16x8*>(peers.base[me] + ws.comb) + (size_t)(t * K + k) * nvec
              : reinterpret_cast<const bf16x8*>(peers.base[loc >> 24] + ws.out_rows) + (size_t)(loc & 0xFFFFFF) * nvec;
          w[k] = weights ? weights[t * K + k] : 1.f;
        }
      }
    }
    for (int c = lane; c < nvec; c += 32) {
      bf16x8 v[KMAX];
#pragma unroll
      for (int k = 0; k < KMAX; ++k)
        if (rows[k]) v[k] = rows[k][c];
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int k = 0; k < KMAX; ++k) {
        if (rows[k]) {
          float f[8];
          unpack8(v[k], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += w[k] * f[j];
        }
      }
      reinterpret_cast<bf16x8*>(y + (size_t)t * H)[c] = pack8(acc);
    }
  }
}

// per-pair scalars pulled from the owners' out_scalars (backward of dispatch_scalars)
__global__ void moe_combine_scalars_kernel(float* __restrict__ s, const int* __restrict__ pair_loc, int n_pairs,
                                           PeerTable peers, WsLayout ws, int world, int me, int epoch, int* status,
                                           unsigned long long limit_ns) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const int* flag = reinterpret_cast<const int*>(peers.base[me] + ws.out_flag) + threadIdx.x;
    if (!wait_flag_ge(flag, epoch, status, limit_ns)) ok = 0;
  }
  __syncthreads();
  for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < n_pairs; p += gridDim.x * blockDim.x) {
    if (!ok) { s[p] = 0.f; continue; }
    const int loc = pair_loc[p];
    s[p] = loc >= 0 ? reinterpret_cast<const float*>(peers.base[loc >> 24] + ws.out_scalars)[loc & 0xFFFFFF] : 0.f;
  }
}

}  // namespace slab

using namespace slab;

// How long a kernel waits for a flag another GPU sets before it gives up and reports TIMEOUT_PEER_FLAG.
// Ranks legitimately drift apart by seconds (first-call library initialisation, stragglers), so the default
// is generous; tests that make a wait run out on purpose pass their own short limit.
static unsigned long long g_wait_limit_ns = 60ull * 1000000000ull;

// Whether the expert-ordered bf16 scatter sends rows with bulk stores out of shared memory (1) or with per-lane
// 16-byte stores (0).
static int g_scatter_bulk = 0;
extern "C" int slab_moe_set_scatter_bulk(int on) {
  g_scatter_bulk = on ? 1 : 0;
  return 0;
}

extern "C" int slab_moe_set_wait_limit_ms(long ms) {
  g_wait_limit_ns = (unsigned long long)(ms < 1 ? 1 : ms) * 1000000ull;
  return 0;
}

static PeerTable make_peers(const long* ptrs, int world) {
  PeerTable t;
  for (int i = 0; i < MAX_WORLD; ++i) t.base[i] = i < world ? reinterpret_cast<uint8_t*>(ptrs[i]) : nullptr;
  return t;
}

static WsLayout make_layout(const long* off) {
  WsLayout w;
  w.counts_all = off[0]; w.counts_flag = off[1]; w.data_flag = off[2]; w.out_flag = off[3];
  w.rows = off[4]; w.row_scales = off[5]; w.scalars = off[6]; w.out_rows = off[7]; w.out_scalars = off[8];
  w.origin = off[9]; w.comb = off[10]; w.push_flag = off[11]; w.eflag = off[12];
  return w;
}

extern "C" int slab_moe_count_blocks(int n_pairs) { return (n_pairs + PAIRS_PER_BLOCK - 1) / PAIRS_PER_BLOCK; }

// Phase 1 of a plan: histogram + publish this rank's counts to all peers.  `peer_ptrs` / `ws_offsets` are
// host arrays (world pointers, 12 region offsets).
extern "C" int slab_moe_count_publish(const int* topk_idx, int n_pairs, int E, int* block_hist, int* send_counts,
                                      const long* peer_ptrs, const long* ws_offsets, int world, int me, int epoch,
                                      int* status, cudaStream_t st) {
  if (E > MAX_EXPERTS || world > MAX_WORLD || E % world) return -100;
  int nb = slab_moe_count_blocks(n_pairs);
  if (nb < 1) nb = 1;
  moe_count_kernel<<<nb, COUNT_THREADS, 0, st>>>(topk_idx, n_pairs, E, block_hist, status);
  moe_publish_kernel<<<1, 512, 0, st>>>(block_hist, nb, E, send_counts, make_peers(peer_ptrs, world),
                                        make_layout(ws_offsets), world, me, epoch);
  return (int)cudaGetLastError();
}

// Phase 2: wait for all counts, derive segments and send bases, assign every pair its destination row.
// `send_counts` (this rank's pairs per expert, written by phase 1), `send_prefix` / `item_prefix` (int [E + 1]) and
// `perm` (int [n_pairs]) feed the expert-ordered scatter; pass null for the last three to skip them.
extern "C" int slab_moe_plan_slots(const int* topk_idx, int n_pairs, int E, const int* block_base,
                                   const long* peer_ptrs, const long* ws_offsets, int world, int me, int epoch,
                                   int pad, int capacity, int* expert_offsets, int* expert_counts, int* send_base,
                                   int* meta, int* pair_loc, int* status, const int* send_counts, int* send_prefix,
                                   int* item_prefix, int* perm, cudaStream_t st) {
  if (E > MAX_EXPERTS || world > MAX_WORLD || capacity >= (1 << 24)) return -100;
  if ((send_prefix == nullptr) != (item_prefix == nullptr) || (send_prefix == nullptr) != (perm == nullptr)) return -101;
  PeerTable pt = make_peers(peer_ptrs, world);
  WsLayout ws = make_layout(ws_offsets);
  moe_plan_kernel<<<1, 512, 0, st>>>(pt, ws, world, me, E, pad, capacity, epoch, expert_offsets, expert_counts,
                                     send_base, meta, status, g_wait_limit_ns, send_counts, send_prefix, item_prefix);
  int nb = slab_moe_count_blocks(n_pairs);
  if (nb < 1) nb = 1;
  moe_slots_kernel<<<nb, COUNT_THREADS, 0, st>>>(topk_idx, n_pairs, E, world, block_base, send_base, capacity,
                                                 pair_loc, status, send_prefix, perm);
  return (int)cudaGetLastError();
}

// Push rows (and one scalar per pair) to their owners; fp8 != 0 quantises 1x128.
extern "C" int slab_moe_scatter(const void* x, const float* pair_scalar, const float* scale_in, const int* pair_loc,
                                int T, int K, int H, const long* peer_ptrs, const long* ws_offsets, int world, int me,
                                int epoch, const int* expert_offsets, const int* expert_counts, int e_local, int pad,
                                int fp8, int* done_counter, int n_blocks, cudaStream_t st) {
  // bf16 rows move as 16-byte vectors (any H % 8 == 0); the fp8 payload is quantised in 128-column blocks
  if ((fp8 ? H % 128 : H % 8) || world > MAX_WORLD) return -100;
  PeerTable pt = make_peers(peer_ptrs, world);
  WsLayout ws = make_layout(ws_offsets);
  if (n_blocks <= 0) n_blocks = 148 * 4;
  const int vpl = (H / 8 + 31) / 32;
#define SLAB_SCATTER(FP8, VPL)                                                                                    \
  moe_scatter_kernel<FP8, VPL><<<n_blocks, 256, 0, st>>>((const __nv_bfloat16*)x, pair_scalar, scale_in, pair_loc, \
                                                          T, K, H, pt, ws, world, me, epoch, expert_offsets,         \
                                                          expert_counts, e_local, pad, done_counter)
  if (vpl > 32) return -100;                      // rows longer than 8192 columns are not covered
  if (fp8) {
    if (vpl <= 8) SLAB_SCATTER(true, 8);
    else if (vpl <= 16) SLAB_SCATTER(true, 16);
    else SLAB_SCATTER(true, 32);
  } else {
    if (vpl <= 8) SLAB_SCATTER(false, 8);
    else if (vpl <= 16) SLAB_SCATTER(false, 16);
    else SLAB_SCATTER(false, 32);
  }
#undef SLAB_SCATTER
  return (int)cudaGetLastError();
}

// Expert-ordered scatter with per-(source, expert) completion flags (see moe_scatter_sorted_kernel).  `perm`,
// `send_counts`, `send_prefix`, `item_prefix` come from the plan; `chunk_done` is a zeroed int [E] the kernel leaves
// zeroed.  part: 0 all destinations, 1 remote only, 2 local only.
extern "C" int slab_moe_scatter_sorted(const void* x, const float* pair_scalar, const float* scale_in,
                                       const int* pair_loc, const int* perm, const int* send_counts,
                                       const int* send_prefix, const int* item_prefix, int T, int K, int H, int E,
                                       const long* peer_ptrs, const long* ws_offsets, int world, int me, int epoch,
                                       const int* expert_offsets, const int* expert_counts, int e_local, int pad,
                                       int fp8, int* chunk_done, int part, int n_blocks, cudaStream_t st) {
  if ((fp8 ? H % 128 : H % 8) || world > MAX_WORLD || E > MAX_EXPERTS || part < 0 || part > 2) return -100;
  PeerTable pt = make_peers(peer_ptrs, world);
  WsLayout ws = make_layout(ws_offsets);
  if (n_blocks <= 0) n_blocks = 148 * 4;
  const int vpl = (H / 8 + 31) / 32;
  if (vpl > 32) return -100;
#define SLAB_SCATTER_S(FP8, VPL, BULK, SMEM)                                                                         \
  moe_scatter_sorted_kernel<FP8, VPL, BULK><<<n_blocks, 256, SMEM, st>>>(                                            \
      (const __nv_bfloat16*)x, pair_scalar, scale_in, pair_loc, perm, send_counts, send_prefix, item_prefix, T, K, H, \
      E, pt, ws, world, me, epoch, expert_offsets, expert_counts, e_local, pad, chunk_done, part)
  if (fp8) {
    if (vpl <= 8) SLAB_SCATTER_S(true, 8, false, 0);
    else if (vpl <= 16) SLAB_SCATTER_S(true, 16, false, 0);
    else SLAB_SCATTER_S(true, 32, false, 0);
  } else if (g_scatter_bulk) {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t err = cudaFuncSetAttribute(moe_scatter_sorted_kernel<false, 8, true>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SCATTER_BULK_SMEM);
      if (err != cudaSuccess) return (int)err;
      attr_set = true;
    }
    SLAB_SCATTER_S(false, 8, true, SCATTER_BULK_SMEM);
  } else {
    if (vpl <= 8) SLAB_SCATTER_S(false, 8, false, 0);
    else if (vpl <= 16) SLAB_SCATTER_S(false, 16, false, 0);
    else SLAB_SCATTER_S(false, 32, false, 0);
  }
#undef SLAB_SCATTER_S
  return (int)cudaGetLastError();
}

// Wait for all per-(source, expert) flags of this rank (world * e_local of them) to reach `epoch`.
extern "C" int slab_moe_wait_experts(const long* peer_ptrs, const long* ws_offsets, int world, int me, int e_local,
                                     int epoch, int* status, cudaStream_t st) {
  WsLayout ws = make_layout(ws_offsets);
  moe_wait_eflags_kernel<<<1, 256, 0, st>>>(make_peers(peer_ptrs, world), ws.eflag, world * e_local, me, epoch, status,
                                            g_wait_limit_ns);
  return (int)cudaGetLastError();
}

extern "C" unsigned long long slab_moe_wait_limit_ns() { return g_wait_limit_ns; }

extern "C" int slab_moe_check_rows(const int* meta, int limit, int* status, int* rows_seen, cudaStream_t st) {
  moe_check_rows_kernel<<<1, 32, 0, st>>>(meta, limit, status, rows_seen);
  return (int)cudaGetLastError();
}

// which: 0 = data_flag (rows arrived), 1 = out_flag, 2 = counts_flag
extern "C" int slab_moe_wait(const long* peer_ptrs, const long* ws_offsets, int world, int me, int epoch, int which,
                             int* status, cudaStream_t st) {
  WsLayout ws = make_layout(ws_offsets);
  long off = which == 0 ? ws.data_flag : (which == 1 ? ws.out_flag : ws.counts_flag);
  moe_wait_flags_kernel<<<1, 32, 0, st>>>(make_peers(peer_ptrs, world), off, world, me, epoch, status, g_wait_limit_ns);
  return (int)cudaGetLastError();
}

// Same wait with a caller-chosen bound (nanoseconds): lets a test make a wait run out quickly.
extern "C" int slab_moe_wait_limit(const long* peer_ptrs, const long* ws_offsets, int world, int me, int epoch,
                                   int which, int* status, long limit_ns, cudaStream_t st) {
  WsLayout ws = make_layout(ws_offsets);
  long off = which == 0 ? ws.data_flag : (which == 1 ? ws.out_flag : ws.counts_flag);
  moe_wait_flags_kernel<<<1, 32, 0, st>>>(make_peers(peer_ptrs, world), off, world, me, epoch, status,
                                          (unsigned long long)limit_ns);
  return (int)cudaGetLastError();
}

extern "C" int slab_moe_signal_out(const long* peer_ptrs, const long* ws_offsets, int world, int me, int epoch,
                                   cudaStream_t st) {
  WsLayout ws = make_layout(ws_offsets);
  moe_signal_kernel<<<1, 32, 0, st>>>(make_peers(peer_ptrs, world), ws.out_flag, world, me, epoch);
  return (int)cudaGetLastError();
}

extern "C" int slab_moe_combine(void* y, const float* weights, const int* pair_loc, int T, int K, int H,
                                const long* peer_ptrs, const long* ws_offsets, int world, int me, int epoch,
                                int* status, int n_blocks, cudaStream_t st) {
  if (H % 8 || K > 16 || world > MAX_WORLD) return -100;
  PeerTable pt = make_peers(peer_ptrs, world);
  WsLayout ws = make_layout(ws_offsets);
  if (n_blocks <= 0) n_blocks = 148 * 4;
  if (K <= 2)
    moe_combine_kernel<2, false><<<n_blocks, 256, 0, st>>>((__nv_bfloat16*)y, weights, pair_loc, T, K, H, pt, ws, world, me, epoch, status, g_wait_limit_ns);
  else if (K <= 4)
    moe_combine_kernel<4, false><<<n_blocks, 256, 0, st>>>((__nv_bfloat16*)y, weights, pair_loc, T, K, H, pt, ws, world, me, epoch, status, g_wait_limit_ns);
  else if (K <= 8)
    moe_combine_kernel<8, false><<<n_blocks, 256, 0, st>>>((__nv_bfloat16*)y, weights, pair_loc, T, K, H, pt, ws, world, me, epoch, status, g_wait_limit_ns);
  else
    moe_combine_kernel<16, false><<<n_blocks, 256, 0, st>>>((__nv_bfloat16*)y, weights, pair_loc, T, K, H, pt, ws, world, me, epoch, status, g_wait_limit_ns);
  return (int)cudaGetLastError();
}

// Reduce the K pushed rows of every token (see PUSHED above); `epoch` is the push epoch of the producing GEMM.
extern "C" int slab_moe_reduce_pairs(void* y, const int* pair_loc, int T, int K, int H, const long* peer_ptrs,
                                     const long* ws_offsets, int world, int me, int epoch, int* status, int n_blocks,
                                     cudaStream_t st) {
  if (H % 8 || K > 16 || world > MAX_WORLD) return -100;
  PeerTable pt = make_peers(peer_ptrs, world);
  WsLayout ws = make_layout(ws_offsets);
  if (n_blocks <= 0) n_blocks = 148 * 4;
  if (K <= 2)
    moe_combine_kernel<2, true><<<n_blocks, 256, 0, st>>>((__nv_bfloat16*)y, nullptr, pair_loc, T, K, H, pt, ws, world, me, epoch, status, g_wait_limit_ns);
  else if (K <= 4)
    moe_combine_kernel<4, true><<<n_blocks, 256, 0, st>>>((__nv_bfloat16*)y, nullptr, pair_loc, T, K, H, pt, ws, world, me, epoch, status, g_wait_limit_ns);
  else if (K <= 8)
    moe_combine_kernel<8, true><<<n_blocks, 256, 0, st>>>((__nv_bfloat16*)y, nullptr, pair_loc, T, K, H, pt, ws, world, me, epoch, status, g_wait_limit_ns);
  else
    moe_combine_kernel<16, true><<<n_blocks, 256, 0, st>>>((__nv_bfloat16*)y, nullptr, pair_loc, T, K, H, pt, ws, world, me, epoch, status, g_wait_limit_ns);
  return (int)cudaGetLastError();
}

extern "C" int slab_moe_combine_scalars(float* s, const int* pair_loc, int n_pairs, const long* peer_ptrs,
                                        const long* ws_offsets, int world, int me, int epoch, int* status,
                                        cudaStream_t st) {
  PeerTable pt = make_peers(peer_ptrs, world);
  WsLayout ws = make_layout(ws_offsets);
  int nb = (n_pairs + 255) / 256;
  if (nb < 1) nb = 1;
  if (nb > 148 * 4) nb = 148 * 4;
  moe_combine_scalars_kernel<<<nb, 256, 0, st>>>(s, pair_loc, n_pairs, pt, ws, world, me, epoch, status, g_wait_limit_ns);
  return (int)cudaGetLastError();
}
