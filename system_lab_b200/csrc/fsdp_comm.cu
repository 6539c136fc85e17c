// FSDP collectives over NVLink peer memory: parameter all-gather and gradient reduce-scatter (with the
// bf16 -> fp32 cast and, optionally, the sharded AdamW update in the same pass).
//
// Each rank owns a symmetric workspace with NSLOT staging slots.  A collective is two launches:
//   stage  : wait until every peer has acknowledged the previous use of the slot (flags of an older call),
//            copy the local operand into the slot, fence, release a per-source "ready" flag on every peer;
//   gather : wait for every source's flag, then pull the peers' slices with 16-byte loads straight into the
//            destination (all-gather) or sum them in fp32 (reduce-scatter); the last block acknowledges the
//            slot to every peer.
// No kernel waits on a flag of its own call that it also sets, so ranks can be emulated phase by phase on
// one GPU.  Waits are bounded (common.cuh) and fail safe: on a timeout the output is left untouched
// (all-gather) or zero (reduce-scatter) and the status word carries the error.
//
// Reference analogues: per-bucket `reduce_scatter_tensor` / `all_gather_into_tensor` of the distributed
// optimizer (notes/2026-04/2026-04-22_gptoss_12_*:38-56), in-collective averaging (:98-108), the in-place P2P
// reduction sketched in moe/research_direction_C.md:236-257, and the multi_tensor Adam tail
// (notes/2026-04/2026-04-22_gptoss_15_*:119-131).
#include "common.cuh"

namespace slab {

constexpr int FS_MAX_WORLD = 16;

struct FsPeers {
  uint8_t* base[FS_MAX_WORLD];
};

// workspace layout (bytes): [0,256) ready flags (int[world]) per slot at slot*1024; acks at 512 + ...
struct FsLayout {
  long ready_flags;   // int [NSLOT][FS_MAX_WORLD]
  long ack_flags;     // int [NSLOT][FS_MAX_WORLD]
  long slots;         // byte offset of slot 0
  long slot_bytes;
};

__global__ void __launch_bounds__(512)
fsdp_stage_kernel(const uint4* __restrict__ src, long n16, FsPeers peers, FsLayout lay, int world, int me, int slot,
                  int epoch, int ack_epoch, int* status, unsigned long long limit_ns, int* done_counter) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (ack_epoch > 0 && threadIdx.x < world) {
    const int* ack = reinterpret_cast<const int*>(peers.base[me] + lay.ack_flags) + slot * FS_MAX_WORLD + threadIdx.x;
    if (!wait_flag_ge(ack, ack_epoch, status, limit_ns)) ok = 0;
  }
  __syncthreads();
  if (ok) {
    uint4* dst = reinterpret_cast<uint4*>(peers.base[me] + lay.slots + slot * lay.slot_bytes);
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n16; i += (long)gridDim.x * blockDim.x) dst[i] = src[i];
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) is_last = (atomicAdd(done_counter, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (is_last) {
    __threadfence_system();
    if (threadIdx.x < world) {
      int* flag = reinterpret_cast<int*>(peers.base[threadIdx.x] + lay.ready_flags) + slot * FS_MAX_WORLD + me;
      st_release_sys(flag, epoch);
    }
    if (threadIdx.x == 0) *done_counter = 0;
  }
}

__device__ __forceinline__ bool fs_wait_ready(const FsPeers& peers, const FsLayout& lay, int world, int me, int slot,
                                              int epoch, int* status, unsigned long long limit_ns, int* ok_smem) {
  if (threadIdx.x == 0) *ok_smem = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const int* flag = reinterpret_cast<const int*>(peers.base[me] + lay.ready_flags) + slot * FS_MAX_WORLD + threadIdx.x;
    if (!wait_flag_ge(flag, epoch, status, limit_ns)) *ok_smem = 0;
  }
  __syncthreads();
  return *ok_smem != 0;
}

__device__ __forceinline__ void fs_ack(const FsPeers& peers, const FsLayout& lay, int world, int me, int slot,
                                       int epoch, int* done_counter) {
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) is_last = (atomicAdd(done_counter, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (is_last) {
    if (threadIdx.x < world) {
      int* ack = reinterpret_cast<int*>(peers.base[threadIdx.x] + lay.ack_flags) + slot * FS_MAX_WORLD + me;
      st_release_sys(ack, epoch);
    }
    if (threadIdx.x == 0) *done_counter = 0;
  }
}

// dst[r * n16 + i] = peer r's staged shard[i]
__global__ void __launch_bounds__(512)
fsdp_gather_kernel(uint4* __restrict__ dst, long n16, FsPeers peers, FsLayout lay, int world, int me, int slot,
                   int epoch, int* status, unsigned long long limit_ns, int* done_counter) {
  __shared__ int ok;
  if (fs_wait_ready(peers, lay, world, me, slot, epoch, status, limit_ns, &ok)) {
    // four peer loads per thread are issued before the first store: four times the bytes in flight over NVLink
    const long total = n16 * world;
    const long stride = (long)gridDim.x * blockDim.x;
    for (long i0 = blockIdx.x * (long)blockDim.x + threadIdx.x; i0 < total; i0 += 4 * stride) {
      uint4 v[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const long i = i0 + q * stride;
        if (i < total) {
          const int r = int(i / n16);
          v[q] = reinterpret_cast<const uint4*>(peers.base[r] + lay.slots + slot * lay.slot_bytes)[i - r * n16];
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const long i = i0 + q * stride;
        if (i < total) dst[i] = v[q];
      }
    }
  }
  fs_ack(peers, lay, world, me, slot, epoch, done_counter);
}

// dst[lo .. hi) (byte offsets inside the gathered buffer) <- the staged shards that hold those bytes.  No
// acknowledgement: the kernel that gathers the rest of the buffer (the fused dense GEMM, or fsdp_gather_kernel)
// acknowledges the slot.  Used for the small tail of a flat group (its 1-D parameters), which the layer reads before
// its first GEMM.
__global__ void __launch_bounds__(256)
fsdp_gather_range_kernel(uint8_t* __restrict__ dst, long lo, long hi, long shard_bytes, FsPeers peers, FsLayout lay,
                         int world, int me, int slot, int epoch, int* status, unsigned long long limit_ns) {
  __shared__ int ok;
  if (!fs_wait_ready(peers, lay, world, me, slot, epoch, status, limit_ns, &ok)) return;
  for (long o = lo + (blockIdx.x * (long)blockDim.x + threadIdx.x) * 16; o < hi; o += (long)gridDim.x * blockDim.x * 16) {
    const int r = (int)(o / shard_bytes);
    *reinterpret_cast<uint4*>(dst + o) =
        *reinterpret_cast<const uint4*>(peers.base[r] + lay.slots + slot * lay.slot_bytes + (o - (long)r * shard_bytes));
  }
}

struct FsAdam {
  float lr, beta1, beta2, eps, wd, bc1, bc2;
  long decay_end;     // elements [0, decay_end) of the shard get weight decay (the tail holds the 1-D parameters)
};

// piece[i] = scale * sum_r peer r's staged grad[me * n8 * 8 + i]  (bf16 in, fp32 accumulate).
// FUSE_ADAM: instead of writing the reduced gradient, apply AdamW to the fp32 master shard / fp32 moments and
// write the bf16 compute copy; sum(g^2) goes to sq_out.
// `mc`: multicast address of the workspaces (the same offsets reach every rank's copy through the switch), or null.
// With it the sum over the ranks is one `multimem.ld_reduce` per 16 bytes: the switch reads every rank's slot, adds in
// fp32 and returns bf16, so a rank's NVLink ingress is its shard once instead of once per peer.
__device__ __forceinline__ void multimem_sum_bf16x8(const void* mc_addr, float (&f)[8]) {
  uint32_t r0, r1, r2, r3;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "l"(mc_addr)
               : "memory");
  bf16x8 v;
  uint32_t* u = reinterpret_cast<uint32_t*>(&v);
  u[0] = r0; u[1] = r1; u[2] = r2; u[3] = r3;
  unpack8(v, f);
}

template <bool FUSE_ADAM>
__global__ void __launch_bounds__(512)
fsdp_reduce_scatter_kernel(const uint8_t* __restrict__ mc, float* __restrict__ piece, long n8, FsPeers peers,
                           FsLayout lay, int world, int me, int slot,
                           int epoch, float scale, float* __restrict__ master, float* __restrict__ m,
                           float* __restrict__ v, __nv_bfloat16* __restrict__ out_bf16, const float* __restrict__ coef,
                           float* __restrict__ sq_out, FsAdam a, int* status, unsigned long long limit_ns,
                           int* done_counter) {
  __shared__ int ok;
  __shared__ float red[32];
  const bool good = fs_wait_ready(peers, lay, world, me, slot, epoch, status, limit_ns, &ok);
  float sq = 0.f;
  const float c = (FUSE_ADAM && coef) ? *coef : 1.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (good && mc) {
      multimem_sum_bf16x8(reinterpret_cast<const bf16x8*>(mc + lay.slots + slot * lay.slot_bytes) + (long)me * n8 + i, acc);
    } else if (good) {
      for (int r = 0; r < world; ++r) {
        const bf16x8* src = reinterpret_cast<const bf16x8*>(peers.base[r] + lay.slots + slot * lay.slot_bytes) + (long)me * n8 + i;
        float f[8];
        unpack8(*src, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= scale;
    if (!FUSE_ADAM) {
      float4* o = reinterpret_cast<float4*>(piece) + 2 * i;
      o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else if (good) {
      float4* pm = reinterpret_cast<float4*>(master) + 2 * i;
      float4* mm = reinterpret_cast<float4*>(m) + 2 * i;
      float4* vm = reinterpret_cast<float4*>(v) + 2 * i;
      float p8[8], m8[8], v8[8];
      const float decay = (i << 3) < a.decay_end ? 1.f - a.lr * a.wd : 1.f;
      *reinterpret_cast<float4*>(p8) = pm[0]; *reinterpret_cast<float4*>(p8 + 4) = pm[1];
      *reinterpret_cast<float4*>(m8) = mm[0]; *reinterpret_cast<float4*>(m8 + 4) = mm[1];
      *reinterpret_cast<float4*>(v8) = vm[0]; *reinterpret_cast<float4*>(v8 + 4) = vm[1];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        sq += acc[j] * acc[j];
        const float g = acc[j] * c;
        m8[j] = a.beta1 * m8[j] + (1.f - a.beta1) * g;
        v8[j] = a.beta2 * v8[j] + (1.f - a.beta2) * g * g;
        p8[j] = p8[j] * decay - a.lr * (m8[j] / a.bc1) / (sqrtf(v8[j] / a.bc2) + a.eps);
      }
      pm[0] = *reinterpret_cast<float4*>(p8); pm[1] = *reinterpret_cast<float4*>(p8 + 4);
      mm[0] = *reinterpret_cast<float4*>(m8); mm[1] = *reinterpret_cast<float4*>(m8 + 4);
      vm[0] = *reinterpret_cast<float4*>(v8); vm[1] = *reinterpret_cast<float4*>(v8 + 4);
      reinterpret_cast<bf16x8*>(out_bf16)[i] = pack8(p8);
    }
  }
  if (FUSE_ADAM && sq_out) {
    sq = warp_sum(sq);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
      atomicAdd(sq_out, t);
    }
  }
  fs_ack(peers, lay, world, me, slot, epoch, done_counter);
}

}  // namespace slab

using namespace slab;

static unsigned long long g_fs_limit_ns = 60ull * 1000000000ull;

extern "C" int slab_fsdp_set_wait_limit_ms(long ms) {
  g_fs_limit_ns = (unsigned long long)(ms < 1 ? 1 : ms) * 1000000ull;
  return 0;
}

static FsPeers fs_peers(const long* ptrs, int world) {
  FsPeers p;
  for (int i = 0; i < FS_MAX_WORLD; ++i) p.base[i] = i < world ? reinterpret_cast<uint8_t*>(ptrs[i]) : nullptr;
  return p;
}
// peer_ptrs[world], when world < FS_MAX_WORLD: multicast address of the workspaces, or 0 (plain peer loads).
static const uint8_t* fs_multicast(const long* ptrs, int world) {
  return world < FS_MAX_WORLD ? reinterpret_cast<const uint8_t*>(ptrs[world]) : nullptr;
}
static FsLayout fs_layout(const long* o) {
  FsLayout l;
  l.ready_flags = o[0]; l.ack_flags = o[1]; l.slots = o[2]; l.slot_bytes = o[3];
  return l;
}
static int fs_grid(long items) {
  long b = (items + 511) / 512;
  return (int)(b < 1 ? 1 : (b > 296 ? 296 : b));
}

// Copy `nbytes` (multiple of 16) from src into this rank's staging slot and publish it.  `ack_epoch` is the
// epoch of the previous call that used this slot (0: none).
extern "C" int slab_fsdp_stage(const void* src, long nbytes, const long* peer_ptrs, const long* layout, int world,
                               int me, int slot, int epoch, int ack_epoch, int* status, int* done_counter,
                               cudaStream_t st) {
  if (nbytes % 16 || world > FS_MAX_WORLD) return -100;
  FsLayout l = fs_layout(layout);
  if (nbytes > l.slot_bytes) return -101;
  fsdp_stage_kernel<<<fs_grid(nbytes / 16), 512, 0, st>>>((const uint4*)src, nbytes / 16, fs_peers(peer_ptrs, world), l,
                                                          world, me, slot, epoch, ack_epoch, status, g_fs_limit_ns,
                                                          done_counter);
  return (int)cudaGetLastError();
}

// dst (world * shard_bytes) <- every peer's staged shard
extern "C" int slab_fsdp_all_gather(void* dst, long shard_bytes, const long* peer_ptrs, const long* layout, int world,
                                    int me, int slot, int epoch, int* status, int* done_counter, cudaStream_t st) {
  if (shard_bytes % 16 || world > FS_MAX_WORLD) return -100;
  fsdp_gather_kernel<<<fs_grid(shard_bytes / 16 * world), 512, 0, st>>>((uint4*)dst, shard_bytes / 16,
                                                                        fs_peers(peer_ptrs, world), fs_layout(layout),
                                                                        world, me, slot, epoch, status, g_fs_limit_ns,
                                                                        done_counter);
  return (int)cudaGetLastError();
}

// piece (fp32, shard_numel) <- scale * sum over peers of their staged bf16 gradient slice `me`.
extern "C" int slab_fsdp_reduce_scatter(float* piece, long shard_numel, const long* peer_ptrs, const long* layout,
                                        int world, int me, int slot, int epoch, float scale, int* status,
                                        int* done_counter, cudaStream_t st) {
  if (shard_numel % 8 || world > FS_MAX_WORLD) return -100;
  FsAdam a{};
  fsdp_reduce_scatter_kernel<false><<<fs_grid(shard_numel / 8), 512, 0, st>>>(
      fs_multicast(peer_ptrs, world), piece, shard_numel / 8, fs_peers(peer_ptrs, world), fs_layout(layout), world, me, slot, epoch, scale, nullptr,
      nullptr, nullptr, nullptr, nullptr, nullptr, a, status, g_fs_limit_ns, done_counter);
  return (int)cudaGetLastError();
}

// Reduce-scatter fused with the sharded AdamW step (fp32 master / moments, bf16 compute copy out).
extern "C" int slab_fsdp_reduce_scatter_adamw(long shard_numel, const long* peer_ptrs, const long* layout, int world,
                                              int me, int slot, int epoch, float scale, float* master, float* m,
                                              float* v, void* out_bf16, const float* coef, float* sq_out, float lr,
                                              float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                                              long decay_end, int* status, int* done_counter, cudaStream_t st) {
  if (shard_numel % 8 || world > FS_MAX_WORLD || decay_end % 8) return -100;
  FsAdam a{lr, beta1, beta2, eps, wd, bc1, bc2, decay_end};
  fsdp_reduce_scatter_kernel<true><<<fs_grid(shard_numel / 8), 512, 0, st>>>(
      fs_multicast(peer_ptrs, world), nullptr, shard_numel / 8, fs_peers(peer_ptrs, world), fs_layout(layout), world, me, slot, epoch, scale, master,
      m, v, (__nv_bfloat16*)out_bf16, coef, sq_out, a, status, g_fs_limit_ns, done_counter);
  return (int)cudaGetLastError();
}

// dst[lo, hi) <- staged shards (see fsdp_gather_range_kernel); lo and hi multiples of 16, the slot not acknowledged.
extern "C" int slab_fsdp_gather_range(void* dst, long lo, long hi, long shard_bytes, const long* peer_ptrs,
                                      const long* layout, int world, int me, int slot, int epoch, int* status,
                                      cudaStream_t st) {
  if (lo % 16 || hi % 16 || shard_bytes % 16 || world > FS_MAX_WORLD || hi > shard_bytes * world) return -100;
  if (hi <= lo) return 0;
  long items = (hi - lo) / 16;
  int grid = (int)((items + 255) / 256);
  if (grid > 296) grid = 296;
  fsdp_gather_range_kernel<<<grid, 256, 0, st>>>((uint8_t*)dst, lo, hi, shard_bytes, fs_peers(peer_ptrs, world),
                                                 fs_layout(layout), world, me, slot, epoch, status, g_fs_limit_ns);
  return (int)cudaGetLastError();
}
