// Peer-memory substrate and the fused ZeRO step over NVLink / NVSwitch.
//
// Symmetric buffers: every rank cudaMalloc's the same sizes, exports IPC handles, and maps every
// peer's buffers, so kernels address peers with plain loads and stores (never TMA, never a
// library kernel given a peer pointer).
//
// Cross-rank ordering uses an epoch barrier in symmetric memory: rank r writes the epoch into
// slot r of every peer's flag array (release, system scope) and waits until all slots of its own
// array reached the epoch (acquire, bounded by the library's wait budget; on expiry the error
// record is set and the kernel returns, so a missing peer gives an exception, not a hang).
//
// Fused optimizer step (one process per GPU, each rank owns one contiguous shard of the flat
// parameter / gradient buffers):
//   zero_reduce_kernel : norm pass — sums the shard's gradient slice from every peer (bf16 -> fp32) and
//                        accumulates Σ g² of the sums for the global norm; the sums are not stored
//   zero_update_kernel : reads every rank's Σ g², sums the shard's slice from every peer again in fp32 (the
//                        gradient AdamW sees is never rounded to bf16), clips, applies AdamW to the fp32
//                        master shard and all-gathers by pushing — writes the new bf16 parameters into
//                        every peer's parameter buffer. The peers' gradient buffers stay untouched until the
//                        closing barrier.
// This replaces reduce-scatter + FusedAdam + all-gather of DeepSpeed ZeRO-2 / FSDP in the
// reference (dllm_parallel/core/optim/zero.py:93-211, :402-462; dllm_parallel/core/optim/fsdp.py:56-114).
#include <cstring>
#include "common.cuh"
#include "api.h"

namespace tdllm {
namespace comm {

constexpr int KID_BARRIER = 10;
constexpr int MAX_RANKS = 16;

struct PeerPtrs {
  void* p[MAX_RANKS];
};

// One block, one thread per rank.
__global__ void barrier_kernel(PeerPtrs flags, int rank, int world, int epoch) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  flag_store_release((int*)flags.p[r] + rank, epoch);       // tell peer r that we arrived
  flag_wait_geq((const int*)flags.p[rank] + r, epoch, KID_BARRIER, r);  // wait for peer r
}

// The arriving half of the barrier alone: tells every peer that this rank's earlier work on the stream (e.g.
// rows it staged for the peers to pull) is done. The peers wait inside the kernel that consumes it.
__global__ void signal_kernel(PeerPtrs flags, int rank, int world, int epoch) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  flag_store_release((int*)flags.p[r] + rank, epoch);
}

__device__ __forceinline__ void acc8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] += t.x;
    f[2 * i + 1] += t.y;
  }
}

// grads.p[r] = base of rank r's flat gradient buffer. Elements [start, start+n) are this rank's shard.
__global__ void zero_reduce_kernel(PeerPtrs grads, int rank, int world, long long start, long long n,
                                   float* sumsq_out, float* __restrict__ reduced) {
  float ss = 0.f;
  const long long n8 = n / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
    for (int k = 0; k < world; ++k) {
      const int r = (rank + 1 + k) % world;  // stagger peers so links are used evenly
      const uint4 v = *reinterpret_cast<const uint4*>((const __nv_bfloat16*)grads.p[r] + start + i * 8);
      acc8(v, f);
    }
    // the sum is never rounded to bf16: it is kept in fp32 when the caller gave a shard-sized scratch
    // (4 bytes per shard element), otherwise zero_update_kernel sums the same values again
    if (reduced) {
      *reinterpret_cast<float4*>(reduced + i * 8) = make_float4(f[0], f[1], f[2], f[3]);
      *reinterpret_cast<float4*>(reduced + i * 8 + 4) = make_float4(f[4], f[5], f[6], f[7]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = warp_sum(ss);
  __shared__ float red[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  if (warp == 0) {
    ss = (lane < (blockDim.x >> 5)) ? red[lane] : 0.f;
    ss = warp_sum(ss);
    if (lane == 0) atomicAdd(sumsq_out, ss);
  }
}

// sumsq.p[r] = address of rank r's Σ g² scalar (symmetric memory). params.p[r] = rank r's flat
// parameter buffer. [start, start+n) is this rank's shard; decay applies to global element
// indices below decay_end.
__global__ void zero_update_kernel(PeerPtrs params, PeerPtrs sumsq, PeerPtrs grads,
                                   const float* __restrict__ reduced, float* master, float* m, float* v, int rank, int world,
                                   long long start, long long n, long long decay_end, float lr,
                                   float beta1, float beta2, float eps, float wd, float bias1,
                                   float bias2, float grad_scale, float max_norm,
                                   float* norm_out) {
  float total = 0.f;
  for (int r = 0; r < world; ++r) total += *(const volatile float*)sumsq.p[r];
  const float norm = sqrtf(total) * grad_scale;
  if (norm_out && blockIdx.x == 0 && threadIdx.x == 0) *norm_out = norm;
  float gs = grad_scale;
  if (max_norm > 0.f && norm > max_norm) gs *= max_norm / (norm + 1e-6f);
  const float inv_b1 = 1.f / bias1;
  const float inv_sqrt_b2 = rsqrtf(bias2);
  const long long n8 = n / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    const long long e0 = i * 8;
    // Σ over ranks of the bf16 gradients, in fp32, in the order zero_reduce_kernel used for the norm
    float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (reduced) {
      *reinterpret_cast<float4*>(g) = *reinterpret_cast<const float4*>(reduced + e0);
      *reinterpret_cast<float4*>(g + 4) = *reinterpret_cast<const float4*>(reduced + e0 + 4);
    } else {
#pragma unroll 1
      for (int k = 0; k < world; ++k) {
        const int r = (rank + 1 + k) % world;
        acc8(*reinterpret_cast<const uint4*>((const __nv_bfloat16*)grads.p[r] + start + e0), g);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= gs;
    float p[8], mm[8], vv[8];
    *reinterpret_cast<float4*>(p) = *reinterpret_cast<const float4*>(master + e0);
    *reinterpret_cast<float4*>(p + 4) = *reinterpret_cast<const float4*>(master + e0 + 4);
    *reinterpret_cast<float4*>(mm) = *reinterpret_cast<const float4*>(m + e0);
    *reinterpret_cast<float4*>(mm + 4) = *reinterpret_cast<const float4*>(m + e0 + 4);
    *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(v + e0);
    *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(v + e0 + 4);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float w = (start + e0 + j < decay_end) ? wd : 0.f;
      mm[j] = beta1 * mm[j] + (1.f - beta1) * g[j];
      vv[j] = beta2 * vv[j] + (1.f - beta2) * g[j] * g[j];
      p[j] = p[j] * (1.f - lr * w) - lr * (mm[j] * inv_b1) / (sqrtf(vv[j]) * inv_sqrt_b2 + eps);
    }
    *reinterpret_cast<float4*>(master + e0) = *reinterpret_cast<float4*>(p);
    *reinterpret_cast<float4*>(master + e0 + 4) = *reinterpret_cast<float4*>(p + 4);
    *reinterpret_cast<float4*>(m + e0) = *reinterpret_cast<float4*>(mm);
    *reinterpret_cast<float4*>(m + e0 + 4) = *reinterpret_cast<float4*>(mm + 4);
    *reinterpret_cast<float4*>(v + e0) = *reinterpret_cast<float4*>(vv);
    *reinterpret_cast<float4*>(v + e0 + 4) = *reinterpret_cast<float4*>(vv + 4);
    uint4 o;
    o.x = pack_bf16x2(p[0], p[1]);
    o.y = pack_bf16x2(p[2], p[3]);
    o.z = pack_bf16x2(p[4], p[5]);
    o.w = pack_bf16x2(p[6], p[7]);
#pragma unroll 1
    for (int k = 0; k < world; ++k) {
      const int r = (rank + k) % world;
      *reinterpret_cast<uint4*>((__nv_bfloat16*)params.p[r] + start + e0) = o;
    }
  }
}


// ---------------------------------------------------------------------------
// Parameter sharding (FSDP): every rank keeps 1/W of each unit (a layer's matrices, the embedding, ...) of
// the bf16 parameters in a symmetric shard buffer. A unit is materialised just before its layer runs by
// pulling the W pieces (fsdp_gather_kernel: plain peer loads, every byte crosses NVLink once), and its
// gradients leave the full-size bf16 gradient buffer as soon as the layer's backward is done:
// fsdp_reduce_kernel pulls this rank's piece from every rank's buffer, sums in fp32 and writes (or adds to)
// the rank's fp32 gradient shard, which the sharded AdamW consumes without another cast.
// Counterparts: torch FSDP's per-module all-gather / reduce-scatter (dllm_parallel/core/optim/fsdp.py:56-114,
// :145-264) and DeepSpeed's reduce-scatter buckets (dllm_parallel/core/optim/zero.py:93-211).
// ---------------------------------------------------------------------------
__global__ void fsdp_gather_kernel(PeerPtrs shards, long long shard_off8, long long shard_len8,
                                   long long unit_len8, int rank, int world, uint4* __restrict__ out) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < unit_len8;
       i += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(i / shard_len8);
    if (!TD_CHECKED(k < world, KID_BARRIER, 0x200 + k)) continue;   // checked builds: the unit must fit its shards
    // the grid-stride walk spreads the blocks over all owners at any moment
    const long long j = i - (long long)k * shard_len8;
    out[i] = reinterpret_cast<const uint4*>(shards.p[k])[shard_off8 + j];
  }
}

__global__ void fsdp_reduce_kernel(PeerPtrs grads, long long my_off8, long long n8, int rank, int world,
                                   float* __restrict__ out, int accumulate) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
    for (int k = 0; k < world; ++k) {
      const int r = (rank + 1 + k) % world;
      acc8(reinterpret_cast<const uint4*>(grads.p[r])[my_off8 + i], f);
    }
    float4* o = reinterpret_cast<float4*>(out + i * 8);
    if (accumulate) {
      const float4 a = o[0], b = o[1];
      f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
      f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
    }
    o[0] = make_float4(f[0], f[1], f[2], f[3]);
    o[1] = make_float4(f[4], f[5], f[6], f[7]);
  }
}

// ---------------------------------------------------------------------------
// Clean K/V exchange of context-sharded block parallelism over peer memory.
//
// gather: every rank owns `count[r]` rows of `row_bytes` bytes in its symmetric staging buffer;
// this rank pulls all of them (its own included) into one local buffer laid out
// [rows of rank 0 ; rows of rank 1 ; ...], so each remote row crosses NVLink exactly once and
// the attention kernel then reads local memory with TMA.
// scatter-reduce: the transpose for gradients — every rank holds partial dK|dV for ALL gathered
// rows in its symmetric buffer (same layout); the owner pulls its slice from every peer, sums
// in fp32 and writes bf16.
// ---------------------------------------------------------------------------
struct RowPlan {
  long long offset[MAX_RANKS + 1];  // prefix sums of rows per rank
};

__global__ void kv_gather_kernel(PeerPtrs staging, RowPlan plan, int rank, int world, int row_vec16,
                                 uint4* __restrict__ out) {
  const long long total = plan.offset[world] * row_vec16;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / row_vec16;
    int r = 0;
    while (row >= plan.offset[r + 1]) ++r;
    const long long local = i - plan.offset[r] * row_vec16;
    out[i] = reinterpret_cast<const uint4*>(staging.p[r])[local];
  }
}

// partial.p[r]: rank r's [total_rows, row_bytes] bf16 partial gradients. Writes this rank's rows.
__global__ void kv_scatter_reduce_kernel(PeerPtrs partial, RowPlan plan, int rank, int world, int row_vec16,
                                         uint4* __restrict__ out) {
  const long long first = plan.offset[rank] * row_vec16;
  const long long n = (plan.offset[rank + 1] - plan.offset[rank]) * row_vec16;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
    for (int k = 0; k < world; ++k) {
      const int r = (rank + 1 + k) % world;
      acc8(reinterpret_cast<const uint4*>(partial.p[r])[first + i], f);
    }
    uint4 o;
    o.x = pack_bf16x2(f[0], f[1]);
    o.y = pack_bf16x2(f[2], f[3]);
    o.z = pack_bf16x2(f[4], f[5]);
    o.w = pack_bf16x2(f[6], f[7]);
    out[i] = o;
  }
}


// ---------------------------------------------------------------------------
// Vocab-parallel cross-entropy: cross-rank finish of the row statistics.
// Every rank holds, per row, the statistics of its vocabulary shard as written by the GEMM's
// statistics epilogue ([M, n_tiles, 3]: max, sum exp, target logit). One warp per row folds the
// tiles into (lse_shard, target_shard), writes the pair into the workspace of every rank
// ([ranks][rows_cap][2] fp32, slot of this rank), the block publishes an epoch flag per
// (rank, block) and waits (bounded) for the peers' flags of the same block, then the warps
// combine: lse = logsumexp over ranks, target = sum over ranks. No collective call.
// ---------------------------------------------------------------------------
constexpr int KID_CE_EXCHANGE = 13;

__global__ void __launch_bounds__(256)
ce_exchange_kernel(const float* __restrict__ stats, int M, int n_tiles, PeerPtrs ws, PeerPtrs flags,
                   int rank, int world, int epoch, long long rows_cap, float* __restrict__ lse_out,
                   float* __restrict__ tgt_out) {
  // the grid is small enough to be resident at once (no block waits for one that cannot start);
  // a warp walks rows blockIdx*8 + warp, + 8*gridDim, ... in both phases
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int stride = gridDim.x * 8;
  for (int row = blockIdx.x * 8 + wib; row < M; row += stride) {
    const float* s = stats + (size_t)row * n_tiles * 3;
    float mx = -INFINITY;
    for (int t = lane; t < n_tiles; t += 32) mx = fmaxf(mx, s[t * 3]);
    mx = warp_max(mx);
    float sum = 0.f, tgt = 0.f;
    for (int t = lane; t < n_tiles; t += 32) {
      const float tm = s[t * 3];
      if (tm > -INFINITY) sum += s[t * 3 + 1] * __expf(tm - mx);
      tgt += s[t * 3 + 2];
    }
    sum = warp_sum(sum);
    tgt = warp_sum(tgt);
    const float lse = (mx > -INFINITY) ? mx + logf(sum) : -INFINITY;
    if (lane < world) {
      float2* dst = (float2*)ws.p[lane] + (size_t)rank * rows_cap + row;
      *dst = make_float2(lse, tgt);
    }
  }
  __threadfence_system();
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const size_t per_rank = gridDim.x;
    flag_store_release((int*)flags.p[threadIdx.x] + (size_t)rank * per_rank + blockIdx.x, epoch);
    if (!flag_wait_geq((const int*)flags.p[rank] + (size_t)threadIdx.x * per_rank + blockIdx.x, epoch,
                       KID_CE_EXCHANGE, (int)threadIdx.x))
      ok_s = 0;
  }
  __syncthreads();
  if (!ok_s) return;
  // combine the shards (read past L1: peers wrote these lines)
  for (int row = blockIdx.x * 8 + wib; row < M; row += stride) {
    float my_l = -INFINITY, my_t = 0.f;
    if (lane < world) {
      const float* src = (const float*)ws.p[rank] + ((size_t)lane * rows_cap + row) * 2;
      asm volatile("ld.global.cg.v2.f32 {%0,%1}, [%2];" : "=f"(my_l), "=f"(my_t) : "l"(src));
    }
    const float m = warp_max(my_l);
    const float e = (my_l > -INFINITY) ? __expf(my_l - m) : 0.f;
    const float se = warp_sum(e);
    const float tg = warp_sum(my_t);
    if (lane == 0) {
      lse_out[row] = (m > -INFINITY) ? m + logf(se) : -INFINITY;
      tgt_out[row] = tg;
    }
  }
}

}  // namespace comm
}  // namespace tdllm

using namespace tdllm;

#define TD_CUDA(call, what)                                                     \
  do {                                                                          \
    cudaError_t e_ = (call);                                                    \
    if (e_ != cudaSuccess) {                                                    \
      tdllm_host::set_last_error(what ": %s", cudaGetErrorString(e_));          \
      return 5;                                                                 \
    }                                                                           \
  } while (0)

extern "C" int tdllm_symm_alloc(long long bytes, void** out) {
  TD_CUDA(cudaMalloc(out, (size_t)bytes), "symm_alloc");
  TD_CUDA(cudaMemset(*out, 0, (size_t)bytes), "symm_alloc memset");
  return 0;
}
extern "C" int tdllm_symm_free(void* p) {
  TD_CUDA(cudaFree(p), "symm_free");
  return 0;
}
// handle_out: 64 bytes
extern "C" int tdllm_ipc_get_handle(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  TD_CUDA(cudaIpcGetMemHandle(&h, p), "ipc_get_handle");
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}
extern "C" int tdllm_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  TD_CUDA(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess), "ipc_open");
  return 0;
}
extern "C" int tdllm_ipc_close(void* p) {
  TD_CUDA(cudaIpcCloseMemHandle(p), "ipc_close");
  return 0;
}

static int fill_peers(comm::PeerPtrs& pp, void* const* ptrs, int world) {
  if (world < 1 || world > comm::MAX_RANKS) {
    tdllm_host::set_last_error("comm: world size %d outside [1, %d]", world, comm::MAX_RANKS);
    return 1;
  }
  for (int i = 0; i < comm::MAX_RANKS; ++i) pp.p[i] = i < world ? ptrs[i] : nullptr;
  return 0;
}

extern "C" int tdllm_symm_barrier(void* const* flag_ptrs, int rank, int world, int epoch, void* stream) {
  comm::PeerPtrs f;
  if (fill_peers(f, flag_ptrs, world)) return 1;
  comm::barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f, rank, world, epoch);
  TD_CUDA(cudaGetLastError(), "symm_barrier launch");
  return 0;
}

extern "C" int tdllm_symm_signal(void* const* flag_ptrs, int rank, int world, int epoch, void* stream) {
  comm::PeerPtrs f;
  if (fill_peers(f, flag_ptrs, world)) return 1;
  comm::signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f, rank, world, epoch);
  TD_CUDA(cudaGetLastError(), "symm_signal launch");
  return 0;
}

// Whole fused step: barrier, pull-reduce, barrier, clip + AdamW + push, barrier.
// epoch is the first of three consecutive barrier epochs used by this call. reduced: fp32 scratch of n elements
// that carries the rank sums from the norm pass to the update pass, or null (the update pass then pulls again).
extern "C" int tdllm_zero_fused_step(void* const* grad_ptrs, void* const* param_ptrs,
                                     void* const* sumsq_ptrs, void* const* flag_ptrs, float* master,
                                     float* m, float* v, int rank, int world, long long start,
                                     long long n, long long decay_end, float lr, float beta1,
                                     float beta2, float eps, float wd, int step, float grad_scale,
                                     float max_norm, float* norm_out, int epoch, float* reduced,
                                     void* stream) {
  comm::PeerPtrs g, p, s, f;
  if (fill_peers(g, grad_ptrs, world) || fill_peers(p, param_ptrs, world) ||
      fill_peers(s, sumsq_ptrs, world) || fill_peers(f, flag_ptrs, world))
    return 1;
  if (n % 8 || start % 8) {
    tdllm_host::set_last_error("zero_fused_step: shard bounds must be multiples of 8 elements");
    return 1;
  }
  cudaStream_t st = (cudaStream_t)stream;
  TD_CUDA(cudaMemsetAsync(sumsq_ptrs[rank], 0, sizeof(float), st), "zero sumsq");
  comm::barrier_kernel<<<1, 32, 0, st>>>(f, rank, world, epoch);
  if (n > 0) {
    const int threads = 256;
    long long blocks = (n / 8 + threads - 1) / threads;
    const long long cap = (long long)tdllm_num_sms() * 8;
    if (blocks > cap) blocks = cap;
    comm::zero_reduce_kernel<<<(unsigned)blocks, threads, 0, st>>>(g, rank, world, start, n,
                                                                  (float*)sumsq_ptrs[rank], reduced);
  }
  comm::barrier_kernel<<<1, 32, 0, st>>>(f, rank, world, epoch + 1);
  if (n > 0) {
    const int threads = 256;
    long long blocks = (n / 8 + threads - 1) / threads;
    const long long cap = (long long)tdllm_num_sms() * 8;
    if (blocks > cap) blocks = cap;
    const float bias1 = 1.f - powf(beta1, (float)step);
    const float bias2 = 1.f - powf(beta2, (float)step);
    comm::zero_update_kernel<<<(unsigned)blocks, threads, 0, st>>>(
        p, s, g, reduced, master, m, v, rank, world, start, n, decay_end,
        lr, beta1, beta2, eps, wd, bias1, bias2, grad_scale, max_norm, norm_out);
  }
  comm::barrier_kernel<<<1, 32, 0, st>>>(f, rank, world, epoch + 2);
  TD_CUDA(cudaGetLastError(), "zero_fused_step launch");
  return 0;
}

static unsigned copy_blocks(long long n16) {
  long long blocks = (n16 + 255) / 256;
  const long long cap = (long long)tdllm_num_sms() * 8;
  return (unsigned)(blocks > cap ? cap : (blocks < 1 ? 1 : blocks));
}

// out[0, unit_len) = concatenation over ranks k of shard k's elements [shard_off, shard_off + shard_len)
// (bf16 elements; all three are multiples of 8). No barrier inside: the caller orders the launch after the
// barrier that follows the owners' last write of their shards.
extern "C" int tdllm_fsdp_gather(void* const* shard_ptrs, long long shard_off, long long shard_len,
                                 long long unit_len, int rank, int world, void* out, void* stream) {
  comm::PeerPtrs sp;
  if (fill_peers(sp, shard_ptrs, world)) return 1;
  if ((shard_off | shard_len | unit_len) % 8 || shard_len <= 0 || unit_len > shard_len * world) {
    tdllm_host::set_last_error("fsdp_gather: offsets and lengths must be multiples of 8 elements and the unit must fit its shards");
    return 1;
  }
  if (unit_len <= 0) return 0;
  comm::fsdp_gather_kernel<<<copy_blocks(unit_len / 8), 256, 0, (cudaStream_t)stream>>>(
      sp, shard_off / 8, shard_len / 8, unit_len / 8, rank, world, (uint4*)out);
  TD_CUDA(cudaGetLastError(), "fsdp_gather launch");
  return 0;
}

// out[0, n) (+)= sum over ranks r of grad buffer r's elements [my_off, my_off + n) (bf16 in, fp32 out).
// The caller places a barrier before (every rank's buffer is complete) and reuses a buffer only after the
// next barrier.
extern "C" int tdllm_fsdp_reduce(void* const* grad_ptrs, long long my_off, long long n, int rank, int world,
                                 float* out, int accumulate, void* stream) {
  comm::PeerPtrs gp;
  if (fill_peers(gp, grad_ptrs, world)) return 1;
  if ((my_off | n) % 8 || ((uintptr_t)out % 16)) {
    tdllm_host::set_last_error("fsdp_reduce: offset and length must be multiples of 8 elements, the output 16-byte aligned");
    return 1;
  }
  if (n <= 0) return 0;
  comm::fsdp_reduce_kernel<<<copy_blocks(n / 8), 256, 0, (cudaStream_t)stream>>>(gp, my_off / 8, n / 8, rank, world,
                                                                                 out, accumulate);
  TD_CUDA(cudaGetLastError(), "fsdp_reduce launch");
  return 0;
}

static int fill_plan(comm::RowPlan& plan, const long long* counts, int world) {
  plan.offset[0] = 0;
  for (int r = 0; r < comm::MAX_RANKS; ++r)
    plan.offset[r + 1] = plan.offset[r] + (r < world ? counts[r] : 0);
  return 0;
}

// Barrier (epoch), then pull every rank's staged rows into `out`. row_bytes % 16 == 0.
extern "C" int tdllm_kv_gather(void* const* staging_ptrs, void* const* flag_ptrs, const long long* counts,
                               int rank, int world, int row_bytes, void* out, int epoch, void* stream) {
  comm::PeerPtrs st, f;
  comm::RowPlan plan;
  if (fill_peers(st, staging_ptrs, world) || fill_peers(f, flag_ptrs, world)) return 1;
  if (row_bytes % 16) {
    tdllm_host::set_last_error("kv_gather: row_bytes must be a multiple of 16");
    return 1;
  }
  fill_plan(plan, counts, world);
  cudaStream_t s = (cudaStream_t)stream;
  comm::barrier_kernel<<<1, 32, 0, s>>>(f, rank, world, epoch);
  const long long total = plan.offset[world] * (row_bytes / 16);
  if (total > 0) {
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)tdllm_num_sms() * 8;
    if (blocks > cap) blocks = cap;
    comm::kv_gather_kernel<<<(unsigned)blocks, 256, 0, s>>>(st, plan, rank, world, row_bytes / 16, (uint4*)out);
  }
  TD_CUDA(cudaGetLastError(), "kv_gather launch");
  return 0;
}

// Barrier (epoch), pull-and-sum this rank's slice of every peer's partial gradients into `out`,
// barrier (epoch + 1) so that nobody overwrites its partial buffer while a peer still reads it.
extern "C" int tdllm_kv_scatter_reduce(void* const* partial_ptrs, void* const* flag_ptrs, const long long* counts,
                                       int rank, int world, int row_bytes, void* out, int epoch, void* stream) {
  comm::PeerPtrs pp, f;
  comm::RowPlan plan;
  if (fill_peers(pp, partial_ptrs, world) || fill_peers(f, flag_ptrs, world)) return 1;
  if (row_bytes % 16) {
    tdllm_host::set_last_error("kv_scatter_reduce: row_bytes must be a multiple of 16");
    return 1;
  }
  fill_plan(plan, counts, world);
  cudaStream_t s = (cudaStream_t)stream;
  comm::barrier_kernel<<<1, 32, 0, s>>>(f, rank, world, epoch);
  const long long n = counts[rank] * (long long)(row_bytes / 16);
  if (n > 0) {
    long long blocks = (n + 255) / 256;
    const long long cap = (long long)tdllm_num_sms() * 8;
    if (blocks > cap) blocks = cap;
    comm::kv_scatter_reduce_kernel<<<(unsigned)blocks, 256, 0, s>>>(pp, plan, rank, world, row_bytes / 16, (uint4*)out);
  }
  comm::barrier_kernel<<<1, 32, 0, s>>>(f, rank, world, epoch + 1);
  TD_CUDA(cudaGetLastError(), "kv_scatter_reduce launch");
  return 0;
}

// Cross-rank finish of vocab-parallel cross-entropy statistics over peer memory (see ce_exchange_kernel).
// ws[d]: rank d's workspace, [world][rows_cap][2] fp32; flags[d]: [world][tdllm_ce_exchange_blocks(rows_cap)] int32,
// zeroed once.
// `epoch` grows per call on one workspace; alternate two workspaces between consecutive calls.
extern "C" int tdllm_ce_exchange(const float* stats, int M, int n_tiles, void* const* ws, void* const* flags,
                                 int rank, int world, int epoch, long long rows_cap, float* lse_out,
                                 float* tgt_out, void* stream) {
  if (M <= 0) return 0;
  if (world < 1 || world > 32 || world > comm::MAX_RANKS || M > rows_cap) {
    tdllm_host::set_last_error("ce_exchange: 1..%d ranks and M <= rows_cap", comm::MAX_RANKS);
    return 1;
  }
  comm::PeerPtrs w, f;
  for (int i = 0; i < world; ++i) { w.p[i] = ws[i]; f.p[i] = flags[i]; }
  // the flag stride is the grid size: fixed by the capacity (and the device), not by M, so that every rank
  // and every call agrees on the layout; at most four blocks per SM, all resident at once
  int blocks = (int)((rows_cap + 7) / 8);
  const int cap = 4 * tdllm_num_sms();
  if (blocks > cap) blocks = cap;
  comm::ce_exchange_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(stats, M, n_tiles, w, f, rank, world, epoch,
                                                                    rows_cap, lse_out, tgt_out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    tdllm_host::set_last_error("ce_exchange launch: %s", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}

extern "C" int tdllm_ce_exchange_blocks(long long rows_cap) {
  long long blocks = (rows_cap + 7) / 8;
  const long long cap = 4LL * tdllm_num_sms();
  return (int)(blocks > cap ? cap : blocks);
}
