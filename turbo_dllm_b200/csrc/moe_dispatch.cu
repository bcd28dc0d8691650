// Expert-parallel dispatch and combine over peer memory (no NCCL call, no host read of the routing).
//
// Every rank owns E_local = E / W experts. One routed batch goes through these phases, all of them kernels on
// the rank's stream:
//   1. counts exchange  : the rank's rows-per-expert histogram is stored into every rank's [W][E] table (plain
//                         peer stores), followed by a flag exchange with bounded waits. Every rank then knows
//                         how many rows each source sends to each expert and derives, on the device, the padded
//                         row layout of every owner (each expert's rows contiguous, segments on 256-row
//                         boundaries, as the grouped GEMM wants them) and its own write offset per expert.
//   2. dispatch          : one warp per (token, choice) copies the token's row straight into the owner's slab
//                         at the expert's segment (16-byte peer stores; the slot inside the segment comes from
//                         a local atomic counter per expert, so no two rows collide). The slot is remembered.
//   3. expert GEMMs      : the owner runs its grouped GEMMs over the slab (csrc/gemm_sm100.cu, grouped form).
//   4. combine           : one warp per token pulls its k expert outputs from the owners' output slabs by the
//                         remembered slots, weights and sums them.
// The backward pass sends weighted output gradients along the same slots (4 reversed), runs the grouped
// backward products, and pulls the input gradients back (2 reversed). A slab that overflows its static capacity
// sets ERR_CAPACITY in the device error record and drops the row; nothing is written out of bounds.
//
// Counterpart of the DeepEP dispatch / combine ops the reference wraps
// (dllm_parallel/core/parallel/expert/deepep.py:122-555) and of its expert-parallel layer
// (dllm_parallel/core/models/backbones/diffusiongemma/expert_parallel.py:71-321).
#include "common.cuh"
#include "api.h"

namespace tdllm {
namespace ep {

constexpr int KID_EP = 14;
constexpr int MAX_RANKS = 16;

struct Peers {
  void* p[MAX_RANKS];
};

// One block. my_counts [E] -> tabs.p[d][rank * E + e] on every rank d, then the flag exchange.
__global__ void counts_exchange_kernel(const int* __restrict__ my_counts, Peers tabs, Peers flags, int rank,
                                       int world, int E, int epoch) {
  for (int i = threadIdx.x; i < E * world; i += blockDim.x) {
    const int d = i / E, e = i - d * E;
    ((int*)tabs.p[d])[rank * E + e] = my_counts[e];
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < world) {
    const int r = threadIdx.x;
    flag_store_release((int*)flags.p[r] + rank, epoch);
    flag_wait_geq((const int*)flags.p[rank] + r, epoch, KID_EP, r);
  }
}

// x [rows, H] bf16; experts [rows * k] (global expert id per item); base [E] first slot of this rank's rows
// inside the expert's segment of the owner's slab; counters [E] zero at launch. One warp per item.
__global__ void dispatch_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ experts,
                                     const float* __restrict__ scale, const long long* __restrict__ base,
                                     int* __restrict__ counters, const int* __restrict__ pos_in,
                                     int* __restrict__ pos_out, Peers slabs, long long items, int k, int h_vec16,
                                     int e_local, long long cap_rows) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long it = (((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5); it < items; it += warps) {
    const int e = experts[it];
    if (!TD_CHECKED(e >= 0 && e / e_local < MAX_RANKS, KID_EP, 0x300)) continue;   // checked builds: a valid expert id
    long long p;
    if (pos_in) {
      p = pos_in[it];                       // the slot this item took in the forward pass
    } else {
      int c = 0;
      if (lane == 0) c = atomicAdd(counters + e, 1);
      c = __shfl_sync(0xffffffffu, c, 0);
      p = base[e] + c;
      if (p >= cap_rows) {
        if (lane == 0) {
          set_error(ERR_CAPACITY, KID_EP, e);
          pos_out[it] = -1;
        }
        continue;
      }
      if (lane == 0) pos_out[it] = (int)p;
    }
    if (p < 0) continue;
    const uint4* src = x + (it / k) * h_vec16;
    uint4* dst = (uint4*)slabs.p[e / e_local] + p * h_vec16;
    if (scale) {
      // backward: the row travels multiplied by the item's routing weight
      const float s = scale[it];
      for (int i = lane; i < h_vec16; i += 32) {
        uint4 v = src[i];
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(h2[j]);
          h2[j] = __floats2bfloat162_rn(f.x * s, f.y * s);
        }
        dst[i] = v;
      }
    } else {
      for (int i = lane; i < h_vec16; i += 32) dst[i] = src[i];
    }
  }
}

// Zeroes the padding rows between an expert's last row and the next 256-row boundary of this rank's slab
// (the weight-gradient product sums over whole segments). begin / count: [E_local].
__global__ void zero_pad_rows_kernel(uint4* __restrict__ slab, const long long* __restrict__ begin,
                                     const long long* __restrict__ count, int h_vec16) {
  const int e = blockIdx.y;
  const long long first = begin[e] + count[e];
  const long long last = begin[e] + (count[e] + 255) / 256 * 256;
  const long long n = (last - first) * h_vec16;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    slab[first * h_vec16 + i] = make_uint4(0, 0, 0, 0);
}

// out[token] = sum_k w[token, k] * y_owner[pos[token, k]] (weights null = plain sum). `keep` (optional,
// [rows * k, H]) receives the pulled rows unweighted: the backward needs them for the routing-weight gradient.
// One warp per token; H = h_vec16 * 8 <= 8192.
__global__ void combine_rows_kernel(uint4* __restrict__ out, const float* __restrict__ weights,
                                    const int* __restrict__ experts, const int* __restrict__ pos, Peers slabs,
                                    uint4* __restrict__ keep, long long rows, int k, int h_vec16, int e_local) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long t = (((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5); t < rows; t += warps) {
    for (int i0 = lane; i0 < h_vec16; i0 += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < k; ++j) {
        const long long it = t * k + j;
        const int p = pos[it];
        uint4 v = make_uint4(0, 0, 0, 0);
        if (p >= 0) {
          const uint4* src = (const uint4*)slabs.p[experts[it] / e_local] + (long long)p * h_vec16 + i0;
          asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                       : "l"(src)
                       : "memory");
        }
        if (keep) keep[it * h_vec16 + i0] = v;
        const float w = weights ? weights[it] : 1.f;
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __bfloat1622float2(h2[q]);
          acc[2 * q] += w * f.x;
          acc[2 * q + 1] += w * f.y;
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      out[t * h_vec16 + i0] = o;
    }
  }
}

// dw[token, k] = <dout[token], y[token, k]> (fp32): gradient of the routing weights. One warp per item.
__global__ void weight_grad_kernel(const uint4* __restrict__ dout, const uint4* __restrict__ y,
                                   float* __restrict__ dw, long long items, int k, int h_vec16) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long it = (((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5); it < items; it += warps) {
    float s = 0.f;
    for (int i = lane; i < h_vec16; i += 32) {
      const uint4 a = dout[(it / k) * h_vec16 + i], b = y[it * h_vec16 + i];
      const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 fa = __bfloat1622float2(ha[q]), fb = __bfloat1622float2(hb[q]);
        s += fa.x * fb.x + fa.y * fb.y;
      }
    }
    s = warp_sum(s);
    if (lane == 0) dw[it] = s;
  }
}

}  // namespace ep
}  // namespace tdllm

using namespace tdllm;

static int ep_fill(ep::Peers& pp, void* const* ptrs, int world) {
  if (world < 1 || world > ep::MAX_RANKS) {
    tdllm_host::set_last_error("ep: world size %d outside [1, %d]", world, ep::MAX_RANKS);
    return 1;
  }
  for (int i = 0; i < ep::MAX_RANKS; ++i) pp.p[i] = i < world ? ptrs[i] : nullptr;
  return 0;
}

static unsigned ep_blocks(long long warps_wanted) {
  long long blocks = (warps_wanted + 7) / 8;
  const long long cap = (long long)tdllm_num_sms() * 16;
  return (unsigned)(blocks > cap ? cap : (blocks < 1 ? 1 : blocks));
}

#define EP_LAUNCH_CHECK(what)                                                   \
  do {                                                                          \
    cudaError_t e_ = cudaGetLastError();                                        \
    if (e_ != cudaSuccess) {                                                    \
      tdllm_host::set_last_error(what ": %s", cudaGetErrorString(e_));          \
      return 4;                                                                 \
    }                                                                           \
  } while (0)

// my_counts [E] int32 (device) -> every rank's table tabs[d] ([world][E] int32, symmetric), then a flag exchange
// over flags[d] (int32[world], symmetric) at `epoch`: on return of the kernel this rank's table is complete.
extern "C" int tdllm_ep_counts_exchange(const int* my_counts, void* const* tabs, void* const* flags, int rank,
                                        int world, int E, int epoch, void* stream) {
  ep::Peers t, f;
  if (ep_fill(t, tabs, world) || ep_fill(f, flags, world)) return 1;
  ep::counts_exchange_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(my_counts, t, f, rank, world, E, epoch);
  EP_LAUNCH_CHECK("ep_counts_exchange launch");
  return 0;
}

// Copies row item / k of x [rows, H] (bf16) into the slab of the owner of experts[item] at slot
// base[expert] + (arrival order), or at pos_in[item] when given (backward: same slots as the forward), optionally
// multiplied by scale[item]. counters [E] int32 must be zero (not used with pos_in). pos_out [items] receives
// the slots (-1 = dropped for lack of capacity, error record set).
extern "C" int tdllm_ep_dispatch(const void* x, const int* experts, const float* scale, const long long* base,
                                 int* counters, const int* pos_in, int* pos_out, void* const* slabs,
                                 long long rows, int k, int H, int e_local, long long cap_rows, int world,
                                 void* stream) {
  ep::Peers s;
  if (ep_fill(s, slabs, world)) return 1;
  if (H % 8 || ((uintptr_t)x % 16)) {
    tdllm_host::set_last_error("ep_dispatch: H must be a multiple of 8 and x 16-byte aligned");
    return 1;
  }
  const long long items = rows * k;
  if (items <= 0) return 0;
  ep::dispatch_rows_kernel<<<ep_blocks(items), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)x, experts, scale, base, counters, pos_in, pos_out, s, items, k, H / 8, e_local, cap_rows);
  EP_LAUNCH_CHECK("ep_dispatch launch");
  return 0;
}

extern "C" int tdllm_ep_zero_pad_rows(void* slab, const long long* begin, const long long* count, int e_local,
                                      int H, void* stream) {
  if (e_local <= 0) return 0;
  dim3 grid(8, e_local);
  ep::zero_pad_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((uint4*)slab, begin, count, H / 8);
  EP_LAUNCH_CHECK("ep_zero_pad_rows launch");
  return 0;
}

extern "C" int tdllm_ep_combine(void* out, const float* weights, const int* experts, const int* pos,
                                void* const* slabs, void* keep, long long rows, int k, int H, int e_local,
                                int world, void* stream) {
  ep::Peers s;
  if (ep_fill(s, slabs, world)) return 1;
  if (H % 8) {
    tdllm_host::set_last_error("ep_combine: H must be a multiple of 8");
    return 1;
  }
  if (rows <= 0) return 0;
  ep::combine_rows_kernel<<<ep_blocks(rows), 256, 0, (cudaStream_t)stream>>>(
      (uint4*)out, weights, experts, pos, s, (uint4*)keep, rows, k, H / 8, e_local);
  EP_LAUNCH_CHECK("ep_combine launch");
  return 0;
}

extern "C" int tdllm_ep_weight_grad(const void* dout, const void* y, float* dw, long long rows, int k, int H,
                                    void* stream) {
  const long long items = rows * k;
  if (items <= 0) return 0;
  ep::weight_grad_kernel<<<ep_blocks(items), 256, 0, (cudaStream_t)stream>>>((const uint4*)dout, (const uint4*)y,
                                                                            dw, items, k, H / 8);
  EP_LAUNCH_CHECK("ep_weight_grad launch");
  return 0;
}
