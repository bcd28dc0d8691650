// Micro-benchmark of the tcgen05.mma issue path: one thread issues `iters` bf16 MMAs of shape
// 128 x N x 16 back to back (operands: zero-filled shared memory or TMEM columns), then commits
// and waits; `accs` accumulators are written in rotation (1 = every MMA depends on the one
// before it). Reports the SM cycles the issuing thread spent in the issue loop and the cycles
// until the last MMA had completed. Tells how small an MMA may be before the single issuing
// thread, not the tensor pipe, sets the pace (attention backward works on 64-query halves).
//
// No counterpart in the reference (its attention kernels are WGMMA/UMMA templates from CUTLASS).
#include "common.cuh"
#include "api.h"

namespace tdllm {
namespace mma_probe {

constexpr int KID = 12;
constexpr int SMEM_BYTES = 2 * 32768 + 1024 + 64;

__global__ void __launch_bounds__(128, 1)
mma_issue_probe_kernel(int n, int iters, int a_from_tmem, int accs, int uniform, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bar = (uint64_t*)(smem + 2 * 32768);
  uint32_t* tmem_slot = (uint32_t*)(bar + 2);
  for (int i = threadIdx.x; i < 2 * 32768 / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(bar), 1);
    fence_mbar_init();
  }
  fence_proxy_async_smem();
  if (threadIdx.x < 32) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (uniform && threadIdx.x < 32) {
    // whole warp runs the loop with identical values; one elected lane issues. Lets the compiler keep
    // descriptors in uniform registers instead of moving them there per instruction.
    const bool leader = elect_one();
    const uint32_t idesc = make_idesc_bf16(128, n, 0, 0);
    const uint32_t a = smem_u32(smem), b = smem_u32(smem + 32768);
    const long long t0 = clock64();
#pragma unroll 1
    for (int i = 0; i < iters; i += 8) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t off = (k & 3) * 32;
        const uint32_t d = tmem_base + 256 + (k & (accs - 1)) * n;
        const uint64_t bd = make_smem_desc_sw128(b + off, 16, 1024);
        const uint64_t ad = make_smem_desc_sw128(a + off, 16, 1024);
        if (leader) {
          if (a_from_tmem)
            tc_mma_ts(d, tmem_base + k * 8, bd, idesc, k >= accs ? 1u : 0u);
          else
            tc_mma_ss(d, ad, bd, idesc, k >= accs ? 1u : 0u);
        }
      }
    }
    const long long t1 = clock64();
    if (leader) tc_commit(smem_u32(bar));
    const bool ok = mbar_wait(smem_u32(bar), 0, KID, 1);
    const long long t2 = clock64();
    if (blockIdx.x == 0 && leader) {
      out[0] = t1 - t0;
      out[1] = ok ? t2 - t0 : -1;
    }
  }
  if (!uniform && threadIdx.x == 0) {
    const uint32_t idesc = make_idesc_bf16(128, n, 0, 0);
    const uint32_t a = smem_u32(smem), b = smem_u32(smem + 32768);
    const long long t0 = clock64();
#pragma unroll 1
    for (int i = 0; i < iters; i += 8) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t off = (k & 3) * 32;   // stays inside one 64-element chunk: B spans at most 256 rows x 128 B
        const uint32_t d = tmem_base + 256 + (k & (accs - 1)) * n;   // `accs` (power of two) accumulators in rotation
        if (a_from_tmem)
          tc_mma_ts(d, tmem_base + k * 8, make_smem_desc_sw128(b + off, 16, 1024), idesc, k >= accs ? 1u : 0u);
        else
          tc_mma_ss(d, make_smem_desc_sw128(a + off, 16, 1024), make_smem_desc_sw128(b + off, 16, 1024),
                    idesc, k >= accs ? 1u : 0u);
      }
    }
    const long long t1 = clock64();
    tc_commit(smem_u32(bar));
    const bool ok = mbar_wait(smem_u32(bar), 0, KID, 1);
    const long long t2 = clock64();
    if (blockIdx.x == 0) {
      out[0] = t1 - t0;
      out[1] = ok ? t2 - t0 : -1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace mma_probe
}  // namespace tdllm

// out: two int64 on the device: cycles spent issuing, cycles until completion (-1: wait ran out).
extern "C" int tdllm_mma_issue_probe(int n, int iters, int a_from_tmem, int accs, int uniform, int ctas,
                                     long long* out, void* stream) {
  using namespace tdllm;
  if (n < 16 || n > 256 || (n % 16) || iters <= 0 || (iters % 8) || ctas <= 0 || (accs != 1 && accs != 2 && accs != 4) ||
      accs * n > 256) {
    tdllm_host::set_last_error("mma_issue_probe: n in 16..256 step 16, accs*n <= 256, iters a positive multiple of 8");
    return 1;
  }
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(mma_probe::mma_issue_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             mma_probe::SMEM_BYTES) != cudaSuccess) {
      tdllm_host::set_last_error("mma_issue_probe: cudaFuncSetAttribute failed");
      return 2;
    }
    attr_set = true;
  }
  mma_probe::mma_issue_probe_kernel<<<ctas, 128, mma_probe::SMEM_BYTES, (cudaStream_t)stream>>>(
      n, iters, a_from_tmem, accs, uniform, out);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
