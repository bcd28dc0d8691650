// Block-diffusion noising in one pass: counter-based Philox4x32-10 uniforms per token, compared
// with the per-(sample, block) move chance, producing noisy ids and labels for one or two
// complementary views (Fast-dLLM v2) including the left shift of the labels.
//
//   u(b, j) = philox(seed, counter = (offset, b * L + j)) in [0, 1)
//   standard : mask = u <= t[b, j / bs] (and eligible);  xt = mask ? mask_id : x0;  label = mask ? x0 : -100
//   v2       : sampled = u < t;  view 0 masks `sampled`, view 1 masks `!sampled` (both and eligible);
//              labels[v, j] = masked_v[j + 1] ? x0[j + 1] : -100 (last position never supervised)
// The same generator is implemented on the host (objectives/philox.py) so CPU runs and tests
// reproduce the device stream bit for bit.
//
// Reference counterpart: eager PyTorch corruption, dllm_parallel/core/objectives/runtime.py:112-212 and
// dllm_parallel/core/objectives/fast_dllm_v2.py:66-179.
#include "common.cuh"
#include "api.h"

namespace tdllm {
namespace noise {

__host__ __device__ inline void philox4x32_10(uint32_t k0, uint32_t k1, uint32_t c[4]) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)M0 * c[0], p1 = (uint64_t)M1 * c[2];
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0, n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1, n3 = (uint32_t)p0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += W0; k1 += W1;
  }
}

__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long offset,
                                           unsigned long long index) {
  uint32_t c[4] = {(uint32_t)index, (uint32_t)(index >> 32), (uint32_t)offset, (uint32_t)(offset >> 32)};
  philox4x32_10((uint32_t)seed, (uint32_t)(seed >> 32), c);
  return (float)(c[0] >> 8) * (1.0f / 16777216.0f);   // 24 random bits -> [0, 1)
}

// x0 [B, L]; t [B, L / bs]; eligible [B, L] or null; outputs [B, V, L]
__global__ void corrupt_kernel(const long long* __restrict__ x0, const float* __restrict__ t,
                               const unsigned char* __restrict__ eligible, long long* __restrict__ xt,
                               long long* __restrict__ labels, int B, int L, int bs, int views, int shift,
                               long long mask_id, unsigned long long seed, unsigned long long offset) {
  const long long n = (long long)B * L;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(i / L), j = (int)(i % L);
    const int nb = L / bs;
    const float u = uniform01(seed, offset, (unsigned long long)i);
    const bool el = eligible ? eligible[i] != 0 : true;
    const float tj = t[b * nb + j / bs];
    const bool sampled = views == 2 ? (u < tj) : (u <= tj);
    const long long tok = x0[i];
    for (int v = 0; v < views; ++v) {
      const bool m = (v == 0 ? sampled : !sampled) && el;
      xt[((long long)b * views + v) * L + j] = m ? mask_id : tok;
      if (!shift) {
        labels[((long long)b * views + v) * L + j] = m ? tok : -100;
      } else {
        if (j > 0) labels[((long long)b * views + v) * L + j - 1] = m ? tok : -100;
        if (j == L - 1) labels[((long long)b * views + v) * L + j] = -100;
      }
    }
  }
}

}  // namespace noise
}  // namespace tdllm

extern "C" int tdllm_corrupt(const long long* x0, const float* t, const unsigned char* eligible, long long* xt,
                             long long* labels, int B, int L, int block_size, int views, int shift_labels,
                             long long mask_id, unsigned long long seed, unsigned long long offset,
                             void* stream) {
  if (B <= 0 || L <= 0) return 0;
  if (L % block_size || (views != 1 && views != 2)) {
    tdllm_host::set_last_error("corrupt: L must be a multiple of block_size and views 1 or 2");
    return 1;
  }
  const long long n = (long long)B * L;
  long long blocks = (n + 255) / 256;
  const long long cap = (long long)tdllm_num_sms() * 8;
  if (blocks > cap) blocks = cap;
  tdllm::noise::corrupt_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      x0, t, eligible, xt, labels, B, L, block_size, views, shift_labels, mask_id, seed, offset);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    tdllm_host::set_last_error("corrupt launch: %s", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}
