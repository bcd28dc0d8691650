// Element-wise half of the wide-head attention path (head_dim 256, 512, any multiple of 64 above 128).
//
// The one-kernel attention of this library keeps S, P and O of a 128-wide head in the 512 TMEM columns of an
// SM; a 256- or 512-wide head does not fit that budget, so wide heads run as tensor-core products around a
// masked softmax: S = Q·Kᵀ, P = softmax(S), O = P·V in the forward pass and the five usual products in the
// backward pass, all through the tcgen05 GEMM of this library over a chunk of query rows and the key tiles
// that chunk can see (ops/wide_attention.py). The kernels here are what lies between the products:
//
//   wide_softmax_kernel      S fp32 [R, N] -> P bf16 [R, N] and the rows' log-sum-exp, under the declarative mask
//                            of the attention kernels (row: lo, hi, grp; key: code)
//   wide_softmax_bwd_kernel  S fp32, dP fp32, lse, delta -> P bf16 (for dV = Pᵀ·dO) and dS = P∘(dP − delta)·scale
//                            bf16 (for dQ = dS·K and dK = dSᵀ·Q)
//
// One CTA per row; a row is read twice in the forward kernel (online max/sum, then the normalised write), which
// stays in L2 for rows of up to a few hundred thousand keys.
// Role of the reference's wide-head attention (dllm_parallel/core/attention/wide_head_attention.py:363-1843),
// which on devices other than Hopper runs a compiled block-sparse path.
#include "common.cuh"
#include "api.h"

namespace tdllm {
namespace wide {

constexpr int THREADS = 256;

__device__ __forceinline__ bool visible(int code, int lo, int hi, int grp) {
  return code >= 0 ? (code >= lo && code < hi) : (code == grp);
}

__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < THREADS / 32) ? red[lane] : -INFINITY;
  r = warp_max(r);
  __syncthreads();
  return r;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < THREADS / 32) ? red[lane] : 0.f;
  r = warp_sum(r);
  __syncthreads();
  return r;
}

// Row r of S belongs to query (r % rows_per_head): the G query heads of a KV head are stacked along the rows.
__global__ void __launch_bounds__(THREADS)
wide_softmax_kernel(const float* __restrict__ S, __nv_bfloat16* __restrict__ P, float* __restrict__ lse,
                    const int* __restrict__ q_lo, const int* __restrict__ q_hi, const int* __restrict__ q_grp,
                    const int* __restrict__ k_code, int rows_per_head, int N, long long lds, long long ldp,
                    float scale) {
  __shared__ float red[32];
  const long long r = blockIdx.x;
  const int qi = (int)(r % rows_per_head);
  const int lo = q_lo[qi], hi = q_hi[qi], grp = q_grp[qi];
  const float* s = S + r * lds;
  __nv_bfloat16* p = P + r * ldp;
  const float sl2 = scale * 1.4426950408889634f;
  float m = -INFINITY;
  for (int j = threadIdx.x * 4; j < N; j += THREADS * 4) {
    const float4 v = *reinterpret_cast<const float4*>(s + j);
    const int4 c = *reinterpret_cast<const int4*>(k_code + j);
    if (visible(c.x, lo, hi, grp)) m = fmaxf(m, v.x);
    if (visible(c.y, lo, hi, grp)) m = fmaxf(m, v.y);
    if (visible(c.z, lo, hi, grp)) m = fmaxf(m, v.z);
    if (visible(c.w, lo, hi, grp)) m = fmaxf(m, v.w);
  }
  m = block_max(m, red);
  if (m == -INFINITY) {          // no visible key: P = 0, lse = -inf
    for (int j = threadIdx.x * 4; j < N; j += THREADS * 4)
      *reinterpret_cast<uint2*>(p + j) = make_uint2(0u, 0u);
    if (threadIdx.x == 0) lse[r] = -INFINITY;
    return;
  }
  const float ml2 = m * sl2;
  float sum = 0.f;
  for (int j = threadIdx.x * 4; j < N; j += THREADS * 4) {
    const float4 v = *reinterpret_cast<const float4*>(s + j);
    const int4 c = *reinterpret_cast<const int4*>(k_code + j);
    if (visible(c.x, lo, hi, grp)) sum += exp2f(v.x * sl2 - ml2);
    if (visible(c.y, lo, hi, grp)) sum += exp2f(v.y * sl2 - ml2);
    if (visible(c.z, lo, hi, grp)) sum += exp2f(v.z * sl2 - ml2);
    if (visible(c.w, lo, hi, grp)) sum += exp2f(v.w * sl2 - ml2);
  }
  sum = block_sum(sum, red);
  const float inv = 1.f / sum;
  for (int j = threadIdx.x * 4; j < N; j += THREADS * 4) {
    const float4 v = *reinterpret_cast<const float4*>(s + j);
    const int4 c = *reinterpret_cast<const int4*>(k_code + j);
    const float a = visible(c.x, lo, hi, grp) ? exp2f(v.x * sl2 - ml2) * inv : 0.f;
    const float b = visible(c.y, lo, hi, grp) ? exp2f(v.y * sl2 - ml2) * inv : 0.f;
    const float cc = visible(c.z, lo, hi, grp) ? exp2f(v.z * sl2 - ml2) * inv : 0.f;
    const float d = visible(c.w, lo, hi, grp) ? exp2f(v.w * sl2 - ml2) * inv : 0.f;
    *reinterpret_cast<uint2*>(p + j) = make_uint2(pack_bf16x2(a, b), pack_bf16x2(cc, d));
  }
  if (threadIdx.x == 0) lse[r] = m * scale + logf(sum);
}

// P = exp(S·scale − lse) under the mask; dS = P∘(dP − delta)·scale. lse is the log-sum-exp over ALL keys of the
// row (merged over chunks of keys or over ranks), so P is the row's true probability on this chunk's keys.
__global__ void __launch_bounds__(THREADS)
wide_softmax_bwd_kernel(const float* __restrict__ S, const float* __restrict__ dP, __nv_bfloat16* __restrict__ P,
                        __nv_bfloat16* __restrict__ dS, const float* __restrict__ lse,
                        const float* __restrict__ delta, const int* __restrict__ q_lo,
                        const int* __restrict__ q_hi, const int* __restrict__ q_grp,
                        const int* __restrict__ k_code, int rows_per_head, int N, long long lds, long long ldp,
                        float scale) {
  const long long r = blockIdx.x;
  const int qi = (int)(r % rows_per_head);
  const int lo = q_lo[qi], hi = q_hi[qi], grp = q_grp[qi];
  const float l = lse[r], dl = delta[r];
  const bool dead = (l == -INFINITY);
  const float sl2 = scale * 1.4426950408889634f, ll2 = l * 1.4426950408889634f;
  const float* s = S + r * lds;
  const float* dp = dP + r * lds;
  for (int j = threadIdx.x * 4; j < N; j += THREADS * 4) {
    const float4 v = *reinterpret_cast<const float4*>(s + j);
    const float4 g = *reinterpret_cast<const float4*>(dp + j);
    const int4 c = *reinterpret_cast<const int4*>(k_code + j);
    const float p0 = (!dead && visible(c.x, lo, hi, grp)) ? exp2f(v.x * sl2 - ll2) : 0.f;
    const float p1 = (!dead && visible(c.y, lo, hi, grp)) ? exp2f(v.y * sl2 - ll2) : 0.f;
    const float p2 = (!dead && visible(c.z, lo, hi, grp)) ? exp2f(v.z * sl2 - ll2) : 0.f;
    const float p3 = (!dead && visible(c.w, lo, hi, grp)) ? exp2f(v.w * sl2 - ll2) : 0.f;
    *reinterpret_cast<uint2*>(P + r * ldp + j) = make_uint2(pack_bf16x2(p0, p1), pack_bf16x2(p2, p3));
    *reinterpret_cast<uint2*>(dS + r * ldp + j) =
        make_uint2(pack_bf16x2(p0 * (g.x - dl) * scale, p1 * (g.y - dl) * scale),
                   pack_bf16x2(p2 * (g.z - dl) * scale, p3 * (g.w - dl) * scale));
  }
}

}  // namespace wide
}  // namespace tdllm

using namespace tdllm;

#define TD_CHECK_LAUNCH(name)                                            \
  do {                                                                   \
    cudaError_t e_ = cudaGetLastError();                                 \
    if (e_ != cudaSuccess) {                                             \
      tdllm_host::set_last_error(name ": %s", cudaGetErrorString(e_));   \
      return 4;                                                          \
    }                                                                    \
  } while (0)

static int wide_check(long long R, int N, long long lds, long long ldp, int rows_per_head) {
  if (R <= 0 || N <= 0 || N % 4 || lds % 4 || ldp % 4 || rows_per_head <= 0) {
    tdllm_host::set_last_error("wide softmax: key count and row strides must be positive multiples of 4");
    return 1;
  }
  if (R > 0x7fffffffLL) {
    tdllm_host::set_last_error("wide softmax: too many rows for one launch");
    return 1;
  }
  return 0;
}

extern "C" int tdllm_wide_softmax(const void* S, void* P, void* lse, const int* q_lo, const int* q_hi,
                                  const int* q_grp, const int* k_code, long long R, int rows_per_head, int N,
                                  long long lds, long long ldp, float scale, void* stream) {
  if (wide_check(R, N, lds, ldp, rows_per_head)) return 1;
  wide::wide_softmax_kernel<<<(unsigned)R, wide::THREADS, 0, (cudaStream_t)stream>>>(
      (const float*)S, (__nv_bfloat16*)P, (float*)lse, q_lo, q_hi, q_grp, k_code, rows_per_head, N, lds, ldp, scale);
  TD_CHECK_LAUNCH("wide_softmax");
  return 0;
}

extern "C" int tdllm_wide_softmax_bwd(const void* S, const void* dP, void* P, void* dS, const void* lse,
                                      const void* delta, const int* q_lo, const int* q_hi, const int* q_grp,
                                      const int* k_code, long long R, int rows_per_head, int N, long long lds,
                                      long long ldp, float scale, void* stream) {
  if (wide_check(R, N, lds, ldp, rows_per_head)) return 1;
  wide::wide_softmax_bwd_kernel<<<(unsigned)R, wide::THREADS, 0, (cudaStream_t)stream>>>(
      (const float*)S, (const float*)dP, (__nv_bfloat16*)P, (__nv_bfloat16*)dS, (const float*)lse,
      (const float*)delta, q_lo, q_hi, q_grp, k_code, rows_per_head, N, lds, ldp, scale);
  TD_CHECK_LAUNCH("wide_softmax_bwd");
  return 0;
}
