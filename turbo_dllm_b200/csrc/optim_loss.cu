// Flat-buffer optimizer kernels (grad-norm, clip + AdamW with fp32 master weights and a
// bf16 working copy) and the small reductions around the fused linear cross-entropy
// (row statistics -> lse / loss; soft-label KL rows), plus the online-softmax merge of
// attention shards.
//
// Reference counterparts: DeepSpeed FusedAdam behind dllm_parallel/core/optim/zero.py:402-462,
// gradient clipping in dllm_parallel/training/optimizer_setup.py:311-372, cross-entropy
// kernels in dllm_parallel/core/csrc/fused_linear_ce/fused_linear_ce_cuda.cu:156-365, and
// the merge kernels of dllm_parallel/core/csrc/cp_fusion/cp_fusion_cuda.cu:24-230.
#include "common.cuh"
#include "api.h"

namespace tdllm {
namespace ol {

// sum of squares of a bf16 buffer, atomically added to *out (fp32); out must be zeroed
__global__ void sumsq_bf16_kernel(const __nv_bfloat16* __restrict__ g, size_t n, float* out) {
  float s = 0.f;
  const size_t n8 = n / 8;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += (size_t)gridDim.x * blockDim.x) {
    const uint4 raw = *reinterpret_cast<const uint4*>(g + i * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      s += f.x * f.x + f.y * f.y;
    }
  }
  if (blockIdx.x == 0)
    for (size_t i = n8 * 8 + threadIdx.x; i < n; i += blockDim.x) {
      const float f = __bfloat162float(g[i]);
      s += f * f;
    }
  s = warp_sum(s);
  __shared__ float red[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = s;
  __syncthreads();
  if (warp == 0) {
    s = (lane < (blockDim.x >> 5)) ? red[lane] : 0.f;
    s = warp_sum(s);
    if (lane == 0) atomicAdd(out, s);
  }
}

// AdamW on a flat shard. grad_scale multiplies the gradient (loss scaling / averaging);
// when sumsq and max_norm > 0 the gradient is also clipped to max_norm using
// norm = sqrt(*sumsq) * grad_scale. step_size = lr / (1 - beta1^t); bias2 = 1 - beta2^t.
__device__ __forceinline__ float grad_as_float(const __nv_bfloat16* g, size_t i) { return __bfloat162float(g[i]); }
__device__ __forceinline__ float grad_as_float(const float* g, size_t i) { return g[i]; }

template <typename G>
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m,
                             float* __restrict__ v, const G* __restrict__ grad,
                             __nv_bfloat16* __restrict__ param, size_t n, float lr, float beta1,
                             float beta2, float eps, float wd, float bias1, float bias2,
                             float grad_scale, const float* __restrict__ sumsq, float max_norm) {
  float gs = grad_scale;
  if (sumsq && max_norm > 0.f) {
    const float norm = sqrtf(*sumsq) * grad_scale;
    if (norm > max_norm) gs *= max_norm / (norm + 1e-6f);
  }
  const float inv_b1 = 1.f / bias1;
  const float inv_sqrt_b2 = rsqrtf(bias2);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x) {
    const float g = grad_as_float(grad, i) * gs;
    float p = master[i];
    const float mi = beta1 * m[i] + (1.f - beta1) * g;
    const float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    p = p * (1.f - lr * wd) - lr * (mi * inv_b1) / (sqrtf(vi) * inv_sqrt_b2 + eps);
    master[i] = p;
    param[i] = __float2bfloat16(p);
  }
}

// Row statistics [M, n_tiles, 3] (max, sum exp, target logit) -> lse[M], and the weighted
// loss sum: out[0] += sum_r weight[r] * (lse[r] - target[r]) over rows with label >= 0,
// out[1] += number of such rows. One warp per row.
__global__ void ce_finalize_kernel(const float* __restrict__ stats, int M, int n_tiles,
                                   const int* __restrict__ labels,
                                   const float* __restrict__ weights, float* __restrict__ lse_out,
                                   float* __restrict__ loss_rows, float* __restrict__ out2) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= M) return;
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
  if (lane == 0) {
    const float lse = mx + logf(sum);
    lse_out[row] = lse;
    const bool valid = labels[row] >= 0;
    const float w = weights ? weights[row] : 1.f;
    const float l = valid ? (lse - tgt) : 0.f;
    if (loss_rows) loss_rows[row] = l;
    if (valid) {
      atomicAdd(out2, l * w);
      atomicAdd(out2 + 1, 1.f);
    }
  }
}

// ---------------------------------------------------------------------------
// Online-softmax merge of attention shard results. State per (row, head): fp32
// numerator[D], running max m, denominator l. One warp per (row, head).
//   merge:    m' = max(m, lse_s); N' = e^{m-m'} N + e^{lse_s-m'} o_s; l' likewise
//   finalize: out = N / l, lse = m + log l
// ---------------------------------------------------------------------------
__global__ void merge_kernel(float* __restrict__ num, float* __restrict__ mrun,
                             float* __restrict__ lrun, const __nv_bfloat16* __restrict__ o_s,
                             const float* __restrict__ lse_s, size_t nrh, int D, int initial) {
  const int lane = threadIdx.x & 31;
  const size_t rh = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (rh >= nrh) return;
  const float ls = lse_s[rh];
  const float m0 = initial ? -INFINITY : mrun[rh];
  const float l0 = initial ? 0.f : lrun[rh];
  const float m1 = fmaxf(m0, ls);
  const float a = (m0 > -INFINITY) ? __expf(m0 - m1) : 0.f;
  const float b = (ls > -INFINITY) ? __expf(ls - m1) : 0.f;
  for (int d = lane; d < D; d += 32) {
    const float prev = initial ? 0.f : num[rh * D + d];
    num[rh * D + d] = a * prev + b * __bfloat162float(o_s[rh * D + d]);
  }
  if (lane == 0) {
    mrun[rh] = m1;
    lrun[rh] = a * l0 + b;
  }
}

__global__ void merge_finalize_kernel(const float* __restrict__ num, const float* __restrict__ mrun,
                                      const float* __restrict__ lrun,
                                      __nv_bfloat16* __restrict__ out, float* __restrict__ lse,
                                      size_t nrh, int D) {
  const int lane = threadIdx.x & 31;
  const size_t rh = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (rh >= nrh) return;
  const float l = lrun[rh];
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int d = lane; d < D; d += 32) out[rh * D + d] = __float2bfloat16(num[rh * D + d] * inv);
  if (lane == 0) lse[rh] = l > 0.f ? mrun[rh] + logf(l) : -INFINITY;
}

// Backward of the merge for one shard: go_s = go * w, dlse_s = w * sum_d go_d (o_s,d - out_d)
// with w = exp(lse_s - lse).
__global__ void merge_bwd_kernel(const __nv_bfloat16* __restrict__ go,
                                 const __nv_bfloat16* __restrict__ out,
                                 const float* __restrict__ lse,
                                 const __nv_bfloat16* __restrict__ o_s,
                                 const float* __restrict__ lse_s, __nv_bfloat16* __restrict__ go_s,
                                 float* __restrict__ dlse_s, size_t nrh, int D) {
  const int lane = threadIdx.x & 31;
  const size_t rh = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (rh >= nrh) return;
  const float ls = lse_s[rh], lf = lse[rh];
  const float w = (ls > -INFINITY && lf > -INFINITY) ? __expf(ls - lf) : 0.f;
  float dot = 0.f;
  for (int d = lane; d < D; d += 32) {
    const float g = __bfloat162float(go[rh * D + d]);
    dot += g * (__bfloat162float(o_s[rh * D + d]) - __bfloat162float(out[rh * D + d]));
    go_s[rh * D + d] = __float2bfloat16(g * w);
  }
  dot = warp_sum(dot);
  if (lane == 0) dlse_s[rh] = w * dot;
}


// ---------------------------------------------------------------------------
// Soft-label distillation over a chunk of rows: KL(teacher || student) from two fp32 logit
// chunks [rows, V], and its gradient w.r.t. the student logits, written as bf16:
//   loss_r = sum_v p_t (log p_t - log p_s),  dlogits = (p_s - p_t) * rowscale[r]
// One block per row; pass A keeps an online (max, sum) pair per thread for both distributions,
// pass B accumulates the loss and writes the gradient. Rows with rowscale == 0 only get zeros.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void online_add(float& m, float& s, float x) {
  if (x > m) {
    s = s * __expf(m - x) + 1.f;
    m = x;
  } else {
    s += __expf(x - m);
  }
}
__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float nm = fmaxf(m, m2);
  if (nm == -INFINITY) return;
  s = s * __expf(m - nm) + s2 * __expf(m2 - nm);
  m = nm;
}

__global__ void kl_rows_kernel(const float* __restrict__ zs, const float* __restrict__ zt,
                               const float* __restrict__ rowscale, float* __restrict__ loss_rows,
                               __nv_bfloat16* __restrict__ dlogits, int V, long long ld) {
  __shared__ float red[4][32];
  const size_t row = blockIdx.x;
  const float* s = zs + row * ld;
  const float* t = zt + row * ld;
  __nv_bfloat16* g = dlogits ? dlogits + row * ld : nullptr;
  const float scale = rowscale[row];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (scale == 0.f) {
    if (g) for (int v = threadIdx.x; v < V; v += blockDim.x) g[v] = __float2bfloat16(0.f);
    if (threadIdx.x == 0) loss_rows[row] = 0.f;
    return;
  }
  float ms = -INFINITY, ss = 0.f, mt = -INFINITY, st = 0.f;
  for (int v = threadIdx.x; v < V; v += blockDim.x) {
    online_add(ms, ss, s[v]);
    online_add(mt, st, t[v]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    online_merge(ms, ss, __shfl_xor_sync(0xffffffffu, ms, o), __shfl_xor_sync(0xffffffffu, ss, o));
    online_merge(mt, st, __shfl_xor_sync(0xffffffffu, mt, o), __shfl_xor_sync(0xffffffffu, st, o));
  }
  if (lane == 0) { red[0][warp] = ms; red[1][warp] = ss; red[2][warp] = mt; red[3][warp] = st; }
  __syncthreads();
  ms = -INFINITY; ss = 0.f; mt = -INFINITY; st = 0.f;
  for (int w = 0; w < nw; ++w) {
    online_merge(ms, ss, red[0][w], red[1][w]);
    online_merge(mt, st, red[2][w], red[3][w]);
  }
  const float lse_s = ms + __logf(ss), lse_t = mt + __logf(st);
  float acc = 0.f;
  for (int v = threadIdx.x; v < V; v += blockDim.x) {
    const float ls = s[v] - lse_s, lt = t[v] - lse_t;
    const float pt = __expf(lt);
    acc += pt * (lt - ls);
    if (g) g[v] = __float2bfloat16((__expf(ls) - pt) * scale);
  }
  acc = warp_sum(acc);
  __syncthreads();
  if (lane == 0) red[0][warp] = acc;
  __syncthreads();
  if (warp == 0) {
    acc = lane < nw ? red[0][lane] : 0.f;
    acc = warp_sum(acc);
    if (lane == 0) loss_rows[row] = acc;
  }
}

}  // namespace ol
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

static inline int grid_for(size_t n, int threads, int per_sm) {
  size_t b = (n + threads - 1) / threads;
  const size_t cap = (size_t)tdllm_num_sms() * per_sm;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

extern "C" int tdllm_sumsq_bf16(const void* g, long long n, float* out, void* stream) {
  if (n <= 0) return 0;
  ol::sumsq_bf16_kernel<<<grid_for((size_t)n / 8 + 1, 256, 8), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)g, (size_t)n, out);
  TD_CHECK_LAUNCH("sumsq");
  return 0;
}

extern "C" int tdllm_adamw(float* master, float* m, float* v, const void* grad, void* param,
                           long long n, float lr, float beta1, float beta2, float eps, float wd,
                           int step, float grad_scale, const float* sumsq, float max_norm,
                           void* stream) {
  if (n <= 0) return 0;
  const float bias1 = 1.f - powf(beta1, (float)step);
  const float bias2 = 1.f - powf(beta2, (float)step);
  ol::adamw_kernel<__nv_bfloat16><<<grid_for((size_t)n, 256, 8), 256, 0, (cudaStream_t)stream>>>(
      master, m, v, (const __nv_bfloat16*)grad, (__nv_bfloat16*)param, (size_t)n, lr, beta1, beta2,
      eps, wd, bias1, bias2, grad_scale, sumsq, max_norm);
  TD_CHECK_LAUNCH("adamw");
  return 0;
}

// Same update from an fp32 gradient (the shard that the fused gradient reduce-scatter leaves behind).
extern "C" int tdllm_adamw_f32grad(float* master, float* m, float* v, const float* grad, void* param,
                                   long long n, float lr, float beta1, float beta2, float eps, float wd,
                                   int step, float grad_scale, const float* sumsq, float max_norm,
                                   void* stream) {
  if (n <= 0) return 0;
  const float bias1 = 1.f - powf(beta1, (float)step);
  const float bias2 = 1.f - powf(beta2, (float)step);
  ol::adamw_kernel<float><<<grid_for((size_t)n, 256, 8), 256, 0, (cudaStream_t)stream>>>(
      master, m, v, grad, (__nv_bfloat16*)param, (size_t)n, lr, beta1, beta2, eps, wd, bias1, bias2,
      grad_scale, sumsq, max_norm);
  TD_CHECK_LAUNCH("adamw_f32grad");
  return 0;
}

extern "C" int tdllm_ce_finalize(const float* stats, int M, int n_tiles, const int* labels,
                                 const float* weights, float* lse_out, float* loss_rows,
                                 float* out2, void* stream) {
  if (M <= 0) return 0;
  ol::ce_finalize_kernel<<<(M + 7) / 8, 256, 0, (cudaStream_t)stream>>>(
      stats, M, n_tiles, labels, weights, lse_out, loss_rows, out2);
  TD_CHECK_LAUNCH("ce_finalize");
  return 0;
}

extern "C" int tdllm_attn_merge(float* num, float* mrun, float* lrun, const void* o_s,
                                const float* lse_s, long long nrh, int D, int initial,
                                void* stream) {
  if (nrh <= 0) return 0;
  ol::merge_kernel<<<(unsigned)((nrh + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      num, mrun, lrun, (const __nv_bfloat16*)o_s, lse_s, (size_t)nrh, D, initial);
  TD_CHECK_LAUNCH("attn_merge");
  return 0;
}
extern "C" int tdllm_attn_merge_finalize(const float* num, const float* mrun, const float* lrun,
                                         void* out, float* lse, long long nrh, int D,
                                         void* stream) {
  if (nrh <= 0) return 0;
  ol::merge_finalize_kernel<<<(unsigned)((nrh + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      num, mrun, lrun, (__nv_bfloat16*)out, lse, (size_t)nrh, D);
  TD_CHECK_LAUNCH("attn_merge_finalize");
  return 0;
}
extern "C" int tdllm_attn_merge_bwd(const void* go, const void* out, const float* lse,
                                    const void* o_s, const float* lse_s, void* go_s,
                                    float* dlse_s, long long nrh, int D, void* stream) {
  if (nrh <= 0) return 0;
  ol::merge_bwd_kernel<<<(unsigned)((nrh + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)go, (const __nv_bfloat16*)out, lse, (const __nv_bfloat16*)o_s, lse_s,
      (__nv_bfloat16*)go_s, dlse_s, (size_t)nrh, D);
  TD_CHECK_LAUNCH("attn_merge_bwd");
  return 0;
}

extern "C" int tdllm_kl_rows(const float* student_logits, const float* teacher_logits, const float* rowscale,
                             float* loss_rows, void* dlogits_bf16, int rows, int V, long long ld,
                             void* stream) {
  if (rows <= 0) return 0;
  ol::kl_rows_kernel<<<rows, 512, 0, (cudaStream_t)stream>>>(student_logits, teacher_logits, rowscale, loss_rows,
                                                           (__nv_bfloat16*)dlogits_bf16, V, ld);
  TD_CHECK_LAUNCH("kl_rows");
  return 0;
}
