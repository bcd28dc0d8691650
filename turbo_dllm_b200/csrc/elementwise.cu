// Bandwidth-bound kernels of the transformer block: RMSNorm (+residual), per-head q/k
// RMSNorm fused with RoPE, SwiGLU, and their backward passes. One pass over HBM each,
// 16-byte vector accesses, fp32 math, bf16 storage.
//
// Counterparts in the reference are eager PyTorch modules (HF RMSNorm / apply_rotary,
// dllm_parallel/core/models/backbones/nemotron/model.py:2236-2241, :3192, :3249) and
// Transformer Engine's LayerNormLinear / ops.SwiGLU (same file :3866-3960, :4149-4160).
#include "common.cuh"
#include "api.h"

namespace tdllm {
namespace ew {

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
  const bf16x8 raw = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(raw.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* f) {
  bf16x8 raw;
#pragma unroll
  for (int i = 0; i < 4; ++i) raw.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = raw;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}

// ---------------------------------------------------------------------------
// RMSNorm forward: h = x (+ res); y = h * rstd * w. One block per row.
// ---------------------------------------------------------------------------
template <int VPT>  // 8-element vectors per thread
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ res,
                                   const __nv_bfloat16* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out,
                                   float* __restrict__ rstd_out, int H, float eps) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int col = (threadIdx.x + i * blockDim.x) * 8;
    if (col < H) {
      load8(x + row * H + col, v[i]);
      if (res) {
        float r[8];
        load8(res + row * H + col, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += r[j];
      }
      if (h_out) {
        store8(h_out + row * H + col, v[i]);
        // normalise what was stored, so forward and recompute agree bit for bit
        load8(h_out + row * H + col, v[i]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / (float)H + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int col = (threadIdx.x + i * blockDim.x) * 8;
    if (col < H) {
      float wv[8], o[8];
      load8(w + col, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rstd * wv[j];
      store8(y + row * H + col, o);
    }
  }
}

// RMSNorm backward. dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres_in);
// dw partials are accumulated per block into dw_partial[gridDim.x, H] (fp32),
// reduced by colsum_kernel. Each block walks rows blockIdx.x, +gridDim.x, ...
template <int VPT>
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                   const __nv_bfloat16* __restrict__ h,
                                   const __nv_bfloat16* __restrict__ w,
                                   const float* __restrict__ rstd_in,
                                   const __nv_bfloat16* __restrict__ dres_in,
                                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial,
                                   int rows, int H) {
  __shared__ float red[32];
  float dwacc[VPT][8];
  float wv[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int col = (threadIdx.x + i * blockDim.x) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
    if (col < H) load8(w + col, wv[i]);
  }
  for (size_t row = blockIdx.x; row < (size_t)rows; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float g[VPT][8], xh[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int col = (threadIdx.x + i * blockDim.x) * 8;
      if (col < H) {
        load8(dy + row * H + col, g[i]);
        load8(h + row * H + col, xh[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] *= rstd;
          dwacc[i][j] += g[i][j] * xh[i][j];
          g[i][j] *= wv[i][j];
          dot += g[i][j] * xh[i][j];
        }
      }
    }
    dot = block_sum(dot, red) / (float)H;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int col = (threadIdx.x + i * blockDim.x) * 8;
      if (col < H) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - xh[i][j] * dot);
        if (dres_in) {
          float r[8];
          load8(dres_in + row * H + col, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        store8(dx + row * H + col, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int col = (threadIdx.x + i * blockDim.x) * 8;
    if (col < H) {
      float* o = dw_partial + (size_t)blockIdx.x * H + col;
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = dwacc[i][j];
    }
  }
}

// out[c] (+)= sum_r part[r, c]; out is bf16 or fp32. A block of 32 x 8 threads owns 32 columns: thread (x, y)
// adds the partial rows y, y + 8, ... of column x (a warp reads 128 contiguous bytes per row), then the eight
// row lanes meet in shared memory. The serial depth is nparts / 8 instead of nparts.
constexpr int COLSUM_COLS = 32;
constexpr int COLSUM_LANES = 8;
__global__ void __launch_bounds__(COLSUM_COLS * COLSUM_LANES)
colsum_kernel(const float* __restrict__ part, int nparts, int H, void* out, int out_fp32, int accumulate) {
  __shared__ float sm[COLSUM_LANES][COLSUM_COLS];
  const int x = threadIdx.x & (COLSUM_COLS - 1), y = threadIdx.x / COLSUM_COLS;
  const int c = blockIdx.x * COLSUM_COLS + x;
  float s0 = 0.f, s1 = 0.f;
  if (c < H) {
    int r = y;
    for (; r + COLSUM_LANES < nparts; r += 2 * COLSUM_LANES) {
      s0 += part[(size_t)r * H + c];
      s1 += part[(size_t)(r + COLSUM_LANES) * H + c];
    }
    if (r < nparts) s0 += part[(size_t)r * H + c];
  }
  sm[y][x] = s0 + s1;
  __syncthreads();
  if (y != 0 || c >= H) return;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < COLSUM_LANES; ++i) s += sm[i][x];
  if (out_fp32) {
    float* o = (float*)out;
    o[c] = accumulate ? o[c] + s : s;
  } else {
    __nv_bfloat16* o = (__nv_bfloat16*)out;
    o[c] = __float2bfloat16(accumulate ? __bfloat162float(o[c]) + s : s);
  }
}


// ---------------------------------------------------------------------------
// q/k per-head RMSNorm + RoPE on the packed projection [rows, (Hq + 2 Hkv) * D].
// One warp per (row, head). V heads are copied through. Rotation pairs (i, i + D/2).
// ---------------------------------------------------------------------------
template <int D>
__global__ void qk_norm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ in,
                                        __nv_bfloat16* __restrict__ out,
                                        const int* __restrict__ pos,
                                        const float* __restrict__ inv_freq,
                                        const __nv_bfloat16* __restrict__ qw,
                                        const __nv_bfloat16* __restrict__ kw, int rows, int Hq,
                                        int Hkv, float eps) {
  constexpr int E = D / 64;  // elements per lane per half
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nheads = Hq + 2 * Hkv;
  const size_t ld = (size_t)nheads * D;
  float fr[E];
#pragma unroll
  for (int e = 0; e < E; ++e) fr[e] = inv_freq[lane * E + e];
  for (size_t row = blockIdx.x; row < (size_t)rows; row += gridDim.x) {
    const float ps = (float)pos[row];
    float cs[E], sn[E];
#pragma unroll
    for (int e = 0; e < E; ++e) sincosf(ps * fr[e], &sn[e], &cs[e]);
    for (int h = warp; h < nheads; h += (blockDim.x >> 5)) {
      const __nv_bfloat16* src = in + row * ld + (size_t)h * D;
      __nv_bfloat16* dst = out + row * ld + (size_t)h * D;
      float a[E], b[E];
#pragma unroll
      for (int e = 0; e < E; ++e) {
        a[e] = __bfloat162float(src[lane * E + e]);
        b[e] = __bfloat162float(src[D / 2 + lane * E + e]);
      }
      if (h < Hq + Hkv) {
        const __nv_bfloat16* w = (h < Hq) ? qw : kw;
        if (w) {
          float ss = 0.f;
#pragma unroll
          for (int e = 0; e < E; ++e) ss += a[e] * a[e] + b[e] * b[e];
          ss = warp_sum(ss);
          const float rstd = rsqrtf(ss / (float)D + eps);
#pragma unroll
          for (int e = 0; e < E; ++e) {
            a[e] *= rstd * __bfloat162float(w[lane * E + e]);
            b[e] *= rstd * __bfloat162float(w[D / 2 + lane * E + e]);
          }
        }
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float x1 = a[e], x2 = b[e];
          a[e] = x1 * cs[e] - x2 * sn[e];
          b[e] = x2 * cs[e] + x1 * sn[e];
        }
      }
#pragma unroll
      for (int e = 0; e < E; ++e) {
        dst[lane * E + e] = __float2bfloat16(a[e]);
        dst[D / 2 + lane * E + e] = __float2bfloat16(b[e]);
      }
    }
  }
}

// Backward of the above. dw_partial: [gridDim.x * warps, 2, D] fp32 (q weights, k weights).
template <int D>
__global__ void qk_norm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dout,
                                        const __nv_bfloat16* __restrict__ in_raw,
                                        __nv_bfloat16* __restrict__ din,
                                        const int* __restrict__ pos,
                                        const float* __restrict__ inv_freq,
                                        const __nv_bfloat16* __restrict__ qw,
                                        const __nv_bfloat16* __restrict__ kw,
                                        float* __restrict__ dw_partial, int rows, int Hq, int Hkv,
                                        float eps) {
  constexpr int E = D / 64;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  const int nheads = Hq + 2 * Hkv;
  const size_t ld = (size_t)nheads * D;
  float fr[E];
  float dwq[2 * E], dwk[2 * E];
#pragma unroll
  for (int e = 0; e < E; ++e) fr[e] = inv_freq[lane * E + e];
#pragma unroll
  for (int e = 0; e < 2 * E; ++e) dwq[e] = dwk[e] = 0.f;
  for (size_t row = blockIdx.x; row < (size_t)rows; row += gridDim.x) {
    const float ps = (float)pos[row];
    float cs[E], sn[E];
#pragma unroll
    for (int e = 0; e < E; ++e) sincosf(ps * fr[e], &sn[e], &cs[e]);
    for (int h = warp; h < nheads; h += nwarps) {
      const __nv_bfloat16* g = dout + row * ld + (size_t)h * D;
      __nv_bfloat16* dst = din + row * ld + (size_t)h * D;
      float ga[E], gb[E];
#pragma unroll
      for (int e = 0; e < E; ++e) {
        ga[e] = __bfloat162float(g[lane * E + e]);
        gb[e] = __bfloat162float(g[D / 2 + lane * E + e]);
      }
      if (h < Hq + Hkv) {
#pragma unroll
        for (int e = 0; e < E; ++e) {  // rotate back
          const float y1 = ga[e], y2 = gb[e];
          ga[e] = y1 * cs[e] + y2 * sn[e];
          gb[e] = y2 * cs[e] - y1 * sn[e];
        }
        const __nv_bfloat16* w = (h < Hq) ? qw : kw;
        if (w) {
          const __nv_bfloat16* src = in_raw + row * ld + (size_t)h * D;
          float xa[E], xb[E];
          float ss = 0.f;
#pragma unroll
          for (int e = 0; e < E; ++e) {
            xa[e] = __bfloat162float(src[lane * E + e]);
            xb[e] = __bfloat162float(src[D / 2 + lane * E + e]);
            ss += xa[e] * xa[e] + xb[e] * xb[e];
          }
          ss = warp_sum(ss);
          const float rstd = rsqrtf(ss / (float)D + eps);
          float dot = 0.f;
#pragma unroll
          for (int e = 0; e < E; ++e) {
            xa[e] *= rstd;
            xb[e] *= rstd;
            if (h < Hq) {
              dwq[e] += ga[e] * xa[e];
              dwq[E + e] += gb[e] * xb[e];
            } else {
              dwk[e] += ga[e] * xa[e];
              dwk[E + e] += gb[e] * xb[e];
            }
            ga[e] *= __bfloat162float(w[lane * E + e]);
            gb[e] *= __bfloat162float(w[D / 2 + lane * E + e]);
            dot += ga[e] * xa[e] + gb[e] * xb[e];
          }
          dot = warp_sum(dot) / (float)D;
#pragma unroll
          for (int e = 0; e < E; ++e) {
            ga[e] = rstd * (ga[e] - xa[e] * dot);
            gb[e] = rstd * (gb[e] - xb[e] * dot);
          }
        }
      }
#pragma unroll
      for (int e = 0; e < E; ++e) {
        dst[lane * E + e] = __float2bfloat16(ga[e]);
        dst[D / 2 + lane * E + e] = __float2bfloat16(gb[e]);
      }
    }
  }
  if (dw_partial) {
    float* o = dw_partial + ((size_t)blockIdx.x * nwarps + warp) * 2 * D;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      o[lane * E + e] = dwq[e];
      o[D / 2 + lane * E + e] = dwq[E + e];
      o[D + lane * E + e] = dwk[e];
      o[D + D / 2 + lane * E + e] = dwk[E + e];
    }
  }
}

// ---------------------------------------------------------------------------
// SwiGLU on interleaved (gate, up) columns: out[r, j] = silu(gu[r, 2j]) * gu[r, 2j+1]
// ---------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ out, size_t n_out8) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_out8;
       i += (size_t)gridDim.x * blockDim.x) {
    float a[8], b[8], o[8];
    load8(gu + i * 16, a);
    load8(gu + i * 16 + 8, b);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[j] = a[2 * j] / (1.f + __expf(-a[2 * j])) * a[2 * j + 1];
      o[4 + j] = b[2 * j] / (1.f + __expf(-b[2 * j])) * b[2 * j + 1];
    }
    store8(out + i * 8, o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                  const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, size_t n_out8) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_out8;
       i += (size_t)gridDim.x * blockDim.x) {
    float a[16], g[8], o[16];
    load8(gu + i * 16, a);
    load8(gu + i * 16 + 8, a + 8);
    load8(dy + i * 8, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gate = a[2 * j], up = a[2 * j + 1];
      const float sig = 1.f / (1.f + __expf(-gate));
      o[2 * j] = g[j] * up * sig * (1.f + gate * (1.f - sig));
      o[2 * j + 1] = g[j] * gate * sig;
    }
    store8(dgu + i * 16, o);
    store8(dgu + i * 16 + 8, o + 8);
  }
}

}  // namespace ew
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

static int norm_threads(int H, int& vpt) {
  // threads * vpt * 8 >= H with vpt in {1,2,4}
  const int vecs = (H + 7) / 8;
  vpt = vecs <= 256 ? 1 : (vecs <= 512 ? 2 : 4);
  int threads = (vecs + vpt - 1) / vpt;
  threads = ((threads + 31) / 32) * 32;
  return threads;
}

extern "C" int tdllm_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y,
                                 void* h_out, float* rstd, int rows, int H, float eps,
                                 void* stream) {
  if (rows <= 0) return 0;
  if (H % 8 || H > 8192) {
    tdllm_host::set_last_error("rmsnorm: hidden size must be a multiple of 8 and <= 8192");
    return 1;
  }
  int vpt;
  const int threads = norm_threads(H, vpt);
  auto xs = (const __nv_bfloat16*)x; auto rs = (const __nv_bfloat16*)res;
  auto ws = (const __nv_bfloat16*)w; auto ys = (__nv_bfloat16*)y; auto hs = (__nv_bfloat16*)h_out;
  cudaStream_t s = (cudaStream_t)stream;
  if (vpt == 1) ew::rmsnorm_fwd_kernel<1><<<rows, threads, 0, s>>>(xs, rs, ws, ys, hs, rstd, H, eps);
  else if (vpt == 2) ew::rmsnorm_fwd_kernel<2><<<rows, threads, 0, s>>>(xs, rs, ws, ys, hs, rstd, H, eps);
  else ew::rmsnorm_fwd_kernel<4><<<rows, threads, 0, s>>>(xs, rs, ws, ys, hs, rstd, H, eps);
  TD_CHECK_LAUNCH("rmsnorm_fwd");
  return 0;
}

// scratch: fp32 [tdllm_rmsnorm_bwd_parts(), H]
extern "C" int tdllm_rmsnorm_bwd_parts(void) { return tdllm_num_sms() * 4; }

extern "C" int tdllm_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd,
                                 const void* dres_in, void* dx, void* dw, int dw_fp32,
                                 int dw_accumulate, float* scratch, int rows, int H,
                                 void* stream) {
  if (rows <= 0) return 0;
  if (H % 8 || H > 8192) {
    tdllm_host::set_last_error("rmsnorm: hidden size must be a multiple of 8 and <= 8192");
    return 1;
  }
  int vpt;
  const int threads = norm_threads(H, vpt);
  int parts = tdllm_rmsnorm_bwd_parts();
  if (parts > rows) parts = rows;
  cudaStream_t s = (cudaStream_t)stream;
  auto a = (const __nv_bfloat16*)dy; auto b = (const __nv_bfloat16*)h;
  auto c = (const __nv_bfloat16*)w; auto d = (const __nv_bfloat16*)dres_in;
  auto o = (__nv_bfloat16*)dx;
  if (vpt == 1) ew::rmsnorm_bwd_kernel<1><<<parts, threads, 0, s>>>(a, b, c, rstd, d, o, scratch, rows, H);
  else if (vpt == 2) ew::rmsnorm_bwd_kernel<2><<<parts, threads, 0, s>>>(a, b, c, rstd, d, o, scratch, rows, H);
  else ew::rmsnorm_bwd_kernel<4><<<parts, threads, 0, s>>>(a, b, c, rstd, d, o, scratch, rows, H);
  TD_CHECK_LAUNCH("rmsnorm_bwd");
  ew::colsum_kernel<<<(H + 31) / 32, 256, 0, s>>>(scratch, parts, H, dw, dw_fp32, dw_accumulate);
  TD_CHECK_LAUNCH("rmsnorm_bwd colsum");
  return 0;
}

extern "C" int tdllm_qk_norm_rope_fwd(const void* in, void* out, const int* pos,
                                      const float* inv_freq, const void* qw, const void* kw,
                                      int rows, int Hq, int Hkv, int D, float eps, void* stream) {
  if (rows <= 0) return 0;
  int grid = rows < tdllm_num_sms() * 8 ? rows : tdllm_num_sms() * 8;
  cudaStream_t s = (cudaStream_t)stream;
  if (D == 128)
    ew::qk_norm_rope_fwd_kernel<128><<<grid, 256, 0, s>>>(
        (const __nv_bfloat16*)in, (__nv_bfloat16*)out, pos, inv_freq, (const __nv_bfloat16*)qw,
        (const __nv_bfloat16*)kw, rows, Hq, Hkv, eps);
  else if (D == 64)
    ew::qk_norm_rope_fwd_kernel<64><<<grid, 256, 0, s>>>(
        (const __nv_bfloat16*)in, (__nv_bfloat16*)out, pos, inv_freq, (const __nv_bfloat16*)qw,
        (const __nv_bfloat16*)kw, rows, Hq, Hkv, eps);
  else if (D == 256)
    ew::qk_norm_rope_fwd_kernel<256><<<grid, 256, 0, s>>>(
        (const __nv_bfloat16*)in, (__nv_bfloat16*)out, pos, inv_freq, (const __nv_bfloat16*)qw,
        (const __nv_bfloat16*)kw, rows, Hq, Hkv, eps);
  else if (D == 512)
    ew::qk_norm_rope_fwd_kernel<512><<<grid, 256, 0, s>>>(
        (const __nv_bfloat16*)in, (__nv_bfloat16*)out, pos, inv_freq, (const __nv_bfloat16*)qw,
        (const __nv_bfloat16*)kw, rows, Hq, Hkv, eps);
  else {
    tdllm_host::set_last_error("qk_norm_rope: head_dim must be 64, 128, 256 or 512");
    return 1;
  }
  TD_CHECK_LAUNCH("qk_norm_rope_fwd");
  return 0;
}

// scratch: fp32 [tdllm_qk_bwd_parts(), 2*D]; dqw/dkw may be null when there is no norm
extern "C" int tdllm_qk_bwd_parts(void) { return tdllm_num_sms() * 4 * 8; }

extern "C" int tdllm_qk_norm_rope_bwd(const void* dout, const void* in_raw, void* din,
                                      const int* pos, const float* inv_freq, const void* qw,
                                      const void* kw, void* dqw, void* dkw, int dw_fp32,
                                      int dw_accumulate, float* scratch, int rows, int Hq,
                                      int Hkv, int D, float eps, void* stream) {
  if (rows <= 0) return 0;
  int grid = tdllm_num_sms() * 4;
  if (grid > rows) grid = rows;
  cudaStream_t s = (cudaStream_t)stream;
  float* part = qw ? scratch : nullptr;
  if (D == 128)
    ew::qk_norm_rope_bwd_kernel<128><<<grid, 256, 0, s>>>(
        (const __nv_bfloat16*)dout, (const __nv_bfloat16*)in_raw, (__nv_bfloat16*)din, pos,
        inv_freq, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, part, rows, Hq, Hkv, eps);
  else if (D == 64)
    ew::qk_norm_rope_bwd_kernel<64><<<grid, 256, 0, s>>>(
        (const __nv_bfloat16*)dout, (const __nv_bfloat16*)in_raw, (__nv_bfloat16*)din, pos,
        inv_freq, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, part, rows, Hq, Hkv, eps);
  else if (D == 256)
    ew::qk_norm_rope_bwd_kernel<256><<<grid, 256, 0, s>>>(
        (const __nv_bfloat16*)dout, (const __nv_bfloat16*)in_raw, (__nv_bfloat16*)din, pos,
        inv_freq, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, part, rows, Hq, Hkv, eps);
  else if (D == 512)
    ew::qk_norm_rope_bwd_kernel<512><<<grid, 256, 0, s>>>(
        (const __nv_bfloat16*)dout, (const __nv_bfloat16*)in_raw, (__nv_bfloat16*)din, pos,
        inv_freq, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, part, rows, Hq, Hkv, eps);
  else {
    tdllm_host::set_last_error("qk_norm_rope: head_dim must be 64, 128, 256 or 512");
    return 1;
  }
  TD_CHECK_LAUNCH("qk_norm_rope_bwd");
  if (part) {
    // partial rows are [q weights | k weights]; reduce both halves with stride 2*D
    const int parts = grid * 8;
    ew::colsum_kernel<<<(2 * D + 31) / 32, 256, 0, s>>>(part, parts, 2 * D, scratch + (size_t)parts * 2 * D,
                                                       1, 0);
    TD_CHECK_LAUNCH("qk colsum");
    const float* red = scratch + (size_t)parts * 2 * D;
    ew::colsum_kernel<<<(D + 31) / 32, 256, 0, s>>>(red, 1, D, dqw, dw_fp32, dw_accumulate);
    ew::colsum_kernel<<<(D + 31) / 32, 256, 0, s>>>(red + D, 1, D, dkw, dw_fp32, dw_accumulate);
    TD_CHECK_LAUNCH("qk colsum2");
  }
  return 0;
}

extern "C" int tdllm_swiglu_fwd(const void* gu, void* out, long long rows, int inter,
                                void* stream) {
  const size_t n8 = (size_t)rows * inter / 8;
  if (n8 == 0) return 0;
  if (inter % 8) {
    tdllm_host::set_last_error("swiglu: intermediate size must be a multiple of 8");
    return 1;
  }
  size_t blocks = (n8 + 255) / 256;
  const size_t cap = (size_t)tdllm_num_sms() * 16;
  ew::swiglu_fwd_kernel<<<(unsigned)(blocks > cap ? cap : blocks), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n8);
  TD_CHECK_LAUNCH("swiglu_fwd");
  return 0;
}

extern "C" int tdllm_swiglu_bwd(const void* dy, const void* gu, void* dgu, long long rows,
                                int inter, void* stream) {
  const size_t n8 = (size_t)rows * inter / 8;
  if (n8 == 0) return 0;
  if (inter % 8) {
    tdllm_host::set_last_error("swiglu: intermediate size must be a multiple of 8");
    return 1;
  }
  size_t blocks = (n8 + 255) / 256;
  const size_t cap = (size_t)tdllm_num_sms() * 16;
  ew::swiglu_bwd_kernel<<<(unsigned)(blocks > cap ? cap : blocks), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, n8);
  TD_CHECK_LAUNCH("swiglu_bwd");
  return 0;
}

// ---------------------------------------------------------------------------
// Allocation-free RMSNorm backward (declared and documented in noalloc.h).
// ---------------------------------------------------------------------------
#include "noalloc.h"

// Partial weight-gradient sums of the allocation-free entry point: one row of H floats per
// thread block. File scope, so the memory belongs to the library image on every device.
static __device__ __align__(256) float g_noalloc_scratch[TDLLM_NOALLOC_PARTS * TDLLM_NOALLOC_MAX_HIDDEN];

// In host code `g_noalloc_scratch` is only a stand-in for the symbol, not a device address,
// so the address is queried once per device and cached here.
static float* noalloc_scratch_for_current_device() {
  static float* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    tdllm_host::set_last_error("rmsnorm_bwd_noalloc: cannot identify the current device");
    return nullptr;
  }
  if (!cached[dev]) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      tdllm_host::set_last_error("rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed: %s",
                                 cudaGetErrorString(e));
      return nullptr;
    }
    cached[dev] = p;
  }
  return cached[dev];
}

extern "C" int tdllm_rmsnorm_bwd_noalloc(const void* dy, const void* h, const void* w,
                                         const float* rstd, const void* dres_in, void* dx,
                                         void* dw, int dw_fp32, int dw_accumulate, int rows, int H,
                                         void* stream) {
  if (rows <= 0) return 0;
  if (H % 8 || H <= 0 || H > TDLLM_NOALLOC_MAX_HIDDEN) {
    tdllm_host::set_last_error(
        "rmsnorm_bwd_noalloc: hidden size %d is outside the built-in scratch area (multiple of 8, at most %d)",
        H, TDLLM_NOALLOC_MAX_HIDDEN);
    return 1;
  }
  float* scratch = noalloc_scratch_for_current_device();
  if (!scratch) return 2;
  int vpt;
  const int threads = norm_threads(H, vpt);
  int parts = TDLLM_NOALLOC_PARTS;
  if (parts > rows) parts = rows;
  cudaStream_t s = (cudaStream_t)stream;
  auto a = (const __nv_bfloat16*)dy; auto b = (const __nv_bfloat16*)h;
  auto c = (const __nv_bfloat16*)w; auto d = (const __nv_bfloat16*)dres_in;
  auto o = (__nv_bfloat16*)dx;
  // every block writes its full row of partial sums, so the array needs no clearing
  if (vpt == 1) ew::rmsnorm_bwd_kernel<1><<<parts, threads, 0, s>>>(a, b, c, rstd, d, o, scratch, rows, H);
  else if (vpt == 2) ew::rmsnorm_bwd_kernel<2><<<parts, threads, 0, s>>>(a, b, c, rstd, d, o, scratch, rows, H);
  else ew::rmsnorm_bwd_kernel<4><<<parts, threads, 0, s>>>(a, b, c, rstd, d, o, scratch, rows, H);
  TD_CHECK_LAUNCH("rmsnorm_bwd_noalloc");
  ew::colsum_kernel<<<(H + 31) / 32, 256, 0, s>>>(scratch, parts, H, dw, dw_fp32, dw_accumulate);
  TD_CHECK_LAUNCH("rmsnorm_bwd_noalloc colsum");
  return 0;
}
