// Chunk-to-chunk state scan of the gated delta rule (sm_100a), forward and backward.
//
// Per (batch, head) a state S [Dk x Dv] is carried over N chunks of C tokens:
//   u_n  = Ut_n - W_n S                       (C x Dv)   corrected values of the chunk
//   o_n  = Qi_n S + QK_n u_n                  (C x Dv)   outputs
//   S   <- t_n S + Ko_n^T u_n                             state in front of chunk n+1
// Ut, W, Qi, Ko (C x Dk or C x Dv), QK (C x C, lower triangular) and t come from batched products
// over all chunks at once; only this scan is sequential. The states in front of every chunk are
// written out: block-diffusion training starts every noisy block from one of them.
//
// One CTA owns one (batch, head) and a slice of 32 value columns; the slice of S lives in shared
// memory for the whole scan, the chunk operands are staged in shared memory one chunk at a time.
// Thread (g, j) = (tid / 32, tid % 32) works on column j: operand reads are warp broadcasts (float4), state
// reads are conflict-free, and four output rows share each state load. The products are C x Dk x 32 per step (C <= 64): the scan is bound by
// the chain of N dependent steps, not by arithmetic, so it runs on the fp32 pipes.
//
// Backward walks the chunks in reverse with dS in shared memory. Gradients that sum over the value
// columns (dW, dQi, dKo, dQK, dt) are written as one partial per column slice and summed by the caller.
//
// Reference counterpart: dllm_parallel/core/kernels/gated_delta_boundary.py:65
// (chunk_gated_delta_rule_fwd_kernel_h_blockdim64) and :435 (its backward).
#include "common.cuh"
#include "api.h"

namespace tdllm {
namespace gdn {

constexpr int DVT = 32;        // value columns per CTA
constexpr int THREADS = 256;   // 8 warps: g = warp index
constexpr int G = THREADS / 32;
constexpr int MAX_C = 64;
constexpr int MAX_DK = 128;

struct FwdParams {
  const float *ut, *w, *qk, *qi, *ko, *total, *s0;
  float *o, *u, *states, *s_final;
  int N, C, Dk, Dv;
};

// shared memory (floats): S [Dk][DVT] | A [C][Dk] (W, then Qi, then Ko) | QK [C][C] | U [C][DVT]
__global__ void __launch_bounds__(THREADS) gdn_scan_fwd_kernel(const FwdParams p) {
  extern __shared__ float sm[];
  const int C = p.C, Dk = p.Dk, Dv = p.Dv, N = p.N;
  float* sS = sm;
  float* sA = sS + Dk * DVT;
  float* sQK = sA + C * Dk;
  float* sU = sQK + C * C;
  const int bh = blockIdx.x, col0 = blockIdx.y * DVT;
  const int tid = threadIdx.x, j = tid & 31, g = tid >> 5;
  for (int i = tid; i < Dk * DVT; i += THREADS) {
    const int k = i / DVT, jj = i % DVT;
    sS[i] = p.s0 ? p.s0[((size_t)bh * Dk + k) * Dv + col0 + jj] : 0.f;
  }
  __syncthreads();
  for (int n = 0; n < N; ++n) {
    const size_t chunk = (size_t)bh * N + n;
    const float* W = p.w + chunk * C * Dk;
    const float* Qi = p.qi + chunk * C * Dk;
    const float* Ko = p.ko + chunk * C * Dk;
    const float* QK = p.qk + chunk * C * C;
    const float* Ut = p.ut + chunk * C * Dv;
    // state in front of the chunk
    for (int i = tid; i < Dk * DVT; i += THREADS)
      p.states[(chunk * Dk + i / DVT) * Dv + col0 + i % DVT] = sS[i];
    for (int i = tid; i < C * Dk; i += THREADS) sA[i] = W[i];
    for (int i = tid; i < C * C; i += THREADS) sQK[i] = QK[i];
    __syncthreads();
    // u = Ut - W S: four rows per pass share every load of the state column; operand rows are read as
    // float4 broadcasts
    for (int c0 = g; c0 < C; c0 += 4 * G) {
      float acc[4];
      const float4* wr[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int c = min(c0 + r * G, C - 1);
        acc[r] = Ut[(size_t)c * Dv + col0 + j];
        wr[r] = reinterpret_cast<const float4*>(sA + c * Dk);
      }
      for (int k4 = 0; k4 < Dk / 4; ++k4) {
        const float s0v = sS[(4 * k4 + 0) * DVT + j], s1v = sS[(4 * k4 + 1) * DVT + j];
        const float s2v = sS[(4 * k4 + 2) * DVT + j], s3v = sS[(4 * k4 + 3) * DVT + j];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float4 a = wr[r][k4];
          acc[r] -= a.x * s0v + a.y * s1v + a.z * s2v + a.w * s3v;
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int c = c0 + r * G;
        if (c < C) {
          sU[c * DVT + j] = acc[r];
          p.u[(chunk * C + c) * Dv + col0 + j] = acc[r];
        }
      }
    }
    __syncthreads();
    for (int i = tid; i < C * Dk; i += THREADS) sA[i] = Qi[i];
    __syncthreads();
    // o = Qi S + QK u
    for (int c0 = g; c0 < C; c0 += 4 * G) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      const float4* qr[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) qr[r] = reinterpret_cast<const float4*>(sA + min(c0 + r * G, C - 1) * Dk);
      for (int k4 = 0; k4 < Dk / 4; ++k4) {
        const float s0v = sS[(4 * k4 + 0) * DVT + j], s1v = sS[(4 * k4 + 1) * DVT + j];
        const float s2v = sS[(4 * k4 + 2) * DVT + j], s3v = sS[(4 * k4 + 3) * DVT + j];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float4 a = qr[r][k4];
          acc[r] += a.x * s0v + a.y * s1v + a.z * s2v + a.w * s3v;
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int c = c0 + r * G;
        if (c < C) {
          float a = acc[r];
          const float* ar = sQK + c * C;
          for (int cc = 0; cc <= c; ++cc) a += ar[cc] * sU[cc * DVT + j];
          p.o[(chunk * C + c) * Dv + col0 + j] = a;
        }
      }
    }
    __syncthreads();
    for (int i = tid; i < C * Dk; i += THREADS) sA[i] = Ko[i];
    __syncthreads();
    // S = t S + Ko^T u
    const float t = p.total[chunk];
    for (int kq = g; kq < Dk / 4; kq += G) {   // four consecutive state rows per pass: one float4 of Ko per token
      const int k = 4 * kq;
      float a0 = t * sS[(k + 0) * DVT + j], a1 = t * sS[(k + 1) * DVT + j];
      float a2 = t * sS[(k + 2) * DVT + j], a3 = t * sS[(k + 3) * DVT + j];
      for (int c = 0; c < C; ++c) {
        const float4 a = *reinterpret_cast<const float4*>(sA + c * Dk + k);
        const float uv = sU[c * DVT + j];
        a0 += a.x * uv;
        a1 += a.y * uv;
        a2 += a.z * uv;
        a3 += a.w * uv;
      }
      sS[(k + 0) * DVT + j] = a0;
      sS[(k + 1) * DVT + j] = a1;
      sS[(k + 2) * DVT + j] = a2;
      sS[(k + 3) * DVT + j] = a3;
    }
    __syncthreads();
  }
  for (int i = tid; i < Dk * DVT; i += THREADS)
    p.s_final[((size_t)bh * Dk + i / DVT) * Dv + col0 + i % DVT] = sS[i];
}

struct BwdParams {
  const float *w, *qk, *qi, *ko, *total, *states, *u;   // forward operands and saved tensors
  const float *d_o, *d_states, *d_sfinal;               // incoming gradients (d_states / d_sfinal may be null)
  float *d_ut, *d_w, *d_qk, *d_qi, *d_ko, *d_total, *d_s0;   // d_w .. d_total carry a slice dimension
  int N, C, Dk, Dv, slices;
};

// shared memory (floats): dS [Dk][DVT+1] | S [Dk][DVT+1] | A [C][Dk] | QK [C][C] | U [C][DVT+1] | dO [C][DVT+1]
// | dU [C][DVT+1] | red [G]
__global__ void __launch_bounds__(THREADS) gdn_scan_bwd_kernel(const BwdParams p) {
  extern __shared__ float sm[];
  const int C = p.C, Dk = p.Dk, Dv = p.Dv, N = p.N;
  constexpr int P = DVT + 1;   // padded row: reads down a column of 32 rows hit 32 banks
  float* sdS = sm;
  float* sS = sdS + Dk * P;
  float* sA = sS + Dk * P;
  float* sQK = sA + C * Dk;
  float* sU = sQK + C * C;
  float* sdO = sU + C * P;
  float* sdU = sdO + C * P;
  float* sRed = sdU + C * P;
  const int bh = blockIdx.x, slice = blockIdx.y, col0 = slice * DVT;
  const int tid = threadIdx.x, j = tid & 31, g = tid >> 5;
  for (int i = tid; i < Dk * DVT; i += THREADS)
    sdS[(i / DVT) * P + i % DVT] =
        p.d_sfinal ? p.d_sfinal[((size_t)bh * Dk + i / DVT) * Dv + col0 + i % DVT] : 0.f;
  __syncthreads();
  for (int n = N - 1; n >= 0; --n) {
    const size_t chunk = (size_t)bh * N + n;
    const size_t part = chunk * p.slices + slice;   // index of this CTA's partial results
    const float* W = p.w + chunk * C * Dk;
    const float* Qi = p.qi + chunk * C * Dk;
    const float* Ko = p.ko + chunk * C * Dk;
    const float* QK = p.qk + chunk * C * C;
    for (int i = tid; i < Dk * DVT; i += THREADS)
      sS[(i / DVT) * P + i % DVT] = p.states[(chunk * Dk + i / DVT) * Dv + col0 + i % DVT];
    for (int i = tid; i < C * DVT; i += THREADS) {
      const int c = i / DVT, jj = i % DVT;
      sU[c * P + jj] = p.u[(chunk * C + c) * Dv + col0 + jj];
      sdO[c * P + jj] = p.d_o[(chunk * C + c) * Dv + col0 + jj];
    }
    for (int i = tid; i < C * C; i += THREADS) sQK[i] = QK[i];
    for (int i = tid; i < C * Dk; i += THREADS) sA[i] = Ko[i];
    __syncthreads();
    // dt = <dS', S> over this slice
    {
      float acc = 0.f;
      for (int k = g; k < Dk; k += G) acc += sdS[k * P + j] * sS[k * P + j];
      for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (j == 0) sRed[g] = acc;
    }
    // du = QK^T dO + Ko dS'
    for (int c0 = g; c0 < C; c0 += 4 * G) {   // four rows per pass share each load of dS'
      float acc[4];
      const float4* kr[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int c = min(c0 + r * G, C - 1);
        float a = 0.f;
        for (int cc = c; cc < C; ++cc) a += sQK[cc * C + c] * sdO[cc * P + j];
        acc[r] = a;
        kr[r] = reinterpret_cast<const float4*>(sA + c * Dk);
      }
      for (int k4 = 0; k4 < Dk / 4; ++k4) {
        const float d0 = sdS[(4 * k4 + 0) * P + j], d1 = sdS[(4 * k4 + 1) * P + j];
        const float d2 = sdS[(4 * k4 + 2) * P + j], d3 = sdS[(4 * k4 + 3) * P + j];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float4 a = kr[r][k4];
          acc[r] += a.x * d0 + a.y * d1 + a.z * d2 + a.w * d3;
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int c = c0 + r * G;
        if (c < C) {
          sdU[c * P + j] = acc[r];
          p.d_ut[(chunk * C + c) * Dv + col0 + j] = acc[r];
        }
      }
    }
    __syncthreads();
    if (tid == 0) {
      float acc = 0.f;
      for (int i = 0; i < G; ++i) acc += sRed[i];
      p.d_total[part] = acc;
    }
    // partial sums over this slice's columns: thread -> one (c, k) / (c, c') entry at a time
    const int KQ = Dk / 4;   // a thread takes entries (c, kk + r * KQ), r = 0..3: the three row operands are loaded once
    for (int i = tid; i < C * KQ; i += THREADS) {
      const int c = i / KQ, kk = i % KQ;
      float aw[4] = {0.f, 0.f, 0.f, 0.f}, aq[4] = {0.f, 0.f, 0.f, 0.f}, ak[4] = {0.f, 0.f, 0.f, 0.f};
      for (int jj = 0; jj < DVT; ++jj) {
        const float du = sdU[c * P + jj], dO = sdO[c * P + jj], uu = sU[c * P + jj];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int k = kk + r * KQ;
          const float sv = sS[k * P + jj];
          aw[r] -= du * sv;
          aq[r] += dO * sv;
          ak[r] += uu * sdS[k * P + jj];
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const size_t at = part * C * Dk + (size_t)c * Dk + kk + r * KQ;
        p.d_w[at] = aw[r];
        p.d_qi[at] = aq[r];
        p.d_ko[at] = ak[r];
      }
    }
    for (int i = tid; i < C * C; i += THREADS) {
      const int c = i / C, cc = i % C;
      float a = 0.f;
      if (cc <= c)
        for (int jj = 0; jj < DVT; ++jj) a += sdO[c * P + jj] * sU[cc * P + jj];
      p.d_qk[part * C * C + i] = a;
    }
    __syncthreads();
    // dS = Qi^T dO + t dS' - W^T du (+ gradient of the state handed out in front of this chunk)
    const float t = p.total[chunk];
    float keep[MAX_DK / G];
    for (int i = tid; i < C * Dk; i += THREADS) sA[i] = Qi[i];
    __syncthreads();
    for (int kq = g, r = 0; kq < Dk / 4; kq += G, ++r) {   // four consecutive state rows: one float4 of Qi per token
      const int k = 4 * kq;
      float a0 = t * sdS[(k + 0) * P + j], a1 = t * sdS[(k + 1) * P + j];
      float a2 = t * sdS[(k + 2) * P + j], a3 = t * sdS[(k + 3) * P + j];
      for (int c = 0; c < C; ++c) {
        const float4 a = *reinterpret_cast<const float4*>(sA + c * Dk + k);
        const float dv = sdO[c * P + j];
        a0 += a.x * dv;
        a1 += a.y * dv;
        a2 += a.z * dv;
        a3 += a.w * dv;
      }
      keep[4 * r + 0] = a0;
      keep[4 * r + 1] = a1;
      keep[4 * r + 2] = a2;
      keep[4 * r + 3] = a3;
    }
    __syncthreads();
    for (int i = tid; i < C * Dk; i += THREADS) sA[i] = W[i];
    __syncthreads();
    for (int kq = g, r = 0; kq < Dk / 4; kq += G, ++r) {
      const int k = 4 * kq;
      float a0 = keep[4 * r + 0], a1 = keep[4 * r + 1], a2 = keep[4 * r + 2], a3 = keep[4 * r + 3];
      for (int c = 0; c < C; ++c) {
        const float4 a = *reinterpret_cast<const float4*>(sA + c * Dk + k);
        const float dv = sdU[c * P + j];
        a0 -= a.x * dv;
        a1 -= a.y * dv;
        a2 -= a.z * dv;
        a3 -= a.w * dv;
      }
      if (p.d_states) {
        const float* ds = p.d_states + (chunk * Dk + k) * Dv + col0 + j;
        a0 += ds[0];
        a1 += ds[Dv];
        a2 += ds[2 * (size_t)Dv];
        a3 += ds[3 * (size_t)Dv];
      }
      sdS[(k + 0) * P + j] = a0;
      sdS[(k + 1) * P + j] = a1;
      sdS[(k + 2) * P + j] = a2;
      sdS[(k + 3) * P + j] = a3;
    }
    __syncthreads();
  }
  for (int i = tid; i < Dk * DVT; i += THREADS)
    p.d_s0[((size_t)bh * Dk + i / DVT) * Dv + col0 + i % DVT] = sdS[(i / DVT) * P + i % DVT];
}

static int check_shape(const char* what, int BH, int N, int C, int Dk, int Dv) {
  if (BH <= 0 || N <= 0 || C <= 0 || C > MAX_C || Dk <= 0 || Dk > MAX_DK || Dk % G || Dv <= 0 || Dv % DVT) {
    tdllm_host::set_last_error("%s: unsupported shape (BH %d, chunks %d, chunk %d <= %d, Dk %d <= %d and a multiple of %d, "
                   "Dv %d a multiple of %d)", what, BH, N, C, MAX_C, Dk, MAX_DK, G, Dv, DVT);
    return 1;
  }
  return 0;
}

}  // namespace gdn
}  // namespace tdllm

using namespace tdllm;

extern "C" int tdllm_gdn_scan_fwd(const float* ut, const float* w, const float* qk, const float* qi, const float* ko,
                                  const float* total, const float* s0, float* o, float* u, float* states,
                                  float* s_final, int BH, int N, int C, int Dk, int Dv, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (gdn::check_shape("gdn_scan_fwd", BH, N, C, Dk, Dv)) return 1;
  gdn::FwdParams p{ut, w, qk, qi, ko, total, s0, o, u, states, s_final, N, C, Dk, Dv};
  const size_t smem = sizeof(float) * ((size_t)Dk * gdn::DVT + (size_t)C * Dk + (size_t)C * C + (size_t)C * gdn::DVT);
  cudaError_t e = cudaFuncSetAttribute(gdn::gdn_scan_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess) {
    gdn::gdn_scan_fwd_kernel<<<dim3(BH, Dv / gdn::DVT), gdn::THREADS, smem, stream>>>(p);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    tdllm_host::set_last_error("gdn_scan_fwd: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

extern "C" int tdllm_gdn_scan_bwd(const float* w, const float* qk, const float* qi, const float* ko, const float* total,
                                  const float* states, const float* u, const float* d_o, const float* d_states,
                                  const float* d_sfinal, float* d_ut, float* d_w, float* d_qk, float* d_qi,
                                  float* d_ko, float* d_total, float* d_s0, int BH, int N, int C, int Dk, int Dv,
                                  void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (gdn::check_shape("gdn_scan_bwd", BH, N, C, Dk, Dv)) return 1;
  const int slices = Dv / gdn::DVT;
  gdn::BwdParams p{w, qk, qi, ko, total, states, u, d_o, d_states, d_sfinal, d_ut, d_w, d_qk, d_qi, d_ko, d_total,
                   d_s0, N, C, Dk, Dv, slices};
  constexpr int P = gdn::DVT + 1;
  const size_t smem = sizeof(float) * (2 * (size_t)Dk * P + (size_t)C * Dk + (size_t)C * C + 3 * (size_t)C * P + gdn::G);
  cudaError_t e = cudaFuncSetAttribute(gdn::gdn_scan_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e == cudaSuccess) {
    gdn::gdn_scan_bwd_kernel<<<dim3(BH, slices), gdn::THREADS, smem, stream>>>(p);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    tdllm_host::set_last_error("gdn_scan_bwd: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}
