// Block-diffusion attention backward, query gradient (sm_100a, head_dim 128).
//
// Same CTA shape as the forward kernel: one 128-row query tile, two query heads that share
// a KV head, two softmax-style warp groups in ping-pong, one TMA warp, one MMA warp.
// Keys are streamed in 64-row sub-tiles so that everything fits TMEM:
//   S_i = Q_i·Kᵀ (64 cols), dP_i = dO_i·Vᵀ (64 cols) for i = 0,1   -> 256 columns
//   dQ_i accumulators (128 cols each)                              -> 256 columns
// The warp group turns (S, dP) into dS = P∘(dP − delta)·scale with P = exp(S·scale − lse),
// writes dS as bf16 over the S columns, and the MMA warp accumulates dQ_i += dS_i·K with
// the A operand read from TMEM and K read MN-major from the same shared-memory tile.
//
// Reference counterpart: the dQ half of the masked FlashAttention backward
// (third_party/flash-attention/hopper/mainloop_bwd_sm90_tma_gmma_ws.hpp, FA4
// flash_bwd_sm100.py), driven from state (out, lse) as in
// dllm_parallel/core/attention/fa4.py:230-296.
#include "common.cuh"
#include "api.h"

namespace tdllm {
namespace attn_dq {

constexpr int KID = 3;
constexpr int BQ = 128;
constexpr int SUB = 64;   // keys per sub-tile
constexpr int HD = 128;
constexpr int QTILE_BYTES = 128 * HD * 2;   // 32 KiB (two 64-column halves)
constexpr int QHALF_BYTES = QTILE_BYTES / 2;
constexpr int KSUB_BYTES = SUB * HD * 2;    // 16 KiB (two halves of 64 rows x 128 B)
constexpr int KHALF_BYTES = KSUB_BYTES / 2;
constexpr int THREADS = 320;
constexpr int SMEM_BYTES = 4 * QTILE_BYTES + 4 * KSUB_BYTES + 512 + 1024;

struct Params {
  int nq_pad, Hq, Hkv;
  const int* q_lo;
  const int* q_hi;
  const int* q_grp;
  const int* k_code;
  const int* tile_ptr;
  const int* tile_idx;
  const int* order;
  const float* lse2;   // [Hq, nq_pad] −lse·log2e (−inf = row without keys)
  const float* delta;  // [Hq, nq_pad] −scale · rowsum(dO∘O)
  float scale_log2, scale;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
      "r"(r[15])
      : "memory");
}
__device__ __forceinline__ bool key_visible(int code, int lo, int hi, int grp) {
  return code >= 0 ? (code >= lo && code < hi) : (code == grp);
}

__global__ void __launch_bounds__(THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                   const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const __grid_constant__ CUtensorMap tm_dq, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                        // 2 x 32 KiB
  uint8_t* sdO = sQ + 2 * QTILE_BYTES;       // 2 x 32 KiB
  uint8_t* sK = sdO + 2 * QTILE_BYTES;       // 2 stages x 16 KiB
  uint8_t* sV = sK + 2 * KSUB_BYTES;         // 2 stages x 16 KiB
  uint64_t* bars = (uint64_t*)(sV + 2 * KSUB_BYTES);
  const uint32_t b0 = smem_u32(bars);
  const uint32_t bar_q = b0;
  const uint32_t bar_kfull = b0 + 8, bar_kempty = b0 + 24, bar_vfull = b0 + 40, bar_vempty = b0 + 56;
  const uint32_t bar_sfull = b0 + 72, bar_pfull = b0 + 88, bar_odone = b0 + 104, bar_epi = b0 + 120;
  uint32_t* tmem_slot = (uint32_t*)(bars + 17);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  const int pairs = G / 2;
  int w = blockIdx.x;
  const int pr = w % pairs;
  w /= pairs;
  const int kvh = w % p.Hkv;
  const int qt = p.order[w / p.Hkv];
  const int h0 = kvh * G + 2 * pr;
  const int list_begin = p.tile_ptr[qt];
  const int n = p.tile_ptr[qt + 1] - list_begin;
  const int* list = p.tile_idx + list_begin;
  const int U = 2 * n;  // 64-key sub-tiles

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_kfull + 8 * s, 1);
      mbar_init(bar_kempty + 8 * s, 1);
      mbar_init(bar_vfull + 8 * s, 1);
      mbar_init(bar_vempty + 8 * s, 1);
      mbar_init(bar_sfull + 8 * s, 1);
      mbar_init(bar_pfull + 8 * s, 128);
      mbar_init(bar_odone + 8 * s, 1);
      mbar_init(bar_epi + 8 * s, 128);
    }
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // columns: S_i at i*128, dP_i at i*128+64, dQ_i at 256+i*128; dS_i aliases S_i[0,32)

  if (warp == 8) {
    if (lane == 0 && n > 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_do);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      mbar_expect_tx(bar_q, 4 * QTILE_BYTES);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          tma_load_2d(smem_u32(sQ + i * QTILE_BYTES + c * QHALF_BYTES), &tm_q, bar_q,
                      (h0 + i) * HD + c * 64, qt * BQ);
          tma_load_2d(smem_u32(sdO + i * QTILE_BYTES + c * QHALF_BYTES), &tm_do, bar_q,
                      (h0 + i) * HD + c * 64, qt * BQ);
        }
      for (int u = 0; u < U; ++u) {
        const int s = u & 1;
        const uint32_t ph = (u >> 1) & 1;
        const int krow = (list[u >> 1] >> 1) * 128 + (u & 1) * SUB;
        if (!mbar_wait(bar_kempty + 8 * s, ph ^ 1, KID, 10)) break;
        mbar_expect_tx(bar_kfull + 8 * s, KSUB_BYTES);
#pragma unroll
        for (int c = 0; c < 2; ++c)
          tma_load_2d(smem_u32(sK + s * KSUB_BYTES + c * KHALF_BYTES), &tm_k, bar_kfull + 8 * s,
                      kvh * HD + c * 64, krow);
        if (!mbar_wait(bar_vempty + 8 * s, ph ^ 1, KID, 11)) break;
        mbar_expect_tx(bar_vfull + 8 * s, KSUB_BYTES);
#pragma unroll
        for (int c = 0; c < 2; ++c)
          tma_load_2d(smem_u32(sV + s * KSUB_BYTES + c * KHALF_BYTES), &tm_v, bar_vfull + 8 * s,
                      kvh * HD + c * 64, krow);
      }
    }
  } else if (warp == 9) {
    // whole warp, identical values; one elected lane issues (keeps descriptors in uniform registers)
    if (n > 0) {
      const bool leader = elect_one();
      const uint32_t idesc_s = make_idesc_bf16(BQ, SUB, 0, 0);   // [128 q] x [64 keys], K = d
      const uint32_t idesc_dq = make_idesc_bf16(BQ, HD, 0, 1);   // [128 q] x [128 d],  K = keys
      auto issue_s_dp = [&](int i, int s) {
        const uint32_t qa = smem_u32(sQ + i * QTILE_BYTES);
        const uint32_t da = smem_u32(sdO + i * QTILE_BYTES);
        const uint32_t ka = smem_u32(sK + s * KSUB_BYTES);
        const uint32_t va = smem_u32(sV + s * KSUB_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t qoff = (k >> 2) * QHALF_BYTES + (k & 3) * 32;
          const uint32_t koff = (k >> 2) * KHALF_BYTES + (k & 3) * 32;
          {
            const uint64_t ad_ = make_smem_desc_sw128(qa + qoff, 16, 1024);
            const uint64_t bd_ = make_smem_desc_sw128(ka + koff, 16, 1024);
            if (leader) tc_mma_ss(tmem_base + i * 128, ad_, bd_, idesc_s, k ? 1u : 0u);
          }
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t qoff = (k >> 2) * QHALF_BYTES + (k & 3) * 32;
          const uint32_t koff = (k >> 2) * KHALF_BYTES + (k & 3) * 32;
          {
            const uint64_t ad_ = make_smem_desc_sw128(da + qoff, 16, 1024);
            const uint64_t bd_ = make_smem_desc_sw128(va + koff, 16, 1024);
            if (leader) tc_mma_ss(tmem_base + i * 128 + 64, ad_, bd_, idesc_s, k ? 1u : 0u);
          }
        }
        if (leader) tc_commit(bar_sfull + 8 * i);
      };
      bool ok = __all_sync(0xffffffffu, mbar_wait(bar_q, 0, KID, 20)) && __all_sync(0xffffffffu, mbar_wait(bar_kfull, 0, KID, 21)) &&
                __all_sync(0xffffffffu, mbar_wait(bar_vfull, 0, KID, 22));
      if (ok) {
        tc_fence_after();
        issue_s_dp(0, 0);
        issue_s_dp(1, 0);
        if (leader) tc_commit(bar_vempty);
      }
      for (int u = 0; u < U && ok; ++u) {
        const int s = u & 1;
        const uint32_t ka = smem_u32(sK + s * KSUB_BYTES);
        for (int i = 0; i < 2; ++i) {
          if (!__all_sync(0xffffffffu, mbar_wait(bar_pfull + 8 * i, u & 1, KID, 23))) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < SUB / 16; ++k)
            {
              const uint64_t bd_ = make_smem_desc_sw128(ka + k * 2048, KHALF_BYTES, 1024);
              if (leader) tc_mma_ts(tmem_base + 256 + i * 128, tmem_base + i * 128 + k * 8, bd_, idesc_dq,
                      (u | k) ? 1u : 0u);
            }
          if (leader && u + 1 == U) tc_commit(bar_odone + 8 * i);
          if (leader && i == 1) tc_commit(bar_kempty + 8 * s);
          if (u + 1 < U) {
            const int s1 = (u + 1) & 1;
            if (i == 0) {
              const uint32_t ph1 = ((u + 1) >> 1) & 1;
              if (!__all_sync(0xffffffffu, mbar_wait(bar_kfull + 8 * s1, ph1, KID, 24)) ||
                  !__all_sync(0xffffffffu, mbar_wait(bar_vfull + 8 * s1, ph1, KID, 25))) { ok = false; break; }
              tc_fence_after();
            }
            issue_s_dp(i, s1);
            if (leader && i == 1) tc_commit(bar_vempty + 8 * s1);
          }
        }
      }
      __syncwarp();
    }
  } else {
    const int i = warp >> 2;
    const int qd = warp & 3;
    const int row = qd * 32 + lane;
    const int grow = qt * BQ + row;
    const int lo = p.q_lo[grow], hi = p.q_hi[grow], grp = p.q_grp[grow];
    const float lse2 = p.lse2[(size_t)(h0 + i) * p.nq_pad + grow];
    const float delta = p.delta[(size_t)(h0 + i) * p.nq_pad + grow];
    const uint32_t t_s = tmem_base + ((uint32_t)(qd * 32) << 16) + i * 128;
    const uint32_t t_dq = tmem_base + ((uint32_t)(qd * 32) << 16) + 256 + i * 128;
    uint32_t rs[64], rp[64];
    bool ok = true;
    for (int u = 0; u < U; ++u) {
      const int ent = list[u >> 1];
      const int* kc = p.k_code + (ent >> 1) * 128 + (u & 1) * SUB;
      if (!mbar_wait(bar_sfull + 8 * i, u & 1, KID, 30)) { ok = false; break; }
      tc_fence_after();
      tmem_ld32(t_s, rs);
      tmem_ld32(t_s + 32, rs + 32);
      tmem_ld32(t_s + 64, rp);
      tmem_ld32(t_s + 96, rp + 32);
      tmem_ld_wait();
      uint32_t pk[32];
      if (ent & 1) {
#pragma unroll
        for (int e = 0; e < 64; e += 2) {
          float p0 = fast_exp2(fmaf(__uint_as_float(rs[e]), p.scale_log2, lse2));
          float p1 = fast_exp2(fmaf(__uint_as_float(rs[e + 1]), p.scale_log2, lse2));
          if (!key_visible(__ldg(kc + e), lo, hi, grp)) p0 = 0.f;
          if (!key_visible(__ldg(kc + e + 1), lo, hi, grp)) p1 = 0.f;
          pk[e >> 1] = pack_bf16x2(p0 * fmaf(__uint_as_float(rp[e]), p.scale, delta),
                                   p1 * fmaf(__uint_as_float(rp[e + 1]), p.scale, delta));
        }
      } else {
#pragma unroll
        for (int e = 0; e < 64; e += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(rs[e]), p.scale_log2, lse2));
          const float p1 = fast_exp2(fmaf(__uint_as_float(rs[e + 1]), p.scale_log2, lse2));
          pk[e >> 1] = pack_bf16x2(p0 * fmaf(__uint_as_float(rp[e]), p.scale, delta),
                                   p1 * fmaf(__uint_as_float(rp[e + 1]), p.scale, delta));
        }
      }
      tmem_st16(t_s, pk);
      tmem_st16(t_s + 16, pk + 16);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar_pfull + 8 * i);
    }
    if (ok && n > 0) ok = mbar_wait(bar_odone + 8 * i, 0, KID, 31);
    if (ok) {
      tc_fence_after();
      uint8_t* st = sQ + i * QTILE_BYTES;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        if (n > 0) {
          tmem_ld32(t_dq + c * 32, rs);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) rs[e] = 0u;
        }
        uint8_t* half = st + (c >> 1) * QHALF_BYTES;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint32_t a[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            a[e] = pack_bf16x2(__uint_as_float(rs[8 * v + 2 * e]), __uint_as_float(rs[8 * v + 2 * e + 1]));
          *reinterpret_cast<uint4*>(half + sw128_offset(row, (c & 1) * 4 + v)) =
              make_uint4(a[0], a[1], a[2], a[3]);
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(bar_epi + 8 * i);
      if (row == 0) {
        if (mbar_wait(bar_epi + 8 * i, 0, KID, 32)) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
            tma_store_2d(&tm_dq, smem_u32(st + c * QHALF_BYTES), (h0 + i) * HD + c * 64, qt * BQ);
          tma_store_commit();
          tma_store_wait_all();
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (error_is_set()) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 9) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// Per (row, head), both NEGATED so that the consumers need one fused multiply-add each:
// delta_s = −scale · sum_d dO·O and lse2 = −lse·log2(e), with lse2 = −inf for rows that saw no key
// (and for padding rows) so that exp2(x + lse2) is exactly 0 there.
// One warp per (row, head). Output layout: delta_s [Hq, nq_pad], lse2 [Hq, nq_pad].
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o,
                                  const __nv_bfloat16* __restrict__ dout,
                                  const float* __restrict__ lse, float* __restrict__ delta,
                                  float* __restrict__ lse2, float scale,
                                  int nq, int nq_pad, int Hq, long long ldo, long long lddo) {
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)nq_pad * Hq) return;
  const int row = (int)(item / Hq), h = (int)(item % Hq);
  float s = 0.f;
  if (row < nq) {
    const uint2 a = *reinterpret_cast<const uint2*>(o + (size_t)row * ldo + h * HD + lane * 4);
    const uint2 b = *reinterpret_cast<const uint2*>(dout + (size_t)row * lddo + h * HD + lane * 4);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const float2 x = __bfloat1622float2(a2[e]), y = __bfloat1622float2(b2[e]);
      s += x.x * y.x + x.y * y.y;
    }
  }
  s = warp_sum(s);
  if (lane == 0) {
    const size_t at = (size_t)h * nq_pad + row;
    const float l = lse[at];
    delta[at] = -s * scale;
    lse2[at] = (row < nq && l > -INFINITY) ? -l * 1.4426950408889634f : -INFINITY;
  }
}

}  // namespace attn_dq
}  // namespace tdllm
