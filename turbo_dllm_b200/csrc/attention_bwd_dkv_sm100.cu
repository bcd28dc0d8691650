// Block-diffusion attention backward, key/value gradients (sm_100a, head_dim 128).
//
// One CTA owns one 128-row key tile of one KV head and walks every (query head of the
// group, visible query tile) pair, so the GQA sum over query heads happens in TMEM and
// dK/dV are written once, without atomics. Everything is computed transposed (keys on
// the TMEM lanes):
//   Sᵀ  = K·Qᵀ   (128 keys x 64 queries)      dPᵀ = V·dOᵀ
//   Pᵀ  = exp(Sᵀ·scale − lse[q])              dSᵀ = Pᵀ∘(dPᵀ − delta[q])·scale
//   dV += Pᵀ·dO                               dK += dSᵀ·Q
// Query tiles are consumed in 64-row halves, half b handled by warp group b, so the
// exponentials of one half overlap the tensor-core work of the other. Pᵀ and dSᵀ are
// written to TMEM as bf16 over the columns they were read from and used as the A operand;
// dO and Q tiles in shared memory serve both as K-major B operands (first two products)
// and as MN-major B operands (last two) — same bytes, two descriptors.
//
// Reference counterpart: dK/dV half of the masked FlashAttention backward
// (third_party/flash-attention/hopper/mainloop_bwd_sm90_tma_gmma_ws.hpp, FA4
// flash_bwd_sm100.py) and the owner-major clean dK/dV buffers of
// dllm_parallel/core/attention/context_parallel_attention.py:820-885.
#include "common.cuh"
#include "api.h"

namespace tdllm {
namespace attn_dkv {

constexpr int KID = 4;
constexpr int HD = 128;
constexpr int TILE_BYTES = 128 * HD * 2;  // 32 KiB
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int THREADS = 320;
constexpr int ROWSTAT_BYTES = 2 * 2 * 128 * 4;  // 2 stages x (lse2[128], delta_s[128])
constexpr int SMEM_BYTES = 6 * TILE_BYTES + 512 + ROWSTAT_BYTES + 1024;

struct Params {
  int nq_pad, Hq, Hkv;
  const int* q_lo;
  const int* q_hi;
  const int* q_grp;
  const int* k_code;
  const int* tile_ptr;  // per key tile: query tiles that see it
  const int* tile_idx;  // q_tile * 2 + needs_mask
  const int* order;     // key tiles, heaviest first
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
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                    const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                    const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                    const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE_BYTES;
  uint8_t* sQ = sV + TILE_BYTES;        // 2 stages
  uint8_t* sdO = sQ + 2 * TILE_BYTES;   // 2 stages
  uint64_t* bars = (uint64_t*)(sdO + 2 * TILE_BYTES);
  const uint32_t b0 = smem_u32(bars);
  const uint32_t bar_kv = b0;
  const uint32_t bar_qfull = b0 + 8, bar_qempty = b0 + 24;
  const uint32_t bar_sfull = b0 + 40, bar_pfull = b0 + 56;
  const uint32_t bar_done = b0 + 72;
  const uint32_t bar_epi = b0 + 80;  // [2]
  uint32_t* tmem_slot = (uint32_t*)(bars + 13);
  float* sStat = (float*)((uint8_t*)bars + 512);  // [stage][lse2 128 | delta_s 128]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  const int kvh = blockIdx.x % p.Hkv;
  const int kt = p.order[blockIdx.x / p.Hkv];
  const int list_begin = p.tile_ptr[kt];
  const int n = p.tile_ptr[kt + 1] - list_begin;
  const int* list = p.tile_idx + list_begin;
  const int items = G * n;   // (query head, query tile) pairs
  const int U = 2 * items;   // 64-query halves

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_qfull + 8 * s, 1);
      mbar_init(bar_qempty + 8 * s, 1);
      mbar_init(bar_sfull + 8 * s, 1);
      mbar_init(bar_pfull + 8 * s, 128);
      mbar_init(bar_epi + 8 * s, 128);
    }
    mbar_init(bar_done, 1);
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
  // columns: ST_b at b*128, dPT_b at b*128+64 (b = half), dV at 256, dK at 384

  if (warp == 8) {
    if (lane == 0 && items > 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_do);
      mbar_expect_tx(bar_kv, 2 * TILE_BYTES);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        tma_load_2d(smem_u32(sK + c * HALF_BYTES), &tm_k, bar_kv, kvh * HD + c * 64, kt * 128);
        tma_load_2d(smem_u32(sV + c * HALF_BYTES), &tm_v, bar_kv, kvh * HD + c * 64, kt * 128);
      }
      for (int it = 0; it < items; ++it) {
        const int s = it & 1;
        const int h = kvh * G + it / n;
        const int qt = list[it % n] >> 1;
        if (!mbar_wait(bar_qempty + 8 * s, ((it >> 1) & 1) ^ 1, KID, 10)) break;
        mbar_expect_tx(bar_qfull + 8 * s, 2 * TILE_BYTES + 1024);
        bulk_load_1d(smem_u32(sStat + s * 256), p.lse2 + (size_t)h * p.nq_pad + qt * 128, 512,
                     bar_qfull + 8 * s);
        bulk_load_1d(smem_u32(sStat + s * 256 + 128), p.delta + (size_t)h * p.nq_pad + qt * 128, 512,
                     bar_qfull + 8 * s);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          tma_load_2d(smem_u32(sQ + s * TILE_BYTES + c * HALF_BYTES), &tm_q, bar_qfull + 8 * s,
                      h * HD + c * 64, qt * 128);
          tma_load_2d(smem_u32(sdO + s * TILE_BYTES + c * HALF_BYTES), &tm_do, bar_qfull + 8 * s,
                      h * HD + c * 64, qt * 128);
        }
      }
    }
  } else if (warp == 9) {
    // whole warp, identical values; one elected lane issues (keeps descriptors in uniform registers)
    if (items > 0) {
      const bool leader = elect_one();
      const uint32_t idesc_st = make_idesc_bf16(128, 64, 0, 0);    // [128 keys] x [64 q], K = d
      const uint32_t idesc_acc = make_idesc_bf16(128, HD, 0, 1);   // [128 keys] x [128 d], K = q
      const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
      // half-tile u: item u>>1, query rows 64*(u&1).. of that item's tile
      auto issue_st = [&](int u) {
        const int s = (u >> 1) & 1, b = u & 1;
        const uint32_t qa = smem_u32(sQ + s * TILE_BYTES) + b * 64 * 128;
        const uint32_t da = smem_u32(sdO + s * TILE_BYTES) + b * 64 * 128;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
          {
            const uint64_t ad_ = make_smem_desc_sw128(ka + off, 16, 1024);
            const uint64_t bd_ = make_smem_desc_sw128(qa + off, 16, 1024);
            if (leader) tc_mma_ss(tmem_base + b * 128, ad_, bd_, idesc_st, k ? 1u : 0u);
          }
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
          {
            const uint64_t ad_ = make_smem_desc_sw128(va + off, 16, 1024);
            const uint64_t bd_ = make_smem_desc_sw128(da + off, 16, 1024);
            if (leader) tc_mma_ss(tmem_base + b * 128 + 64, ad_, bd_, idesc_st, k ? 1u : 0u);
          }
        }
        if (leader) tc_commit(bar_sfull + 8 * b);
      };
      bool ok = __all_sync(0xffffffffu, mbar_wait(bar_kv, 0, KID, 20)) && __all_sync(0xffffffffu, mbar_wait(bar_qfull, 0, KID, 21));
      if (ok) {
        tc_fence_after();
        issue_st(0);
        issue_st(1);
      }
      for (int u = 0; u < U && ok; ++u) {
        const int s = (u >> 1) & 1, b = u & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(bar_pfull + 8 * b, (u >> 1) & 1, KID, 22))) break;
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ + s * TILE_BYTES) + b * 64 * 128;
        const uint32_t da = smem_u32(sdO + s * TILE_BYTES) + b * 64 * 128;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          {
            const uint64_t bd_ = make_smem_desc_sw128(da + k * 2048, HALF_BYTES, 1024);
            if (leader) tc_mma_ts(tmem_base + 256, tmem_base + b * 128 + k * 8, bd_, idesc_acc,
                    (u | k) ? 1u : 0u);
          }
#pragma unroll
        for (int k = 0; k < 4; ++k)
          {
            const uint64_t bd_ = make_smem_desc_sw128(qa + k * 2048, HALF_BYTES, 1024);
            if (leader) tc_mma_ts(tmem_base + 384, tmem_base + b * 128 + 64 + k * 8, bd_, idesc_acc,
                    (u | k) ? 1u : 0u);
          }
        if (leader && b == 1) tc_commit(bar_qempty + 8 * s);
        if (leader && u + 1 == U) tc_commit(bar_done);
        if (u + 2 < U) {
          if (b == 0) {
            const int it1 = (u + 2) >> 1;
            if (!__all_sync(0xffffffffu, mbar_wait(bar_qfull + 8 * (it1 & 1), (it1 >> 1) & 1, KID, 23))) break;
            tc_fence_after();
          }
          issue_st(u + 2);
        }
      }
      __syncwarp();
    }
  } else {
    const int b = warp >> 2;   // which 64-query half this group handles
    const int qd = warp & 3;
    const int row = qd * 32 + lane;   // key row inside the tile
    const int kcode = p.k_code[kt * 128 + row];
    const uint32_t t_s = tmem_base + ((uint32_t)(qd * 32) << 16) + b * 128;
    uint32_t rs[64], rp[64];
    bool ok = true;
    for (int it = 0; it < items; ++it) {
      const int ent = list[it % n];
      const int qrow0 = (ent >> 1) * 128 + b * 64;
      const float* sl = sStat + (it & 1) * 256 + b * 64;   // lse2 of this half's 64 queries
      const float* sd = sl + 128;                          // delta_s
      if (!mbar_wait(bar_sfull + 8 * b, it & 1, KID, 30)) { ok = false; break; }
      tc_fence_after();
      tmem_ld32(t_s, rs);
      tmem_ld32(t_s + 32, rs + 32);
      tmem_ld32(t_s + 64, rp);
      tmem_ld32(t_s + 96, rp + 32);
      tmem_ld_wait();
      uint32_t pk[32], dk[32];
      if (ent & 1) {
#pragma unroll
        for (int e = 0; e < 64; e += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(sl + e);
          const float4 d4 = *reinterpret_cast<const float4*>(sd + e);
          const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
          const float dv[4] = {d4.x, d4.y, d4.z, d4.w};
          float pv[4], ds[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const int g = qrow0 + e + t;
            float pr = fast_exp2(fmaf(__uint_as_float(rs[e + t]), p.scale_log2, lv[t]));
            if (!key_visible(kcode, __ldg(p.q_lo + g), __ldg(p.q_hi + g), __ldg(p.q_grp + g))) pr = 0.f;
            pv[t] = pr;
            ds[t] = pr * fmaf(__uint_as_float(rp[e + t]), p.scale, dv[t]);
          }
          pk[e >> 1] = pack_bf16x2(pv[0], pv[1]);
          pk[(e >> 1) + 1] = pack_bf16x2(pv[2], pv[3]);
          dk[e >> 1] = pack_bf16x2(ds[0], ds[1]);
          dk[(e >> 1) + 1] = pack_bf16x2(ds[2], ds[3]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 64; e += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(sl + e);
          const float4 d4 = *reinterpret_cast<const float4*>(sd + e);
          const float p0 = fast_exp2(fmaf(__uint_as_float(rs[e]), p.scale_log2, l4.x));
          const float p1 = fast_exp2(fmaf(__uint_as_float(rs[e + 1]), p.scale_log2, l4.y));
          const float p2 = fast_exp2(fmaf(__uint_as_float(rs[e + 2]), p.scale_log2, l4.z));
          const float p3 = fast_exp2(fmaf(__uint_as_float(rs[e + 3]), p.scale_log2, l4.w));
          pk[e >> 1] = pack_bf16x2(p0, p1);
          pk[(e >> 1) + 1] = pack_bf16x2(p2, p3);
          dk[e >> 1] = pack_bf16x2(p0 * fmaf(__uint_as_float(rp[e]), p.scale, d4.x),
                                   p1 * fmaf(__uint_as_float(rp[e + 1]), p.scale, d4.y));
          dk[(e >> 1) + 1] = pack_bf16x2(p2 * fmaf(__uint_as_float(rp[e + 2]), p.scale, d4.z),
                                         p3 * fmaf(__uint_as_float(rp[e + 3]), p.scale, d4.w));
        }
      }
      tmem_st16(t_s, pk);
      tmem_st16(t_s + 16, pk + 16);
      tmem_st16(t_s + 64, dk);
      tmem_st16(t_s + 80, dk + 16);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar_pfull + 8 * b);
    }
    // epilogue: group 0 stores dV, group 1 stores dK
    if (ok && items > 0) ok = mbar_wait(bar_done, 0, KID, 31);
    if (ok) {
      tc_fence_after();
      const uint32_t t_acc = tmem_base + ((uint32_t)(qd * 32) << 16) + 256 + b * 128;
      uint8_t* st = sQ + b * TILE_BYTES;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        if (items > 0) {
          tmem_ld32(t_acc + c * 32, rs);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) rs[e] = 0u;
        }
        uint8_t* half = st + (c >> 1) * HALF_BYTES;
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
      mbar_arrive(bar_epi + 8 * b);
      if (row == 0) {
        if (mbar_wait(bar_epi + 8 * b, 0, KID, 32)) {
          const CUtensorMap* tm = b ? &tm_dk : &tm_dv;
#pragma unroll
          for (int c = 0; c < 2; ++c)
            tma_store_2d(tm, smem_u32(st + c * HALF_BYTES), kvh * HD + c * 64, kt * 128);
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

}  // namespace attn_dkv
}  // namespace tdllm
