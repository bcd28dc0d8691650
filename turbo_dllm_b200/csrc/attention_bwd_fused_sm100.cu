// Block-diffusion attention backward in one pass (sm_100a, head_dim 128): dK, dV and dQ.
//
// One CTA owns one 128-row key tile of one KV head and walks every (query head of the
// group, visible query tile) pair in units of 64 queries. Everything is computed transposed
// (keys on the TMEM lanes):
//   Sᵀ  = K·Qᵀ   (128 keys x 64 queries)      dPᵀ = V·dOᵀ
//   Pᵀ  = exp(Sᵀ·scale − lse[q])              dSᵀ = Pᵀ∘(dPᵀ − delta[q])·scale   (packed fp32x2 arithmetic)
//   dV += Pᵀ·dO        dK += dSᵀ·Q            dQᵀ = Kᵀ·dSᵀ   (128 d x 64 queries)
// Five tensor-core products per tile pair: the score and dP tiles are computed once and
// feed all three gradients (separate dQ and dK/dV kernels need seven). dK/dV accumulate in
// TMEM over the whole walk (the GQA sum over query heads included) and are stored once.
// dQᵀ of one unit is a partial sum over this key tile only: it is read back from TMEM, staged
// in shared memory as [query][d] fp32 and added to an fp32 accumulator in global memory by
// TMA reduce-add copies (16 query rows of 512 bytes per copy). A small kernel afterwards
// casts the accumulator to bf16.
//
// The walk of a key tile is cut into chunks of consecutive query tiles and the grid runs chunk by
// chunk (all key tiles of chunk 0, then chunk 1, ...): the rows of the dQ accumulator that a chunk
// touches then stay in L2 while every key tile adds to them, instead of going to DRAM and back once
// per wave of CTAs. The price: dK/dV of a CTA are partial sums too, added to fp32 accumulators by the
// same kind of copy when the CTA ends (128 KiB per CTA against 32 KiB per 64-query unit for dQ).
//
// Warps: 0-15 do the element-wise work as four groups of four (unit parity b = warp/8, 32 of the
// unit's 64 queries each), warp 16 issues TMA loads, warp 17 issues the MMAs. Units alternate
// between two TMEM slots, so the exponentials of one unit overlap the products of the other.
//
// TMEM, per slot b at column 128·b: [0,64) Sᵀ fp32, rewritten in place as bf16 (per 32-query group:
// Pᵀ in 16 columns, dSᵀ in the next 16; A operands of the dV and dK products); [64,128) dPᵀ fp32,
// reused as the dQᵀ accumulator once its values are in registers. dV at 256, dK at 384. dSᵀ also
// goes to shared memory as bf16 (one 128-byte swizzled row of 64 queries per key): the B operand
// of the dQᵀ product, whose A operand is the K tile read MN-major (same bytes as the Sᵀ product).
//
// Context-sharded form (template argument CSBP): key tiles [0, nlt) are this rank's own rows, key tiles from
// nlt on are clean rows of the other ranks of the context-parallel group (their K|V were brought into
// kv_rem by the forward kernel). The dK/dV partial sums of a remote key tile never touch this GPU's memory:
// the epilogue adds them, fp32, straight into the owner's accumulator through peer memory (vector
// red.add over NVLink, one 16-byte packet per four values), while later work items of the grid are still in
// their products. The owner casts its accumulator once every rank has passed the barrier that follows the
// kernel. Replaces the clean-gradient reduce-scatter of
// dllm_parallel/core/attention/context_parallel_attention.py:760-885 and its overlap with the local
// backward (:2292-2312).
//
// Reference counterpart: the masked FlashAttention backward
// (third_party/flash-attention/hopper/mainloop_bwd_sm90_tma_gmma_ws.hpp, FA4
// flash_bwd_sm100.py: five products, dQ by reduce-add) and the owner-major clean dK/dV
// buffers of dllm_parallel/core/attention/context_parallel_attention.py:820-885.
#include "common.cuh"
#include "api.h"

namespace tdllm {
namespace attn_fused {

constexpr int KID = 5;
constexpr int HD = 128;
constexpr int KV_TILE_BYTES = 128 * HD * 2;   // 32 KiB: 128 keys, two 64-column halves
constexpr int KV_HALF_BYTES = KV_TILE_BYTES / 2;
constexpr int QS_BYTES = 64 * HD * 2;         // 16 KiB: 64 queries of Q (or dO), two 64-column halves
constexpr int QS_HALF_BYTES = QS_BYTES / 2;
constexpr int STAGES = 3;
constexpr int DS_BYTES = 128 * 64 * 2;        // 16 KiB: dSᵀ of one unit, [128 keys][64 queries] bf16
constexpr int RED_BYTES = 16 * HD * 4;        // 8 KiB per group: 16 query rows of dQ, fp32
constexpr int THREADS = 576;
constexpr int OFF_Q = 2 * KV_TILE_BYTES;
constexpr int OFF_DO = OFF_Q + STAGES * QS_BYTES;
constexpr int OFF_DS = OFF_DO + STAGES * QS_BYTES;
constexpr int OFF_RED = OFF_DS + 2 * DS_BYTES;
constexpr int OFF_BARS = OFF_RED + 4 * RED_BYTES;
constexpr int OFF_STAT = OFF_BARS + 512;      // [stage][lse2 64 | delta_s 64] fp32
// no alignment slack: the kernel checks that its dynamic shared memory starts 1 KiB aligned
constexpr int SMEM_BYTES = OFF_STAT + STAGES * 128 * 4;
static_assert(SMEM_BYTES <= 232448, "shared memory budget of one CTA");
static_assert(OFF_Q + 2 * 65536 <= OFF_RED, "dK/dV staging must not reach the dQ staging rows");

constexpr int MAX_PEERS = 16;
// Where the gradients of remote key rows go: segment s = the rows of one peer, in the order of the forward
// pull (rank+1, rank+2, ...).
struct PushPlan {
  float* dk[MAX_PEERS];               // segment s: the owner's dK accumulator [rows][Hkv*128] fp32 (peer memory)
  float* dv[MAX_PEERS];
  long long seg_begin[MAX_PEERS + 1]; // first remote row of segment s
  long long dst_row0[MAX_PEERS];      // row of the owner's accumulator that takes the segment's first row
  long long n_rows;                   // remote rows
  int nseg, nlt;
};

struct Params {
  int nq_pad, Hq, Hkv;
  const int* q_lo;
  const int* q_hi;
  const int* q_grp;
  const int* k_code;
  int nkt;              // key tiles
  const int* tile_ptr;  // per work item (chunk * nkt + key tile): the chunk's query tiles that see the key tile
  const int* tile_idx;  // q_tile * 2 + needs_mask
  const int* order;     // non-empty work items: chunk by chunk, heaviest first inside a chunk
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
__device__ __forceinline__ void red_add_peer_f32x4(float* dst, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__uint_as_float(a)),
               "f"(__uint_as_float(b)), "f"(__uint_as_float(c)), "f"(__uint_as_float(d))
               : "memory");
}

template <bool CSBP>
__global__ void __launch_bounds__(THREADS, 1)
attn_bwd_fused_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                      const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const __grid_constant__ CUtensorMap tm_dkacc, const __grid_constant__ CUtensorMap tm_dvacc,
                      const __grid_constant__ CUtensorMap tm_dqacc, const __grid_constant__ CUtensorMap tm_kr,
                      const __grid_constant__ CUtensorMap tm_vr, const Params p,
                      const __grid_constant__ PushPlan pp) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {   // swizzled tiles need 1 KiB alignment; nothing has been set up yet
    if (threadIdx.x == 0) set_error(ERR_BAD_INDEX, KID, 1);
    return;
  }
  uint8_t* sK = smem;
  uint8_t* sV = sK + KV_TILE_BYTES;
  uint8_t* sQ = smem + OFF_Q;     // [stage]
  uint8_t* sdO = smem + OFF_DO;   // [stage]
  uint8_t* sdS = smem + OFF_DS;   // [slot]
  uint8_t* sRed = smem + OFF_RED; // [group]
  uint64_t* bars = (uint64_t*)(smem + OFF_BARS);
  float* sStat = (float*)(smem + OFF_STAT);
  const uint32_t b0 = smem_u32(bars);
  const uint32_t bar_kv = b0;
  const uint32_t bar_qfull = b0 + 8, bar_qempty = b0 + 32;            // [3] each
  const uint32_t bar_sfull = b0 + 56, bar_pfull = b0 + 72;            // [2] each
  const uint32_t bar_dqfull = b0 + 88, bar_dqread = b0 + 104;         // [2] each
  const uint32_t bar_done = b0 + 120;
  const uint32_t bar_epi = b0 + 128;                                  // [2]
  uint32_t* tmem_slot = (uint32_t*)(bars + 20);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  const int kvh = blockIdx.x % p.Hkv;
  const int work = p.order[blockIdx.x / p.Hkv];
  const int kt = work % p.nkt;
  const int list_begin = p.tile_ptr[work];
  const int n = p.tile_ptr[work + 1] - list_begin;
  const int* list = p.tile_idx + list_begin;
  const int items = G * n;   // (query head, query tile) pairs
  const int U = 2 * items;   // 64-query units

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_qfull + 8 * s, 1);
      mbar_init(bar_qempty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_sfull + 8 * s, 1);
      mbar_init(bar_pfull + 8 * s, 256);
      mbar_init(bar_dqfull + 8 * s, 1);
      mbar_init(bar_dqread + 8 * s, 256);
      mbar_init(bar_epi + 8 * s, 256);
    }
    mbar_init(bar_done, 1);
    fence_mbar_init();
  }
  if (warp == 17) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // columns: ST_b at b*128, dPT_b / dQT_b at b*128+64 (b = unit parity), dV at 256, dK at 384

  if (warp == 16) {
    if (lane == 0 && items > 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_do);
      mbar_expect_tx(bar_kv, 2 * KV_TILE_BYTES);
      const bool remote = CSBP && kt >= pp.nlt;
      const CUtensorMap* mk = remote ? &tm_kr : &tm_k;
      const CUtensorMap* mv = remote ? &tm_vr : &tm_v;
      const int krow = (remote ? kt - pp.nlt : kt) * 128;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        tma_load_2d(smem_u32(sK + c * KV_HALF_BYTES), mk, bar_kv, kvh * HD + c * 64, krow);
        tma_load_2d(smem_u32(sV + c * KV_HALF_BYTES), mv, bar_kv, kvh * HD + c * 64, krow);
      }
      int st = 0;
      uint32_t ph = 0;
      for (int u = 0; u < U; ++u) {
        const int it = u >> 1, b = u & 1;
        const int h = kvh * G + it / n;
        const int qrow = (list[it % n] >> 1) * 128 + b * 64;
        if (!mbar_wait_spin(bar_qempty + 8 * st, ph ^ 1, KID, 10)) break;
        mbar_expect_tx(bar_qfull + 8 * st, 2 * QS_BYTES + 512);
        bulk_load_1d(smem_u32(sStat + st * 128), p.lse2 + (size_t)h * p.nq_pad + qrow, 256,
                     bar_qfull + 8 * st);
        bulk_load_1d(smem_u32(sStat + st * 128 + 64), p.delta + (size_t)h * p.nq_pad + qrow, 256,
                     bar_qfull + 8 * st);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          tma_load_2d(smem_u32(sQ + st * QS_BYTES + c * QS_HALF_BYTES), &tm_q, bar_qfull + 8 * st,
                      h * HD + c * 64, qrow);
          tma_load_2d(smem_u32(sdO + st * QS_BYTES + c * QS_HALF_BYTES), &tm_do, bar_qfull + 8 * st,
                      h * HD + c * 64, qrow);
        }
        if (++st == STAGES) {
          st = 0;
          ph ^= 1;
        }
      }
    }
  } else if (warp == 17) {
    // The whole warp runs this loop with identical values and one elected lane issues: descriptors
    // then live in uniform registers. Issuing from a divergent `lane == 0` branch costs about 130
    // cycles per MMA on the issuing thread (measured), more than these small MMAs take to execute.
    if (items > 0) {
      const bool leader = elect_one();
      const uint32_t idesc_st = make_idesc_bf16(128, 64, 0, 0);    // [128 keys] x [64 q], K = d
      const uint32_t idesc_acc = make_idesc_bf16(128, HD, 0, 1);   // [128 keys] x [128 d], K = q
      const uint32_t idesc_dq = make_idesc_bf16(HD, 64, 1, 1);     // [128 d] x [64 q], K = keys
      const uint32_t ka = smem_u32(sK), va = smem_u32(sV), sa = smem_u32(sdS);
      auto wait_all = [&](uint32_t bar, uint32_t parity, int detail) {
        return __all_sync(0xffffffffu, mbar_wait_spin(bar, parity, KID, detail));
      };
      // unit u lives in stage u % 3 and TMEM slot u & 1
      auto issue_s = [&](int b, int st) {
        const uint32_t qa = smem_u32(sQ + st * QS_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t ad = make_smem_desc_sw128(ka + (k >> 2) * KV_HALF_BYTES + (k & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(qa + (k >> 2) * QS_HALF_BYTES + (k & 3) * 32, 16, 1024);
          if (leader) tc_mma_ss(tmem_base + b * 128, ad, bd, idesc_st, k ? 1u : 0u);
        }
      };
      // dPᵀ overwrites the columns that held the previous dQᵀ of this slot: issue only after the
      // slot's warp groups have read that dQᵀ back. Completes the pair (Sᵀ, dPᵀ) of a unit.
      auto issue_dp = [&](int b, int st) {
        const uint32_t da = smem_u32(sdO + st * QS_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t ad = make_smem_desc_sw128(va + (k >> 2) * KV_HALF_BYTES + (k & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(da + (k >> 2) * QS_HALF_BYTES + (k & 3) * 32, 16, 1024);
          if (leader) tc_mma_ss(tmem_base + b * 128 + 64, ad, bd, idesc_st, k ? 1u : 0u);
        }
        if (leader) tc_commit(bar_sfull + 8 * b);
      };
      bool ok = wait_all(bar_kv, 0, 20) && wait_all(bar_qfull, 0, 21);
      if (ok) {
        tc_fence_after();
        issue_s(0, 0);
        issue_dp(0, 0);
        ok = wait_all(bar_qfull + 8, 0, 21);   // U >= 2 always
      }
      if (ok) {
        tc_fence_after();
        issue_s(1, 1);
        issue_dp(1, 1);
      }
      int st = 0;            // stage of unit u
      int st2 = 2;           // stage of unit u + 2
      uint32_t ph2 = 0;      // phase of that stage's "full" barrier for unit u + 2
      for (int u = 0; u < U && ok; ++u) {
        const int b = u & 1;
        if (!wait_all(bar_pfull + 8 * b, (u >> 1) & 1, 22)) break;
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ + st * QS_BYTES);
        const uint32_t da = smem_u32(sdO + st * QS_BYTES);
        // dQᵀ first: its read-back by the warp groups then overlaps the dV and dK products, and
        // the next dPᵀ of this slot (which reuses the columns) can follow in the same round
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t ad = make_smem_desc_sw128(ka + k * 2048, KV_HALF_BYTES, 1024);
          const uint64_t bd = make_smem_desc_sw128(sa + b * DS_BYTES + k * 2048, DS_BYTES, 1024);
          if (leader) tc_mma_ss(tmem_base + b * 128 + 64, ad, bd, idesc_dq, k ? 1u : 0u);
        }
        if (leader) tc_commit(bar_dqfull + 8 * b);
        // A operands in TMEM: queries 16k..16k+15 of the unit sit in 8 columns; the two 32-query
        // groups of a unit each own 32 columns (Pᵀ in the first 16, dSᵀ in the last 16)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t bd = make_smem_desc_sw128(da + k * 2048, QS_HALF_BYTES, 1024);
          if (leader)
            tc_mma_ts(tmem_base + 256, tmem_base + b * 128 + (k >> 1) * 32 + (k & 1) * 8, bd, idesc_acc,
                      (u | k) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t bd = make_smem_desc_sw128(qa + k * 2048, QS_HALF_BYTES, 1024);
          if (leader)
            tc_mma_ts(tmem_base + 384, tmem_base + b * 128 + 16 + (k >> 1) * 32 + (k & 1) * 8, bd, idesc_acc,
                      (u | k) ? 1u : 0u);
        }
        if (leader) {
          tc_commit(bar_qempty + 8 * st);
          if (u + 1 == U) tc_commit(bar_done);
        }
        if (u + 2 < U) {
          if (!wait_all(bar_qfull + 8 * st2, ph2, 23)) break;
          tc_fence_after();
          issue_s(b, st2);
          if (!wait_all(bar_dqread + 8 * b, (u >> 1) & 1, 24)) break;
          tc_fence_after();
          issue_dp(b, st2);
        }
        if (++st == STAGES) st = 0;
        if (++st2 == STAGES) {
          st2 = 0;
          ph2 ^= 1;
        }
      }
      __syncwarp();
    }
  } else {
    // four groups of four warps: unit parity b, and within a unit 32 of its 64 queries
    const int b = warp >> 3;
    const int sub = (warp >> 2) & 1;
    const int grp = warp >> 2;
    const int qd = warp & 3;
    const int row = qd * 32 + lane;   // key row inside the tile (TMEM lane); d index for dQᵀ
    const int kcode = p.k_code[kt * 128 + row];
    const uint32_t t_s = tmem_base + ((uint32_t)(qd * 32) << 16) + b * 128;
    float* red = (float*)(sRed + grp * RED_BYTES);
    const bool issuer = (qd == 0 && lane == 0);   // issues and tracks this group's reduce-add copies
    int st = b;   // stage of unit 2*it + b
    for (int it = 0; it < items; ++it) {
      const int ent = list[it % n];
      const int qrow0 = (ent >> 1) * 128 + b * 64 + sub * 32;
      const float* sl = sStat + st * 128 + sub * 32;   // lse2 of this group's 32 queries
      const float* sd = sl + 64;                       // delta_s
      bool good = __all_sync(0xffffffffu, mbar_wait_spin(bar_sfull + 8 * b, it & 1, KID, 30));
      if (good) {
        tc_fence_after();
        // two chunks of 16 queries: keeps the live registers under the 96 this block size allows
        // (spilled values come back through L2, since nearly all of L1 is shared memory here)
        uint32_t pk[16], dk[16];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t rs[16], rp[16];
          tmem_ld16(t_s + sub * 32 + c * 16, rs);
          tmem_ld16(t_s + 64 + sub * 32 + c * 16, rp);
          tmem_ld_wait();
          if (ent & 1) {
#pragma unroll
            for (int e = 0; e < 16; e += 4) {
              const float4 l4 = *reinterpret_cast<const float4*>(sl + c * 16 + e);
              const float4 d4 = *reinterpret_cast<const float4*>(sd + c * 16 + e);
              const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
              const float dv[4] = {d4.x, d4.y, d4.z, d4.w};
              float pv[4], ds[4];
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                const int g = qrow0 + c * 16 + e + t;
                float pr = fast_exp2(fmaf(__uint_as_float(rs[e + t]), p.scale_log2, lv[t]));
                if (!key_visible(kcode, __ldg(p.q_lo + g), __ldg(p.q_hi + g), __ldg(p.q_grp + g))) pr = 0.f;
                pv[t] = pr;
                ds[t] = pr * fmaf(__uint_as_float(rp[e + t]), p.scale, dv[t]);
              }
              pk[c * 8 + (e >> 1)] = pack_bf16x2(pv[0], pv[1]);
              pk[c * 8 + (e >> 1) + 1] = pack_bf16x2(pv[2], pv[3]);
              dk[c * 8 + (e >> 1)] = pack_bf16x2(ds[0], ds[1]);
              dk[c * 8 + (e >> 1) + 1] = pack_bf16x2(ds[2], ds[3]);
            }
          } else {
            // two queries per instruction: t = s·scale_log2 + (−lse2), u = dP·scale + (−delta_s), dS = p·u
            const uint64_t sc_l2 = pair_f32(p.scale_log2, p.scale_log2), sc = pair_f32(p.scale, p.scale);
#pragma unroll
            for (int e = 0; e < 16; e += 4) {
              const float4 l4 = *reinterpret_cast<const float4*>(sl + c * 16 + e);
              const float4 d4 = *reinterpret_cast<const float4*>(sd + c * 16 + e);
              const uint64_t t01 = fma_f32x2(pair_f32(__uint_as_float(rs[e]), __uint_as_float(rs[e + 1])), sc_l2,
                                             pair_f32(l4.x, l4.y));
              const uint64_t t23 = fma_f32x2(pair_f32(__uint_as_float(rs[e + 2]), __uint_as_float(rs[e + 3])), sc_l2,
                                             pair_f32(l4.z, l4.w));
              const uint64_t u01 = fma_f32x2(pair_f32(__uint_as_float(rp[e]), __uint_as_float(rp[e + 1])), sc,
                                             pair_f32(d4.x, d4.y));
              const uint64_t u23 = fma_f32x2(pair_f32(__uint_as_float(rp[e + 2]), __uint_as_float(rp[e + 3])), sc,
                                             pair_f32(d4.z, d4.w));
              float t0, t1, t2, t3;
              unpair_f32(t01, t0, t1);
              unpair_f32(t23, t2, t3);
              const float p0 = fast_exp2(t0), p1 = fast_exp2(t1), p2 = fast_exp2(t2), p3 = fast_exp2(t3);
              float s0, s1, s2, s3;
              unpair_f32(mul_f32x2(pair_f32(p0, p1), u01), s0, s1);
              unpair_f32(mul_f32x2(pair_f32(p2, p3), u23), s2, s3);
              pk[c * 8 + (e >> 1)] = pack_bf16x2(p0, p1);
              pk[c * 8 + (e >> 1) + 1] = pack_bf16x2(p2, p3);
              dk[c * 8 + (e >> 1)] = pack_bf16x2(s0, s1);
              dk[c * 8 + (e >> 1) + 1] = pack_bf16x2(s2, s3);
            }
          }
        }
        // in place over the 32 Sᵀ columns this group has just read (the other group of the unit may
        // still be reading its own): Pᵀ in the first 16, dSᵀ in the last 16
        tmem_st16(t_s + sub * 32, pk);
        tmem_st16(t_s + sub * 32 + 16, dk);
        {
          uint8_t* srow = sdS + b * DS_BYTES;   // this key's 64 queries: one swizzled 128-byte row
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(srow + sw128_offset(row, sub * 4 + j)) =
                make_uint4(dk[4 * j], dk[4 * j + 1], dk[4 * j + 2], dk[4 * j + 3]);
        }
        tmem_st_wait();
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(bar_pfull + 8 * b);
        // dQᵀ of this unit: lanes = d, columns = the unit's 64 queries
        good = __all_sync(0xffffffffu, mbar_wait_spin(bar_dqfull + 8 * b, it & 1, KID, 33));
      }
      // the group's staging rows are free once its previous copy has read them; the vote keeps the
      // four warps together (a warp whose wait ran out takes the others out with it)
      if (issuer) tma_store_wait_read<0>();
      if (!named_bar_all(1 + grp, 128, good)) break;
      tc_fence_after();
      const int h = kvh * G + it / n;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rq[16];
        tmem_ld16(t_s + 64 + sub * 32 + c * 16, rq);
        tmem_ld_wait();
        if (c == 1) {
          tc_fence_before();
          mbar_arrive(bar_dqread + 8 * b);
          if (issuer) tma_store_wait_read<0>();
          named_bar_sync(1 + grp, 128);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) red[j * HD + row] = __uint_as_float(rq[j]);
        fence_proxy_async_smem();
        named_bar_sync(1 + grp, 128);
        if (issuer) {
          tma_reduce_add_2d(&tm_dqacc, smem_u32(red), h * HD, qrow0 + c * 16);
          tma_store_commit();
        }
      }
      st += 2;
      if (st >= STAGES) st -= STAGES;
    }
    if (issuer) tma_store_wait_all();
    // epilogue: the groups of slot 0 add dV, those of slot 1 add dK to the fp32 accumulators: fp32 tile
    // staged as four [128 keys][32 columns] swizzled blocks (64 KiB per tensor, over the Q / dO / dSᵀ
    // buffers, which nothing reads any more once the last product has completed)
    bool ok = !error_is_set();
    if (ok && items > 0) ok = mbar_wait_spin(bar_done, 0, KID, 31);
    if (CSBP && ok && items > 0 && kt >= pp.nlt) {
      // a peer's key rows: this thread's row (TMEM lane) goes to the owner's accumulator, 64 of the 128
      // columns per thread (the two groups of a slot split them), four values per packet
      tc_fence_after();
      const uint32_t t_acc = tmem_base + ((uint32_t)(qd * 32) << 16) + 256 + b * 128;
      const long long rrow = (long long)(kt - pp.nlt) * 128 + row;
      int s = 0;
      while (s + 1 < pp.nseg && rrow >= pp.seg_begin[s + 1]) ++s;
      const bool live = rrow < pp.n_rows;
      float* base = b ? pp.dk[s] : pp.dv[s];
      float* dst = base + (pp.dst_row0[s] + (rrow - pp.seg_begin[s])) * ((long long)p.Hkv * HD) + kvh * HD;
      uint32_t rs[32];
#pragma unroll 1
      for (int c = 2 * sub; c < 2 * sub + 2; ++c) {
        tmem_ld32(t_acc + c * 32, rs);
        tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int v = 0; v < 8; ++v)
            red_add_peer_f32x4(dst + c * 32 + 4 * v, rs[4 * v], rs[4 * v + 1], rs[4 * v + 2], rs[4 * v + 3]);
        }
      }
    } else if (ok && items > 0) {
      tc_fence_after();
      const uint32_t t_acc = tmem_base + ((uint32_t)(qd * 32) << 16) + 256 + b * 128;
      uint8_t* stg = smem + OFF_Q + b * 65536;
      uint32_t rs[32];
#pragma unroll 1
      for (int c = 2 * sub; c < 2 * sub + 2; ++c) {
        tmem_ld32(t_acc + c * 32, rs);
        tmem_ld_wait();
        uint8_t* blk = stg + c * 16384;
#pragma unroll
        for (int v = 0; v < 8; ++v)
          *reinterpret_cast<uint4*>(blk + sw128_offset(row, v)) =
              make_uint4(rs[4 * v], rs[4 * v + 1], rs[4 * v + 2], rs[4 * v + 3]);
      }
      fence_proxy_async_smem();
      mbar_arrive(bar_epi + 8 * b);
      if (row == 0 && sub == 0) {
        if (mbar_wait_spin(bar_epi + 8 * b, 0, KID, 32)) {
          const CUtensorMap* tm = b ? &tm_dkacc : &tm_dvacc;
#pragma unroll
          for (int c = 0; c < 4; ++c)
            tma_reduce_add_2d(tm, smem_u32(stg + c * 16384), kvh * HD + c * 32, kt * 128);
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
  if (warp == 17) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace attn_fused
}  // namespace tdllm
