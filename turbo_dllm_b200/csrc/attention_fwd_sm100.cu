// Block-diffusion attention forward for sm_100a (head_dim 128).
//
// One CTA owns one 128-row query tile and TWO query heads that share a KV head, so every
// K/V tile it streams in is used by two independent softmax pipelines ("ping-pong"):
//   warps 0-3  softmax group 0 (head h0)      warp 8  TMA producer (Q once, K/V stream)
//   warps 4-7  softmax group 1 (head h1)      warp 9  tcgen05.mma issuer
// S = Q·Kᵀ lands in TMEM, is read with tcgen05.ld, exponentiated, written back to TMEM as
// bf16 P over the same columns and consumed by O += P·V (A operand from TMEM). O stays in
// TMEM for the whole tile list and is rescaled lazily (only when the running max grows
// by more than 2^8), so no correction warps are needed.
//
// Masking is declarative. Each query row carries (lo, hi, grp); each key carries one code:
//   code >= 0 : a clean key at coordinate `code`  -> visible iff lo <= code < hi
//   code <  0 : a noisy key of block -(code+1)    -> visible iff code == grp
// which expresses "bidirectional inside a noisy block, noisy block b sees clean blocks < b,
// clean block c sees clean blocks <= c, clean never sees noisy", sliding windows and several
// sequences per batch (coordinates are offset per sequence). The host passes, per query tile,
// the list of key tiles that contain any visible key and whether the tile needs the
// per-element predicate; fully visible tiles skip it.
//
// This is the sm_100a counterpart of the reference's masked FlashAttention paths:
// third_party/flash-attention/hopper/mask.h:165 (BDLM mask), dllm_parallel/core/attention/fa4.py:71-132
// (mask_mod) and the predicate of dllm_parallel/core/attention/context_parallel_attention.py:119-144.
// It returns (out, lse) so shard results can be merged across K/V owners.
//
// Context-sharded form (template argument CSBP): key tiles [0, nlt) are this rank's own rows and are read
// in place; key tiles [nlt, nlt + nrt) are clean K|V rows owned by the peers of the context-parallel group.
// Two extra warps per CTA ("pullers") fetch those rows from the peers' symmetric staging buffers with plain
// 16-byte peer loads into a buffer in this GPU's memory, 16 rows per claim from a shared counter, and count
// finished claims per key tile; the TMA warp waits (bounded) for a remote tile's count before it loads the
// tile. Each remote row crosses NVLink once, the tiles of this rank run while the first remote rows arrive,
// and the pull of later tiles overlaps the products of earlier ones. No TMA touches a peer's memory.
// Counterpart: the asynchronous clean K/V all-gather overlapped with the local attention in
// dllm_parallel/core/attention/context_parallel_attention.py:2315-2691 (:701-741 for the gather itself).
#include <cstring>
#include "common.cuh"
#include "peer_pull.cuh"
#include "api.h"

namespace tdllm {
namespace attn {

constexpr int KID = 2;  // kernel id in the error record
constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int HD = 128;
constexpr int TILE_BYTES = 128 * HD * 2;  // 32 KiB: two 64-column halves of 128 rows x 128 B
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int KV_STAGES = 2;
constexpr int THREADS = 576;   // 16 softmax warps (2 heads x 2 column halves x 4 lane quarters), TMA warp 16, MMA warp 17
constexpr int THREADS_CSBP = 640;   // + puller warps 18 and 19
constexpr int KID_PULL = 6;         // error-record id of the pull side of the context-sharded form
using peer::MAX_PEERS;
using peer::PULL_ROWS;
using peer::PullPlan;
constexpr int SMEM_BYTES = 2 * TILE_BYTES + 2 * KV_STAGES * TILE_BYTES + 512 + 2048 + 1024;   // + barriers + row exchange

struct FwdParams {
  int nq_pad;          // query rows padded to a multiple of 128
  int Hq, Hkv;
  const int* q_lo;     // [nq_pad]
  const int* q_hi;     // [nq_pad]
  const int* q_grp;    // [nq_pad]
  const int* k_code;   // [nk_pad]
  const int* tile_ptr; // [n_qtiles + 1]
  const int* tile_idx; // entries: kv_tile * 2 + needs_mask
  const int* order;    // [n_qtiles] query tiles, heaviest first
  float* lse;          // [Hq, nq_pad]
  float scale_log2;    // softmax scale * log2(e)
  float scale;         // softmax scale
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

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

__device__ __forceinline__ bool key_visible(int code, int lo, int hi, int grp) {
  return code >= 0 ? (code >= lo && code < hi) : (code == grp);
}

template <bool CSBP>
__global__ void __launch_bounds__(CSBP ? THREADS_CSBP : THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                const __grid_constant__ CUtensorMap tm_kr, const __grid_constant__ CUtensorMap tm_vr,
                const FwdParams p, const __grid_constant__ PullPlan pl) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                                   // 2 heads x 32 KiB
  uint8_t* sK = sQ + 2 * TILE_BYTES;                    // KV_STAGES x 32 KiB
  uint8_t* sV = sK + KV_STAGES * TILE_BYTES;            // KV_STAGES x 32 KiB
  uint64_t* bars = (uint64_t*)(sV + KV_STAGES * TILE_BYTES);
  const uint32_t b0 = smem_u32(bars);
  const uint32_t bar_q = b0;
  const uint32_t bar_kfull = b0 + 8;         // [2]
  const uint32_t bar_kempty = b0 + 24;       // [2]
  const uint32_t bar_vfull = b0 + 40;        // [2]
  const uint32_t bar_vempty = b0 + 56;       // [2]
  const uint32_t bar_sfull = b0 + 72;        // [2] S_i ready
  const uint32_t bar_pfull = b0 + 88;        // [2] P_i written
  const uint32_t bar_odone = b0 + 104;       // [2] last P·V of head i complete
  const uint32_t bar_epi = b0 + 120;         // [2] output staged in shared memory
  uint32_t* tmem_slot = (uint32_t*)(bars + 17);
  float* sX = (float*)((uint8_t*)bars + 512);   // [head][column half][128 rows]: row maxima, then row sums

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // work decomposition
  const int G = p.Hq / p.Hkv;
  const int pairs = (G + 1) / 2;   // an odd group's last CTA runs its single head in both pipelines
  int w = blockIdx.x;
  const int pr = w % pairs;
  w /= pairs;
  const int kvh = w % p.Hkv;
  const int qt = p.order[w / p.Hkv];
  const int h0 = kvh * G + 2 * pr;
  const int h_last = kvh * G + G - 1;
  const int list_begin = p.tile_ptr[qt];
  const int n = p.tile_ptr[qt + 1] - list_begin;
  const int* list = p.tile_idx + list_begin;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_kfull + 8 * s, 1);
      mbar_init(bar_kempty + 8 * s, 1);
      mbar_init(bar_vfull + 8 * s, 1);
      mbar_init(bar_vempty + 8 * s, 1);
      mbar_init(bar_sfull + 8 * s, 1);
      mbar_init(bar_pfull + 8 * s, 256);
      mbar_init(bar_odone + 8 * s, 1);
      mbar_init(bar_epi + 8 * s, 256);
    }
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
  // TMEM columns: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_i aliases S_i[0,64)

  if (warp == 16) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && n > 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      if (CSBP) {
        tma_prefetch_desc(&tm_kr);
        tma_prefetch_desc(&tm_vr);
      }
      mbar_expect_tx(bar_q, 2 * TILE_BYTES);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int c = 0; c < 2; ++c)
          tma_load_2d(smem_u32(sQ + i * TILE_BYTES + c * HALF_BYTES), &tm_q, bar_q,
                      min(h0 + i, h_last) * HD + c * 64, qt * BQ);
      for (int j = 0; j < n; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        int kt = list[j] >> 1;
        const CUtensorMap* mk = &tm_k;
        const CUtensorMap* mv = &tm_v;
        if (CSBP && kt >= pl.nlt) {
          // a peer's rows: wait until the pullers have brought the whole tile into local memory
          kt -= pl.nlt;
          if (!peer::count_wait_geq(pl.tile_ready + kt, pl.tile_target, KID_PULL, 100)) break;
          peer::fence_proxy_async_global();
          mk = &tm_kr;
          mv = &tm_vr;
        }
        if (!mbar_wait_spin(bar_kempty + 8 * s, ph ^ 1, KID, 10)) break;
        mbar_expect_tx(bar_kfull + 8 * s, TILE_BYTES);
#pragma unroll
        for (int c = 0; c < 2; ++c)
          tma_load_2d(smem_u32(sK + s * TILE_BYTES + c * HALF_BYTES), mk, bar_kfull + 8 * s,
                      kvh * HD + c * 64, kt * BKV);
        if (!mbar_wait_spin(bar_vempty + 8 * s, ph ^ 1, KID, 11)) break;
        mbar_expect_tx(bar_vfull + 8 * s, TILE_BYTES);
#pragma unroll
        for (int c = 0; c < 2; ++c)
          tma_load_2d(smem_u32(sV + s * TILE_BYTES + c * HALF_BYTES), mv, bar_vfull + 8 * s,
                      kvh * HD + c * 64, kt * BKV);
      }
    }
  } else if (warp == 17) {
    // ------------------------------ MMA issuer --------------------------------
    // whole warp, identical values, one elected lane issues (descriptors stay in uniform registers;
    // issuing from a divergent lane-0 branch costs ~130 cycles per MMA on the issuing thread)
    if (n > 0) {
      const bool leader = elect_one();
      const uint32_t idesc_qk = make_idesc_bf16(BQ, BKV, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(BQ, HD, 0, 1);
      auto wait_all = [&](uint32_t bar, uint32_t parity, int detail) {
        return __all_sync(0xffffffffu, mbar_wait_spin(bar, parity, KID, detail));
      };
      auto issue_qk = [&](int i, int s) {
        const uint32_t qa = smem_u32(sQ + i * TILE_BYTES);
        const uint32_t ka = smem_u32(sK + s * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
          const uint64_t ad = make_smem_desc_sw128(qa + off, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(ka + off, 16, 1024);
          if (leader) tc_mma_ss(tmem_base + i * 128, ad, bd, idesc_qk, k ? 1u : 0u);
        }
        if (leader) tc_commit(bar_sfull + 8 * i);
      };
      bool ok = wait_all(bar_q, 0, 20) && wait_all(bar_kfull, 0, 21);
      if (ok) {
        tc_fence_after();
        issue_qk(0, 0);
        issue_qk(1, 0);
        if (leader) tc_commit(bar_kempty);
      }
      for (int j = 0; j < n && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!wait_all(bar_vfull + 8 * s, ph, 22)) break;
        const uint32_t va = smem_u32(sV + s * TILE_BYTES);
        for (int i = 0; i < 2; ++i) {
          if (!wait_all(bar_pfull + 8 * i, j & 1, 23)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < BKV / 16; ++k) {
            const uint64_t bd = make_smem_desc_sw128(va + k * 2048, HALF_BYTES, 1024);
            if (leader)
              tc_mma_ts(tmem_base + 256 + i * 128, tmem_base + i * 128 + k * 8, bd, idesc_pv, (j | k) ? 1u : 0u);
          }
          if (leader) {
            if (j + 1 == n) tc_commit(bar_odone + 8 * i);
            if (i == 1) tc_commit(bar_vempty + 8 * s);
          }
          if (j + 1 < n) {
            const int s1 = (j + 1) & 1;
            if (i == 0) {
              if (!wait_all(bar_kfull + 8 * s1, ((j + 1) >> 1) & 1, 24)) { ok = false; break; }
              tc_fence_after();
            }
            issue_qk(i, s1);
            if (i == 1 && leader) tc_commit(bar_kempty + 8 * s1);
          }
        }
      }
      __syncwarp();
    }
  } else if (CSBP && warp >= 18) {
    // ------------------------------ pullers (context-sharded form) -------------
    peer::pull_remote_rows(pl, lane, KID_PULL);
  } else {
    // ------------------------------ softmax groups -----------------------------
    // four warps per (head, column half): a thread owns one query row and 64 of the tile's 128 keys;
    // the two threads of a row meet through shared memory for the row maximum (every tile) and the
    // row sum (once, at the end)
    const int i = warp >> 3;          // which head of the pair
    const int sub = (warp >> 2) & 1;  // which 64 keys of a tile
    const int qd = warp & 3;          // TMEM lane quarter
    const int row = qd * 32 + lane;
    const int grow = qt * BQ + row;
    const uint32_t t_s = tmem_base + ((uint32_t)(qd * 32) << 16) + i * 128;
    const uint32_t t_o = tmem_base + ((uint32_t)(qd * 32) << 16) + 256 + i * 128;
    float* xmine = sX + (i * 2 + sub) * 128 + row;
    const float* xother = sX + (i * 2 + (sub ^ 1)) * 128 + row;
    float m_used = -INFINITY;  // max the stored probabilities are relative to (raw score units)
    float l = 0.f;             // this thread's share of the row sum
    uint32_t r[64];
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      const int ent = list[j];
      const int* kc = p.k_code + (ent >> 1) * BKV + sub * 64;
      bool good = __all_sync(0xffffffffu, mbar_wait_spin(bar_sfull + 8 * i, j & 1, KID, 30));
      if (good) {
        tc_fence_after();
        tmem_ld32(t_s + sub * 64, r);
        tmem_ld32(t_s + sub * 64 + 32, r + 32);
        tmem_ld_wait();
        if (ent & 1) {
          const int lo = __ldg(p.q_lo + grow), hi = __ldg(p.q_hi + grow), grp = __ldg(p.q_grp + grow);
#pragma unroll
          for (int e = 0; e < 64; ++e)
            if (!key_visible(__ldg(kc + e), lo, hi, grp)) r[e] = 0xff800000u;  // -inf
        }
        float mx = -INFINITY;
#pragma unroll
        for (int e = 0; e < 64; ++e) mx = fmaxf(mx, __uint_as_float(r[e]));
        *xmine = mx;
      }
      // the barrier also orders the P stores below after the partner's loads of its score columns
      if (!named_bar_all(1 + i, 256, good)) { ok = false; break; }
      float mx = fmaxf(*xmine, *xother);
      // lazy rescale: keep the old reference max unless the new one is 2^8 larger (both threads of a
      // row take the same decision: same inputs)
      float alpha = 1.f;
      if (mx > -INFINITY && (m_used == -INFINITY || (mx - m_used) * p.scale_log2 > 8.f)) {
        alpha = (m_used == -INFINITY) ? 0.f : fast_exp2((m_used - mx) * p.scale_log2);
        m_used = mx;
      }
      l *= alpha;
      if (__any_sync(0xffffffffu, alpha != 1.f) && j > 0) {
        uint32_t ro[16];
#pragma unroll 1
        for (int c = 4 * sub; c < 4 * sub + 4; ++c) {   // this thread's half of the accumulator columns
          tmem_ld16(t_o + c * 16, ro);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) ro[e] = __float_as_uint(__uint_as_float(ro[e]) * alpha);
          tmem_st16(t_o + c * 16, ro);
        }
      }
      // probabilities -> bf16 P in TMEM over the S columns; masked scores are -inf -> exactly 0
      const float mref = (m_used == -INFINITY) ? 0.f : m_used * p.scale_log2;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[8];
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(r[c * 16 + e]), p.scale_log2, -mref));
          const float p1 = fast_exp2(fmaf(__uint_as_float(r[c * 16 + e + 1]), p.scale_log2, -mref));
          l += p0 + p1;
          pk[e >> 1] = pack_bf16x2(p0, p1);
        }
        tmem_st8(t_s + sub * 32 + c * 8, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar_pfull + 8 * i);
    }
    // epilogue: O / l -> bf16 -> shared staging (the Q tile of this head) -> TMA store
    if (ok && n > 0) ok = mbar_wait_spin(bar_odone + 8 * i, 0, KID, 31);
    // row sum over both column halves (every thread takes part in the exchange, also after a failed wait)
    *xmine = l;
    ok = named_bar_all(1 + i, 256, ok);
    if (ok) {
      l += *xother;
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      uint8_t* st = sQ + i * TILE_BYTES;
      uint32_t ro[32];
#pragma unroll 1
      for (int c = 2 * sub; c < 2 * sub + 2; ++c) {
        if (n > 0) {
          tmem_ld32(t_o + c * 32, ro);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) ro[e] = 0u;
        }
        uint8_t* half = st + (c >> 1) * HALF_BYTES;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint32_t a[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            a[e] = pack_bf16x2(__uint_as_float(ro[8 * v + 2 * e]) * inv,
                               __uint_as_float(ro[8 * v + 2 * e + 1]) * inv);
          *reinterpret_cast<uint4*>(half + sw128_offset(row, (c & 1) * 4 + v)) =
              make_uint4(a[0], a[1], a[2], a[3]);
        }
      }
      if (sub == 0)
        p.lse[(size_t)min(h0 + i, h_last) * p.nq_pad + grow] = l > 0.f ? m_used * p.scale + __logf(l) : -INFINITY;
      fence_proxy_async_smem();
      mbar_arrive(bar_epi + 8 * i);
      if (row == 0 && sub == 0) {
        if (mbar_wait_spin(bar_epi + 8 * i, 0, KID, 32)) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
            tma_store_2d(&tm_o, smem_u32(st + c * HALF_BYTES), min(h0 + i, h_last) * HD + c * 64, qt * BQ);
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

}  // namespace attn
}  // namespace tdllm

using namespace tdllm;

namespace tdllm_host {
int encode_rows_tmap(CUtensorMap* out, const void* base, long long cols, long long rows,
                     long long ld_elems, int box_rows) {
  uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows};
  uint64_t strides[1] = {(uint64_t)ld_elems * 2};
  uint32_t box[2] = {64, (uint32_t)box_rows};
  return encode_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_128B);
}
}  // namespace tdllm_host

static int attn_fwd_check(const char* who, int Hq, int Hkv, const long long* lds, const void* const* ptrs, int n) {
  if (Hq % Hkv) {
    tdllm_host::set_last_error("%s: %d query heads do not divide over %d KV heads", who, Hq, Hkv);
    return 1;
  }
  for (int i = 0; i < n; ++i)
    if ((lds[i] % 8) || ((uintptr_t)ptrs[i] % 16)) {
      tdllm_host::set_last_error("%s: operand %d needs a 16-byte aligned base and row stride", who, i);
      return 1;
    }
  return 0;
}

// q [nq, Hq*128] (row stride ldq), k/v [nk, Hkv*128], o [nq, Hq*128], lse [Hq, nq_pad].
// Row metadata arrays are padded to nq_pad / nk_pad (multiples of 128) by the caller.
extern "C" int tdllm_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                              int nq, int nk, int Hq, int Hkv, long long ldq, long long ldk,
                              long long ldv, long long ldo, const int* q_lo, const int* q_hi,
                              const int* q_grp, const int* k_code, const int* tile_ptr,
                              const int* tile_idx, const int* order, int n_qtiles, float scale,
                              void* stream) {
  using namespace tdllm::attn;
  if (nq <= 0) return 0;
  const long long lds[4] = {ldq, ldk, ldv, ldo};
  const void* ptrs[4] = {q, k, v, o};
  if (attn_fwd_check("attn_fwd", Hq, Hkv, lds, ptrs, 4)) return 1;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_BYTES);
    if (e != cudaSuccess) {
      tdllm_host::set_last_error("attn_fwd: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return 2;
    }
    attr_set = true;
  }
  CUtensorMap tq, tk, tv, to;
  if (tdllm_host::encode_rows_tmap(&tq, q, (long long)Hq * HD, nq, ldq, 128)) return 3;
  if (tdllm_host::encode_rows_tmap(&tk, k, (long long)Hkv * HD, nk, ldk, 128)) return 3;
  if (tdllm_host::encode_rows_tmap(&tv, v, (long long)Hkv * HD, nk, ldv, 128)) return 3;
  if (tdllm_host::encode_rows_tmap(&to, o, (long long)Hq * HD, nq, ldo, 128)) return 3;
  FwdParams p;
  p.nq_pad = n_qtiles * BQ;
  p.Hq = Hq; p.Hkv = Hkv;
  p.q_lo = q_lo; p.q_hi = q_hi; p.q_grp = q_grp; p.k_code = k_code;
  p.tile_ptr = tile_ptr; p.tile_idx = tile_idx; p.order = order;
  p.lse = lse;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  PullPlan pl;
  memset(&pl, 0, sizeof(pl));
  const int grid = n_qtiles * Hkv * ((Hq / Hkv + 1) / 2);
  attn_fwd_kernel<false><<<grid, THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(tq, tk, tv, to, tk, tv, p, pl);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    tdllm_host::set_last_error("attn_fwd launch: %s", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}

// Context-sharded forward. Keys are this rank's nk_loc rows (k_loc / v_loc, read in place) followed, from key
// tile ceil(nk_loc / 128) on, by the clean K|V rows of the other ranks of the group: kv_rem
// [n_rem, 2*Hkv*128] bf16 in this GPU's memory is filled inside the kernel from the peers' staged rows
// (staging[r]: rank r's [counts[r], 2*Hkv*128] rows as mapped here; peers are visited in the order rank+1,
// rank+2, ...). ready[r]: rank r's int32[world] flag array as mapped here; rank r stores `ready_epoch` into
// slot r of every array once its rows are staged (tdllm_symm_signal). counter: one int32 of scratch, zeroed
// here; tile_ready: int32 per remote key tile, zeroed once by the caller and never reset, with `launch_no`
// the 1-based number of this call on those counters. k_code and the tile lists index the concatenated keys.
extern "C" int tdllm_attn_fwd_csbp(const void* q, const void* k_loc, const void* v_loc, void* kv_rem, void* o,
                                   float* lse, int nq, int nk_loc, long long n_rem, int Hq, int Hkv,
                                   long long ldq, long long ldk, long long ldv, long long ldo, const int* q_lo,
                                   const int* q_hi, const int* q_grp, const int* k_code, const int* tile_ptr,
                                   const int* tile_idx, const int* order, int n_qtiles, float scale,
                                   void* const* staging, void* const* ready, const long long* counts, int rank,
                                   int world, int ready_epoch, int* counter, int* tile_ready, int launch_no,
                                   void* stream) {
  using namespace tdllm::attn;
  if (nq <= 0) return 0;
  const long long ldr = 2LL * Hkv * HD;
  const long long lds[5] = {ldq, ldk, ldv, ldo, ldr};
  const void* ptrs[5] = {q, k_loc, v_loc, o, kv_rem};
  if (attn_fwd_check("attn_fwd_csbp", Hq, Hkv, lds, ptrs, 5)) return 1;
  if (world < 2 || world > MAX_PEERS || rank < 0 || rank >= world) {
    tdllm_host::set_last_error("attn_fwd_csbp: 2..%d ranks (got %d)", MAX_PEERS, world);
    return 1;
  }
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_BYTES);
    if (e != cudaSuccess) {
      tdllm_host::set_last_error("attn_fwd_csbp: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return 2;
    }
    attr_set = true;
  }
  PullPlan pl;
  memset(&pl, 0, sizeof(pl));
  long long total = 0;
  pl.nseg = world - 1;
  for (int s = 0; s < world - 1; ++s) {
    const int peer = (rank + 1 + s) % world;
    pl.src[s] = (const uint4*)staging[peer];
    pl.ready[s] = (const int*)ready[rank] + peer;
    pl.seg_begin[s] = total;
    pl.dst_begin[s] = total;
    total += counts[peer];
  }
  for (int s = world - 1; s <= MAX_PEERS; ++s) pl.seg_begin[s] = total;
  if (total != n_rem) {
    tdllm_host::set_last_error("attn_fwd_csbp: peers hold %lld rows, caller expects %lld", total, n_rem);
    return 1;
  }
  pl.dst = (uint4*)kv_rem;
  pl.counter = counter;
  pl.tile_ready = tile_ready;
  pl.n_rows = n_rem;
  pl.want = ready_epoch;
  pl.row_vec16 = (int)(ldr * 2 / 16);
  pl.nlt = (nk_loc + BKV - 1) / BKV;
  pl.nrt = (int)((n_rem + BKV - 1) / BKV);
  pl.tile_target = launch_no * (BKV / PULL_ROWS);
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemsetAsync(counter, 0, sizeof(int), st) != cudaSuccess) {
    tdllm_host::set_last_error("attn_fwd_csbp: clearing the claim counter failed");
    return 5;
  }
  CUtensorMap tq, tk, tv, to, tkr, tvr;
  if (tdllm_host::encode_rows_tmap(&tq, q, (long long)Hq * HD, nq, ldq, 128)) return 3;
  if (tdllm_host::encode_rows_tmap(&tk, k_loc, (long long)Hkv * HD, nk_loc, ldk, 128)) return 3;
  if (tdllm_host::encode_rows_tmap(&tv, v_loc, (long long)Hkv * HD, nk_loc, ldv, 128)) return 3;
  if (tdllm_host::encode_rows_tmap(&to, o, (long long)Hq * HD, nq, ldo, 128)) return 3;
  const long long rem_rows = n_rem > 0 ? n_rem : 1;
  if (tdllm_host::encode_rows_tmap(&tkr, kv_rem, (long long)Hkv * HD, rem_rows, ldr, 128)) return 3;
  if (tdllm_host::encode_rows_tmap(&tvr, (const __nv_bfloat16*)kv_rem + (long long)Hkv * HD, (long long)Hkv * HD,
                                   rem_rows, ldr, 128))
    return 3;
  FwdParams p;
  p.nq_pad = n_qtiles * BQ;
  p.Hq = Hq; p.Hkv = Hkv;
  p.q_lo = q_lo; p.q_hi = q_hi; p.q_grp = q_grp; p.k_code = k_code;
  p.tile_ptr = tile_ptr; p.tile_idx = tile_idx; p.order = order;
  p.lse = lse;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int grid = n_qtiles * Hkv * ((Hq / Hkv + 1) / 2);
  attn_fwd_kernel<true><<<grid, THREADS_CSBP, SMEM_BYTES, st>>>(tq, tk, tv, to, tkr, tvr, p, pl);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    tdllm_host::set_last_error("attn_fwd_csbp launch: %s", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}
