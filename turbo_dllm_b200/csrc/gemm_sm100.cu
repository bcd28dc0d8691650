// Persistent bf16 GEMM for sm_100a: TMA (local memory) -> 128B-swizzled shared memory ->
// tcgen05.mma (one issuing thread) -> fp32 accumulators in TMEM (double buffered) ->
// tcgen05.ld epilogue -> shared staging -> TMA store.
//
//   D[M,N] (+)= A * B with  A given as [M,K] (K-major) or [K,M] (MN-major)
//                           B given as [N,K] (K-major) or [K,N] (MN-major)
//
// That covers the three products of a linear layer y = x W^T without any transpose
// copy: forward (K,K), input gradient (K,MN), weight gradient (MN,MN).
//
// Epilogues: plain store (bf16 or fp32, optional accumulate into the destination),
// SwiGLU on interleaved gate/up columns, cross-entropy row statistics (no logits
// written), cross-entropy gradient of the logits (written as bf16), and an all-reduce over
// peer memory for products whose K dimension is split over ranks (row-parallel linears):
// every epilogue warp writes its bf16 partial slice into the workspace of every other rank (plain
// peer stores), publishes a per-(tile, warp) flag, waits for the peers' flags of the same slice and
// adds their partials (+ residual) to its own fp32 accumulator, which never leaves TMEM. Ranks
// walk the tiles in the same order, so the exchange of one tile overlaps the tensor-core work on
// the next (two accumulator buffers); no collective call is involved.
//
// Sequence parallelism inside a tensor-parallel group adds two fused forms (template argument AG, rs_rows):
//   all-gather -> GEMM : A's rows are sharded over the ranks. Two extra warps per CTA pull the peers' rows into
//     this GPU's copy of A (plain peer loads, 16-row pieces claimed from a shared counter, one arrival counter
//     per 128-row tile) while the tiles of this rank's own rows run; the TMA warp waits (bounded) for a remote
//     tile's counter before loading it. The tile walk starts at this rank's rows and follows the pull order.
//   GEMM -> reduce-scatter : the all-reduce epilogue with an owner per row tile. A tile owned by a peer is pushed
//     to that peer only and not stored here; a tile this rank owns waits for the peers' partials and is stored
//     to the rank's [M / ranks, N] output. Rank r starts its walk at the rows of rank r+1 and reaches its own
//     rows last, so the ranks push to different owners at any moment and an owner's waits are short.
// Counterpart: Transformer Engine's userbuffers overlap (dllm_parallel/core/parallel/transformer_engine.py:84-139)
// behind dllm_parallel/core/parallel/tensor_parallel/sequence_parallel.py:158-285.
//
// This replaces the library GEMMs the reference calls (cublasGemmEx in
// dllm_parallel/core/csrc/fused_linear_ce/fused_linear_ce_cuda.cu:618-791 and the
// torch / Transformer Engine linears of
// dllm_parallel/core/models/backbones/nemotron/model.py:3727-4190).
#include <cstring>
#include "common.cuh"
#include "peer_pull.cuh"
#include "api.h"

namespace tdllm {

constexpr int GEMM_KERNEL_ID = 1;
constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int EPI_WARPS = 4;
constexpr int EPI_BUF_BYTES = 32 * 128;  // one warp: 32 rows x 128 bytes
constexpr int GEMM_THREADS = 32 * (2 + EPI_WARPS);
constexpr int GEMM_THREADS_AG = GEMM_THREADS + 64;   // + two puller warps (all-gather fused into the product)
constexpr int KID_GEMM_PULL = 7;
constexpr int SMEM_EPI = EPI_WARPS * 2 * EPI_BUF_BYTES;

// PAIR = 1: one CTA per 128 x 256 tile. PAIR = 2: a cluster of two CTAs per 256 x 256 tile
// (tcgen05 cta_group::2): each CTA loads its own 128 rows of A and half of the B tile, so
// every MMA reads 8 KiB of shared memory per SM instead of 12 KiB; the single-CTA form is bound by
// that read (171 cycles per 128x256x16 MMA measured, against 128 of tensor work).
template <int PAIR>
struct Cfg {
  static constexpr int B_ROWS = BN / PAIR;
  static constexpr int B_STAGE_BYTES = B_ROWS * BK * 2;        // 32 or 16 KiB
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGES = PAIR == 2 ? 6 : 4;
  static constexpr int SMEM_TILES = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = SMEM_TILES + SMEM_EPI + 256 + 1024;  // + barriers + align slack
};

enum EpilogueMode : int {
  EPI_STORE = 0,     // D = acc (bf16 or fp32), optional D += acc
  EPI_SWIGLU = 1,    // D[:, j] = silu(acc[:, 2j]) * acc[:, 2j+1], bf16, N_out = N/2
  EPI_CE_STATS = 2,  // per (row, n-tile): max, sum exp, target logit -> fp32 scratch
  EPI_CE_GRAD = 3,   // D = (exp(acc - lse[row]) - onehot(label[row])) * rowscale[row], bf16
  EPI_ALLREDUCE = 4, // D = sum over ranks of acc (+ C), bf16, partial tiles exchanged through peer memory
};
constexpr int AR_MAX_RANKS = 8;

struct GemmParams {
  int M, N, K;
  int a_mn_major, b_mn_major;
  int mode;
  int out_fp32;
  int accumulate;
  int m_tiles, n_tiles;
  // accumulate path: D = acc + C, where C is the destination itself or a separate tensor
  // of the destination's dtype (fused residual add)
  const void* c_ptr;
  long long ldc;  // elements
  // cross-entropy epilogues
  const int* labels;      // [M], negative = ignored row
  const float* lse;       // [M]
  const float* rowscale;  // [M]
  float* stats;           // [M, n_tiles, 3]
  int exclude_index;      // column removed from the softmax (-1 = none)
  float softcap;          // 0 = off
  // all-reduce epilogue: workspace of rank d (as mapped here) holds [ranks][ar_rows][N] bf16 partials,
  // flags of rank d hold [ranks][tiles * 4] epochs (one per source rank, 128-row tile and 32-row warp slice)
  int ar_world, ar_rank, ar_epoch;
  long long ar_rows;
  void* ar_ws[AR_MAX_RANKS];
  int* ar_flags[AR_MAX_RANKS];
  void* ar_out;       // destination (this rank's memory), row stride ar_ldd elements
  long long ar_ldd;
  // grouped products (experts): per 128-row tile of M, the group whose slice of B is used (B's row
  // coordinate is shifted by group * b_group_rows) and/or the range of K blocks to run over (ragged K:
  // each group of output rows sums over its own rows of the operands). Null = plain GEMM.
  const int* mt_group;
  long long b_group_rows;
  long long a_group_rows;   // A's M coordinate is shifted back by group * a_group_rows (per-group outputs)
  const int* mt_kbegin;
  const int* mt_kend;
  // sequence-parallel forms
  int m_rot;        // the tile walk starts at this group of PAIR row tiles and wraps around
  int rs_rows;      // > 0: reduce-scatter epilogue, rank r owns rows [r * rs_rows, (r + 1) * rs_rows)
  int ag_rows;      // > 0: all-gather form, rank r's rows of A are [r * ag_rows, (r + 1) * ag_rows)
  int ag_rank;
};

__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int& m, int& n, int m_rot = 0) {
  constexpr int G = 8;
  const int per_group = G * n_tiles;
  const int g = t / per_group;
  const int first_m = g * G;
  const int gsz = min(m_tiles - first_m, G);
  const int r = t - g * per_group;
  m = first_m + r % gsz + m_rot;
  if (m >= m_tiles) m -= m_tiles;
  n = r / gsz;
}

__device__ __forceinline__ float apply_softcap(float x, float cap) {
  return cap > 0.f ? cap * tanhf(x / cap) : x;
}

template <int PAIR, bool AG>
__global__ void __launch_bounds__(AG ? GEMM_THREADS_AG : GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_d, const GemmParams p,
                 const __grid_constant__ peer::PullPlan pl) {
  constexpr int STAGES = Cfg<PAIR>::STAGES;
  constexpr int STAGE_BYTES = Cfg<PAIR>::STAGE_BYTES;
  constexpr int SMEM_TILES = Cfg<PAIR>::SMEM_TILES;
  constexpr int B_ROWS = Cfg<PAIR>::B_ROWS;
  extern __shared__ uint8_t smem_raw[];
  // the two CTAs of a pair must use identical offsets: the window bases are equally aligned
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* epi_smem = smem + SMEM_TILES;
  uint64_t* bars = (uint64_t*)(epi_smem + SMEM_EPI);
  // bars: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], then tmem base word
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * STAGES;
  const uint32_t bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // a pair walks 256-row tiles together; CTA `rank` owns the rank-th 128 rows of each
  const int rank = PAIR == 2 ? (int)cluster_ctarank() : 0;
  const int m_groups = (p.m_tiles + PAIR - 1) / PAIR;
  const int num_tiles = m_groups * p.n_tiles;
  const int walker = blockIdx.x / PAIR, walkers = gridDim.x / PAIR;
  const int k_blocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, EPI_WARPS * PAIR);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    if (PAIR == 2) {
      tmem_alloc_pair(smem_u32(tmem_slot), 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), 512);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if (PAIR == 2) cluster_sync_all();   // the peer's barriers exist before anything is sent to them
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = walker; t < num_tiles && ok; t += walkers) {
        int tm, tn;
        tile_coords(t, m_groups, p.n_tiles, tm, tn, p.m_rot);
        tm = tm * PAIR + rank;
        const int b_row0 = tn * BN + rank * B_ROWS;
        const int tml = min(tm, p.m_tiles - 1);   // a pair's second CTA may sit past the last row tile
        const int b_shift = p.mt_group ? (int)(p.mt_group[tml] * p.b_group_rows) : 0;
        const int a_m0 = tm * BM - (p.mt_group ? (int)(p.mt_group[tml] * p.a_group_rows) : 0);
        const int kb0 = p.mt_kbegin ? p.mt_kbegin[tml] : 0;
        const int kb1 = p.mt_kend ? p.mt_kend[tml] : k_blocks;
        if (AG && tm < p.m_tiles && (tm * BM) / p.ag_rows != p.ag_rank) {
          // rows of a peer: wait until the pullers have brought this 128-row tile into local memory
          if (!peer::count_wait_geq(pl.tile_ready + tm, pl.tile_target, KID_GEMM_PULL, 100)) {
            ok = false;
            break;
          }
          peer::fence_proxy_async_global();
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, GEMM_KERNEL_ID, 10)) {
            ok = false;
            break;
          }
          // pair: both CTAs' bytes are credited to CTA 0's barrier, which expects the sum
          const uint32_t full = PAIR == 2 ? ((bar_full + 8 * stage) & PEER_BIT_MASK) : (bar_full + 8 * stage);
          if (rank == 0) mbar_expect_tx(bar_full + 8 * stage, STAGE_BYTES * PAIR);
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
          auto load = [&](uint32_t dst, const CUtensorMap* m, int x, int y) {
            if (PAIR == 2) tma_load_2d_pair(dst, m, full, x, y);
            else tma_load_2d(dst, m, full, x, y);
          };
          if (!p.a_mn_major) {
            load(sa, &tmap_a, kb * BK, a_m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) load(sa + c * (BK * 128), &tmap_a, a_m0 + c * 64, kb * BK);
          }
          if (!p.b_mn_major) {
            load(sb, &tmap_b, kb * BK, b_row0 + b_shift);
          } else {
#pragma unroll
            for (int c = 0; c < B_ROWS / 64; ++c)
              load(sb + c * (BK * 128), &tmap_b, b_row0 + c * 64, kb * BK + b_shift);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    // whole warp with identical values; one elected lane issues, so that the descriptors stay in
    // uniform registers (a divergent lane-0 branch makes every MMA cost ~130 cycles to issue)
    if (rank == 0) {   // in a pair, CTA 0 issues for both
      const bool leader = elect_one();
      const uint32_t idesc = make_idesc_bf16(BM * PAIR, BN, p.a_mn_major, p.b_mn_major);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = walker; t < num_tiles && ok; t += walkers, ++it) {
        const int buf = it & 1;
        const uint32_t tphase = (it >> 1) & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(bar_tempty + 8 * buf, tphase ^ 1, GEMM_KERNEL_ID, 20))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        int kb0 = 0, kb1 = k_blocks;
        if (p.mt_kbegin) {
          int tm_, tn_;
          tile_coords(t, m_groups, p.n_tiles, tm_, tn_, p.m_rot);
          const int tml = min(tm_ * PAIR, p.m_tiles - 1);
          kb0 = p.mt_kbegin[tml];
          kb1 = p.mt_kend[tml];
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(bar_full + 8 * stage, phase, GEMM_KERNEL_ID, 21))) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: step 32 bytes inside the 128-byte swizzled row.
            // MN-major: step 16 rows of 128 bytes.
            const uint64_t ad = p.a_mn_major
                                    ? make_smem_desc_sw128(sa + k * (UMMA_K * 128), BK * 128, 1024)
                                    : make_smem_desc_sw128(sa + k * (UMMA_K * 2), 16, 1024);
            const uint64_t bd = p.b_mn_major
                                    ? make_smem_desc_sw128(sb + k * (UMMA_K * 128), BK * 128, 1024)
                                    : make_smem_desc_sw128(sb + k * (UMMA_K * 2), 16, 1024);
            if (leader) {
              if (PAIR == 2) tc_mma_ss_pair(d_tmem, ad, bd, idesc, ((kb - kb0) | k) ? 1u : 0u);
              else tc_mma_ss(d_tmem, ad, bd, idesc, ((kb - kb0) | k) ? 1u : 0u);
            }
          }
          if (leader) {
            if (PAIR == 2) tc_commit_pair(bar_empty + 8 * stage, 3);
            else tc_commit(bar_empty + 8 * stage);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok && leader) {
          if (PAIR == 2) tc_commit_pair(bar_tfull + 8 * buf, 3);
          else tc_commit(bar_tfull + 8 * buf);
        }
      }
      __syncwarp();
    }
  } else if (AG && warp >= 2 + EPI_WARPS) {
    // ------------------------------ pullers (all-gather form) -----------------
    peer::pull_remote_rows(pl, lane, KID_GEMM_PULL);
  } else {
    // ------------------------------ epilogue warps ----------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;
    uint8_t* my_stage = epi_smem + (warp - 2) * 2 * EPI_BUF_BYTES;
    int sbuf = 0;
    int it = 0;
    for (int t = walker; t < num_tiles; t += walkers, ++it) {
      int tm, tn;
      tile_coords(t, m_groups, p.n_tiles, tm, tn, p.m_rot);
      tm = tm * PAIR + rank;
      const int buf = it & 1;
      const uint32_t tphase = (it >> 1) & 1;
      if (!mbar_wait(bar_tfull + 8 * buf, tphase, GEMM_KERNEL_ID, 30)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
      const int gm = tm * BM + row;
      const int n0 = tn * BN;
      uint32_t r[32];
      // reduce-scatter form: the owner of this row tile, and the shift from global to the owner's local rows
      const int owner = p.rs_rows > 0 ? min((tm * BM) / p.rs_rows, p.ar_world - 1) : p.ar_rank;
      const int row_shift = p.rs_rows > 0 ? owner * p.rs_rows : 0;
      bool skip_store = false;
      // a group without rows runs no MMA: its accumulator is undefined and counts as zero
      const bool empty_k = p.mt_kbegin && p.mt_kbegin[min(tm, p.m_tiles - 1)] >= p.mt_kend[min(tm, p.m_tiles - 1)];

      if (p.mode == EPI_ALLREDUCE) {
        // 1. this warp's 32 x 256 partial, as bf16, into the workspace of every OTHER rank (slot of
        //    this rank); the fp32 accumulator stays in TMEM for step 2
        const bool live = tm < p.m_tiles;   // a pair's second CTA may sit past the last row tile
        const size_t slot = (size_t)p.ar_rank * p.ar_rows * p.N;
        const bool push = p.rs_rows == 0 || owner != p.ar_rank;   // an owner keeps its own partial in TMEM
        skip_store = p.rs_rows > 0 && owner != p.ar_rank;
#pragma unroll 1
        for (int c = 0; c < BN / 64 && live && push; ++c) {
          uint8_t* st = my_stage + sbuf * EPI_BUF_BYTES;
          if (lane == 0) tma_store_wait_read<1>();   // an earlier tile's TMA store may still read this buffer
          __syncwarp();
#pragma unroll 1
          for (int h = 0; h < 2; ++h) {
            tmem_ld32(taddr + c * 64 + h * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t a0 = pack_bf16x2(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1]));
              const uint32_t a1 = pack_bf16x2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
              const uint32_t a2 = pack_bf16x2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
              const uint32_t a3 = pack_bf16x2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
              *reinterpret_cast<uint4*>(st + sw128_offset(lane, h * 4 + i)) = make_uint4(a0, a1, a2, a3);
            }
          }
          __syncwarp();
          // 32 rows x 128 bytes: lane l moves the 16-byte pieces l, l+32, ... (8 consecutive lanes = one row)
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int piece = k * 32 + lane;
            const int rr = piece >> 3, ch = piece & 7;
            const int grow = tm * BM + q * 32 + rr;
            const int col = n0 + c * 64 + ch * 8;
            if (grow < p.M && col < p.N) {
              const uint4 v = *reinterpret_cast<const uint4*>(st + sw128_offset(rr, ch));
              const size_t off = slot + (size_t)(grow - row_shift) * p.N + col;
              if (p.rs_rows > 0) {
                *reinterpret_cast<uint4*>((__nv_bfloat16*)p.ar_ws[owner] + off) = v;
              } else {
                for (int d = 0; d < p.ar_world; ++d)
                  if (d != p.ar_rank) *reinterpret_cast<uint4*>((__nv_bfloat16*)p.ar_ws[d] + off) = v;
              }
            }
          }
          __syncwarp();
          sbuf ^= 1;
        }
        // publish the slice to the peers, then wait (bounded) for theirs: ranks run the same tile
        // order, so after the first tile this wait is short
        __threadfence_system();
        __syncwarp();
        const int fidx = (tm * p.n_tiles + tn) * 4 + q;
        const size_t per_rank_flags = (size_t)p.m_tiles * p.n_tiles * 4;
        bool ok_ar = true;
        if (live && lane < p.ar_world && lane != p.ar_rank) {
          if (p.rs_rows == 0) {
            flag_store_release(p.ar_flags[lane] + (size_t)p.ar_rank * per_rank_flags + fidx, p.ar_epoch);
            ok_ar = flag_wait_geq(p.ar_flags[p.ar_rank] + (size_t)lane * per_rank_flags + fidx, p.ar_epoch,
                                  GEMM_KERNEL_ID, 40 + lane);
          } else if (owner != p.ar_rank) {
            if (lane == owner)
              flag_store_release(p.ar_flags[owner] + (size_t)p.ar_rank * per_rank_flags + fidx, p.ar_epoch);
          } else {
            ok_ar = flag_wait_geq(p.ar_flags[p.ar_rank] + (size_t)lane * per_rank_flags + fidx, p.ar_epoch,
                                  GEMM_KERNEL_ID, 40 + lane);
          }
        }
        if (!__all_sync(0xffffffffu, ok_ar)) break;
        // 2. falls into the bf16 store path below, which adds the peers' partials (and C) to the accumulator
      }
      if (skip_store) {
        // reduce-scatter form, a peer owns this tile: the partial has been pushed, nothing is stored here
      } else if (p.mode == EPI_CE_STATS) {
        float mx = -INFINITY, sum = 0.f, tgt = 0.f;
        const int label = (gm < p.M) ? p.labels[gm] : -1;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
          float cmx = -INFINITY;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int col = n0 + c * 32 + j;
            float v = apply_softcap(__uint_as_float(r[j]), p.softcap);
            if (col == label) tgt = v;
            v = (col < p.N && col != p.exclude_index) ? v : -INFINITY;
            r[j] = __float_as_uint(v);
            cmx = fmaxf(cmx, v);
          }
          const float nmx = fmaxf(mx, cmx);
          if (nmx > -INFINITY) {
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) s += __expf(__uint_as_float(r[j]) - nmx);
            sum = sum * __expf(mx - nmx) + s;
            mx = nmx;
          }
        }
        if (gm < p.M) {
          float* o = p.stats + ((size_t)gm * p.n_tiles + tn) * 3;
          o[0] = mx;
          o[1] = sum;
          o[2] = (label >= n0 && label < n0 + BN) ? tgt : 0.f;
        }
      } else if (p.mode == EPI_SWIGLU) {
#pragma unroll 1
        for (int c = 0; c < BN / 128; ++c) {
          uint8_t* st = my_stage + sbuf * EPI_BUF_BYTES;
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
#pragma unroll 1
          for (int h = 0; h < 4; ++h) {
            tmem_ld32(taddr + c * 128 + h * 32, r);
            tmem_ld_wait();
            if (empty_k) {
#pragma unroll
              for (int j = 0; j < 32; ++j) r[j] = 0u;
            }
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float g0 = __uint_as_float(r[4 * j]), u0 = __uint_as_float(r[4 * j + 1]);
              const float g1 = __uint_as_float(r[4 * j + 2]), u1 = __uint_as_float(r[4 * j + 3]);
              o[j] = pack_bf16x2(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
              *reinterpret_cast<uint4*>(st + sw128_offset(lane, h * 2 + i)) =
                  make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmap_d, smem_u32(st), tn * (BN / 2) + c * 64, tm * BM + q * 32);
            tma_store_commit();
          }
          sbuf ^= 1;
        }
      } else if (p.out_fp32) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint8_t* st = my_stage + sbuf * EPI_BUF_BYTES;
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
            if (empty_k) {
#pragma unroll
              for (int j = 0; j < 32; ++j) r[j] = 0u;
            }
          if (p.accumulate && gm < p.M) {
            const float* dp = (const float*)p.c_ptr + (size_t)gm * p.ldc + n0 + c * 32;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (n0 + c * 32 + j < p.N) {
                const float4 v = *reinterpret_cast<const float4*>(dp + j);
                r[j] = __float_as_uint(__uint_as_float(r[j]) + v.x);
                r[j + 1] = __float_as_uint(__uint_as_float(r[j + 1]) + v.y);
                r[j + 2] = __float_as_uint(__uint_as_float(r[j + 2]) + v.z);
                r[j + 3] = __float_as_uint(__uint_as_float(r[j + 3]) + v.w);
              }
            }
          }
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<uint4*>(st + sw128_offset(lane, i)) =
                make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmap_d, smem_u32(st), n0 + c * 32, tm * BM + q * 32);
            tma_store_commit();
          }
          sbuf ^= 1;
        }
      } else {
        // bf16 destination: plain store, accumulate, or cross-entropy logit gradient
        float row_lse = 0.f, row_scale = 0.f;
        int label = -1;
        if (p.mode == EPI_CE_GRAD && gm < p.M) {
          row_lse = p.lse[gm];
          row_scale = p.rowscale[gm];
          label = p.labels[gm];
        }
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint8_t* st = my_stage + sbuf * EPI_BUF_BYTES;
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
#pragma unroll 1
          for (int h = 0; h < 2; ++h) {
            const int cbase = n0 + c * 64 + h * 32;
            tmem_ld32(taddr + c * 64 + h * 32, r);
            tmem_ld_wait();
            if (empty_k) {
#pragma unroll
              for (int j = 0; j < 32; ++j) r[j] = 0u;
            }
            if (p.mode == EPI_CE_GRAD) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int col = cbase + j;
                const float x = __uint_as_float(r[j]);
                float v = x, dcap = 1.f;
                if (p.softcap > 0.f) {
                  const float th = tanhf(x / p.softcap);
                  v = p.softcap * th;
                  dcap = 1.f - th * th;
                }
                float g = (col == p.exclude_index) ? 0.f : __expf(v - row_lse);
                if (col == label) g -= 1.f;
                r[j] = __float_as_uint(g * row_scale * dcap);
              }
            } else if (p.mode == EPI_ALLREDUCE && gm < p.M) {
              // partial sums of the other ranks, landed in this rank's workspace (read past L1: a peer
              // wrote them), plus the optional C operand
              const __nv_bfloat16* ws = (const __nv_bfloat16*)p.ar_ws[p.ar_rank];
              // sources two at a time, all eight 16-byte loads in flight before the first add
              for (int s0 = 0; s0 <= p.ar_world; s0 += 2) {
                uint4 v[2][4];
                bool use[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                  const int s = s0 + u;
                  use[u] = s <= p.ar_world && s != p.ar_rank && !(s == p.ar_world && !p.accumulate);
                  const __nv_bfloat16* dp = (s >= p.ar_world)
                                                ? (const __nv_bfloat16*)p.c_ptr + (size_t)(gm - row_shift) * p.ldc + cbase
                                                : ws + ((size_t)s * p.ar_rows + (gm - row_shift)) * p.N + cbase;
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    v[u][j] = make_uint4(0, 0, 0, 0);
                    if (use[u] && cbase + j * 8 < p.N)
                      asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
                                   : "=r"(v[u][j].x), "=r"(v[u][j].y), "=r"(v[u][j].z), "=r"(v[u][j].w)
                                   : "l"(dp + j * 8));
                  }
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) {
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v[u][j]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                      const float2 f = __bfloat1622float2(h2[e]);   // zeros where nothing was loaded
                      r[j * 8 + 2 * e] = __float_as_uint(__uint_as_float(r[j * 8 + 2 * e]) + f.x);
                      r[j * 8 + 2 * e + 1] = __float_as_uint(__uint_as_float(r[j * 8 + 2 * e + 1]) + f.y);
                    }
                  }
                }
              }
            } else if (p.accumulate && gm < p.M) {
              const __nv_bfloat16* dp = (const __nv_bfloat16*)p.c_ptr + (size_t)gm * p.ldc + cbase;
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                if (cbase + j < p.N) {
                  const uint4 v = *reinterpret_cast<const uint4*>(dp + j);
                  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(h2[e]);
                    r[j + 2 * e] = __float_as_uint(__uint_as_float(r[j + 2 * e]) + f.x);
                    r[j + 2 * e + 1] = __float_as_uint(__uint_as_float(r[j + 2 * e + 1]) + f.y);
                  }
                }
              }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t a0 = pack_bf16x2(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1]));
              const uint32_t a1 = pack_bf16x2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
              const uint32_t a2 = pack_bf16x2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
              const uint32_t a3 = pack_bf16x2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
              *reinterpret_cast<uint4*>(st + sw128_offset(lane, h * 4 + i)) = make_uint4(a0, a1, a2, a3);
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmap_d, smem_u32(st), n0 + c * 64, tm * BM + q * 32 - row_shift);
            tma_store_commit();
          }
          sbuf ^= 1;
        }
      }
      // accumulator buffer is free again
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR == 2) mbar_arrive_cluster((bar_tempty + 8 * buf) & PEER_BIT_MASK);   // CTA 0 counts both
        else mbar_arrive(bar_tempty + 8 * buf);
      }
    }
    if (lane == 0) tma_store_wait_all();
  }

  // common exit: every role arrives here, also after a failed wait
  tc_fence_before();
  if (PAIR == 2) cluster_sync_all();   // neither CTA leaves while the other may still read or signal it
  else __syncthreads();
  if (error_is_set()) {
    // loads that were issued before an abort may still be landing in shared memory
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    if (PAIR == 2) cluster_sync_all();
    else __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    if (PAIR == 2) tmem_dealloc_pair(tmem_base, 512);
    else tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace tdllm

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
using namespace tdllm;

static thread_local long long g_b_rows_override = 0;   // rows of the whole (all groups) B operand
static thread_local long long g_a_m_override = 0;      // extent of A along M when outputs are stacked per group

struct GroupConfig {
  const int* mt_group;
  long long b_group_rows;
  long long a_group_rows;
  long long a_m_total;   // extent of A along M (0 = M)
  const int* mt_kbegin;
  const int* mt_kend;
};

struct ArConfig {
  int world, rank, epoch;
  long long rows;
  void* const* ws;
  void* const* flags;
  int rs_rows;   // > 0: reduce-scatter form, rows per rank
};

// all-gather form: A's rows are sharded over the ranks (`rows` each); bufs[r] = rank r's copy of the whole A
// (symmetric memory, rank r's own rows already in place), ready[r] = rank r's int32[world] flag array
struct AgConfig {
  int world, rank, epoch;
  long long rows;
  void* const* bufs;
  void* const* ready;
  int* counter;
  int* tile_ready;
  int launch_no;
};

static int gemm_impl(const void* A, const void* B, void* D, int M, int N, int K, long long lda,
                     long long ldb, long long ldd, int a_mn_major, int b_mn_major, int out_fp32,
                     int accumulate, int mode, const int* labels, const float* lse,
                     const float* rowscale, float* stats, int exclude_index, float softcap,
                     int max_ctas, const void* c_src, long long ldc, const ArConfig* ar, const GroupConfig* grp,
                     void* stream, const AgConfig* ag = nullptr) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (ar && ar->rs_rows > 0 && (ar->rs_rows % (2 * BM) || (long long)ar->rs_rows * ar->world != M)) {
    tdllm_host::set_last_error("gemm: reduce-scatter epilogue needs M = ranks * rows with rows a multiple of %d", 2 * BM);
    return 1;
  }
  if (ag && (ag->world < 2 || ag->world > AR_MAX_RANKS || ag->rows % (2 * BM) || ag->rows * ag->world != M ||
             a_mn_major || (lda != K) || grp)) {
    tdllm_host::set_last_error("gemm: all-gather form needs 2..%d ranks, a dense K-major A of ranks * rows rows, rows a "
                               "multiple of %d", AR_MAX_RANKS, 2 * BM);
    return 1;
  }
  if (mode == EPI_ALLREDUCE) {
    if (!ar || ar->world < 2 || ar->world > AR_MAX_RANKS || ar->rank < 0 || ar->rank >= ar->world ||
        out_fp32 || (N % 8) || ar->rows < (ar->rs_rows > 0 ? ar->rs_rows : M)) {
      tdllm_host::set_last_error("gemm: all-reduce epilogue needs 2..%d ranks, bf16 output, N %% 8 == 0 and a "
                                 "workspace of at least M rows", AR_MAX_RANKS);
      return 1;
    }
  }
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)A % 16) || ((uintptr_t)B % 16)) {
    tdllm_host::set_last_error("gemm: operands need 16-byte aligned base and row stride");
    return 1;
  }
  if (mode == EPI_SWIGLU && (N % 2 || out_fp32 || accumulate)) {
    tdllm_host::set_last_error("gemm: swiglu epilogue needs even N and a bf16 plain store");
    return 1;
  }
  if (mode == EPI_CE_GRAD && (out_fp32 || accumulate)) {
    tdllm_host::set_last_error("gemm: ce-grad epilogue writes bf16 without accumulate");
    return 1;
  }
  static bool attr_set = false;
  static int max_pairs = 0;   // clusters of two that fit on the device at once (0 = pairs unavailable)
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg<1>::SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemm_bf16_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               Cfg<2>::SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemm_bf16_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               Cfg<1>::SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemm_bf16_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               Cfg<2>::SMEM_BYTES);
    if (e != cudaSuccess) {
      tdllm_host::set_last_error("gemm: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return 2;
    }
    const char* env = getenv("TDLLM_GEMM_PAIR");
    if (!(env && env[0] == '0')) {
      cudaLaunchConfig_t cfg = {};
      cudaLaunchAttribute at;
      at.id = cudaLaunchAttributeClusterDimension;
      at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
      cfg.gridDim = dim3(2 * 74); cfg.blockDim = dim3(GEMM_THREADS);
      cfg.dynamicSmemBytes = Cfg<2>::SMEM_BYTES; cfg.attrs = &at; cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, gemm_bf16_kernel<2, false>, &cfg) == cudaSuccess && n > 0) max_pairs = n;
      else (void)cudaGetLastError();
    }
    attr_set = true;
  }
  // pairs pay off when there are at least two 128-row tiles to share a B tile
  const bool pair = max_pairs > 0 && M > BM;
  CUtensorMap ta, tb, td;
  {
    uint64_t dims[2], strides[1];
    uint32_t box[2];
    const uint64_t a_m = (uint64_t)(g_a_m_override ? g_a_m_override : M);
    if (!a_mn_major) {
      dims[0] = (uint64_t)K; dims[1] = a_m; box[0] = BK; box[1] = BM;
    } else {
      dims[0] = a_m; dims[1] = (uint64_t)K; box[0] = 64; box[1] = BK;
    }
    strides[0] = (uint64_t)lda * 2;
    if (tdllm_host::encode_tmap(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B)) return 3;
    if (!b_mn_major) {
      dims[0] = (uint64_t)K; dims[1] = (uint64_t)(g_b_rows_override ? g_b_rows_override : N);
      box[0] = BK; box[1] = pair ? BN / 2 : BN;
    } else {
      dims[0] = (uint64_t)N; dims[1] = (uint64_t)(g_b_rows_override ? g_b_rows_override : K);
      box[0] = 64; box[1] = BK;
    }
    strides[0] = (uint64_t)ldb * 2;
    if (tdllm_host::encode_tmap(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B)) return 3;
    if (mode == EPI_CE_STATS) {
      td = ta;  // unused by this epilogue
    } else {
      const int n_out = (mode == EPI_SWIGLU) ? N / 2 : N;
      const int esz = out_fp32 ? 4 : 2;
      if (((uint64_t)ldd * esz) % 16 || ((uintptr_t)D % 16)) {
        tdllm_host::set_last_error("gemm: destination needs 16-byte aligned base and row stride");
        return 1;
      }
      // reduce-scatter form: the destination holds the owner's rows only
      dims[0] = (uint64_t)n_out; dims[1] = (uint64_t)((ar && ar->rs_rows > 0) ? ar->rs_rows : M);
      box[0] = out_fp32 ? 32 : 64; box[1] = 32;
      strides[0] = (uint64_t)ldd * esz;
      if (tdllm_host::encode_tmap(&td, out_fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                                  2, D, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return 3;
    }
  }
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major;
  p.mode = mode; p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.m_tiles = (M + BM - 1) / BM; p.n_tiles = (N + BN - 1) / BN;
  p.c_ptr = c_src ? c_src : D;
  p.ldc = c_src ? ldc : ldd;
  if (accumulate && ((uintptr_t)p.c_ptr % 16 || (p.ldc * (out_fp32 ? 4 : 2)) % 16)) {
    tdllm_host::set_last_error("gemm: accumulate source needs 16-byte aligned base and row stride");
    return 1;
  }
  p.labels = labels; p.lse = lse; p.rowscale = rowscale; p.stats = stats;
  p.exclude_index = exclude_index; p.softcap = softcap;
  p.mt_group = grp ? grp->mt_group : nullptr; p.b_group_rows = grp ? grp->b_group_rows : 0;
  p.a_group_rows = grp ? grp->a_group_rows : 0;
  p.mt_kbegin = grp ? grp->mt_kbegin : nullptr; p.mt_kend = grp ? grp->mt_kend : nullptr;
  p.ar_world = 0; p.ar_rank = 0; p.ar_epoch = 0; p.ar_rows = 0; p.ar_out = D; p.ar_ldd = ldd;
  for (int i = 0; i < AR_MAX_RANKS; ++i) { p.ar_ws[i] = nullptr; p.ar_flags[i] = nullptr; }
  p.m_rot = 0; p.rs_rows = 0; p.ag_rows = 0; p.ag_rank = 0;
  if (mode == EPI_ALLREDUCE) {
    p.ar_world = ar->world; p.ar_rank = ar->rank; p.ar_epoch = ar->epoch; p.ar_rows = ar->rows;
    for (int i = 0; i < ar->world; ++i) { p.ar_ws[i] = ar->ws[i]; p.ar_flags[i] = (int*)ar->flags[i]; }
    if (ar->rs_rows > 0) {
      // start at the rows of the next rank, reach the own rows last (see the file header)
      p.rs_rows = ar->rs_rows;
      p.m_rot = (int)(((long long)((ar->rank + 1) % ar->world) * ar->rs_rows) / (BM * (pair ? 2 : 1)));
    }
  }
  peer::PullPlan pl;
  memset(&pl, 0, sizeof(pl));
  if (ag) {
    p.ag_rows = (int)ag->rows; p.ag_rank = ag->rank;
    p.m_rot = (int)(((long long)ag->rank * ag->rows) / (BM * (pair ? 2 : 1)));   // own rows first
    const long long row_bytes = (long long)K * 2;
    long long total = 0;
    pl.nseg = ag->world - 1;
    for (int sgm = 0; sgm < ag->world - 1; ++sgm) {
      const int peer_rank = (ag->rank + 1 + sgm) % ag->world;
      pl.src[sgm] = (const uint4*)((const char*)ag->bufs[peer_rank] + (long long)peer_rank * ag->rows * row_bytes);
      pl.ready[sgm] = (const int*)ag->ready[ag->rank] + peer_rank;
      pl.seg_begin[sgm] = total;
      pl.dst_begin[sgm] = (long long)peer_rank * ag->rows;
      total += ag->rows;
    }
    for (int sgm = ag->world - 1; sgm <= peer::MAX_PEERS; ++sgm) pl.seg_begin[sgm] = total;
    pl.dst = (uint4*)ag->bufs[ag->rank];
    pl.counter = ag->counter;
    pl.tile_ready = ag->tile_ready;
    pl.n_rows = total;
    pl.want = ag->epoch;
    pl.row_vec16 = (int)(row_bytes / 16);
    pl.tile_target = ag->launch_no * (peer::TILE_ROWS / peer::PULL_ROWS);
    if (cudaMemsetAsync(ag->counter, 0, sizeof(int), (cudaStream_t)stream) != cudaSuccess) {
      tdllm_host::set_last_error("gemm: clearing the claim counter failed");
      return 5;
    }
  }
  cudaError_t e;
  if (pair) {
    const int tiles = ((p.m_tiles + 1) / 2) * p.n_tiles;
    int pairs = max_ctas > 0 ? (max_ctas / 2 > 0 ? max_ctas / 2 : 1) : max_pairs;
    if (pairs > max_pairs) pairs = max_pairs;
    if (pairs > tiles) pairs = tiles;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(ag ? GEMM_THREADS_AG : GEMM_THREADS);
    cfg.dynamicSmemBytes = Cfg<2>::SMEM_BYTES; cfg.stream = (cudaStream_t)stream;
    cfg.attrs = &at; cfg.numAttrs = 1;
    if (ag) e = cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<2, true>, ta, tb, td, p, pl);
    else e = cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<2, false>, ta, tb, td, p, pl);
  } else {
    const int tiles = p.m_tiles * p.n_tiles;
    int ctas = max_ctas > 0 ? max_ctas : tdllm_num_sms();
    if (ctas > tiles) ctas = tiles;
    if (ag)
      gemm_bf16_kernel<1, true><<<ctas, GEMM_THREADS_AG, Cfg<1>::SMEM_BYTES, (cudaStream_t)stream>>>(ta, tb, td, p, pl);
    else
      gemm_bf16_kernel<1, false><<<ctas, GEMM_THREADS, Cfg<1>::SMEM_BYTES, (cudaStream_t)stream>>>(ta, tb, td, p, pl);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    tdllm_host::set_last_error("gemm launch: %s", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}

extern "C" int tdllm_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K,
                               long long lda, long long ldb, long long ldd, int a_mn_major,
                               int b_mn_major, int out_fp32, int accumulate, int mode,
                               const int* labels, const float* lse, const float* rowscale,
                               float* stats, int exclude_index, float softcap, int max_ctas,
                               const void* c_src, long long ldc, void* stream) {
  if (mode == EPI_ALLREDUCE) {
    tdllm_host::set_last_error("gemm: the all-reduce epilogue is reached through tdllm_gemm_allreduce_bf16");
    return 1;
  }
  return gemm_impl(A, B, D, M, N, K, lda, ldb, ldd, a_mn_major, b_mn_major, out_fp32, accumulate, mode,
                   labels, lse, rowscale, stats, exclude_index, softcap, max_ctas, c_src, ldc, nullptr, nullptr, stream);
}

// D = sum over the `world` ranks of (A_r * B_r) (+ C): every rank calls this with its K-slice of A and B.
// ws[d] / flags[d]: rank d's workspace ([world][ws_rows][N] bf16) and flag array ([world][m_tiles*n_tiles*4]
// int32, zero at allocation) as mapped into this process; `epoch` must grow from call to call on one
// workspace, and two workspaces must alternate between consecutive calls (a rank may start the next call
// while a peer still sums the previous one).
extern "C" int tdllm_gemm_allreduce_bf16(const void* A, const void* B, void* D, int M, int N, int K,
                                         long long lda, long long ldb, long long ldd, int a_mn_major,
                                         int b_mn_major, const void* c_src, long long ldc, int world,
                                         int rank, int epoch, long long ws_rows, void* const* ws,
                                         void* const* flags, int max_ctas, void* stream) {
  ArConfig ar{world, rank, epoch, ws_rows, ws, flags, 0};
  return gemm_impl(A, B, D, M, N, K, lda, ldb, ldd, a_mn_major, b_mn_major, 0, c_src != nullptr, EPI_ALLREDUCE,
                   nullptr, nullptr, nullptr, nullptr, -1, 0.f, max_ctas, c_src, ldc, &ar, nullptr, stream);
}

// GEMM -> reduce-scatter over peer memory: D_local[M / world, N] = rows [rank * M / world, ...) of
// sum over ranks of (A_r * B_r) (+ C_local, the same rows of a residual). Same workspace contract as
// tdllm_gemm_allreduce_bf16, with ws_rows >= M / world (a workspace keeps only the owner's rows).
extern "C" int tdllm_gemm_reduce_scatter_bf16(const void* A, const void* B, void* D_local, int M, int N, int K,
                                              long long lda, long long ldb, long long ldd, int a_mn_major,
                                              int b_mn_major, const void* c_local, long long ldc, int world,
                                              int rank, int epoch, long long ws_rows, void* const* ws,
                                              void* const* flags, int max_ctas, void* stream) {
  if (world < 2 || M % world || ws_rows < M / world) {
    tdllm_host::set_last_error("gemm_reduce_scatter: M must divide by the ranks and the workspace hold M / ranks rows");
    return 1;
  }
  ArConfig ar{world, rank, epoch, ws_rows, ws, flags, M / world};
  // the destination tensor map spans the owner's rows only: stores of other tiles never happen
  return gemm_impl(A, B, D_local, M, N, K, lda, ldb, ldd, a_mn_major, b_mn_major, 0, c_local != nullptr,
                   EPI_ALLREDUCE, nullptr, nullptr, nullptr, nullptr, -1, 0.f, max_ctas, c_local, ldc, &ar, nullptr,
                   stream);
}

// all-gather -> GEMM over peer memory: D[M, N] = A * B where A's rows are sharded over the ranks. bufs[r]: rank
// r's [M, K] bf16 copy of A in symmetric memory as mapped here; this rank's own rows [rank * M / world, ...) are
// already in bufs[rank]; the other rows are pulled inside the kernel once the owners have stored `epoch` into
// slot `owner` of every rank's ready array (tdllm_symm_signal after they wrote their rows). counter: one int32,
// zeroed here; tile_ready: one int32 per 128-row tile of A, zeroed once by the caller, `launch_no` = 1-based
// number of this call on those counters. mode: EPI_STORE or EPI_SWIGLU.
extern "C" int tdllm_gemm_allgather_bf16(void* const* bufs, const void* B, void* D, int M, int N, int K,
                                         long long ldb, long long ldd, int b_mn_major, int mode, int world,
                                         int rank, int epoch, void* const* ready, int* counter, int* tile_ready,
                                         int launch_no, int max_ctas, void* stream) {
  if (mode != EPI_STORE && mode != EPI_SWIGLU) {
    tdllm_host::set_last_error("gemm_allgather: only the store and SwiGLU epilogues");
    return 1;
  }
  if (world < 2 || M % world) {
    tdllm_host::set_last_error("gemm_allgather: M must divide by the ranks");
    return 1;
  }
  AgConfig ag{world, rank, epoch, M / world, bufs, ready, counter, tile_ready, launch_no};
  return gemm_impl(bufs[rank], B, D, M, N, K, K, ldb, ldd, 0, b_mn_major, 0, 0, mode, nullptr, nullptr, nullptr,
                   nullptr, -1, 0.f, max_ctas, nullptr, 0, nullptr, nullptr, stream, &ag);
}

// Grouped product over row tiles (experts): tile tm of M uses the slice `mt_group[tm]` of B (B's row coordinate
// shifted by mt_group[tm] * b_group_rows, A's M coordinate shifted back by mt_group[tm] * a_group_rows with
// A spanning a_m_total along M; pass null / 0 for none) and runs over K blocks [mt_kbegin[tm], mt_kend[tm])
// (64-element blocks; null = all of K). The tables live on the device, one entry per 128-row tile of M; both
// tiles of a 256-row pair must agree. `b_rows_total`: rows of the whole B operand (all groups).
// mode: EPI_STORE or EPI_SWIGLU.
extern "C" int tdllm_gemm_grouped_bf16(const void* A, const void* B, void* D, int M, int N, int K,
                                       long long lda, long long ldb, long long ldd, int a_mn_major,
                                       int b_mn_major, int accumulate, int mode, const int* mt_group,
                                       long long b_group_rows, long long b_rows_total, long long a_group_rows,
                                       long long a_m_total, const int* mt_kbegin, const int* mt_kend,
                                       int max_ctas, void* stream) {
  if (mode != EPI_STORE && mode != EPI_SWIGLU) {
    tdllm_host::set_last_error("gemm_grouped: only the store and SwiGLU epilogues are grouped");
    return 1;
  }
  GroupConfig g{mt_group, b_group_rows, a_group_rows, a_m_total, mt_kbegin, mt_kend};
  g_b_rows_override = b_rows_total;
  g_a_m_override = a_m_total;
  const int rc = gemm_impl(A, B, D, M, N, K, lda, ldb, ldd, a_mn_major, b_mn_major, 0, accumulate, mode, nullptr,
                           nullptr, nullptr, nullptr, -1, 0.f, max_ctas, nullptr, 0, nullptr, &g, stream);
  g_b_rows_override = 0;
  g_a_m_override = 0;
  return rc;
}

extern "C" int tdllm_gemm_flag_count(int M, int N) { return ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * 4; }

extern "C" int tdllm_gemm_n_tiles(int N) { return (N + BN - 1) / BN; }
