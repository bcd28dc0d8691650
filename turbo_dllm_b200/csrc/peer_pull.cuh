// In-kernel pull of rows that live in other GPUs' memory into a buffer of this GPU, shared by the kernels that
// fuse an all-gather with their tensor-core work (context-sharded attention, sequence-parallel GEMM).
//
// The remote rows form segments, one per peer, in the order this rank visits its peers (rank+1, rank+2, ... so
// that no owner serves every puller at once). Puller warps of all resident CTAs claim 16-row pieces from a
// shared counter, copy them with plain 16-byte peer loads (never TMA, never a library copy) and count finished
// claims per 128-row tile of the destination; a consumer waits (bounded) until a tile's count says that all its
// rows have arrived and then reads the tile from local memory with TMA. Every remote row crosses NVLink once.
#pragma once
#include "common.cuh"

namespace tdllm {
namespace peer {

constexpr int MAX_PEERS = 16;
constexpr int PULL_ROWS = 16;       // rows per claim; a 128-row tile is complete after 8 claims
constexpr int TILE_ROWS = 128;

struct PullPlan {
  const uint4* src[MAX_PEERS];        // segment s: first row of the peer's rows (peer memory)
  const int* ready[MAX_PEERS];        // segment s: word in THIS rank's flag array that the peer sets to `want`
  long long seg_begin[MAX_PEERS + 1]; // first remote row of segment s (prefix sums of the peers' row counts)
  long long dst_begin[MAX_PEERS];     // row of the destination buffer that takes the segment's first row
  uint4* dst;                         // destination rows, row_vec16 16-byte pieces each, in this GPU's memory
  int* counter;                       // claim counter, zero at launch
  int* tile_ready;                    // finished claims per 128-row tile of the destination, cumulative over launches
  long long n_rows;                   // remote rows
  int nseg, want, row_vec16;
  int nlt, nrt;                       // attention: local and remote key tiles
  int tile_target;                    // count a tile has reached when all its rows of this launch are in
};

__device__ __forceinline__ uint4 ld_peer16(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}
// bounded wait on a counter in this GPU's memory that other CTAs of the launch advance
__device__ __forceinline__ bool count_wait_geq(const int* flag, int want, int kernel_id, int detail) {
  const unsigned long long t0 = globaltimer_ns();
  const unsigned long long budget = g_tdllm_timeout_ns;
#pragma unroll 1
  while (true) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= want) return true;
    if (error_is_set()) return false;
    if (globaltimer_ns() - t0 > budget) {
      set_error(ERR_WAIT_TIMEOUT, kernel_id, detail);
      return false;
    }
    __nanosleep(32);
  }
}

// One puller warp: claims 16-row pieces of the remote rows until none is left. Segment boundaries and
// destination offsets must be multiples of 16 rows for a piece to count toward one tile only, or else the
// caller sizes `tile_ready` by remote-row tiles (attention) where a piece may straddle segments.
__device__ __forceinline__ void pull_remote_rows(const PullPlan& pl, int lane, int kernel_id) {
  const int n_claims = (int)((pl.n_rows + PULL_ROWS - 1) / PULL_ROWS);
  const int tile_claims = TILE_ROWS / PULL_ROWS;
  const int padded_claims = (n_claims + tile_claims - 1) / tile_claims * tile_claims;
  uint32_t seen = 0;   // segments whose owner has been seen ready
  // every pass takes one claim off the shared counter: at most padded_claims + 1 passes per warp
#pragma unroll 1
  for (int pass = 0; pass <= padded_claims; ++pass) {
    int c = 0;
    if (lane == 0) c = atomicAdd(pl.counter, 1);
    c = __shfl_sync(0xffffffffu, c, 0);
    if (c >= padded_claims) break;
    long long row = (long long)c * PULL_ROWS;
    const long long row_end = min(row + PULL_ROWS, pl.n_rows);
    long long first_dst = -1;
    bool ok = true;
#pragma unroll 1
    while (row < row_end) {
      int s = 0;
      while (s + 1 < pl.nseg && row >= pl.seg_begin[s + 1]) ++s;
      const long long run_end = min(row_end, pl.seg_begin[s + 1]);
      if (!((seen >> s) & 1u)) {
        int good = 1;
        if (lane == 0) good = flag_wait_geq(pl.ready[s], pl.want, kernel_id, s) ? 1 : 0;
        if (!__shfl_sync(0xffffffffu, good, 0)) { ok = false; break; }
        seen |= 1u << s;
      }
      const long long drow = pl.dst_begin[s] + (row - pl.seg_begin[s]);
      // checked builds: the claim must lie inside its segment and map to a row of the destination buffer
      if (!TD_CHECKED(s < pl.nseg && row >= pl.seg_begin[s] && run_end <= pl.seg_begin[s + 1] && drow >= 0,
                      kernel_id, 0x100 + s)) {
        ok = false;
        break;
      }
      if (first_dst < 0) first_dst = drow;
      const uint4* src = pl.src[s] + (row - pl.seg_begin[s]) * pl.row_vec16;
      uint4* dst = pl.dst + drow * pl.row_vec16;
      const long long n = (run_end - row) * pl.row_vec16;
#pragma unroll 1
      for (long long i = lane; i < n; i += 32 * 8) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (i + u * 32 < n) v[u] = ld_peer16(src + i + u * 32);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (i + u * 32 < n) dst[i + u * 32] = v[u];
      }
      row = run_end;
    }
    if (!ok) break;   // the error record is set: every waiter of the launch leaves its loop
    // the rows are read by TMA (async proxy) in other CTAs: order them before the count
    fence_proxy_async_global();
    __threadfence();
    __syncwarp();
    // pieces past the last remote row (padding of the last tile) count toward that tile
    const long long tile = first_dst >= 0 ? first_dst / TILE_ROWS
                                          : (pl.dst_begin[pl.nseg - 1] + pl.n_rows - 1 - pl.seg_begin[pl.nseg - 1]) / TILE_ROWS;
    if (lane == 0)
      asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(pl.tile_ready + tile) : "memory");
  }
}

}  // namespace peer
}  // namespace tdllm
