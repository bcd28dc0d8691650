// C ABI of the sm_100a kernel library (libtdllm_kernels.so). Python binds it with ctypes;
// every function takes raw device pointers and a cudaStream_t passed as void*.
// Functions return 0 on success; tdllm_last_error() describes a non-zero return.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- runtime -------------------------------------------------------------
const char* tdllm_last_error(void);
int tdllm_num_sms(void);
// copies the 8-word device error record to out (synchronises the device)
int tdllm_get_error(int* out8);
int tdllm_clear_error(void);
// budget of every bounded device-side wait, in nanoseconds (default 2 s)
int tdllm_set_wait_timeout_ns(unsigned long long ns);
// test hook: a kernel that waits on an mbarrier nobody arrives on; must come back with
// ERR_WAIT_TIMEOUT in the error record and leave the context usable
int tdllm_test_wait_timeout(void* stream);

// ---- GEMM ----------------------------------------------------------------
int tdllm_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, long long lda,
                    long long ldb, long long ldd, int a_mn_major, int b_mn_major, int out_fp32,
                    int accumulate, int mode, const int* labels, const float* lse,
                    const float* rowscale, float* stats, int exclude_index, float softcap,
                    int max_ctas, const void* c_src, long long ldc, void* stream);
int tdllm_gemm_n_tiles(int N);

// Row-parallel product with the all-reduce done in the epilogue over peer memory: D = sum_r A_r * B_r (+ C).
// ws[d] / flags[d]: rank d's workspace ([world][ws_rows][N] bf16) and flags ([world][tdllm_gemm_flag_count(M,N)]
// int32, zeroed once) as mapped here. `epoch` grows per call on one workspace; alternate two workspaces.
int tdllm_gemm_allreduce_bf16(const void* A, const void* B, void* D, int M, int N, int K, long long lda,
                              long long ldb, long long ldd, int a_mn_major, int b_mn_major,
                              const void* c_src, long long ldc, int world, int rank, int epoch,
                              long long ws_rows, void* const* ws, void* const* flags, int max_ctas,
                              void* stream);
int tdllm_gemm_flag_count(int M, int N);
// Sequence-parallel forms (see gemm_sm100.cu): GEMM -> reduce-scatter and all-gather -> GEMM in one kernel each.
int tdllm_gemm_reduce_scatter_bf16(const void* A, const void* B, void* D_local, int M, int N, int K, long long lda,
                                   long long ldb, long long ldd, int a_mn_major, int b_mn_major,
                                   const void* c_local, long long ldc, int world, int rank, int epoch,
                                   long long ws_rows, void* const* ws, void* const* flags, int max_ctas,
                                   void* stream);
int tdllm_gemm_allgather_bf16(void* const* bufs, const void* B, void* D, int M, int N, int K, long long ldb,
                              long long ldd, int b_mn_major, int mode, int world, int rank, int epoch,
                              void* const* ready, int* counter, int* tile_ready, int launch_no, int max_ctas,
                              void* stream);

// Cross-rank finish of vocab-parallel CE statistics over peer memory: lse = logsumexp over ranks of the
// shard lse, target = sum of the shard target logits. ws[d]: [world][rows_cap][2] fp32, flags[d]:
// [world][tdllm_ce_exchange_blocks(rows_cap)] int32 (zeroed once); growing epoch, two alternating workspaces.
int tdllm_ce_exchange(const float* stats, int M, int n_tiles, void* const* ws, void* const* flags, int rank,
                      int world, int epoch, long long rows_cap, float* lse_out, float* tgt_out, void* stream);
int tdllm_ce_exchange_blocks(long long rows_cap);

// Grouped product (experts): per 128-row tile of M a slice of B (row coordinate shifted by mt_group[tm] *
// b_group_rows) and/or a range of 64-element K blocks; tables on the device, null = not used.
int tdllm_gemm_grouped_bf16(const void* A, const void* B, void* D, int M, int N, int K, long long lda,
                            long long ldb, long long ldd, int a_mn_major, int b_mn_major, int accumulate,
                            int mode, const int* mt_group, long long b_group_rows, long long b_rows_total,
                            long long a_group_rows, long long a_m_total, const int* mt_kbegin,
                            const int* mt_kend, int max_ctas, void* stream);

// ---- normalisation / rotary / activation ---------------------------------
int tdllm_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out,
                      float* rstd, int rows, int H, float eps, void* stream);
int tdllm_rmsnorm_bwd_parts(void);
int tdllm_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd,
                      const void* dres_in, void* dx, void* dw, int dw_fp32, int dw_accumulate,
                      float* scratch, int rows, int H, void* stream);
int tdllm_qk_norm_rope_fwd(const void* in, void* out, const int* pos, const float* inv_freq,
                           const void* qw, const void* kw, int rows, int Hq, int Hkv, int D,
                           float eps, void* stream);
int tdllm_qk_bwd_parts(void);
int tdllm_qk_norm_rope_bwd(const void* dout, const void* in_raw, void* din, const int* pos,
                           const float* inv_freq, const void* qw, const void* kw, void* dqw,
                           void* dkw, int dw_fp32, int dw_accumulate, float* scratch, int rows,
                           int Hq, int Hkv, int D, float eps, void* stream);
int tdllm_swiglu_fwd(const void* gu, void* out, long long rows, int inter, void* stream);
int tdllm_swiglu_bwd(const void* dy, const void* gu, void* dgu, long long rows, int inter,
                     void* stream);

// ---- wide-head attention: the masked softmax between the tensor-core products ----
// S fp32 [R, N] (row stride lds) -> P bf16 [R, N] (row stride ldp), lse [R]. Row r uses the mask entries of
// query (r % rows_per_head).
int tdllm_wide_softmax(const void* S, void* P, void* lse, const int* q_lo, const int* q_hi, const int* q_grp,
                       const int* k_code, long long R, int rows_per_head, int N, long long lds, long long ldp,
                       float scale, void* stream);
// P = exp(S*scale - lse) under the mask, dS = P * (dP - delta) * scale (both bf16, row stride ldp).
int tdllm_wide_softmax_bwd(const void* S, const void* dP, void* P, void* dS, const void* lse,
                           const void* delta, const int* q_lo, const int* q_hi, const int* q_grp,
                           const int* k_code, long long R, int rows_per_head, int N, long long lds,
                           long long ldp, float scale, void* stream);

// ---- optimizer / loss reductions / attention-state merge -------------------
int tdllm_sumsq_bf16(const void* g, long long n, float* out, void* stream);
int tdllm_adamw(float* master, float* m, float* v, const void* grad, void* param, long long n,
                float lr, float beta1, float beta2, float eps, float wd, int step,
                float grad_scale, const float* sumsq, float max_norm, void* stream);
int tdllm_adamw_f32grad(float* master, float* m, float* v, const float* grad, void* param, long long n,
                        float lr, float beta1, float beta2, float eps, float wd, int step,
                        float grad_scale, const float* sumsq, float max_norm, void* stream);
int tdllm_ce_finalize(const float* stats, int M, int n_tiles, const int* labels,
                      const float* weights, float* lse_out, float* loss_rows, float* out2,
                      void* stream);
int tdllm_kl_rows(const float* student_logits, const float* teacher_logits, const float* rowscale,
                  float* loss_rows, void* dlogits_bf16, int rows, int V, long long ld, void* stream);
int tdllm_attn_merge(float* num, float* mrun, float* lrun, const void* o_s, const float* lse_s,
                     long long nrh, int D, int initial, void* stream);
int tdllm_attn_merge_finalize(const float* num, const float* mrun, const float* lrun, void* out,
                              float* lse, long long nrh, int D, void* stream);
int tdllm_attn_merge_bwd(const void* go, const void* out, const float* lse, const void* o_s,
                         const float* lse_s, void* go_s, float* dlse_s, long long nrh, int D,
                         void* stream);

// ---- block-diffusion attention (head_dim 128) ------------------------------
int tdllm_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int nq,
                   int nk, int Hq, int Hkv, long long ldq, long long ldk, long long ldv,
                   long long ldo, const int* q_lo, const int* q_hi, const int* q_grp,
                   const int* k_code, const int* tile_ptr, const int* tile_idx, const int* order,
                   int n_qtiles, float scale, void* stream);

// Context-sharded forward: keys = this rank's rows, then the peers' clean K|V rows, pulled from the peers'
// staged rows into kv_rem by two extra warps per CTA while the tiles of local keys run (see
// attention_fwd_sm100.cu for the argument contract).
int tdllm_attn_fwd_csbp(const void* q, const void* k_loc, const void* v_loc, void* kv_rem, void* o, float* lse,
                        int nq, int nk_loc, long long n_rem, int Hq, int Hkv, long long ldq, long long ldk,
                        long long ldv, long long ldo, const int* q_lo, const int* q_hi, const int* q_grp,
                        const int* k_code, const int* tile_ptr, const int* tile_idx, const int* order,
                        int n_qtiles, float scale, void* const* staging, void* const* ready,
                        const long long* counts, int rank, int world, int ready_epoch, int* counter,
                        int* tile_ready, int launch_no, void* stream);

// dq/dk/dv may point into one packed [rows, (Hq+2Hkv)*128] buffer; delta is fp32 scratch
// [2, Hq, n_qtiles*128]; f_* lists are per query tile, b_* lists per key tile.
int tdllm_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                   void* dq, void* dk, void* dv, const float* lse, float* delta, int nq, int nk,
                   int Hq, int Hkv, long long ldq, long long ldk, long long ldv, long long ldo,
                   long long lddo, long long lddq, long long lddk, long long lddv,
                   const int* q_lo, const int* q_hi, const int* q_grp, const int* k_code,
                   const int* f_ptr, const int* f_idx, const int* f_order, const int* b_ptr,
                   const int* b_idx, const int* b_order, int n_qtiles, int n_ktiles, float scale,
                   void* stream);

// One-pass backward (five tensor-core products per tile pair instead of seven). dQ, dK and dV are
// summed in `acc`, fp32 scratch of n_qtiles*128*Hq*128 + 2*n_ktiles*128*Hkv*128 floats that this call
// zeroes, then cast. Work item c*n_ktiles + kt = the query tiles of chunk c that see key tile kt
// (w_ptr: one entry per item plus one; w_order: the n_work non-empty items, chunk by chunk).
int tdllm_attn_bwd_fused(const void* q, const void* k, const void* v, const void* o, const void* dout,
                         void* dq, void* dk, void* dv, const float* lse, float* delta, float* acc,
                         int nq, int nk, int Hq, int Hkv, long long ldq, long long ldk, long long ldv,
                         long long ldo, long long lddo, long long lddq, long long lddk,
                         long long lddv, const int* q_lo, const int* q_hi, const int* q_grp,
                         const int* k_code, const int* w_ptr, const int* w_idx, const int* w_order,
                         int n_work, int n_qtiles, int n_ktiles, float scale, void* stream);

// Context-sharded one-pass backward: gradients of the peers' key rows are added to the owners' fp32
// accumulators through peer memory from the kernel's epilogue (see attention_bwd_host.cu).
int tdllm_attn_bwd_fused_csbp(const void* q, const void* k_loc, const void* v_loc, const void* kv_rem,
                              const void* o, const void* dout, void* dq, void* dk, void* dv, const float* lse,
                              float* delta, float* dq_acc, void* const* acc_dk, void* const* acc_dv,
                              long long acc_rows, void* next_acc, long long next_bytes, int nq, int nk_loc,
                              long long n_rem, int Hq, int Hkv, long long ldq, long long ldk, long long ldv,
                              long long ldo, long long lddo, long long lddq, long long lddk, long long lddv,
                              const int* q_lo, const int* q_hi, const int* q_grp, const int* k_code,
                              const int* w_ptr, const int* w_idx, const int* w_order, int n_work, int n_qtiles,
                              int n_ktiles, float scale, const long long* counts, const long long* dst_row0,
                              void* const* flags, int rank, int world, int epoch, void* stream);

// ---- peer memory and the fused ZeRO step -----------------------------------
int tdllm_symm_alloc(long long bytes, void** out);
int tdllm_symm_free(void* p);
int tdllm_ipc_get_handle(void* p, void* handle_out64);
int tdllm_ipc_open(const void* handle64, void** out);
int tdllm_ipc_close(void* p);
int tdllm_symm_barrier(void* const* flag_ptrs, int rank, int world, int epoch, void* stream);
// the arriving half of the barrier alone (consumers wait inside their own kernels)
int tdllm_symm_signal(void* const* flag_ptrs, int rank, int world, int epoch, void* stream);
int tdllm_zero_fused_step(void* const* grad_ptrs, void* const* param_ptrs, void* const* sumsq_ptrs,
                          void* const* flag_ptrs, float* master, float* m, float* v, int rank,
                          int world, long long start, long long n, long long decay_end, float lr,
                          float beta1, float beta2, float eps, float wd, int step, float grad_scale,
                          float max_norm, float* norm_out, int epoch, float* reduced, void* stream);

// Parameter sharding: materialise a unit from the ranks' bf16 shards / reduce a unit's bf16 gradients into this
// rank's fp32 shard (see comm.cu).
int tdllm_fsdp_gather(void* const* shard_ptrs, long long shard_off, long long shard_len, long long unit_len,
                      int rank, int world, void* out, void* stream);
int tdllm_fsdp_reduce(void* const* grad_ptrs, long long my_off, long long n, int rank, int world, float* out,
                      int accumulate, void* stream);

int tdllm_kv_gather(void* const* staging_ptrs, void* const* flag_ptrs, const long long* counts, int rank,
                    int world, int row_bytes, void* out, int epoch, void* stream);
int tdllm_kv_scatter_reduce(void* const* partial_ptrs, void* const* flag_ptrs, const long long* counts,
                            int rank, int world, int row_bytes, void* out, int epoch, void* stream);

// ---- expert-parallel dispatch / combine over peer memory (moe_dispatch.cu) -------------
int tdllm_ep_counts_exchange(const int* my_counts, void* const* tabs, void* const* flags, int rank, int world,
                             int E, int epoch, void* stream);
int tdllm_ep_dispatch(const void* x, const int* experts, const float* scale, const long long* base, int* counters,
                      const int* pos_in, int* pos_out, void* const* slabs, long long rows, int k, int H,
                      int e_local, long long cap_rows, int world, void* stream);
int tdllm_ep_zero_pad_rows(void* slab, const long long* begin, const long long* count, int e_local, int H,
                           void* stream);
int tdllm_ep_combine(void* out, const float* weights, const int* experts, const int* pos, void* const* slabs,
                     void* keep, long long rows, int k, int H, int e_local, int world, void* stream);
int tdllm_ep_weight_grad(const void* dout, const void* y, float* dw, long long rows, int k, int H, void* stream);

// ---- gated delta rule: chunk-to-chunk state scan ---------------------------------
// All tensors fp32 and contiguous. ut/o/u: [BH, N, C, Dv]; w/qi/ko: [BH, N, C, Dk]; qk: [BH, N, C, C];
// total: [BH, N]; s0 (may be null)/s_final: [BH, Dk, Dv]; states: [BH, N, Dk, Dv] (state in front of each chunk).
// C <= 64, Dk <= 128 and a multiple of 8, Dv a multiple of 32.
int tdllm_gdn_scan_fwd(const float* ut, const float* w, const float* qk, const float* qi, const float* ko,
                       const float* total, const float* s0, float* o, float* u, float* states, float* s_final,
                       int BH, int N, int C, int Dk, int Dv, void* stream);
// d_states / d_sfinal may be null. d_w, d_qi, d_ko: [BH, N, Dv/32, C, Dk]; d_qk: [BH, N, Dv/32, C, C];
// d_total: [BH, N, Dv/32]: partial sums per slice of 32 value columns, to be summed over that axis.
int tdllm_gdn_scan_bwd(const float* w, const float* qk, const float* qi, const float* ko, const float* total,
                       const float* states, const float* u, const float* d_o, const float* d_states,
                       const float* d_sfinal, float* d_ut, float* d_w, float* d_qk, float* d_qi, float* d_ko,
                       float* d_total, float* d_s0, int BH, int N, int C, int Dk, int Dv, void* stream);

// ---- noising ---------------------------------------------------------------
int tdllm_corrupt(const long long* x0, const float* t, const unsigned char* eligible, long long* xt,
                  long long* labels, int B, int L, int block_size, int views, int shift_labels,
                  long long mask_id, unsigned long long seed, unsigned long long offset, void* stream);

#ifdef __cplusplus
}
#endif
