// Host entry points of the attention backward: row statistics (delta·scale, lse·log2e) into the
// caller's scratch [2, Hq, n_qtiles*128], then either the dQ kernel (per query tile) and the
// dK/dV kernel (per key tile), or the one-pass kernel (per key tile) that also accumulates dQ
// in an fp32 scratch, followed by a cast.
#include <cstring>
#include "attention_bwd_dq_sm100.cu"
#include "attention_bwd_dkv_sm100.cu"
#include "attention_bwd_fused_sm100.cu"

using namespace tdllm;

extern "C" int tdllm_attn_bwd(const void* q, const void* k, const void* v, const void* o,
                              const void* dout, void* dq, void* dk, void* dv, const float* lse,
                              float* delta, int nq, int nk, int Hq, int Hkv, long long ldq,
                              long long ldk, long long ldv, long long ldo, long long lddo,
                              long long lddq, long long lddk, long long lddv, const int* q_lo,
                              const int* q_hi, const int* q_grp, const int* k_code,
                              const int* f_ptr, const int* f_idx, const int* f_order,
                              const int* b_ptr, const int* b_idx, const int* b_order,
                              int n_qtiles, int n_ktiles, float scale, void* stream) {
  if (nq <= 0 || nk <= 0) return 0;
  if (Hq % Hkv || (Hq / Hkv) % 2) {
    tdllm_host::set_last_error("attn_bwd: query heads per KV head must be even (got %d/%d)", Hq, Hkv);
    return 1;
  }
  const long long lds[8] = {ldq, ldk, ldv, ldo, lddo, lddq, lddk, lddv};
  const void* ptrs[8] = {q, k, v, o, dout, dq, dk, dv};
  for (int i = 0; i < 8; ++i)
    if ((lds[i] % 8) || ((uintptr_t)ptrs[i] % 16)) {
      tdllm_host::set_last_error("attn_bwd: operand %d needs 16-byte aligned base and row stride", i);
      return 1;
    }
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e1 = cudaFuncSetAttribute(attn_dq::attn_bwd_dq_kernel,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          attn_dq::SMEM_BYTES);
    cudaError_t e2 = cudaFuncSetAttribute(attn_dkv::attn_bwd_dkv_kernel,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          attn_dkv::SMEM_BYTES);
    if (e1 != cudaSuccess || e2 != cudaSuccess) {
      tdllm_host::set_last_error("attn_bwd: cudaFuncSetAttribute failed");
      return 2;
    }
    attr_set = true;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const int nq_pad = n_qtiles * 128;
  {
    const long long items = (long long)nq_pad * Hq;
    attn_dq::attn_delta_kernel<<<(unsigned)((items + 7) / 8), 256, 0, s>>>(
        (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, lse, delta, delta + (size_t)Hq * nq_pad, scale,
        nq, nq_pad, Hq, ldo, lddo);
  }
  CUtensorMap tq, tdo, tk, tv, tk64, tv64, tdq, tdk, tdv;
  const long long qc = (long long)Hq * 128, kc = (long long)Hkv * 128;
  if (tdllm_host::encode_rows_tmap(&tq, q, qc, nq, ldq, 128) ||
      tdllm_host::encode_rows_tmap(&tdo, dout, qc, nq, lddo, 128) ||
      tdllm_host::encode_rows_tmap(&tk, k, kc, nk, ldk, 128) ||
      tdllm_host::encode_rows_tmap(&tv, v, kc, nk, ldv, 128) ||
      tdllm_host::encode_rows_tmap(&tk64, k, kc, nk, ldk, 64) ||
      tdllm_host::encode_rows_tmap(&tv64, v, kc, nk, ldv, 64) ||
      tdllm_host::encode_rows_tmap(&tdq, dq, qc, nq, lddq, 128) ||
      tdllm_host::encode_rows_tmap(&tdk, dk, kc, nk, lddk, 128) ||
      tdllm_host::encode_rows_tmap(&tdv, dv, kc, nk, lddv, 128))
    return 3;
  {
    attn_dq::Params p;
    p.nq_pad = nq_pad; p.Hq = Hq; p.Hkv = Hkv;
    p.q_lo = q_lo; p.q_hi = q_hi; p.q_grp = q_grp; p.k_code = k_code;
    p.tile_ptr = f_ptr; p.tile_idx = f_idx; p.order = f_order;
    p.lse2 = delta + (size_t)Hq * nq_pad; p.delta = delta;
    p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
    const int grid = n_qtiles * Hkv * (Hq / Hkv / 2);
    attn_dq::attn_bwd_dq_kernel<<<grid, attn_dq::THREADS, attn_dq::SMEM_BYTES, s>>>(
        tq, tdo, tk64, tv64, tdq, p);
  }
  {
    attn_dkv::Params p;
    p.nq_pad = nq_pad; p.Hq = Hq; p.Hkv = Hkv;
    p.q_lo = q_lo; p.q_hi = q_hi; p.q_grp = q_grp; p.k_code = k_code;
    p.tile_ptr = b_ptr; p.tile_idx = b_idx; p.order = b_order;
    p.lse2 = delta + (size_t)Hq * nq_pad; p.delta = delta;
    p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
    const int grid = n_ktiles * Hkv;
    attn_dkv::attn_bwd_dkv_kernel<<<grid, attn_dkv::THREADS, attn_dkv::SMEM_BYTES, s>>>(
        tq, tdo, tk, tv, tdk, tdv, p);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    tdllm_host::set_last_error("attn_bwd launch: %s", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}

namespace tdllm {
// fp32 [rows, cols] accumulator -> bf16 rows of a (possibly wider) destination
__global__ void acc_cast_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ out, int rows,
                                int cols, long long ld_out) {
  const long long per_row = cols / 4;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)rows * per_row) return;
  const long long r = i / per_row, c = (i % per_row) * 4;
  const float4 v = *reinterpret_cast<const float4*>(acc + r * cols + c);
  uint2 o;
  o.x = pack_bf16x2(v.x, v.y);
  o.y = pack_bf16x2(v.z, v.w);
  *reinterpret_cast<uint2*>(out + r * ld_out + c) = o;
}
}  // namespace tdllm

// One-pass variant. `acc`: fp32 scratch of n_qtiles*128*Hq*128 + 2*n_ktiles*128*Hkv*128 floats (dQ, dK, dV
// accumulators, zeroed here). Work items (`w_*`): for chunk c of query tiles and key tile kt, item
// c*n_ktiles + kt lists the chunk's query tiles that see the key tile (w_ptr has one entry per item
// plus one); `w_order` names the non-empty items, chunk by chunk.
extern "C" int tdllm_attn_bwd_fused(const void* q, const void* k, const void* v, const void* o,
                                    const void* dout, void* dq, void* dk, void* dv, const float* lse,
                                    float* delta, float* acc, int nq, int nk, int Hq, int Hkv,
                                    long long ldq, long long ldk, long long ldv, long long ldo,
                                    long long lddo, long long lddq, long long lddk, long long lddv,
                                    const int* q_lo, const int* q_hi, const int* q_grp,
                                    const int* k_code, const int* w_ptr, const int* w_idx,
                                    const int* w_order, int n_work, int n_qtiles, int n_ktiles,
                                    float scale, void* stream) {
  if (nq <= 0 || nk <= 0) return 0;
  if (Hq % Hkv) {
    tdllm_host::set_last_error("attn_bwd_fused: %d query heads do not divide over %d KV heads", Hq, Hkv);
    return 1;
  }
  const long long lds[8] = {ldq, ldk, ldv, ldo, lddo, lddq, lddk, lddv};
  const void* ptrs[8] = {q, k, v, o, dout, dq, dk, dv};
  for (int i = 0; i < 8; ++i)
    if ((lds[i] % 8) || ((uintptr_t)ptrs[i] % 16)) {
      tdllm_host::set_last_error("attn_bwd_fused: operand %d needs 16-byte aligned base and row stride", i);
      return 1;
    }
  if ((uintptr_t)acc % 128) {
    tdllm_host::set_last_error("attn_bwd_fused: accumulator scratch must be 128-byte aligned");
    return 1;
  }
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_fused::attn_bwd_fused_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             attn_fused::SMEM_BYTES) != cudaSuccess) {
      tdllm_host::set_last_error("attn_bwd_fused: cudaFuncSetAttribute failed");
      return 2;
    }
    attr_set = true;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const int nq_pad = n_qtiles * 128, nk_pad = n_ktiles * 128;
  const long long qc = (long long)Hq * 128, kc = (long long)Hkv * 128;
  float* dq_acc = acc;
  float* dk_acc = dq_acc + (size_t)nq_pad * qc;
  float* dv_acc = dk_acc + (size_t)nk_pad * kc;
  cudaMemsetAsync(acc, 0, ((size_t)nq_pad * qc + 2 * (size_t)nk_pad * kc) * sizeof(float), s);
  {
    const long long items = (long long)nq_pad * Hq;
    attn_dq::attn_delta_kernel<<<(unsigned)((items + 7) / 8), 256, 0, s>>>(
        (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, lse, delta, delta + (size_t)Hq * nq_pad, scale,
        nq, nq_pad, Hq, ldo, lddo);
  }
  CUtensorMap tq, tdo, tk, tv, tdk, tdv, tacc;
  {
    // fp32 accumulators as [rows][heads*128]; one reduce-add copy moves 16 query rows (dQ) or a
    // swizzled block of 128 key rows x 32 columns (dK, dV) of one head
    uint64_t dims[2] = {(uint64_t)qc, (uint64_t)nq_pad};
    uint64_t strides[1] = {(uint64_t)qc * sizeof(float)};
    uint32_t box[2] = {128, 16};
    if (tdllm_host::encode_tmap(&tacc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, dq_acc, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_NONE))
      return 3;
    dims[0] = (uint64_t)kc; dims[1] = (uint64_t)nk_pad;
    strides[0] = (uint64_t)kc * sizeof(float);
    box[0] = 32; box[1] = 128;
    if (tdllm_host::encode_tmap(&tdk, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, dk_acc, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B) ||
        tdllm_host::encode_tmap(&tdv, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, dv_acc, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B))
      return 3;
  }
  if (tdllm_host::encode_rows_tmap(&tq, q, qc, nq, ldq, 64) ||
      tdllm_host::encode_rows_tmap(&tdo, dout, qc, nq, lddo, 64) ||
      tdllm_host::encode_rows_tmap(&tk, k, kc, nk, ldk, 128) ||
      tdllm_host::encode_rows_tmap(&tv, v, kc, nk, ldv, 128))
    return 3;
  if (n_work > 0) {
    attn_fused::Params p;
    p.nq_pad = nq_pad; p.Hq = Hq; p.Hkv = Hkv; p.nkt = n_ktiles;
    p.q_lo = q_lo; p.q_hi = q_hi; p.q_grp = q_grp; p.k_code = k_code;
    p.tile_ptr = w_ptr; p.tile_idx = w_idx; p.order = w_order;
    p.lse2 = delta + (size_t)Hq * nq_pad; p.delta = delta;
    p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
    attn_fused::PushPlan pp;
    memset(&pp, 0, sizeof(pp));
    attn_fused::attn_bwd_fused_kernel<false><<<n_work * Hkv, attn_fused::THREADS, attn_fused::SMEM_BYTES, s>>>(
        tq, tdo, tk, tv, tdk, tdv, tacc, tk, tv, p, pp);
  }
  {
    const long long n4 = (long long)nq * (qc / 4);
    acc_cast_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, s>>>(dq_acc, (__nv_bfloat16*)dq, nq, (int)qc, lddq);
    const long long k4 = (long long)nk * (kc / 4);
    acc_cast_kernel<<<(unsigned)((k4 + 255) / 256), 256, 0, s>>>(dk_acc, (__nv_bfloat16*)dk, nk, (int)kc, lddk);
    acc_cast_kernel<<<(unsigned)((k4 + 255) / 256), 256, 0, s>>>(dv_acc, (__nv_bfloat16*)dv, nk, (int)kc, lddv);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    tdllm_host::set_last_error("attn_bwd_fused launch: %s", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}

// Context-sharded one-pass backward. Keys as in tdllm_attn_fwd_csbp: this rank's nk_loc rows, then (from key
// tile ceil(nk_loc/128) on) the peers' clean rows held in kv_rem. dq_acc: fp32 scratch of n_qtiles*128*Hq*128
// floats, zeroed here. acc_dk[r] / acc_dv[r]: rank r's fp32 accumulators [acc_rows][Hkv*128] in symmetric
// memory as mapped here; they must be zero when the first rank starts (the caller alternates two sets:
// `next_acc` / `next_bytes` name this rank's other set, which is zeroed here, before this rank arrives at the
// barrier, for the following call). Gradients of this rank's key rows are added to acc_*[rank] at their row;
// gradients of a peer's clean rows are added to the peer's set at row dst_row0[peer] + (row within the peer's
// staged rows). After the kernel: barrier over `flags` at `epoch` (bounded waits), then dq, dk and dv
// ([nq] and [nk_loc] rows, bf16) are cast from dq_acc and this rank's set.
extern "C" int tdllm_attn_bwd_fused_csbp(
    const void* q, const void* k_loc, const void* v_loc, const void* kv_rem, const void* o, const void* dout,
    void* dq, void* dk, void* dv, const float* lse, float* delta, float* dq_acc, void* const* acc_dk,
    void* const* acc_dv, long long acc_rows, void* next_acc, long long next_bytes, int nq, int nk_loc,
    long long n_rem, int Hq, int Hkv, long long ldq, long long ldk, long long ldv, long long ldo, long long lddo,
    long long lddq, long long lddk, long long lddv, const int* q_lo, const int* q_hi, const int* q_grp,
    const int* k_code, const int* w_ptr, const int* w_idx, const int* w_order, int n_work, int n_qtiles,
    int n_ktiles, float scale, const long long* counts, const long long* dst_row0, void* const* flags, int rank,
    int world, int epoch, void* stream) {
  if (nq <= 0) return 0;
  if (Hq % Hkv) {
    tdllm_host::set_last_error("attn_bwd_fused_csbp: %d query heads do not divide over %d KV heads", Hq, Hkv);
    return 1;
  }
  if (world < 2 || world > attn_fused::MAX_PEERS || rank < 0 || rank >= world) {
    tdllm_host::set_last_error("attn_bwd_fused_csbp: 2..%d ranks (got %d)", attn_fused::MAX_PEERS, world);
    return 1;
  }
  const long long ldr = 2LL * Hkv * 128;
  const long long lds[9] = {ldq, ldk, ldv, ldo, lddo, lddq, lddk, lddv, ldr};
  const void* ptrs[9] = {q, k_loc, v_loc, o, dout, dq, dk, dv, kv_rem};
  for (int i = 0; i < 9; ++i)
    if ((lds[i] % 8) || ((uintptr_t)ptrs[i] % 16)) {
      tdllm_host::set_last_error("attn_bwd_fused_csbp: operand %d needs 16-byte aligned base and row stride", i);
      return 1;
    }
  const int nlt = (nk_loc + 127) / 128;
  if ((uintptr_t)dq_acc % 128 || (uintptr_t)acc_dk[rank] % 128 || (uintptr_t)acc_dv[rank] % 128 ||
      acc_rows < (long long)nlt * 128) {
    tdllm_host::set_last_error("attn_bwd_fused_csbp: accumulators must be 128-byte aligned and hold %d rows", nlt * 128);
    return 1;
  }
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_fused::attn_bwd_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             attn_fused::SMEM_BYTES) != cudaSuccess) {
      tdllm_host::set_last_error("attn_bwd_fused_csbp: cudaFuncSetAttribute failed");
      return 2;
    }
    attr_set = true;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const int nq_pad = n_qtiles * 128;
  const long long qc = (long long)Hq * 128, kc = (long long)Hkv * 128;
  cudaMemsetAsync(dq_acc, 0, (size_t)nq_pad * qc * sizeof(float), s);
  if (next_acc && next_bytes > 0) cudaMemsetAsync(next_acc, 0, (size_t)next_bytes, s);
  {
    const long long items = (long long)nq_pad * Hq;
    attn_dq::attn_delta_kernel<<<(unsigned)((items + 7) / 8), 256, 0, s>>>(
        (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, lse, delta, delta + (size_t)Hq * nq_pad, scale,
        nq, nq_pad, Hq, ldo, lddo);
  }
  float* my_dk = (float*)acc_dk[rank];
  float* my_dv = (float*)acc_dv[rank];
  CUtensorMap tq, tdo, tk, tv, tkr, tvr, tdk, tdv, tacc;
  {
    uint64_t dims[2] = {(uint64_t)qc, (uint64_t)nq_pad};
    uint64_t strides[1] = {(uint64_t)qc * sizeof(float)};
    uint32_t box[2] = {128, 16};
    if (tdllm_host::encode_tmap(&tacc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, dq_acc, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_NONE))
      return 3;
    dims[0] = (uint64_t)kc; dims[1] = (uint64_t)nlt * 128;
    strides[0] = (uint64_t)kc * sizeof(float);
    box[0] = 32; box[1] = 128;
    if (tdllm_host::encode_tmap(&tdk, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, my_dk, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B) ||
        tdllm_host::encode_tmap(&tdv, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, my_dv, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B))
      return 3;
  }
  const long long rem_rows = n_rem > 0 ? n_rem : 1;
  if (tdllm_host::encode_rows_tmap(&tq, q, qc, nq, ldq, 64) ||
      tdllm_host::encode_rows_tmap(&tdo, dout, qc, nq, lddo, 64) ||
      tdllm_host::encode_rows_tmap(&tk, k_loc, kc, nk_loc, ldk, 128) ||
      tdllm_host::encode_rows_tmap(&tv, v_loc, kc, nk_loc, ldv, 128) ||
      tdllm_host::encode_rows_tmap(&tkr, kv_rem, kc, rem_rows, ldr, 128) ||
      tdllm_host::encode_rows_tmap(&tvr, (const __nv_bfloat16*)kv_rem + kc, kc, rem_rows, ldr, 128))
    return 3;
  if (n_work > 0) {
    attn_fused::Params p;
    p.nq_pad = nq_pad; p.Hq = Hq; p.Hkv = Hkv; p.nkt = n_ktiles;
    p.q_lo = q_lo; p.q_hi = q_hi; p.q_grp = q_grp; p.k_code = k_code;
    p.tile_ptr = w_ptr; p.tile_idx = w_idx; p.order = w_order;
    p.lse2 = delta + (size_t)Hq * nq_pad; p.delta = delta;
    p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
    attn_fused::PushPlan pp;
    memset(&pp, 0, sizeof(pp));
    long long total = 0;
    pp.nseg = world - 1;
    for (int sgm = 0; sgm < world - 1; ++sgm) {
      const int peer = (rank + 1 + sgm) % world;
      pp.dk[sgm] = (float*)acc_dk[peer];
      pp.dv[sgm] = (float*)acc_dv[peer];
      pp.seg_begin[sgm] = total;
      pp.dst_row0[sgm] = dst_row0[peer];
      total += counts[peer];
    }
    for (int sgm = world - 1; sgm <= attn_fused::MAX_PEERS; ++sgm) pp.seg_begin[sgm] = total;
    if (total != n_rem) {
      tdllm_host::set_last_error("attn_bwd_fused_csbp: peers hold %lld rows, caller expects %lld", total, n_rem);
      return 1;
    }
    pp.n_rows = n_rem;
    pp.nlt = nlt;
    attn_fused::attn_bwd_fused_kernel<true><<<n_work * Hkv, attn_fused::THREADS, attn_fused::SMEM_BYTES, s>>>(
        tq, tdo, tk, tv, tdk, tdv, tacc, tkr, tvr, p, pp);
  }
  // every rank's partial sums for this rank's rows are in place once all ranks have passed this point
  if (tdllm_symm_barrier(flags, rank, world, epoch, stream)) return 5;
  {
    const long long n4 = (long long)nq * (qc / 4);
    acc_cast_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, s>>>(dq_acc, (__nv_bfloat16*)dq, nq, (int)qc, lddq);
    const long long k4 = (long long)nk_loc * (kc / 4);
    acc_cast_kernel<<<(unsigned)((k4 + 255) / 256), 256, 0, s>>>(my_dk, (__nv_bfloat16*)dk, nk_loc, (int)kc, lddk);
    acc_cast_kernel<<<(unsigned)((k4 + 255) / 256), 256, 0, s>>>(my_dv, (__nv_bfloat16*)dv, nk_loc, (int)kc, lddv);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    tdllm_host::set_last_error("attn_bwd_fused_csbp launch: %s", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}
