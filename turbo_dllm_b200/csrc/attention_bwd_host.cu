// Host entry points of the attention backward: row statistics (delta·scale, lse·log2e) into the
// caller's scratch [2, Hq, n_qtiles*128], then either the dQ kernel (per query tile) and the
// dK/dV kernel (per key tile), or the one-pass kernel (per key tile) that also accumulates dQ
// in an fp32 scratch, followed by a cast.
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
__global__ void dq_cast_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int nq,
                               int cols, long long lddq) {
  const long long per_row = cols / 4;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)nq * per_row) return;
  const long long r = i / per_row, c = (i % per_row) * 4;
  const float4 v = *reinterpret_cast<const float4*>(acc + r * cols + c);
  uint2 o;
  o.x = pack_bf16x2(v.x, v.y);
  o.y = pack_bf16x2(v.z, v.w);
  *reinterpret_cast<uint2*>(dq + r * lddq + c) = o;
}
}  // namespace tdllm

// One-pass variant: same operands plus `dq_acc`, fp32 scratch [n_qtiles*128, Hq, 128] (zeroed
// here). The forward-side tile lists (f_*) are not needed.
extern "C" int tdllm_attn_bwd_fused(const void* q, const void* k, const void* v, const void* o,
                                    const void* dout, void* dq, void* dk, void* dv, const float* lse,
                                    float* delta, float* dq_acc, int nq, int nk, int Hq, int Hkv,
                                    long long ldq, long long ldk, long long ldv, long long ldo,
                                    long long lddo, long long lddq, long long lddk, long long lddv,
                                    const int* q_lo, const int* q_hi, const int* q_grp,
                                    const int* k_code, const int* b_ptr, const int* b_idx,
                                    const int* b_order, int n_qtiles, int n_ktiles, float scale,
                                    void* stream) {
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
  if ((uintptr_t)dq_acc % 128) {
    tdllm_host::set_last_error("attn_bwd_fused: dq accumulator must be 128-byte aligned");
    return 1;
  }
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_fused::attn_bwd_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             attn_fused::SMEM_BYTES) != cudaSuccess) {
      tdllm_host::set_last_error("attn_bwd_fused: cudaFuncSetAttribute failed");
      return 2;
    }
    attr_set = true;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const int nq_pad = n_qtiles * 128;
  const long long qc = (long long)Hq * 128, kc = (long long)Hkv * 128;
  cudaMemsetAsync(dq_acc, 0, (size_t)nq_pad * qc * sizeof(float), s);
  {
    const long long items = (long long)nq_pad * Hq;
    attn_dq::attn_delta_kernel<<<(unsigned)((items + 7) / 8), 256, 0, s>>>(
        (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, lse, delta, delta + (size_t)Hq * nq_pad, scale,
        nq, nq_pad, Hq, ldo, lddo);
  }
  CUtensorMap tq, tdo, tk, tv, tdk, tdv, tacc;
  {
    // fp32 accumulator as [nq_pad rows][Hq*128]; one reduce-add copy moves 16 rows of one head
    const uint64_t dims[2] = {(uint64_t)qc, (uint64_t)nq_pad};
    const uint64_t strides[1] = {(uint64_t)qc * sizeof(float)};
    const uint32_t box[2] = {128, 16};
    if (tdllm_host::encode_tmap(&tacc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, dq_acc, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_NONE))
      return 3;
  }
  if (tdllm_host::encode_rows_tmap(&tq, q, qc, nq, ldq, 64) ||
      tdllm_host::encode_rows_tmap(&tdo, dout, qc, nq, lddo, 64) ||
      tdllm_host::encode_rows_tmap(&tk, k, kc, nk, ldk, 128) ||
      tdllm_host::encode_rows_tmap(&tv, v, kc, nk, ldv, 128) ||
      tdllm_host::encode_rows_tmap(&tdk, dk, kc, nk, lddk, 128) ||
      tdllm_host::encode_rows_tmap(&tdv, dv, kc, nk, lddv, 128))
    return 3;
  attn_fused::Params p;
  p.nq_pad = nq_pad; p.Hq = Hq; p.Hkv = Hkv;
  p.q_lo = q_lo; p.q_hi = q_hi; p.q_grp = q_grp; p.k_code = k_code;
  p.tile_ptr = b_ptr; p.tile_idx = b_idx; p.order = b_order;
  p.lse2 = delta + (size_t)Hq * nq_pad; p.delta = delta;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  attn_fused::attn_bwd_fused_kernel<<<n_ktiles * Hkv, attn_fused::THREADS, attn_fused::SMEM_BYTES, s>>>(
      tq, tdo, tk, tv, tdk, tdv, tacc, p);
  {
    const long long n4 = (long long)nq * (qc / 4);
    dq_cast_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, s>>>(dq_acc, (__nv_bfloat16*)dq, nq, (int)qc, lddq);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    tdllm_host::set_last_error("attn_bwd_fused launch: %s", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}
