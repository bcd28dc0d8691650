// Library runtime: error record, wait budget, tensor-map encoding through the driver
// entry point, and the bounded-wait self test.
#include <cstdarg>
#include <cstdio>
#include <cudaTypedefs.h>
#include "common.cuh"
#include "api.h"

namespace tdllm {
__device__ int g_tdllm_error[8] = {0, 0, 0, 0, 0, 0, 0, 0};
__device__ unsigned long long g_tdllm_timeout_ns = 2000000000ull;

__global__ void wait_timeout_test_kernel() {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
  }
  __syncthreads();
  // nobody ever arrives: the wait must run out of budget and come back
  if (threadIdx.x == 0) mbar_wait(smem_u32(&bar), 0, /*kernel_id=*/99, /*detail=*/7);
  __syncthreads();
}
}  // namespace tdllm

namespace tdllm_host {
static thread_local char g_err[512] = "";
const char* last_error() { return g_err; }
void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !p) {
    set_last_error("cuTensorMapEncodeTiled entry point unavailable: %s", cudaGetErrorString(e));
    return nullptr;
  }
  fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
  return fn;
}

int encode_tmap(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base,
                const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                CUtensorMapSwizzle swz) {
  auto fn = get_encode();
  if (!fn) return 1;
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  auto encode = [&]() {
    return fn(out, dt, (cuuint32_t)rank, const_cast<void*>(base), (const cuuint64_t*)dims,
              (const cuuint64_t*)strides_bytes, (const cuuint32_t*)box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r = encode();
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // a thread that has made no runtime call yet (an autograd worker) has no current context for
    // this driver entry point; a runtime no-op binds the device's primary context to the thread
    (void)cudaFree(nullptr);
    r = encode();
  }
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled failed: code %d (rank %d dims %llu,%llu stride %llu box %u,%u)",
                   (int)r, rank, (unsigned long long)dims[0], (unsigned long long)dims[1],
                   (unsigned long long)strides_bytes[0], box[0], box[1]);
    return 1;
  }
  return 0;
}
}  // namespace tdllm_host

extern "C" const char* tdllm_last_error(void) { return tdllm_host::last_error(); }

extern "C" int tdllm_num_sms(void) {
  static int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!sms[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    sms[dev] = n;
  }
  return sms[dev];
}

extern "C" int tdllm_get_error(int* out8) {
  cudaError_t e = cudaMemcpyFromSymbol(out8, tdllm::g_tdllm_error, 8 * sizeof(int));
  if (e != cudaSuccess) {
    tdllm_host::set_last_error("get_error: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}
extern "C" int tdllm_clear_error(void) {
  int z[8] = {0};
  cudaError_t e = cudaMemcpyToSymbol(tdllm::g_tdllm_error, z, sizeof(z));
  if (e != cudaSuccess) {
    tdllm_host::set_last_error("clear_error: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}
extern "C" int tdllm_set_wait_timeout_ns(unsigned long long ns) {
  cudaError_t e = cudaMemcpyToSymbol(tdllm::g_tdllm_timeout_ns, &ns, sizeof(ns));
  if (e != cudaSuccess) {
    tdllm_host::set_last_error("set_wait_timeout: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}
extern "C" int tdllm_test_wait_timeout(void* stream) {
  tdllm::wait_timeout_test_kernel<<<1, 32, 0, (cudaStream_t)stream>>>();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    tdllm_host::set_last_error("wait test launch: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}
