// Host-side shared helpers: last-error string, tensor-map encoding via the
// driver entry point, per-device status block, exported C accessors.
#include "host.h"

#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

namespace hmf {

static thread_local char g_last_error[512] = {0};

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return HMF_OK;
  set_last_error("CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), what);
  return HMF_ERR_CUDA;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaFree(0);  // make sure this runtime instance is attached to the device's primary context
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)p;
  });
  return fn;
}

int make_tensor_map(CUtensorMap* out, const void* base, int elem, int rank, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, int swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled entry point not available");
    return HMF_ERR_CUDA;
  }
  if (rank < 1 || rank > 5) {
    set_last_error("tensor map rank %d out of range", rank);
    return HMF_ERR_BAD_ARG;
  }
  if (((uintptr_t)base & 15) != 0) {
    set_last_error("tensor map base %p is not 16-byte aligned", base);
    return HMF_ERR_BAD_ARG;
  }
  CUtensorMapDataType dt;
  int esize;
  switch (elem) {
    case 0: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; esize = 2; break;
    case 1: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; esize = 4; break;
    case 2: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; esize = 1; break;
    case 3: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; esize = 2; break;
    default:
      set_last_error("tensor map element kind %d unknown", elem);
      return HMF_ERR_BAD_ARG;
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bdim[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
    if (box[i] == 0 || box[i] > 256) {
      set_last_error("tensor map box[%d]=%u out of range", i, box[i]);
      return HMF_ERR_BAD_ARG;
    }
  }
  for (int i = 1; i < rank; ++i) {
    gstr[i - 1] = strides_bytes[i];
    if (strides_bytes[i] % 16 != 0) {
      set_last_error("tensor map stride[%d]=%llu bytes is not a multiple of 16", i,
                     (unsigned long long)strides_bytes[i]);
      return HMF_ERR_BAD_ARG;
    }
  }
  if (((uint64_t)box[0] * esize) % 16 != 0) {
    set_last_error("tensor map inner box %u x %d bytes is not a multiple of 16", box[0], esize);
    return HMF_ERR_BAD_ARG;
  }
  CUtensorMapSwizzle sw = swizzle == 3   ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B
                                         : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = fn(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bdim, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    int n = 0;
    for (int i = 0; i < rank && n < 200; ++i)
      n += snprintf(buf + n, sizeof(buf) - n, " d%d=%llu/s%llu/b%u", i, (unsigned long long)dims[i],
                    (unsigned long long)(i > 0 ? strides_bytes[i] : 0), box[i]);
    set_last_error("cuTensorMapEncodeTiled failed with %d (base %p rank %d:%s)", (int)r, base, rank, buf);
    return HMF_ERR_CUDA;
  }
  return HMF_OK;
}

int make_map_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                     uint64_t row_stride_elems, uint32_t box_rows, uint32_t box_cols) {
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[2] = {2, row_stride_elems * 2};
  uint32_t box[2] = {box_cols, box_rows};
  return make_tensor_map(out, base, 0, 2, dims, strides, box, 3);
}

// One status block per device, living in a __device__ array (no allocation).
__device__ unsigned int g_status_block[4];

unsigned int* status_ptr() {
  static unsigned int* ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ptrs[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_block) != cudaSuccess) return nullptr;
    ptrs[dev] = (unsigned int*)p;
  }
  return ptrs[dev];
}

static cudaDeviceProp& props() {
  static cudaDeviceProp p[64];
  static bool have[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!have[dev]) {
    cudaGetDeviceProperties(&p[dev], dev);
    have[dev] = true;
  }
  return p[dev];
}
int sm_count() { return props().multiProcessorCount; }
int max_smem_optin() { return (int)props().sharedMemPerBlockOptin; }

}  // namespace hmf

HMF_API const char* hmf_last_error() { return hmf::g_last_error; }

// Copies the 4-word status block of the current device to `out` (synchronises
// the given stream first) and, when `reset` is non-zero, clears it.
HMF_API int hmf_read_status(unsigned int* out, int reset, cudaStream_t stream) {
  unsigned int* p = hmf::status_ptr();
  if (!p) {
    hmf::set_last_error("status block unavailable");
    return HMF_ERR_CUDA;
  }
  HMF_CHECK_CUDA(cudaStreamSynchronize(stream));
  HMF_CHECK_CUDA(cudaMemcpy(out, p, 4 * sizeof(unsigned int), cudaMemcpyDeviceToHost));
  if (reset) HMF_CHECK_CUDA(cudaMemset(p, 0, 4 * sizeof(unsigned int)));
  return HMF_OK;
}

// Binds the calling host thread to a device in this library's runtime instance (and makes that
// device's primary context current).  Needed once per thread that launches kernels, e.g. the
// autograd worker threads, which otherwise have no current context.
HMF_API int hmf_set_device(int index) {
  HMF_CHECK_CUDA(cudaSetDevice(index));
  HMF_CHECK_CUDA(cudaFree(0));
  return HMF_OK;
}

HMF_API int hmf_sm_count() { return hmf::sm_count(); }
HMF_API int hmf_abi_version() { return 1; }
