// Host-side helpers shared by the launchers: error codes, tensor-map encoding
// through the driver entry point (no link-time dependency on libcuda), device
// properties cache.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define HMF_API extern "C" __attribute__((visibility("default")))

// Return codes of every exported launcher.
enum HmfError : int {
  HMF_OK = 0,
  HMF_ERR_BAD_ARG = -1,      // shape / alignment / null pointer rejected before launch
  HMF_ERR_CUDA = -2,         // a CUDA runtime call failed; see hmf_last_error()
  HMF_ERR_UNSUPPORTED = -3,  // configuration not built
  HMF_ERR_TOO_LARGE = -4,    // beyond a documented static limit
};

namespace hmf {

void set_last_error(const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

// Encodes a tiled tensor map for a row-major tensor of up to 5 dims.
// dims/strides are innermost-first; strides[0] is implied by the element size;
// strides[i>0] are in BYTES and must be multiples of 16; box is in elements.
// swizzle: 0 none, 1 32B, 2 64B, 3 128B.   elem: 0 bf16, 1 fp32, 2 u8, 3 fp16
int make_tensor_map(CUtensorMap* out, const void* base, int elem, int rank, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, int swizzle);

// Convenience: 2-D row-major [rows, cols] bf16 with 128B swizzle and box [box_rows, 64].
int make_map_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                     uint64_t row_stride_elems, uint32_t box_rows, uint32_t box_cols);

// Device pointer to the 4-word status block of the current device (lazily allocated).
unsigned int* status_ptr();

int sm_count();
int max_smem_optin();

}  // namespace hmf

#define HMF_CHECK_CUDA(expr)                                  \
  do {                                                        \
    int _e = ::hmf::check_cuda((expr), #expr);                \
    if (_e != HMF_OK) return _e;                              \
  } while (0)

#define HMF_REQUIRE(cond, ...)                                \
  do {                                                        \
    if (!(cond)) {                                            \
      ::hmf::set_last_error(__VA_ARGS__);                     \
      return HMF_ERR_BAD_ARG;                                 \
    }                                                         \
  } while (0)
