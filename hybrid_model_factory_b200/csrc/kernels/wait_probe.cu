// Bounded-wait self test: one thread waits for a flag with the same helper the peer-memory kernels use
// (`wait_flag_sys`), with a caller-chosen time limit.  When nothing raises the flag the wait runs out, the kernel
// records code kFlagTimeout in the status block and returns normally: the context stays usable.
#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
__global__ void wait_probe_kernel(const unsigned int* flag, unsigned int want, unsigned long long limit_ns,
                                  unsigned int* status, int* result) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *result = wait_flag_sys(flag, want, limit_ns, status, 0x900) ? 1 : 0;
}
}  // namespace hmf

using namespace hmf;

// result: 1 = flag reached `want`, 0 = the wait ran out (status block holds the error).
HMF_API int hmf_wait_probe(const unsigned int* flag, unsigned int want, unsigned long long limit_ns, int* result,
                           cudaStream_t st) {
  HMF_REQUIRE(limit_ns <= 1000000000ull, "wait_probe: limit %llu ns above one second", limit_ns);
  wait_probe_kernel<<<1, 32, 0, st>>>(flag, want, limit_ns, status_ptr(), result);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}
