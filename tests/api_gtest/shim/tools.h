// Stand-in for the header of the same name in the reference's test harness
// (test/mlu_op_gtest/include/tools.h), which the reference's API tests include
// through api_test_tools.h.  The original pulls in the protobuf-generated test-case
// classes and the vendor's device-management header, neither of which exists
// here; the API tests themselves only use what is below: the check macros of
// check_tools.h and the vendor runtime's allocation / queue calls, mapped to the
// CUDA runtime (or to the host heap when the process has no CUDA device: every
// API test fails or succeeds in the argument checks, so the pointers are never
// dereferenced).
#ifndef MLUOP_B200_TESTS_API_GTEST_SHIM_TOOLS_H_
#define MLUOP_B200_TESTS_API_GTEST_SHIM_TOOLS_H_

#include <cuda_runtime_api.h>

#include <cstdlib>
#include <sstream>
#include <stdexcept>
#include <string>

#include "core/logging.h"
#include "core/tensor.h"
#include "gtest/gtest.h"
#include "mlu_op.h"

#ifndef unlikely
#define unlikely(x) __builtin_expect(!!(x), 0)
#endif

#define GTEST_CHECK(condition, ...)                                                                   \
  if (unlikely(!(condition))) {                                                                       \
    ADD_FAILURE() << "Check failed: " #condition ". ";                                                \
    throw std::invalid_argument(std::string(__FILE__) + " +" + std::to_string(__LINE__));             \
  }

typedef int cnrtRet_t;
static const cnrtRet_t cnrtSuccess = 0;

namespace mluop_api_gtest_shim {
inline bool haveDevice() {
  static const bool have = [] {
    int n = 0;
    const bool ok = cudaGetDeviceCount(&n) == cudaSuccess && n > 0;
    (void)cudaGetLastError();
    return ok;
  }();
  return have;
}
}  // namespace mluop_api_gtest_shim

inline cnrtRet_t cnrtMalloc(void **ptr, size_t bytes) {
  if (mluop_api_gtest_shim::haveDevice()) return cudaMalloc(ptr, bytes ? bytes : 1) == cudaSuccess ? 0 : 1;
  // 256-byte aligned like a device allocation
  return posix_memalign(ptr, 256, bytes ? bytes : 1) == 0 ? 0 : 1;
}
inline cnrtRet_t cnrtFree(void *ptr) {
  if (mluop_api_gtest_shim::haveDevice()) return cudaFree(ptr) == cudaSuccess ? 0 : 1;
  std::free(ptr);
  return 0;
}
inline cnrtRet_t cnrtQueueSync(cnrtQueue_t queue) {
  if (!mluop_api_gtest_shim::haveDevice()) return 0;
  return cudaStreamSynchronize(queue) == cudaSuccess ? 0 : 1;
}

#define CNRT_CHECK(call)                                                                             \
  do {                                                                                               \
    if ((call) != cnrtSuccess) throw std::runtime_error(std::string("runtime call failed: ") + #call); \
  } while (0)

#endif  // MLUOP_B200_TESTS_API_GTEST_SHIM_TOOLS_H_
