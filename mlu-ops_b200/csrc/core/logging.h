// Logging and argument-check macros of the host side.
//
// Conventions follow the reference (core/logging.h:93-230): a failed
// PARAM_CHECK logs one ERROR line and returns MLUOP_STATUS_BAD_PARAM, a strided
// (non-contiguous) descriptor returns MLUOP_STATUS_NOT_SUPPORTED, a failed
// launch returns MLUOP_STATUS_EXECUTION_FAILED.  Output goes to stderr;
// MLUOP_MIN_LOG_LEVEL (0 info, 1 warning, 2 error, 3 silent) filters it and
// MLUOP_MIN_VLOG_LEVEL enables VLOG(n).
#ifndef MLUOP_B200_CORE_LOGGING_H_
#define MLUOP_B200_CORE_LOGGING_H_

#include <cstdint>
#include <sstream>
#include <string>

#include "mlu_op.h"

namespace mluop {

enum LogLevel { LOG_INFO = 0, LOG_WARNING = 1, LOG_ERROR = 2 };

int minLogLevel();
int minVlogLevel();

// Collects one message and writes it on destruction.
class LogLine {
 public:
  LogLine(int level, const char *file, int line);
  ~LogLine();
  std::ostream &stream() { return os_; }

 private:
  int level_;
  std::ostringstream os_;
};

bool isStrideTensor(int dim, const int64_t *dims, const int64_t *strides);

}  // namespace mluop

#define MLUOP_LOG_INFO ::mluop::LOG_INFO
#define MLUOP_LOG_WARNING ::mluop::LOG_WARNING
#define MLUOP_LOG_ERROR ::mluop::LOG_ERROR
#define LOG(level)                                  \
  if (MLUOP_LOG_##level >= ::mluop::minLogLevel())  \
  ::mluop::LogLine(MLUOP_LOG_##level, __FILE__, __LINE__).stream()
#define VLOG(n)                        \
  if ((n) <= ::mluop::minVlogLevel())  \
  ::mluop::LogLine(::mluop::LOG_INFO, __FILE__, __LINE__).stream()

#define PARAM_CHECK(api, condition, ...)                                  \
  if (!(condition)) {                                                     \
    LOG(ERROR) << api << " Check failed: " #condition ". " #__VA_ARGS__; \
    return MLUOP_STATUS_BAD_PARAM;                                        \
  }

#define PARAM_CHECK_V2(api, condition, ...)                              \
  if (!(condition)) {                                                    \
    LOG(ERROR) << api << " Check failed: " #condition ". " __VA_ARGS__; \
    return MLUOP_STATUS_BAD_PARAM;                                       \
  }

#define PARAM_CHECK_EQ(api, a, b)                                  \
  if (!((a) == (b))) {                                             \
    LOG(ERROR) << api << " Check failed: " #a " == " #b ". ";     \
    return MLUOP_STATUS_BAD_PARAM;                                 \
  }

#define PARAM_CHECK_LE(api, a, b)                                  \
  if (!((a) <= (b))) {                                             \
    LOG(ERROR) << api << " Check failed: " #a " <= " #b ". ";     \
    return MLUOP_STATUS_BAD_PARAM;                                 \
  }

#define INTERNAL_CHECK(api, condition)                           \
  if (!(condition)) {                                            \
    LOG(ERROR) << api << " An internal error occured. " #condition; \
    return MLUOP_STATUS_INTERNAL_ERROR;                          \
  }

#define CHECK_RETURN(api, status)                                           \
  {                                                                         \
    mluOpStatus_t status__ = (status);                                      \
    if (status__ != MLUOP_STATUS_SUCCESS) {                                 \
      LOG(ERROR) << api << " BAD return status: " #status " returns "       \
                 << status__ << " (FILE: " << __FILE__ << ", LINE: "        \
                 << __LINE__ << ").";                                       \
      return status__;                                                      \
    }                                                                       \
  }

// Non-contiguous tensors are not supported anywhere on this path.
#define STRIDE_TENSOR_CHECK(api, desc, reason)                                 \
  if ((desc) != NULL && mluOpGetTensorElementNum(desc) != 0 &&                 \
      ::mluop::isStrideTensor((desc)->getDim(), (desc)->getDims(),             \
                              (desc)->getStrides())) {                         \
    LOG(ERROR) << api << " stride tensor is not supported. " << reason;        \
    return MLUOP_STATUS_NOT_SUPPORTED;                                         \
  }

// Runs a launch expression, then maps a launch error to EXECUTION_FAILED.
#define KERNEL_CHECK(...)                                                       \
  {                                                                             \
    (void)cudaGetLastError();                                                   \
    __VA_ARGS__;                                                                \
    cudaError_t kernel_check_err__ = cudaPeekAtLastError();                     \
    if (kernel_check_err__ != cudaSuccess) {                                    \
      LOG(ERROR) << "Check failed: Found " << cudaGetErrorString(kernel_check_err__) \
                 << " after invoke kernel " #__VA_ARGS__;                       \
      return MLUOP_STATUS_EXECUTION_FAILED;                                     \
    }                                                                           \
  }

#define LARGE_TENSOR_NUM ((uint64_t)2147483648)  // 2^31, reference core/logging.h:37

// MLUOP_CHECK(call): for test and example code, not for the library itself; a status
// other than success is logged and thrown (reference core/logging.h:232-234, core/util.cpp:30-41).
#include <stdexcept>
inline void mluOpCheck(mluOpStatus_t result, char const *const func, const char *const file, int const line) {
  if (result != MLUOP_STATUS_SUCCESS) {
    const std::string error = "\"" + std::string(mluOpGetErrorString(result)) + " in " + std::string(func) + "\"";
    LOG(ERROR) << error << " (" << file << ":" << line << ")";
    throw std::runtime_error(error);
  }
}
#define MLUOP_CHECK(val) mluOpCheck((val), #val, __FILE__, __LINE__)

#endif  // MLUOP_B200_CORE_LOGGING_H_
