// Optional per-launch timing with CUDA events (see include/mlu_op_trace.h).
#ifndef MLUOP_B200_CORE_TRACE_H_
#define MLUOP_B200_CORE_TRACE_H_

#include <cuda_runtime_api.h>

namespace mluop {
namespace trace {

bool enabled();

// Brackets the launches issued during its lifetime with two events on `stream`.
// `name` must be a string literal (it is kept by pointer).
class Scope {
 public:
  Scope(const char *name, cudaStream_t stream, double algorithmic_bytes = 0.0, double flops = 0.0);
  ~Scope();
  Scope(const Scope &) = delete;
  Scope &operator=(const Scope &) = delete;

 private:
  int slot_;
  cudaStream_t stream_;
};

}  // namespace trace
}  // namespace mluop

#endif  // MLUOP_B200_CORE_TRACE_H_
