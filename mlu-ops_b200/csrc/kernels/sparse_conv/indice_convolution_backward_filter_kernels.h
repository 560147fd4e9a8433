// Device side of the filter gradient of the sparse convolution: workspace plan
// and launch sequence.  Argument checks live in
// indice_convolution_backward_filter.cpp.
#ifndef MLUOP_B200_KERNELS_SPARSE_CONV_INDICE_CONVOLUTION_BACKWARD_FILTER_KERNELS_H_
#define MLUOP_B200_KERNELS_SPARSE_CONV_INDICE_CONVOLUTION_BACKWARD_FILTER_KERNELS_H_

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

namespace mluop {
namespace sparse_conv {

struct FilterGradProblem {
  int64_t L;      // rows of features (= indice_pairs dims[2])
  int64_t n_out;  // rows of output_grad
  int32_t K;      // kernel volume
  int32_t ci, co;
  int32_t is_half;
  // Device-visible host word (or null) that a kernel's error path stores its error
  // bits into, so that the next entry point on the handle can report them.
  int32_t *sticky_status;
};

// The pair list of every kernel offset is cut into segments of seg_pairs pairs;
// one thread block sums one segment into a float [Ci][Co] partial, a second
// kernel adds the partials of an offset in ascending segment order.  The result
// therefore does not depend on how blocks are scheduled.
struct FilterGradWorkspacePlan {
  size_t counts;   // int32[K]: pair counts
  size_t partial;  // float[K][max_segments][Ci][Co]
  // tensor-memory kernel (half, 64 input channels): its own scratch, laid over `partial`
  int32_t use_tc;
  size_t tc_status;   // int32: error bits of the kernel's bounded waits
  size_t tc_table;    // int32[K][n_pad]: the forward convolution's neighbour table
  size_t tc_partial;  // float[blocks][pairs][128][Co]
  size_t total;
  int32_t seg_pairs;
  int32_t max_segments;  // segments of the longest pair list
};

FilterGradWorkspacePlan planFilterGradWorkspace(const FilterGradProblem &p, const int64_t *indice_num,
                                                int sm_count);

// filters_grad is written as [K][Ci][Co] in the problem's data type.
cudaError_t launchIndiceConvolutionBackwardFilter(const FilterGradProblem &p,
                                                  const FilterGradWorkspacePlan &plan,
                                                  const void *features, const void *output_grad,
                                                  const int32_t *indice_pairs,
                                                  const int64_t *indice_num, void *workspace,
                                                  void *filters_grad, int sm_count, cudaStream_t stream,
                                                  const int32_t *forward_table = nullptr);

// Whether a call with these shapes and pointers runs from the forward convolution's neighbour
// table (the tensor-memory kernel) and can therefore take the caller's copy of it.
bool filterGradRunsFromTable(const FilterGradProblem &p, const FilterGradWorkspacePlan &plan, const void *features,
                             const void *output_grad);

}  // namespace sparse_conv
}  // namespace mluop

#endif  // MLUOP_B200_KERNELS_SPARSE_CONV_INDICE_CONVOLUTION_BACKWARD_FILTER_KERNELS_H_
