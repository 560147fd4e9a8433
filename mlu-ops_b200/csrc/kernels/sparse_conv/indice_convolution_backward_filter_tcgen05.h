// Filter gradient of the sparse convolution on the tcgen05 tensor cores: plan
// and launch (half; 64 input channels with 64 or 128 output channels, 32 with 32 or 64).
#ifndef MLUOP_B200_KERNELS_SPARSE_CONV_INDICE_CONVOLUTION_BACKWARD_FILTER_TCGEN05_H_
#define MLUOP_B200_KERNELS_SPARSE_CONV_INDICE_CONVOLUTION_BACKWARD_FILTER_TCGEN05_H_

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

#include "kernels/sparse_conv/indice_convolution_backward_filter_kernels.h"

namespace mluop {
namespace sparse_conv {

struct FilterGradTcPlan {
  int32_t groups;            // groups of kernel offsets; a block serves one group
  int32_t bundles_per_group;  // bundles of 128 / Ci offsets (one accumulator each) a block keeps in tensor memory
  int32_t blocks_per_group;  // blocks that share a group's tiles of 128 output rows
  int64_t n_pad;             // rows of the neighbour table (n_out padded)
  size_t table_bytes;        // int32[K][n_pad]
  size_t partial_bytes;      // float[groups * blocks_per_group][bundles_per_group][128][Co]
};

// Decided from the shape alone, so that the workspace query and the call agree;
// MLUOP_B200_FILTER_GRAD_KERNEL=mma turns the tensor-memory kernel off, =tcgen05 also
// sends 32 input channels to it (slower there than the pair-list kernel; kept selectable
// and tested).
bool filterGradTcShapeEligible(const FilterGradProblem &p);

FilterGradTcPlan planFilterGradTc(const FilterGradProblem &p, int sm_count);

// table, partial and status (one int32 of error bits) are 256-byte aligned
// device buffers of the sizes the plan gives; filters_grad is written as half
// [K][Ci][Co].  external_table: the forward convolution's neighbour table if the
// caller has it (then `table` is unused and nothing is built), else null.
cudaError_t launchFilterGradTcgen05(const FilterGradProblem &p, const FilterGradTcPlan &plan, const void *features,
                                    const void *output_grad, const int32_t *indice_pairs,
                                    const int64_t *indice_num, int32_t *table, float *partial, int32_t *status,
                                    void *filters_grad, int sm_count, double bytes, double flops,
                                    cudaStream_t stream, const int32_t *external_table = nullptr);

}  // namespace sparse_conv
}  // namespace mluop

#endif  // MLUOP_B200_KERNELS_SPARSE_CONV_INDICE_CONVOLUTION_BACKWARD_FILTER_TCGEN05_H_
