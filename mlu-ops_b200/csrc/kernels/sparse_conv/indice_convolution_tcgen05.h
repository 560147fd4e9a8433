// tcgen05 / tensor-memory variant of the convolution kernel: half, channel
// counts that are multiples of 8 up to 128 (run at the next of 16 / 32 / 64 / 128
// with zero padding on chip), kernel volume up to 128.
#ifndef MLUOP_B200_KERNELS_SPARSE_CONV_INDICE_CONVOLUTION_TCGEN05_H_
#define MLUOP_B200_KERNELS_SPARSE_CONV_INDICE_CONVOLUTION_TCGEN05_H_

#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include "kernels/sparse_conv/indice_convolution_kernels.h"

namespace mluop {
namespace sparse_conv {

bool tcgen05Eligible(const ConvProblem &p, const void *features, const void *out);
// The channel count the kernel runs a count of c at (16, 32, 64 or 128), 0 if unsupported.
// The repacked filter the kernel reads is [K][padded Co][padded Ci], zero in the padding.
int tcgen05PaddedChannels(int c);

// status: one int32 of device memory, zero before the launch; a non-zero value
// afterwards means a bounded wait inside the kernel gave up (bit 0 producer on a gather stage,
// bit 1 MMA issuer, bit 2 epilogue, bit 3 producer on a filter buffer).
cudaError_t launchConvTcgen05(const ConvProblem &p, const ConvWorkspacePlan &plan, const __half *features,
                              const __half *filter_kcoci, const int32_t *nbr, __half *out, int32_t *status,
                              double algo_bytes, double algo_flops, cudaStream_t stream);

}  // namespace sparse_conv
}  // namespace mluop

#endif  // MLUOP_B200_KERNELS_SPARSE_CONV_INDICE_CONVOLUTION_TCGEN05_H_
