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
// The repacked filter holds [padded Co][padded Ci] values per offset, zero in the padding.
int tcgen05PaddedChannels(int c);

// The kernel reads the filter of one kernel offset with ONE bulk copy, so the repacked filter is
// the byte image of its shared-memory operand: per offset, for every block of up to 64 contracted
// channels (`row_bytes` = 2 * min(c_pad, 64) per produced channel, blocks `block_stride` bytes
// apart), rows of the n_pad produced channels with their 16-byte chunks XOR-swizzled the way
// tcgen05.mma expects (chunk ^= (byte offset >> 7) & (row_bytes / 16 - 1)).
struct Tcgen05FilterImage {
  int row_bytes;
  int block_stride;
  int bytes_per_offset;
};
inline Tcgen05FilterImage tcgen05FilterImage(int c_pad, int n_pad) {
  Tcgen05FilterImage im;
  const int block_k = c_pad < 64 ? c_pad : 64;
  im.row_bytes = block_k * 2;
  im.block_stride = (n_pad * im.row_bytes + 1023) / 1024 * 1024;
  im.bytes_per_offset = (c_pad / block_k) * im.block_stride;
  return im;
}

// status: one int32 of device memory, zero before the launch; a non-zero value
// afterwards means a bounded wait inside the kernel gave up (bit 0 producer on a gather stage,
// bit 1 MMA issuer on a stage, bit 2 epilogue, bit 3 producer on a filter buffer, bit 4 MMA issuer on a filter).
cudaError_t launchConvTcgen05(const ConvProblem &p, const ConvWorkspacePlan &plan, const __half *features,
                              const __half *filter_image, const int32_t *nbr, __half *out, int32_t *status,
                              double algo_bytes, double algo_flops, cudaStream_t stream);

}  // namespace sparse_conv
}  // namespace mluop

#endif  // MLUOP_B200_KERNELS_SPARSE_CONV_INDICE_CONVOLUTION_TCGEN05_H_
