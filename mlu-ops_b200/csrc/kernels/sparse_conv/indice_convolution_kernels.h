// Device side of the sparse convolution forward and of its input gradient:
// workspace plan and launch sequence.  Argument checks live in
// indice_convolution_forward.cpp and indice_convolution_backward_data.cpp.
#ifndef MLUOP_B200_KERNELS_SPARSE_CONV_INDICE_CONVOLUTION_KERNELS_H_
#define MLUOP_B200_KERNELS_SPARSE_CONV_INDICE_CONVOLUTION_KERNELS_H_

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

namespace mluop {
namespace sparse_conv {

// Output rows owned by one thread block of the tensor-core kernel; the
// neighbour table is padded to a multiple of it.
constexpr int kConvTileRows = 128;
// The neighbour table is padded to a multiple of this many rows (the largest
// block of rows any kernel variant owns).
constexpr int kConvPadRows = 512;

enum FilterLayout { kFilterArray = 0, kFilterNDHWC = 1, kFilterNCDHW = 2 };

struct ConvProblem {
  int64_t L;        // input rows
  int64_t n_out;    // output rows
  int32_t K;        // kernel volume
  int32_t ci, co;
  int32_t is_half;  // 1: half, 0: float
  int32_t filter_layout;
  // 0: forward, features [L,ci] -> features_out [n_out,co].
  // 1: input gradient, output_grad [n_out,co] -> input_grad [L,ci]: the same
  //    computation with the two row sets, the two ids of a pair and the two
  //    channel axes of the filter exchanged.
  int32_t backward_data;
  // 1 (input gradient from a caller's table only): the table is the FORWARD table of a submanifold
  // rulebook with centred padding, whose pairs are symmetric - (i, o) at offset k goes with (o, i)
  // at offset K-1-k - so the output row input row i feeds through offset k stands in forward table
  // row K-1-k at column i.  Only the tensor-memory kernel reads a table this way.
  int32_t mirror_table;
  // Device-visible host word (or null) that a kernel's error path stores its error
  // bits into, so that the next entry point on the handle can report them.
  int32_t *sticky_status;
};

struct ConvWorkspacePlan {
  size_t status;     // int32[64]: [0] error bits of the tensor-memory kernel's bounded waits
  size_t filter;     // T[K][Co][Ci]: filter repacked so that the contracted axis is contiguous
                     // (input gradient: T[K][Ci][Co])
  size_t neighbour;  // int32[K][n_pad]: source row feeding (k, destination row), -1 if none
  size_t counts;     // int32[K]: pair counts, only used when K is too large for kernel arguments
  size_t total;
  int64_t n_pad;
};

// external_table: the neighbour table lives in a buffer of the caller (see
// launchIndiceConvolutionSteps), the workspace holds the rest.
ConvWorkspacePlan planConvWorkspace(const ConvProblem &p, bool external_table = false);

// Whether the convolution of this problem (either direction) and these row arrays runs on the
// tensor-memory kernel (the only one that reads a mirrored table).
bool convRunsOnTensorMemory(const ConvProblem &p, const void *rows_in, const void *rows_out);

// Bytes of a neighbour table int32[K][n_pad] for this problem and direction.
size_t neighbourTableBytes(const ConvProblem &p);
// Whether the pair counts of K offsets fit the kernel-argument path that building a
// table without a workspace relies on.
bool neighbourTableCountsFit(int32_t K);

// Enqueues filter repack, neighbour-table build and the convolution kernel.
// indice_num is the caller's host array.  `rows_in` are the rows that are
// gathered (features, or output_grad for the input gradient), `rows_out` the
// rows that are produced (features_out, or input_grad).
cudaError_t launchIndiceConvolution(const ConvProblem &p, const ConvWorkspacePlan &plan,
                                    const void *rows_in, const void *filters,
                                    const int32_t *indice_pairs, const int64_t *indice_num,
                                    void *workspace, void *rows_out, int sm_count,
                                    cudaStream_t stream);

// The same launch sequence with the neighbour table in a caller buffer, run in
// part: a rulebook that feeds several convolutions needs its table built once.
enum NeighbourTableSteps {
  kTableBuildAndConvolve = 0,  // what launchIndiceConvolution does
  kTableBuildOnly = 1,         // memset + build into external_table; features, filters, workspace, rows_out unused
  kTableConvolveOnly = 2,      // filter repack + convolution reading external_table
};
cudaError_t launchIndiceConvolutionSteps(const ConvProblem &p, const ConvWorkspacePlan &plan,
                                         const void *rows_in, const void *filters,
                                         const int32_t *indice_pairs, const int64_t *indice_num,
                                         void *workspace, void *rows_out, int sm_count,
                                         cudaStream_t stream, int32_t *external_table, int steps);

}  // namespace sparse_conv
}  // namespace mluop

#endif  // MLUOP_B200_KERNELS_SPARSE_CONV_INDICE_CONVOLUTION_KERNELS_H_
