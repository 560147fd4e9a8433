// mluOpIndiceConvolutionBackwardData / mluOpGetIndiceConvolutionBackwardDataWorkspaceSize:
// argument checks and dispatch (reference
// kernels/sparse_conv/indice_convolution_backward_data/indice_convolution_backward_data.cpp:
// foolCheckNoPtr :34-232, foolCheck :277-307, workspace query :358-566,
// compute entry :568-959).
//
//   input_grad[i,:] = sum_k sum_{(i,o) in pairs_k} output_grad[o,:] * W_k^T
//
// The reference runs, per kernel offset, a gather of output_grad rows, a matmul
// with the transposed filter slice, a scatter into a zeroed copy of input_grad
// and an add.  Here it is the forward computation with the two row sets
// exchanged: a neighbour table input row -> output row per offset, then one
// kernel that owns a tile of input_grad rows and sums over the offsets in
// ascending order (no atomics, every row written once).
//
// The order of the checks, and the status each returns, follows the reference.
// One limit differs: the reference refuses more than 1,000,000 input rows
// (get_indice_pairs_structs.h:36); here the bound is only that every tensor has
// fewer than 2^31 elements.
#include <cuda_runtime_api.h>

#include <cstdlib>
#include <string>

#include "core/context.h"
#include "core/logging.h"
#include "core/tensor.h"
#include "kernels/sparse_conv/indice_convolution_kernels.h"

using mluop::sparse_conv::ConvProblem;
using mluop::sparse_conv::ConvWorkspacePlan;

namespace {

struct FilterDims {
  int64_t kd = 1, kh = 1, kw = 1, dyc = 1, dxc = 1;
  int64_t K() const { return kd * kh * kw; }
};

// reference :103-124
FilterDims readFilterDims(const mluOpTensorDescriptor_t filters_desc) {
  FilterDims f;
  if (filters_desc->getLayout() != MLUOP_LAYOUT_ARRAY) {
    f.kh = mluOpGetTensordimH(filters_desc);
    f.kw = mluOpGetTensordimW(filters_desc);
    f.dyc = mluOpGetTensordimN(filters_desc);
    f.dxc = mluOpGetTensordimC(filters_desc);
    if (filters_desc->getDim() == 5) f.kd = mluOpGetTensordimD(filters_desc);
  } else {
    const int n = filters_desc->getDim();
    if (n == 5) f.kd = filters_desc->getDimIndex(0);
    f.kh = filters_desc->getDimIndex(n - 4);
    f.kw = filters_desc->getDimIndex(n - 3);
    f.dxc = filters_desc->getDimIndex(n - 2);
    f.dyc = filters_desc->getDimIndex(n - 1);
  }
  return f;
}

int filterLayoutCode(mluOpTensorLayout_t layout) {
  switch (layout) {
    case MLUOP_LAYOUT_NHWC:
    case MLUOP_LAYOUT_NDHWC:
      return mluop::sparse_conv::kFilterNDHWC;  // [Co][K][Ci]
    case MLUOP_LAYOUT_NCHW:
    case MLUOP_LAYOUT_NCDHW:
      return mluop::sparse_conv::kFilterNCDHW;  // [Co][Ci][K]
    default:
      return mluop::sparse_conv::kFilterArray;  // HWCN, ARRAY: [K][Ci][Co]
  }
}

int64_t maxCount(const int64_t indice_num[], int64_t K) {
  int64_t m = 0;
  for (int64_t k = 0; k < K; ++k) m = indice_num[k] > m ? indice_num[k] : m;
  return m;
}

mluOpStatus_t foolCheckNoPtr(const std::string &api, mluOpHandle_t handle,
                             const mluOpTensorDescriptor_t output_grad_desc,
                             const mluOpTensorDescriptor_t filters_desc,
                             const mluOpTensorDescriptor_t indice_pairs_desc, const int64_t indice_num[],
                             const int64_t inverse, const int64_t sub_m,
                             const mluOpTensorDescriptor_t input_grad_desc, bool *is_zero) {
  PARAM_CHECK(api, handle != nullptr);
  PARAM_CHECK(api, output_grad_desc != nullptr);
  PARAM_CHECK(api, filters_desc != nullptr);
  PARAM_CHECK(api, indice_pairs_desc != nullptr);
  PARAM_CHECK(api, input_grad_desc != nullptr);
  // The reference dereferences indice_num without a check; a null array is a caller error.
  PARAM_CHECK(api, indice_num != nullptr);

  if (handle->arch < MLUOP_MLU370) {
    LOG(ERROR) << api << " needs a compute-capability 10.x device; this handle's device is not one.";
    return MLUOP_STATUS_ARCH_MISMATCH;
  }

  PARAM_CHECK_EQ(api, output_grad_desc->getDim(), 2);
  PARAM_CHECK(api, filters_desc->getDim() == 4 || filters_desc->getDim() == 5);
  PARAM_CHECK_EQ(api, indice_pairs_desc->getDim(), 3);
  PARAM_CHECK_EQ(api, input_grad_desc->getDim(), 2);
  PARAM_CHECK(api, indice_pairs_desc->getDimIndex(1) == 2);

  PARAM_CHECK(api, output_grad_desc->getDtype() == MLUOP_DTYPE_FLOAT ||
                       output_grad_desc->getDtype() == MLUOP_DTYPE_HALF);
  PARAM_CHECK(api, filters_desc->getDtype() == MLUOP_DTYPE_FLOAT ||
                       filters_desc->getDtype() == MLUOP_DTYPE_HALF);
  PARAM_CHECK(api, input_grad_desc->getDtype() == MLUOP_DTYPE_FLOAT ||
                       input_grad_desc->getDtype() == MLUOP_DTYPE_HALF);
  PARAM_CHECK(api, indice_pairs_desc->getDtype() == MLUOP_DTYPE_INT32);

  const mluOpTensorLayout_t layout = filters_desc->getLayout();
  const bool layout_ok = layout == MLUOP_LAYOUT_NHWC || layout == MLUOP_LAYOUT_NCHW ||
                         layout == MLUOP_LAYOUT_HWCN || layout == MLUOP_LAYOUT_NCDHW ||
                         layout == MLUOP_LAYOUT_NDHWC || layout == MLUOP_LAYOUT_ARRAY;
  if (!layout_ok) {
    LOG(ERROR) << api << " The filters tensor only supports NHWC/NCHW/HWCN/NCDHW/NDHWC/ARRAY layout.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  // A 4-D tag on a 5-D filter (or the reverse) would make the dimension getters read the wrong axes.
  const bool tag_4d = layout == MLUOP_LAYOUT_NHWC || layout == MLUOP_LAYOUT_NCHW || layout == MLUOP_LAYOUT_HWCN;
  const bool tag_5d = layout == MLUOP_LAYOUT_NDHWC || layout == MLUOP_LAYOUT_NCDHW;
  if ((tag_4d && filters_desc->getDim() != 4) || (tag_5d && filters_desc->getDim() != 5)) {
    LOG(ERROR) << api << " The filters layout " << mluop::getNameOfTensorLayout(layout) << " does not match its "
               << filters_desc->getDim() << " dimensions.";
    return MLUOP_STATUS_BAD_PARAM;
  }

  STRIDE_TENSOR_CHECK(api + ":", output_grad_desc, "output_grad_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", filters_desc, "filters_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", indice_pairs_desc, "indice_pairs_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", input_grad_desc, "input_grad_desc must be contiguous");

  const FilterDims f = readFilterDims(filters_desc);
  const int64_t K = f.K();

  PARAM_CHECK(api, inverse == 0 || inverse == 1);
  PARAM_CHECK(api, sub_m == 0 || sub_m == 1);
  // indice_num has one entry per row of indice_pairs; never read past that
  const int64_t listed = K < indice_pairs_desc->getDimIndex(0) ? K : indice_pairs_desc->getDimIndex(0);
  for (int64_t k = 0; k < listed; ++k) {
    PARAM_CHECK(api, indice_num[k] >= 0);
  }
  if (inverse == 1) {
    LOG(ERROR) << api << " Not support inverse == 1 yet.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }
  if (K != indice_pairs_desc->getDimIndex(0)) {
    LOG(ERROR) << api << " The dims[0] of indice_pairs should be equal to the multiple of kd, kh and kw.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (output_grad_desc->getDimIndex(1) != f.dyc) {
    LOG(ERROR) << api << " The dims[1] of output_grad should be equal to dyc of filters tensor.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (input_grad_desc->getDimIndex(1) != f.dxc) {
    LOG(ERROR) << api << " The dims[1] of input_grad should be equal to dxc of filters tensor.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (input_grad_desc->getDimIndex(0) != indice_pairs_desc->getDimIndex(2)) {
    LOG(ERROR) << api << " The dims[0] of input_grad should be equal to the dims[2] of indice_pairs.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  const int64_t max_indice_num = maxCount(indice_num, K);
  if (indice_pairs_desc->getDimIndex(2) < max_indice_num) {
    LOG(ERROR) << api << " The data in indice_num array should be smaller or equal to the dims[2] of indice_pairs.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (sub_m == 1) {
    if (input_grad_desc->getDimIndex(0) != output_grad_desc->getDimIndex(0)) {
      LOG(ERROR) << api << " The dims[0] of input_grad should be equal to the dims[0] of output_grad when sub_m is 1.";
      return MLUOP_STATUS_BAD_PARAM;
    }
    if (K > 0 && indice_num[K / 2] < max_indice_num) {
      LOG(ERROR) << api << " The middle number of the indice_num array should be the maximum of the array when "
                 << "sub_m is 1. Now the maximum is " << max_indice_num << " while the middle number of the array is "
                 << indice_num[K / 2] << ".";
      return MLUOP_STATUS_BAD_PARAM;
    }
  }
  if (output_grad_desc->getDimIndex(0) < max_indice_num) {
    LOG(ERROR) << api << " The dims[0] of output_grad should be larger than or equal to the maximum number of "
               << "indice_num.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (sub_m == 1 && K % 2 == 0) {
    LOG(ERROR) << api << " When sub_m value is 1, the filters dims (Kd, Kh & Kw) should be odd numbers.";
    return MLUOP_STATUS_BAD_PARAM;
  }

  PARAM_CHECK(api, output_grad_desc->getDtype() == input_grad_desc->getDtype());
  PARAM_CHECK(api, output_grad_desc->getDtype() == filters_desc->getDtype());

  const uint64_t input_grad_count = mluOpGetTensorElementNum(input_grad_desc);
  const uint64_t output_grad_count = mluOpGetTensorElementNum(output_grad_desc);
  const uint64_t filter_count = mluOpGetTensorElementNum(filters_desc);
  const uint64_t indice_pairs_count = mluOpGetTensorElementNum(indice_pairs_desc);
  if (input_grad_count >= LARGE_TENSOR_NUM || output_grad_count >= LARGE_TENSOR_NUM ||
      filter_count >= LARGE_TENSOR_NUM || indice_pairs_count >= LARGE_TENSOR_NUM) {
    LOG(ERROR) << api << " Max tensor number overflow. Tensors must have fewer than 2^31 elements.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }

  if (input_grad_count == 0 || output_grad_count == 0 || filter_count == 0 || indice_pairs_count == 0) {
    VLOG(5) << api << " Skip zero element tensor.";
    *is_zero = true;
  }
  return MLUOP_STATUS_SUCCESS;
}

ConvProblem makeProblem(mluOpHandle_t handle, const mluOpTensorDescriptor_t output_grad_desc,
                        const mluOpTensorDescriptor_t filters_desc,
                        const mluOpTensorDescriptor_t input_grad_desc) {
  const FilterDims f = readFilterDims(filters_desc);
  ConvProblem p{};
  p.L = input_grad_desc->getDimIndex(0);
  p.n_out = output_grad_desc->getDimIndex(0);
  p.K = (int32_t)f.K();
  p.ci = (int32_t)f.dxc;
  p.co = (int32_t)f.dyc;
  p.is_half = output_grad_desc->getDtype() == MLUOP_DTYPE_HALF;
  p.filter_layout = filterLayoutCode(filters_desc->getLayout());
  p.backward_data = 1;
  p.sticky_status = handle->host_only ? nullptr : handle->host_words + mluOpContext::kStickyWord;
  return p;
}

}  // namespace

extern "C" {

mluOpStatus_t MLUOP_WIN_API mluOpGetIndiceConvolutionBackwardDataWorkspaceSize(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t output_grad_desc,
    const mluOpTensorDescriptor_t filters_desc, const mluOpTensorDescriptor_t indice_pairs_desc,
    const mluOpTensorDescriptor_t input_grad_desc, const int64_t indice_num[], const int64_t inverse,
    size_t *workspace_size) {
  const std::string api = "[mluOpGetIndiceConvolutionBackwardDataWorkspaceSize]";
  if (workspace_size == nullptr) {
    LOG(ERROR) << api << " The pointer workspace_size should not be nullptr.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  bool is_zero = false;
  mluOpStatus_t st = foolCheckNoPtr(api, handle, output_grad_desc, filters_desc, indice_pairs_desc, indice_num,
                                    inverse, 0, input_grad_desc, &is_zero);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  if (is_zero) return MLUOP_STATUS_SUCCESS;
  const ConvProblem p = makeProblem(handle, output_grad_desc, filters_desc, input_grad_desc);
  *workspace_size = mluop::sparse_conv::planConvWorkspace(p).total;
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpIndiceConvolutionBackwardData(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t output_grad_desc, const void *output_grad,
    const mluOpTensorDescriptor_t filters_desc, const void *filters,
    const mluOpTensorDescriptor_t indice_pairs_desc, const void *indice_pairs, const int64_t indice_num[],
    const int64_t inverse, const int64_t sub_m, void *workspace, const size_t workspace_size,
    const mluOpTensorDescriptor_t input_grad_desc, void *input_grad) {
  const std::string api = "[mluOpIndiceConvolutionBackwardData]";
  bool is_zero = false;
  mluOpStatus_t st = foolCheckNoPtr(api, handle, output_grad_desc, filters_desc, indice_pairs_desc, indice_num,
                                    inverse, sub_m, input_grad_desc, &is_zero);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  if (is_zero) return MLUOP_STATUS_SUCCESS;
  PARAM_CHECK(api, output_grad != nullptr);
  PARAM_CHECK(api, filters != nullptr);
  PARAM_CHECK(api, indice_pairs != nullptr);
  PARAM_CHECK(api, input_grad != nullptr);
  if (workspace_size > 0) {
    PARAM_CHECK(api, workspace != nullptr);
  }
  const ConvProblem p = makeProblem(handle, output_grad_desc, filters_desc, input_grad_desc);
  const ConvWorkspacePlan plan = mluop::sparse_conv::planConvWorkspace(p);
  if (workspace_size < plan.total || workspace == nullptr) {
    LOG(ERROR) << api << " workspace of " << workspace_size << " bytes is smaller than the " << plan.total
               << " bytes mluOpGetIndiceConvolutionBackwardDataWorkspaceSize reports.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (handle->host_only) {
    LOG(ERROR) << api << " this handle was created without a CUDA device; nothing can be launched.";
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  if (mluop::takeStickyDeviceError(handle, std::string(api).c_str())) return MLUOP_STATUS_EXECUTION_FAILED;
  cudaError_t err = mluop::sparse_conv::launchIndiceConvolution(
      p, plan, output_grad, filters, static_cast<const int32_t *>(indice_pairs), indice_num, workspace,
      input_grad, handle->sm_count, handle->queue);
  if (err != cudaSuccess) {
    LOG(ERROR) << api << " launch failed: " << cudaGetErrorString(err);
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  // See mluOpIndiceConvolutionForward: MLUOP_B200_CHECK_STATUS=1 makes the call wait
  // for the stream and report a kernel whose bounded waits gave up.
  if (mluop::checkStatusRequested()) {
    int32_t word = 0;
    const char *base = reinterpret_cast<const char *>((reinterpret_cast<size_t>(workspace) + 255) / 256 * 256);
    err = cudaMemcpyAsync(&word, base + plan.status, sizeof(word), cudaMemcpyDeviceToHost, handle->queue);
    if (err == cudaSuccess) err = cudaStreamSynchronize(handle->queue);
    if (err != cudaSuccess) {
      LOG(ERROR) << api << " execution failed: " << cudaGetErrorString(err);
      return MLUOP_STATUS_EXECUTION_FAILED;
    }
    if (word != 0) {
      handle->host_words[mluOpContext::kStickyWord] = 0;  // reported here; not again by the next call
      LOG(ERROR) << api << " device reported error bits " << word << " (a bounded wait gave up).";
      return MLUOP_STATUS_EXECUTION_FAILED;
    }
  }
  return MLUOP_STATUS_SUCCESS;
}

// ---- neighbour-table fast path (no counterpart in the reference) -------------
//
// mluOpIndiceConvolutionBackwardData turns indice_pairs into its table (for every
// kernel offset and INPUT row the output row it feeds) on every call.  Layers that
// share a rulebook can build that table once and run each input gradient from it.

mluOpStatus_t MLUOP_WIN_API mluOpGetIndiceInputNeighbourTableSize(mluOpHandle_t handle,
                                                                  const mluOpTensorDescriptor_t indice_pairs_desc,
                                                                  size_t *table_size) {
  const std::string api = "[mluOpGetIndiceInputNeighbourTableSize]";
  PARAM_CHECK(api, handle != nullptr);
  PARAM_CHECK(api, indice_pairs_desc != nullptr);
  PARAM_CHECK(api, table_size != nullptr);
  PARAM_CHECK(api, indice_pairs_desc->getDim() == 3 && indice_pairs_desc->getDimIndex(1) == 2);
  PARAM_CHECK(api, indice_pairs_desc->getDtype() == MLUOP_DTYPE_INT32);
  ConvProblem p{};
  p.L = indice_pairs_desc->getDimIndex(2);
  p.K = (int32_t)indice_pairs_desc->getDimIndex(0);
  p.backward_data = 1;
  *table_size = mluop::sparse_conv::neighbourTableBytes(p);
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpBuildIndiceInputNeighbourTable(mluOpHandle_t handle,
                                                                const mluOpTensorDescriptor_t indice_pairs_desc,
                                                                const void *indice_pairs, const int64_t indice_num[],
                                                                const int64_t num_act_out, void *table,
                                                                const size_t table_size) {
  const std::string api = "[mluOpBuildIndiceInputNeighbourTable]";
  PARAM_CHECK(api, handle != nullptr);
  PARAM_CHECK(api, indice_pairs_desc != nullptr);
  PARAM_CHECK(api, indice_num != nullptr);
  PARAM_CHECK(api, indice_pairs_desc->getDim() == 3 && indice_pairs_desc->getDimIndex(1) == 2);
  PARAM_CHECK(api, indice_pairs_desc->getDtype() == MLUOP_DTYPE_INT32);
  PARAM_CHECK(api, num_act_out >= 0);
  STRIDE_TENSOR_CHECK(api + ":", indice_pairs_desc, "indice_pairs_desc must be contiguous");
  if (mluOpGetTensorElementNum(indice_pairs_desc) >= LARGE_TENSOR_NUM) {
    LOG(ERROR) << api << " Max tensor number overflow. Tensors must have fewer than 2^31 elements.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }
  ConvProblem p{};
  p.L = indice_pairs_desc->getDimIndex(2);
  p.n_out = num_act_out;
  p.K = (int32_t)indice_pairs_desc->getDimIndex(0);
  p.backward_data = 1;
  for (int32_t k = 0; k < p.K; ++k) {
    PARAM_CHECK(api, indice_num[k] >= 0 && indice_num[k] <= p.L);
  }
  if (!mluop::sparse_conv::neighbourTableCountsFit(p.K)) {
    LOG(ERROR) << api << " kernel volumes above 128 are not supported by the table path.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }
  const size_t need = mluop::sparse_conv::neighbourTableBytes(p);
  if (need == 0 || p.L == 0) return MLUOP_STATUS_SUCCESS;
  PARAM_CHECK(api, indice_pairs != nullptr);
  PARAM_CHECK(api, table != nullptr);
  PARAM_CHECK(api, reinterpret_cast<size_t>(table) % 16 == 0);
  if (table_size < need) {
    LOG(ERROR) << api << " table of " << table_size << " bytes is smaller than the " << need
               << " bytes mluOpGetIndiceInputNeighbourTableSize reports.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (handle->host_only) {
    LOG(ERROR) << api << " this handle was created without a CUDA device; nothing can be launched.";
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  if (mluop::takeStickyDeviceError(handle, std::string(api).c_str())) return MLUOP_STATUS_EXECUTION_FAILED;
  const ConvWorkspacePlan plan = mluop::sparse_conv::planConvWorkspace(p, true);
  cudaError_t err = mluop::sparse_conv::launchIndiceConvolutionSteps(
      p, plan, nullptr, nullptr, static_cast<const int32_t *>(indice_pairs), indice_num, nullptr, nullptr,
      handle->sm_count, handle->queue, static_cast<int32_t *>(table), mluop::sparse_conv::kTableBuildOnly);
  if (err != cudaSuccess) {
    LOG(ERROR) << api << " launch failed: " << cudaGetErrorString(err);
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpGetIndiceConvolutionBackwardDataFromTableWorkspaceSize(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t output_grad_desc,
    const mluOpTensorDescriptor_t filters_desc, const mluOpTensorDescriptor_t indice_pairs_desc,
    const mluOpTensorDescriptor_t input_grad_desc, const int64_t indice_num[], const int64_t inverse,
    size_t *workspace_size) {
  const std::string api = "[mluOpGetIndiceConvolutionBackwardDataFromTableWorkspaceSize]";
  PARAM_CHECK(api, workspace_size != nullptr);
  bool is_zero = false;
  mluOpStatus_t st = foolCheckNoPtr(api, handle, output_grad_desc, filters_desc, indice_pairs_desc, indice_num,
                                    inverse, 0, input_grad_desc, &is_zero);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  *workspace_size = 0;
  if (is_zero) return MLUOP_STATUS_SUCCESS;
  const ConvProblem p = makeProblem(handle, output_grad_desc, filters_desc, input_grad_desc);
  *workspace_size = mluop::sparse_conv::planConvWorkspace(p, true).total;
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpIndiceConvolutionBackwardDataFromTable(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t output_grad_desc, const void *output_grad,
    const mluOpTensorDescriptor_t filters_desc, const void *filters,
    const mluOpTensorDescriptor_t indice_pairs_desc, const void *table, const size_t table_size,
    const int64_t indice_num[], const int64_t inverse, const int64_t sub_m, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t input_grad_desc, void *input_grad) {
  const std::string api = "[mluOpIndiceConvolutionBackwardDataFromTable]";
  bool is_zero = false;
  mluOpStatus_t st = foolCheckNoPtr(api, handle, output_grad_desc, filters_desc, indice_pairs_desc, indice_num,
                                    inverse, sub_m, input_grad_desc, &is_zero);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  if (is_zero) return MLUOP_STATUS_SUCCESS;
  PARAM_CHECK(api, output_grad != nullptr);
  PARAM_CHECK(api, filters != nullptr);
  PARAM_CHECK(api, table != nullptr);
  PARAM_CHECK(api, input_grad != nullptr);
  PARAM_CHECK(api, workspace != nullptr);
  PARAM_CHECK(api, reinterpret_cast<size_t>(table) % 16 == 0);  // read 16 bytes at a time
  const ConvProblem p = makeProblem(handle, output_grad_desc, filters_desc, input_grad_desc);
  if (!mluop::sparse_conv::neighbourTableCountsFit(p.K)) {
    LOG(ERROR) << api << " kernel volumes above 128 are not supported by the table path.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }
  const ConvWorkspacePlan plan = mluop::sparse_conv::planConvWorkspace(p, true);
  const size_t need = mluop::sparse_conv::neighbourTableBytes(p);
  if (workspace_size < plan.total || table_size < need) {
    LOG(ERROR) << api << " workspace (" << workspace_size << " of " << plan.total << " bytes) or table ("
               << table_size << " of " << need << " bytes) is smaller than the size queries report.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (handle->host_only) {
    LOG(ERROR) << api << " this handle was created without a CUDA device; nothing can be launched.";
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  if (mluop::takeStickyDeviceError(handle, std::string(api).c_str())) return MLUOP_STATUS_EXECUTION_FAILED;
  cudaError_t err = mluop::sparse_conv::launchIndiceConvolutionSteps(
      p, plan, output_grad, filters, nullptr, indice_num, workspace, input_grad, handle->sm_count, handle->queue,
      const_cast<int32_t *>(static_cast<const int32_t *>(table)), mluop::sparse_conv::kTableConvolveOnly);
  if (err != cudaSuccess) {
    LOG(ERROR) << api << " launch failed: " << cudaGetErrorString(err);
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  return MLUOP_STATUS_SUCCESS;
}

// The input gradient of a SUBMANIFOLD layer with centred padding straight from the rulebook's
// FORWARD table (the one the forward convolutions run from): its pairs are symmetric, (i, o) at
// offset k goes with (o, i) at offset K-1-k, so the kernel reads the forward table with the
// offsets mirrored and no table of the opposite direction is ever built.  The caller vouches
// for the geometry (stride 1, dilation 1, odd kernel extents, pad = extent / 2: what
// mluOpGetIndicePairsWithNeighbourTable accepts).  Only the tensor-memory kernel reads a table
// this way: other shapes are MLUOP_STATUS_NOT_SUPPORTED before anything is enqueued, and the
// caller uses mluOpIndiceConvolutionBackwardDataFromTable with an input table.  Workspace as for
// that entry point.
mluOpStatus_t MLUOP_WIN_API mluOpIndiceConvolutionBackwardDataFromForwardTable(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t output_grad_desc, const void *output_grad,
    const mluOpTensorDescriptor_t filters_desc, const void *filters,
    const mluOpTensorDescriptor_t indice_pairs_desc, const void *table, const size_t table_size,
    const int64_t indice_num[], const int64_t inverse, const int64_t sub_m, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t input_grad_desc, void *input_grad) {
  const std::string api = "[mluOpIndiceConvolutionBackwardDataFromForwardTable]";
  bool is_zero = false;
  mluOpStatus_t st = foolCheckNoPtr(api, handle, output_grad_desc, filters_desc, indice_pairs_desc, indice_num,
                                    inverse, sub_m, input_grad_desc, &is_zero);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  if (is_zero) return MLUOP_STATUS_SUCCESS;
  PARAM_CHECK(api, output_grad != nullptr);
  PARAM_CHECK(api, filters != nullptr);
  PARAM_CHECK(api, table != nullptr);
  PARAM_CHECK(api, input_grad != nullptr);
  PARAM_CHECK(api, workspace != nullptr);
  PARAM_CHECK(api, reinterpret_cast<size_t>(table) % 16 == 0);  // read 16 bytes at a time
  PARAM_CHECK(api, sub_m == 1);  // only a submanifold rulebook is symmetric
  ConvProblem p = makeProblem(handle, output_grad_desc, filters_desc, input_grad_desc);
  PARAM_CHECK(api, p.L == p.n_out);
  p.mirror_table = 1;
  if (!mluop::sparse_conv::neighbourTableCountsFit(p.K) ||
      !mluop::sparse_conv::convRunsOnTensorMemory(p, output_grad, input_grad)) {
    // an answer, not an error: callers try this entry point first
    VLOG(5) << api << " only the tensor-memory kernel (half, channel counts that are multiples of 8 up to 128, "
            << "16-byte aligned rows, kernel volume up to 128) reads a mirrored table.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }
  const ConvWorkspacePlan plan = mluop::sparse_conv::planConvWorkspace(p, true);
  const size_t need = mluop::sparse_conv::neighbourTableBytes(p);
  if (workspace_size < plan.total || table_size < need) {
    LOG(ERROR) << api << " workspace (" << workspace_size << " of " << plan.total << " bytes) or table ("
               << table_size << " of " << need << " bytes) is smaller than the size queries report.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (handle->host_only) {
    LOG(ERROR) << api << " this handle was created without a CUDA device; nothing can be launched.";
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  if (mluop::takeStickyDeviceError(handle, std::string(api).c_str())) return MLUOP_STATUS_EXECUTION_FAILED;
  cudaError_t err = mluop::sparse_conv::launchIndiceConvolutionSteps(
      p, plan, output_grad, filters, nullptr, indice_num, workspace, input_grad, handle->sm_count, handle->queue,
      const_cast<int32_t *>(static_cast<const int32_t *>(table)), mluop::sparse_conv::kTableConvolveOnly);
  if (err != cudaSuccess) {
    LOG(ERROR) << api << " launch failed: " << cudaGetErrorString(err);
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  return MLUOP_STATUS_SUCCESS;
}

}  // extern "C"
