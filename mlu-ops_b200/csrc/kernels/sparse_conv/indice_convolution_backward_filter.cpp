// mluOpIndiceConvolutionBackwardFilter / mluOpGetIndiceConvolutionBackwardFilterWorkspaceSize:
// argument checks and dispatch (reference
// kernels/sparse_conv/indice_convolution_backward_filter/indice_convolution_backward_filter.cpp:
// indiceConvDtypeVaild :100-172, baseParamCheck :174-258, workspace query :531-568,
// compute entry :570-620).
//
//   filters_grad[k,c,n] = sum_{(i,o) in pairs_k} features[i,c] * output_grad[o,n]
//
// The order of the checks, and the status each returns, follows the reference.
// Like the reference, the result is always written in [kd,kh,kw,Ci,Co] order and
// the channel counts are read from the last two dimensions of filters_grad
// (reference :226-235: "only DHWCN/HWCN layout of filter_grad is supported").
// Two differences: the reference refuses more than 1,000,000 input rows
// (get_indice_pairs_structs.h:36), here the bound is only that every tensor has
// fewer than 2^31 elements; descriptors here carry no separate on-chip data
// type, so the reference's checks of it have nothing to look at.
#include <cuda_runtime_api.h>

#include <string>

#include "core/context.h"
#include "core/logging.h"
#include "core/tensor.h"
#include "kernels/sparse_conv/indice_convolution_backward_filter_kernels.h"
#include "kernels/sparse_conv/indice_convolution_kernels.h"

using mluop::sparse_conv::FilterGradProblem;
using mluop::sparse_conv::FilterGradWorkspacePlan;

namespace {

bool isFloatDtype(mluOpDataType_t t) { return t == MLUOP_DTYPE_HALF || t == MLUOP_DTYPE_FLOAT; }

std::string shapeString(const mluOpTensorDescriptor_t d) {
  std::string s = "[";
  for (int i = 0; i < d->getDim(); ++i) s += (i ? "," : "") + std::to_string(d->getDimIndex(i));
  return s + "]";
}

mluOpStatus_t baseParamCheck(const std::string &api, mluOpHandle_t handle,
                             const mluOpTensorDescriptor_t features_desc,
                             const mluOpTensorDescriptor_t output_grad_desc,
                             const mluOpTensorDescriptor_t indice_pairs_desc,
                             const mluOpTensorDescriptor_t filters_grad_desc, const int64_t indice_num[],
                             const int64_t inverse) {
  PARAM_CHECK(api, handle != nullptr);
  PARAM_CHECK(api, features_desc != nullptr);
  PARAM_CHECK(api, output_grad_desc != nullptr);
  PARAM_CHECK(api, indice_pairs_desc != nullptr);
  PARAM_CHECK(api, filters_grad_desc != nullptr);
  PARAM_CHECK(api, indice_num != nullptr);
  PARAM_CHECK(api, inverse == 0);

  STRIDE_TENSOR_CHECK(api + ":", features_desc, "features_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", output_grad_desc, "output_grad_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", indice_pairs_desc, "indice_pairs_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", filters_grad_desc, "filters_grad_desc must be contiguous");

  if (handle->arch < MLUOP_MLU370) {
    LOG(ERROR) << api << " needs a compute-capability 10.x device; this handle's device is not one.";
    return MLUOP_STATUS_ARCH_MISMATCH;
  }

  const mluOpDataType_t in_t = features_desc->getDtype();
  const mluOpDataType_t dy_t = output_grad_desc->getDtype();
  const mluOpDataType_t dw_t = filters_grad_desc->getDtype();
  if (indice_pairs_desc->getDtype() != MLUOP_DTYPE_INT32) {
    LOG(ERROR) << api << " indice_pairs_desc only supports data type int32. But now the data type is "
               << mluop::getNameOfDataType(indice_pairs_desc->getDtype()) << ".";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (in_t != dy_t || in_t != dw_t || !isFloatDtype(in_t)) {
    LOG(ERROR) << api << " The data type of features_desc, output_grad_desc and filters_grad_desc should be the "
               << "same and the three should be either half or float. But now the data types are "
               << mluop::getNameOfDataType(in_t) << "-" << mluop::getNameOfDataType(dy_t) << "-"
               << mluop::getNameOfDataType(dw_t) << ".";
    return MLUOP_STATUS_BAD_PARAM;
  }

  if (mluOpGetTensorElementNum(features_desc) >= LARGE_TENSOR_NUM ||
      mluOpGetTensorElementNum(output_grad_desc) >= LARGE_TENSOR_NUM ||
      mluOpGetTensorElementNum(indice_pairs_desc) >= LARGE_TENSOR_NUM ||
      mluOpGetTensorElementNum(filters_grad_desc) >= LARGE_TENSOR_NUM) {
    LOG(ERROR) << api << " Overflow max tensor num. Tensors must have fewer than 2^31 elements.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }

  bool shape_ok = features_desc->getDim() == 2 && output_grad_desc->getDim() == 2 &&
                  indice_pairs_desc->getDim() == 3 &&
                  (filters_grad_desc->getDim() == 4 || filters_grad_desc->getDim() == 5);
  if (shape_ok) {
    const int n = filters_grad_desc->getDim();
    const int64_t ci = filters_grad_desc->getDimIndex(n - 2);
    const int64_t co = filters_grad_desc->getDimIndex(n - 1);
    const int64_t kd = n == 4 ? 1 : filters_grad_desc->getDimIndex(0);
    const int64_t kh = filters_grad_desc->getDimIndex(n - 4);
    const int64_t kw = filters_grad_desc->getDimIndex(n - 3);
    shape_ok = ci == features_desc->getDimIndex(1) && co == output_grad_desc->getDimIndex(1) &&
               features_desc->getDimIndex(0) == indice_pairs_desc->getDimIndex(2) &&
               indice_pairs_desc->getDimIndex(1) == 2 && kd * kh * kw == indice_pairs_desc->getDimIndex(0);
  }
  if (!shape_ok) {
    LOG(ERROR) << api << " Shape check failed! Now the shapes are features_desc" << shapeString(features_desc)
               << ", output_grad_desc" << shapeString(output_grad_desc) << ", indice_pairs_desc"
               << shapeString(indice_pairs_desc) << ", and filters_grad_desc"
               << shapeString(filters_grad_desc) << ".";
    return MLUOP_STATUS_BAD_PARAM;
  }
  return MLUOP_STATUS_SUCCESS;
}

// Every pair count must fit its list (the reference leaves this to the matmul it
// calls; here a count is a loop bound on the GPU).  Checked after the
// zero-element return, like the reference's own use of the counts.
mluOpStatus_t pairCountCheck(const std::string &api, const mluOpTensorDescriptor_t indice_pairs_desc,
                             const int64_t indice_num[]) {
  const int64_t K = indice_pairs_desc->getDimIndex(0);
  for (int64_t k = 0; k < K; ++k) {
    const std::string where = "k: " + std::to_string(k) + ".";
    PARAM_CHECK_V2(api, indice_num[k] >= 0 && indice_num[k] <= indice_pairs_desc->getDimIndex(2), << where);
  }
  return MLUOP_STATUS_SUCCESS;
}

bool anyZeroElement(const mluOpTensorDescriptor_t a, const mluOpTensorDescriptor_t b,
                    const mluOpTensorDescriptor_t c, const mluOpTensorDescriptor_t d) {
  return mluOpGetTensorElementNum(a) == 0 || mluOpGetTensorElementNum(b) == 0 ||
         mluOpGetTensorElementNum(c) == 0 || mluOpGetTensorElementNum(d) == 0;
}

FilterGradProblem makeProblem(const mluOpTensorDescriptor_t features_desc,
                              const mluOpTensorDescriptor_t output_grad_desc,
                              const mluOpTensorDescriptor_t indice_pairs_desc) {
  FilterGradProblem p{};
  p.L = features_desc->getDimIndex(0);
  p.n_out = output_grad_desc->getDimIndex(0);
  p.K = (int32_t)indice_pairs_desc->getDimIndex(0);
  p.ci = (int32_t)features_desc->getDimIndex(1);
  p.co = (int32_t)output_grad_desc->getDimIndex(1);
  p.is_half = features_desc->getDtype() == MLUOP_DTYPE_HALF;
  return p;
}

// The tensor-memory kernel records a bounded wait that gave up in a status word of the workspace
// (and in the handle's sticky word).  MLUOP_B200_CHECK_STATUS=1 makes the call wait for the
// stream and report it itself (debugging and tests).
mluOpStatus_t reportKernelStatus(const std::string &api, mluOpHandle_t handle, const FilterGradProblem &p,
                                 const FilterGradWorkspacePlan &plan, const void *features, const void *output_grad,
                                 const void *workspace) {
  if (!mluop::checkStatusRequested() ||
      !mluop::sparse_conv::filterGradRunsFromTable(p, plan, features, output_grad)) {
    return MLUOP_STATUS_SUCCESS;
  }
  int32_t word = 0;
  const char *base = reinterpret_cast<const char *>((reinterpret_cast<size_t>(workspace) + 255) / 256 * 256);
  cudaError_t err = cudaMemcpyAsync(&word, base + plan.tc_status, sizeof(word), cudaMemcpyDeviceToHost, handle->queue);
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
  return MLUOP_STATUS_SUCCESS;
}

}  // namespace

extern "C" {

mluOpStatus_t MLUOP_WIN_API mluOpGetIndiceConvolutionBackwardFilterWorkspaceSize(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc,
    const mluOpTensorDescriptor_t output_grad_desc, const mluOpTensorDescriptor_t indice_pairs_desc,
    const mluOpTensorDescriptor_t filters_grad_desc, const int64_t indice_num[], const int64_t inverse,
    const int64_t sub_m, size_t *size) {
  const std::string api = "[mluOpGetIndiceConvolutionBackwardFilterWorkspaceSize]";
  (void)sub_m;
  PARAM_CHECK(api, size != nullptr);
  mluOpStatus_t st = baseParamCheck(api, handle, features_desc, output_grad_desc, indice_pairs_desc,
                                    filters_grad_desc, indice_num, inverse);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  if (anyZeroElement(features_desc, output_grad_desc, indice_pairs_desc, filters_grad_desc)) {
    VLOG(5) << api << " Skip zero element tensor.";
    return MLUOP_STATUS_SUCCESS;
  }
  st = pairCountCheck(api, indice_pairs_desc, indice_num);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  const FilterGradProblem p = makeProblem(features_desc, output_grad_desc, indice_pairs_desc);
  *size = mluop::sparse_conv::planFilterGradWorkspace(p, indice_num, handle->sm_count).total;
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpIndiceConvolutionBackwardFilter(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc, const void *features,
    const mluOpTensorDescriptor_t output_grad_desc, const void *output_grad,
    const mluOpTensorDescriptor_t indice_pairs_desc, const void *indice_pairs, const int64_t indice_num[],
    const int64_t inverse, const int64_t sub_m, void *workspace, const size_t workspace_size,
    const mluOpTensorDescriptor_t filters_grad_desc, void *filters_grad) {
  const std::string api = "[mluOpIndiceConvolutionBackwardFilter]";
  (void)sub_m;
  mluOpStatus_t st = baseParamCheck(api, handle, features_desc, output_grad_desc, indice_pairs_desc,
                                    filters_grad_desc, indice_num, inverse);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  if (anyZeroElement(features_desc, output_grad_desc, indice_pairs_desc, filters_grad_desc)) {
    VLOG(5) << api << " Skip zero element tensor.";
    return MLUOP_STATUS_SUCCESS;
  }
  st = pairCountCheck(api, indice_pairs_desc, indice_num);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  PARAM_CHECK(api, features != nullptr);
  PARAM_CHECK(api, output_grad != nullptr);
  PARAM_CHECK(api, indice_pairs != nullptr);
  PARAM_CHECK(api, filters_grad != nullptr);
  if (workspace_size > 0) {
    PARAM_CHECK(api, workspace != nullptr);
  }
  FilterGradProblem p = makeProblem(features_desc, output_grad_desc, indice_pairs_desc);
  p.sticky_status = handle->host_only ? nullptr : handle->host_words + mluOpContext::kStickyWord;
  const FilterGradWorkspacePlan plan =
      mluop::sparse_conv::planFilterGradWorkspace(p, indice_num, handle->sm_count);
  if (workspace_size < plan.total || workspace == nullptr) {
    LOG(ERROR) << api << " workspace of " << workspace_size << " bytes is smaller than the " << plan.total
               << " bytes mluOpGetIndiceConvolutionBackwardFilterWorkspaceSize reports.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (handle->host_only) {
    LOG(ERROR) << api << " this handle was created without a CUDA device; nothing can be launched.";
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  if (mluop::takeStickyDeviceError(handle, std::string(api).c_str())) return MLUOP_STATUS_EXECUTION_FAILED;
  cudaError_t err = mluop::sparse_conv::launchIndiceConvolutionBackwardFilter(
      p, plan, features, output_grad, static_cast<const int32_t *>(indice_pairs), indice_num, workspace,
      filters_grad, handle->sm_count, handle->queue);
  if (err != cudaSuccess) {
    LOG(ERROR) << api << " launch failed: " << cudaGetErrorString(err);
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  return reportKernelStatus(api, handle, p, plan, features, output_grad, workspace);
}

// ---- neighbour-table fast path (no counterpart in the reference) -------------
//
// The tensor-memory kernel works from the FORWARD convolution's neighbour table
// (mluOpBuildIndiceNeighbourTable, or the one mluOpGetIndicePairsWithNeighbourTable
// emitted) and builds it from indice_pairs on every call; a caller that kept the
// table hands it over instead.  Shapes the kernel does not take (anything but half
// with 64 input and 64 or 128 output channels) are MLUOP_STATUS_NOT_SUPPORTED: the
// caller uses mluOpIndiceConvolutionBackwardFilter.  The workspace is the one
// mluOpGetIndiceConvolutionBackwardFilterWorkspaceSize reports.

mluOpStatus_t MLUOP_WIN_API mluOpIndiceConvolutionBackwardFilterFromTable(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc, const void *features,
    const mluOpTensorDescriptor_t output_grad_desc, const void *output_grad,
    const mluOpTensorDescriptor_t indice_pairs_desc, const void *table, const size_t table_size,
    const int64_t indice_num[], const int64_t inverse, const int64_t sub_m, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t filters_grad_desc, void *filters_grad) {
  const std::string api = "[mluOpIndiceConvolutionBackwardFilterFromTable]";
  (void)sub_m;
  mluOpStatus_t st = baseParamCheck(api, handle, features_desc, output_grad_desc, indice_pairs_desc,
                                    filters_grad_desc, indice_num, inverse);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  if (anyZeroElement(features_desc, output_grad_desc, indice_pairs_desc, filters_grad_desc)) {
    VLOG(5) << api << " Skip zero element tensor.";
    return MLUOP_STATUS_SUCCESS;
  }
  st = pairCountCheck(api, indice_pairs_desc, indice_num);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  PARAM_CHECK(api, features != nullptr);
  PARAM_CHECK(api, output_grad != nullptr);
  PARAM_CHECK(api, table != nullptr);
  PARAM_CHECK(api, filters_grad != nullptr);
  PARAM_CHECK(api, workspace != nullptr);
  PARAM_CHECK(api, reinterpret_cast<size_t>(table) % 16 == 0);  // read 16 bytes at a time
  FilterGradProblem p = makeProblem(features_desc, output_grad_desc, indice_pairs_desc);
  p.sticky_status = handle->host_only ? nullptr : handle->host_words + mluOpContext::kStickyWord;
  const FilterGradWorkspacePlan plan =
      mluop::sparse_conv::planFilterGradWorkspace(p, indice_num, handle->sm_count);
  if (!mluop::sparse_conv::filterGradRunsFromTable(p, plan, features, output_grad)) {
    // an answer, not an error: callers try this entry point first
    VLOG(5) << api << " only half tensors with 64 input and 64 or 128 output channels (16-byte aligned) run "
            << "from a neighbour table; use mluOpIndiceConvolutionBackwardFilter.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }
  mluop::sparse_conv::ConvProblem cp{};
  cp.L = p.L;
  cp.n_out = p.n_out;
  cp.K = p.K;
  const size_t need = mluop::sparse_conv::neighbourTableBytes(cp);
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
  cudaError_t err = mluop::sparse_conv::launchIndiceConvolutionBackwardFilter(
      p, plan, features, output_grad, nullptr, indice_num, workspace, filters_grad, handle->sm_count, handle->queue,
      static_cast<const int32_t *>(table));
  if (err != cudaSuccess) {
    LOG(ERROR) << api << " launch failed: " << cudaGetErrorString(err);
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  return reportKernelStatus(api, handle, p, plan, features, output_grad, workspace);
}

}  // extern "C"
