// mluOpIndiceConvolutionForward / mluOpGetIndiceConvolutionForwardWorkspaceSize:
// argument checks and dispatch (reference
// kernels/sparse_conv/indice_convolution_forward/indice_convolution_forward.cpp:
// foolProof :37-169, workspace query :581-619, compute entry :621-686).
//
// The order of the checks, and which status each one returns, follows the
// reference.  One limit differs: the reference refuses more than 1,000,000
// input rows (get_indice_pairs_structs.h:36); here the bound is only that
// every tensor has fewer than 2^31 elements.
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

struct FilterShape {
  int64_t ci = 0, co = 0, num_filter = 0;
  int layout = 0;
};

FilterShape readFilterShape(const mluOpTensorDescriptor_t filters_desc) {
  FilterShape s;
  if (filters_desc->getLayout() == MLUOP_LAYOUT_ARRAY) {
    s.ci = filters_desc->getDimIndex(3);
    s.co = filters_desc->getDimIndex(4);
    s.num_filter = filters_desc->getDimIndex(0) * filters_desc->getDimIndex(1) * filters_desc->getDimIndex(2);
    s.layout = mluop::sparse_conv::kFilterArray;
  } else {
    s.ci = mluOpGetTensordimC(filters_desc);
    s.co = mluOpGetTensordimN(filters_desc);
    s.num_filter =
        mluOpGetTensordimD(filters_desc) * mluOpGetTensordimH(filters_desc) * mluOpGetTensordimW(filters_desc);
    s.layout = filters_desc->getLayout() == MLUOP_LAYOUT_NDHWC ? mluop::sparse_conv::kFilterNDHWC
                                                               : mluop::sparse_conv::kFilterNCDHW;
  }
  return s;
}

mluOpStatus_t foolProof(const std::string &api, mluOpHandle_t handle,
                        const mluOpTensorDescriptor_t features_desc,
                        const mluOpTensorDescriptor_t filters_desc,
                        const mluOpTensorDescriptor_t indice_pairs_desc, const int64_t indice_num[],
                        const int64_t num_act_out, const int64_t inverse, const int64_t sub_m,
                        const mluOpTensorDescriptor_t features_out_desc) {
  PARAM_CHECK(api, handle != nullptr);
  PARAM_CHECK(api, features_desc != nullptr);
  PARAM_CHECK(api, filters_desc != nullptr);
  PARAM_CHECK(api, indice_pairs_desc != nullptr);
  PARAM_CHECK(api, indice_num != nullptr);
  PARAM_CHECK(api, features_out_desc != nullptr);

  if (handle->arch < MLUOP_MLU370) {
    LOG(ERROR) << api << " needs a compute-capability 10.x device; this handle's device is not one.";
    return MLUOP_STATUS_ARCH_MISMATCH;
  }

  PARAM_CHECK(api, features_desc->getDtype() == MLUOP_DTYPE_FLOAT ||
                       features_desc->getDtype() == MLUOP_DTYPE_HALF);
  PARAM_CHECK(api, filters_desc->getDtype() == MLUOP_DTYPE_FLOAT ||
                       filters_desc->getDtype() == MLUOP_DTYPE_HALF);
  PARAM_CHECK(api, indice_pairs_desc->getDtype() == MLUOP_DTYPE_INT32);
  PARAM_CHECK(api, features_out_desc->getDtype() == MLUOP_DTYPE_FLOAT ||
                       features_out_desc->getDtype() == MLUOP_DTYPE_HALF);
  PARAM_CHECK(api, features_desc->getDtype() == features_out_desc->getDtype() &&
                       features_desc->getDtype() == filters_desc->getDtype());

  PARAM_CHECK(api, sub_m == 0 || sub_m == 1);
  PARAM_CHECK(api, inverse == 0 || inverse == 1);
  if (inverse != 0) {
    LOG(ERROR) << api << " inverse is: " << inverse << ", which is not supported now.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }

  if (filters_desc->getLayout() != MLUOP_LAYOUT_NDHWC && filters_desc->getLayout() != MLUOP_LAYOUT_NCDHW &&
      filters_desc->getLayout() != MLUOP_LAYOUT_ARRAY) {
    LOG(ERROR) << api << " The layout of filters is: "
               << mluop::getNameOfTensorLayout(filters_desc->getLayout()) << ", which is not supported now.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }

  PARAM_CHECK(api, features_desc->getDim() == 2);
  PARAM_CHECK(api, indice_pairs_desc->getDim() == 3);
  PARAM_CHECK(api, features_out_desc->getDim() == 2);
  if (filters_desc->getDim() != 5) {
    LOG(ERROR) << api << " The filters dimension number only support 5 currently, but filters dimension "
               << "number is :" << filters_desc->getDim() << ".";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }

  STRIDE_TENSOR_CHECK(api + ":", features_desc, "features_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", filters_desc, "filters_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", indice_pairs_desc, "indice_pairs_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", features_out_desc, "features_out_desc must be contiguous");

  if (mluOpGetTensorElementNum(features_desc) >= LARGE_TENSOR_NUM ||
      mluOpGetTensorElementNum(filters_desc) >= LARGE_TENSOR_NUM ||
      mluOpGetTensorElementNum(indice_pairs_desc) >= LARGE_TENSOR_NUM ||
      mluOpGetTensorElementNum(features_out_desc) >= LARGE_TENSOR_NUM) {
    LOG(ERROR) << api << " Max tensor number overflow. Tensors must have fewer than 2^31 elements.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }

  const FilterShape fs = readFilterShape(filters_desc);

  PARAM_CHECK(api, features_desc->getDimIndex(0) == indice_pairs_desc->getDimIndex(2));
  PARAM_CHECK(api, features_desc->getDimIndex(1) == fs.ci);
  PARAM_CHECK(api, indice_pairs_desc->getDimIndex(0) == fs.num_filter);
  PARAM_CHECK(api, indice_pairs_desc->getDimIndex(1) == 2);
  PARAM_CHECK(api, features_out_desc->getDimIndex(0) == num_act_out);
  PARAM_CHECK(api, features_out_desc->getDimIndex(1) == fs.co);

  for (int64_t i = 0; i < fs.num_filter; ++i) {
    const std::string where = "i: " + std::to_string(i) + ".";
    PARAM_CHECK_V2(api, indice_num[i] >= 0 && indice_num[i] <= features_desc->getDimIndex(0), << where);
  }
  return MLUOP_STATUS_SUCCESS;
}

bool anyZeroElement(const mluOpTensorDescriptor_t a, const mluOpTensorDescriptor_t b,
                    const mluOpTensorDescriptor_t c, const mluOpTensorDescriptor_t d) {
  return mluOpGetTensorElementNum(a) == 0 || mluOpGetTensorElementNum(b) == 0 ||
         mluOpGetTensorElementNum(c) == 0 || mluOpGetTensorElementNum(d) == 0;
}

ConvProblem makeProblem(mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc,
                        const mluOpTensorDescriptor_t filters_desc, int64_t num_act_out) {
  const FilterShape fs = readFilterShape(filters_desc);
  ConvProblem p{};
  p.L = features_desc->getDimIndex(0);
  p.n_out = num_act_out;
  p.K = (int32_t)fs.num_filter;
  p.ci = (int32_t)fs.ci;
  p.co = (int32_t)fs.co;
  p.is_half = features_desc->getDtype() == MLUOP_DTYPE_HALF;
  p.filter_layout = fs.layout;
  p.sticky_status = handle->host_only ? nullptr : handle->host_words + mluOpContext::kStickyWord;
  return p;
}

}  // namespace

extern "C" {

mluOpStatus_t MLUOP_WIN_API mluOpGetIndiceConvolutionForwardWorkspaceSize(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc,
    const mluOpTensorDescriptor_t filters_desc, const mluOpTensorDescriptor_t indice_pairs_desc,
    const mluOpTensorDescriptor_t features_out_desc, const int64_t indice_num[], const int64_t num_act_out,
    const int64_t inverse, const int64_t sub_m, size_t *size) {
  const std::string api = "[mluOpGetIndiceConvolutionForwardWorkspaceSize]";
  mluOpStatus_t st = foolProof(api, handle, features_desc, filters_desc, indice_pairs_desc, indice_num,
                               num_act_out, inverse, sub_m, features_out_desc);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  if (anyZeroElement(features_desc, indice_pairs_desc, filters_desc, features_out_desc)) {
    VLOG(5) << api << " Skip zero element tensor.";
    return MLUOP_STATUS_SUCCESS;
  }
  PARAM_CHECK(api, size != nullptr);
  const ConvProblem p = makeProblem(handle, features_desc, filters_desc, num_act_out);
  *size = mluop::sparse_conv::planConvWorkspace(p).total;
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpIndiceConvolutionForward(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc, const void *features,
    const mluOpTensorDescriptor_t filters_desc, const void *filters,
    const mluOpTensorDescriptor_t indice_pairs_desc, const void *indice_pairs, const int64_t indice_num[],
    const int64_t num_act_out, const int64_t inverse, const int64_t sub_m, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t features_out_desc, void *features_out) {
  const std::string api = "[mluOpIndiceConvolutionForward]";
  mluOpStatus_t st = foolProof(api, handle, features_desc, filters_desc, indice_pairs_desc, indice_num,
                               num_act_out, inverse, sub_m, features_out_desc);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  if (anyZeroElement(filters_desc, features_desc, indice_pairs_desc, features_out_desc)) {
    VLOG(5) << api << " Skip zero element tensor.";
    return MLUOP_STATUS_SUCCESS;
  }
  PARAM_CHECK(api, features != nullptr);
  PARAM_CHECK(api, filters != nullptr);
  PARAM_CHECK(api, indice_pairs != nullptr);
  PARAM_CHECK(api, features_out != nullptr);
  if (workspace_size > 0) {
    PARAM_CHECK(api, workspace != nullptr);
  }
  const ConvProblem p = makeProblem(handle, features_desc, filters_desc, num_act_out);
  const ConvWorkspacePlan plan = mluop::sparse_conv::planConvWorkspace(p);
  if (workspace_size < plan.total || workspace == nullptr) {
    LOG(ERROR) << api << " workspace of " << workspace_size << " bytes is smaller than the " << plan.total
               << " bytes mluOpGetIndiceConvolutionForwardWorkspaceSize reports.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (handle->host_only) {
    LOG(ERROR) << api << " this handle was created without a CUDA device; nothing can be launched.";
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  if (mluop::takeStickyDeviceError(handle, std::string(api).c_str())) return MLUOP_STATUS_EXECUTION_FAILED;
  cudaError_t err = mluop::sparse_conv::launchIndiceConvolution(
      p, plan, features, filters, static_cast<const int32_t *>(indice_pairs), indice_num, workspace,
      features_out, handle->sm_count, handle->queue);
  if (err != cudaSuccess) {
    LOG(ERROR) << api << " launch failed: " << cudaGetErrorString(err);
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  // The call is asynchronous; a kernel whose bounded waits gave up records that
  // in a status word of the workspace.  MLUOP_B200_CHECK_STATUS=1 makes the call
  // wait for the stream and report such a failure (debugging and tests).
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
// mluOpIndiceConvolutionForward turns indice_pairs into its neighbour table on
// every call.  Layers that share a rulebook (the submanifold blocks of a
// backbone) can build the table once and run each convolution from it.

mluOpStatus_t MLUOP_WIN_API mluOpGetIndiceNeighbourTableSize(mluOpHandle_t handle,
                                                             const mluOpTensorDescriptor_t indice_pairs_desc,
                                                             const int64_t num_act_out, size_t *table_size) {
  const std::string api = "[mluOpGetIndiceNeighbourTableSize]";
  PARAM_CHECK(api, handle != nullptr);
  PARAM_CHECK(api, indice_pairs_desc != nullptr);
  PARAM_CHECK(api, table_size != nullptr);
  PARAM_CHECK(api, indice_pairs_desc->getDim() == 3 && indice_pairs_desc->getDimIndex(1) == 2);
  PARAM_CHECK(api, indice_pairs_desc->getDtype() == MLUOP_DTYPE_INT32);
  PARAM_CHECK(api, num_act_out >= 0);
  ConvProblem p{};
  p.L = indice_pairs_desc->getDimIndex(2);
  p.n_out = num_act_out;
  p.K = (int32_t)indice_pairs_desc->getDimIndex(0);
  *table_size = mluop::sparse_conv::neighbourTableBytes(p);
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpBuildIndiceNeighbourTable(mluOpHandle_t handle,
                                                           const mluOpTensorDescriptor_t indice_pairs_desc,
                                                           const void *indice_pairs, const int64_t indice_num[],
                                                           const int64_t num_act_out, void *table,
                                                           const size_t table_size) {
  const std::string api = "[mluOpBuildIndiceNeighbourTable]";
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
               << " bytes mluOpGetIndiceNeighbourTableSize reports.";
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

mluOpStatus_t MLUOP_WIN_API mluOpGetIndiceConvolutionForwardFromTableWorkspaceSize(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc,
    const mluOpTensorDescriptor_t filters_desc, const mluOpTensorDescriptor_t indice_pairs_desc,
    const mluOpTensorDescriptor_t features_out_desc, const int64_t indice_num[], const int64_t num_act_out,
    const int64_t inverse, const int64_t sub_m, size_t *size) {
  const std::string api = "[mluOpGetIndiceConvolutionForwardFromTableWorkspaceSize]";
  mluOpStatus_t st = foolProof(api, handle, features_desc, filters_desc, indice_pairs_desc, indice_num,
                               num_act_out, inverse, sub_m, features_out_desc);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  PARAM_CHECK(api, size != nullptr);
  *size = 0;
  if (anyZeroElement(features_desc, indice_pairs_desc, filters_desc, features_out_desc)) return MLUOP_STATUS_SUCCESS;
  const ConvProblem p = makeProblem(handle, features_desc, filters_desc, num_act_out);
  *size = mluop::sparse_conv::planConvWorkspace(p, true).total;
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpIndiceConvolutionForwardFromTable(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc, const void *features,
    const mluOpTensorDescriptor_t filters_desc, const void *filters,
    const mluOpTensorDescriptor_t indice_pairs_desc, const void *table, const size_t table_size,
    const int64_t indice_num[], const int64_t num_act_out, const int64_t inverse, const int64_t sub_m,
    void *workspace, const size_t workspace_size, const mluOpTensorDescriptor_t features_out_desc,
    void *features_out) {
  const std::string api = "[mluOpIndiceConvolutionForwardFromTable]";
  mluOpStatus_t st = foolProof(api, handle, features_desc, filters_desc, indice_pairs_desc, indice_num,
                               num_act_out, inverse, sub_m, features_out_desc);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  if (anyZeroElement(filters_desc, features_desc, indice_pairs_desc, features_out_desc)) {
    VLOG(5) << api << " Skip zero element tensor.";
    return MLUOP_STATUS_SUCCESS;
  }
  PARAM_CHECK(api, features != nullptr);
  PARAM_CHECK(api, filters != nullptr);
  PARAM_CHECK(api, table != nullptr);
  PARAM_CHECK(api, features_out != nullptr);
  PARAM_CHECK(api, workspace != nullptr);
  PARAM_CHECK(api, reinterpret_cast<size_t>(table) % 16 == 0);  // read 16 bytes at a time
  const ConvProblem p = makeProblem(handle, features_desc, filters_desc, num_act_out);
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
      p, plan, features, filters, nullptr, indice_num, workspace, features_out, handle->sm_count, handle->queue,
      const_cast<int32_t *>(static_cast<const int32_t *>(table)), mluop::sparse_conv::kTableConvolveOnly);
  if (err != cudaSuccess) {
    LOG(ERROR) << api << " launch failed: " << cudaGetErrorString(err);
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  return MLUOP_STATUS_SUCCESS;
}

}  // extern "C"
