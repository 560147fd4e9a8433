// mluOpGetIndicePairs / mluOpGetIndicePairsWorkspaceSize: argument checks,
// workspace plan and launch (reference
// kernels/sparse_conv/get_indice_pairs/get_indice_pairs.cpp:78-277 for the
// checks and their order, normal_get_indice_pairs.cpp:193-261 for the
// workspace query, :831-1153 for the computation these kernels replace).
//
// Differences from the reference, all documented for callers:
//   * the cap of 1,000,000 input voxels (get_indice_pairs_structs.h:36) is
//     lifted; the limits are the structural ones (every tensor below 2^31
//     elements, batch*D*H*W + 1 below 2^31 for both spaces);
//   * in submanifold mode num_act_out is set to the number of input voxels
//     (the reference leaves the field untouched);
//   * out_indices rows past the active count are set to -1, as the
//     reference's CPU implementation does;
//   * an input row whose batch index or coordinates lie outside the declared
//     batch / input space produces no pair (the reference reads out of bounds).
#include <cuda_runtime_api.h>

#include <cstdlib>
#include <string>

#include "core/context.h"
#include "core/logging.h"
#include "core/tensor.h"
#include "kernels/sparse_conv/get_indice_pairs_kernels.h"
#include "kernels/sparse_conv/sparse_conv_desc.h"

using mluop::sparse_conv::PairsGeometry;
using mluop::sparse_conv::PairsWorkspacePlan;

namespace {

mluOpStatus_t internalGetIndicePairs(mluOpHandle_t handle, const std::string &api,
                                     mluOpSparseConvolutionDescriptor_t conv_desc,
                                     const mluOpTensorDescriptor_t indices_desc, const void *indices,
                                     void *workspace, size_t workspace_size,
                                     const mluOpTensorDescriptor_t indice_pairs_desc, void *indice_pairs,
                                     const mluOpTensorDescriptor_t out_indices_desc, void *out_indices,
                                     const mluOpTensorDescriptor_t indice_num_desc, void *indice_num,
                                     bool is_get_workspace, size_t *return_ws, bool with_table = false,
                                     void *table = NULL, size_t table_size = 0) {
  PARAM_CHECK(api, handle != NULL);
  PARAM_CHECK(api, conv_desc != NULL);
  PARAM_CHECK(api, indices_desc != NULL);
  PARAM_CHECK(api, indice_pairs_desc != NULL);
  PARAM_CHECK(api, out_indices_desc != NULL);
  PARAM_CHECK(api, indice_num_desc != NULL);

  if (handle->arch < MLUOP_MLU370) {
    LOG(ERROR) << api << " needs a compute-capability 10.x device; this handle's device is not one.";
    return MLUOP_STATUS_ARCH_MISMATCH;
  }
  const int spatial = conv_desc->dimNb - 2;
  PARAM_CHECK(api, conv_desc->dimNb == 5);

  PARAM_CHECK(api, indices_desc->getDim() == 2);
  PARAM_CHECK(api, indice_pairs_desc->getDim() == 3);
  PARAM_CHECK(api, out_indices_desc->getDim() == 2);
  PARAM_CHECK(api, indice_num_desc->getDim() == 1);
  PARAM_CHECK(api, indices_desc->getDimIndex(1) == 4);
  PARAM_CHECK(api, out_indices_desc->getDimIndex(1) == 4);
  PARAM_CHECK(api, indice_pairs_desc->getDimIndex(1) == 2);

  PARAM_CHECK(api, indice_pairs_desc->getDimIndex(2) == indices_desc->getDimIndex(0));
  PARAM_CHECK(api, indice_pairs_desc->getDimIndex(0) == indice_num_desc->getDimIndex(0));
  int64_t kernel_volume = 1, output_spaces = conv_desc->batch, input_spaces = conv_desc->batch;
  for (int i = 0; i < spatial; ++i) {
    kernel_volume *= conv_desc->filter_space[i];
    output_spaces *= conv_desc->output_space[i];
    input_spaces *= conv_desc->input_space[i];
  }
  PARAM_CHECK_LE(api, indices_desc->getDimIndex(0), input_spaces);
  for (int i = 0; i < spatial; ++i) {
    const std::string where = "i: " + std::to_string(i) + ".";
    PARAM_CHECK_V2(api, conv_desc->pad[i] >= 0, << where);
    PARAM_CHECK_V2(api, conv_desc->dilation[i] >= 1, << where);
    PARAM_CHECK_V2(api, conv_desc->stride[i] >= 1, << where);
    if (conv_desc->dilation[i] != 1 && conv_desc->stride[i] != 1) {
      LOG(ERROR) << api << " dilation[" << i << "] and stride[" << i << "] cannot both differ from 1.";
      return MLUOP_STATUS_BAD_PARAM;
    }
  }
  PARAM_CHECK(api, indice_pairs_desc->getDimIndex(0) == kernel_volume);
  PARAM_CHECK_LE(api, kernel_volume, 4096);
  PARAM_CHECK_LE(api, out_indices_desc->getDimIndex(0), output_spaces);

  STRIDE_TENSOR_CHECK(api, indices_desc, "indices_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api, indice_pairs_desc, "indice_pairs_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api, out_indices_desc, "out_indices_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api, indice_num_desc, "indice_num_desc must be contiguous");

  if (mluOpGetTensorElementNum(indices_desc) >= LARGE_TENSOR_NUM ||
      mluOpGetTensorElementNum(out_indices_desc) >= LARGE_TENSOR_NUM ||
      mluOpGetTensorElementNum(indice_pairs_desc) >= LARGE_TENSOR_NUM ||
      mluOpGetTensorElementNum(indice_num_desc) >= LARGE_TENSOR_NUM) {
    LOG(ERROR) << api << " Overflow max tensor num. Tensors must have fewer than 2^31 elements.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }
  // Linear voxel indices are int32 (and one sentinel past the end is used by
  // callers that follow the reference's conventions).
  if ((uint64_t)output_spaces + 1 >= LARGE_TENSOR_NUM || (uint64_t)input_spaces + 1 >= LARGE_TENSOR_NUM) {
    LOG(ERROR) << api << " batch * D * H * W must stay below 2^31 - 1 for the input and the output space.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }

  PARAM_CHECK_EQ(api, indices_desc->getDtype(), MLUOP_DTYPE_INT32);
  PARAM_CHECK_EQ(api, indice_pairs_desc->getDtype(), MLUOP_DTYPE_INT32);
  PARAM_CHECK_EQ(api, out_indices_desc->getDtype(), MLUOP_DTYPE_INT32);
  PARAM_CHECK_EQ(api, indice_num_desc->getDtype(), MLUOP_DTYPE_INT32);

  const int sub_m = conv_desc->sub_m;
  if (sub_m) {
    for (int i = 0; i < spatial; ++i) {
      const std::string where = "i: " + std::to_string(i) + ".";
      PARAM_CHECK_V2(api, conv_desc->input_space[i] == conv_desc->output_space[i], << where);
      PARAM_CHECK_V2(api, conv_desc->stride[i] == 1, << where);
      PARAM_CHECK_V2(api, conv_desc->dilation[i] == 1, << where);
    }
  }

  if (mluOpGetTensorElementNum(indices_desc) == 0 || mluOpGetTensorElementNum(indice_pairs_desc) == 0 ||
      mluOpGetTensorElementNum(out_indices_desc) == 0 || mluOpGetTensorElementNum(indice_num_desc) == 0) {
    conv_desc->num_act_out = 0;
    if (is_get_workspace && return_ws) *return_ws = 0;
    return MLUOP_STATUS_SUCCESS;
  }

  PairsGeometry g{};
  g.L = (int32_t)indices_desc->getDimIndex(0);
  g.K = (int32_t)kernel_volume;
  g.batch = conv_desc->batch;
  g.out_vol = 1;
  for (int i = 0; i < 3; ++i) {
    g.ks[i] = conv_desc->filter_space[i];
    g.pad[i] = conv_desc->pad[i];
    g.stride[i] = conv_desc->stride[i];
    g.stride_shift[i] = -1;
    for (int sh = 0; sh < 31; ++sh)
      if ((1 << sh) == conv_desc->stride[i]) g.stride_shift[i] = sh;
    g.dil[i] = conv_desc->dilation[i];
    g.in_space[i] = conv_desc->input_space[i];
    g.out_space[i] = conv_desc->output_space[i];
    g.out_vol *= conv_desc->output_space[i];
  }
  g.sub_m = sub_m ? 1 : 0;
  const PairsWorkspacePlan plan = mluop::sparse_conv::planPairsWorkspace(g);

  if (is_get_workspace) {
    *return_ws = plan.total;
    return MLUOP_STATUS_SUCCESS;
  }

  PARAM_CHECK(api, indices != NULL);
  PARAM_CHECK(api, indice_pairs != NULL);
  PARAM_CHECK(api, out_indices != NULL);
  PARAM_CHECK(api, indice_num != NULL);
  // The kernels read and write coordinate rows (four int32) as one 16-byte word.
  PARAM_CHECK(api, reinterpret_cast<size_t>(indices) % 16 == 0);
  PARAM_CHECK(api, reinterpret_cast<size_t>(out_indices) % 16 == 0);
  PARAM_CHECK(api, reinterpret_cast<size_t>(indice_pairs) % 4 == 0);
  PARAM_CHECK(api, reinterpret_cast<size_t>(indice_num) % 4 == 0);
  if (workspace_size != 0) {
    PARAM_CHECK(api, workspace != NULL);
  }
  if (workspace_size < plan.total || workspace == NULL) {
    LOG(ERROR) << api << " workspace of " << workspace_size << " bytes is smaller than the "
               << plan.total << " bytes mluOpGetIndicePairsWorkspaceSize reports.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  int32_t *neighbour_table = NULL;
  if (with_table) {
    if (!mluop::sparse_conv::pairsCanEmitTable(g, plan)) {
      LOG(ERROR) << api << " the rulebook kernels emit a neighbour table only for submanifold rulebooks with odd "
                 << "kernel sizes up to volume 32, unit stride and dilation and pad = size / 2; build the table "
                 << "from indice_pairs with mluOpBuildIndiceNeighbourTable instead.";
      return MLUOP_STATUS_NOT_SUPPORTED;
    }
    PARAM_CHECK(api, table != NULL);
    PARAM_CHECK(api, reinterpret_cast<size_t>(table) % 16 == 0);
    const size_t need = (size_t)g.K * (size_t)mluop::sparse_conv::pairsTableStride(g.L) * sizeof(int32_t);
    if (table_size < need) {
      LOG(ERROR) << api << " table of " << table_size << " bytes is smaller than the " << need
                 << " bytes mluOpGetIndiceNeighbourTableSize reports.";
      return MLUOP_STATUS_BAD_PARAM;
    }
    neighbour_table = static_cast<int32_t *>(table);
  }
  if (handle->host_only) {
    LOG(ERROR) << api << " this handle was created without a CUDA device; nothing can be launched.";
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  if (mluop::takeStickyDeviceError(handle, std::string(api).c_str())) return MLUOP_STATUS_EXECUTION_FAILED;

  cudaStream_t stream = handle->queue;
  int32_t *status_host = handle->host_words;
  cudaError_t err = mluop::sparse_conv::launchGetIndicePairs(
      g, plan, static_cast<const int32_t *>(indices), workspace, static_cast<int32_t *>(indice_pairs),
      static_cast<int32_t *>(out_indices), out_indices_desc->getDimIndex(0),
      static_cast<int32_t *>(indice_num), status_host, neighbour_table, stream);
  if (err != cudaSuccess) {
    LOG(ERROR) << api << " launch failed: " << cudaGetErrorString(err);
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  if (sub_m && !mluop::checkStatusRequested()) {
    // No host read is needed: the active outputs are the inputs.  (With
    // MLUOP_B200_CHECK_STATUS=1 the call waits and reports device error bits.)
    conv_desc->num_act_out = g.L;
    return MLUOP_STATUS_SUCCESS;
  }
  // The caller sizes features_out by the number of active outputs, so this
  // one value has to reach the host before the call returns.
  err = cudaStreamSynchronize(stream);
  if (err != cudaSuccess) {
    LOG(ERROR) << api << " execution failed: " << cudaGetErrorString(err);
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  // this call reports its own error bits below; they need not be reported a second time
  static_assert(mluOpContext::kStickyWord == 2, "publishStatusKernel ORs the error bits into word 2");
  status_host[mluOpContext::kStickyWord] = 0;
  if (status_host[0] & mluop::sparse_conv::kPairsErrOutIndicesSmall) {
    LOG(ERROR) << api << " out_indices has " << out_indices_desc->getDimIndex(0) << " rows but "
               << status_host[1] << " output voxels are active.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (status_host[0] != 0) {
    LOG(ERROR) << api << " device reported error bits " << status_host[0] << ".";
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  conv_desc->num_act_out = sub_m ? g.L : status_host[1];
  return MLUOP_STATUS_SUCCESS;
}

}  // namespace

extern "C" {

mluOpStatus_t MLUOP_WIN_API mluOpGetIndicePairs(
    mluOpHandle_t handle, mluOpSparseConvolutionDescriptor_t sparse_conv_desc,
    const mluOpTensorDescriptor_t indices_desc, const void *indices, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t indice_pairs_desc, void *indice_pairs,
    const mluOpTensorDescriptor_t out_indices_desc, void *out_indices,
    const mluOpTensorDescriptor_t indice_num_desc, void *indice_num) {
  return internalGetIndicePairs(handle, "[mluOpGetIndicesPairs]", sparse_conv_desc, indices_desc, indices,
                                workspace, workspace_size, indice_pairs_desc, indice_pairs,
                                out_indices_desc, out_indices, indice_num_desc, indice_num, false, NULL);
}

// No counterpart in the reference: mluOpGetIndicePairs that also leaves the
// neighbour table of the rulebook in `table` (see the neighbour-table entry
// points next to mluOpIndiceConvolutionForward).  The probe kernel has every
// match in hand, so the table costs one more coalesced store per slot and the
// separate build (a memset and a scatter over all pairs) disappears.
mluOpStatus_t MLUOP_WIN_API mluOpGetIndicePairsWithNeighbourTable(
    mluOpHandle_t handle, mluOpSparseConvolutionDescriptor_t sparse_conv_desc,
    const mluOpTensorDescriptor_t indices_desc, const void *indices, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t indice_pairs_desc, void *indice_pairs,
    const mluOpTensorDescriptor_t out_indices_desc, void *out_indices,
    const mluOpTensorDescriptor_t indice_num_desc, void *indice_num, void *table, const size_t table_size) {
  return internalGetIndicePairs(handle, "[mluOpGetIndicePairsWithNeighbourTable]", sparse_conv_desc, indices_desc,
                                indices, workspace, workspace_size, indice_pairs_desc, indice_pairs,
                                out_indices_desc, out_indices, indice_num_desc, indice_num, false, NULL, true, table,
                                table_size);
}

mluOpStatus_t MLUOP_WIN_API mluOpGetIndicePairsWorkspaceSize(
    mluOpHandle_t handle, mluOpSparseConvolutionDescriptor_t sparse_conv_desc,
    const mluOpTensorDescriptor_t indices_desc, const mluOpTensorDescriptor_t indice_pairs_desc,
    const mluOpTensorDescriptor_t out_indices_desc, const mluOpTensorDescriptor_t indice_num_desc,
    size_t *workspace_size) {
  const std::string api = "[mluOpGetIndicePairsWorkspaceSize]";
  PARAM_CHECK(api, handle != NULL);
  PARAM_CHECK(api, sparse_conv_desc != NULL);
  PARAM_CHECK(api, indices_desc != NULL);
  PARAM_CHECK(api, indice_pairs_desc != NULL);
  PARAM_CHECK(api, out_indices_desc != NULL);
  PARAM_CHECK(api, indice_num_desc != NULL);
  PARAM_CHECK(api, workspace_size != NULL);
  if (mluOpGetTensorElementNum(indices_desc) == 0 || mluOpGetTensorElementNum(indice_pairs_desc) == 0 ||
      mluOpGetTensorElementNum(out_indices_desc) == 0 || mluOpGetTensorElementNum(indice_num_desc) == 0) {
    workspace_size[0] = 0;
    return MLUOP_STATUS_SUCCESS;
  }
  return internalGetIndicePairs(handle, api, sparse_conv_desc, indices_desc, NULL, NULL, 0,
                                indice_pairs_desc, NULL, out_indices_desc, NULL, indice_num_desc, NULL,
                                true, workspace_size);
}

}  // extern "C"
