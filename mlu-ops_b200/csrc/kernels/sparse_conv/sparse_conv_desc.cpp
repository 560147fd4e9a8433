// Sparse-convolution descriptor API (reference
// kernels/sparse_conv/get_indice_pairs/get_indice_pairs_structs.cpp:31-134).
// Status codes per entry point are the reference's: Create(NULL) ->
// NOT_INITIALIZED, Destroy(NULL) -> EXECUTION_FAILED, GetNumActOut(NULL) ->
// NOT_INITIALIZED, every rejected Set argument -> BAD_PARAM.
#include "kernels/sparse_conv/sparse_conv_desc.h"

#include <new>
#include <string>

#include "core/logging.h"

extern "C" {

mluOpStatus_t MLUOP_WIN_API
mluOpCreateSparseConvolutionDescriptor(mluOpSparseConvolutionDescriptor_t *desc) {
  if (desc == NULL) {
    LOG(ERROR) << "mluOpCreateSparseConvolutionDescriptor failed, can't create desc when desc == NULL.";
    return MLUOP_STATUS_NOT_INITIALIZED;
  }
  *desc = new (std::nothrow) mluOpSparseConvolutionStruct();
  return *desc ? MLUOP_STATUS_SUCCESS : MLUOP_STATUS_ALLOC_FAILED;
}

mluOpStatus_t MLUOP_WIN_API mluOpSetSparseConvolutionDescriptor(
    mluOpSparseConvolutionDescriptor_t desc, int dimNb, int batch, const int pad[], const int stride[],
    const int dilation[], const int input_space[], const int filter_space[], const int output_space[],
    const int sub_m, const int transpose, const int inverse) {
  const std::string api = "[mluOpSetSparseConvolutionDescriptor]";
  PARAM_CHECK(api, desc != NULL);
  PARAM_CHECK(api, pad != NULL);
  PARAM_CHECK(api, stride != NULL);
  PARAM_CHECK(api, dilation != NULL);
  PARAM_CHECK(api, input_space != NULL);
  PARAM_CHECK(api, filter_space != NULL);
  PARAM_CHECK(api, output_space != NULL);
  if (dimNb != 5) {
    LOG(ERROR) << api << " only 3-D convolution is supported: dimNb must be 5, got " << dimNb << ".";
    return MLUOP_STATUS_BAD_PARAM;
  }
  desc->dimNb = dimNb;
  if (batch <= 0) {
    LOG(ERROR) << api << " batch must be positive, got " << batch << ".";
    return MLUOP_STATUS_BAD_PARAM;
  }
  desc->batch = batch;
  desc->sub_m = sub_m;
  if (transpose != 0) {
    LOG(ERROR) << api << " transpose is not supported, got " << transpose << ".";
    return MLUOP_STATUS_BAD_PARAM;
  }
  desc->transpose = transpose;
  if (inverse != 0) {
    LOG(ERROR) << api << " inverse is not supported, got " << inverse << ".";
    return MLUOP_STATUS_BAD_PARAM;
  }
  desc->inverse = inverse;
  for (int i = 0; i < dimNb - 2; ++i) {
    const std::string where = "idx: " + std::to_string(i) + ".";
    PARAM_CHECK_V2(api, pad[i] >= 0, << where);
    desc->pad[i] = pad[i];
    PARAM_CHECK_V2(api, stride[i] >= 1, << where);
    desc->stride[i] = stride[i];
    PARAM_CHECK_V2(api, dilation[i] >= 1, << where);
    desc->dilation[i] = dilation[i];
    PARAM_CHECK_V2(api, input_space[i] >= 1, << where);
    desc->input_space[i] = input_space[i];
    PARAM_CHECK_V2(api, filter_space[i] >= 1, << where);
    desc->filter_space[i] = filter_space[i];
    PARAM_CHECK_V2(api, output_space[i] >= 1, << where);
    desc->output_space[i] = output_space[i];
  }
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API
mluOpGetSparseConvolutionNumActOut(mluOpSparseConvolutionDescriptor_t desc, int *num_act_out) {
  if (desc == NULL || num_act_out == NULL) {
    LOG(ERROR) << "mluOpGetSparseConvolutionNumActOut failed: NULL pointer passed to this API.";
    return MLUOP_STATUS_NOT_INITIALIZED;
  }
  *num_act_out = desc->num_act_out;
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API
mluOpDestroySparseConvolutionDescriptor(mluOpSparseConvolutionDescriptor_t desc) {
  if (desc == NULL) {
    LOG(ERROR) << "mluOpDestroySparseConvolutionDescriptor failed: NULL pointer passed to this API.";
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  delete desc;
  return MLUOP_STATUS_SUCCESS;
}

}  // extern "C"
