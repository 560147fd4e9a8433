// A C++ caller of the C ABI, written the way the reference's API tests call it
// (test/mlu_op_gtest/api_gtest/src/gtest/indice_convolution_forward/indice_convolution_forward.cpp:
// create a handle, descriptors, then expect MLUOP_STATUS_BAD_PARAM for every
// missing argument).  Built and run by tests/test_symbols.py against
// libmluops_b200.so with a host-only handle, so it needs no GPU.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "mlu_op.h"

#define EXPECT(cond)                                                        \
  do {                                                                      \
    if (!(cond)) {                                                          \
      std::fprintf(stderr, "%s:%d: check failed: %s\n", __FILE__, __LINE__, #cond); \
      return 1;                                                             \
    }                                                                       \
  } while (0)

int main() {
  mluOpHandle_t handle = nullptr;
  EXPECT(mluOpCreate(&handle) == MLUOP_STATUS_SUCCESS);
  int major = 0, minor = 0, patch = 0;
  mluOpGetLibVersion(&major, &minor, &patch);
  EXPECT(major == 1);

  mluOpTensorDescriptor_t features, filters, pairs, out;
  EXPECT(mluOpCreateTensorDescriptor(&features) == MLUOP_STATUS_SUCCESS);
  EXPECT(mluOpCreateTensorDescriptor(&filters) == MLUOP_STATUS_SUCCESS);
  EXPECT(mluOpCreateTensorDescriptor(&pairs) == MLUOP_STATUS_SUCCESS);
  EXPECT(mluOpCreateTensorDescriptor(&out) == MLUOP_STATUS_SUCCESS);
  const int f_dims[2] = {2, 3}, w_dims[5] = {5, 1, 2, 2, 3}, p_dims[3] = {4, 2, 2}, o_dims[2] = {9, 5};
  EXPECT(mluOpSetTensorDescriptor(features, MLUOP_LAYOUT_ARRAY, MLUOP_DTYPE_FLOAT, 2, f_dims) == MLUOP_STATUS_SUCCESS);
  EXPECT(mluOpSetTensorDescriptor(filters, MLUOP_LAYOUT_NDHWC, MLUOP_DTYPE_FLOAT, 5, w_dims) == MLUOP_STATUS_SUCCESS);
  EXPECT(mluOpSetTensorDescriptor(pairs, MLUOP_LAYOUT_ARRAY, MLUOP_DTYPE_INT32, 3, p_dims) == MLUOP_STATUS_SUCCESS);
  EXPECT(mluOpSetTensorDescriptor(out, MLUOP_LAYOUT_ARRAY, MLUOP_DTYPE_FLOAT, 2, o_dims) == MLUOP_STATUS_SUCCESS);
  EXPECT(mluOpGetTensorElementNum(filters) == 60);

  const int64_t indice_num[4] = {1, 1, 1, 1};
  size_t workspace_size = 0;
  EXPECT(mluOpGetIndiceConvolutionForwardWorkspaceSize(handle, features, filters, pairs, out, indice_num, 9, 0, 0,
                                                       &workspace_size) == MLUOP_STATUS_SUCCESS);
  EXPECT(workspace_size > 0);
  std::vector<char> dummy(4096);
  void *p = dummy.data();
  // every missing argument is MLUOP_STATUS_BAD_PARAM, as in the reference's tests
  EXPECT(mluOpIndiceConvolutionForward(nullptr, features, p, filters, p, pairs, p, indice_num, 9, 0, 0, p, 64, out, p) ==
         MLUOP_STATUS_BAD_PARAM);
  EXPECT(mluOpIndiceConvolutionForward(handle, nullptr, p, filters, p, pairs, p, indice_num, 9, 0, 0, p, 64, out, p) ==
         MLUOP_STATUS_BAD_PARAM);
  EXPECT(mluOpIndiceConvolutionForward(handle, features, nullptr, filters, p, pairs, p, indice_num, 9, 0, 0, p, 64, out,
                                       p) == MLUOP_STATUS_BAD_PARAM);
  EXPECT(mluOpIndiceConvolutionForward(handle, features, p, filters, p, pairs, p, nullptr, 9, 0, 0, p, 64, out, p) ==
         MLUOP_STATUS_BAD_PARAM);
  EXPECT(mluOpIndiceConvolutionForward(handle, features, p, filters, p, pairs, p, indice_num, 9, 1, 0, p, 64, out, p) ==
         MLUOP_STATUS_NOT_SUPPORTED);
  // all checks pass: a handle without a device cannot launch
  EXPECT(mluOpIndiceConvolutionForward(handle, features, p, filters, p, pairs, p, indice_num, 9, 0, 0, p, workspace_size,
                                       out, p) == MLUOP_STATUS_EXECUTION_FAILED);

  // sparse convolution descriptor and the rulebook's checks
  mluOpSparseConvolutionDescriptor_t conv = nullptr;
  EXPECT(mluOpCreateSparseConvolutionDescriptor(&conv) == MLUOP_STATUS_SUCCESS);
  const int pad[3] = {1, 1, 1}, stride[3] = {1, 1, 1}, dilation[3] = {1, 1, 1};
  const int in_space[3] = {4, 4, 4}, filter_space[3] = {3, 3, 3}, out_space[3] = {4, 4, 4};
  EXPECT(mluOpSetSparseConvolutionDescriptor(conv, 5, 1, pad, stride, dilation, in_space, filter_space, out_space, 1, 0,
                                             0) == MLUOP_STATUS_SUCCESS);
  EXPECT(mluOpSetSparseConvolutionDescriptor(conv, 4, 1, pad, stride, dilation, in_space, filter_space, out_space, 1, 0,
                                             0) != MLUOP_STATUS_SUCCESS);
  EXPECT(mluOpGetIndicePairs(handle, conv, nullptr, p, p, 64, pairs, p, out, p, features, p) == MLUOP_STATUS_BAD_PARAM);

  // the neighbour-table extensions: declared for C callers too, same conventions
  size_t table_size = 0;
  EXPECT(mluOpGetIndiceNeighbourTableSize(handle, pairs, 9, &table_size) == MLUOP_STATUS_SUCCESS && table_size > 0);
  EXPECT(mluOpGetIndiceInputNeighbourTableSize(handle, pairs, &table_size) == MLUOP_STATUS_SUCCESS && table_size > 0);
  EXPECT(mluOpBuildIndiceNeighbourTable(nullptr, pairs, p, indice_num, 9, p, table_size) == MLUOP_STATUS_BAD_PARAM);
  EXPECT(mluOpBuildIndiceInputNeighbourTable(nullptr, pairs, p, indice_num, 9, p, table_size) == MLUOP_STATUS_BAD_PARAM);
  EXPECT(mluOpIndiceConvolutionForwardFromTable(nullptr, features, p, filters, p, pairs, p, table_size, indice_num, 9, 0,
                                                0, p, 64, out, p) == MLUOP_STATUS_BAD_PARAM);
  EXPECT(mluOpIndiceConvolutionBackwardDataFromTable(nullptr, out, p, filters, p, pairs, p, table_size, indice_num, 0, 0,
                                                     p, 64, features, p) == MLUOP_STATUS_BAD_PARAM);
  EXPECT(mluOpIndiceConvolutionBackwardDataFromForwardTable(nullptr, out, p, filters, p, pairs, p, table_size,
                                                            indice_num, 0, 1, p, 64, features, p) ==
         MLUOP_STATUS_BAD_PARAM);
  EXPECT(mluOpIndiceConvolutionBackwardFilterFromTable(nullptr, features, p, out, p, pairs, p, table_size, indice_num,
                                                       0, 0, p, 64, filters, p) == MLUOP_STATUS_BAD_PARAM);
  EXPECT(mluOpGetIndicePairsWithNeighbourTable(handle, conv, nullptr, p, p, 64, pairs, p, out, p, features, p, p,
                                               table_size) == MLUOP_STATUS_BAD_PARAM);

  EXPECT(mluOpDestroySparseConvolutionDescriptor(conv) == MLUOP_STATUS_SUCCESS);
  EXPECT(mluOpDestroyTensorDescriptor(features) == MLUOP_STATUS_SUCCESS);
  EXPECT(mluOpDestroyTensorDescriptor(filters) == MLUOP_STATUS_SUCCESS);
  EXPECT(mluOpDestroyTensorDescriptor(pairs) == MLUOP_STATUS_SUCCESS);
  EXPECT(mluOpDestroyTensorDescriptor(out) == MLUOP_STATUS_SUCCESS);
  EXPECT(mluOpDestroy(handle) == MLUOP_STATUS_SUCCESS);
  std::puts("abi_check: ok");
  return 0;
}
