// mluOpDynamicPointToVoxelBackward / mluOpGetDynamicPointToVoxelBackwardWorkspaceSize
// (reference kernels/dynamic_point_to_voxel/dynamic_point_to_voxel_backward/
// dynamic_point_to_voxel_backward.cpp: parameter check :34-186, compute entry
// :232-340, workspace query :342-387; device code
// dynamic_point_to_voxel_backward_union1.mlu).
//
// Gradient of the maximum reduction: of the points of a voxel, the one with the
// smallest index whose feature equals the voxel's maximum receives the voxel's
// gradient, per channel; every other entry of grad_feats is zero.
//   fillKernel         voxel_from[v][c] = N ("none")
//   findSourceKernel   one thread per (point, channel): atomicMin of the point
//                      index where the feature equals the voxel's maximum
//   scatterKernel      one thread per (voxel, channel): grad_feats[voxel_from][c]
// The order of the checks and their status codes follow the reference; its limit
// on N and C (the working set had to fit one core's scratch memory) does not
// apply here.  The workspace is int32[M][C] (the reference's is the same array).
#include <cuda_runtime.h>

#include <string>

#include "core/context.h"
#include "core/logging.h"
#include "core/tensor.h"
#include "core/trace.h"
#include "mlu_op.h"

namespace {

__global__ void __launch_bounds__(256) fillKernel(int32_t *__restrict__ dst, int64_t count, int32_t value) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = value;
}

__global__ void __launch_bounds__(256)
findSourceKernel(const float *__restrict__ feats, const float *__restrict__ voxel_feats,
                 const int32_t *__restrict__ point2voxel_map, const int32_t *__restrict__ voxel_num, int64_t n,
                 int c_num, int64_t voxel_rows, int32_t *__restrict__ voxel_from) {
  const int64_t voxels = *voxel_num < voxel_rows ? *voxel_num : voxel_rows;
  const int64_t total = n * c_num;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t x = e / c_num;
    const int c = (int)(e % c_num);
    const int32_t v = point2voxel_map[x];
    if (v < 0 || v >= voxels) continue;
    if (feats[e] == voxel_feats[(int64_t)v * c_num + c]) atomicMin(&voxel_from[(int64_t)v * c_num + c], (int32_t)x);
  }
}

__global__ void __launch_bounds__(256)
scatterKernel(const float *__restrict__ grad_voxel_feats, const int32_t *__restrict__ voxel_from,
              const int32_t *__restrict__ voxel_num, int64_t n, int c_num, int64_t voxel_rows,
              float *__restrict__ grad_feats) {
  const int64_t voxels = *voxel_num < voxel_rows ? *voxel_num : voxel_rows;
  const int64_t total = voxels * c_num;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (int64_t)gridDim.x * blockDim.x) {
    const int32_t x = voxel_from[e];
    if (x < n) grad_feats[(int64_t)x * c_num + (e % c_num)] = grad_voxel_feats[e];
  }
}

unsigned gridFor(int64_t work) {
  int64_t b = (work + 255) / 256;
  if (b < 1) b = 1;
  if (b > 148 * 32) b = 148 * 32;
  return (unsigned)b;
}

mluOpStatus_t paramCheck(const std::string &api, const mluOpHandle_t handle, const mluOpReduceMode_t reduce_type,
                         const mluOpTensorDescriptor_t grad_voxel_feats_desc, const void *grad_voxel_feats,
                         const mluOpTensorDescriptor_t feats_desc, const void *feats,
                         const mluOpTensorDescriptor_t voxel_feats_desc, const void *voxel_feats,
                         const mluOpTensorDescriptor_t point2voxel_map_desc, const void *point2voxel_map,
                         const mluOpTensorDescriptor_t voxel_points_count_desc, const void *voxel_points_count,
                         const mluOpTensorDescriptor_t voxel_num_desc, const void *voxel_num, void *workspace,
                         const size_t workspace_size, const mluOpTensorDescriptor_t grad_feats_desc,
                         void *grad_feats, bool check_pointers, bool *zero_element) {
  PARAM_CHECK(api, handle != nullptr);
  if (handle->arch < MLUOP_MLU370) {
    LOG(ERROR) << api << " needs a compute-capability 10.x device; this handle's device is not one.";
    return MLUOP_STATUS_ARCH_MISMATCH;
  }
  PARAM_CHECK(api, grad_voxel_feats_desc != nullptr);
  PARAM_CHECK(api, feats_desc != nullptr);
  PARAM_CHECK(api, voxel_feats_desc != nullptr);
  PARAM_CHECK(api, point2voxel_map_desc != nullptr);
  PARAM_CHECK(api, voxel_points_count_desc != nullptr);
  PARAM_CHECK(api, voxel_num_desc != nullptr);
  if (check_pointers) {
    PARAM_CHECK(api, grad_feats_desc != nullptr);
  }
  STRIDE_TENSOR_CHECK(api + ":", grad_voxel_feats_desc, "grad_voxel_feats_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", feats_desc, "feats_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", voxel_feats_desc, "voxel_feats_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", point2voxel_map_desc, "point2voxel_map_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", voxel_points_count_desc, "voxel_points_count_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", voxel_num_desc, "voxel_num_desc must be contiguous");
  PARAM_CHECK(api, grad_voxel_feats_desc->getDtype() == MLUOP_DTYPE_FLOAT);
  PARAM_CHECK(api, feats_desc->getDtype() == MLUOP_DTYPE_FLOAT);
  PARAM_CHECK(api, voxel_feats_desc->getDtype() == MLUOP_DTYPE_FLOAT);
  PARAM_CHECK(api, point2voxel_map_desc->getDtype() == MLUOP_DTYPE_INT32);
  PARAM_CHECK(api, voxel_points_count_desc->getDtype() == MLUOP_DTYPE_INT32);
  PARAM_CHECK(api, voxel_num_desc->getDtype() == MLUOP_DTYPE_INT32);
  PARAM_CHECK(api, grad_voxel_feats_desc->getDim() == 2);
  PARAM_CHECK(api, feats_desc->getDim() == 2);
  PARAM_CHECK(api, voxel_feats_desc->getDim() == 2);
  PARAM_CHECK(api, point2voxel_map_desc->getDim() == 1);
  PARAM_CHECK(api, voxel_points_count_desc->getDim() == 1);
  PARAM_CHECK(api, voxel_num_desc->getDim() == 1);
  PARAM_CHECK(api, feats_desc->getDimIndex(1) == grad_voxel_feats_desc->getDimIndex(1));
  PARAM_CHECK(api, voxel_feats_desc->getDimIndex(0) == grad_voxel_feats_desc->getDimIndex(0));
  PARAM_CHECK(api, voxel_feats_desc->getDimIndex(1) == grad_voxel_feats_desc->getDimIndex(1));
  PARAM_CHECK(api, point2voxel_map_desc->getDimIndex(0) == feats_desc->getDimIndex(0));
  PARAM_CHECK(api, voxel_points_count_desc->getDimIndex(0) == grad_voxel_feats_desc->getDimIndex(0));
  PARAM_CHECK(api, voxel_num_desc->getDimIndex(0) == 1);
  PARAM_CHECK(api, feats_desc->getDimIndex(0) >= grad_voxel_feats_desc->getDimIndex(0));
  if (check_pointers) {
    STRIDE_TENSOR_CHECK(api + ":", grad_feats_desc, "grad_feats_desc must be contiguous");
    PARAM_CHECK(api, grad_feats_desc->getDtype() == MLUOP_DTYPE_FLOAT);
    PARAM_CHECK(api, grad_feats_desc->getDim() == 2);
    PARAM_CHECK(api, grad_feats_desc->getDimIndex(0) == feats_desc->getDimIndex(0));
    PARAM_CHECK(api, grad_feats_desc->getDimIndex(1) == grad_voxel_feats_desc->getDimIndex(1));
  }
  if (reduce_type != MLUOP_REDUCE_DMAX) {
    LOG(ERROR) << api << " only supports max reduce in current version. ";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (mluOpGetTensorElementNum(grad_voxel_feats_desc) >= LARGE_TENSOR_NUM ||
      mluOpGetTensorElementNum(feats_desc) >= LARGE_TENSOR_NUM) {
    LOG(ERROR) << api << " Overflow max tensor num. Tensors must have fewer than 2^31 elements.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }
  if (!check_pointers) return MLUOP_STATUS_SUCCESS;
  if (mluOpGetTensorElementNum(grad_feats_desc) == 0) {
    *zero_element = true;
    return MLUOP_STATUS_SUCCESS;
  }
  if (mluOpGetTensorElementNum(grad_voxel_feats_desc) != 0) {
    PARAM_CHECK(api, grad_voxel_feats != nullptr);
  }
  PARAM_CHECK(api, feats != nullptr);
  if (mluOpGetTensorElementNum(voxel_feats_desc) != 0) {
    PARAM_CHECK(api, voxel_feats != nullptr);
  }
  PARAM_CHECK(api, point2voxel_map != nullptr);
  if (mluOpGetTensorElementNum(voxel_points_count_desc) != 0) {
    PARAM_CHECK(api, voxel_points_count != nullptr);
  }
  PARAM_CHECK(api, voxel_num != nullptr);
  PARAM_CHECK(api, grad_feats != nullptr);
  if (workspace_size != 0) {
    PARAM_CHECK(api, workspace != nullptr);
  }
  return MLUOP_STATUS_SUCCESS;
}

size_t workspaceBytes(const mluOpTensorDescriptor_t grad_voxel_feats_desc) {
  return (size_t)mluOpGetTensorElementNum(grad_voxel_feats_desc) * sizeof(int32_t);
}

}  // namespace

extern "C" {

mluOpStatus_t MLUOP_WIN_API mluOpGetDynamicPointToVoxelBackwardWorkspaceSize(
    const mluOpHandle_t handle, const mluOpReduceMode_t reduce_type,
    const mluOpTensorDescriptor_t grad_voxel_feats_desc, const mluOpTensorDescriptor_t feats_desc,
    const mluOpTensorDescriptor_t voxel_feats_desc, const mluOpTensorDescriptor_t point2voxel_map_desc,
    const mluOpTensorDescriptor_t voxel_points_count_desc, const mluOpTensorDescriptor_t voxel_num_desc,
    size_t *workspace_size) {
  const std::string api = "[mluOpGetDynamicPointToVoxelBackwardWorkspaceSize]";
  bool zero = false;
  mluOpStatus_t st = paramCheck(api, handle, reduce_type, grad_voxel_feats_desc, nullptr, feats_desc, nullptr,
                                voxel_feats_desc, nullptr, point2voxel_map_desc, nullptr, voxel_points_count_desc,
                                nullptr, voxel_num_desc, nullptr, nullptr, 0, nullptr, nullptr, false, &zero);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  PARAM_CHECK(api, workspace_size != nullptr);
  *workspace_size = workspaceBytes(grad_voxel_feats_desc);
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpDynamicPointToVoxelBackward(
    const mluOpHandle_t handle, const mluOpReduceMode_t reduce_type,
    const mluOpTensorDescriptor_t grad_voxel_feats_desc, const void *grad_voxel_feats,
    const mluOpTensorDescriptor_t feats_desc, const void *feats, const mluOpTensorDescriptor_t voxel_feats_desc,
    const void *voxel_feats, const mluOpTensorDescriptor_t point2voxel_map_desc, const void *point2voxel_map,
    const mluOpTensorDescriptor_t voxel_points_count_desc, const void *voxel_points_count,
    const mluOpTensorDescriptor_t voxel_num_desc, const void *voxel_num, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t grad_feats_desc, void *grad_feats) {
  const std::string api = "[mluOpDynamicPointToVoxelBackward]";
  bool zero = false;
  mluOpStatus_t st = paramCheck(api, handle, reduce_type, grad_voxel_feats_desc, grad_voxel_feats, feats_desc, feats,
                                voxel_feats_desc, voxel_feats, point2voxel_map_desc, point2voxel_map,
                                voxel_points_count_desc, voxel_points_count, voxel_num_desc, voxel_num, workspace,
                                workspace_size, grad_feats_desc, grad_feats, true, &zero);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  if (zero) {
    VLOG(5) << api << " Skip zero element tensor.";
    return MLUOP_STATUS_SUCCESS;
  }
  const int64_t n = feats_desc->getDimIndex(0);
  const int c_num = (int)feats_desc->getDimIndex(1);
  const int64_t voxel_rows = grad_voxel_feats_desc->getDimIndex(0);
  const size_t need = workspaceBytes(grad_voxel_feats_desc);
  if (need > 0 && (workspace == nullptr || workspace_size < need)) {
    LOG(ERROR) << api << " workspace of " << workspace_size << " bytes is smaller than the " << need
               << " bytes mluOpGetDynamicPointToVoxelBackwardWorkspaceSize reports.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (handle->host_only) {
    LOG(ERROR) << api << " this handle was created without a CUDA device; nothing can be launched.";
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  cudaStream_t stream = handle->queue;
  cudaError_t err = cudaMemsetAsync(grad_feats, 0, (size_t)n * c_num * sizeof(float), stream);
  if (err == cudaSuccess && voxel_rows > 0) {
    int32_t *voxel_from = static_cast<int32_t *>(workspace);
    mluop::trace::Scope t("dynamicPointToVoxelBackwardKernels", stream,
                          8.0 * n * c_num + 16.0 * voxel_rows * c_num);
    fillKernel<<<gridFor(voxel_rows * c_num), 256, 0, stream>>>(voxel_from, voxel_rows * c_num, (int32_t)n);
    findSourceKernel<<<gridFor(n * c_num), 256, 0, stream>>>(
        static_cast<const float *>(feats), static_cast<const float *>(voxel_feats),
        static_cast<const int32_t *>(point2voxel_map), static_cast<const int32_t *>(voxel_num), n, c_num,
        voxel_rows, voxel_from);
    scatterKernel<<<gridFor(voxel_rows * c_num), 256, 0, stream>>>(
        static_cast<const float *>(grad_voxel_feats), voxel_from, static_cast<const int32_t *>(voxel_num), n, c_num,
        voxel_rows, static_cast<float *>(grad_feats));
    err = cudaGetLastError();
  }
  if (err != cudaSuccess) {
    LOG(ERROR) << api << " launch failed: " << cudaGetErrorString(err);
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  return MLUOP_STATUS_SUCCESS;
}

}  // extern "C"
