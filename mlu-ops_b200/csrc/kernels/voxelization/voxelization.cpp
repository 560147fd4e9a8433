// mluOpVoxelization / mluOpGetVoxelizationWorkspaceSize: argument checks and
// dispatch (reference kernels/voxelization/voxelization.cpp: voxelizationParamCheck
// :56-176, workspace query :178-224, compute entry :226-366).
//
// The order of the checks, and the status each returns, follows the reference.
// Differences: the data pointers are checked (the reference checks only the
// workspace pointer), and a workspace smaller than the query result is rejected
// with MLUOP_STATUS_BAD_PARAM.  The size the query returns is this
// implementation's own (hash table and per-voxel lists instead of the reference's
// 6 * num_points words).
#include <cuda_runtime_api.h>

#include <cstdlib>
#include <string>

#include "core/context.h"
#include "core/logging.h"
#include "core/tensor.h"
#include "kernels/voxelization/voxelization_kernels.h"

using mluop::voxelization::VoxelProblem;
using mluop::voxelization::VoxelWorkspacePlan;

namespace {

mluOpStatus_t paramCheck(const std::string &api, const mluOpHandle_t handle,
                         const mluOpTensorDescriptor_t points_desc, const mluOpTensorDescriptor_t voxel_size_desc,
                         const mluOpTensorDescriptor_t coors_range_desc, const int32_t max_points,
                         const int32_t max_voxels, const int32_t NDim, const bool deterministic,
                         const mluOpTensorDescriptor_t voxels_desc, const mluOpTensorDescriptor_t coors_desc,
                         const mluOpTensorDescriptor_t num_points_per_voxel_desc,
                         const mluOpTensorDescriptor_t voxel_num_desc, bool *is_zero_element) {
  if (handle->arch < MLUOP_MLU370) {
    LOG(ERROR) << api << " needs a compute-capability 10.x device; this handle's device is not one.";
    return MLUOP_STATUS_ARCH_MISMATCH;
  }
  if (!deterministic) {
    LOG(ERROR) << api << " Currently, Non-deterministic mode not supported.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  PARAM_CHECK_EQ(api, points_desc->getDim(), 2);
  PARAM_CHECK_EQ(api, voxel_size_desc->getDim(), 1);
  PARAM_CHECK_EQ(api, voxel_size_desc->getDimIndex(0), 3);
  PARAM_CHECK_EQ(api, coors_range_desc->getDim(), 1);
  PARAM_CHECK_EQ(api, coors_range_desc->getDimIndex(0), 6);
  PARAM_CHECK_EQ(api, voxels_desc->getDim(), 3);
  PARAM_CHECK_EQ(api, voxels_desc->getDimIndex(0), max_voxels);
  PARAM_CHECK_EQ(api, voxels_desc->getDimIndex(1), max_points);
  PARAM_CHECK_EQ(api, voxels_desc->getDimIndex(2), points_desc->getDimIndex(1));
  PARAM_CHECK_EQ(api, coors_desc->getDim(), 2);
  PARAM_CHECK_EQ(api, coors_desc->getDimIndex(0), max_voxels);
  PARAM_CHECK_EQ(api, coors_desc->getDimIndex(1), 3);
  PARAM_CHECK_EQ(api, num_points_per_voxel_desc->getDim(), 1);
  PARAM_CHECK_EQ(api, num_points_per_voxel_desc->getDimIndex(0), max_voxels);
  PARAM_CHECK_EQ(api, voxel_num_desc->getDim(), 1);
  PARAM_CHECK_EQ(api, voxel_num_desc->getDimIndex(0), 1);
  PARAM_CHECK_EQ(api, NDim, 3);

  STRIDE_TENSOR_CHECK(api + ":", points_desc, "points_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", voxel_size_desc, "voxel_size_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", coors_range_desc, "coors_range_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", voxels_desc, "voxels_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", coors_desc, "coors_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", num_points_per_voxel_desc, "num_points_per_voxel_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", voxel_num_desc, "voxel_num_desc must be contiguous");

  PARAM_CHECK(api, points_desc->getDtype() == MLUOP_DTYPE_FLOAT);
  PARAM_CHECK(api, voxel_size_desc->getDtype() == MLUOP_DTYPE_FLOAT);
  PARAM_CHECK(api, coors_range_desc->getDtype() == MLUOP_DTYPE_FLOAT);
  PARAM_CHECK(api, voxels_desc->getDtype() == MLUOP_DTYPE_FLOAT);
  PARAM_CHECK(api, coors_desc->getDtype() == MLUOP_DTYPE_INT32);
  PARAM_CHECK(api, num_points_per_voxel_desc->getDtype() == MLUOP_DTYPE_INT32);
  PARAM_CHECK(api, voxel_num_desc->getDtype() == MLUOP_DTYPE_INT32);

  const uint64_t points_n = mluOpGetTensorElementNum(points_desc);
  if (points_n >= LARGE_TENSOR_NUM || mluOpGetTensorElementNum(voxels_desc) >= LARGE_TENSOR_NUM ||
      mluOpGetTensorElementNum(coors_desc) >= LARGE_TENSOR_NUM ||
      mluOpGetTensorElementNum(num_points_per_voxel_desc) >= LARGE_TENSOR_NUM) {
    LOG(ERROR) << api << " Overflow max tensor num. Tensors must have fewer than 2^31 elements.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }
  *is_zero_element = false;
  if (points_n == 0) {
    LOG(ERROR) << api << " Check failed: Input zero element tensor.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (max_points == 0 || max_voxels == 0) {
    *is_zero_element = true;
    return MLUOP_STATUS_SUCCESS;
  }
  // a point needs x, y and z (the reference reads them unchecked)
  PARAM_CHECK(api, points_desc->getDimIndex(1) >= 3);
  return MLUOP_STATUS_SUCCESS;
}

VoxelProblem makeProblem(const mluOpTensorDescriptor_t points_desc, int32_t max_points, int32_t max_voxels) {
  VoxelProblem p{};
  p.num_points = points_desc->getDimIndex(0);
  p.num_features = (int32_t)points_desc->getDimIndex(1);
  p.max_points = max_points;
  p.max_voxels = max_voxels;
  return p;
}

}  // namespace

extern "C" {

mluOpStatus_t MLUOP_WIN_API mluOpGetVoxelizationWorkspaceSize(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t points_desc,
    const mluOpTensorDescriptor_t voxel_size_desc, const mluOpTensorDescriptor_t coors_range_desc,
    const int32_t max_points, const int32_t max_voxels, const int32_t NDim, const bool deterministic,
    const mluOpTensorDescriptor_t voxels_desc, const mluOpTensorDescriptor_t coors_desc,
    const mluOpTensorDescriptor_t num_points_per_voxel_desc, const mluOpTensorDescriptor_t voxel_num_desc,
    size_t *size) {
  const std::string api = "[mluOpGetVoxelizationWorkspaceSize]";
  PARAM_CHECK(api, handle != nullptr);
  PARAM_CHECK(api, points_desc != nullptr);
  PARAM_CHECK(api, voxel_size_desc != nullptr);
  PARAM_CHECK(api, coors_range_desc != nullptr);
  PARAM_CHECK(api, voxels_desc != nullptr);
  PARAM_CHECK(api, coors_desc != nullptr);
  PARAM_CHECK(api, num_points_per_voxel_desc != nullptr);
  PARAM_CHECK(api, voxel_num_desc != nullptr);
  PARAM_CHECK(api, size != nullptr);
  bool is_zero = false;
  mluOpStatus_t st = paramCheck(api, handle, points_desc, voxel_size_desc, coors_range_desc, max_points, max_voxels,
                                NDim, deterministic, voxels_desc, coors_desc, num_points_per_voxel_desc,
                                voxel_num_desc, &is_zero);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  if (is_zero) {
    VLOG(5) << api << " Skip output zero element tensor.";
    return MLUOP_STATUS_SUCCESS;
  }
  *size = mluop::voxelization::planVoxelWorkspace(makeProblem(points_desc, max_points, max_voxels)).total;
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpVoxelization(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t points_desc, const void *points,
    const mluOpTensorDescriptor_t voxel_size_desc, const void *voxel_size,
    const mluOpTensorDescriptor_t coors_range_desc, const void *coors_range, const int32_t max_points,
    const int32_t max_voxels, const int32_t NDim, const bool deterministic, void *workspace,
    size_t workspace_size, const mluOpTensorDescriptor_t voxels_desc, void *voxels,
    const mluOpTensorDescriptor_t coors_desc, void *coors,
    const mluOpTensorDescriptor_t num_points_per_voxel_desc, void *num_points_per_voxel,
    const mluOpTensorDescriptor_t voxel_num_desc, void *voxel_num) {
  const std::string api = "[mluOpVoxelization]";
  PARAM_CHECK(api, handle != nullptr);
  PARAM_CHECK(api, points_desc != nullptr);
  PARAM_CHECK(api, voxel_size_desc != nullptr);
  PARAM_CHECK(api, coors_range_desc != nullptr);
  PARAM_CHECK(api, voxels_desc != nullptr);
  PARAM_CHECK(api, coors_desc != nullptr);
  PARAM_CHECK(api, num_points_per_voxel_desc != nullptr);
  PARAM_CHECK(api, voxel_num_desc != nullptr);
  bool is_zero = false;
  mluOpStatus_t st = paramCheck(api, handle, points_desc, voxel_size_desc, coors_range_desc, max_points, max_voxels,
                                NDim, deterministic, voxels_desc, coors_desc, num_points_per_voxel_desc,
                                voxel_num_desc, &is_zero);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  if (workspace_size > 0) {
    PARAM_CHECK(api, workspace != nullptr);
  }
  if (is_zero) {
    VLOG(5) << api << " Skip output zero element tensor.";
    return MLUOP_STATUS_SUCCESS;
  }
  PARAM_CHECK(api, points != nullptr);
  PARAM_CHECK(api, voxel_size != nullptr);
  PARAM_CHECK(api, coors_range != nullptr);
  PARAM_CHECK(api, voxels != nullptr);
  PARAM_CHECK(api, coors != nullptr);
  PARAM_CHECK(api, num_points_per_voxel != nullptr);
  PARAM_CHECK(api, voxel_num != nullptr);
  const VoxelProblem p = makeProblem(points_desc, max_points, max_voxels);
  const VoxelWorkspacePlan plan = mluop::voxelization::planVoxelWorkspace(p);
  if (workspace_size < plan.total || workspace == nullptr) {
    LOG(ERROR) << api << " workspace of " << workspace_size << " bytes is smaller than the " << plan.total
               << " bytes mluOpGetVoxelizationWorkspaceSize reports.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (handle->host_only) {
    LOG(ERROR) << api << " this handle was created without a CUDA device; nothing can be launched.";
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  cudaError_t err = mluop::voxelization::launchVoxelization(
      p, plan, static_cast<const float *>(points), static_cast<const float *>(voxel_size),
      static_cast<const float *>(coors_range), workspace, static_cast<float *>(voxels),
      static_cast<int32_t *>(coors), static_cast<int32_t *>(num_points_per_voxel),
      static_cast<int32_t *>(voxel_num), handle->queue);
  if (err != cudaSuccess) {
    LOG(ERROR) << api << " launch failed: " << cudaGetErrorString(err);
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  if (mluop::checkStatusRequested()) {
    int32_t word = 0;
    const char *base = reinterpret_cast<const char *>((reinterpret_cast<size_t>(workspace) + 255) / 256 * 256);
    err = cudaMemcpyAsync(&word, base + plan.status, sizeof(word), cudaMemcpyDeviceToHost, handle->queue);
    if (err == cudaSuccess) err = cudaStreamSynchronize(handle->queue);
    if (err != cudaSuccess || word != 0) {
      LOG(ERROR) << api << " execution failed: "
                 << (err != cudaSuccess ? cudaGetErrorString(err) : "the hash table overflowed");
      return MLUOP_STATUS_EXECUTION_FAILED;
    }
  }
  return MLUOP_STATUS_SUCCESS;
}

}  // extern "C"
