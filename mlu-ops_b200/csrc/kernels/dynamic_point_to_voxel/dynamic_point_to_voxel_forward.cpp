// mluOpDynamicPointToVoxelForward / mluOpGetDynamicPointToVoxelForwardWorkspaceSize:
// argument checks and dispatch (reference kernels/dynamic_point_to_voxel/
// dynamic_point_to_voxel_forward/dynamic_point_to_voxel_forward.cpp: parameter
// check :70-191, workspace query :193-224, compute entry :226-352).
//
// The order of the checks, and the status each returns, follows the reference.
// The workspace size is this implementation's own (two copies of 16-byte sort
// records and the radix-sort counters, where the reference asks its vendor
// library's "unique" for a size); a workspace smaller than the query result is
// rejected with MLUOP_STATUS_BAD_PARAM.
#include <cuda_runtime_api.h>

#include <string>

#include "core/context.h"
#include "core/logging.h"
#include "core/tensor.h"
#include "kernels/dynamic_point_to_voxel/dynamic_point_to_voxel_forward_kernels.h"

using mluop::dynamic_point_to_voxel::PointToVoxelProblem;
using mluop::dynamic_point_to_voxel::PointToVoxelWorkspacePlan;

extern "C" {

mluOpStatus_t MLUOP_WIN_API mluOpGetDynamicPointToVoxelForwardWorkspaceSize(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t feats_desc, const mluOpTensorDescriptor_t coors_desc,
    size_t *workspace_size) {
  const std::string api = "[mluOpGetDynamicPointToVoxelForwardWorkspaceSize]";
  PARAM_CHECK(api, handle != nullptr);
  if (handle->arch < MLUOP_MLU370) {
    LOG(ERROR) << api << " needs a compute-capability 10.x device; this handle's device is not one.";
    return MLUOP_STATUS_ARCH_MISMATCH;
  }
  PARAM_CHECK(api, feats_desc != nullptr);
  PARAM_CHECK(api, coors_desc != nullptr);
  PARAM_CHECK(api, workspace_size != nullptr);
  PARAM_CHECK(api, coors_desc->getDim() == 2);
  PointToVoxelProblem p{};
  p.num_points = coors_desc->getDimIndex(0);
  *workspace_size = mluop::dynamic_point_to_voxel::planPointToVoxelWorkspace(p).total;
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpDynamicPointToVoxelForward(
    const mluOpHandle_t handle, const mluOpReduceMode_t reduce_type, const mluOpTensorDescriptor_t feats_desc,
    const void *feats, const mluOpTensorDescriptor_t coors_desc, void *coors, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t voxel_feats_desc, void *voxel_feats,
    const mluOpTensorDescriptor_t voxel_coors_desc, void *voxel_coors,
    const mluOpTensorDescriptor_t point2voxel_map_desc, void *point2voxel_map,
    const mluOpTensorDescriptor_t voxel_points_count_desc, void *voxel_points_count,
    const mluOpTensorDescriptor_t voxel_num_desc, void *voxel_num) {
  const std::string api = "[mluOpDynamicPointToVoxelForward]";
  PARAM_CHECK(api, handle != nullptr);
  if (handle->arch < MLUOP_MLU370) {
    LOG(ERROR) << api << " needs a compute-capability 10.x device; this handle's device is not one.";
    return MLUOP_STATUS_ARCH_MISMATCH;
  }
  PARAM_CHECK(api, feats_desc != nullptr);
  PARAM_CHECK(api, coors_desc != nullptr);
  PARAM_CHECK(api, voxel_feats_desc != nullptr);
  PARAM_CHECK(api, voxel_coors_desc != nullptr);
  PARAM_CHECK(api, point2voxel_map_desc != nullptr);
  PARAM_CHECK(api, voxel_points_count_desc != nullptr);
  PARAM_CHECK(api, voxel_num_desc != nullptr);
  PARAM_CHECK(api, feats_desc->getDim() == 2);
  PARAM_CHECK(api, coors_desc->getDim() == 2);
  PARAM_CHECK(api, voxel_feats_desc->getDim() == 2);
  PARAM_CHECK(api, voxel_coors_desc->getDim() == 2);
  PARAM_CHECK(api, point2voxel_map_desc->getDim() == 1);
  PARAM_CHECK(api, voxel_points_count_desc->getDim() == 1);
  PARAM_CHECK(api, voxel_num_desc->getDim() == 1);
  STRIDE_TENSOR_CHECK(api + ":", feats_desc, "feats_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", coors_desc, "coors_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", voxel_feats_desc, "voxel_feats_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", voxel_coors_desc, "voxel_coors_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", point2voxel_map_desc, "point2voxel_map_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", voxel_points_count_desc, "voxel_points_count_desc must be contiguous");
  STRIDE_TENSOR_CHECK(api + ":", voxel_num_desc, "voxel_num_desc must be contiguous");
  PARAM_CHECK(api, feats_desc->getDtype() == MLUOP_DTYPE_FLOAT);
  PARAM_CHECK(api, coors_desc->getDtype() == MLUOP_DTYPE_INT32);
  PARAM_CHECK(api, point2voxel_map_desc->getDtype() == MLUOP_DTYPE_INT32);
  PARAM_CHECK(api, voxel_feats_desc->getDtype() == feats_desc->getDtype());
  PARAM_CHECK(api, voxel_coors_desc->getDtype() == coors_desc->getDtype());
  PARAM_CHECK(api, voxel_points_count_desc->getDtype() == point2voxel_map_desc->getDtype());
  PARAM_CHECK(api, voxel_num_desc->getDtype() == point2voxel_map_desc->getDtype());
  if (reduce_type != MLUOP_REDUCE_DMAX && reduce_type != MLUOP_REDUCE_DMEAN) {
    LOG(ERROR) << api << " Only support max and mean. Please check reduce_type!";
    return MLUOP_STATUS_BAD_PARAM;
  }
  PARAM_CHECK(api, feats_desc->getDimIndex(0) == coors_desc->getDimIndex(0));
  PARAM_CHECK(api, feats_desc->getDimIndex(0) == point2voxel_map_desc->getDimIndex(0));
  PARAM_CHECK(api, voxel_feats_desc->getDimIndex(0) == voxel_coors_desc->getDimIndex(0));
  PARAM_CHECK(api, voxel_feats_desc->getDimIndex(0) == voxel_points_count_desc->getDimIndex(0));
  PARAM_CHECK(api, voxel_num_desc->getDimIndex(0) == 1);
  PARAM_CHECK(api, feats_desc->getDimIndex(1) == voxel_feats_desc->getDimIndex(1));
  PARAM_CHECK(api, coors_desc->getDimIndex(1) == voxel_coors_desc->getDimIndex(1));
  PARAM_CHECK(api, coors_desc->getDimIndex(1) == 3);
  PARAM_CHECK(api, feats_desc->getDimIndex(0) >= voxel_feats_desc->getDimIndex(0));
  if (mluOpGetTensorElementNum(feats_desc) >= LARGE_TENSOR_NUM ||
      mluOpGetTensorElementNum(coors_desc) >= LARGE_TENSOR_NUM) {
    LOG(ERROR) << api << " Overflow max tensor num. Tensors must have fewer than 2^31 elements.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }
  if (mluOpGetTensorElementNum(feats_desc) == 0 || mluOpGetTensorElementNum(coors_desc) == 0) {
    VLOG(5) << api << " Skip zero element tensor.";
    return MLUOP_STATUS_SUCCESS;
  }
  if (workspace_size > 0) {
    PARAM_CHECK(api, workspace != nullptr);
  }
  PARAM_CHECK(api, feats != nullptr);
  PARAM_CHECK(api, coors != nullptr);
  PARAM_CHECK(api, voxel_feats != nullptr);
  PARAM_CHECK(api, voxel_coors != nullptr);
  PARAM_CHECK(api, point2voxel_map != nullptr);
  PARAM_CHECK(api, voxel_points_count != nullptr);
  PARAM_CHECK(api, voxel_num != nullptr);

  PointToVoxelProblem p{};
  p.num_points = feats_desc->getDimIndex(0);
  p.num_feats = (int32_t)feats_desc->getDimIndex(1);
  p.voxel_rows = voxel_feats_desc->getDimIndex(0);
  p.reduce_max = reduce_type == MLUOP_REDUCE_DMAX;
  const PointToVoxelWorkspacePlan plan = mluop::dynamic_point_to_voxel::planPointToVoxelWorkspace(p);
  if (workspace_size < plan.total || workspace == nullptr) {
    LOG(ERROR) << api << " workspace of " << workspace_size << " bytes is smaller than the " << plan.total
               << " bytes mluOpGetDynamicPointToVoxelForwardWorkspaceSize reports.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  if (handle->host_only) {
    LOG(ERROR) << api << " this handle was created without a CUDA device; nothing can be launched.";
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  cudaError_t err = mluop::dynamic_point_to_voxel::launchDynamicPointToVoxelForward(
      p, plan, static_cast<const float *>(feats), static_cast<int32_t *>(coors), workspace,
      static_cast<float *>(voxel_feats), static_cast<int32_t *>(voxel_coors),
      static_cast<int32_t *>(point2voxel_map), static_cast<int32_t *>(voxel_points_count),
      static_cast<int32_t *>(voxel_num), handle->queue);
  if (err != cudaSuccess) {
    LOG(ERROR) << api << " launch failed: " << cudaGetErrorString(err);
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  return MLUOP_STATUS_SUCCESS;
}

}  // extern "C"
