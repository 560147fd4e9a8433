// Device side of hard voxelization (deterministic mode): workspace plan and
// launch sequence.  Argument checks live in voxelization.cpp.
#ifndef MLUOP_B200_KERNELS_VOXELIZATION_VOXELIZATION_KERNELS_H_
#define MLUOP_B200_KERNELS_VOXELIZATION_VOXELIZATION_KERNELS_H_

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

namespace mluop {
namespace voxelization {

// Points handled by one thread block of the numbering kernels.
constexpr int kChunkPoints = 1024;

struct VoxelProblem {
  int64_t num_points;
  int32_t num_features;
  int32_t max_points;
  int32_t max_voxels;
};

// Byte offsets of the scratch arrays inside the (256-byte aligned) workspace.
struct VoxelWorkspacePlan {
  size_t status;       // int32[64]: [0] error bits, [1] number of voxels before the max_voxels cap
  size_t keys;         // uint64[capacity]: linear voxel index + 1 per hash slot (0 = empty)
  size_t first;        // int32[capacity]: smallest point index of the slot's voxel
  size_t voxel_of;     // int32[capacity]: output row of the slot's voxel, -1 when past max_voxels
  size_t slot_of;      // int32[num_points]: hash slot of the point's voxel, -1 outside the range
  size_t chunk_count;  // int32[chunks]: first points per chunk, then their exclusive prefix
  size_t lists;        // int32[max_voxels][max_points]: point indices of a voxel, ascending
  size_t total;
  uint32_t capacity;   // power of two >= 2 * num_points
  int32_t chunks;
};

VoxelWorkspacePlan planVoxelWorkspace(const VoxelProblem &p);

constexpr int kVoxelErrHashFull = 1;  // a probe ran through the whole table

cudaError_t launchVoxelization(const VoxelProblem &p, const VoxelWorkspacePlan &plan, const float *points,
                               const float *voxel_size, const float *coors_range, void *workspace,
                               float *voxels, int32_t *coors, int32_t *num_points_per_voxel,
                               int32_t *voxel_num, cudaStream_t stream);

}  // namespace voxelization
}  // namespace mluop

#endif  // MLUOP_B200_KERNELS_VOXELIZATION_VOXELIZATION_KERNELS_H_
