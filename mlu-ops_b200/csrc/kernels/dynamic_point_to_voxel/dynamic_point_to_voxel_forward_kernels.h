// Device side of dynamic point-to-voxel scatter (forward): workspace plan and
// launch sequence.  Argument checks live in dynamic_point_to_voxel_forward.cpp.
#ifndef MLUOP_B200_KERNELS_DYNAMIC_POINT_TO_VOXEL_FORWARD_KERNELS_H_
#define MLUOP_B200_KERNELS_DYNAMIC_POINT_TO_VOXEL_FORWARD_KERNELS_H_

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

namespace mluop {
namespace dynamic_point_to_voxel {

// Records sorted by one thread block per radix pass; points numbered by one block
// of the segment kernels.
constexpr int kSortTile = 2048;
constexpr int kRadixBins = 256;
// 12 byte digits of the three coordinates (last coordinate least significant) and
// one digit for the "no voxel" flag on top.
constexpr int kRadixPasses = 13;

struct PointToVoxelProblem {
  int64_t num_points;
  int32_t num_feats;
  int64_t voxel_rows;  // rows of the voxel_* outputs (<= num_points)
  int32_t reduce_max;  // 1: maximum, 0: mean
};

struct PointToVoxelWorkspacePlan {
  size_t records;     // uint4[2][num_points]: {c0, c1, c2, point index | invalid << 31}, ping-pong
  size_t block_hist;  // int32[256][tiles]: digit counts per tile, then per digit their exclusive prefix
  size_t source;      // int32[32]: which half of `records` a pass reads; then int32[256] digit totals
  size_t chunk_count; // int32[tiles]: segment heads per tile, then exclusive prefix
  size_t seg_start;   // int32[num_points + 1]: first sorted position of every voxel
  size_t total;
  int32_t tiles;
};

PointToVoxelWorkspacePlan planPointToVoxelWorkspace(const PointToVoxelProblem &p);

cudaError_t launchDynamicPointToVoxelForward(const PointToVoxelProblem &p, const PointToVoxelWorkspacePlan &plan,
                                             const float *feats, int32_t *coors, void *workspace,
                                             float *voxel_feats, int32_t *voxel_coors, int32_t *point2voxel_map,
                                             int32_t *voxel_points_count, int32_t *voxel_num,
                                             cudaStream_t stream);

}  // namespace dynamic_point_to_voxel
}  // namespace mluop

#endif  // MLUOP_B200_KERNELS_DYNAMIC_POINT_TO_VOXEL_FORWARD_KERNELS_H_
