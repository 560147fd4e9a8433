/*
 * CPU oracle for hard voxelization (deterministic mode).  TEST INFRASTRUCTURE ONLY.
 *
 * Restates the reference's CPU implementation,
 * test/mlu_op_gtest/pb_gtest/src/zoo/voxelization/voxelization.cpp:
 *   :129-163 dynamicVoxelize        coordinates (z, y, x) of every point, -1 when outside
 *   :165-206 pointToVoxelidx        rank of a point among the earlier points of its voxel
 *                                   (-1 from max_points on) and the index of the voxel's
 *                                   first point
 *   :208-234 determinVoxelNum       voxels numbered in the order of their first points,
 *                                   at most max_voxels; points per voxel
 *   :236-270 assignPointToVoxel / assignVoxelCoors
 *   :272-330 deterministic_hard_voxelize (grid size = round((max - min) / voxel_size))
 * The reference's loops are quadratic in the number of points; this restatement
 * keeps their results and is quadratic too (tests use a few thousand points).
 *
 * Outputs follow the library's types: coors, num_points_per_voxel and voxel_num are
 * int32 (the reference's CPU path holds them as float copies of the same integers),
 * and rows the operator does not assign are zero (the reference fills the three
 * output tensors with zeros first, kernels/voxelization/voxelization.cpp:296-321).
 *
 * Parity status: pinned against the reference's own function bodies compiled by
 * oracle/build_ref.py and against tests/golden/voxelization_golden.npz.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

int mluops_oracle_voxelization(const float *points, int64_t num_points, int64_t num_features,
                               const float *voxel_size, const float *coors_range,
                               int32_t max_points, int32_t max_voxels, float *voxels,
                               int32_t *coors, int32_t *num_points_per_voxel, int32_t *voxel_num) {
  const int NDim = 3;
  const int32_t grid_x = (int32_t)roundf((coors_range[3] - coors_range[0]) / voxel_size[0]);
  const int32_t grid_y = (int32_t)roundf((coors_range[4] - coors_range[1]) / voxel_size[1]);
  const int32_t grid_z = (int32_t)roundf((coors_range[5] - coors_range[2]) / voxel_size[2]);
  memset(voxels, 0, sizeof(float) * (size_t)max_voxels * max_points * num_features);
  memset(coors, 0, sizeof(int32_t) * (size_t)max_voxels * NDim);
  memset(num_points_per_voxel, 0, sizeof(int32_t) * (size_t)max_voxels);
  *voxel_num = 0;
  if (num_points == 0) return 0;
  int32_t *c = (int32_t *)malloc(sizeof(int32_t) * (size_t)num_points * NDim);
  int32_t *first = (int32_t *)malloc(sizeof(int32_t) * (size_t)num_points);
  int32_t *rank = (int32_t *)malloc(sizeof(int32_t) * (size_t)num_points);
  int32_t *voxel_of = (int32_t *)malloc(sizeof(int32_t) * (size_t)num_points);
  if (!c || !first || !rank || !voxel_of) return -1;

  for (int64_t i = 0; i < num_points; ++i) {
    const float *p = points + i * num_features;
    int32_t *o = c + i * NDim;
    o[0] = o[1] = o[2] = -1;
    const int32_t cx = (int32_t)floorf((p[0] - coors_range[0]) / voxel_size[0]);
    if (cx < 0 || cx >= grid_x) continue;
    const int32_t cy = (int32_t)floorf((p[1] - coors_range[1]) / voxel_size[1]);
    if (cy < 0 || cy >= grid_y) continue;
    const int32_t cz = (int32_t)floorf((p[2] - coors_range[2]) / voxel_size[2]);
    if (cz < 0 || cz >= grid_z) continue;
    o[0] = cz; o[1] = cy; o[2] = cx;
  }

  for (int64_t i = 0; i < num_points; ++i) {
    const int32_t *ci = c + i * NDim;
    if (ci[0] == -1) {
      first[i] = -1;
      rank[i] = -1;
      continue;
    }
    int32_t num = 0;
    for (int64_t j = 0; j < i; ++j) {
      const int32_t *cj = c + j * NDim;
      if (cj[0] == -1) continue;
      if (cj[0] == ci[0] && cj[1] == ci[1] && cj[2] == ci[2]) {
        ++num;
        if (num == 1) first[i] = (int32_t)j;
        else if (num >= max_points) break;
      }
    }
    if (num == 0) first[i] = (int32_t)i;
    rank[i] = num < max_points ? num : -1;
  }

  int32_t count = 0;
  for (int64_t i = 0; i < num_points; ++i) {
    voxel_of[i] = -1;
    if (rank[i] == -1) continue;
    if (rank[i] == 0) {
      if (count >= max_voxels) continue;
      voxel_of[i] = count;
      num_points_per_voxel[count] = 1;
      ++count;
    } else {
      const int32_t v = voxel_of[first[i]];
      if (v != -1) {
        voxel_of[i] = v;
        num_points_per_voxel[v] += 1;
      }
    }
  }
  *voxel_num = count;

  for (int64_t i = 0; i < num_points; ++i) {
    if (rank[i] < 0 || voxel_of[i] < 0) continue;
    memcpy(voxels + ((size_t)voxel_of[i] * max_points + rank[i]) * num_features,
           points + i * num_features, sizeof(float) * (size_t)num_features);
    if (rank[i] == 0) memcpy(coors + (size_t)voxel_of[i] * NDim, c + i * NDim, sizeof(int32_t) * NDim);
  }
  free(c); free(first); free(rank); free(voxel_of);
  return 0;
}
