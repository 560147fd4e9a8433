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

/*
 * Dynamic point-to-voxel scatter, forward (reference
 * test/mlu_op_gtest/pb_gtest/src/zoo/dynamic_point_to_voxel_forward/
 * dynamic_point_to_voxel_forward.cpp:107-247):
 *   rows of coors with a negative entry become (-1,-1,-1) (in place);
 *   point indices are sorted by their coordinates (lexicographic) and made
 *   unique; a leading (-1,-1,-1) voxel is dropped; point2voxel_map, the points
 *   per voxel; voxel_feats starts at -1.17549e38 (maximum) or 0 (mean) in every
 *   row and is reduced over the points in index order, the mean as
 *   sum_i feats_i / count.
 * The reference sorts with std::sort, which may order equal coordinates
 * differently; nothing that is output depends on that order.
 * reduce_max: 1 maximum, 0 mean.  voxel_rows: rows of the voxel_* outputs.
 */
static const int32_t *dpv_coors;
static int dpv_cmp(const void *a, const void *b) {
  const int32_t i = *(const int32_t *)a, j = *(const int32_t *)b;
  for (int d = 0; d < 3; ++d) {
    if (dpv_coors[i * 3 + d] < dpv_coors[j * 3 + d]) return -1;
    if (dpv_coors[i * 3 + d] > dpv_coors[j * 3 + d]) return 1;
  }
  return (i > j) - (i < j);
}

int mluops_oracle_dynamic_point_to_voxel_forward(const float *feats, int32_t *coors, int64_t n,
                                                 int64_t c_num, int64_t voxel_rows, int32_t reduce_max,
                                                 float *voxel_feats, int32_t *voxel_coors,
                                                 int32_t *point2voxel_map, int32_t *voxel_points_count,
                                                 int32_t *voxel_num) {
  for (int64_t i = 0; i < n; ++i)
    if (coors[i * 3] < 0 || coors[i * 3 + 1] < 0 || coors[i * 3 + 2] < 0)
      coors[i * 3] = coors[i * 3 + 1] = coors[i * 3 + 2] = -1;
  int32_t *order = (int32_t *)malloc(sizeof(int32_t) * (size_t)(n > 0 ? n : 1));
  if (!order) return -1;
  for (int64_t i = 0; i < n; ++i) order[i] = (int32_t)i;
  dpv_coors = coors;
  qsort(order, (size_t)n, sizeof(int32_t), dpv_cmp);
  const float fill = reduce_max ? -1.17549e38f : 0.0f;
  for (int64_t i = 0; i < voxel_rows * c_num; ++i) voxel_feats[i] = fill;
  int32_t voxels = 0;
  for (int64_t s = 0; s < n;) {
    int64_t e = s + 1;
    while (e < n && memcmp(coors + (size_t)order[s] * 3, coors + (size_t)order[e] * 3, 12) == 0) ++e;
    const int invalid = coors[(size_t)order[s] * 3] == -1;
    for (int64_t q = s; q < e; ++q) point2voxel_map[order[q]] = invalid ? -1 : voxels;
    if (!invalid) {
      if (voxels < voxel_rows) {
        memcpy(voxel_coors + (size_t)voxels * 3, coors + (size_t)order[s] * 3, 12);
        voxel_points_count[voxels] = (int32_t)(e - s);
      }
      ++voxels;
    }
    s = e;
  }
  *voxel_num = voxels;
  for (int64_t i = 0; i < n; ++i) {
    const int32_t v = point2voxel_map[i];
    if (v < 0 || v >= voxel_rows) continue;
    const int32_t count = voxel_points_count[v];
    for (int64_t c = 0; c < c_num; ++c) {
      float *dst = voxel_feats + (size_t)v * c_num + c;
      const float x = feats[i * c_num + c];
      if (reduce_max) {
        if (x >= *dst) *dst = x;
      } else {
        volatile float term = x / count;
        *dst += term;
      }
    }
  }
  free(order);
  return 0;
}

/*
 * Gradient of the maximum reduction of the dynamic point-to-voxel scatter
 * (reference test/mlu_op_gtest/pb_gtest/src/zoo/dynamic_point_to_voxel_backward/
 * dynamic_point_to_voxel_backward.cpp:108-163): per voxel and channel the
 * smallest point index whose feature equals the voxel's maximum receives the
 * voxel's gradient; everything else in grad_feats [n,c] is zero.
 */
int mluops_oracle_dynamic_point_to_voxel_backward(const float *grad_voxel_feats, const float *feats,
                                                  const float *voxel_feats, const int32_t *point2voxel_map,
                                                  int32_t voxel_num, int64_t n, int64_t c_num,
                                                  float *grad_feats) {
  memset(grad_feats, 0, sizeof(float) * (size_t)(n * c_num));
  if (voxel_num <= 0 || n == 0) return 0;
  int32_t *from = (int32_t *)malloc(sizeof(int32_t) * (size_t)voxel_num * c_num);
  if (!from) return -1;
  for (int64_t i = 0; i < (int64_t)voxel_num * c_num; ++i) from[i] = (int32_t)n;
  for (int64_t x = 0; x < n; ++x) {
    const int32_t v = point2voxel_map[x];
    if (v == -1) continue;
    for (int64_t c = 0; c < c_num; ++c)
      if (feats[x * c_num + c] == voxel_feats[(int64_t)v * c_num + c] && x < from[(int64_t)v * c_num + c])
        from[(int64_t)v * c_num + c] = (int32_t)x;
  }
  for (int64_t v = 0; v < voxel_num; ++v)
    for (int64_t c = 0; c < c_num; ++c)
      if (from[v * c_num + c] < n) grad_feats[(int64_t)from[v * c_num + c] * c_num + c] = grad_voxel_feats[v * c_num + c];
  free(from);
  return 0;
}
