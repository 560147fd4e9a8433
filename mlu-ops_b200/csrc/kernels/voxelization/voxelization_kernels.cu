// Hard voxelization (deterministic mode) for sm_100a.
//
// The operator groups points [N,F] into voxels of a regular grid: the voxels are
// numbered in the order of their first points, a voxel keeps its first max_points
// points in index order, and at most max_voxels voxels are kept (reference
// kernels/voxelization/voxelization.cpp:277-361 and voxelization_kernel.mlu: four
// kernels, of which the one that finds a point's rank inside its voxel compares
// every point with all earlier points, and the one that numbers the voxels runs
// on a single core).
//
// Here every step is linear in the number of points and parallel, and still
// deterministic:
//   hashPointsKernel     voxel coordinates of a point -> 64-bit key -> hash slot
//                        (CAS insert); atomicMin keeps the voxel's first point
//   countFirstsKernel /  a point is the first of its voxel iff first[slot] == its
//   scanChunksKernel /   index; an exclusive prefix sum of those flags in point
//   numberVoxelsKernel   order is the voxel numbering of the reference; voxels past
//                        max_voxels get -1; coors and voxel_num are written here
//   insertPointsKernel   every point of a kept voxel walks the voxel's list of
//                        max_points slots with atomicMin, carrying the larger index
//                        onward: whatever the interleaving, slot m ends up with the
//                        (m+1)-th smallest index, i.e. the points in index order
//   gatherVoxelsKernel   voxels[v][m][:] = points[list[v][m]][:] (zeros where empty),
//                        num_points_per_voxel[v] = filled slots
// All arithmetic on coordinates is the reference's float arithmetic
// (floorf((p - min) / size), grid = round((max - min) / size)), so coors are
// bit-exact.
#include "kernels/voxelization/voxelization_kernels.h"

#include <cuda_runtime.h>

#include "core/trace.h"

namespace mluop {
namespace voxelization {

namespace {

inline size_t alignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

constexpr int32_t kEmptyIndex = 0x7f7f7f7f;  // what a 0x7f byte fill leaves; above every point index

struct Grid {
  float min_x, min_y, min_z, size_x, size_y, size_z;
  int32_t nx, ny, nz;
};

__device__ __forceinline__ Grid readGrid(const float *__restrict__ voxel_size,
                                         const float *__restrict__ coors_range) {
  Grid g;
  g.size_x = voxel_size[0]; g.size_y = voxel_size[1]; g.size_z = voxel_size[2];
  g.min_x = coors_range[0]; g.min_y = coors_range[1]; g.min_z = coors_range[2];
  g.nx = (int32_t)roundf(__fdiv_rn(__fsub_rn(coors_range[3], g.min_x), g.size_x));
  g.ny = (int32_t)roundf(__fdiv_rn(__fsub_rn(coors_range[4], g.min_y), g.size_y));
  g.nz = (int32_t)roundf(__fdiv_rn(__fsub_rn(coors_range[5], g.min_z), g.size_z));
  return g;
}

// (z, y, x) of a point, false when it lies outside the grid.
__device__ __forceinline__ bool voxelOf(const Grid &g, const float *__restrict__ p, int32_t &cz, int32_t &cy,
                                        int32_t &cx) {
  cx = (int32_t)floorf(__fdiv_rn(__fsub_rn(p[0], g.min_x), g.size_x));
  if (cx < 0 || cx >= g.nx) return false;
  cy = (int32_t)floorf(__fdiv_rn(__fsub_rn(p[1], g.min_y), g.size_y));
  if (cy < 0 || cy >= g.ny) return false;
  cz = (int32_t)floorf(__fdiv_rn(__fsub_rn(p[2], g.min_z), g.size_z));
  return cz >= 0 && cz < g.nz;
}

__device__ __forceinline__ uint32_t hashKey(uint64_t key) {
  key ^= key >> 33;
  key *= 0xff51afd7ed558ccdull;
  key ^= key >> 33;
  return (uint32_t)key;
}

__global__ void __launch_bounds__(256)
hashPointsKernel(const float *__restrict__ points, int64_t n, int f, const float *__restrict__ voxel_size,
                 const float *__restrict__ coors_range, unsigned long long *__restrict__ keys,
                 int32_t *__restrict__ first, uint32_t capacity, int32_t *__restrict__ slot_of,
                 int32_t *__restrict__ status) {
  const Grid g = readGrid(voxel_size, coors_range);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int32_t cz, cy, cx;
    if (!voxelOf(g, points + i * f, cz, cy, cx)) {
      slot_of[i] = -1;
      continue;
    }
    const unsigned long long key = ((unsigned long long)cz * g.ny + cy) * g.nx + cx + 1ull;  // 0 = empty
    uint32_t slot = hashKey(key) & (capacity - 1);
    int32_t found = -1;
    for (uint32_t probe = 0; probe < capacity; ++probe) {
      const unsigned long long seen = atomicCAS(&keys[slot], 0ull, key);
      if (seen == 0ull || seen == key) {
        found = (int32_t)slot;
        break;
      }
      slot = (slot + 1) & (capacity - 1);
    }
    if (found < 0) {
      atomicOr(status, kVoxelErrHashFull);
      slot_of[i] = -1;
      continue;
    }
    atomicMin(&first[found], (int32_t)i);
    slot_of[i] = found;
  }
}

__device__ __forceinline__ bool isFirst(const int32_t *__restrict__ slot_of, const int32_t *__restrict__ first,
                                        int64_t i, int64_t n) {
  if (i >= n) return false;
  const int32_t s = slot_of[i];
  return s >= 0 && first[s] == (int32_t)i;
}

__global__ void __launch_bounds__(256)
countFirstsKernel(const int32_t *__restrict__ slot_of, const int32_t *__restrict__ first, int64_t n,
                  int32_t *__restrict__ chunk_count) {
  const int64_t base = (int64_t)blockIdx.x * kChunkPoints;
  int local = 0;
  for (int r = threadIdx.x; r < kChunkPoints; r += 256) local += isFirst(slot_of, first, base + r, n) ? 1 : 0;
  __shared__ int warp_sum[8];
  for (int o = 16; o > 0; o >>= 1) local += __shfl_down_sync(0xffffffffu, local, o);
  if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
    for (int w = 0; w < 8; ++w) s += warp_sum[w];
    chunk_count[blockIdx.x] = s;
  }
}

// One block: exclusive prefix of the chunk counts in place; total to status[1] and,
// capped, to voxel_num.
__global__ void __launch_bounds__(1024)
scanChunksKernel(int32_t *__restrict__ chunk_count, int chunks, int32_t max_voxels, int32_t *__restrict__ status,
                 int32_t *__restrict__ voxel_num) {
  __shared__ int32_t warp_total[32];
  __shared__ int32_t carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < chunks; base += 1024) {
    const int i = base + threadIdx.x;
    const int32_t v = i < chunks ? chunk_count[i] : 0;
    int32_t incl = v;
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t t = __shfl_up_sync(0xffffffffu, incl, o);
      if ((threadIdx.x & 31) >= o) incl += t;
    }
    if ((threadIdx.x & 31) == 31) warp_total[threadIdx.x >> 5] = incl;
    __syncthreads();
    if (threadIdx.x < 32) {
      int32_t w = warp_total[threadIdx.x];
      for (int o = 1; o < 32; o <<= 1) {
        const int32_t t = __shfl_up_sync(0xffffffffu, w, o);
        if (threadIdx.x >= o) w += t;
      }
      warp_total[threadIdx.x] = w;  // inclusive over warps
    }
    __syncthreads();
    const int32_t before = carry + (threadIdx.x >= 32 ? warp_total[(threadIdx.x >> 5) - 1] : 0);
    if (i < chunks) chunk_count[i] = before + incl - v;
    __syncthreads();
    if (threadIdx.x == 0) carry += warp_total[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    status[1] = carry;
    *voxel_num = carry < max_voxels ? carry : max_voxels;
  }
}

__global__ void __launch_bounds__(256)
numberVoxelsKernel(const float *__restrict__ points, int64_t n, int f, const float *__restrict__ voxel_size,
                   const float *__restrict__ coors_range, const int32_t *__restrict__ slot_of,
                   const int32_t *__restrict__ first, const int32_t *__restrict__ chunk_offset,
                   int32_t max_voxels, int32_t *__restrict__ voxel_of, int32_t *__restrict__ coors) {
  const Grid g = readGrid(voxel_size, coors_range);
  const int64_t base = (int64_t)blockIdx.x * kChunkPoints;
  __shared__ int32_t warp_total[8];
  __shared__ int32_t running;
  if (threadIdx.x == 0) running = chunk_offset[blockIdx.x];
  __syncthreads();
  // four rounds of 256 consecutive points keep the numbering in point order
  for (int round = 0; round < kChunkPoints / 256; ++round) {
    const int64_t i = base + round * 256 + threadIdx.x;
    const bool flag = isFirst(slot_of, first, i, n);
    const unsigned ballot = __ballot_sync(0xffffffffu, flag);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) warp_total[warp] = __popc(ballot);
    __syncthreads();
    int32_t before = running;
    for (int w = 0; w < warp; ++w) before += warp_total[w];
    const int32_t id = before + __popc(ballot & ((1u << lane) - 1u));
    if (flag) {
      const int32_t s = slot_of[i];
      if (id < max_voxels) {
        voxel_of[s] = id;
        int32_t cz, cy, cx;
        voxelOf(g, points + i * f, cz, cy, cx);
        coors[(size_t)id * 3 + 0] = cz;
        coors[(size_t)id * 3 + 1] = cy;
        coors[(size_t)id * 3 + 2] = cx;
      } else {
        voxel_of[s] = -1;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int32_t s = 0;
      for (int w = 0; w < 8; ++w) s += warp_total[w];
      running += s;
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(256)
insertPointsKernel(const int32_t *__restrict__ slot_of, const int32_t *__restrict__ voxel_of, int64_t n,
                   int32_t max_points, int32_t *__restrict__ lists) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int32_t s = slot_of[i];
    if (s < 0) continue;
    const int32_t v = voxel_of[s];
    if (v < 0) continue;
    int32_t *list = lists + (size_t)v * max_points;
    int32_t carried = (int32_t)i;
    for (int m = 0; m < max_points; ++m) {
      const int32_t old = atomicMin(&list[m], carried);
      if (old == kEmptyIndex) break;       // took an empty slot
      if (old > carried) carried = old;    // took the slot of a later point: that one moves on
    }
  }
}

__global__ void __launch_bounds__(256)
gatherVoxelsKernel(const float *__restrict__ points, int f, const int32_t *__restrict__ lists,
                   const int32_t *__restrict__ voxel_num, int32_t max_voxels, int32_t max_points,
                   float *__restrict__ voxels, int32_t *__restrict__ num_points_per_voxel) {
  const int32_t kept = *voxel_num;
  const int64_t per_voxel = (int64_t)max_points * f;
  const int64_t total = (int64_t)max_voxels * per_voxel;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t v = e / per_voxel;
    const int m = (int)((e % per_voxel) / f), c = (int)(e % f);
    float value = 0.0f;
    if (v < kept) {
      const int32_t idx = lists[v * max_points + m];
      if (idx != kEmptyIndex) value = points[(int64_t)idx * f + c];
    }
    voxels[e] = value;
    if (m == 0 && c == 0) {
      int32_t count = 0;
      if (v < kept)
        for (int q = 0; q < max_points; ++q) count += lists[v * max_points + q] != kEmptyIndex ? 1 : 0;
      num_points_per_voxel[v] = count;
    }
  }
}

unsigned gridFor(int64_t work, int threads) {
  int64_t b = (work + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > 148 * 32) b = 148 * 32;
  return (unsigned)b;
}

}  // namespace

VoxelWorkspacePlan planVoxelWorkspace(const VoxelProblem &p) {
  VoxelWorkspacePlan plan{};
  uint32_t cap = 1024;
  while ((int64_t)cap < 2 * p.num_points) cap <<= 1;
  plan.capacity = cap;
  plan.chunks = (int32_t)((p.num_points + kChunkPoints - 1) / kChunkPoints);
  size_t off = 0;
  plan.status = off;
  off = alignUp(off + 64 * sizeof(int32_t), 256);
  plan.keys = off;
  off = alignUp(off + (size_t)cap * sizeof(uint64_t), 256);
  plan.first = off;
  off = alignUp(off + (size_t)cap * sizeof(int32_t), 256);
  plan.voxel_of = off;
  off = alignUp(off + (size_t)cap * sizeof(int32_t), 256);
  plan.slot_of = off;
  off = alignUp(off + (size_t)p.num_points * sizeof(int32_t), 256);
  plan.chunk_count = off;
  off = alignUp(off + (size_t)(plan.chunks > 0 ? plan.chunks : 1) * sizeof(int32_t), 256);
  plan.lists = off;
  off = alignUp(off + (size_t)p.max_voxels * p.max_points * sizeof(int32_t), 256);
  plan.total = off + 256;
  return plan;
}

cudaError_t launchVoxelization(const VoxelProblem &p, const VoxelWorkspacePlan &plan, const float *points,
                               const float *voxel_size, const float *coors_range, void *workspace,
                               float *voxels, int32_t *coors, int32_t *num_points_per_voxel,
                               int32_t *voxel_num, cudaStream_t stream) {
  char *base = reinterpret_cast<char *>(alignUp(reinterpret_cast<size_t>(workspace), 256));
  int32_t *status = reinterpret_cast<int32_t *>(base + plan.status);
  unsigned long long *keys = reinterpret_cast<unsigned long long *>(base + plan.keys);
  int32_t *first = reinterpret_cast<int32_t *>(base + plan.first);
  int32_t *voxel_of = reinterpret_cast<int32_t *>(base + plan.voxel_of);
  int32_t *slot_of = reinterpret_cast<int32_t *>(base + plan.slot_of);
  int32_t *chunk_count = reinterpret_cast<int32_t *>(base + plan.chunk_count);
  int32_t *lists = reinterpret_cast<int32_t *>(base + plan.lists);
  const int64_t n = p.num_points;
  const int f = p.num_features;
  cudaError_t err;
  {
    trace::Scope t("memset:voxel_tables", stream, 16.0 * plan.capacity + 4.0 * p.max_voxels * p.max_points);
    if ((err = cudaMemsetAsync(status, 0, 64 * sizeof(int32_t), stream)) != cudaSuccess) return err;
    if ((err = cudaMemsetAsync(keys, 0, (size_t)plan.capacity * sizeof(uint64_t), stream)) != cudaSuccess) return err;
    // first and lists start "empty": a 0x7f fill is 0x7f7f7f7f, above every point index
    if ((err = cudaMemsetAsync(first, 0x7f, (size_t)plan.capacity * sizeof(int32_t), stream)) != cudaSuccess)
      return err;
    if ((err = cudaMemsetAsync(lists, 0x7f, (size_t)p.max_voxels * p.max_points * sizeof(int32_t), stream)) !=
        cudaSuccess)
      return err;
    if ((err = cudaMemsetAsync(coors, 0, (size_t)p.max_voxels * 3 * sizeof(int32_t), stream)) != cudaSuccess)
      return err;
  }
  {
    trace::Scope t("hashPointsKernel", stream, (double)n * (12.0 + 4.0 + 12.0));
    hashPointsKernel<<<gridFor(n, 256), 256, 0, stream>>>(points, n, f, voxel_size, coors_range, keys, first,
                                                          plan.capacity, slot_of, status);
  }
  {
    trace::Scope t("countFirstsKernel", stream, 8.0 * n);
    countFirstsKernel<<<(unsigned)plan.chunks, 256, 0, stream>>>(slot_of, first, n, chunk_count);
  }
  {
    trace::Scope t("scanChunksKernel", stream, 8.0 * plan.chunks);
    scanChunksKernel<<<1, 1024, 0, stream>>>(chunk_count, plan.chunks, p.max_voxels, status, voxel_num);
  }
  {
    trace::Scope t("numberVoxelsKernel", stream, 8.0 * n + 12.0 * p.max_voxels);
    numberVoxelsKernel<<<(unsigned)plan.chunks, 256, 0, stream>>>(points, n, f, voxel_size, coors_range, slot_of,
                                                                  first, chunk_count, p.max_voxels, voxel_of,
                                                                  coors);
  }
  {
    trace::Scope t("insertPointsKernel", stream, 12.0 * n);
    insertPointsKernel<<<gridFor(n, 256), 256, 0, stream>>>(slot_of, voxel_of, n, p.max_points, lists);
  }
  {
    const int64_t out = (int64_t)p.max_voxels * p.max_points * f;
    trace::Scope t("gatherVoxelsKernel", stream, 8.0 * out + 4.0 * p.max_voxels * p.max_points);
    gatherVoxelsKernel<<<gridFor(out, 256), 256, 0, stream>>>(points, f, lists, voxel_num, p.max_voxels,
                                                              p.max_points, voxels, num_points_per_voxel);
  }
  return cudaGetLastError();
}

}  // namespace voxelization
}  // namespace mluop
