// Dynamic point-to-voxel scatter (forward) for sm_100a.
//
// Points with integer voxel coordinates coors [N,3] are grouped by voxel: the
// distinct coordinates in ascending lexicographic order (voxel_coors), the voxel
// of every point (point2voxel_map, -1 for a point with a negative coordinate),
// the points per voxel, and per voxel the maximum or the mean of the features of
// its points (reference kernels/dynamic_point_to_voxel/dynamic_point_to_voxel_forward/
// dynamic_point_to_voxel_forward.cpp:226-352: a mask-fill kernel, the vendor
// library's sort-based "unique", a fill and an atomic reduce kernel).
//
// Here one stable least-significant-digit radix sort of the records
// {c0, c1, c2, point index} does all the grouping:
//   makeRecordsKernel      coordinates with a negative entry become (-1,-1,-1) in
//                          coors (as the reference does, in place) and get the
//                          "no voxel" flag, the most significant sort digit
//   histKernel / scanDigitRowsKernel / scatterKernel, once per 8-bit digit (13
//                          passes): per-tile digit counts, per digit an exclusive
//                          scan over the tiles (256 blocks), stable scatter (ranks
//                          inside a tile from warp match masks and per-warp counts,
//                          no atomics).  A digit on which all records agree is
//                          seen in the digit totals and its scatter is skipped, so
//                          small coordinates cost few passes; nothing is decided
//                          on the host
//   countHeadsKernel / scanHeadsKernel / numberSegmentsKernel
//                          a sorted record starts a voxel when its coordinates
//                          differ from its predecessor's; the prefix sum of those
//                          flags numbers the voxels in ascending order
//   reduceSegmentsKernel   one thread per (voxel, channel) walks the voxel's
//                          records, which the stable sort left in point order:
//                          the mean is summed in exactly the reference's order
//                          (sum of feats / count), so it is reproducible, and no
//                          float atomics are needed
#include "kernels/dynamic_point_to_voxel/dynamic_point_to_voxel_forward_kernels.h"

#include <cuda_runtime.h>

#include <cmath>

#include "core/trace.h"

namespace mluop {
namespace dynamic_point_to_voxel {

namespace {

inline size_t alignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

constexpr unsigned kInvalidBit = 0x80000000u;

__device__ __forceinline__ unsigned digitOf(const uint4 &r, int pass) {
  if (pass < 4) return (r.z >> (8 * pass)) & 0xffu;
  if (pass < 8) return (r.y >> (8 * (pass - 4))) & 0xffu;
  if (pass < 12) return (r.x >> (8 * (pass - 8))) & 0xffu;
  return r.w >> 31;
}

__global__ void __launch_bounds__(256)
makeRecordsKernel(int32_t *__restrict__ coors, int64_t n, uint4 *__restrict__ records, int32_t *__restrict__ source) {
  if (blockIdx.x == 0 && threadIdx.x == 0) source[0] = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int32_t a = coors[i * 3], b = coors[i * 3 + 1], c = coors[i * 3 + 2];
    uint4 r;
    if (a < 0 || b < 0 || c < 0) {
      coors[i * 3] = -1;
      coors[i * 3 + 1] = -1;
      coors[i * 3 + 2] = -1;
      r = make_uint4(0u, 0u, 0u, (unsigned)i | kInvalidBit);
    } else {
      r = make_uint4((unsigned)a, (unsigned)b, (unsigned)c, (unsigned)i);
    }
    records[i] = r;
  }
}

// block_hist[digit][tile] = records of the tile with that digit.
__global__ void __launch_bounds__(256)
histKernel(const uint4 *__restrict__ records, int64_t n, int pass, const int32_t *__restrict__ source, int tiles,
           int32_t *__restrict__ block_hist) {
  __shared__ int32_t hist[kRadixBins];
  hist[threadIdx.x] = 0;
  __syncthreads();
  const uint4 *src = records + (size_t)source[pass] * n;
  const int64_t base = (int64_t)blockIdx.x * kSortTile;
  for (int r = threadIdx.x; r < kSortTile; r += 256) {
    const int64_t i = base + r;
    if (i < n) atomicAdd(&hist[digitOf(src[i], pass)], 1);
  }
  __syncthreads();
  block_hist[(size_t)threadIdx.x * tiles + blockIdx.x] = hist[threadIdx.x];
}

// Block d: exclusive scan of digit d's counts over the tiles, in place, and the
// digit's total.  (The offsets of the digits themselves are 256 numbers: every
// block of the scatter kernel adds them up for itself.)
__global__ void __launch_bounds__(256)
scanDigitRowsKernel(int32_t *__restrict__ block_hist, int tiles, int32_t *__restrict__ digit_total) {
  __shared__ int32_t warp_total[8];
  __shared__ int32_t carry;
  int32_t *row = block_hist + (size_t)blockIdx.x * tiles;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < tiles; base += 256) {
    const int i = base + threadIdx.x;
    const int32_t v = i < tiles ? row[i] : 0;
    int32_t incl = v;
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t t = __shfl_up_sync(0xffffffffu, incl, o);
      if ((threadIdx.x & 31) >= o) incl += t;
    }
    if ((threadIdx.x & 31) == 31) warp_total[threadIdx.x >> 5] = incl;
    __syncthreads();
    int32_t before = carry;
    for (int w = 0; w < (threadIdx.x >> 5); ++w) before += warp_total[w];
    if (i < tiles) row[i] = before + incl - v;
    __syncthreads();
    if (threadIdx.x == 255) carry = before + incl;
    __syncthreads();
  }
  if (threadIdx.x == 0) digit_total[blockIdx.x] = carry;
}

// Stable scatter of one tile.  A pass on whose digit all records agree moves
// nothing: it is skipped and the next pass reads the same half of the ping-pong
// buffer (every block reaches that decision from the 256 digit totals; block 0
// records it for the kernels that follow).
__global__ void __launch_bounds__(256)
scatterKernel(uint4 *__restrict__ records, int64_t n, int pass, int32_t *__restrict__ source, int tiles,
              const int32_t *__restrict__ block_hist, const int32_t *__restrict__ digit_total) {
  __shared__ int32_t warp_count[8][kRadixBins];  // this round: records per (warp, digit)
  __shared__ int32_t running[kRadixBins];        // records of earlier rounds per digit
  __shared__ int32_t digit_base[kRadixBins];     // records with a smaller digit
  __shared__ int32_t warp_sums[8];
  __shared__ int32_t single_digit;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  {
    if (threadIdx.x == 0) single_digit = 0;
    const int32_t mine = digit_total[threadIdx.x];
    int32_t incl = mine;
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    int32_t before = 0;
    for (int w = 0; w < warp; ++w) before += warp_sums[w];
    digit_base[threadIdx.x] = before + incl - mine;
    if ((int64_t)mine == n) single_digit = 1;
    running[threadIdx.x] = 0;
    __syncthreads();
  }
  const int from = source[pass];
  const int to = single_digit ? from : 1 - from;
  if (blockIdx.x == 0 && threadIdx.x == 0) source[pass + 1] = to;
  if (single_digit) return;
  const uint4 *src = records + (size_t)from * n;
  uint4 *dst = records + (size_t)to * n;
  const int64_t base = (int64_t)blockIdx.x * kSortTile;
  for (int round = 0; round < kSortTile / 256; ++round) {
    for (int w = 0; w < 8; ++w) warp_count[w][threadIdx.x] = 0;
    __syncthreads();
    const int64_t i = base + round * 256 + threadIdx.x;
    const bool live = i < n;
    uint4 r = make_uint4(0u, 0u, 0u, 0u);
    unsigned digit = 0;
    if (live) {
      r = src[i];
      digit = digitOf(r, pass);
    }
    // lanes of the warp with the same digit; dead lanes match only each other
    const unsigned peers = __match_any_sync(0xffffffffu, live ? digit : 0xffffffffu);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (live && rank_in_warp == 0) warp_count[warp][digit] = __popc(peers);
    __syncthreads();
    // thread d: exclusive prefix of digit d over the warps, on top of the earlier rounds
    {
      int32_t before = running[threadIdx.x];
      for (int w = 0; w < 8; ++w) {
        const int32_t c = warp_count[w][threadIdx.x];
        warp_count[w][threadIdx.x] = before;
        before += c;
      }
      running[threadIdx.x] = before;
    }
    __syncthreads();
    if (live) {
      const int64_t pos = (int64_t)digit_base[digit] + block_hist[(size_t)digit * tiles + blockIdx.x] +
                          warp_count[warp][digit] + rank_in_warp;
      dst[pos] = r;
    }
    __syncthreads();
  }
}

// ---- segments ----------------------------------------------------------------

__device__ __forceinline__ bool isHead(const uint4 *__restrict__ sorted, int64_t i, int64_t n) {
  if (i >= n) return false;
  const uint4 r = sorted[i];
  if (r.w & kInvalidBit) return false;
  if (i == 0) return true;
  const uint4 q = sorted[i - 1];
  return r.x != q.x || r.y != q.y || r.z != q.z;
}

__global__ void __launch_bounds__(256)
countHeadsKernel(const uint4 *__restrict__ records, int64_t n, const int32_t *__restrict__ source,
                 int32_t *__restrict__ chunk_count) {
  const uint4 *sorted = records + (size_t)source[kRadixPasses] * n;
  const int64_t base = (int64_t)blockIdx.x * kSortTile;
  int local = 0;
  for (int r = threadIdx.x; r < kSortTile; r += 256) local += isHead(sorted, base + r, n) ? 1 : 0;
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

// One block: exclusive prefix of the per-tile head counts in place; voxel_num = total.
__global__ void __launch_bounds__(1024)
scanHeadsKernel(int32_t *__restrict__ chunk_count, int tiles, int32_t *__restrict__ voxel_num) {
  __shared__ int32_t warp_total[32];
  __shared__ int32_t carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < tiles; base += 1024) {
    const int i = base + threadIdx.x;
    const int32_t v = i < tiles ? chunk_count[i] : 0;
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
      warp_total[threadIdx.x] = w;
    }
    __syncthreads();
    const int32_t before = carry + (threadIdx.x >= 32 ? warp_total[(threadIdx.x >> 5) - 1] : 0);
    if (i < tiles) chunk_count[i] = before + incl - v;
    __syncthreads();
    if (threadIdx.x == 0) carry += warp_total[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) *voxel_num = carry;
}

// Voxel of every sorted record; coordinates and first position of every voxel;
// seg_start[voxel_num] = number of records that have a voxel.
__global__ void __launch_bounds__(256)
numberSegmentsKernel(const uint4 *__restrict__ records, int64_t n, const int32_t *__restrict__ source,
                     const int32_t *__restrict__ chunk_offset, const int32_t *__restrict__ voxel_num,
                     int64_t voxel_rows, int32_t *__restrict__ voxel_coors, int32_t *__restrict__ point2voxel_map,
                     int32_t *__restrict__ seg_start) {
  const uint4 *sorted = records + (size_t)source[kRadixPasses] * n;
  const int64_t base = (int64_t)blockIdx.x * kSortTile;
  __shared__ int32_t warp_total[8];
  __shared__ int32_t running;
  if (threadIdx.x == 0) running = chunk_offset[blockIdx.x];
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int round = 0; round < kSortTile / 256; ++round) {
    const int64_t i = base + round * 256 + threadIdx.x;
    const bool head = isHead(sorted, i, n);
    const unsigned ballot = __ballot_sync(0xffffffffu, head);
    if (lane == 0) warp_total[warp] = __popc(ballot);
    __syncthreads();
    int32_t heads_before = running;
    for (int w = 0; w < warp; ++w) heads_before += warp_total[w];
    // heads at or before this record, minus one: the record's voxel
    const int32_t vid = heads_before + __popc(ballot & ((2u << lane) - 1u)) - 1;
    if (i < n) {
      const uint4 r = sorted[i];
      const bool valid = !(r.w & kInvalidBit);
      point2voxel_map[r.w & ~kInvalidBit] = valid ? vid : -1;
      if (head) {
        if (vid < voxel_rows) {  // outputs with fewer rows than voxels keep the first rows
          voxel_coors[(size_t)vid * 3 + 0] = (int32_t)r.x;
          voxel_coors[(size_t)vid * 3 + 1] = (int32_t)r.y;
          voxel_coors[(size_t)vid * 3 + 2] = (int32_t)r.z;
        }
        seg_start[vid] = (int32_t)i;
      }
      // the first record without a voxel (or the end of the array) closes the last voxel
      if (!valid && (i == 0 || !(sorted[i - 1].w & kInvalidBit))) seg_start[*voxel_num] = (int32_t)i;
      if (valid && i == n - 1) seg_start[*voxel_num] = (int32_t)n;
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
reduceSegmentsKernel(const float *__restrict__ feats, int c_num, const uint4 *__restrict__ records, int64_t n,
                     const int32_t *__restrict__ source, const int32_t *__restrict__ seg_start,
                     const int32_t *__restrict__ voxel_num, int64_t voxel_rows, int reduce_max,
                     float *__restrict__ voxel_feats, int32_t *__restrict__ voxel_points_count,
                     int32_t *__restrict__ voxel_coors) {
  const uint4 *sorted = records + (size_t)source[kRadixPasses] * n;
  const int32_t voxels = *voxel_num;
  const int64_t total = voxel_rows * c_num;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t v = e / c_num;
    const int c = (int)(e % c_num);
    if (v >= voxels) {
      // rows past voxel_num: the fill value of the reduction, zero counts and coordinates
      voxel_feats[e] = reduce_max ? -INFINITY : 0.0f;
      if (c == 0) {
        voxel_points_count[v] = 0;
        voxel_coors[v * 3] = voxel_coors[v * 3 + 1] = voxel_coors[v * 3 + 2] = 0;
      }
      continue;
    }
    const int32_t begin = seg_start[v], end = seg_start[v + 1];
    const int32_t count = end - begin;
    if (c == 0) voxel_points_count[v] = count;
    float acc = reduce_max ? -INFINITY : 0.0f;
    if (reduce_max) {
      for (int32_t i = begin; i < end; ++i) {
        const float x = feats[(int64_t)(sorted[i].w & ~kInvalidBit) * c_num + c];
        if (x >= acc) acc = x;
      }
    } else {
      const float divisor = (float)count;
      for (int32_t i = begin; i < end; ++i)
        acc = __fadd_rn(acc, __fdiv_rn(feats[(int64_t)(sorted[i].w & ~kInvalidBit) * c_num + c], divisor));
    }
    voxel_feats[e] = acc;
  }
}

unsigned gridFor(int64_t work, int threads) {
  int64_t b = (work + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > 148 * 32) b = 148 * 32;
  return (unsigned)b;
}

}  // namespace

PointToVoxelWorkspacePlan planPointToVoxelWorkspace(const PointToVoxelProblem &p) {
  PointToVoxelWorkspacePlan plan{};
  plan.tiles = (int32_t)((p.num_points + kSortTile - 1) / kSortTile);
  if (plan.tiles < 1) plan.tiles = 1;
  size_t off = 0;
  plan.records = off;
  off = alignUp(off + 2 * (size_t)p.num_points * sizeof(uint4), 256);
  plan.block_hist = off;
  off = alignUp(off + (size_t)kRadixBins * plan.tiles * sizeof(int32_t), 256);
  plan.source = off;
  off = alignUp(off + (32 + kRadixBins) * sizeof(int32_t), 256);
  plan.chunk_count = off;
  off = alignUp(off + (size_t)plan.tiles * sizeof(int32_t), 256);
  plan.seg_start = off;
  off = alignUp(off + ((size_t)p.num_points + 1) * sizeof(int32_t), 256);
  plan.total = off + 256;
  return plan;
}

cudaError_t launchDynamicPointToVoxelForward(const PointToVoxelProblem &p, const PointToVoxelWorkspacePlan &plan,
                                             const float *feats, int32_t *coors, void *workspace,
                                             float *voxel_feats, int32_t *voxel_coors, int32_t *point2voxel_map,
                                             int32_t *voxel_points_count, int32_t *voxel_num,
                                             cudaStream_t stream) {
  char *base = reinterpret_cast<char *>(alignUp(reinterpret_cast<size_t>(workspace), 256));
  uint4 *records = reinterpret_cast<uint4 *>(base + plan.records);
  int32_t *block_hist = reinterpret_cast<int32_t *>(base + plan.block_hist);
  int32_t *source = reinterpret_cast<int32_t *>(base + plan.source);
  int32_t *digit_total = source + 32;  // int32[256] after the pass table
  int32_t *chunk_count = reinterpret_cast<int32_t *>(base + plan.chunk_count);
  int32_t *seg_start = reinterpret_cast<int32_t *>(base + plan.seg_start);
  const int64_t n = p.num_points;
  {
    trace::Scope t("makeRecordsKernel", stream, 28.0 * n);
    makeRecordsKernel<<<gridFor(n, 256), 256, 0, stream>>>(coors, n, records, source);
  }
  {
    trace::Scope t("radixSortPasses", stream, 13.0 * 16.0 * n + 32.0 * n);
    for (int pass = 0; pass < kRadixPasses; ++pass) {
      histKernel<<<(unsigned)plan.tiles, 256, 0, stream>>>(records, n, pass, source, plan.tiles, block_hist);
      scanDigitRowsKernel<<<kRadixBins, 256, 0, stream>>>(block_hist, plan.tiles, digit_total);
      scatterKernel<<<(unsigned)plan.tiles, 256, 0, stream>>>(records, n, pass, source, plan.tiles, block_hist,
                                                             digit_total);
    }
  }
  {
    trace::Scope t("numberSegmentsKernels", stream, 48.0 * n);
    countHeadsKernel<<<(unsigned)plan.tiles, 256, 0, stream>>>(records, n, source, chunk_count);
    scanHeadsKernel<<<1, 1024, 0, stream>>>(chunk_count, plan.tiles, voxel_num);
    numberSegmentsKernel<<<(unsigned)plan.tiles, 256, 0, stream>>>(records, n, source, chunk_count, voxel_num,
                                                                  p.voxel_rows, voxel_coors, point2voxel_map,
                                                                  seg_start);
  }
  {
    trace::Scope t("reduceSegmentsKernel", stream, 4.0 * n * p.num_feats + 4.0 * p.voxel_rows * p.num_feats);
    reduceSegmentsKernel<<<gridFor(p.voxel_rows * p.num_feats, 256), 256, 0, stream>>>(
        feats, p.num_feats, records, n, source, seg_start, voxel_num, p.voxel_rows, p.reduce_max, voxel_feats,
        voxel_points_count, voxel_coors);
  }
  return cudaGetLastError();
}

}  // namespace dynamic_point_to_voxel
}  // namespace mluop
