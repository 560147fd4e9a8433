// Rulebook generation kernels for sm_100a.
//
// What is computed (semantics of the reference's device path,
// kernels/sparse_conv/get_indice_pairs/normal_get_indice_pairs.cpp:831-1153 and
// get_indice_pairs_block.mlu:41-466, and of its CPU path): for input voxel j at
// (b, z, y, x) and kernel offset k = (kd*KH + kh)*KW + kw, the output
// coordinate per dim is o = (i + pad - k_dim*dilation) / stride, valid when the
// division is exact and 0 <= o < out_dim.
//   default mode: the active outputs are the distinct valid linear indices
//     b*Do*Ho*Wo + (d*Ho + h)*Wo + w in ascending order; pair (j, rank).
//   submanifold mode: outputs are the inputs themselves; pair (j, j') when an
//     input j' sits at the output coordinate (largest j' wins for a repeated
//     coordinate).
//   indice_pairs[k,0,:] lists j ascending, [k,1,:] the matching output id, -1
//   from position indice_num[k] on.
//
// How: everything is exact int32 arithmetic and every result is deterministic.
//   subm     hash table lin(j) -> j  (64-bit slots, CAS insert + atomicMax so a
//            repeated coordinate keeps the largest j), then one probe per (k,j).
//   default  one occupancy bit per output cell (atomicOr), a prefix popcount
//            over the bit words gives each active cell its ascending rank, the
//            same pass decodes out_indices; one {bits, rank} load per (k,j).
//   both     the matched id of every (k,j) is staged in [K][L] order while
//            per-tile counts are taken; an exclusive scan over tiles per k
//            gives every tile its write offset; an order-preserving block
//            compaction writes the pair lists and the -1 tails, every output
//            word exactly once.
// All loops that walk the hash table are bounded by its capacity and report
// through a status word instead of spinning.
#include "kernels/sparse_conv/get_indice_pairs_kernels.h"

#include <cuda_runtime.h>

#include "core/trace.h"

namespace mluop {
namespace sparse_conv {

namespace {

constexpr unsigned long long kEmptySlot = 0xFFFFFFFFFFFFFFFFull;

__host__ __device__ inline size_t alignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

__device__ __forceinline__ uint32_t mixKey(uint32_t x) {
  x ^= x >> 16;
  x *= 0x85ebca6bu;
  x ^= x >> 13;
  x *= 0xc2b2ae35u;
  x ^= x >> 16;
  return x;
}

// Exclusive scan of one int per thread over the block; *total gets the sum.
// blockDim.x must be a multiple of 32 and at most 1024.
__device__ __forceinline__ int blockExclusiveScan(int v, int *total, int *warp_sums /* [32] shared */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += n;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const int nwarps = blockDim.x >> 5;
    int w = lane < nwarps ? warp_sums[lane] : 0;
    int wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int n = __shfl_up_sync(0xffffffffu, wi, d);
      if (lane >= d) wi += n;
    }
    warp_sums[lane] = wi - w;  // exclusive prefix of warp sums
    if (lane == 31) warp_sums[32] = wi;
  }
  __syncthreads();
  int result = incl - v + warp_sums[warp];
  *total = warp_sums[32];
  __syncthreads();  // warp_sums may be reused by the caller's next scan
  return result;
}

__device__ __forceinline__ bool rowInRange(const int4 c, const PairsGeometry &g) {
  return (unsigned)c.x < (unsigned)g.batch && (unsigned)c.y < (unsigned)g.in_space[0] &&
         (unsigned)c.z < (unsigned)g.in_space[1] && (unsigned)c.w < (unsigned)g.in_space[2];
}

// ---------------------------------------------------------------- subm hash

__global__ void __launch_bounds__(256)
hashInsertKernel(PairsGeometry g, const int4 *__restrict__ indices, unsigned long long *slots,
                 uint32_t mask, int32_t *status) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= g.L) return;
  const int4 c = indices[j];
  if (!rowInRange(c, g)) return;
  const uint32_t lin =
      (uint32_t)(((c.x * g.in_space[0] + c.y) * g.in_space[1] + c.z) * g.in_space[2] + c.w);
  const unsigned long long packed = ((unsigned long long)lin << 32) | (uint32_t)j;
  uint32_t h = mixKey(lin) & mask;
  for (uint32_t probe = 0; probe <= mask; ++probe) {
    unsigned long long cur = slots[h];
    if (cur == kEmptySlot) {
      cur = atomicCAS(&slots[h], kEmptySlot, packed);
      if (cur == kEmptySlot) return;
    }
    if ((uint32_t)(cur >> 32) == lin) {
      atomicMax(&slots[h], packed);  // same key: keep the largest row id
      return;
    }
    h = (h + 1) & mask;
  }
  atomicOr(status, kPairsErrHashFull);
}

__device__ __forceinline__ int hashLookup(const unsigned long long *__restrict__ slots, uint32_t mask,
                                          uint32_t lin, int32_t *status) {
  uint32_t h = mixKey(lin) & mask;
  for (uint32_t probe = 0; probe <= mask; ++probe) {
    const unsigned long long cur = __ldg(slots + h);
    const uint32_t key = (uint32_t)(cur >> 32);
    if (key == lin) return (int)(uint32_t)cur;
    if (key == 0xFFFFFFFFu) return -1;
    h = (h + 1) & mask;
  }
  atomicOr(status, kPairsErrHashFull);
  return -1;
}

// ------------------------------------------------------- default-mode bits

// Sets the occupancy bit of every valid output cell.
__global__ void __launch_bounds__(256)
markOutputsKernel(PairsGeometry g, const int4 *__restrict__ indices, uint2 *rank_table) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= g.L) return;
  const int4 c = indices[j];
  if (!rowInRange(c, g)) return;
  const int base_b = c.x * g.out_vol;
  for (int kd = 0; kd < g.ks[0]; ++kd) {
    const int td = c.y + g.pad[0] - kd * g.dil[0];
    if (td < 0 || td % g.stride[0]) continue;
    const int od = td / g.stride[0];
    if (od >= g.out_space[0]) continue;
    for (int kh = 0; kh < g.ks[1]; ++kh) {
      const int th = c.z + g.pad[1] - kh * g.dil[1];
      if (th < 0 || th % g.stride[1]) continue;
      const int oh = th / g.stride[1];
      if (oh >= g.out_space[1]) continue;
      for (int kw = 0; kw < g.ks[2]; ++kw) {
        const int tw = c.w + g.pad[2] - kw * g.dil[2];
        if (tw < 0 || tw % g.stride[2]) continue;
        const int ow = tw / g.stride[2];
        if (ow >= g.out_space[2]) continue;
        const uint32_t lin = (uint32_t)(base_b + (od * g.out_space[1] + oh) * g.out_space[2] + ow);
        const uint32_t bit = 1u << (lin & 31);
        uint32_t *word = &rank_table[lin >> 5].x;
        if (!(*(volatile uint32_t *)word & bit)) atomicOr(word, bit);
      }
    }
  }
}

// chunk_count[c] = set bits in words [c*1024, (c+1)*1024)
__global__ void __launch_bounds__(256)
countBitsKernel(const uint2 *__restrict__ rank_table, int64_t words, int32_t *chunk_count) {
  __shared__ int warp_sums[33];
  const int64_t w0 = (int64_t)blockIdx.x * kRankChunkWords + threadIdx.x * 4;
  int n = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (w0 + i < words) n += __popc(rank_table[w0 + i].x);
  int total;
  blockExclusiveScan(n, &total, warp_sums);
  if (threadIdx.x == 0) chunk_count[blockIdx.x] = total;
}

// In-place exclusive scan of `n` ints by one block; writes the grand total.
__global__ void __launch_bounds__(1024)
scanSingleBlockKernel(int32_t *data, int n, int32_t *total_out) {
  __shared__ int warp_sums[33];
  int running = 0;
  for (int start = 0; start < n; start += blockDim.x) {
    const int i = start + threadIdx.x;
    const int v = i < n ? data[i] : 0;
    int total;
    const int excl = blockExclusiveScan(v, &total, warp_sums);
    if (i < n) data[i] = running + excl;
    running += total;
  }
  if (threadIdx.x == 0) *total_out = running;
}

// Gives every occupancy word its exclusive rank and writes the coordinates of
// the active cells, in ascending linear order, to out_indices.
__global__ void __launch_bounds__(256)
rankAndDecodeKernel(PairsGeometry g, uint2 *rank_table, int64_t words,
                    const int32_t *__restrict__ chunk_offset, int4 *out_indices, int64_t out_rows,
                    int32_t *status) {
  __shared__ int warp_sums[33];
  const int64_t w0 = (int64_t)blockIdx.x * kRankChunkWords + threadIdx.x * 4;
  uint32_t bits[4];
  int n = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    bits[i] = (w0 + i < words) ? rank_table[w0 + i].x : 0u;
    n += __popc(bits[i]);
  }
  int total;
  int rank = blockExclusiveScan(n, &total, warp_sums) + chunk_offset[blockIdx.x];
  const int hw = g.out_space[1] * g.out_space[2];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (w0 + i >= words) break;
    rank_table[w0 + i].y = (uint32_t)rank;
    uint32_t b = bits[i];
    while (b) {
      const int bit = __ffs(b) - 1;
      b &= b - 1;
      int lin = (int)((w0 + i) * 32 + bit);
      int4 o;
      o.x = lin / g.out_vol;
      lin -= o.x * g.out_vol;
      o.y = lin / hw;
      lin -= o.y * hw;
      o.z = lin / g.out_space[2];
      o.w = lin - o.z * g.out_space[2];
      if (rank < out_rows) {
        out_indices[rank] = o;
      } else {
        atomicOr(status, kPairsErrOutIndicesSmall);
      }
      ++rank;
    }
  }
}

// out_indices rows from the active count on are -1 (the CPU path initialises
// the whole tensor to -1 before filling it).
__global__ void __launch_bounds__(256)
fillInactiveRowsKernel(int4 *out_indices, int64_t out_rows, const int32_t *n_active) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r < out_rows && r >= *n_active) out_indices[r] = make_int4(-1, -1, -1, -1);
}

// ------------------------------------------------------------ probe + count

// One thread per input voxel walks the K offsets.  match[k][j] = output id or
// -1; tile_count[k][tile] = matches of this tile at offset k.
template <bool SUBM>
__global__ void __launch_bounds__(kPairsTile)
probeCountKernel(PairsGeometry g, const int4 *__restrict__ indices,
                 const unsigned long long *__restrict__ slots, uint32_t mask,
                 const uint2 *__restrict__ rank_table, int32_t *__restrict__ match,
                 int32_t *__restrict__ tile_count, int tiles, int32_t *status) {
  extern __shared__ int s_count[];  // [K]
  for (int k = threadIdx.x; k < g.K; k += blockDim.x) s_count[k] = 0;
  __syncthreads();
  const int j = blockIdx.x * kPairsTile + threadIdx.x;
  const bool live = j < g.L;
  int4 c = make_int4(0, 0, 0, 0);
  if (live) c = indices[j];
  const bool row_ok = live && rowInRange(c, g);
  const int base_b = c.x * g.out_vol;
  const int lane = threadIdx.x & 31;
  int k = 0;
  for (int kd = 0; kd < g.ks[0]; ++kd) {
    const int td = c.y + g.pad[0] - kd * g.dil[0];
    const int od = td / g.stride[0];
    const bool vd = row_ok && td >= 0 && (td - od * g.stride[0]) == 0 && od < g.out_space[0];
    for (int kh = 0; kh < g.ks[1]; ++kh) {
      const int th = c.z + g.pad[1] - kh * g.dil[1];
      const int oh = th / g.stride[1];
      const bool vh = vd && th >= 0 && (th - oh * g.stride[1]) == 0 && oh < g.out_space[1];
      for (int kw = 0; kw < g.ks[2]; ++kw, ++k) {
        const int tw = c.w + g.pad[2] - kw * g.dil[2];
        const int ow = tw / g.stride[2];
        const bool ok = vh && tw >= 0 && (tw - ow * g.stride[2]) == 0 && ow < g.out_space[2];
        int v = -1;
        if (ok) {
          const uint32_t lin = (uint32_t)(base_b + (od * g.out_space[1] + oh) * g.out_space[2] + ow);
          if (SUBM) {
            v = hashLookup(slots, mask, lin, status);
          } else {
            const uint2 e = __ldg(rank_table + (lin >> 5));
            v = (int)(e.y + __popc(e.x & ((1u << (lin & 31)) - 1u)));
          }
        }
        if (live) match[(size_t)k * g.L + j] = v;
        const unsigned m = __ballot_sync(0xffffffffu, v >= 0);
        if (lane == 0 && m) atomicAdd(&s_count[k], __popc(m));
      }
    }
  }
  __syncthreads();
  for (int kk = threadIdx.x; kk < g.K; kk += blockDim.x)
    tile_count[(size_t)kk * tiles + blockIdx.x] = s_count[kk];
}

// Per offset k (one block each): exclusive scan of the tile counts in place,
// indice_num[k] = total.
__global__ void __launch_bounds__(1024)
scanTilesKernel(int32_t *tile_count, int tiles, int32_t *indice_num) {
  __shared__ int warp_sums[33];
  int32_t *row = tile_count + (size_t)blockIdx.x * tiles;
  int running = 0;
  for (int start = 0; start < tiles; start += blockDim.x) {
    const int i = start + threadIdx.x;
    const int v = i < tiles ? row[i] : 0;
    int total;
    const int excl = blockExclusiveScan(v, &total, warp_sums);
    if (i < tiles) row[i] = running + excl;
    running += total;
  }
  if (threadIdx.x == 0) indice_num[blockIdx.x] = running;
}

// Block (segment of kWriteSegTiles tiles, k): order-preserving compaction of each
// tile's matches into the two rows of indice_pairs[k], plus the -1 tail for the
// positions the segment covers.  Every word of indice_pairs is written exactly
// once.  A tile without a match (its count is the difference of neighbouring
// offsets) is not read at all.
constexpr int kWriteSegTiles = 8;

__global__ void __launch_bounds__(kPairsTile)
writePairsKernel(int L, const int32_t *__restrict__ match, const int32_t *__restrict__ tile_offset,
                 int tiles, const int32_t *__restrict__ indice_num, int32_t *__restrict__ indice_pairs) {
  __shared__ int warp_count[2][kPairsTile / 32];
  const int k = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int total = indice_num[k];
  const int32_t *offsets = tile_offset + (size_t)k * tiles;
  const int32_t *match_row = match + (size_t)k * L;
  int32_t *in_row = indice_pairs + (size_t)k * 2 * L;
  int32_t *out_row = in_row + L;
  int buffers_used = 0;
  for (int i = 0; i < kWriteSegTiles; ++i) {
    const int tile = blockIdx.x * kWriteSegTiles + i;
    if (tile >= tiles) break;
    const int j = tile * kPairsTile + threadIdx.x;
    const int first = offsets[tile];
    const int next = tile + 1 < tiles ? offsets[tile + 1] : total;
    if (next > first) {  // same decision in every thread of the block
      const int v = j < L ? match_row[j] : -1;
      const unsigned hits = __ballot_sync(0xffffffffu, v >= 0);
      int *counts = warp_count[buffers_used & 1];
      ++buffers_used;
      if (lane == 0) counts[warp] = __popc(hits);
      __syncthreads();
      if (v >= 0) {
        int p = first + __popc(hits & ((1u << lane) - 1u));
        for (int w = 0; w < warp; ++w) p += counts[w];
        in_row[p] = j;
        out_row[p] = v;
      }
    }
    if (j < L && j >= total) {
      in_row[j] = -1;
      out_row[j] = -1;
    }
  }
}

}  // namespace

PairsWorkspacePlan planPairsWorkspace(const PairsGeometry &g) {
  PairsWorkspacePlan p{};
  p.tiles = (g.L + kPairsTile - 1) / kPairsTile;
  size_t off = 0;
  p.status = off;
  off = alignUp(off + 64 * sizeof(int32_t), 256);
  p.match = off;
  off = alignUp(off + (size_t)g.K * g.L * sizeof(int32_t), 256);
  p.tile_count = off;
  off = alignUp(off + (size_t)g.K * p.tiles * sizeof(int32_t), 256);
  p.table = off;
  if (g.sub_m) {
    uint32_t cap = 64;
    while ((uint64_t)cap < 2ull * (uint64_t)g.L) cap <<= 1;
    p.hash_capacity = cap;
    off = alignUp(off + (size_t)cap * sizeof(unsigned long long), 256);
    p.chunk_count = off;
  } else {
    const int64_t cells = (int64_t)g.batch * g.out_vol;
    p.rank_words = (cells + 31) / 32;
    p.rank_chunks = (int32_t)((p.rank_words + kRankChunkWords - 1) / kRankChunkWords);
    off = alignUp(off + (size_t)p.rank_words * sizeof(uint2), 256);
    p.chunk_count = off;
    off = alignUp(off + (size_t)p.rank_chunks * sizeof(int32_t), 256);
  }
  p.total = off + 256;  // slack to align the caller's pointer
  return p;
}

cudaError_t launchGetIndicePairs(const PairsGeometry &g, const PairsWorkspacePlan &plan,
                                 const int32_t *indices, void *workspace, int32_t *indice_pairs,
                                 int32_t *out_indices, int64_t out_rows, int32_t *indice_num,
                                 int32_t *status_host, cudaStream_t stream) {
  char *base = reinterpret_cast<char *>(alignUp(reinterpret_cast<size_t>(workspace), 256));
  int32_t *status = reinterpret_cast<int32_t *>(base + plan.status);
  int32_t *match = reinterpret_cast<int32_t *>(base + plan.match);
  int32_t *tile_count = reinterpret_cast<int32_t *>(base + plan.tile_count);
  const int4 *rows = reinterpret_cast<const int4 *>(indices);
  const int tiles = plan.tiles;
  const size_t count_smem = (size_t)g.K * sizeof(int);
  const double L = g.L, KL = (double)g.K * g.L;
  cudaError_t err;

  if ((err = cudaMemsetAsync(status, 0, 64 * sizeof(int32_t), stream)) != cudaSuccess) return err;
  if (g.sub_m) {
    unsigned long long *slots = reinterpret_cast<unsigned long long *>(base + plan.table);
    const uint32_t mask = plan.hash_capacity - 1;
    {
      trace::Scope t("memset:hash_table", stream, 8.0 * plan.hash_capacity);
      if ((err = cudaMemsetAsync(slots, 0xFF, (size_t)plan.hash_capacity * sizeof(unsigned long long),
                                 stream)) != cudaSuccess)
        return err;
    }
    {
      trace::Scope t("hashInsertKernel", stream, 16.0 * L + 8.0 * L);
      hashInsertKernel<<<tiles, kPairsTile, 0, stream>>>(g, rows, slots, mask, status);
    }
    {
      // out_indices = indices for the first L rows, -1 beyond
      trace::Scope t("memcpy:out_indices", stream, 32.0 * L);
      const int64_t copy_rows = out_rows < g.L ? out_rows : (int64_t)g.L;
      if ((err = cudaMemcpyAsync(out_indices, indices, (size_t)copy_rows * 4 * sizeof(int32_t),
                                 cudaMemcpyDeviceToDevice, stream)) != cudaSuccess)
        return err;
      if (out_rows > g.L) {
        if ((err = cudaMemsetAsync(out_indices + (size_t)g.L * 4, 0xFF,
                                   (size_t)(out_rows - g.L) * 4 * sizeof(int32_t), stream)) != cudaSuccess)
          return err;
      }
    }
    {
      trace::Scope t("probeCountKernel<subm>", stream, 16.0 * L + 4.0 * KL);
      probeCountKernel<true><<<tiles, kPairsTile, count_smem, stream>>>(
          g, rows, slots, mask, nullptr, match, tile_count, tiles, status);
    }
  } else {
    uint2 *rank_table = reinterpret_cast<uint2 *>(base + plan.table);
    int32_t *chunk_count = reinterpret_cast<int32_t *>(base + plan.chunk_count);
    const double words = (double)plan.rank_words;
    {
      trace::Scope t("memset:rank_table", stream, 8.0 * words);
      if ((err = cudaMemsetAsync(rank_table, 0, (size_t)plan.rank_words * sizeof(uint2), stream)) !=
          cudaSuccess)
        return err;
    }
    {
      trace::Scope t("markOutputsKernel", stream, 16.0 * L);
      markOutputsKernel<<<tiles, kPairsTile, 0, stream>>>(g, rows, rank_table);
    }
    {
      trace::Scope t("countBitsKernel", stream, 8.0 * words);
      countBitsKernel<<<plan.rank_chunks, 256, 0, stream>>>(rank_table, plan.rank_words, chunk_count);
    }
    {
      trace::Scope t("scanSingleBlockKernel", stream, 8.0 * plan.rank_chunks);
      scanSingleBlockKernel<<<1, 1024, 0, stream>>>(chunk_count, plan.rank_chunks, status + 1);
    }
    {
      trace::Scope t("rankAndDecodeKernel", stream, 16.0 * words);
      rankAndDecodeKernel<<<plan.rank_chunks, 256, 0, stream>>>(
          g, rank_table, plan.rank_words, chunk_count, reinterpret_cast<int4 *>(out_indices), out_rows,
          status);
    }
    {
      trace::Scope t("fillInactiveRowsKernel", stream, 16.0 * (double)out_rows);
      const unsigned fill_blocks = (unsigned)((out_rows + 255) / 256);
      fillInactiveRowsKernel<<<fill_blocks, 256, 0, stream>>>(reinterpret_cast<int4 *>(out_indices),
                                                             out_rows, status + 1);
    }
    {
      trace::Scope t("probeCountKernel<default>", stream, 16.0 * L + 4.0 * KL);
      probeCountKernel<false><<<tiles, kPairsTile, count_smem, stream>>>(
          g, rows, nullptr, 0, rank_table, match, tile_count, tiles, status);
    }
  }
  {
    trace::Scope t("scanTilesKernel", stream, 8.0 * g.K * tiles);
    scanTilesKernel<<<g.K, 1024, 0, stream>>>(tile_count, tiles, indice_num);
  }
  {
    trace::Scope t("writePairsKernel", stream, 12.0 * KL);
    const unsigned segments = (unsigned)((tiles + kWriteSegTiles - 1) / kWriteSegTiles);
    writePairsKernel<<<dim3(segments, g.K), kPairsTile, 0, stream>>>(g.L, match, tile_count, tiles, indice_num,
                                                                    indice_pairs);
  }
  if ((err = cudaGetLastError()) != cudaSuccess) return err;
  return cudaMemcpyAsync(status_host, status, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, stream);
}

}  // namespace sparse_conv
}  // namespace mluop
