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
//
// Lookup structure, one of
//   rank       (default mode) one occupancy bit per output cell (atomicOr); a
//              prefix popcount over the bit words gives each active cell its
//              ascending rank and the same pass decodes out_indices; a lookup is
//              one {bits, rank} load and neighbouring cells share words.
//   hash       (submanifold, sparse grid) table lin(j) -> j in 64-bit slots, CAS
//              insert + atomicMax so a repeated coordinate keeps the largest j.
//   rank+perm  (submanifold, dense grid) the occupancy/rank table over the
//              input grid plus perm[rank] = row id (atomicMax): a miss costs one
//              shared word, a hit one more load.
//
// Pair lists, one of
//   two pass   (default) matches are staged in [K][L] order with per-tile
//              counts, an exclusive scan over tiles per offset gives the write
//              offsets, a compaction kernel writes lists and -1 tails, every
//              word of indice_pairs exactly once.
//   single pass (opt-in, kernel volume <= 32): a block takes a tile of 256 voxels by
//              ticket, keeps the tile's matches in shared memory, publishes its
//              per-offset counts and obtains its write offsets by decoupled
//              look-back over the preceding tiles' descriptors, then writes its
//              pairs in place; a second kernel writes the -1 tails.  indice_pairs
//              is written exactly once and nothing is staged in global memory.
//
// Every wait is bounded: hash probes by the table capacity, the look-back spin
// by about one second of clock; both report through a status word instead of
// spinning on.
#include "kernels/sparse_conv/get_indice_pairs_kernels.h"

#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <string>

#include "core/trace.h"

namespace mluop {
namespace sparse_conv {

namespace {

constexpr unsigned long long kEmptySlot = 0xFFFFFFFFFFFFFFFFull;
constexpr long long kLookBackCycles = 2000000000ll;  // a look-back wait gives up after about a second

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
// blockDim.x must be a multiple of 32 and at most 1024; warp_sums holds 33 ints.
__device__ __forceinline__ int blockExclusiveScan(int v, int *total, int *warp_sums) {
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

__device__ __forceinline__ int warpSum(int v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

__device__ __forceinline__ bool rowInRange(const int4 c, const PairsGeometry &g) {
  return (unsigned)c.x < (unsigned)g.batch && (unsigned)c.y < (unsigned)g.in_space[0] &&
         (unsigned)c.z < (unsigned)g.in_space[1] && (unsigned)c.w < (unsigned)g.in_space[2];
}

__device__ __forceinline__ uint32_t inputLinear(const int4 c, const PairsGeometry &g) {
  return (uint32_t)(((c.x * g.in_space[0] + c.y) * g.in_space[1] + c.z) * g.in_space[2] + c.w);
}

struct LookupTables {
  const unsigned long long *slots;  // hash
  uint32_t mask;
  const uint2 *rank_table;  // rank, rank + perm
  const int32_t *perm;      // rank + perm
};

// ---------------------------------------------------------------- hash table

__global__ void __launch_bounds__(256)
hashInsertKernel(PairsGeometry g, const int4 *__restrict__ indices, unsigned long long *slots,
                 uint32_t mask, int32_t *status) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= g.L) return;
  const int4 c = indices[j];
  if (!rowInRange(c, g)) return;
  const uint32_t lin = inputLinear(c, g);
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

// ------------------------------------------------------- occupancy-bit table

__device__ __forceinline__ void setBit(uint2 *rank_table, uint32_t lin) {
  const uint32_t bit = 1u << (lin & 31);
  uint32_t *word = &rank_table[lin >> 5].x;
  if (!(*(volatile uint32_t *)word & bit)) atomicOr(word, bit);
}

// default mode: the occupancy bit of every valid output cell
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
        setBit(rank_table, (uint32_t)(base_b + (od * g.out_space[1] + oh) * g.out_space[2] + ow));
      }
    }
  }
}

// submanifold mode: the occupancy bit of every input voxel
__global__ void __launch_bounds__(256)
markInputsKernel(PairsGeometry g, const int4 *__restrict__ indices, uint2 *rank_table) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= g.L) return;
  const int4 c = indices[j];
  if (rowInRange(c, g)) setBit(rank_table, inputLinear(c, g));
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

// Gives every occupancy word its exclusive rank; with DECODE also writes the
// coordinates of the active cells, in ascending linear order, to out_indices.
template <bool DECODE>
__global__ void __launch_bounds__(256)
rankKernel(PairsGeometry g, uint2 *rank_table, int64_t words, const int32_t *__restrict__ chunk_offset,
           int4 *out_indices, int64_t out_rows, int32_t *status) {
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
    if (!DECODE) {
      rank += __popc(bits[i]);
      continue;
    }
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

// submanifold rank + perm: perm[rank of voxel j's cell] = j (largest j wins)
__global__ void __launch_bounds__(256)
permKernel(PairsGeometry g, const int4 *__restrict__ indices, const uint2 *__restrict__ rank_table,
           int32_t *perm) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= g.L) return;
  const int4 c = indices[j];
  if (!rowInRange(c, g)) return;
  const uint32_t lin = inputLinear(c, g);
  const uint2 e = __ldg(rank_table + (lin >> 5));
  atomicMax(&perm[e.y + __popc(e.x & ((1u << (lin & 31)) - 1u))], j);
}

// out_indices rows from the active count on are -1 (the CPU path initialises
// the whole tensor to -1 before filling it).
__global__ void __launch_bounds__(256)
fillInactiveRowsKernel(int4 *out_indices, int64_t out_rows, const int32_t *n_active) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r < out_rows && r >= *n_active) out_indices[r] = make_int4(-1, -1, -1, -1);
}

// ------------------------------------------------------------------- lookups

template <int LOOKUP>
__device__ __forceinline__ int lookupOutput(const LookupTables &t, uint32_t lin, int32_t *status) {
  if (LOOKUP == kLookupHash) return hashLookup(t.slots, t.mask, lin, status);
  const uint2 e = __ldg(t.rank_table + (lin >> 5));
  const uint32_t bit = lin & 31;
  if (LOOKUP == kLookupRank) return (int)(e.y + __popc(e.x & ((1u << bit) - 1u)));  // always occupied
  if (!((e.x >> bit) & 1u)) return -1;
  return __ldg(t.perm + e.y + __popc(e.x & ((1u << bit) - 1u)));
}

// t / stride when the division is exact (t >= 0): shift for power-of-two strides.
__device__ __forceinline__ bool exactDivide(int t, int stride, int shift, int *q) {
  if (shift >= 0) {
    *q = t >> shift;
    return (t & (stride - 1)) == 0;
  }
  *q = t / stride;
  return t - *q * stride == 0;
}

// Walks the K offsets of one voxel; emit(k, output id or -1) is called for every k in order.
template <int LOOKUP, typename Emit>
__device__ __forceinline__ void walkOffsets(const PairsGeometry &g, const LookupTables &tables, const int4 c,
                                            bool row_ok, int32_t *status, Emit emit) {
  const int base_b = c.x * g.out_vol;
  int k = 0;
  for (int kd = 0; kd < g.ks[0]; ++kd) {
    const int td = c.y + g.pad[0] - kd * g.dil[0];
    int od;
    const bool vd = exactDivide(td, g.stride[0], g.stride_shift[0], &od) && row_ok && td >= 0 && od < g.out_space[0];
    for (int kh = 0; kh < g.ks[1]; ++kh) {
      const int th = c.z + g.pad[1] - kh * g.dil[1];
      int oh;
      const bool vh = exactDivide(th, g.stride[1], g.stride_shift[1], &oh) && vd && th >= 0 && oh < g.out_space[1];
      const int base_row = base_b + (od * g.out_space[1] + oh) * g.out_space[2];
      for (int kw = 0; kw < g.ks[2]; ++kw, ++k) {
        const int tw = c.w + g.pad[2] - kw * g.dil[2];
        int ow;
        const bool ok = exactDivide(tw, g.stride[2], g.stride_shift[2], &ow) && vh && tw >= 0 && ow < g.out_space[2];
        int v = -1;
        if (ok) v = lookupOutput<LOOKUP>(tables, (uint32_t)(base_row + ow), status);
        emit(k, v);
      }
    }
  }
}

// ------------------------------------------------------------ single pass

constexpr uint32_t kStateAggregate = 1u << 30;  // the tile's own count is known
constexpr uint32_t kStatePrefix = 2u << 30;     // the inclusive count up to this tile is known
constexpr uint32_t kStateValue = (1u << 30) - 1u;
constexpr int kTileWarps = kPairsTile / 32;

// One block per tile of 256 voxels (tiles are handed out by ticket so that every
// tile a block waits for is already running or done).
//   1. probe: match[k][thread] and per-warp counts in shared memory
//   2. per offset k (warps share the offsets): publish the tile's count, look
//      back over earlier tiles until a published prefix is met, publish the
//      inclusive prefix; the last tile writes indice_num
//   3. write the tile's pairs at offset + rank inside the tile, ascending j
template <int LOOKUP>
__global__ void __launch_bounds__(kPairsTile)
probeWriteKernel(PairsGeometry g, const int4 *__restrict__ indices, LookupTables tables, uint32_t *tile_state,
                 int tiles, int32_t *__restrict__ indice_pairs, int32_t *__restrict__ indice_num,
                 int32_t *status) {
  extern __shared__ int smem_i[];
  int *match_s = smem_i;                            // [K][256]
  int *warp_count_s = match_s + g.K * kPairsTile;    // [K][8]
  int *offset_s = warp_count_s + g.K * kTileWarps;   // [K]
  __shared__ int tile_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) tile_s = atomicAdd(status + 2, 1);
  __syncthreads();
  const int tile = tile_s;
  const int j = tile * kPairsTile + threadIdx.x;
  const bool live = j < g.L;
  int4 c = make_int4(0, 0, 0, 0);
  if (live) c = indices[j];
  walkOffsets<LOOKUP>(g, tables, c, live && rowInRange(c, g), status, [&](int k, int v) {
    match_s[k * kPairsTile + threadIdx.x] = v;
    const unsigned hits = __ballot_sync(0xffffffffu, v >= 0);
    if (lane == 0) warp_count_s[k * kTileWarps + warp] = __popc(hits);
  });
  __syncthreads();

  for (int k = warp; k < g.K; k += kTileWarps) {
    const int mine = warpSum(lane < kTileWarps ? warp_count_s[k * kTileWarps + lane] : 0);
    volatile uint32_t *state = tile_state + (size_t)k * tiles;
    int before = 0;
    if (tile > 0) {
      if (lane == 0) state[tile] = kStateAggregate | (uint32_t)mine;
      int pos = tile - 1;  // the window covers tiles pos, pos-1, ..., pos-31
      const long long t0 = clock64();
      for (;;) {
        const int idx = pos - lane;
        uint32_t w = 2u << 30;  // before tile 0: prefix 0
        if (idx >= 0) w = state[idx];
        const unsigned prefix_lanes = __ballot_sync(0xffffffffu, (w >> 30) == 2u);
        const int first = prefix_lanes ? __ffs(prefix_lanes) - 1 : 31;
        const unsigned needed = first == 31 ? 0xffffffffu : ((2u << first) - 1u);
        const unsigned empty_lanes = __ballot_sync(0xffffffffu, (w >> 30) == 0u);
        if (empty_lanes & needed) {  // a tile in the window has not published yet
          if (clock64() - t0 > kLookBackCycles) {
            if (lane == 0) atomicOr(status, kPairsErrLookBack);
            break;
          }
          continue;
        }
        before += warpSum(lane <= first ? (int)(w & kStateValue) : 0);
        if (prefix_lanes) break;
        pos -= 32;
      }
    }
    if (lane == 0) {
      state[tile] = kStatePrefix | (uint32_t)(before + mine);
      offset_s[k] = before;
      if (tile == tiles - 1) indice_num[k] = before + mine;
    }
  }
  __syncthreads();

  for (int k = 0; k < g.K; ++k) {
    const int v = match_s[k * kPairsTile + threadIdx.x];
    const unsigned hits = __ballot_sync(0xffffffffu, v >= 0);
    if (v >= 0) {
      int p = offset_s[k] + __popc(hits & ((1u << lane) - 1u));
      for (int w = 0; w < warp; ++w) p += warp_count_s[k * kTileWarps + w];
      int32_t *in_row = indice_pairs + (size_t)k * 2 * g.L;
      in_row[p] = j;
      in_row[g.L + p] = v;
    }
  }
}

// -1 from position indice_num[k] on, both rows of every offset.
__global__ void __launch_bounds__(256)
fillTailsKernel(int L, const int32_t *__restrict__ indice_num, int32_t *__restrict__ indice_pairs) {
  const int k = blockIdx.y;
  const int first = indice_num[k];
  const int base = blockIdx.x * 2048;
  if (base + 2048 <= first) return;
  int32_t *in_row = indice_pairs + (size_t)k * 2 * L;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int p = base + i * 256 + threadIdx.x;
    if (p >= first && p < L) {
      in_row[p] = -1;
      in_row[L + p] = -1;
    }
  }
}

// ---------------------------------------------------------------- two pass

// match[k][j] = output id or -1; tile_count[k][tile] = matches of this tile at offset k.
template <int LOOKUP>
__global__ void __launch_bounds__(kPairsTile)
probeCountKernel(PairsGeometry g, const int4 *__restrict__ indices, LookupTables tables,
                 int32_t *__restrict__ match, int32_t *__restrict__ tile_count, int tiles, int32_t *status) {
  // match rows are tiles*256 entries long: every thread of every tile stores, and
  // the compaction kernel can read them 16 bytes at a time
  extern __shared__ int s_count[];  // [K]
  for (int k = threadIdx.x; k < g.K; k += blockDim.x) s_count[k] = 0;
  __syncthreads();
  const int j = blockIdx.x * kPairsTile + threadIdx.x;
  const bool live = j < g.L;
  int4 c = make_int4(0, 0, 0, 0);
  if (live) c = indices[j];
  const int lane = threadIdx.x & 31;
  int32_t *match_col = match + j;
  const size_t row_stride = (size_t)tiles * kPairsTile;
  walkOffsets<LOOKUP>(g, tables, c, live && rowInRange(c, g), status, [&](int k, int v) {
    *match_col = v;
    match_col += row_stride;
    const unsigned m = __ballot_sync(0xffffffffu, v >= 0);
    if (lane == 0 && m) atomicAdd(&s_count[k], __popc(m));
  });
  __syncthreads();
  for (int kk = threadIdx.x; kk < g.K; kk += blockDim.x)
    tile_count[(size_t)kk * tiles + blockIdx.x] = s_count[kk];
}

// Per offset k (one block each): exclusive scan of the tile counts in place,
// indice_num[k] = counts[k] = total.
__global__ void __launch_bounds__(1024)
scanTilesKernel(int32_t *tile_count, int tiles, int32_t *indice_num, int32_t *counts) {
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
  if (threadIdx.x == 0) {
    // The caller's indice_num may be pinned host memory (it wants the counts on the
    // host anyway); later kernels read the copy that stays in the workspace.
    indice_num[blockIdx.x] = running;
    counts[blockIdx.x] = running;
  }
}

// Block (segment of 8 tiles = 2048 positions, k): order-preserving compaction of
// the segment's matches into the two rows of indice_pairs[k], plus the -1 tail
// for the positions the segment covers.  Every word of indice_pairs is written
// exactly once.  A thread compacts four consecutive entries (one 16-byte load);
// half a segment without a match (its count is the difference of neighbouring
// tile offsets) is not read at all.
constexpr int kWriteSegTiles = 8;
constexpr int kWriteHalfTiles = 4;  // tiles covered by one 256-thread x 4-entry sweep

__global__ void __launch_bounds__(kPairsTile)
writePairsKernel(int L, const int32_t *__restrict__ match, const int32_t *__restrict__ tile_offset,
                 int tiles, const int32_t *__restrict__ indice_num, int32_t *__restrict__ indice_pairs) {
  __shared__ int warp_total[2][kTileWarps];
  const int k = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int total = indice_num[k];
  const size_t row_stride = (size_t)tiles * kPairsTile;
  const int32_t *offsets = tile_offset + (size_t)k * tiles;
  const int32_t *match_row = match + (size_t)k * row_stride;
  int32_t *in_row = indice_pairs + (size_t)k * 2 * L;
  int32_t *out_row = in_row + L;
  int buffers_used = 0;
#pragma unroll 1
  for (int half = 0; half < kWriteSegTiles / kWriteHalfTiles; ++half) {
    const int tile0 = blockIdx.x * kWriteSegTiles + half * kWriteHalfTiles;
    if (tile0 >= tiles) break;
    const int j0 = tile0 * kPairsTile;
    const int tile_end = min(tile0 + kWriteHalfTiles, tiles);
    const int first = offsets[tile0];
    const int next = tile_end < tiles ? offsets[tile_end] : total;
    if (next > first) {  // same decision in every thread of the block
      const int jt = j0 + 4 * threadIdx.x;
      int4 v = make_int4(-1, -1, -1, -1);
      if ((size_t)jt < row_stride) v = *reinterpret_cast<const int4 *>(match_row + jt);
      const int mine = (v.x >= 0) + (v.y >= 0) + (v.z >= 0) + (v.w >= 0);
      int incl = mine;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
      }
      int *totals = warp_total[buffers_used & 1];
      ++buffers_used;
      if (lane == 31) totals[warp] = incl;
      __syncthreads();
      int p = first + incl - mine;
      for (int w = 0; w < warp; ++w) p += totals[w];
      if (v.x >= 0) { in_row[p] = jt; out_row[p] = v.x; ++p; }
      if (v.y >= 0) { in_row[p] = jt + 1; out_row[p] = v.y; ++p; }
      if (v.z >= 0) { in_row[p] = jt + 2; out_row[p] = v.z; ++p; }
      if (v.w >= 0) { in_row[p] = jt + 3; out_row[p] = v.w; }
    }
#pragma unroll
    for (int i = 0; i < kWriteHalfTiles; ++i) {
      const int j = j0 + i * kPairsTile + threadIdx.x;
      if (j < L && j >= total) {
        in_row[j] = -1;
        out_row[j] = -1;
      }
    }
  }
}

std::string envChoice(const char *name) {
  const char *v = std::getenv(name);
  return v ? std::string(v) : std::string();
}

}  // namespace

PairsWorkspacePlan planPairsWorkspace(const PairsGeometry &g) {
  // MLUOP_B200_PAIRS_LOOKUP=hash|rank overrides the automatic choice of the
  // submanifold lookup structure; MLUOP_B200_PAIRS_PATH=fused selects the
  // single-pass pair-list path (both are cross-checked by the tests).
  static const std::string lookup_env = envChoice("MLUOP_B200_PAIRS_LOOKUP");
  static const std::string path_env = envChoice("MLUOP_B200_PAIRS_PATH");
  PairsWorkspacePlan p{};
  p.tiles = (g.L + kPairsTile - 1) / kPairsTile;
  const int64_t cells = (int64_t)g.batch * g.out_vol;  // submanifold: input space == output space
  if (!g.sub_m) {
    p.lookup = kLookupRank;
  } else if (lookup_env == "hash") {
    p.lookup = kLookupHash;
  } else if (lookup_env == "rank") {
    p.lookup = kLookupRankPerm;
  } else {
    p.lookup = cells <= kDenseCellsPerVoxel * (int64_t)g.L ? kLookupRankPerm : kLookupHash;
  }
  // The single-pass path is opt-in: on B200 about a thousand tiles finish their
  // probes in lockstep, so the look-back chain (32 tiles per L2 round trip, per
  // offset) costs more than the staged matches of the two-pass path save.
  p.fused = (g.K <= kFusedMaxOffsets && path_env == "fused") ? 1 : 0;
  size_t off = 0;
  p.status = off;
  off = alignUp(off + 64 * sizeof(int32_t), 256);
  p.counts = off;
  off = alignUp(off + (size_t)g.K * sizeof(int32_t), 256);
  p.tile_state = off;
  p.match = off;
  p.tile_count = off;
  if (p.fused) {
    off = alignUp(off + (size_t)g.K * p.tiles * sizeof(uint32_t), 256);
  } else {
    off = alignUp(off + (size_t)g.K * p.tiles * kPairsTile * sizeof(int32_t), 256);
    p.tile_count = off;
    off = alignUp(off + (size_t)g.K * p.tiles * sizeof(int32_t), 256);
  }
  p.table = off;
  p.chunk_count = off;
  p.perm = off;
  // Test hook: MLUOP_B200_TEST_HASH_CAPACITY=<n> makes submanifold rulebooks use the hash
  // table with at most n slots (rounded down to a power of two, at least 64), so that the
  // "table full" error path can be exercised: probes are bounded by the capacity, the
  // kernels record kPairsErrHashFull and carry on.
  uint32_t cap_limit = 0;
  if (g.sub_m) {
    if (const char *v = std::getenv("MLUOP_B200_TEST_HASH_CAPACITY")) cap_limit = (uint32_t)std::strtoul(v, nullptr, 10);
    if (cap_limit) p.lookup = kLookupHash;
  }
  if (p.lookup == kLookupHash) {
    uint32_t cap = 64;
    while ((uint64_t)cap < 2ull * (uint64_t)g.L && (cap_limit == 0 || cap * 2 <= cap_limit)) cap <<= 1;
    p.hash_capacity = cap;
    off = alignUp(off + (size_t)cap * sizeof(unsigned long long), 256);
  } else {
    p.rank_words = (cells + 31) / 32;
    p.rank_chunks = (int32_t)((p.rank_words + kRankChunkWords - 1) / kRankChunkWords);
    off = alignUp(off + (size_t)p.rank_words * sizeof(uint2), 256);
    p.chunk_count = off;
    off = alignUp(off + (size_t)p.rank_chunks * sizeof(int32_t), 256);
    if (p.lookup == kLookupRankPerm) {
      p.perm = off;
      off = alignUp(off + (size_t)g.L * sizeof(int32_t), 256);
    }
  }
  p.total = off + 256;  // slack to align the caller's pointer
  return p;
}

namespace {

template <int LOOKUP>
void launchPairLists(const PairsGeometry &g, const PairsWorkspacePlan &plan, const int4 *rows,
                     const LookupTables &tables, char *base, int32_t *indice_pairs, int32_t *indice_num,
                     int32_t *status, cudaStream_t stream) {
  const int tiles = plan.tiles;
  const double L = g.L, KL = (double)g.K * g.L;
  static const char *names_fused[] = {"probeWriteKernel<rank>", "probeWriteKernel<hash>",
                                      "probeWriteKernel<rank+perm>"};
  static const char *names_count[] = {"probeCountKernel<rank>", "probeCountKernel<hash>",
                                      "probeCountKernel<rank+perm>"};
  if (plan.fused) {
    uint32_t *tile_state = reinterpret_cast<uint32_t *>(base + plan.tile_state);
    {
      trace::Scope t("memset:tile_state", stream, 4.0 * g.K * tiles);
      cudaMemsetAsync(tile_state, 0, (size_t)g.K * tiles * sizeof(uint32_t), stream);
    }
    {
      // per voxel: its coordinates; the matched pairs are written by this kernel
      trace::Scope t(names_fused[LOOKUP], stream, 16.0 * L);
      const size_t smem = (size_t)g.K * (kPairsTile + kTileWarps + 1) * sizeof(int);
      probeWriteKernel<LOOKUP><<<tiles, kPairsTile, smem, stream>>>(g, rows, tables, tile_state, tiles,
                                                                    indice_pairs, indice_num, status);
    }
    {
      trace::Scope t("fillTailsKernel", stream, 8.0 * KL);
      fillTailsKernel<<<dim3((unsigned)((g.L + 2047) / 2048), g.K), 256, 0, stream>>>(g.L, indice_num,
                                                                                     indice_pairs);
    }
    return;
  }
  int32_t *match = reinterpret_cast<int32_t *>(base + plan.match);
  int32_t *tile_count = reinterpret_cast<int32_t *>(base + plan.tile_count);
  int32_t *counts = reinterpret_cast<int32_t *>(base + plan.counts);
  {
    trace::Scope t(names_count[LOOKUP], stream, 16.0 * L + 4.0 * KL);
    probeCountKernel<LOOKUP><<<tiles, kPairsTile, (size_t)g.K * sizeof(int), stream>>>(
        g, rows, tables, match, tile_count, tiles, status);
  }
  {
    trace::Scope t("scanTilesKernel", stream, 8.0 * g.K * tiles);
    scanTilesKernel<<<g.K, 1024, 0, stream>>>(tile_count, tiles, indice_num, counts);
  }
  {
    trace::Scope t("writePairsKernel", stream, 12.0 * KL);
    const unsigned segments = (unsigned)((tiles + kWriteSegTiles - 1) / kWriteSegTiles);
    writePairsKernel<<<dim3(segments, g.K), kPairsTile, 0, stream>>>(g.L, match, tile_count, tiles, counts,
                                                                    indice_pairs);
  }
}

__global__ void publishStatusKernel(const int32_t *__restrict__ status, volatile int32_t *status_host) {
  const int32_t bits = status[0];
  status_host[0] = bits;
  status_host[1] = status[1];
  if (bits) status_host[2] |= bits;  // sticky: reported and cleared by the next entry point on the handle
  __threadfence_system();
}

}  // namespace

cudaError_t launchGetIndicePairs(const PairsGeometry &g, const PairsWorkspacePlan &plan,
                                 const int32_t *indices, void *workspace, int32_t *indice_pairs,
                                 int32_t *out_indices, int64_t out_rows, int32_t *indice_num,
                                 int32_t *status_host, cudaStream_t stream) {
  char *base = reinterpret_cast<char *>(alignUp(reinterpret_cast<size_t>(workspace), 256));
  int32_t *status = reinterpret_cast<int32_t *>(base + plan.status);
  const int4 *rows = reinterpret_cast<const int4 *>(indices);
  const int tiles = plan.tiles;
  const double L = g.L;
  LookupTables tables{};
  cudaError_t err;

  if ((err = cudaMemsetAsync(status, 0, 64 * sizeof(int32_t), stream)) != cudaSuccess) return err;

  if (plan.lookup == kLookupHash) {
    unsigned long long *slots = reinterpret_cast<unsigned long long *>(base + plan.table);
    tables.slots = slots;
    tables.mask = plan.hash_capacity - 1;
    {
      trace::Scope t("memset:hash_table", stream, 8.0 * plan.hash_capacity);
      if ((err = cudaMemsetAsync(slots, 0xFF, (size_t)plan.hash_capacity * sizeof(unsigned long long),
                                 stream)) != cudaSuccess)
        return err;
    }
    trace::Scope t("hashInsertKernel", stream, 16.0 * L + 8.0 * L);
    hashInsertKernel<<<tiles, kPairsTile, 0, stream>>>(g, rows, slots, tables.mask, status);
  } else {
    uint2 *rank_table = reinterpret_cast<uint2 *>(base + plan.table);
    int32_t *chunk_count = reinterpret_cast<int32_t *>(base + plan.chunk_count);
    const double words = (double)plan.rank_words;
    tables.rank_table = rank_table;
    {
      trace::Scope t("memset:rank_table", stream, 8.0 * words);
      if ((err = cudaMemsetAsync(rank_table, 0, (size_t)plan.rank_words * sizeof(uint2), stream)) !=
          cudaSuccess)
        return err;
    }
    if (g.sub_m) {
      trace::Scope t("markInputsKernel", stream, 16.0 * L);
      markInputsKernel<<<tiles, kPairsTile, 0, stream>>>(g, rows, rank_table);
    } else {
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
    if (g.sub_m) {
      int32_t *perm = reinterpret_cast<int32_t *>(base + plan.perm);
      tables.perm = perm;
      {
        trace::Scope t("rankKernel", stream, 16.0 * words);
        rankKernel<false><<<plan.rank_chunks, 256, 0, stream>>>(g, rank_table, plan.rank_words, chunk_count,
                                                               nullptr, 0, status);
      }
      if ((err = cudaMemsetAsync(perm, 0xFF, (size_t)g.L * sizeof(int32_t), stream)) != cudaSuccess) return err;
      trace::Scope t("permKernel", stream, 20.0 * L);
      permKernel<<<tiles, kPairsTile, 0, stream>>>(g, rows, rank_table, perm);
    } else {
      {
        trace::Scope t("rankAndDecodeKernel", stream, 16.0 * words);
        rankKernel<true><<<plan.rank_chunks, 256, 0, stream>>>(g, rank_table, plan.rank_words, chunk_count,
                                                              reinterpret_cast<int4 *>(out_indices), out_rows,
                                                              status);
      }
      trace::Scope t("fillInactiveRowsKernel", stream, 16.0 * (double)out_rows);
      const unsigned fill_blocks = (unsigned)((out_rows + 255) / 256);
      fillInactiveRowsKernel<<<fill_blocks, 256, 0, stream>>>(reinterpret_cast<int4 *>(out_indices), out_rows,
                                                             status + 1);
    }
  }

  if (g.sub_m) {
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

  switch (plan.lookup) {
    case kLookupHash:
      launchPairLists<kLookupHash>(g, plan, rows, tables, base, indice_pairs, indice_num, status, stream);
      break;
    case kLookupRankPerm:
      launchPairLists<kLookupRankPerm>(g, plan, rows, tables, base, indice_pairs, indice_num, status, stream);
      break;
    default:
      launchPairLists<kLookupRank>(g, plan, rows, tables, base, indice_pairs, indice_num, status, stream);
      break;
  }
  if ((err = cudaGetLastError()) != cudaSuccess) return err;
  // status_host is pinned, device-mapped host memory: a one-thread kernel stores the
  // two words there, so the read-back does not queue behind whatever large
  // transfers the application has on the copy engines.
  publishStatusKernel<<<1, 1, 0, stream>>>(status, status_host);
  return cudaGetLastError();
}

}  // namespace sparse_conv
}  // namespace mluop
