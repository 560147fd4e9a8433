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
// One cudaMemsetAsync clears all scratch that must start at zero (status words,
// scan descriptors, lookup table), then
//
//   lookup structure, one of
//     rank       (default mode) markOutputsKernel sets one occupancy bit per valid
//                output cell; rankScanKernel turns the bit words into {bits,
//                exclusive rank} in one pass (chained scan over chunks of words
//                with decoupled look-back) and decodes out_indices in ascending
//                order.
//     hash       (submanifold, sparse grid) hashInsertKernel: lin(j) -> j in
//                64-bit slots, CAS insert + atomicMax so that a repeated coordinate
//                keeps the largest j.
//     rank+perm  (submanifold, dense grid) the same occupancy/rank table over the
//                input grid plus permKernel: perm[rank] = row id.
//
//   pair lists, one of
//     single pass (kernel volume <= 32) pairListsKernel: a block takes a tile of
//                256 voxels by ticket, probes its K x 256 slots (3x3x3 kernels with
//                stride 1 or 2 run a fully unrolled walk that keeps the matches
//                in registers), publishes its K counts as one descriptor and
//                obtains its K write offsets by a two-level look-back (tiles of
//                its group of 32, then group descriptors), and writes its pairs
//                in place.  Nothing is staged in global memory and one chain of
//                K-wide descriptors serves all offsets.
//     two pass   (larger kernel volumes) matches staged in [K][L] order with
//                per-tile counts, a scan per offset, a compaction kernel.
//   finishPairsKernel writes the -1 tails of indice_pairs, the -1 rows of
//   out_indices past the active count, and hands {error bits, active count} to
//   the host.
//
// Every wait is bounded: hash probes by the table capacity, look-back spins by
// about 0.2 s of clock, with the give-up decision taken by the whole warp;
// both report through the status word (and the handle's sticky host word)
// instead of spinning on.
#include "kernels/sparse_conv/get_indice_pairs_kernels.h"

#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <string>

#include "core/trace.h"

namespace mluop {
namespace sparse_conv {

namespace {

constexpr long long kLookBackCycles = 400000000ll;  // a look-back wait gives up after about 0.2 s

// status words (int32) at the start of the workspace
constexpr int kStatusErrors = 0;       // error bits
constexpr int kStatusActive = 1;       // number of active outputs (default mode)
constexpr int kStatusTileTicket = 2;   // tiles handed out by pairListsKernel
constexpr int kStatusChunkTicket = 3;  // chunks handed out by rankScanKernel

// look-back descriptor words: 2-bit state, 30-bit value
constexpr uint32_t kFlagAggregate = 1u << 30;  // value = this unit's own count
constexpr uint32_t kFlagPrefix = 2u << 30;     // value = inclusive count up to and including this unit
constexpr uint32_t kValueMask = (1u << 30) - 1u;
constexpr int kGroupTiles = 32;  // tiles per group of the two-level look-back
constexpr int kDescWords = 32;   // words per K-wide descriptor (kernel volumes up to 32)
static_assert(kFusedMaxOffsets <= kDescWords, "one descriptor word per kernel offset");

__host__ __device__ inline size_t alignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct ErrorSink {
  int32_t *status;  // status words in the workspace
  int32_t *sticky;  // device-visible host word of the handle, or null
};

__device__ __forceinline__ void raiseError(const ErrorSink &sink, int code) {
  atomicOr(sink.status + kStatusErrors, code);
  if (sink.sticky) {
    volatile int32_t *w = sink.sticky;
    *w = *w | code;
    __threadfence_system();
  }
}

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
  const unsigned long long *slots;  // hash: (lin + 1) << 32 | row id, 0 = empty
  uint32_t mask;
  const uint2 *rank_table;  // rank, rank + perm: {occupancy bits, exclusive rank}
  const int32_t *perm;      // rank + perm: row id + 1 of the r-th occupied cell
};

// ---------------------------------------------------------------- hash table

__global__ void __launch_bounds__(256)
hashInsertKernel(PairsGeometry g, const int4 *__restrict__ indices, unsigned long long *slots,
                 uint32_t mask, ErrorSink sink) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= g.L) return;
  const int4 c = indices[j];
  if (!rowInRange(c, g)) return;
  const uint32_t key = inputLinear(c, g) + 1u;
  const unsigned long long packed = ((unsigned long long)key << 32) | (uint32_t)j;
  uint32_t h = mixKey(key) & mask;
  for (uint32_t probe = 0; probe <= mask; ++probe) {
    unsigned long long cur = slots[h];
    if (cur == 0ull) {
      cur = atomicCAS(&slots[h], 0ull, packed);
      if (cur == 0ull) return;
    }
    if ((uint32_t)(cur >> 32) == key) {
      atomicMax(&slots[h], packed);  // same key: keep the largest row id
      return;
    }
    h = (h + 1) & mask;
  }
  raiseError(sink, kPairsErrHashFull);
}

__device__ __forceinline__ int hashLookup(const unsigned long long *__restrict__ slots, uint32_t mask,
                                          uint32_t lin, const ErrorSink &sink) {
  const uint32_t want = lin + 1u;
  uint32_t h = mixKey(want) & mask;
  for (uint32_t probe = 0; probe <= mask; ++probe) {
    const unsigned long long cur = __ldg(slots + h);
    const uint32_t key = (uint32_t)(cur >> 32);
    if (key == want) return (int)(uint32_t)cur;
    if (key == 0u) return -1;
    h = (h + 1) & mask;
  }
  raiseError(sink, kPairsErrHashFull);
  return -1;
}

// ------------------------------------------------------- occupancy-bit table

// A reduction: nothing is returned, so the thread does not wait for it (reading the
// word first to spare the atomic made every bit a dependent round trip).
__device__ __forceinline__ void setBit(uint2 *rank_table, uint32_t lin) {
  atomicOr(&rank_table[lin >> 5].x, 1u << (lin & 31));
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

// The same for a 3x3x3 kernel with stride 2 and dilation 1: per dimension only the
// offsets with the parity of (i + pad) can be valid, at most two of the three.
__global__ void __launch_bounds__(256)
markOutputsCube3Stride2Kernel(PairsGeometry g, const int4 *__restrict__ indices, uint2 *rank_table) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= g.L) return;
  const int4 c = indices[j];
  if (!rowInRange(c, g)) return;
  int o[3][2];
  bool ok[3][2];
  const int i3[3] = {c.y, c.z, c.w};
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    const int t0 = i3[d] + g.pad[d];
    const int k0 = t0 & 1;  // the smallest offset with t = t0 - k even
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      const int kk = k0 + 2 * a, t = t0 - kk;
      o[d][a] = t >> 1;
      ok[d][a] = kk < 3 && t >= 0 && o[d][a] < g.out_space[d];
    }
  }
  const int base_b = c.x * g.out_vol;
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int b = 0; b < 2; ++b)
#pragma unroll
      for (int e = 0; e < 2; ++e)
        if (ok[0][a] && ok[1][b] && ok[2][e])
          setBit(rank_table, (uint32_t)(base_b + (o[0][a] * g.out_space[1] + o[1][b]) * g.out_space[2] + o[2][e]));
}

// submanifold mode: the occupancy bit of every input voxel
__global__ void __launch_bounds__(256)
markInputsKernel(PairsGeometry g, const int4 *__restrict__ indices, uint2 *rank_table) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= g.L) return;
  const int4 c = indices[j];
  if (rowInRange(c, g)) setBit(rank_table, inputLinear(c, g));
}

// Exclusive prefix of `mine` over the units before `unit` by decoupled look-back
// over one-word descriptors; called by one whole warp, every lane gets the result.
// The unit's own aggregate is published first and its inclusive prefix last.
// Returns -1 when a wait ran out (decided by the whole warp).
__device__ __forceinline__ int lookBackOneWord(uint32_t *desc, int unit, int mine) {
  const int lane = threadIdx.x & 31;
  volatile uint32_t *state = desc;
  int before = 0;
  if (unit > 0) {
    if (lane == 0) state[unit] = kFlagAggregate | (uint32_t)mine;
    int pos = unit - 1;  // the window covers units pos, pos-1, ..., pos-31
    const long long t0 = clock64();
    for (;;) {
      const int idx = pos - lane;
      uint32_t w = kFlagPrefix;  // before unit 0: prefix 0
      if (idx >= 0) w = state[idx];
      const unsigned prefix_lanes = __ballot_sync(0xffffffffu, (w >> 30) == 2u);
      const int first = prefix_lanes ? __ffs(prefix_lanes) - 1 : 31;
      const unsigned needed = first == 31 ? 0xffffffffu : ((2u << first) - 1u);
      const unsigned empty_lanes = __ballot_sync(0xffffffffu, (w >> 30) == 0u);
      if (empty_lanes & needed) {  // a unit in the window has not published yet
        const bool late = clock64() - t0 > kLookBackCycles;
        if (__any_sync(0xffffffffu, late)) return -1;
        continue;
      }
      before += warpSum(lane <= first ? (int)(w & kValueMask) : 0);
      if (prefix_lanes) break;
      pos -= 32;
    }
  }
  if (lane == 0) state[unit] = kFlagPrefix | (uint32_t)(before + mine);
  return before;
}

// One pass over the occupancy words: chunk c = words [c*W, (c+1)*W), 8 words per
// thread.  Counts the chunk's bits, gets the count of all earlier chunks by
// look-back (chunks are handed out by ticket, so every chunk waited for is already
// running), stores each word's exclusive rank next to its bits and, with DECODE,
// writes the coordinates of the chunk's active cells to out_indices in ascending
// linear order.  The last chunk leaves the total in status[kStatusActive].
// The chunk size is chosen per call (8, 4, 2 or 1 words per thread) so that small grids
// still spread over all SMs: the decode of a chunk is serial per thread.
template <bool DECODE, int kRankWordsPerThread>
__global__ void __launch_bounds__(256)
rankScanKernel(PairsGeometry g, uint2 *rank_table, int64_t words, int chunks, uint32_t *chunk_desc,
               int4 *out_indices, int64_t out_rows, ErrorSink sink) {
  constexpr int kRankChunkWords = 256 * kRankWordsPerThread;
  __shared__ int warp_sums[33];
  __shared__ int chunk_s, before_s;
  if (threadIdx.x == 0) chunk_s = atomicAdd(sink.status + kStatusChunkTicket, 1);
  __syncthreads();
  const int chunk = chunk_s;
  const int64_t w0 = (int64_t)chunk * kRankChunkWords + threadIdx.x * kRankWordsPerThread;
  uint32_t bits[kRankWordsPerThread];
  int n = 0;
  if (kRankWordsPerThread >= 2 && w0 + kRankWordsPerThread <= words) {
    const uint4 *src = reinterpret_cast<const uint4 *>(rank_table + w0);  // two {bits, rank} entries per load
#pragma unroll
    for (int i = 0; i < kRankWordsPerThread / 2; ++i) {
      const uint4 v = src[i];
      bits[2 * i] = v.x;
      bits[2 * i + 1] = v.z;
    }
  } else {
#pragma unroll
    for (int i = 0; i < kRankWordsPerThread; ++i) bits[i] = (w0 + i < words) ? rank_table[w0 + i].x : 0u;
  }
#pragma unroll
  for (int i = 0; i < kRankWordsPerThread; ++i) n += __popc(bits[i]);
  int total;
  const int excl = blockExclusiveScan(n, &total, warp_sums);
  if (threadIdx.x < 32) {
    const int before = lookBackOneWord(chunk_desc, chunk, total);
    if (threadIdx.x == 0) {
      before_s = before < 0 ? 0 : before;
      if (before < 0) raiseError(sink, kPairsErrLookBack);
      if (chunk == chunks - 1) sink.status[kStatusActive] = before_s + total;
    }
  }
  __syncthreads();
  int rank = excl + before_s;
  const int hw = g.out_space[1] * g.out_space[2];
#pragma unroll
  for (int i = 0; i < kRankWordsPerThread; ++i) {
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
        raiseError(sink, kPairsErrOutIndicesSmall);
      }
      ++rank;
    }
  }
}

// submanifold rank + perm: perm[rank of voxel j's cell] = j + 1 (largest j wins; 0 = none)
__global__ void __launch_bounds__(256)
permKernel(PairsGeometry g, const int4 *__restrict__ indices, const uint2 *__restrict__ rank_table,
           int32_t *perm) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= g.L) return;
  const int4 c = indices[j];
  if (!rowInRange(c, g)) return;
  const uint32_t lin = inputLinear(c, g);
  const uint2 e = __ldg(rank_table + (lin >> 5));
  atomicMax(&perm[e.y + __popc(e.x & ((1u << (lin & 31)) - 1u))], j + 1);
}

// ------------------------------------------------------------------- lookups

template <int LOOKUP>
__device__ __forceinline__ int lookupOutput(const LookupTables &t, uint32_t lin, const ErrorSink &sink) {
  if (LOOKUP == kLookupHash) return hashLookup(t.slots, t.mask, lin, sink);
  const uint2 e = __ldg(t.rank_table + (lin >> 5));
  const uint32_t bit = lin & 31;
  if (LOOKUP == kLookupRank) return (int)(e.y + __popc(e.x & ((1u << bit) - 1u)));  // always occupied
  if (!((e.x >> bit) & 1u)) return -1;
  return __ldg(t.perm + e.y + __popc(e.x & ((1u << bit) - 1u))) - 1;
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
                                            bool row_ok, const ErrorSink &sink, Emit emit) {
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
        if (ok) v = lookupOutput<LOOKUP>(tables, (uint32_t)(base_row + ow), sink);
        emit(k, v);
      }
    }
  }
}

// The same walk for a 3x3x3 kernel with dilation 1 and stride SHIFT+1 in {1, 2},
// fully unrolled: the index arithmetic is hoisted per dimension, the 27 lookups
// are independent loads, and the results stay in registers.
template <int LOOKUP, int SHIFT>
__device__ __forceinline__ void walkCube3(const PairsGeometry &g, const LookupTables &tables, const int4 c,
                                          bool row_ok, const ErrorSink &sink, int (&v)[27]) {
  bool ok_d[3], ok_h[3], ok_w[3];
  int o_d[3], o_h[3], o_w[3];
#pragma unroll
  for (int kk = 0; kk < 3; ++kk) {
    const int td = c.y + g.pad[0] - kk, th = c.z + g.pad[1] - kk, tw = c.w + g.pad[2] - kk;
    o_d[kk] = td >> SHIFT;
    o_h[kk] = th >> SHIFT;
    o_w[kk] = tw >> SHIFT;
    ok_d[kk] = row_ok && td >= 0 && (td & SHIFT) == 0 && o_d[kk] < g.out_space[0];
    ok_h[kk] = th >= 0 && (th & SHIFT) == 0 && o_h[kk] < g.out_space[1];
    ok_w[kk] = tw >= 0 && (tw & SHIFT) == 0 && o_w[kk] < g.out_space[2];
  }
  const int base_b = c.x * g.out_vol;
#pragma unroll
  for (int kd = 0; kd < 3; ++kd) {
#pragma unroll
    for (int kh = 0; kh < 3; ++kh) {
      const bool ok_dh = ok_d[kd] && ok_h[kh];
      const int base_row = base_b + (o_d[kd] * g.out_space[1] + o_h[kh]) * g.out_space[2];
#pragma unroll
      for (int kw = 0; kw < 3; ++kw) {
        int r = -1;
        if (ok_dh && ok_w[kw]) r = lookupOutput<LOOKUP>(tables, (uint32_t)(base_row + o_w[kw]), sink);
        v[(kd * 3 + kh) * 3 + kw] = r;
      }
    }
  }
}

// ------------------------------------------------------------ single pass

constexpr int kTileWarps = kPairsTile / 32;

enum WalkKind { kWalkGeneric = 0, kWalkCube3Stride1 = 1, kWalkCube3Stride2 = 2 };

struct PairListScratch {
  uint32_t *tile_desc;   // [tiles][32]   aggregate of a tile per offset
  uint32_t *group_desc;  // [groups][32]  aggregate / inclusive prefix of a group of 32 tiles per offset
  uint32_t *group_sum;   // [groups][32]  running sum of the group's tile aggregates
  int32_t *group_done;   // [groups]      tiles of the group that have published
};

// Exclusive prefix of this tile's per-offset counts (lane = offset k), by one warp.
//   1. publish the tile's aggregate; add it to the group's running sum; the tile
//      that completes its group publishes the group's aggregate
//   2. sum the aggregates of the earlier tiles of the own group
//   3. walk back over the group descriptors until an inclusive prefix is met, and
//      publish the inclusive prefix of the preceding group for those that follow
// Tiles are handed out by ticket, so everything waited for is running or done,
// and nothing that is waited for waits for this tile.  Returns false when a wait
// ran out; every exit is taken by the whole warp.
__device__ __forceinline__ bool tilePrefix(const PairListScratch &s, int tile, int tiles, int mine, int *before_out) {
  constexpr unsigned kFull = 0xffffffffu;
  const int lane = threadIdx.x & 31;
  const int group = tile / kGroupTiles, first_tile = group * kGroupTiles;
  const int group_size = min(kGroupTiles, tiles - first_tile);
  volatile uint32_t *tile_desc = s.tile_desc;
  volatile uint32_t *group_desc = s.group_desc;
  tile_desc[(size_t)tile * kDescWords + lane] = kFlagAggregate | (uint32_t)mine;
  atomicAdd(&s.group_sum[(size_t)group * kDescWords + lane], (uint32_t)mine);
  __threadfence();
  __syncwarp();  // every lane's addition is ordered before lane 0's arrival count
  int arrived = 0;
  if (lane == 0) arrived = atomicAdd(&s.group_done[group], 1);
  arrived = __shfl_sync(kFull, arrived, 0);
  if (arrived == group_size - 1) {  // every tile of the group has added its counts
    __threadfence();
    const uint32_t sum = atomicAdd(&s.group_sum[(size_t)group * kDescWords + lane], 0u);
    group_desc[(size_t)group * kDescWords + lane] = kFlagAggregate | sum;
  }
  const long long t0 = clock64();
  int before = 0;
  // earlier tiles of the own group, four descriptors in flight at a time
  for (int t = first_tile; t < tile; t += 4) {
    uint32_t w[4];
    for (;;) {
      bool missing = false;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        w[u] = 1u << 30;  // past the own tile: an aggregate of zero
        if (t + u < tile) w[u] = tile_desc[(size_t)(t + u) * kDescWords + lane];
        missing |= (w[u] >> 30) == 0u;
      }
      if (!__any_sync(kFull, missing)) break;
      if (__any_sync(kFull, clock64() - t0 > kLookBackCycles)) return false;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) before += (int)(w[u] & kValueMask);
  }
  // groups before the own one; a lane is done when it has met an inclusive prefix
  int groups_before = 0;
  bool open = group > 0;
  for (int gg = group - 1; gg >= 0; --gg) {
    if (!__any_sync(kFull, open)) break;
    uint32_t w = 0u;
    for (;;) {
      if (open) w = group_desc[(size_t)gg * kDescWords + lane];
      if (!__any_sync(kFull, open && (w >> 30) == 0u)) break;
      if (__any_sync(kFull, clock64() - t0 > kLookBackCycles)) return false;
    }
    if (open) {
      groups_before += (int)(w & kValueMask);
      if ((w >> 30) == 2u) open = false;
    }
  }
  if (group > 0) group_desc[(size_t)(group - 1) * kDescWords + lane] = kFlagPrefix | (uint32_t)groups_before;
  *before_out = before + groups_before;
  return true;
}

// One block per tile of 256 voxels.
//   A. probe: the tile's K x 256 matches (registers for the unrolled 3x3x3 walks,
//      shared memory otherwise) and per-warp counts; submanifold mode also copies
//      the tile's rows of indices to out_indices, and with `table` the matches are
//      written to table[K-1-k][j] (the neighbour table of a submanifold rulebook
//      with centred padding: the input row feeding output row j at offset K-1-k),
//      -1 in the padding rows
//   B. warp 0: the tile's write offsets for all K offsets (tilePrefix); the last
//      tile writes indice_num
//   C. the tile's pairs, ascending j, at offset + rank inside the tile
// Resident blocks per SM the compiler has to leave room for.  A tile's life is a chain
// of dependent memory latencies (coordinates, lookups, look-back, stores), so the kernel
// is bound by the number of tiles in flight: 6 blocks (40 registers, a few spilled
// words) measured faster than 4 (64 registers, none).
#ifndef MLUOP_B200_PAIRS_MIN_BLOCKS
#define MLUOP_B200_PAIRS_MIN_BLOCKS 6
#endif
template <int LOOKUP, int WALK>
__global__ void __launch_bounds__(kPairsTile, MLUOP_B200_PAIRS_MIN_BLOCKS)
pairListsKernel(PairsGeometry g, const int4 *__restrict__ indices, LookupTables tables, PairListScratch scratch,
                int tiles, int32_t *__restrict__ indice_pairs, int32_t *__restrict__ indice_num,
                int32_t *__restrict__ counts, int4 *__restrict__ out_indices, int64_t out_rows,
                int32_t *__restrict__ table, int64_t table_stride, ErrorSink sink) {
  extern __shared__ int match_s[];  // generic walk: [K][256]
  __shared__ int warp_base_s[kDescWords][kTileWarps];
  __shared__ int offset_s[kDescWords];
  __shared__ int tile_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) tile_s = atomicAdd(sink.status + kStatusTileTicket, 1);
  __syncthreads();
  const int tile = tile_s;
  const int j = tile * kPairsTile + threadIdx.x;
  const bool live = j < g.L;
  int4 c = make_int4(0, 0, 0, 0);
  if (live) c = indices[j];
  const bool row_ok = live && rowInRange(c, g);
  if (g.sub_m && live && j < out_rows) out_indices[j] = c;

  int v[27];
  if (WALK == kWalkGeneric) {
    walkOffsets<LOOKUP>(g, tables, c, row_ok, sink, [&](int k, int r) {
      match_s[k * kPairsTile + threadIdx.x] = r;
      const unsigned hits = __ballot_sync(0xffffffffu, r >= 0);
      if (lane == 0) warp_base_s[k][warp] = __popc(hits);
    });
  } else {
    walkCube3<LOOKUP, WALK == kWalkCube3Stride2 ? 1 : 0>(g, tables, c, row_ok, sink, v);
#pragma unroll
    for (int k = 0; k < 27; ++k) {
      const unsigned hits = __ballot_sync(0xffffffffu, v[k] >= 0);
      if (lane == 0) warp_base_s[k][warp] = __popc(hits);
    }
  }
  if (table != nullptr) {
    // rows [L, table_stride) are padding; the last tile also covers the 256 rows past its own
    const bool second = tile == tiles - 1 && (int64_t)j + kPairsTile < table_stride;
    if (WALK == kWalkGeneric) {
      for (int k = 0; k < g.K; ++k) {
        int32_t *row = table + (size_t)(g.K - 1 - k) * table_stride;
        if (j < table_stride) row[j] = match_s[k * kPairsTile + threadIdx.x];
        if (second) row[j + kPairsTile] = -1;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 27; ++k) {
        int32_t *row = table + (size_t)(26 - k) * table_stride;
        if (j < table_stride) row[j] = v[k];
        if (second) row[j + kPairsTile] = -1;
      }
    }
  }
  __syncthreads();

  if (warp == 0) {
    int mine = 0;
    if (lane < g.K) {
#pragma unroll
      for (int w = 0; w < kTileWarps; ++w) {
        const int n = warp_base_s[lane][w];
        warp_base_s[lane][w] = mine;  // exclusive count of the warps before w
        mine += n;
      }
    }
    int before = 0;
    if (!tilePrefix(scratch, tile, tiles, mine, &before)) {
      if (lane == 0) raiseError(sink, kPairsErrLookBack);
      before = 0;
    }
    offset_s[lane] = before;
    if (tile == tiles - 1 && lane < g.K) {
      // indice_num may be pinned host memory (the caller wants the counts on the host
      // anyway); later kernels read the copy that stays in the workspace
      indice_num[lane] = before + mine;
      counts[lane] = before + mine;
    }
  }
  __syncthreads();

  const unsigned lower = (1u << lane) - 1u;
  if (WALK == kWalkGeneric) {
    for (int k = 0; k < g.K; ++k) {
      const int r = match_s[k * kPairsTile + threadIdx.x];
      const unsigned hits = __ballot_sync(0xffffffffu, r >= 0);
      if (r >= 0) {
        const int p = offset_s[k] + warp_base_s[k][warp] + __popc(hits & lower);
        int32_t *in_row = indice_pairs + (size_t)k * 2 * g.L;
        in_row[p] = j;
        in_row[g.L + p] = r;
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < 27; ++k) {
      const unsigned hits = __ballot_sync(0xffffffffu, v[k] >= 0);
      if (v[k] >= 0) {
        const int p = offset_s[k] + warp_base_s[k][warp] + __popc(hits & lower);
        int32_t *in_row = indice_pairs + (size_t)k * 2 * g.L;
        in_row[p] = j;
        in_row[g.L + p] = v[k];
      }
    }
  }
}

// Last kernel of every rulebook.
//   blockIdx.y < K: -1 from position indice_num[k] on, both rows of offset k
//     (nothing to do when the two-pass compaction already wrote its tails)
//   blockIdx.y == K: out_indices rows from the active count (default mode) or
//     from L (submanifold mode) on are -1, as the CPU path leaves them; block
//     (0, K) also hands {error bits, active count} to the host.
// A thread fills four consecutive words with one 16-byte store: positions are
// grouped in fours that start where the row's address is 16-byte aligned.
constexpr int kFinishSpan = 256 * 16;  // positions per block

__global__ void __launch_bounds__(256)
finishPairsKernel(int L, int K, int sub_m, int write_tails, const int32_t *__restrict__ counts,
                  int32_t *__restrict__ indice_pairs, int4 *__restrict__ out_indices, int64_t out_rows,
                  const int32_t *__restrict__ status, volatile int32_t *status_host) {
  const int k = blockIdx.y;
  if (k == K) {
    const int64_t first = sub_m ? (int64_t)L : (int64_t)status[kStatusActive];
    for (int64_t r = first + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < out_rows;
         r += (int64_t)gridDim.x * blockDim.x)
      out_indices[r] = make_int4(-1, -1, -1, -1);
    if (blockIdx.x == 0 && threadIdx.x == 0 && status_host != nullptr) {
      const int32_t bits = status[kStatusErrors];
      status_host[0] = bits;
      status_host[1] = sub_m ? L : status[kStatusActive];
      if (bits) status_host[2] |= bits;  // sticky: reported and cleared by the next entry point on the handle
      __threadfence_system();
    }
    return;
  }
  if (!write_tails) return;
  const int first = counts[k];
  const int base = blockIdx.x * kFinishSpan;
  if (base + kFinishSpan <= first) return;
#pragma unroll
  for (int row = 0; row < 2; ++row) {
    int32_t *dst = indice_pairs + ((size_t)k * 2 + row) * L;
    const int skew = (int)((reinterpret_cast<size_t>(dst) >> 2) & 3);  // words past a 16-byte boundary
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int p0 = base + (i * 256 + threadIdx.x) * 4 - skew;  // dst + p0 is 16-byte aligned
      if (p0 >= first && p0 >= 0 && p0 + 3 < L) {
        *reinterpret_cast<int4 *>(dst + p0) = make_int4(-1, -1, -1, -1);
      } else {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int p = p0 + u;
          if (p >= first && p >= 0 && p < L) dst[p] = -1;
        }
      }
    }
  }
}

// ---------------------------------------------------------------- two pass

// match[k][j] = output id or -1; tile_count[k][tile] = matches of this tile at offset k.
template <int LOOKUP>
__global__ void __launch_bounds__(kPairsTile)
probeCountKernel(PairsGeometry g, const int4 *__restrict__ indices, LookupTables tables,
                 int32_t *__restrict__ match, int32_t *__restrict__ tile_count, int tiles,
                 int4 *__restrict__ out_indices, int64_t out_rows, ErrorSink sink) {
  // match rows are tiles*256 entries long: every thread of every tile stores, and
  // the compaction kernel can read them 16 bytes at a time
  extern __shared__ int s_count[];  // [K]
  for (int k = threadIdx.x; k < g.K; k += blockDim.x) s_count[k] = 0;
  __syncthreads();
  const int j = blockIdx.x * kPairsTile + threadIdx.x;
  const bool live = j < g.L;
  int4 c = make_int4(0, 0, 0, 0);
  if (live) c = indices[j];
  if (g.sub_m && live && j < out_rows) out_indices[j] = c;
  const int lane = threadIdx.x & 31;
  int32_t *match_col = match + j;
  const size_t row_stride = (size_t)tiles * kPairsTile;
  walkOffsets<LOOKUP>(g, tables, c, live && rowInRange(c, g), sink, [&](int k, int v) {
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
  // submanifold lookup structure; MLUOP_B200_PAIRS_PATH=twopass selects the
  // staged pair-list path for every kernel volume (both are cross-checked by the tests).
  static const std::string lookup_env = envChoice("MLUOP_B200_PAIRS_LOOKUP");
  static const std::string path_env = envChoice("MLUOP_B200_PAIRS_PATH");
  PairsWorkspacePlan p{};
  p.tiles = (g.L + kPairsTile - 1) / kPairsTile;
  p.groups = (p.tiles + kGroupTiles - 1) / kGroupTiles;
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
  // Test hook: MLUOP_B200_TEST_HASH_CAPACITY=<n> makes submanifold rulebooks use the hash
  // table with at most n slots (rounded down to a power of two, at least 64), so that the
  // "table full" error path can be exercised: probes are bounded by the capacity, the
  // kernels record kPairsErrHashFull and carry on.
  uint32_t cap_limit = 0;
  if (g.sub_m) {
    if (const char *v = std::getenv("MLUOP_B200_TEST_HASH_CAPACITY")) cap_limit = (uint32_t)std::strtoul(v, nullptr, 10);
    if (cap_limit) p.lookup = kLookupHash;
  }
  p.fused = (g.K <= kFusedMaxOffsets && path_env != "twopass") ? 1 : 0;

  // scratch that must start at zero, cleared by one memset: [0, zero_end)
  size_t off = 0;
  p.status = off;
  off = alignUp(off + 64 * sizeof(int32_t), 256);
  p.counts = off;
  off = alignUp(off + (size_t)g.K * sizeof(int32_t), 256);
  p.tile_desc = p.group_desc = p.group_sum = p.group_done = off;
  if (p.fused) {
    p.tile_desc = off;
    off = alignUp(off + (size_t)p.tiles * kDescWords * sizeof(uint32_t), 256);
    p.group_desc = off;
    off = alignUp(off + (size_t)p.groups * kDescWords * sizeof(uint32_t), 256);
    p.group_sum = off;
    off = alignUp(off + (size_t)p.groups * kDescWords * sizeof(uint32_t), 256);
    p.group_done = off;
    off = alignUp(off + (size_t)p.groups * sizeof(int32_t), 256);
  }
  p.table = off;
  p.chunk_desc = off;
  p.perm = off;
  if (p.lookup == kLookupHash) {
    uint32_t cap = 64;
    while ((uint64_t)cap < 2ull * (uint64_t)g.L && (cap_limit == 0 || cap * 2 <= cap_limit)) cap <<= 1;
    p.hash_capacity = cap;
    off = alignUp(off + (size_t)cap * sizeof(unsigned long long), 256);
  } else {
    p.rank_words = (cells + 31) / 32;
    // up to 8 words per thread, fewer while that leaves less than about four chunks per SM
    p.rank_words_per_thread = 8;
    while (p.rank_words_per_thread > 1 && p.rank_words / (256 * p.rank_words_per_thread) < 600) p.rank_words_per_thread /= 2;
    const int64_t chunk_words = 256 * p.rank_words_per_thread;
    p.rank_chunks = (int32_t)((p.rank_words + chunk_words - 1) / chunk_words);
    off = alignUp(off + (size_t)p.rank_words * sizeof(uint2), 256);
    p.chunk_desc = off;
    off = alignUp(off + (size_t)p.rank_chunks * sizeof(uint32_t), 256);
    if (p.lookup == kLookupRankPerm) {
      p.perm = off;
      off = alignUp(off + (size_t)g.L * sizeof(int32_t), 256);
    }
  }
  p.zero_end = off;
  // scratch that is fully written before it is read
  p.match = p.tile_count = off;
  if (!p.fused) {
    off = alignUp(off + (size_t)g.K * p.tiles * kPairsTile * sizeof(int32_t), 256);
    p.tile_count = off;
    off = alignUp(off + (size_t)g.K * p.tiles * sizeof(int32_t), 256);
  }
  p.total = off + 256;  // slack to align the caller's pointer
  return p;
}

int64_t pairsTableStride(int64_t rows) { return (rows + kPairsTablePadRows - 1) / kPairsTablePadRows * kPairsTablePadRows; }

bool pairsCanEmitTable(const PairsGeometry &g, const PairsWorkspacePlan &plan) {
  if (!g.sub_m || !plan.fused) return false;
  for (int i = 0; i < 3; ++i)
    if (g.stride[i] != 1 || g.dil[i] != 1 || (g.ks[i] & 1) == 0 || g.pad[i] != g.ks[i] / 2) return false;
  return true;
}

namespace {

struct PairListArgs {
  const int4 *rows;
  LookupTables tables;
  PairListScratch scratch;
  int32_t *indice_pairs, *indice_num, *counts;
  int4 *out_indices;
  int64_t out_rows;
  int32_t *table;
  int64_t table_stride;
  ErrorSink sink;
};

template <int LOOKUP, int WALK>
void launchFused(const PairsGeometry &g, const PairsWorkspacePlan &plan, const PairListArgs &a,
                 cudaStream_t stream) {
  static const char *names[3][3] = {
      {"pairListsKernel<rank>", "pairListsKernel<rank,3x3x3 s1>", "pairListsKernel<rank,3x3x3 s2>"},
      {"pairListsKernel<hash>", "pairListsKernel<hash,3x3x3 s1>", "pairListsKernel<hash,3x3x3 s2>"},
      {"pairListsKernel<rank+perm>", "pairListsKernel<rank+perm,3x3x3 s1>", "pairListsKernel<rank+perm,3x3x3 s2>"}};
  const size_t smem = WALK == kWalkGeneric ? (size_t)g.K * kPairsTile * sizeof(int) : 0;
  auto kernel = pairListsKernel<LOOKUP, WALK>;
  // per voxel its coordinates (submanifold: and their copy in out_indices); the pairs
  // themselves are counted with the kernel that completes indice_pairs
  trace::Scope t(names[LOOKUP][WALK], stream, 16.0 * g.L + (g.sub_m ? 16.0 * g.L : 0.0));
  kernel<<<plan.tiles, kPairsTile, smem, stream>>>(g, a.rows, a.tables, a.scratch, plan.tiles, a.indice_pairs,
                                                   a.indice_num, a.counts, a.out_indices, a.out_rows, a.table,
                                                   a.table_stride, a.sink);
}

template <int LOOKUP>
void launchPairLists(const PairsGeometry &g, const PairsWorkspacePlan &plan, const PairListArgs &a, char *base,
                     cudaStream_t stream) {
  if (plan.fused) {
    const bool cube3 = g.ks[0] == 3 && g.ks[1] == 3 && g.ks[2] == 3 && g.dil[0] == 1 && g.dil[1] == 1 && g.dil[2] == 1;
    const bool s1 = g.stride[0] == 1 && g.stride[1] == 1 && g.stride[2] == 1;
    const bool s2 = g.stride[0] == 2 && g.stride[1] == 2 && g.stride[2] == 2;
    if (cube3 && s1) {
      launchFused<LOOKUP, kWalkCube3Stride1>(g, plan, a, stream);
    } else if (cube3 && s2) {
      launchFused<LOOKUP, kWalkCube3Stride2>(g, plan, a, stream);
    } else {
      launchFused<LOOKUP, kWalkGeneric>(g, plan, a, stream);
    }
    return;
  }
  const int tiles = plan.tiles;
  const double L = g.L, KL = (double)g.K * g.L;
  static const char *names_count[] = {"probeCountKernel<rank>", "probeCountKernel<hash>",
                                      "probeCountKernel<rank+perm>"};
  int32_t *match = reinterpret_cast<int32_t *>(base + plan.match);
  int32_t *tile_count = reinterpret_cast<int32_t *>(base + plan.tile_count);
  {
    trace::Scope t(names_count[LOOKUP], stream, 16.0 * L + 4.0 * KL);
    probeCountKernel<LOOKUP><<<tiles, kPairsTile, (size_t)g.K * sizeof(int), stream>>>(
        g, a.rows, a.tables, match, tile_count, tiles, a.out_indices, a.out_rows, a.sink);
  }
  {
    trace::Scope t("scanTilesKernel", stream, 8.0 * g.K * tiles);
    scanTilesKernel<<<g.K, 1024, 0, stream>>>(tile_count, tiles, a.indice_num, a.counts);
  }
  {
    trace::Scope t("writePairsKernel", stream, 12.0 * KL);
    const unsigned segments = (unsigned)((tiles + kWriteSegTiles - 1) / kWriteSegTiles);
    writePairsKernel<<<dim3(segments, g.K), kPairsTile, 0, stream>>>(g.L, match, tile_count, tiles, a.counts,
                                                                    a.indice_pairs);
  }
}

template <bool DECODE>
void launchRankScan(const PairsGeometry &g, const PairsWorkspacePlan &plan, uint2 *rank_table, uint32_t *chunk_desc,
                    int4 *out_indices, int64_t out_rows, const ErrorSink &sink, cudaStream_t stream) {
  const int chunks = plan.rank_chunks;
  switch (plan.rank_words_per_thread) {
    case 8:
      rankScanKernel<DECODE, 8><<<chunks, 256, 0, stream>>>(g, rank_table, plan.rank_words, chunks, chunk_desc,
                                                           out_indices, out_rows, sink);
      break;
    case 4:
      rankScanKernel<DECODE, 4><<<chunks, 256, 0, stream>>>(g, rank_table, plan.rank_words, chunks, chunk_desc,
                                                           out_indices, out_rows, sink);
      break;
    case 2:
      rankScanKernel<DECODE, 2><<<chunks, 256, 0, stream>>>(g, rank_table, plan.rank_words, chunks, chunk_desc,
                                                           out_indices, out_rows, sink);
      break;
    default:
      rankScanKernel<DECODE, 1><<<chunks, 256, 0, stream>>>(g, rank_table, plan.rank_words, chunks, chunk_desc,
                                                           out_indices, out_rows, sink);
      break;
  }
}

}  // namespace

cudaError_t launchGetIndicePairs(const PairsGeometry &g, const PairsWorkspacePlan &plan,
                                 const int32_t *indices, void *workspace, int32_t *indice_pairs,
                                 int32_t *out_indices, int64_t out_rows, int32_t *indice_num,
                                 int32_t *status_host, int32_t *neighbour_table, cudaStream_t stream) {
  char *base = reinterpret_cast<char *>(alignUp(reinterpret_cast<size_t>(workspace), 256));
  int32_t *status = reinterpret_cast<int32_t *>(base + plan.status);
  const int4 *rows = reinterpret_cast<const int4 *>(indices);
  const int tiles = plan.tiles;
  const double L = g.L, KL = (double)g.K * g.L;
  const ErrorSink sink{status, status_host ? status_host + 2 : nullptr};
  cudaError_t err;

  {
    trace::Scope t("memset:rulebook_scratch", stream, (double)plan.zero_end);
    if ((err = cudaMemsetAsync(base, 0, plan.zero_end, stream)) != cudaSuccess) return err;
  }

  PairListArgs a{};
  a.rows = rows;
  a.indice_pairs = indice_pairs;
  a.indice_num = indice_num;
  a.counts = reinterpret_cast<int32_t *>(base + plan.counts);
  a.out_indices = reinterpret_cast<int4 *>(out_indices);
  a.out_rows = out_rows;
  a.table = neighbour_table;
  a.table_stride = pairsTableStride(g.L);
  a.sink = sink;
  a.scratch.tile_desc = reinterpret_cast<uint32_t *>(base + plan.tile_desc);
  a.scratch.group_desc = reinterpret_cast<uint32_t *>(base + plan.group_desc);
  a.scratch.group_sum = reinterpret_cast<uint32_t *>(base + plan.group_sum);
  a.scratch.group_done = reinterpret_cast<int32_t *>(base + plan.group_done);

  if (plan.lookup == kLookupHash) {
    unsigned long long *slots = reinterpret_cast<unsigned long long *>(base + plan.table);
    a.tables.slots = slots;
    a.tables.mask = plan.hash_capacity - 1;
    trace::Scope t("hashInsertKernel", stream, 16.0 * L + 8.0 * L);
    hashInsertKernel<<<tiles, kPairsTile, 0, stream>>>(g, rows, slots, a.tables.mask, sink);
  } else {
    uint2 *rank_table = reinterpret_cast<uint2 *>(base + plan.table);
    uint32_t *chunk_desc = reinterpret_cast<uint32_t *>(base + plan.chunk_desc);
    const double words = (double)plan.rank_words;
    a.tables.rank_table = rank_table;
    if (g.sub_m) {
      trace::Scope t("markInputsKernel", stream, 16.0 * L);
      markInputsKernel<<<tiles, kPairsTile, 0, stream>>>(g, rows, rank_table);
    } else {
      trace::Scope t("markOutputsKernel", stream, 16.0 * L);
      bool cube3_s2 = true;
      for (int i = 0; i < 3; ++i) cube3_s2 = cube3_s2 && g.ks[i] == 3 && g.stride[i] == 2 && g.dil[i] == 1;
      if (cube3_s2) {
        markOutputsCube3Stride2Kernel<<<tiles, kPairsTile, 0, stream>>>(g, rows, rank_table);
      } else {
        markOutputsKernel<<<tiles, kPairsTile, 0, stream>>>(g, rows, rank_table);
      }
    }
    if (g.sub_m) {
      int32_t *perm = reinterpret_cast<int32_t *>(base + plan.perm);
      a.tables.perm = perm;
      {
        trace::Scope t("rankScanKernel", stream, 16.0 * words);
        launchRankScan<false>(g, plan, rank_table, chunk_desc, nullptr, 0, sink, stream);
      }
      trace::Scope t("permKernel", stream, 20.0 * L);
      permKernel<<<tiles, kPairsTile, 0, stream>>>(g, rows, rank_table, perm);
    } else {
      trace::Scope t("rankScanKernel<decode>", stream, 16.0 * words);
      launchRankScan<true>(g, plan, rank_table, chunk_desc, reinterpret_cast<int4 *>(out_indices), out_rows, sink,
                           stream);
    }
  }

  switch (plan.lookup) {
    case kLookupHash:
      launchPairLists<kLookupHash>(g, plan, a, base, stream);
      break;
    case kLookupRankPerm:
      launchPairLists<kLookupRankPerm>(g, plan, a, base, stream);
      break;
    default:
      launchPairLists<kLookupRank>(g, plan, a, base, stream);
      break;
  }
  if ((err = cudaGetLastError()) != cudaSuccess) return err;
  {
    // -1 tails of indice_pairs (8 bytes per unused slot) and -1 rows of out_indices.  The
    // status words reach the host through device-mapped pinned memory, so the read-back
    // does not queue behind whatever large transfers the application has on the copy engines.
    trace::Scope t("finishPairsKernel", stream, 8.0 * KL);
    const unsigned spans = (unsigned)(((int64_t)g.L + 3 + kFinishSpan - 1) / kFinishSpan);
    finishPairsKernel<<<dim3(spans, g.K + 1), 256, 0, stream>>>(g.L, g.K, g.sub_m, plan.fused, a.counts,
                                                                indice_pairs, reinterpret_cast<int4 *>(out_indices),
                                                                out_rows, status, status_host);
  }
  return cudaGetLastError();
}

}  // namespace sparse_conv
}  // namespace mluop
