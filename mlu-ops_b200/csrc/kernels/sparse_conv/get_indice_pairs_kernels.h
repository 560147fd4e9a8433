// Device side of rulebook generation: geometry block, workspace plan and the
// launch sequence.  The host entry points in get_indice_pairs.cpp do the
// argument checks and call into here.
#ifndef MLUOP_B200_KERNELS_SPARSE_CONV_GET_INDICE_PAIRS_KERNELS_H_
#define MLUOP_B200_KERNELS_SPARSE_CONV_GET_INDICE_PAIRS_KERNELS_H_

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

namespace mluop {
namespace sparse_conv {

// Input voxels handled by one thread block of the probe and write kernels.
constexpr int kPairsTile = 256;
// 32-bit occupancy words handled by one thread block of the rank kernels.
constexpr int kRankChunkWords = 1024;

struct PairsGeometry {
  int32_t L;      // active input voxels
  int32_t K;      // kernel volume
  int32_t batch;
  int32_t ks[3], pad[3], stride[3], dil[3];
  int32_t stride_shift[3];  // log2(stride) when the stride is a power of two, else -1
  int32_t in_space[3], out_space[3];
  int32_t out_vol;  // Do*Ho*Wo
  int32_t sub_m;
};

// How (k, voxel) -> output id is looked up.
enum PairsLookup {
  kLookupRank = 0,      // default mode: occupancy bits + prefix rank over the output grid
  kLookupHash = 1,      // submanifold, sparse grid: hash table lin -> row id
  kLookupRankPerm = 2,  // submanifold, dense grid: occupancy bits + rank, then rank -> row id
};

// A submanifold rulebook uses the occupancy-bit table instead of the hash table
// when the grid has at most this many cells per input voxel: the table is then
// small, and neighbouring cells share its words, which a hash table cannot offer.
constexpr int64_t kDenseCellsPerVoxel = 512;
// Kernel volumes up to this size can take the opt-in single-pass path (matches
// of a tile stay in shared memory).
constexpr int kFusedMaxOffsets = 32;

// Byte offsets of the scratch arrays inside the (256-byte aligned) workspace.
struct PairsWorkspacePlan {
  size_t status;      // int32[64]: [0] error bits, [1] number of active outputs, [2] tile ticket counter
  size_t counts;      // int32[K]: pair counts, the copy the kernels read (indice_num may be host memory)
  size_t tile_state;  // fused path: uint32[K][tiles] look-back descriptors {2-bit state, 30-bit count}
  size_t match;       // two-pass path: int32[K][tiles*256] output id matched by (k, j), -1 if none
  size_t tile_count;  // two-pass path: int32[K][tiles] matches per tile, then exclusive offsets
  size_t table;       // hash: uint64[capacity] slots; rank: uint2[words] {occupancy bits, exclusive rank}
  size_t chunk_count; // rank: int32[chunks]
  size_t perm;        // rank + perm: int32[L] row id of the r-th occupied cell
  size_t total;       // bytes including alignment slack
  int32_t tiles;
  int32_t lookup;          // PairsLookup
  int32_t fused;           // 1: single-pass path
  uint32_t hash_capacity;  // hash: power of two >= 2L
  int64_t rank_words;      // rank: ceil(cells / 32)
  int32_t rank_chunks;
};

PairsWorkspacePlan planPairsWorkspace(const PairsGeometry &g);

// Error bits in status[0].
constexpr int kPairsErrHashFull = 1;         // hash probe ran through the whole table
constexpr int kPairsErrOutIndicesSmall = 2;  // more active outputs than out_indices rows
constexpr int kPairsErrLookBack = 4;         // a bounded look-back wait gave up

// Enqueues the whole rulebook computation on `stream`.  status_host (pinned,
// device-mapped host memory) receives {error bits, number of active outputs}
// from a last one-thread kernel; the caller synchronises when it needs them.
cudaError_t launchGetIndicePairs(const PairsGeometry &g, const PairsWorkspacePlan &plan,
                                 const int32_t *indices, void *workspace, int32_t *indice_pairs,
                                 int32_t *out_indices, int64_t out_rows, int32_t *indice_num,
                                 int32_t *status_host, cudaStream_t stream);

}  // namespace sparse_conv
}  // namespace mluop

#endif  // MLUOP_B200_KERNELS_SPARSE_CONV_GET_INDICE_PAIRS_KERNELS_H_
