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
// A neighbour table emitted by the rulebook has rows padded to a multiple of this
// many entries (the padding of the convolution's neighbour table).
constexpr int kPairsTablePadRows = 512;

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
constexpr int64_t kDenseCellsPerVoxel = 1024;
// Kernel volumes up to this size take the single-pass pair-list path (one
// descriptor word per offset; matches of a tile stay on chip).
constexpr int kFusedMaxOffsets = 32;

// Byte offsets of the scratch arrays inside the (256-byte aligned) workspace.
// Everything in [0, zero_end) is cleared by one memset at the start of a call.
struct PairsWorkspacePlan {
  size_t status;      // int32[64]: [0] error bits, [1] number of active outputs, [2] tile ticket, [3] chunk ticket
  size_t counts;      // int32[K]: pair counts, the copy the kernels read (indice_num may be host memory)
  size_t tile_desc;   // single pass: uint32[tiles][32] per-offset counts of a tile {2-bit state, 30-bit count}
  size_t group_desc;  // single pass: uint32[groups][32] aggregate / inclusive prefix of a group of 32 tiles
  size_t group_sum;   // single pass: uint32[groups][32] running sums of the groups
  size_t group_done;  // single pass: int32[groups] tiles of a group that have published
  size_t table;       // hash: uint64[capacity] slots; rank: uint2[words] {occupancy bits, exclusive rank}
  size_t chunk_desc;  // rank: uint32[chunks] look-back descriptors of the rank scan
  size_t perm;        // rank + perm: int32[L] row id + 1 of the r-th occupied cell
  size_t zero_end;    // end of the region that must start at zero
  size_t match;       // two pass: int32[K][tiles*256] output id matched by (k, j), -1 if none
  size_t tile_count;  // two pass: int32[K][tiles] matches per tile, then exclusive offsets
  size_t total;       // bytes including alignment slack
  int32_t tiles;
  int32_t groups;
  int32_t lookup;          // PairsLookup
  int32_t fused;           // 1: single-pass path
  uint32_t hash_capacity;  // hash: power of two >= 2L
  int64_t rank_words;      // rank: ceil(cells / 32)
  int32_t rank_words_per_thread;  // rank: 8, 4, 2 or 1 occupancy words per thread of the scan
  int32_t rank_chunks;            // rank: chunks of 256 * rank_words_per_thread words
};

PairsWorkspacePlan planPairsWorkspace(const PairsGeometry &g);

// Error bits in status[0].
constexpr int kPairsErrHashFull = 1;         // hash probe ran through the whole table
constexpr int kPairsErrOutIndicesSmall = 2;  // more active outputs than out_indices rows
constexpr int kPairsErrLookBack = 4;         // a bounded look-back wait gave up

// Row stride (entries) of a neighbour table with `rows` rows per offset.
int64_t pairsTableStride(int64_t rows);
// Whether the rulebook kernels can emit the neighbour table themselves: a
// submanifold rulebook on the single-pass path with odd kernel sizes, unit stride
// and dilation and centred padding (pad = size / 2).  The table entry of (offset
// k, output row r) is then the match of input row r at the mirrored offset K-1-k.
bool pairsCanEmitTable(const PairsGeometry &g, const PairsWorkspacePlan &plan);

// Enqueues the whole rulebook computation on `stream`.  status_host (pinned,
// device-mapped host memory, three words) receives {error bits, number of active
// outputs} from the last kernel and error bits are ORed into its third word; the
// caller synchronises when it needs them.  neighbour_table (optional, only when
// pairsCanEmitTable) receives int32[K][pairsTableStride(L)].
cudaError_t launchGetIndicePairs(const PairsGeometry &g, const PairsWorkspacePlan &plan,
                                 const int32_t *indices, void *workspace, int32_t *indice_pairs,
                                 int32_t *out_indices, int64_t out_rows, int32_t *indice_num,
                                 int32_t *status_host, int32_t *neighbour_table, cudaStream_t stream);

}  // namespace sparse_conv
}  // namespace mluop

#endif  // MLUOP_B200_KERNELS_SPARSE_CONV_GET_INDICE_PAIRS_KERNELS_H_
