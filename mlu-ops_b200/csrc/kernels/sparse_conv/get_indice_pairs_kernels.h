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
  int32_t in_space[3], out_space[3];
  int32_t out_vol;  // Do*Ho*Wo
  int32_t sub_m;
};

// Byte offsets of the scratch arrays inside the (256-byte aligned) workspace.
struct PairsWorkspacePlan {
  size_t status;      // int32[64]: [0] error bits, [1] number of active outputs
  size_t match;       // int32[K][L]: output id matched by (k, j), -1 if none
  size_t tile_count;  // int32[K][tiles]: matches per tile, then exclusive offsets
  size_t table;       // subm: uint64[capacity] hash slots; default: uint2[words] {bits, rank}
  size_t chunk_count; // default mode: int32[chunks]
  size_t total;       // bytes including alignment slack
  int32_t tiles;
  uint32_t hash_capacity;  // subm: power of two >= 2L
  int64_t rank_words;      // default: ceil(batch*out_vol / 32)
  int32_t rank_chunks;
};

PairsWorkspacePlan planPairsWorkspace(const PairsGeometry &g);

// Error bits in status[0].
constexpr int kPairsErrHashFull = 1;      // hash probe ran through the whole table
constexpr int kPairsErrOutIndicesSmall = 2;  // more active outputs than out_indices rows

// Enqueues the whole rulebook computation on `stream`.  n_out_host (pinned)
// receives {error bits, number of active outputs} by an async copy that is
// ordered after the kernels; the caller synchronises when it needs them.
cudaError_t launchGetIndicePairs(const PairsGeometry &g, const PairsWorkspacePlan &plan,
                                 const int32_t *indices, void *workspace, int32_t *indice_pairs,
                                 int32_t *out_indices, int64_t out_rows, int32_t *indice_num,
                                 int32_t *status_host, cudaStream_t stream);

}  // namespace sparse_conv
}  // namespace mluop

#endif  // MLUOP_B200_KERNELS_SPARSE_CONV_GET_INDICE_PAIRS_KERNELS_H_
