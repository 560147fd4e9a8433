// Filter gradient of the sparse convolution on the 5th-generation tensor cores
// (tcgen05) of sm_100a: half inputs with 32 or 64 input channels, fp32 accumulation
// in tensor memory.
//
//   filters_grad[k,c,n] = sum_j features[nbr[k][j], c] * output_grad[j, n]
//
// where nbr is the neighbour table of the forward convolution (input row feeding
// output row j through offset k, -1 if none).  Per offset this is a product
// whose long (contracted) axis is the list of output rows, so the roles of the
// forward kernel are turned round: the block keeps the [Ci x Co] sums of its
// offsets in tensor memory for the whole kernel and streams tiles of 128 output
// rows past them.
//
// Work split.  128 / Ci offsets (a "bundle": two at 64 channels, four at 32) share
// one accumulator of 128 lanes (lanes h*Ci .. h*Ci+Ci-1: the input channels of the
// bundle's h-th offset) and Co columns.  Tensor memory holds 512/Co such bundles
// (and the kernel keeps at most 16 offsets' table entries in registers), so the
// offsets are cut into groups and a block serves one group.  The blocks of a group
// (one per SM) take the tiles of 128 output rows round-robin.
//
// Per tile the eight producer warps copy the tile's output_grad rows to shared
// memory once (contiguous rows, cp.async) and, for every bundle with at least one
// live row in the tile, gather the feature rows of its offsets into a stage
// of the ring (rows without a neighbour are zero-filled, nothing is fetched).
// Both operands lie row-major in shared memory - the contracted axis (rows) is
// the slow one - which tcgen05.mma reads as "MN-major" operands: an issuing
// thread (there are two, each owning every other accumulator) issues 8 MMAs
// (M=128, N=Co, K=16 rows each) per bundle and tile and releases the stage with
// tcgen05.commit.  Producers, issuer and epilogue each
// derive which bundles are live from the table itself (a warp reads the tile's
// 128 entries of an offset with one 16-byte load per lane and votes), so no
// flags travel between them.
//
// After its last tile the block reads its accumulators back (tcgen05.ld) and
// writes them as a float partial; reduceFilterGradTcKernel adds the partials of
// a group's blocks in ascending block order and converts to half.  Tiles are
// dealt statically, so the result does not depend on scheduling.
//
// A row of output_grad that has no neighbour at an offset meets a zero-filled
// feature row, so unlike a walk over the pair lists an infinity or NaN in such a
// row reaches that offset's gradient as NaN (0 x inf).
//
// Every mbarrier wait is bounded (tcgen05_primitives.cuh); a waiter that gives
// up takes its warp to the common exit, where copies in flight are drained,
// outstanding MMAs are seen out and tensor memory is freed.
#include "kernels/sparse_conv/indice_convolution_backward_filter_tcgen05.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <string>

#include "core/trace.h"
#include "kernels/sparse_conv/indice_convolution_kernels.h"
#include "kernels/sparse_conv/tcgen05_primitives.cuh"

namespace mluop {
namespace sparse_conv {

namespace {

using namespace tc;

constexpr int kTile = kConvTileRows;  // 128 output rows per tile
constexpr int kProducerWarps = 8;      // warps 0-7: gather; warps 0-3 also read the sums back
constexpr int kProducerThreads = kProducerWarps * 32;
constexpr int kIssuerWarp = kProducerWarps;  // first MMA-issuing warp; it also owns the tensor-memory allocation
// Two issuing threads (one per warp): a single thread's wait / issue / release loop handles an item
// in no less than about 300 clocks plus the time its MMAs are accepted in, and was the slowest
// part of the chain.  Accumulator q belongs to issuer q % kIssuers, so every sum still sees its
// tiles in one fixed order.
constexpr int kIssuers = 2;
constexpr int kThreads = kProducerThreads + 32 * kIssuers;
constexpr int kMaxGroupOffsets = 16;  // offsets whose table entries a thread keeps in registers
constexpr long long kWaitCycles = 2000000000ll;  // a wait gives up after about one second
constexpr int kErrProducerStage = 1, kErrIssuerStage = 2, kErrAccum = 4, kErrGradTile = 8, kErrIssuerGrad = 16;

// An operand tile in shared memory: 128 rows (the contracted axis) of up to 64 halfs,
// `row_bytes` apart, 16-byte chunks XOR-swizzled over `row_bytes`; wider rows are split
// into 64-half atoms `kTileBytes` apart.
template <int CHANNELS>
struct OperandTile {
  static constexpr int kAtomChannels = CHANNELS < 64 ? CHANNELS : 64;
  static constexpr int kAtoms = CHANNELS / kAtomChannels;
  static constexpr int kRowBytes = kAtomChannels * 2;              // 64 or 128
  static constexpr unsigned kSwizzleMask = kRowBytes / 16 - 1;     // 3 or 7
  static constexpr unsigned long long kLayoutType = kRowBytes == 128 ? 2 : 4;  // 128-byte / 64-byte swizzle
  static constexpr int kTileBytes = kTile * kRowBytes;             // one atom: 8 or 16 KB
  static constexpr int kBytes = kAtoms * kTileBytes;
  static constexpr int kGroupStride = 8 * kRowBytes;               // between groups of 8 rows
  static constexpr int kStepBytes = 16 * kRowBytes;                // 16 rows of the contracted axis (one MMA)
};

template <int CI, int CO>
struct GradTcConfig {
  using A = OperandTile<CI>;   // the gathered rows of ONE offset
  using G = OperandTile<CO>;   // a tile of output_grad rows
  static constexpr int kOffsetsPerBundle = kTile / CI;  // 2 or 4: together 128 accumulator lanes
  static constexpr int kBundlesByTmem = 512 / CO;
  static constexpr int kBundlesByRegs = kMaxGroupOffsets / kOffsetsPerBundle;
  static constexpr int kBundlesPerGroup = kBundlesByTmem < kBundlesByRegs ? kBundlesByTmem : kBundlesByRegs;
  static constexpr int kOffsetsPerGroup = kBundlesPerGroup * kOffsetsPerBundle;
  static constexpr int kTmemCols = kBundlesPerGroup * CO;  // 128, 256 or 512 (a power of two)
  static constexpr int kAStageBytes = kOffsetsPerBundle * A::kBytes;  // 32 KB: the gathered rows of a bundle
  static constexpr int kGradBufBytes = G::kBytes;
  static constexpr int kGradBufs = 2;
  // as many stages as shared memory holds: the gathers are latency-bound, what counts is bytes in flight
  static constexpr int kAStages = (227 * 1024 - 2048 - kGradBufs * kGradBufBytes) / kAStageBytes;
  static constexpr size_t kSmemBytes = 1024 + (size_t)kAStages * kAStageBytes + (size_t)kGradBufs * kGradBufBytes;
  // D fp32, A and B fp16, both MN-major (bits 15 and 16), N = CO, M = 128
  static constexpr unsigned kIdesc =
      (1u << 4) | (1u << 15) | (1u << 16) | ((unsigned)(CO >> 3) << 17) | ((unsigned)(kTile >> 4) << 24);
};

// Descriptor of an MN-major operand tile: the elements of an atom's M (or N) axis are
// contiguous (one row per step of the contracted axis), groups of 8 rows are
// kGroupStride bytes apart (stride byte offset) and the next atom of the M/N axis starts
// `atom_stride` bytes further (leading byte offset).
template <typename Tile>
__device__ __forceinline__ unsigned long long makeDescMn(unsigned smem_byte_addr, unsigned atom_stride) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_byte_addr & 0x3FFFFu) >> 4);
  d |= (unsigned long long)(atom_stride >> 4) << 16;
  d |= (unsigned long long)((unsigned)Tile::kGroupStride >> 4) << 32;
  d |= 1ull << 46;
  d |= Tile::kLayoutType << 61;
  return d;
}

// Liveness of a tile's offsets, in two steps so that the loads of the next tile can be in
// flight while the current one is processed.  loadTileEntries: lane l of the calling warp
// loads the table entries of rows 4l..4l+3 of the tile for each of the group's offsets
// (all -1 past the last tile or offset).  voteTileLive: bit j of the result is set when
// some row of the tile has a neighbour at offset k0 + j; every lane gets the same mask.
template <int OFFSETS>
__device__ __forceinline__ void loadTileEntries(const int32_t *__restrict__ nbr, int64_t n_pad, int64_t tile,
                                                int64_t n_tiles, int k0, int k_end, int lane, int4 (&v)[OFFSETS]) {
#pragma unroll
  for (int j = 0; j < OFFSETS; ++j) {
    if (k0 + j < k_end && tile < n_tiles) {
      v[j] = __ldg(reinterpret_cast<const int4 *>(nbr + (size_t)(k0 + j) * n_pad + tile * kTile) + lane);
    } else {
      v[j] = make_int4(-1, -1, -1, -1);
    }
  }
}
template <int OFFSETS>
__device__ __forceinline__ unsigned voteTileLive(const int4 (&v)[OFFSETS]) {
  unsigned mask = 0u;
#pragma unroll
  for (int j = 0; j < OFFSETS; ++j) {
    if (__ballot_sync(0xffffffffu, (v[j].x & v[j].y & v[j].z & v[j].w) >= 0)) mask |= 1u << j;
  }
  return mask;
}

template <int CI, int CO>
__global__ void __launch_bounds__(kThreads, 1)
filterGradTcgen05Kernel(const __half *__restrict__ features, const __half *__restrict__ output_grad,
                        const int32_t *__restrict__ nbr, int64_t n_out, int64_t n_pad, int K, int bundles_per_group,
                        int blocks_per_group, float *__restrict__ partial, int32_t *status_word, int32_t *sticky, long long wait_limit,
                        int test_drop_release) {
  using Cfg = GradTcConfig<CI, CO>;
  using ATile = typename Cfg::A;
  using GTile = typename Cfg::G;
  constexpr int S = Cfg::kAStages, NG = Cfg::kGradBufs, OPB = Cfg::kOffsetsPerBundle, OPG = Cfg::kOffsetsPerGroup;
  constexpr int kTmemCols = Cfg::kTmemCols;
  constexpr int kGradChunks = CO / 8;  // 16-byte chunks of one output_grad row
  extern __shared__ unsigned char smem_raw[];
  unsigned char *a_ring = reinterpret_cast<unsigned char *>((reinterpret_cast<size_t>(smem_raw) + 1023) & ~(size_t)1023);
  unsigned char *g_ring = a_ring + (size_t)S * Cfg::kAStageBytes;
  // a_full: one set of barriers per issuer.  An mbarrier wait names a phase by its parity only, so a
  // waiter must see every phase of a barrier: an issuer that waited on a stage only when the item in it
  // is its own would skip phases and take a stage that is still being filled for one that is ready.
  // The producers arrive on the barrier of the issuer that owns the item.
  __shared__ unsigned long long a_full[kIssuers][S], a_empty[S], g_full[NG], g_empty[NG], accum_bar, drain_bar[kIssuers];
  __shared__ unsigned tmem_base_s;
  __shared__ int abort_s;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = blockIdx.x / blocks_per_group, member = blockIdx.x % blocks_per_group;
  // the group's offsets: bundles_per_group (<= kBundlesPerGroup) bundles from offset k0 on
  const int k0 = group * OPB * bundles_per_group;
  const int k_end = K < k0 + OPB * bundles_per_group ? K : k0 + OPB * bundles_per_group;
  const int64_t n_tiles = (n_out + kTile - 1) / kTile;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      for (int i = 0; i < kIssuers; ++i) mbarInit(&a_full[i][s], kProducerThreads);
      mbarInit(&a_empty[s], 1);
    }
    for (int g = 0; g < NG; ++g) {
      mbarInit(&g_full[g], kProducerThreads);
      mbarInit(&g_empty[g], kIssuers);
    }
    mbarInit(&accum_bar, kIssuers);
    for (int i = 0; i < kIssuers; ++i) mbarInit(&drain_bar[i], 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == kIssuerWarp) tmemAlloc(&tmem_base_s, kTmemCols);
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const unsigned tmem_base = tmem_base_s;
  volatile int *abort_flag = &abort_s;
  const ErrorSink status{status_word, sticky};

  if (warp < kProducerWarps) {
    // ------------------------------------------------------------ producers
    // Eight warps, so that every scheduler of the SM has two to hide instruction latency
    // with (four warps, one per scheduler, ran at a fifth of the issue rate).  Warp w
    // gathers rows 16w..16w+15 of every offset of a bundle.  A lane holds table entries of
    // row 16w + (l & 15): register j for offset 2j + (l >> 4) of the bundle, and hands them
    // to the lanes that fetch that row by shuffle; consecutive lanes fetch consecutive
    // 16-byte chunks of a feature row (CPR per row), so one warp instruction touches
    // 32 / CPR rows.
    constexpr int CPR = CI / 8;                 // 16-byte chunks per feature row: 4 or 8
    constexpr int kRowsPerInstr = 32 / CPR;     // 8 or 4
    constexpr int kInstrPerOffset = 16 / kRowsPerInstr;  // 2 or 4
    const int rr0 = lane / CPR, chunk = lane % CPR;
    const int my_row = warp * 16 + (lane & 15), my_half = lane >> 4;
    unsigned a_off[kInstrPerOffset];
#pragma unroll
    for (int i = 0; i < kInstrPerOffset; ++i) {
      const int row = warp * 16 + rr0 + i * kRowsPerInstr;
      unsigned off = (unsigned)(row * ATile::kRowBytes + chunk * 16);
      off ^= ((off >> 7) & ATile::kSwizzleMask) << 4;
      a_off[i] = off;
    }
    const unsigned a_ring_addr = smemAddr(a_ring), g_ring_addr = smemAddr(g_ring);
    const __half *feat_chunk = features + chunk * 8;

    int s = 0;
    unsigned a_parity = 0, items = 0, ever_live = 0u;
    bool ok = true;
    int64_t n_mine = 0;
    // table entries of the next tile, for the vote
    int4 vote_next[OPG];
    loadTileEntries<OPG>(nbr, n_pad, member, n_tiles, k0, k_end, lane, vote_next);
    for (int64_t tile = member; tile < n_tiles && ok; tile += blocks_per_group, ++n_mine) {
      const int64_t row0 = tile * kTile;
      const unsigned live = voteTileLive<OPG>(vote_next);
      loadTileEntries<OPG>(nbr, n_pad, tile + blocks_per_group, n_tiles, k0, k_end, lane, vote_next);
      ever_live |= live;
      // this tile's rows of output_grad
      const int g = (int)(n_mine % NG);
      if (n_mine >= NG) {
        if (!mbarWaitWarp(&g_empty[g], (unsigned)((n_mine / NG) - 1) & 1u, abort_flag, status, kErrGradTile,
                          wait_limit)) {
          ok = false;
          break;
        }
      }
      if (live) {
        const unsigned g_addr = g_ring_addr + (unsigned)g * Cfg::kGradBufBytes;
#pragma unroll
        for (int i = 0; i < kGradChunks * kTile / kProducerThreads; ++i) {
          const int e = tid + i * kProducerThreads;
          const int row = e / kGradChunks, c = e % kGradChunks;
          constexpr int kAtomChunks = GTile::kRowBytes / 16;
          unsigned off = (unsigned)(row * GTile::kRowBytes + (c % kAtomChunks) * 16);
          off ^= ((off >> 7) & GTile::kSwizzleMask) << 4;
          const bool valid = row0 + row < n_out;
          cpAsync16(g_addr + (unsigned)(c / kAtomChunks) * GTile::kTileBytes + off,
                    output_grad + (valid ? (size_t)(row0 + row) * CO + c * 8 : 0), valid);
        }
      }
      cpAsyncArriveOn(&g_full[g]);
      // the gathered feature rows of every live pair
      // (a real loop: unrolled over the pairs its body no longer fits the instruction cache)
      unsigned todo = 0u;  // bit q: bundle q has a live offset
#pragma unroll
      for (int q = 0; q < Cfg::kBundlesPerGroup; ++q)
        if ((live >> (q * OPB)) & ((1u << OPB) - 1u)) todo |= 1u << q;
#pragma unroll 1
      while (todo && ok) {
        const int q = __ffs(todo) - 1;
        todo &= todo - 1u;
        // this lane's table entries (row 16w + (l & 15)); the lines are in L1 since the vote
        int idx[OPB / 2];
#pragma unroll
        for (int j = 0; j < OPB / 2; ++j) {
          const int k = k0 + q * OPB + 2 * j + my_half;
          idx[j] = k < k_end ? __ldg(nbr + (size_t)k * n_pad + row0 + my_row) : -1;
        }
        if (items >= (unsigned)S) {
          if (!mbarWaitWarp(&a_empty[s], a_parity ^ 1u, abort_flag, status, kErrProducerStage, wait_limit)) {
            ok = false;
            continue;
          }
        }
        const unsigned stage_addr = a_ring_addr + (unsigned)s * Cfg::kAStageBytes;
#pragma unroll
        for (int h = 0; h < OPB; ++h) {
#pragma unroll
          for (int i = 0; i < kInstrPerOffset; ++i) {
            const int src_row = __shfl_sync(0xffffffffu, idx[h >> 1], (h & 1) * 16 + rr0 + i * kRowsPerInstr);
            const bool valid = src_row >= 0;
            cpAsync16(stage_addr + (unsigned)h * ATile::kBytes + a_off[i], feat_chunk + (valid ? (size_t)src_row * CI : 0),
                      valid);
          }
        }
        cpAsyncArriveOn(&a_full[q % kIssuers][s]);
        ++items;
        if (++s == S) {
          s = 0;
          a_parity ^= 1u;
        }
      }
    }
    cpAsyncWaitAll();

    // ------------------------------------------------------------- epilogue
    bool have_acc = ok && items > 0;
    if (have_acc) have_acc = mbarWaitWarp(&accum_bar, 0, abort_flag, status, kErrAccum, wait_limit);
    tcFenceAfter();
    if (ok && !*abort_flag && warp < 4) {
      float *dst_block = partial + (size_t)blockIdx.x * bundles_per_group * kTile * CO;
#pragma unroll 1
      for (int q = 0; q < bundles_per_group; ++q) {
        const bool touched = have_acc && ((ever_live >> (q * OPB)) & ((1u << OPB) - 1u));
        float *dst = dst_block + ((size_t)q * kTile + tid) * CO;
#pragma unroll
        for (int c0 = 0; c0 < CO; c0 += 16) {
          unsigned v[16];
          if (touched) {
            tmemLoad16(tmem_base + ((unsigned)(warp * 32) << 16) + (unsigned)(q * CO + c0), v);
            tmemLoadWait();
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0u;
          }
#pragma unroll
          for (int i = 0; i < 16; i += 4)
            *reinterpret_cast<uint4 *>(dst + c0 + i) = make_uint4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
      }
    }
    tcFenceBefore();
  } else {
    // ------------------------------------------------------------ MMA issuers
    // The whole warp derives the live bundles of a tile; lane 0 issues those of its accumulators.
    const int me = warp - kIssuerWarp;
    const unsigned long long a_desc0 = makeDescMn<ATile>(smemAddr(a_ring), ATile::kBytes);
    const unsigned long long g_desc0 = makeDescMn<GTile>(smemAddr(g_ring), GTile::kTileBytes);
    unsigned started = 0u;  // bundles whose accumulator has been written
    int s = 0;
    unsigned items = 0, my_items = 0;  // items: all of the block's, my_items: this issuer's
    unsigned my_phase = 0u;  // bit s: parity of the next phase of a_full[me][s]
    bool ok = true;
    int64_t n_mine = 0;
    int4 vote_next[OPG];
    loadTileEntries<OPG>(nbr, n_pad, member, n_tiles, k0, k_end, lane, vote_next);
    for (int64_t tile = member; tile < n_tiles && ok; tile += blocks_per_group, ++n_mine) {
      const unsigned live = voteTileLive<OPG>(vote_next);
      loadTileEntries<OPG>(nbr, n_pad, tile + blocks_per_group, n_tiles, k0, k_end, lane, vote_next);
      const int g = (int)(n_mine % NG);
      if (lane == 0) {
        ok = mbarWait(&g_full[g], (unsigned)(n_mine / NG) & 1u, abort_flag, status, kErrIssuerGrad, wait_limit);
        const unsigned long long g_desc = g_desc0 + (unsigned long long)((g * Cfg::kGradBufBytes) >> 4);
        for (int q = 0; q < Cfg::kBundlesPerGroup && ok; ++q) {
          if (!((live >> (q * OPB)) & ((1u << OPB) - 1u))) continue;
          if (q % kIssuers == me) {
            // the phase of MY barrier of this stage: it advances only when an item of mine uses the stage
            if (!mbarWait(&a_full[me][s], (my_phase >> s) & 1u, abort_flag, status, kErrIssuerStage, wait_limit)) {
              ok = false;
              break;
            }
            fenceProxyAsync();
            tcFenceAfter();
            const unsigned long long a_desc = a_desc0 + (unsigned long long)((s * Cfg::kAStageBytes) >> 4);
            const unsigned d_addr = tmem_base + (unsigned)(q * CO);
#pragma unroll
            for (int j = 0; j < kTile / 16; ++j) {
              // 16 rows of the contracted axis per MMA: 16 rows further in both operands
              umma(d_addr, a_desc + (unsigned long long)((j * ATile::kStepBytes) >> 4),
                   g_desc + (unsigned long long)((j * GTile::kStepBytes) >> 4), Cfg::kIdesc,
                   (((started >> q) & 1u) || j > 0) ? 1u : 0u);
            }
            started |= 1u << q;
            my_phase ^= 1u << s;
            // the stage may be refilled once these MMAs have read it (test hook: the first issuer's first
            // release is withheld, so that the producers' wait for that stage runs out)
            if (!(test_drop_release && me == 0 && my_items == 0)) ummaCommit(&a_empty[s]);
            ++my_items;
          }
          ++items;
          if (++s == S) s = 0;
        }
        // the tile's output_grad rows are free once both issuers' MMAs issued so far are done
        if (ok) ummaCommit(&g_empty[g]);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    }
    if (lane == 0) {
      if (ok && items > 0 && !*abort_flag) {
        ummaCommit(&accum_bar);
      } else if (my_items > 0) {
        // leaving early: see the outstanding MMAs out before tensor memory is freed
        ummaCommit(&drain_bar[me]);
        const long long t0 = clock64();
        while (!mbarTryWait(&drain_bar[me], 0) && clock64() - t0 <= wait_limit) {
        }
      }
    }
    __syncwarp();
    tcFenceBefore();
  }
  __syncthreads();
  if (warp == kIssuerWarp) {
    tcFenceAfter();
    tmemDealloc(tmem_base, kTmemCols);
  }
}

// filters_grad[k][c][n] = sum over the blocks of k's group, in ascending block
// order, of partial[block][bundle of k][lane (k % offsets per bundle) * Ci + c][n].
__global__ void __launch_bounds__(256)
reduceFilterGradTcKernel(const float *__restrict__ partial, int K, int ci, int co, int bundles_per_group,
                         int blocks_per_group, __half *__restrict__ filters_grad) {
  const int64_t total = (int64_t)K * ci * co;
  const int offsets_per_bundle = kTile / ci;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int n = (int)(i % co);
    const int c = (int)((i / co) % ci);
    const int k = (int)(i / ((int64_t)co * ci));
    const int bundle = k / offsets_per_bundle, group = bundle / bundles_per_group, q = bundle % bundles_per_group;
    const size_t block_stride = (size_t)bundles_per_group * kTile * co;
    const float *src = partial + (size_t)group * blocks_per_group * block_stride +
                       ((size_t)q * kTile + (size_t)(k % offsets_per_bundle) * ci + c) * co + n;
    float v = 0.0f;
    for (int b = 0; b < blocks_per_group; ++b) v += src[(size_t)b * block_stride];
    filters_grad[i] = __float2half_rn(v);
  }
}

template <int CI, int CO>
cudaError_t launchGradTc(const FilterGradProblem &p, const FilterGradTcPlan &plan, const __half *features,
                         const __half *output_grad, const int32_t *nbr, float *partial, int32_t *status,
                         double bytes, double flops, cudaStream_t stream) {
  using Cfg = GradTcConfig<CI, CO>;
  auto kernel = filterGradTcgen05Kernel<CI, CO>;
  cudaError_t err =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::kSmemBytes);
  if (err != cudaSuccess) return err;
  static const std::string name = "filterGradTcgen05Kernel<" + std::to_string(CI) + "," + std::to_string(CO) + ">";
  trace::Scope t(name.c_str(), stream, bytes, flops);
  // Test hook: MLUOP_B200_TEST_FILTER_GRAD_WAIT=<cycles> gives every wait that limit and withholds one
  // stage release per block, so that the producers' bounded wait runs out: the kernel must record the
  // error, leave through its common exit (copies drained, MMAs seen out, tensor memory freed) and
  // return.  Nothing faults or spins on.
  long long wait_limit = kWaitCycles;
  int test_drop_release = 0;
  if (const char *hook = std::getenv("MLUOP_B200_TEST_FILTER_GRAD_WAIT")) {
    const long long cycles = std::atoll(hook);
    if (cycles > 0) {
      wait_limit = cycles;
      test_drop_release = 1;
    }
  }
  kernel<<<(unsigned)(plan.groups * plan.blocks_per_group), kThreads, Cfg::kSmemBytes, stream>>>(
      features, output_grad, nbr, p.n_out, plan.n_pad, p.K, plan.bundles_per_group, plan.blocks_per_group, partial,
      status, p.sticky_status, wait_limit, test_drop_release);
  return cudaGetLastError();
}

// bundles a group may hold for this shape (tensor-memory columns, table entries in registers)
int maxBundlesPerGroup(int ci, int co) {
  const int by_tmem = 512 / co, by_regs = kMaxGroupOffsets / (kTile / ci);
  return by_tmem < by_regs ? by_tmem : by_regs;
}

}  // namespace

bool filterGradTcShapeEligible(const FilterGradProblem &p) {
  const char *forced = std::getenv("MLUOP_B200_FILTER_GRAD_KERNEL");  // read per call: tests switch it
  const std::string choice = forced ? forced : "";
  if (choice == "mma") return false;
  // 32 input channels run correctly but slower than the pair-list kernel (0.79 vs 0.56 ms for the two
  // 32->32 layers of the c2 backbone: an item costs the same hand-offs for half the arithmetic), so they
  // take this kernel only on request.
  const bool wide = p.ci == 64 && (p.co == 64 || p.co == 128);
  const bool narrow = p.ci == 32 && (p.co == 32 || p.co == 64) && choice == "tcgen05";
  return p.is_half && (wide || narrow) && p.K >= 1 && p.K <= 128 && p.n_out >= 1 && neighbourTableCountsFit(p.K);
}

FilterGradTcPlan planFilterGradTc(const FilterGradProblem &p, int sm_count) {
  FilterGradTcPlan plan{};
  const int sms = sm_count > 0 ? sm_count : 148;
  // as few groups as the kernel allows, the bundles spread evenly over them
  const int offsets_per_bundle = kTile / p.ci;
  const int bundles = (p.K + offsets_per_bundle - 1) / offsets_per_bundle;
  const int max_per_group = maxBundlesPerGroup(p.ci, p.co);
  plan.groups = (bundles + max_per_group - 1) / max_per_group;
  plan.bundles_per_group = (bundles + plan.groups - 1) / plan.groups;
  const int64_t tiles = (p.n_out + kTile - 1) / kTile;
  int64_t per_group = sms / plan.groups;
  if (per_group < 1) per_group = 1;
  if (per_group > tiles) per_group = tiles;
  plan.blocks_per_group = (int32_t)per_group;
  plan.n_pad = (p.n_out + kConvPadRows - 1) / kConvPadRows * kConvPadRows;
  plan.table_bytes = (size_t)p.K * plan.n_pad * sizeof(int32_t);
  plan.partial_bytes =
      (size_t)plan.groups * plan.blocks_per_group * plan.bundles_per_group * kTile * p.co * sizeof(float);
  return plan;
}

cudaError_t launchFilterGradTcgen05(const FilterGradProblem &p, const FilterGradTcPlan &plan, const void *features,
                                    const void *output_grad, const int32_t *indice_pairs,
                                    const int64_t *indice_num, int32_t *table, float *partial, int32_t *status,
                                    void *filters_grad, int sm_count, double bytes, double flops,
                                    cudaStream_t stream, const int32_t *external_table) {
  // 1. the forward convolution's neighbour table: the caller's, or built from the pair lists
  cudaError_t err = cudaSuccess;
  if (external_table != nullptr) {
    table = const_cast<int32_t *>(external_table);
  } else {
    ConvProblem cp{};
    cp.L = p.L;
    cp.n_out = p.n_out;
    cp.K = p.K;
    cp.ci = p.ci;
    cp.co = p.co;
    cp.is_half = 1;
    cp.sticky_status = p.sticky_status;
    const ConvWorkspacePlan conv_plan = planConvWorkspace(cp, /*external_table=*/true);
    err = launchIndiceConvolutionSteps(cp, conv_plan, nullptr, nullptr, indice_pairs, indice_num, nullptr, nullptr,
                                       sm_count, stream, table, kTableBuildOnly);
    if (err != cudaSuccess) return err;
  }
  if ((err = cudaMemsetAsync(status, 0, sizeof(int32_t), stream)) != cudaSuccess) return err;
  // 2. partial sums of every block
  const __half *f = static_cast<const __half *>(features);
  const __half *g = static_cast<const __half *>(output_grad);
  if (p.ci == 64 && p.co == 64) {
    err = launchGradTc<64, 64>(p, plan, f, g, table, partial, status, bytes, flops, stream);
  } else if (p.ci == 64) {
    err = launchGradTc<64, 128>(p, plan, f, g, table, partial, status, bytes, flops, stream);
  } else if (p.co == 32) {
    err = launchGradTc<32, 32>(p, plan, f, g, table, partial, status, bytes, flops, stream);
  } else {
    err = launchGradTc<32, 64>(p, plan, f, g, table, partial, status, bytes, flops, stream);
  }
  if (err != cudaSuccess) return err;
  // 3. blocks of a group added in a fixed order
  const int64_t total = (int64_t)p.K * p.ci * p.co;
  const unsigned blocks = (unsigned)((total + 255) / 256 < 2048 ? (total + 255) / 256 : 2048);
  trace::Scope t("reduceFilterGradTcKernel", stream, (double)plan.partial_bytes + 2.0 * (double)total);
  reduceFilterGradTcKernel<<<blocks, 256, 0, stream>>>(partial, p.K, p.ci, p.co, plan.bundles_per_group,
                                                       plan.blocks_per_group, static_cast<__half *>(filters_grad));
  return cudaGetLastError();
}

}  // namespace sparse_conv
}  // namespace mluop
