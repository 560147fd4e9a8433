// Filter gradient of the sparse convolution on the 5th-generation tensor cores
// (tcgen05) of sm_100a: half inputs with 64 input channels, fp32 accumulation in
// tensor memory.
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
// Work split.  Two offsets share one accumulator of 128 lanes (lanes 0-63: the 64
// input channels of offset 2q, lanes 64-127: those of offset 2q+1) and Co
// columns; 512 columns of tensor memory hold 512/Co such pairs, so the offsets
// are cut into groups of that many pairs and a block serves one group.  The
// blocks of a group (one per SM) take the tiles of 128 output rows round-robin.
//
// Per tile the eight producer warps copy the tile's output_grad rows to shared
// memory once (contiguous rows, cp.async) and, for every pair with at least one
// live row in the tile, gather the feature rows of its two offsets into a stage
// of the ring (rows without a neighbour are zero-filled, nothing is fetched).
// Both operands lie row-major in shared memory - the contracted axis (rows) is
// the slow one - which tcgen05.mma reads as "MN-major" operands: one elected
// thread issues 8 MMAs (M=128, N=Co, K=16 rows each) per pair and tile and
// releases the stage with tcgen05.commit.  Producers, issuer and epilogue each
// derive which pairs are live from the table itself (a warp reads the tile's
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
constexpr int kCi = 64;               // input channels (one 128-byte swizzle atom per row)
constexpr int kProducerWarps = 8;      // warps 0-7: gather; warps 0-3 also read the sums back
constexpr int kProducerThreads = kProducerWarps * 32;
constexpr int kIssuerWarp = kProducerWarps;  // tensor-memory allocation and MMA issue
constexpr int kThreads = kProducerThreads + 32;
constexpr int kSubTileBytes = kTile * kCi * 2;  // [128 rows][64 halfs], rows 128 bytes apart
constexpr int kTmemCols = 512;
constexpr long long kWaitCycles = 2000000000ll;  // a wait gives up after about one second
constexpr int kErrProducerStage = 1, kErrIssuerStage = 2, kErrAccum = 4, kErrGradTile = 8, kErrIssuerGrad = 16;

template <int CO>
struct GradTcConfig {
  static constexpr int kPairsPerGroup = kTmemCols / CO;  // accumulators of 128 lanes x CO columns
  static constexpr int kOffsetsPerGroup = 2 * kPairsPerGroup;
  // as many stages as shared memory holds: the gathers are latency-bound, what counts is bytes in flight
  static constexpr int kAStages = CO == 64 ? 6 : 5;
  static constexpr int kAStageBytes = 2 * kSubTileBytes;         // the gathered rows of two offsets
  static constexpr int kGradBufBytes = (CO / 64) * kSubTileBytes;  // one tile of output_grad rows
  static constexpr int kGradBufs = 2;
  static constexpr size_t kSmemBytes = 1024 + (size_t)kAStages * kAStageBytes + (size_t)kGradBufs * kGradBufBytes;
  // D fp32, A and B fp16, both MN-major (bits 15 and 16), N = CO, M = 128
  static constexpr unsigned kIdesc =
      (1u << 4) | (1u << 15) | (1u << 16) | ((unsigned)(CO >> 3) << 17) | ((unsigned)(kTile >> 4) << 24);
};

// Descriptor of an MN-major operand with the 128-byte swizzle: 64 elements of the
// M (or N) axis are contiguous (one 128-byte row per step of the contracted axis),
// groups of 8 such rows are 1024 bytes apart (stride byte offset) and the next 64
// elements of the M/N axis start `atom_stride` bytes further (leading byte offset).
__device__ __forceinline__ unsigned long long makeDescMn(unsigned smem_byte_addr, unsigned atom_stride) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_byte_addr & 0x3FFFFu) >> 4);
  d |= (unsigned long long)(atom_stride >> 4) << 16;
  d |= (unsigned long long)(1024u >> 4) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
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

template <int CO>
__global__ void __launch_bounds__(kThreads, 1)
filterGradTcgen05Kernel(const __half *__restrict__ features, const __half *__restrict__ output_grad,
                        const int32_t *__restrict__ nbr, int64_t n_out, int64_t n_pad, int K, int pairs_per_group,
                        int blocks_per_group, float *__restrict__ partial, int32_t *status_word, int32_t *sticky, long long wait_limit) {
  using Cfg = GradTcConfig<CO>;
  constexpr int S = Cfg::kAStages, NG = Cfg::kGradBufs, PPG = Cfg::kPairsPerGroup, OPG = Cfg::kOffsetsPerGroup;
  constexpr int kGradChunks = CO / 8;  // 16-byte chunks of one output_grad row
  extern __shared__ unsigned char smem_raw[];
  unsigned char *a_ring = reinterpret_cast<unsigned char *>((reinterpret_cast<size_t>(smem_raw) + 1023) & ~(size_t)1023);
  unsigned char *g_ring = a_ring + (size_t)S * Cfg::kAStageBytes;
  __shared__ unsigned long long a_full[S], a_empty[S], g_full[NG], g_empty[NG], accum_bar, drain_bar;
  __shared__ unsigned tmem_base_s;
  __shared__ int abort_s;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = blockIdx.x / blocks_per_group, member = blockIdx.x % blocks_per_group;
  // the group's offsets: pairs_per_group (<= PPG) pairs from offset k0 on
  const int k0 = group * 2 * pairs_per_group;
  const int k_end = K < k0 + 2 * pairs_per_group ? K : k0 + 2 * pairs_per_group;
  const int64_t n_tiles = (n_out + kTile - 1) / kTile;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbarInit(&a_full[s], kProducerThreads);
      mbarInit(&a_empty[s], 1);
    }
    for (int g = 0; g < NG; ++g) {
      mbarInit(&g_full[g], kProducerThreads);
      mbarInit(&g_empty[g], 1);
    }
    mbarInit(&accum_bar, 1);
    mbarInit(&drain_bar, 1);
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
    // with (four warps, one per scheduler, ran at a fifth of the issue rate and the kernel
    // was bound by that, not by the copies or the MMAs).  Warp w gathers rows 16w..16w+15 of
    // both offsets of a pair: lane l holds the table entry of row 16w + (l & 15) for offset
    // 2q + (l >> 4) and hands it to the lanes that fetch that row by shuffle; consecutive
    // lanes fetch consecutive 16-byte chunks of a feature row (8 per row), so one warp
    // instruction touches four rows.
    const int rr0 = lane >> 3, chunk = lane & 7;
    const int my_row = warp * 16 + (lane & 15), my_half = lane >> 4;
    unsigned a_off[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = warp * 16 + rr0 + i * 4;
      unsigned off = (unsigned)(row * 128 + chunk * 16);
      off ^= ((off >> 7) & 7u) << 4;
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
          unsigned off = (unsigned)(row * 128 + (c & 7) * 16);
          off ^= ((off >> 7) & 7u) << 4;
          const bool valid = row0 + row < n_out;
          cpAsync16(g_addr + (unsigned)(c >> 3) * kSubTileBytes + off,
                    output_grad + (valid ? (size_t)(row0 + row) * CO + c * 8 : 0), valid);
        }
      }
      cpAsyncArriveOn(&g_full[g]);
      // the gathered feature rows of every live pair
      // (a real loop: unrolled over the pairs its body no longer fits the instruction cache)
      unsigned todo = (live | (live >> 1)) & 0x55555555u;  // bit 2q: pair q has a live offset
#pragma unroll 1
      while (todo && ok) {
        const int q = (__ffs(todo) - 1) >> 1;
        todo &= todo - 1u;
        // this lane's table entry: row 16w + (l & 15) of offset 2q + (l >> 4); the line is in L1 since the vote
        const int k = k0 + 2 * q + my_half;
        const int idx = k < k_end ? __ldg(nbr + (size_t)k * n_pad + row0 + my_row) : -1;
        if (items >= (unsigned)S) {
          if (!mbarWaitWarp(&a_empty[s], a_parity ^ 1u, abort_flag, status, kErrProducerStage, wait_limit)) {
            ok = false;
            continue;
          }
        }
        const unsigned stage_addr = a_ring_addr + (unsigned)s * Cfg::kAStageBytes;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int src_row = __shfl_sync(0xffffffffu, idx, h * 16 + rr0 + i * 4);
            const bool valid = src_row >= 0;
            cpAsync16(stage_addr + (unsigned)h * kSubTileBytes + a_off[i], feat_chunk + (valid ? (size_t)src_row * kCi : 0),
                      valid);
          }
        }
        cpAsyncArriveOn(&a_full[s]);
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
      float *dst_block = partial + (size_t)blockIdx.x * pairs_per_group * kTile * CO;
#pragma unroll 1
      for (int q = 0; q < pairs_per_group; ++q) {
        const bool touched = have_acc && ((ever_live >> (2 * q)) & 3u);
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
    // ------------------------------------------------------------ MMA issuer
    // The whole warp derives the live pairs of a tile; lane 0 issues.
    const unsigned long long a_desc0 = makeDescMn(smemAddr(a_ring), kSubTileBytes);
    const unsigned long long g_desc0 = makeDescMn(smemAddr(g_ring), kSubTileBytes);
    unsigned started = 0u;  // pairs whose accumulator has been written
    int s = 0;
    unsigned a_parity = 0, items = 0;
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
        for (int q = 0; q < PPG && ok; ++q) {
          if (!((live >> (2 * q)) & 3u)) continue;
          if (!mbarWait(&a_full[s], a_parity, abort_flag, status, kErrIssuerStage, wait_limit)) {
            ok = false;
            break;
          }
          fenceProxyAsync();
          tcFenceAfter();
          const unsigned long long a_desc = a_desc0 + (unsigned long long)((s * Cfg::kAStageBytes) >> 4);
          const unsigned d_addr = tmem_base + (unsigned)(q * CO);
#pragma unroll
          for (int j = 0; j < kTile / 16; ++j) {
            // 16 rows of the contracted axis per MMA: 2048 bytes further in both operands
            umma(d_addr, a_desc + (unsigned long long)((j * 2048) >> 4), g_desc + (unsigned long long)((j * 2048) >> 4),
                 Cfg::kIdesc, (((started >> q) & 1u) || j > 0) ? 1u : 0u);
          }
          started |= 1u << q;
          ummaCommit(&a_empty[s]);
          ++items;
          if (++s == S) {
            s = 0;
            a_parity ^= 1u;
          }
        }
        // the tile's output_grad rows are free once the MMAs issued so far are done
        if (ok) ummaCommit(&g_empty[g]);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    }
    if (lane == 0) {
      if (ok && items > 0 && !*abort_flag) {
        ummaCommit(&accum_bar);
      } else if (items > 0) {
        // leaving early: see the outstanding MMAs out before tensor memory is freed
        ummaCommit(&drain_bar);
        const long long t0 = clock64();
        while (!mbarTryWait(&drain_bar, 0) && clock64() - t0 <= wait_limit) {
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
// order, of partial[block][pair of k][lane (k & 1) * 64 + c][n].
__global__ void __launch_bounds__(256)
reduceFilterGradTcKernel(const float *__restrict__ partial, int K, int co, int pairs_per_group, int blocks_per_group,
                         __half *__restrict__ filters_grad) {
  const int64_t total = (int64_t)K * kCi * co;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int n = (int)(i % co);
    const int c = (int)((i / co) % kCi);
    const int k = (int)(i / ((int64_t)co * kCi));
    const int pair = k >> 1, group = pair / pairs_per_group, q = pair % pairs_per_group;
    const size_t block_stride = (size_t)pairs_per_group * kTile * co;
    const float *src = partial + (size_t)group * blocks_per_group * block_stride +
                       ((size_t)q * kTile + (size_t)(k & 1) * kCi + c) * co + n;
    float v = 0.0f;
    for (int b = 0; b < blocks_per_group; ++b) v += src[(size_t)b * block_stride];
    filters_grad[i] = __float2half_rn(v);
  }
}

template <int CO>
cudaError_t launchGradTc(const FilterGradProblem &p, const FilterGradTcPlan &plan, const __half *features,
                         const __half *output_grad, const int32_t *nbr, float *partial, int32_t *status,
                         double bytes, double flops, cudaStream_t stream) {
  using Cfg = GradTcConfig<CO>;
  auto kernel = filterGradTcgen05Kernel<CO>;
  cudaError_t err =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::kSmemBytes);
  if (err != cudaSuccess) return err;
  static const std::string name = "filterGradTcgen05Kernel<64," + std::to_string(CO) + ">";
  trace::Scope t(name.c_str(), stream, bytes, flops);
  kernel<<<(unsigned)(plan.groups * plan.blocks_per_group), kThreads, Cfg::kSmemBytes, stream>>>(
      features, output_grad, nbr, p.n_out, plan.n_pad, p.K, plan.pairs_per_group, plan.blocks_per_group, partial, status, p.sticky_status,
      kWaitCycles);
  return cudaGetLastError();
}

}  // namespace

bool filterGradTcShapeEligible(const FilterGradProblem &p) {
  const char *forced = std::getenv("MLUOP_B200_FILTER_GRAD_KERNEL");  // read per call: tests switch it
  if (forced && std::string(forced) == "mma") return false;
  return p.is_half && p.ci == kCi && (p.co == 64 || p.co == 128) && p.K >= 1 && p.K <= 128 && p.n_out >= 1 &&
         neighbourTableCountsFit(p.K);
}

FilterGradTcPlan planFilterGradTc(const FilterGradProblem &p, int sm_count) {
  FilterGradTcPlan plan{};
  const int sms = sm_count > 0 ? sm_count : 148;
  // as few groups as tensor memory allows, the pairs spread evenly over them
  const int max_pairs_per_group = kTmemCols / p.co;
  const int pairs = (p.K + 1) / 2;
  plan.groups = (pairs + max_pairs_per_group - 1) / max_pairs_per_group;
  plan.pairs_per_group = (pairs + plan.groups - 1) / plan.groups;
  const int64_t tiles = (p.n_out + kTile - 1) / kTile;
  int64_t per_group = sms / plan.groups;
  if (per_group < 1) per_group = 1;
  if (per_group > tiles) per_group = tiles;
  plan.blocks_per_group = (int32_t)per_group;
  plan.n_pad = (p.n_out + kConvPadRows - 1) / kConvPadRows * kConvPadRows;
  plan.table_bytes = (size_t)p.K * plan.n_pad * sizeof(int32_t);
  plan.partial_bytes =
      (size_t)plan.groups * plan.blocks_per_group * plan.pairs_per_group * kTile * p.co * sizeof(float);
  return plan;
}

cudaError_t launchFilterGradTcgen05(const FilterGradProblem &p, const FilterGradTcPlan &plan, const void *features,
                                    const void *output_grad, const int32_t *indice_pairs,
                                    const int64_t *indice_num, int32_t *table, float *partial, int32_t *status,
                                    void *filters_grad, int sm_count, double bytes, double flops,
                                    cudaStream_t stream) {
  // 1. the forward convolution's neighbour table, from the pair lists
  ConvProblem cp{};
  cp.L = p.L;
  cp.n_out = p.n_out;
  cp.K = p.K;
  cp.ci = p.ci;
  cp.co = p.co;
  cp.is_half = 1;
  cp.sticky_status = p.sticky_status;
  const ConvWorkspacePlan conv_plan = planConvWorkspace(cp, /*external_table=*/true);
  cudaError_t err = launchIndiceConvolutionSteps(cp, conv_plan, nullptr, nullptr, indice_pairs, indice_num, nullptr,
                                                 nullptr, sm_count, stream, table, kTableBuildOnly);
  if (err != cudaSuccess) return err;
  if ((err = cudaMemsetAsync(status, 0, sizeof(int32_t), stream)) != cudaSuccess) return err;
  // 2. partial sums of every block
  const __half *f = static_cast<const __half *>(features);
  const __half *g = static_cast<const __half *>(output_grad);
  if (p.co == 64) {
    err = launchGradTc<64>(p, plan, f, g, table, partial, status, bytes, flops, stream);
  } else {
    err = launchGradTc<128>(p, plan, f, g, table, partial, status, bytes, flops, stream);
  }
  if (err != cudaSuccess) return err;
  // 3. blocks of a group added in a fixed order
  const int64_t total = (int64_t)p.K * p.ci * p.co;
  const unsigned blocks = (unsigned)((total + 255) / 256 < 2048 ? (total + 255) / 256 : 2048);
  trace::Scope t("reduceFilterGradTcKernel", stream, (double)plan.partial_bytes + 2.0 * (double)total);
  reduceFilterGradTcKernel<<<blocks, 256, 0, stream>>>(partial, p.K, p.co, plan.pairs_per_group,
                                                       plan.blocks_per_group, static_cast<__half *>(filters_grad));
  return cudaGetLastError();
}

}  // namespace sparse_conv
}  // namespace mluop
