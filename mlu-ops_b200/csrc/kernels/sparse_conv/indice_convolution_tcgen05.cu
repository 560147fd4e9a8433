// Sparse convolution forward on the 5th-generation tensor cores (tcgen05) of
// sm_100a: half inputs, fp32 accumulation in tensor memory.
//
// One thread block owns a few consecutive tiles of 128 output rows and keeps
// one [128 x Co] fp32 accumulator per tile in TMEM for the whole kernel.  It
// walks the kernel offsets in ascending order; for each offset k the filter
// slice W_k ([Co x Ci], Ci contiguous) arrives in shared memory by ONE bulk copy
// (the repacked filter is the byte image of the operand, swizzle included) and is
// reused by all tiles of the block, and for every tile with at least one live
// row at k (a per-tile bit mask the block derives from the neighbour table)
//   * four producer warps (one thread per output row) gather the input rows
//     named by the neighbour table into a shared-memory A tile with cp.async
//     (16-byte chunks; rows without a neighbour are zero-filled, nothing is
//     fetched for them); A and W_k are written in the K-major swizzled layout
//     tcgen05.mma reads;
//   * one elected thread issues Ci/16 tcgen05.mma instructions (M=128, N=Co,
//     K=16) that accumulate into the tile's TMEM columns, then tcgen05.commit
//     releases the stage (and, after the last tile of k, the filter buffer).
// Stages form a ring guarded by mbarriers (full: one arrival per producer thread,
// delivered by cp.async.mbarrier.arrive when that thread's copies have landed;
// empty: one arrival from tcgen05.commit).  After the last offset the producer warps read the
// accumulators back with tcgen05.ld, round to half and store each output row
// once.  The reduction over offsets happens in TMEM in a fixed order, so the
// result is deterministic.
//
// Every mbarrier wait is bounded: after about one second the waiter records an
// error in the status word, raises a block-wide abort flag and every role
// falls through to the common exit, where outstanding cp.async groups are
// drained (cp.async.wait_all) and TMEM is freed.  The host side reports a non-zero status word as
// MLUOP_STATUS_EXECUTION_FAILED when asked to check it.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <string>

#include "core/trace.h"
#include "kernels/sparse_conv/indice_convolution_kernels.h"
#include "kernels/sparse_conv/indice_convolution_tcgen05.h"
#include "kernels/sparse_conv/tcgen05_primitives.cuh"

namespace mluop {
namespace sparse_conv {

namespace {

constexpr int kTile = kConvTileRows;      // 128 output rows = 128 TMEM lanes
constexpr int kProducerThreads = 128;     // warps 0-3: gather, then epilogue
constexpr int kThreads = 160;             // + warp 4: TMEM allocation and MMA issue
constexpr int kMaxOffsets = 128;           // kernel volumes up to 5x5x5
constexpr int kMaskWords = kMaxOffsets / 32;
constexpr long long kWaitCycles = 2000000000ll;  // a wait gives up after about one second (default)

using namespace tc;

// Tile configuration.  A block owns TILES consecutive tiles of 128 output rows
// and one [128 x CO] fp32 accumulator per tile in tensor memory.
template <int CI, int CO>
struct TcConfig {
  // K is split into blocks of at most 64 halfs (128 bytes, one swizzle atom wide)
  static constexpr int kBlockK = CI < 64 ? CI : 64;
  static constexpr int kKBlocks = CI / kBlockK;
  static constexpr int kRowBytes = kBlockK * 2;                 // 32, 64 or 128
  static constexpr unsigned kSwizzleMask = kRowBytes / 16 - 1;  // 1, 3 or 7: XOR of 16-byte chunk index
  // tcgen05 shared-memory descriptor layout type: 128B = 2, 64B = 4, 32B = 6
  static constexpr unsigned long long kLayoutType = kRowBytes == 128 ? 2 : (kRowBytes == 64 ? 4 : 6);
  static constexpr int kABlockBytes = kTile * kRowBytes;
  static constexpr int kBBlockBytes = CO * kRowBytes;
  static constexpr int kBBlockStride = (kBBlockBytes + 1023) / 1024 * 1024;
  static constexpr int kAStageBytes = kKBlocks * kABlockBytes;  // one gathered [128 x CI] tile
  static constexpr int kBBufBytes = kKBlocks * kBBlockStride;   // one filter slice W_k [CO x CI]
  static constexpr int kTiles = 2;                              // tiles per block
  static constexpr int kTmemCols = kTiles * CO < 32 ? 32 : kTiles * CO;  // 64, 128 or 256
  static constexpr int kBlocksPerSmByTmem = 512 / kTmemCols;
  // filter slices and gathered tiles in flight; sized so that as many blocks share an SM as
  // tensor memory allows (128 input channels: 2 x 32 KB tiles + one 32 KB slice = two blocks
  // per SM, which hides more latency than a third stage and a second slice in one block)
  static constexpr int kBBuffers = CI >= 128 ? 1 : 2;
  static constexpr int kAStages = 2;
  static constexpr int kChunksPerRow = CI / 8;  // 16-byte chunks of one feature row
  // instruction descriptor: D fp32, A and B fp16, both K-major, N = CO, M = 128
  static constexpr unsigned kIdesc = (1u << 4) | ((unsigned)(CO >> 3) << 17) | ((unsigned)(kTile >> 4) << 24);
  static constexpr size_t kOperandBytes = (size_t)kAStages * kAStageBytes + (size_t)kBBuffers * kBBufBytes;
  // Dynamic shared memory: operands (+ alignment slack), raised where needed so
  // that no more blocks fit on an SM than tensor memory has columns for.
  static size_t smemBytes() {
    size_t need = 1024 + kOperandBytes;
    const size_t per_block_floor = (size_t)(227 * 1024) / (kBlocksPerSmByTmem + 1) + 1024;
    return need > per_block_floor ? need : per_block_floor;
  }
};

// Descriptor of a K-major swizzled operand block whose rows are kRowBytes apart:
// start address, stride between 8-row groups (8 * kRowBytes), descriptor version 1.
template <typename Cfg>
__device__ __forceinline__ unsigned long long makeDesc(unsigned smem_byte_addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_byte_addr & 0x3FFFFu) >> 4);
  d |= (unsigned long long)((8u * Cfg::kRowBytes) >> 4) << 32;
  d |= 1ull << 46;
  d |= Cfg::kLayoutType << 61;
  return d;
}

// Work items of a block: (offset k ascending, tile t ascending) for which the
// tile has at least one live row at k.  The list is built once per block in
// shared memory, two bytes per item: bit 15 = first item of its offset, bits
// 2..14 = k, bits 0..1 = t.  Producers and the MMA issuer walk the same list.
constexpr int kMaxItems = 2 * kMaxOffsets;
constexpr unsigned kItemFirst = 0x8000u;
__device__ __forceinline__ int itemOffset(unsigned code) { return (int)((code >> 2) & 0x1FFFu); }
__device__ __forceinline__ int itemTile(unsigned code) { return (int)(code & 3u); }

template <int CI, int CO>
__global__ void __launch_bounds__(kThreads)
convTcgen05Kernel(const __half *__restrict__ features, const __half *__restrict__ filter_image,
                  const int32_t *__restrict__ nbr, int64_t n_out, int64_t n_pad, int K, int ci_real, int co_real,
                  __half *__restrict__ out, int32_t *status_word, int32_t *sticky, long long wait_limit,
                  int test_drop_release, int mirror) {
  using Cfg = TcConfig<CI, CO>;
  constexpr int S = Cfg::kAStages, NB = Cfg::kBBuffers, T = Cfg::kTiles;
  constexpr int CPR = Cfg::kChunksPerRow;  // 16-byte chunks per feature row
  extern __shared__ unsigned char smem_raw[];
  // operand blocks must sit on 1024-byte boundaries (swizzle atoms)
  unsigned char *a_ring = reinterpret_cast<unsigned char *>((reinterpret_cast<size_t>(smem_raw) + 1023) & ~(size_t)1023);
  unsigned char *b_ring = a_ring + (size_t)S * Cfg::kAStageBytes;
  __shared__ unsigned long long a_full[S], a_empty[S], b_full[NB], b_empty[NB], accum_bar, drain_bar;
  __shared__ unsigned tmem_base_s;
  static_assert(T <= 2, "kMaxItems holds two tiles per offset");
  __shared__ unsigned masks_s[T][kMaskWords];
  __shared__ unsigned short items_s[kMaxItems];
  __shared__ int n_items_s;
  __shared__ int abort_s;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t row0 = (int64_t)blockIdx.x * (T * kTile);

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbarInit(&a_full[s], kProducerThreads);
      mbarInit(&a_empty[s], 1);
    }
    for (int b = 0; b < NB; ++b) {
      mbarInit(&b_full[b], 1);
      mbarInit(&b_empty[b], 1);
    }
    mbarInit(&accum_bar, 1);
    mbarInit(&drain_bar, 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (tid < T * kMaskWords) masks_s[tid / kMaskWords][tid % kMaskWords] = 0u;
  if (warp == 4) tmemAlloc(&tmem_base_s, Cfg::kTmemCols);
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  // Live masks: bit k of masks_s[t] is set when some row of tile t has a
  // neighbour at offset k.  Each warp scans (offset, tile) slices of the table,
  // four rows per lane.
  // (eight slices' loads are issued before the first vote, so a warp pays the memory latency
  // once per eight slices, not once per slice)
  for (int e0 = warp; e0 < K * T; e0 += 8 * (kThreads / 32)) {
    int4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int e = e0 + u * (kThreads / 32);
      v[u] = make_int4(-1, -1, -1, -1);
      // (mirror: offset k reads table row K-1-k, see launchConvTcgen05)
      if (e < K * T) {
        const int row_k = mirror ? K - 1 - e / T : e / T;
        v[u] = __ldg(reinterpret_cast<const int4 *>(nbr + (size_t)row_k * n_pad + row0 + (e % T) * kTile) + lane);
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int e = e0 + u * (kThreads / 32);
      const unsigned any = __ballot_sync(0xffffffffu, (v[u].x & v[u].y & v[u].z & v[u].w) >= 0);
      if (lane == 0 && any && e < K * T) atomicOr(&masks_s[e % T][(e / T) >> 5], 1u << ((e / T) & 31));
    }
  }
  __syncthreads();
  if (tid == 0) {
    int n = 0;
    for (int k = 0; k < K; ++k) {
      unsigned first = kItemFirst;
      for (int t = 0; t < T; ++t) {
        if ((masks_s[t][k >> 5] >> (k & 31)) & 1u) {
          items_s[n++] = (unsigned short)(first | (unsigned)(k << 2) | (unsigned)t);
          first = 0u;
        }
      }
    }
    n_items_s = n;
  }
  __syncthreads();
  const int n_items = n_items_s;
  const unsigned tmem_base = tmem_base_s;
  volatile int *abort_flag = &abort_s;
  const ErrorSink status{status_word, sticky};

  if (warp < 4) {
    // ------------------------------------------------------------ producers
    // Warp w gathers rows 32w..32w+31 of every tile; lane l holds the neighbour
    // id of row 32w+l and hands it to the lanes that fetch that row by shuffle.
    // Consecutive lanes fetch consecutive 16-byte chunks of one feature row, so a
    // warp instruction touches 32/CPR rows.  Every byte of a stage is written by
    // cp.async (zero fill for rows without a neighbour: nothing is read), and
    // each thread lets the stage's mbarrier collect one arrival when its own
    // copies have landed, so producers never wait for data: as many gathers are
    // in flight as there are stages.
    constexpr int kRowsPerInstr = 32 / CPR > 0 ? 32 / CPR : 1;  // rows one warp instruction covers (CPR <= 32)
    const int rr0 = lane / CPR;         // row (within the instruction's rows) this lane fetches
    const int chunk = lane % CPR;       // its 16-byte chunk of the row
    unsigned a_off[CPR];                // byte offset of (row, chunk) inside a stage, swizzled
#pragma unroll
    for (int i = 0; i < CPR; ++i) {
      const int row = warp * 32 + rr0 + i * kRowsPerInstr;
      const int kb = chunk / (Cfg::kRowBytes / 16), cc = chunk % (Cfg::kRowBytes / 16);
      unsigned off = (unsigned)(row * Cfg::kRowBytes + cc * 16);
      off ^= ((off >> 7) & Cfg::kSwizzleMask) << 4;
      a_off[i] = (unsigned)(kb * Cfg::kABlockBytes) + off;
    }
    const unsigned a_ring_addr = smemAddr(a_ring);
    const __half *feat_chunk = features + chunk * 8;
    const bool chunk_in_row = chunk * 8 < ci_real;  // channels past ci_real are zero fill (padded Ci)
    const int32_t *nbr_rows = nbr + row0 + tid;

    int s = 0, b = -1;
    unsigned a_parity = 0, b_uses = 0;  // a_parity: parity of the current pass over the stage ring
    int idx_next = -1;
    if (n_items > 0) {
      const unsigned c0 = items_s[0];
      idx_next = __ldg(nbr_rows + (size_t)(mirror ? K - 1 - itemOffset(c0) : itemOffset(c0)) * n_pad + itemTile(c0) * kTile);
    }
    for (int it = 0; it < n_items; ++it) {
      const unsigned code = items_s[it];
      const int idx = idx_next;
      if (it + 1 < n_items) {
        const unsigned c1 = items_s[it + 1];
        idx_next = __ldg(nbr_rows + (size_t)(mirror ? K - 1 - itemOffset(c1) : itemOffset(c1)) * n_pad + itemTile(c1) * kTile);
      }
      if (it >= S) {
        if (!mbarWaitWarp(&a_empty[s], a_parity ^ 1u, abort_flag, status, 1, wait_limit)) break;
      }
      if (code & kItemFirst) {
        // The filter slice of offset k: one bulk copy of its shared-memory image, issued by one
        // thread of warp 0 once the MMAs that read the buffer's previous slice are done; its
        // bytes are counted by b_full[b], which the issuer waits for.
        if (++b == NB) b = 0;
        if (warp == 0) {
          if (b_uses >= (unsigned)NB) {
            if (!mbarWaitWarp(&b_empty[b], ((b_uses / NB) - 1u) & 1u, abort_flag, status, 8, wait_limit)) break;
          }
          if (lane == 0) {
            mbarArriveExpectTx(&b_full[b], (unsigned)Cfg::kBBufBytes);
            bulkCopyToShared(smemAddr(b_ring + (size_t)b * Cfg::kBBufBytes),
                             reinterpret_cast<const unsigned char *>(filter_image) + (size_t)itemOffset(code) * Cfg::kBBufBytes,
                             (unsigned)Cfg::kBBufBytes, &b_full[b]);
          }
          __syncwarp();
        }
        ++b_uses;
      }
      const unsigned stage_addr = a_ring_addr + (unsigned)s * Cfg::kAStageBytes;
#pragma unroll
      for (int i = 0; i < CPR; ++i) {
        const int src_row = __shfl_sync(0xffffffffu, idx, rr0 + i * kRowsPerInstr);
        const bool valid = src_row >= 0 && chunk_in_row;
        cpAsync16(stage_addr + a_off[i], feat_chunk + (valid ? (size_t)src_row * ci_real : 0), valid);
      }
      cpAsyncArriveOn(&a_full[s]);
      if (++s == S) {
        s = 0;
        a_parity ^= 1u;
      }
    }
    cpAsyncWaitAll();
    if (tid == 0 && *abort_flag) {
      // leaving early: a bulk copy may still be writing a filter buffer; see it out (bounded)
      for (int i = 0; i < NB && (unsigned)i < b_uses; ++i) {
        const unsigned use = b_uses - 1u - (unsigned)i;  // the i-th last slice sent
        const long long t0 = clock64();
        while (!mbarTryWait(&b_full[use % NB], (use / NB) & 1u) && clock64() - t0 <= wait_limit) {
        }
      }
    }

    // ------------------------------------------------------------- epilogue
    bool have_acc = n_items > 0;
    if (have_acc) have_acc = mbarWaitWarp(&accum_bar, 0, abort_flag, status, 4, wait_limit);
    tcFenceAfter();
    if (!*abort_flag) {
#pragma unroll 1
      for (int t = 0; t < T; ++t) {
        const int64_t r = row0 + t * kTile + tid;
        unsigned live = 0u;
#pragma unroll
        for (int w = 0; w < kMaskWords; ++w) live |= masks_s[t][w];
        const bool tile_has_acc = have_acc && live != 0u;
        __half *dst = out + (size_t)r * co_real;
#pragma unroll
        for (int c0 = 0; c0 < CO; c0 += 16) {
          unsigned v[16];
          if (tile_has_acc) {
            tmemLoad16(tmem_base + ((unsigned)(warp * 32) << 16) + (unsigned)(t * CO + c0), v);
            tmemLoadWait();
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0u;
          }
          if (r < n_out) {
            __half2 h[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
              h[i] = __floats2half2_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
            // columns past co_real belong to the padding of Co
            if (c0 + 8 <= co_real) *reinterpret_cast<uint4 *>(dst + c0) = *reinterpret_cast<uint4 *>(&h[0]);
            if (c0 + 16 <= co_real) *reinterpret_cast<uint4 *>(dst + c0 + 8) = *reinterpret_cast<uint4 *>(&h[4]);
          }
        }
      }
    }
    tcFenceBefore();
  } else {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const unsigned long long a_desc0 = makeDesc<Cfg>(smemAddr(a_ring));
      const unsigned long long b_desc0 = makeDesc<Cfg>(smemAddr(b_ring));
      unsigned started = 0;  // tiles whose accumulator has been written
      unsigned b_firsts = 0;  // offsets begun so far
      int s = 0, b = -1;
      unsigned a_parity = 0;
      int it = 0;
      for (; it < n_items; ++it) {
        const unsigned code = items_s[it];
        const int t = itemTile(code);
        if (code & kItemFirst) {
          if (++b == NB) b = 0;
          if (!mbarWait(&b_full[b], (b_firsts / NB) & 1u, abort_flag, status, 16, wait_limit)) break;
          ++b_firsts;
        }
        if (!mbarWait(&a_full[s], a_parity, abort_flag, status, 2, wait_limit)) break;
        fenceProxyAsync();
        tcFenceAfter();
        // only the start-address field (16-byte units) differs between stages and K steps
        const unsigned long long a_desc = a_desc0 + (unsigned long long)((s * Cfg::kAStageBytes) >> 4);
        const unsigned long long b_desc = b_desc0 + (unsigned long long)((b * Cfg::kBBufBytes) >> 4);
        const unsigned d_addr = tmem_base + (unsigned)(t * CO);
#pragma unroll
        for (int j = 0; j < CI / 16; ++j) {
          constexpr int kStep = 32;  // bytes of K per MMA
          const int kb = (j * kStep) / Cfg::kRowBytes, within = (j * kStep) % Cfg::kRowBytes;
          umma(d_addr, a_desc + (unsigned long long)((kb * Cfg::kABlockBytes + within) >> 4),
               b_desc + (unsigned long long)((kb * Cfg::kBBlockStride + within) >> 4), Cfg::kIdesc,
               (((started >> t) & 1u) || j > 0) ? 1u : 0u);
        }
        started |= 1u << t;
        // the stage may be refilled once these MMAs have read it (test hook: the first release of a
        // block is withheld, so that the producers' wait for that stage runs out)
        if (!(test_drop_release && it == 0)) ummaCommit(&a_empty[s]);
        // last item of offset k: its filter slice is free once these MMAs are done
        if (it + 1 == n_items || (items_s[it + 1] & kItemFirst)) ummaCommit(&b_empty[b]);
        if (++s == S) {
          s = 0;
          a_parity ^= 1u;
        }
      }
      if (it == n_items && n_items > 0 && !*abort_flag) {
        ummaCommit(&accum_bar);
      } else if (it > 0) {
        // Leaving early: the MMAs issued so far may still be running, and tensor memory must not
        // be freed under them (the next block could be given the same columns).  One more
        // commit and one more bounded wait, whose outcome changes nothing, see them out.
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
  if (warp == 4) {
    tcFenceAfter();
    tmemDealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int CI, int CO>
cudaError_t launchTc(const ConvProblem &p, const ConvWorkspacePlan &plan, const __half *features,
                     const __half *filter, const int32_t *nbr, __half *out, int32_t *status, double algo_bytes,
                     double algo_flops, cudaStream_t stream) {
  using Cfg = TcConfig<CI, CO>;
  auto kernel = convTcgen05Kernel<CI, CO>;
  const size_t smem = Cfg::smemBytes();
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) return err;
  const unsigned blocks = (unsigned)(plan.n_pad / (Cfg::kTiles * kTile));
  // the input gradient runs the same kernel; its launches are listed apart in the trace
  static const std::string name = "convTcgen05Kernel<" + std::to_string(CI) + "," + std::to_string(CO) + ">";
  static const std::string name_dgrad = name + ":input_grad";
  trace::Scope t(p.backward_data ? name_dgrad.c_str() : name.c_str(), stream, algo_bytes, algo_flops);
  // Test hook: MLUOP_B200_TEST_CONV_WAIT=<cycles> gives every wait that limit and withholds the
  // first stage release of every block, so that the producers' bounded wait runs out: the kernel
  // must record the error, leave through its common exit (copies drained, tensor memory freed) and
  // return.  Nothing faults or spins on.
  long long wait_limit = kWaitCycles;
  int test_drop_release = 0;
  if (const char *hook = std::getenv("MLUOP_B200_TEST_CONV_WAIT")) {
    const long long cycles = std::atoll(hook);
    if (cycles > 0) {
      wait_limit = cycles;
      test_drop_release = 1;
    }
  }
  kernel<<<blocks, kThreads, smem, stream>>>(features, filter, nbr, p.n_out, plan.n_pad, p.K, p.ci, p.co, out, status,
                                             p.sticky_status, wait_limit, test_drop_release, p.mirror_table);
  return cudaGetLastError();
}

template <int CI>
cudaError_t dispatchCo(const ConvProblem &p, const ConvWorkspacePlan &plan, const __half *features,
                       const __half *filter, const int32_t *nbr, __half *out, int32_t *status, double algo_bytes,
                       double algo_flops, cudaStream_t stream) {
  switch (tcgen05PaddedChannels(p.co)) {
    case 16: return launchTc<CI, 16>(p, plan, features, filter, nbr, out, status, algo_bytes, algo_flops, stream);
    case 32: return launchTc<CI, 32>(p, plan, features, filter, nbr, out, status, algo_bytes, algo_flops, stream);
    case 64: return launchTc<CI, 64>(p, plan, features, filter, nbr, out, status, algo_bytes, algo_flops, stream);
    case 128: return launchTc<CI, 128>(p, plan, features, filter, nbr, out, status, algo_bytes, algo_flops, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

int tcgen05PaddedChannels(int c) {
  if (c < 8 || c > 128 || c % 8) return 0;
  return c <= 16 ? 16 : (c <= 32 ? 32 : (c <= 64 ? 64 : 128));
}

bool tcgen05Eligible(const ConvProblem &p, const void *features, const void *out) {
  return p.is_half && p.K <= kMaxOffsets && tcgen05PaddedChannels(p.ci) && tcgen05PaddedChannels(p.co) &&
         (reinterpret_cast<size_t>(features) % 16 == 0) && (reinterpret_cast<size_t>(out) % 16 == 0);
}

cudaError_t launchConvTcgen05(const ConvProblem &p, const ConvWorkspacePlan &plan, const __half *features,
                              const __half *filter_image, const int32_t *nbr, __half *out, int32_t *status,
                              double algo_bytes, double algo_flops, cudaStream_t stream) {
  switch (tcgen05PaddedChannels(p.ci)) {
    case 16: return dispatchCo<16>(p, plan, features, filter_image, nbr, out, status, algo_bytes, algo_flops, stream);
    case 32: return dispatchCo<32>(p, plan, features, filter_image, nbr, out, status, algo_bytes, algo_flops, stream);
    case 64: return dispatchCo<64>(p, plan, features, filter_image, nbr, out, status, algo_bytes, algo_flops, stream);
    case 128: return dispatchCo<128>(p, plan, features, filter_image, nbr, out, status, algo_bytes, algo_flops, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace sparse_conv
}  // namespace mluop
