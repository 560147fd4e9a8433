// Sparse convolution forward on the 5th-generation tensor cores (tcgen05) of
// sm_100a: half inputs, fp32 accumulation in tensor memory.
//
// One thread block owns 128 output rows and keeps their [128 x Co] fp32
// accumulator in TMEM for the whole kernel.  It walks the kernel offsets that
// have at least one live row in the tile, in ascending order; per offset
//   * four producer warps (one thread per output row) gather the input rows
//     named by the neighbour table into a shared-memory A tile with cp.async
//     (16-byte chunks, zero fill for rows without a neighbour) and copy W_k
//     ([Co x Ci], Ci contiguous) into a B tile; both tiles are written in the
//     K-major swizzled layout tcgen05.mma reads;
//   * one elected thread issues Ci/16 tcgen05.mma instructions (M=128, N=Co,
//     K=16) that accumulate into TMEM, then tcgen05.commit releases the stage.
// Stages form a ring guarded by mbarriers (full: 128 producer arrivals after
// cp.async.wait_group + fence.proxy.async; empty: one arrival from
// tcgen05.commit).  After the last offset the producer warps read the
// accumulator back with tcgen05.ld, round to half and store each output row
// once.  The reduction over offsets happens in TMEM in a fixed order, so the
// result is deterministic.
//
// Every mbarrier wait is bounded: after about one second the waiter records an
// error in the status word, raises a block-wide abort flag and every role
// falls through to the common exit, where outstanding cp.async groups are
// drained and TMEM is freed.  The host side reports a non-zero status word as
// MLUOP_STATUS_EXECUTION_FAILED when asked to check it.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <string>

#include "core/trace.h"
#include "kernels/sparse_conv/indice_convolution_kernels.h"
#include "kernels/sparse_conv/indice_convolution_tcgen05.h"

namespace mluop {
namespace sparse_conv {

namespace {

constexpr int kTile = kConvTileRows;      // 128 output rows = 128 TMEM lanes
constexpr int kProducerThreads = 128;     // warps 0-3: gather, then epilogue
constexpr int kThreads = 160;             // + warp 4: TMEM allocation and MMA issue
constexpr int kMaxOffsets = 32;
constexpr long long kWaitCycles = 2000000000ll;  // a wait gives up after about one second

__device__ __forceinline__ unsigned smemAddr(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbarInit(unsigned long long *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smemAddr(bar)), "r"(count));
}
__device__ __forceinline__ void mbarArrive(unsigned long long *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ bool mbarTryWait(unsigned long long *bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smemAddr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and raises the abort flag) when the phase did
// not complete within kWaitCycles clock cycles or another waiter already gave up.
__device__ __forceinline__ bool mbarWait(unsigned long long *bar, unsigned parity, volatile int *abort_flag,
                                         int32_t *status, int code) {
  if (mbarTryWait(bar, parity)) return true;
  const long long t0 = clock64();
  for (unsigned spin = 1;; ++spin) {
    if (mbarTryWait(bar, parity)) return true;
    if ((spin & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitCycles) break;
    }
  }
  *abort_flag = 1;
  atomicOr(status, code);
  return false;
}

__device__ __forceinline__ void cpAsync16(unsigned smem, const void *gmem, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cpAsyncCommit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cpAsyncWait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fenceProxyAsync() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void tcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

__device__ __forceinline__ void tmemAlloc(unsigned *smem_dst, unsigned cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smemAddr(smem_dst)),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmemDealloc(unsigned taddr, unsigned cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                     unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread has finished.
__device__ __forceinline__ void ummaCommit(unsigned long long *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smemAddr(bar))
               : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns of TMEM -> 16 registers per thread.
__device__ __forceinline__ void tmemLoad16(unsigned taddr, unsigned (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmemLoadWait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

template <int CI, int CO, int STAGES>
struct TcConfig {
  // K is split into blocks of at most 64 halfs (128 bytes, one swizzle atom wide)
  static constexpr int kBlockK = CI < 64 ? CI : 64;
  static constexpr int kKBlocks = CI / kBlockK;
  static constexpr int kRowBytes = kBlockK * 2;                 // 32, 64 or 128
  static constexpr unsigned kSwizzleMask = kRowBytes / 16 - 1;  // 1, 3 or 7: XOR of 16-byte chunk index
  // tcgen05 shared-memory descriptor layout type: 128B = 2, 64B = 4, 32B = 6
  static constexpr unsigned long long kLayoutType = kRowBytes == 128 ? 2 : (kRowBytes == 64 ? 4 : 6);
  static constexpr int kABlockBytes = kTile * kRowBytes;
  static constexpr int kBBlockBytes = CO * kRowBytes;  // a multiple of 1024 when CO*kRowBytes >= 1024
  static constexpr int kBBlockStride = (kBBlockBytes + 1023) / 1024 * 1024;
  static constexpr int kAStageBytes = kKBlocks * kABlockBytes;
  static constexpr int kBStageBytes = kKBlocks * kBBlockStride;
  static constexpr int kStageBytes = kAStageBytes + kBStageBytes;
  static constexpr int kTmemCols = CO < 32 ? 32 : CO;
  static constexpr int kChunksPerRow = CI / 8;  // 16-byte chunks of one feature row
  // instruction descriptor: D fp32, A and B fp16, both K-major, N = CO, M = 128
  static constexpr unsigned kIdesc = (1u << 4) | ((unsigned)(CO >> 3) << 17) | ((unsigned)(kTile >> 4) << 24);
  static size_t smemBytes(int K) {
    return 1024 /* alignment slack */ + (size_t)STAGES * kStageBytes + (size_t)K * kTile * sizeof(int32_t) + 1024;
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

template <int CI, int CO, int STAGES>
__global__ void __launch_bounds__(kThreads)
convTcgen05Kernel(const __half *__restrict__ features, const __half *__restrict__ filter_kcoci,
                  const int32_t *__restrict__ nbr, int64_t n_out, int64_t n_pad, int K,
                  __half *__restrict__ out, int32_t *status) {
  using Cfg = TcConfig<CI, CO, STAGES>;
  extern __shared__ unsigned char smem_raw[];
  // operand blocks must sit on 1024-byte boundaries (swizzle atoms)
  unsigned char *stage_base =
      reinterpret_cast<unsigned char *>((reinterpret_cast<size_t>(smem_raw) + 1023) & ~(size_t)1023);
  int32_t *nbr_s = reinterpret_cast<int32_t *>(stage_base + (size_t)STAGES * Cfg::kStageBytes);  // [K][128]
  __shared__ unsigned long long full_bar[STAGES], empty_bar[STAGES], accum_bar;
  __shared__ unsigned tmem_base_s;
  __shared__ int klist_s[kMaxOffsets];
  __shared__ unsigned live_mask_s;
  __shared__ int n_live_s;
  __shared__ int abort_s;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t r0 = (int64_t)blockIdx.x * kTile;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbarInit(&full_bar[s], kProducerThreads);
      mbarInit(&empty_bar[s], 1);
    }
    mbarInit(&accum_bar, 1);
    live_mask_s = 0;
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 4) tmemAlloc(&tmem_base_s, Cfg::kTmemCols);
  for (int e = tid; e < K * kTile; e += kThreads) {
    const int k = e / kTile, r = e % kTile;
    nbr_s[e] = nbr[(size_t)k * n_pad + r0 + r];
  }
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  if (warp < 4) {
    unsigned mine = 0;
    for (int k = 0; k < K; ++k) {
      const unsigned any = __ballot_sync(0xffffffffu, nbr_s[k * kTile + tid] >= 0);
      if (any) mine |= 1u << k;
    }
    if (lane == 0 && mine) atomicOr(&live_mask_s, mine);
  }
  __syncthreads();
  if (tid == 0) {
    int n = 0;
    for (int k = 0; k < K; ++k)
      if ((live_mask_s >> k) & 1u) klist_s[n++] = k;
    n_live_s = n;
  }
  __syncthreads();
  const int n_live = n_live_s;
  const unsigned tmem_base = tmem_base_s;
  volatile int *abort_flag = &abort_s;

  if (warp < 4) {
    // ------------------------------------------------------------ producers
    const int row = tid;  // tile row this thread gathers
    constexpr int kLag = STAGES > 2 ? 2 : 1;  // cp.async groups allowed in flight before signalling
    int signalled = 0;
    for (int it = 0; it < n_live; ++it) {
      const int s = it % STAGES;
      if (it >= STAGES) {
        if (!mbarWait(&empty_bar[s], ((it / STAGES) - 1) & 1, abort_flag, status, 1)) break;
      }
      const int k = klist_s[it];
      unsigned char *a_stage = stage_base + (size_t)s * Cfg::kStageBytes;
      unsigned char *b_stage = a_stage + Cfg::kAStageBytes;
      const int idx = nbr_s[k * kTile + row];
      const __half *src = features + (idx >= 0 ? (size_t)idx * CI : 0);
#pragma unroll
      for (int c = 0; c < Cfg::kChunksPerRow; ++c) {
        const int kb = c / (Cfg::kRowBytes / 16), cc = c % (Cfg::kRowBytes / 16);
        unsigned off = (unsigned)(row * Cfg::kRowBytes + cc * 16);
        off ^= ((off >> 7) & Cfg::kSwizzleMask) << 4;
        cpAsync16(smemAddr(a_stage + kb * Cfg::kABlockBytes + off), src + c * 8, idx >= 0);
      }
      const __half *wk = filter_kcoci + (size_t)k * CO * CI;
      for (int e = tid; e < CO * Cfg::kChunksPerRow; e += kProducerThreads) {
        const int n = e / Cfg::kChunksPerRow, c = e % Cfg::kChunksPerRow;
        const int kb = c / (Cfg::kRowBytes / 16), cc = c % (Cfg::kRowBytes / 16);
        unsigned off = (unsigned)(n * Cfg::kRowBytes + cc * 16);
        off ^= ((off >> 7) & Cfg::kSwizzleMask) << 4;
        cpAsync16(smemAddr(b_stage + kb * Cfg::kBBlockStride + off), wk + (size_t)n * CI + c * 8, true);
      }
      cpAsyncCommit();
      if (it >= kLag) {
        cpAsyncWait<kLag>();
        fenceProxyAsync();
        mbarArrive(&full_bar[signalled % STAGES]);
        ++signalled;
      }
    }
    cpAsyncWait<0>();
    fenceProxyAsync();
    if (!*abort_flag) {
      for (; signalled < n_live; ++signalled) mbarArrive(&full_bar[signalled % STAGES]);
    }

    // ------------------------------------------------------------- epilogue
    const int64_t r = r0 + row;
    bool have_acc = n_live > 0;
    if (have_acc) have_acc = mbarWait(&accum_bar, 0, abort_flag, status, 4);
    tcFenceAfter();
    if (!*abort_flag) {
      __half *dst = out + (size_t)r * CO;
#pragma unroll
      for (int c0 = 0; c0 < CO; c0 += 16) {
        unsigned v[16];
        if (have_acc) {
          tmemLoad16(tmem_base + ((unsigned)(warp * 32) << 16) + (unsigned)c0, v);
          tmemLoadWait();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = 0u;
        }
        if (r < n_out) {
          uint4 lo, hi;
          __half2 h[8];
#pragma unroll
          for (int i = 0; i < 8; ++i)
            h[i] = __floats2half2_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
          lo = *reinterpret_cast<uint4 *>(&h[0]);
          hi = *reinterpret_cast<uint4 *>(&h[4]);
          *reinterpret_cast<uint4 *>(dst + c0) = lo;
          *reinterpret_cast<uint4 *>(dst + c0 + 8) = hi;
        }
      }
    }
    tcFenceBefore();
  } else {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      for (int it = 0; it < n_live; ++it) {
        const int s = it % STAGES;
        if (!mbarWait(&full_bar[s], (it / STAGES) & 1, abort_flag, status, 2)) break;
        tcFenceAfter();
        const unsigned a_addr = smemAddr(stage_base + (size_t)s * Cfg::kStageBytes);
        const unsigned b_addr = a_addr + Cfg::kAStageBytes;
#pragma unroll
        for (int j = 0; j < CI / 16; ++j) {
          const int kb = (j * 32) / Cfg::kRowBytes, within = (j * 32) % Cfg::kRowBytes;
          const unsigned long long a_desc = makeDesc<Cfg>(a_addr + kb * Cfg::kABlockBytes + within);
          const unsigned long long b_desc = makeDesc<Cfg>(b_addr + kb * Cfg::kBBlockStride + within);
          umma(tmem_base, a_desc, b_desc, Cfg::kIdesc, (it > 0 || j > 0) ? 1u : 0u);
        }
        ummaCommit(&empty_bar[s]);  // the stage may be refilled once these MMAs have read it
      }
      if (n_live > 0 && !*abort_flag) ummaCommit(&accum_bar);
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

template <int CI, int CO, int STAGES>
cudaError_t launchTc(const ConvProblem &p, const ConvWorkspacePlan &plan, const __half *features,
                     const __half *filter, const int32_t *nbr, __half *out, int32_t *status, double algo_bytes,
                     double algo_flops, cudaStream_t stream) {
  using Cfg = TcConfig<CI, CO, STAGES>;
  auto kernel = convTcgen05Kernel<CI, CO, STAGES>;
  const size_t smem = Cfg::smemBytes(p.K);
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) return err;
  const unsigned blocks = (unsigned)(plan.n_pad / kTile);
  static const std::string name = "convTcgen05Kernel<" + std::to_string(CI) + "," + std::to_string(CO) + ">";
  trace::Scope t(name.c_str(), stream, algo_bytes, algo_flops);
  kernel<<<blocks, kThreads, smem, stream>>>(features, filter, nbr, p.n_out, plan.n_pad, p.K, out, status);
  return cudaGetLastError();
}

template <int CI>
cudaError_t dispatchCo(const ConvProblem &p, const ConvWorkspacePlan &plan, const __half *features,
                       const __half *filter, const int32_t *nbr, __half *out, int32_t *status, double algo_bytes,
                       double algo_flops, cudaStream_t stream) {
  constexpr int kStages = CI >= 128 ? 3 : 4;
  switch (p.co) {
    case 16: return launchTc<CI, 16, kStages>(p, plan, features, filter, nbr, out, status, algo_bytes, algo_flops, stream);
    case 32: return launchTc<CI, 32, kStages>(p, plan, features, filter, nbr, out, status, algo_bytes, algo_flops, stream);
    case 64: return launchTc<CI, 64, kStages>(p, plan, features, filter, nbr, out, status, algo_bytes, algo_flops, stream);
    case 128: return launchTc<CI, 128, kStages>(p, plan, features, filter, nbr, out, status, algo_bytes, algo_flops, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

bool tcgen05Eligible(const ConvProblem &p, const void *features, const void *out) {
  auto ok = [](int c) { return c == 16 || c == 32 || c == 64 || c == 128; };
  return p.is_half && p.K <= kMaxOffsets && ok(p.ci) && ok(p.co) &&
         (reinterpret_cast<size_t>(features) % 16 == 0) && (reinterpret_cast<size_t>(out) % 16 == 0);
}

cudaError_t launchConvTcgen05(const ConvProblem &p, const ConvWorkspacePlan &plan, const __half *features,
                              const __half *filter_kcoci, const int32_t *nbr, __half *out, int32_t *status,
                              double algo_bytes, double algo_flops, cudaStream_t stream) {
  switch (p.ci) {
    case 16: return dispatchCo<16>(p, plan, features, filter_kcoci, nbr, out, status, algo_bytes, algo_flops, stream);
    case 32: return dispatchCo<32>(p, plan, features, filter_kcoci, nbr, out, status, algo_bytes, algo_flops, stream);
    case 64: return dispatchCo<64>(p, plan, features, filter_kcoci, nbr, out, status, algo_bytes, algo_flops, stream);
    case 128: return dispatchCo<128>(p, plan, features, filter_kcoci, nbr, out, status, algo_bytes, algo_flops, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace sparse_conv
}  // namespace mluop
