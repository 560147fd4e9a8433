// Inline-PTX wrappers shared by the tensor-core (tcgen05) kernels of the sparse
// convolution: shared-memory addresses, mbarriers with BOUNDED waits, cp.async
// with zero fill, tensor-memory allocation, tcgen05.mma / commit / ld.
//
// Every wait gives up after a caller-given number of clock cycles: the waiter
// records an error bit in a status word (and in the handle's sticky host word),
// raises a block-wide abort flag and returns false, so that every role of the
// kernel can fall through to its common exit.
#ifndef MLUOP_B200_KERNELS_SPARSE_CONV_TCGEN05_PRIMITIVES_CUH_
#define MLUOP_B200_KERNELS_SPARSE_CONV_TCGEN05_PRIMITIVES_CUH_

#include <cuda_runtime.h>

#include <cstdint>

namespace mluop {
namespace sparse_conv {
namespace tc {

__device__ __forceinline__ unsigned smemAddr(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbarInit(unsigned long long *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smemAddr(bar)), "r"(count));
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
struct ErrorSink {
  int32_t *status;  // status word in the workspace
  int32_t *sticky;  // device-visible host word of the handle, or null
};
__device__ __forceinline__ void raiseWaitError(const ErrorSink &sink, int code) {
  atomicOr(sink.status, code);
  if (sink.sticky) {
    *reinterpret_cast<volatile int32_t *>(sink.sticky) = code << 8;
    __threadfence_system();
  }
}
// Bounded wait of ONE thread (the MMA issuer).  Returns false (and raises the abort
// flag) when the phase did not complete within `limit` clock cycles or another
// waiter already gave up.
__device__ __forceinline__ bool mbarWait(unsigned long long *bar, unsigned parity, volatile int *abort_flag,
                                         const ErrorSink &sink, int code, long long limit) {
  if (mbarTryWait(bar, parity)) return true;
  const long long t0 = clock64();
  for (unsigned spin = 1;; ++spin) {
    if (mbarTryWait(bar, parity)) return true;
    if ((spin & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit) break;
    }
  }
  *abort_flag = 1;
  raiseWaitError(sink, code);
  return false;
}
// The same wait for a whole warp, called by all 32 lanes at the same point of the
// program.  The lanes poll on their own, but they leave together: the result is a
// vote, so a lane that gave up (or saw the abort flag) takes the whole warp to the
// exit and no lane goes on to a warp-wide shuffle without the others.
__device__ __forceinline__ bool mbarWaitWarp(unsigned long long *bar, unsigned parity, volatile int *abort_flag,
                                             const ErrorSink &sink, int code, long long limit) {
  bool ok = mbarTryWait(bar, parity);
  if (!ok) {
    const long long t0 = clock64();
    for (unsigned spin = 1;; ++spin) {
      if (mbarTryWait(bar, parity)) {
        ok = true;
        break;
      }
      if ((spin & 63u) == 0u) {
        if (*abort_flag) break;
        if (clock64() - t0 > limit) {
          *abort_flag = 1;
          raiseWaitError(sink, code);
          break;
        }
      }
    }
  }
  return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ void cpAsync16(unsigned smem, const void *gmem, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem), "l"(gmem), "r"(bytes) : "memory");
}
// Makes the mbarrier receive one arrival (one of its expected arrivals) once all
// cp.async operations this thread has issued so far have landed in shared memory.
__device__ __forceinline__ void cpAsyncArriveOn(unsigned long long *bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(smemAddr(bar)) : "memory");
}
// One arrival on an mbarrier of this block that also announces `bytes` of bulk-copy data: the
// barrier's phase completes when the arrivals are in and that many bytes have landed.
__device__ __forceinline__ void mbarArriveExpectTx(unsigned long long *bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smemAddr(bar)), "r"(bytes) : "memory");
}
// Bulk copy (the TMA engine, no tensor map) of `bytes` contiguous bytes from global to this
// block's shared memory; both addresses 16-byte aligned, bytes a multiple of 16.  Completion is
// reported to the mbarrier as transferred bytes.  No multicast.
__device__ __forceinline__ void bulkCopyToShared(unsigned smem_dst, const void *gmem_src, unsigned bytes,
                                                 unsigned long long *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(smem_dst),
               "l"(gmem_src), "r"(bytes), "r"(smemAddr(bar))
               : "memory");
}
__device__ __forceinline__ void cpAsyncWaitAll() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }
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

}  // namespace tc
}  // namespace sparse_conv
}  // namespace mluop

#endif  // MLUOP_B200_KERNELS_SPARSE_CONV_TCGEN05_PRIMITIVES_CUH_
