// Microbenchmark of the producer / issuer hand-off the tensor-core kernels are built on, with
// no data moved and no MMA issued: P producer warps and one issuer thread pass S ring stages
// back and forth through two mbarriers per stage (full: producers -> issuer, empty: issuer ->
// producers), 4,000 items per block.  What is varied is HOW each side arrives:
//   full  by thread : every producer thread lets the barrier collect an arrival through
//                     cp.async.mbarrier.arrive.noinc (what a cp.async gather needs);
//   full  by warp   : lane 0 of every producer warp arrives with mbarrier.arrive;
//   empty by commit : the issuer releases a stage with tcgen05.commit (what a stage read by
//                     tcgen05.mma needs);
//   empty by arrive : the issuer releases it with mbarrier.arrive.
// Output: one line per combination, clocks per item as block 0 sees them.  The difference
// between the lines is the cost of the arrival mechanism itself, the floor under any kernel
// that hands a stage over once per item.
//
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o ring_handoff ring_handoff.cu
#include <cuda_runtime.h>

#include <cstdio>

__device__ __forceinline__ unsigned smemAddr(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbarInit(unsigned long long *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smemAddr(bar)), "r"(count));
}
__device__ __forceinline__ bool mbarTryWait(unsigned long long *bar, unsigned parity) {
  unsigned ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok)
               : "r"(smemAddr(bar)), "r"(parity)
               : "memory");
  return ok != 0;
}
// gives up after about a second and raises the block's abort flag
__device__ __forceinline__ bool mbarWaitBounded(unsigned long long *bar, unsigned parity, volatile int *abort_flag) {
  if (mbarTryWait(bar, parity)) return true;
  const long long t0 = clock64();
  for (unsigned spin = 1;; ++spin) {
    if (mbarTryWait(bar, parity)) return true;
    if ((spin & 63u) == 0u && (*abort_flag || clock64() - t0 > 2000000000ll)) break;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void mbarArrive(unsigned long long *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ void cpAsyncArriveOn(unsigned long long *bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ void ummaCommit(unsigned long long *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smemAddr(bar))
               : "memory");
}

constexpr int kMaxStages = 8;

template <int P_WARPS, int S, bool FULL_BY_THREAD, bool EMPTY_BY_COMMIT>
__global__ void __launch_bounds__(P_WARPS * 32 + 32) handoffKernel(int items, long long *cycles_out, int *err) {
  extern __shared__ unsigned char pad[];  // only sets how many blocks share an SM
  __shared__ unsigned long long full_bar[kMaxStages], empty_bar[kMaxStages];
  __shared__ unsigned tmem_base_s;
  __shared__ int abort_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbarInit(&full_bar[s], FULL_BY_THREAD ? P_WARPS * 32 : P_WARPS);
      mbarInit(&empty_bar[s], 1);
    }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == P_WARPS) {  // tcgen05.commit belongs to a block that owns tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smemAddr(&tmem_base_s)), "r"(32u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  volatile int *abort_flag = &abort_s;
  if (warp < P_WARPS) {
    int s = 0;
    unsigned parity = 0;
    for (int it = 0; it < items; ++it) {
      if (it >= S && !mbarWaitBounded(&empty_bar[s], parity ^ 1u, abort_flag)) break;
      if (FULL_BY_THREAD) {
        cpAsyncArriveOn(&full_bar[s]);
      } else {
        __syncwarp();
        if (lane == 0) mbarArrive(&full_bar[s]);
      }
      if (++s == S) {
        s = 0;
        parity ^= 1u;
      }
    }
  } else if (lane == 0) {
    int s = 0;
    unsigned parity = 0;
    const long long t0 = clock64();
    int it = 0;
    for (; it < items; ++it) {
      if (!mbarWaitBounded(&full_bar[s], parity, abort_flag)) break;
      if (EMPTY_BY_COMMIT) {
        ummaCommit(&empty_bar[s]);
      } else {
        mbarArrive(&empty_bar[s]);
      }
      if (++s == S) {
        s = 0;
        parity ^= 1u;
      }
    }
    const long long t1 = clock64();
    if (it < items) atomicExch(err, 1);
    if (blockIdx.x == 0) cycles_out[0] = t1 - t0;
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == P_WARPS) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base_s), "r"(32u) : "memory");
  }
}

template <int P_WARPS, int S, bool FULL_BY_THREAD, bool EMPTY_BY_COMMIT>
void run(int ctas_per_sm, long long *d_cycles, int *d_err, int sms) {
  const int items = 4000;
  size_t smem = (size_t)(227 * 1024) / ctas_per_sm - 2048;
  auto kernel = handoffKernel<P_WARPS, S, FULL_BY_THREAD, EMPTY_BY_COMMIT>;
  cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  cudaMemset(d_err, 0, sizeof(int));
  kernel<<<sms * ctas_per_sm, P_WARPS * 32 + 32, smem>>>(200, d_cycles, d_err);  // warm-up
  kernel<<<sms * ctas_per_sm, P_WARPS * 32 + 32, smem>>>(items, d_cycles, d_err);
  const cudaError_t st = cudaDeviceSynchronize();
  long long cyc = 0;
  int err = 0;
  cudaMemcpy(&cyc, d_cycles, sizeof(cyc), cudaMemcpyDeviceToHost);
  cudaMemcpy(&err, d_err, sizeof(err), cudaMemcpyDeviceToHost);
  printf("producer_warps=%d stages=%d ctas_per_sm=%d full=%s empty=%s clk_per_item=%.1f err=%d %s\n", P_WARPS, S,
         ctas_per_sm, FULL_BY_THREAD ? "thread" : "warp", EMPTY_BY_COMMIT ? "commit" : "arrive", (double)cyc / items,
         err || st != cudaSuccess, st == cudaSuccess ? "" : cudaGetErrorString(st));
}

int main() {
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  long long *d_cycles;
  int *d_err;
  cudaMalloc(&d_cycles, sizeof(long long));
  cudaMalloc(&d_err, sizeof(int));
  // the filter-gradient kernel's shape: 8 producer warps, 6 stages, one block per SM
  run<8, 6, true, true>(1, d_cycles, d_err, sms);
  run<8, 6, false, true>(1, d_cycles, d_err, sms);
  run<8, 6, true, false>(1, d_cycles, d_err, sms);
  run<8, 6, false, false>(1, d_cycles, d_err, sms);
  run<8, 2, true, true>(1, d_cycles, d_err, sms);
  // the forward kernel's shape: 4 producer warps, 2 stages, four blocks per SM
  run<4, 2, true, true>(1, d_cycles, d_err, sms);
  run<4, 2, true, true>(4, d_cycles, d_err, sms);
  run<4, 2, false, true>(4, d_cycles, d_err, sms);
  run<4, 2, true, false>(4, d_cycles, d_err, sms);
  run<4, 2, false, false>(4, d_cycles, d_err, sms);
  cudaFree(d_cycles);
  cudaFree(d_err);
  return 0;
}
