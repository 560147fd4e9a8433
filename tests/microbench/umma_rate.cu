// Microbenchmark behind the shared-memory roofline of the tensor-core convolution kernel:
// cycles per tcgen05.mma (cta_group::1, kind::f16, M = 128, K = 16, both operands K-major in
// shared memory with the 128-byte swizzle) as a function of N and of the number of CTAs
// resident per SM.  One thread per CTA issues 16,000 back-to-back MMAs on two alternating
// A tiles and one B tile, commits them to an mbarrier and waits (bounded); the kernel is
// timed with CUDA events and block 0 reports its own clock64() span.
//
// The second table ("mn-major") repeats the measurement with both operands MN-major (rows of
// the contracted axis 128 bytes apart, the layout the filter-gradient kernel feeds the
// tensor cores from): A is [128 rows of K][128 of M] as two 64-wide atoms, B [128 rows of K][N].
//
// What it shows on B200: the cost of an MMA is max(math, operand bytes / 128 B per clock):
// N = 64 costs 48 clocks (4 KB of A + 2 KB of B), not the 32 clocks of its 262,144 flops;
// N = 128 costs 64 (8 KB of operands, and 64 clocks of math); N = 256 costs 128
// (math-bound).  More CTAs per SM do not raise the SM's rate.
//
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o umma_rate umma_rate.cu
// Output: one line per (N, CTAs per SM): "N=<n> ctas_per_sm=<c> clk_per_mma=<block 0's
// cycles per MMA> sm_clk_per_mma=<kernel time x 1.965 GHz / MMAs per SM> tflops=<...> err=<0|1>"
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>

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
// gives up after about a second
__device__ __forceinline__ bool mbarWaitBounded(unsigned long long *bar, unsigned parity) {
  const long long t0 = clock64();
  while (!mbarTryWait(bar, parity)) {
    if (clock64() - t0 > 2000000000ll) return false;
  }
  return true;
}
__device__ __forceinline__ void umma(unsigned d, unsigned long long a, unsigned long long b, unsigned idesc,
                                     unsigned accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d),
               "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
               : "memory");
}
__device__ __forceinline__ void ummaCommit(unsigned long long *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smemAddr(bar))
               : "memory");
}

// K-major operand block, 128-byte swizzle: rows of 64 halfs, 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long makeDesc(unsigned addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
  d |= (unsigned long long)(1024u >> 4) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// MN-major operand, 128-byte swizzle: 64 elements of M (or N) contiguous per row of the contracted
// axis, 8-row groups 1024 bytes apart, the next 64 elements of M/N 16 KB further.
__device__ __forceinline__ unsigned long long makeDescMn(unsigned addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
  d |= (unsigned long long)(16384u >> 4) << 16;
  d |= (unsigned long long)(1024u >> 4) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

template <int N, bool MN>
__global__ void __launch_bounds__(64) rateKernel(int groups, long long *cycles_out, int *err) {
  extern __shared__ unsigned char raw[];
  unsigned char *base = (unsigned char *)(((size_t)raw + 1023) & ~(size_t)1023);
  unsigned char *a_ring = base;             // 2 tiles x [128 x 64] half = 2 x 16 KB
  unsigned char *b_buf = base + 2 * 16384;  // [N x 64] half (MN-major: [128 x N] half as N/64 blocks of 16 KB)
  constexpr int kBBytes = MN ? (N / 64) * 16384 : N * 128;
  __shared__ unsigned long long done_bar;
  __shared__ unsigned tmem_base_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr unsigned kCols = N < 32 ? 32 : N;
  if (tid == 0) {
    mbarInit(&done_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  for (int i = tid; i < (2 * 16384 + kBBytes) / 4; i += blockDim.x) ((unsigned *)base)[i] = 0x3c003c00u;  // ones
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smemAddr(&tmem_base_s)),
                 "r"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem = tmem_base_s;
  constexpr unsigned idesc =
      (1u << 4) | (MN ? (3u << 15) : 0u) | ((unsigned)(N >> 3) << 17) | ((unsigned)(128 >> 4) << 24);
  if (warp == 1) {
    if (lane == 0) {
      const unsigned long long a0 = MN ? makeDescMn(smemAddr(a_ring)) : makeDesc(smemAddr(a_ring));
      const unsigned long long b0 = MN ? makeDescMn(smemAddr(b_buf)) : makeDesc(smemAddr(b_buf));
      const long long t0 = clock64();
      for (int it = 0; it < groups; ++it) {
        if (MN) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // four K steps of 16 rows (2048 bytes) down the 128 rows
            const unsigned long long step = (unsigned long long)(((((it & 1) * 4 + j) * 2048)) >> 4);
            umma(tmem, a0 + step, b0 + step, idesc, (it | j) ? 1u : 0u);
          }
        } else {
          const unsigned long long a = a0 + (unsigned long long)(((it & 1) * 16384) >> 4);
#pragma unroll
          for (int j = 0; j < 4; ++j)  // four K steps of 16 halfs (32 bytes) inside the 128-byte rows
            umma(tmem, a + (unsigned long long)((j * 32) >> 4), b0 + (unsigned long long)((j * 32) >> 4), idesc,
                 (it | j) ? 1u : 0u);
        }
      }
      ummaCommit(&done_bar);
      const bool ok = mbarWaitBounded(&done_bar, 0);
      const long long t1 = clock64();
      if (!ok) atomicExch(err, 1);
      if (blockIdx.x == 0) cycles_out[0] = t1 - t0;
    }
    __syncwarp();
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kCols) : "memory");
  }
}

template <int N, bool MN = false>
void run(int ctas_per_sm, long long *d_cycles, int *d_err, int sms) {
  const int groups = 4000;
  const size_t need = 1024 + 2 * 16384 + (MN ? (N / 64) * 16384 : N * 128);
  // dynamic shared memory padded so that exactly ctas_per_sm blocks fit an SM
  size_t smem = (size_t)(227 * 1024) / ctas_per_sm - 2048;
  if (smem < need) smem = need;
  cudaFuncSetAttribute(rateKernel<N, MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  cudaMemset(d_err, 0, sizeof(int));
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  rateKernel<N, MN><<<sms * ctas_per_sm, 64, smem>>>(200, d_cycles, d_err);  // warm-up
  cudaEventRecord(e0);
  rateKernel<N, MN><<<sms * ctas_per_sm, 64, smem>>>(groups, d_cycles, d_err);
  cudaEventRecord(e1);
  const cudaError_t st = cudaDeviceSynchronize();
  float ms = 0;
  cudaEventElapsedTime(&ms, e0, e1);
  long long cyc = 0;
  int err = 0;
  cudaMemcpy(&cyc, d_cycles, sizeof(cyc), cudaMemcpyDeviceToHost);
  cudaMemcpy(&err, d_err, sizeof(err), cudaMemcpyDeviceToHost);
  const double mmas = 4.0 * groups;
  const double flops = 2.0 * 128 * N * 16 * mmas * sms * ctas_per_sm;
  printf("%sN=%d ctas_per_sm=%d clk_per_mma=%.1f sm_clk_per_mma=%.1f tflops=%.1f err=%d %s\n", MN ? "mn-major " : "", N, ctas_per_sm,
         cyc / mmas, ms * 1e-3 * 1.965e9 / (mmas * ctas_per_sm), flops / (ms * 1e-3) / 1e12,
         err || st != cudaSuccess, st == cudaSuccess ? "" : cudaGetErrorString(st));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
}

int main() {
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  long long *d_cycles;
  int *d_err;
  cudaMalloc(&d_cycles, sizeof(long long));
  cudaMalloc(&d_err, sizeof(int));
  for (int ctas = 1; ctas <= 4; ctas *= 2) {
    run<16>(ctas, d_cycles, d_err, sms);
    run<32>(ctas, d_cycles, d_err, sms);
    run<64>(ctas, d_cycles, d_err, sms);
    run<128>(ctas, d_cycles, d_err, sms);
    if (ctas <= 2) run<256>(ctas, d_cycles, d_err, sms);
  }
  for (int ctas = 1; ctas <= 2; ctas *= 2) {
    run<64, true>(ctas, d_cycles, d_err, sms);
    run<128, true>(ctas, d_cycles, d_err, sms);
    run<256, true>(ctas, d_cycles, d_err, sms);
  }
  cudaFree(d_cycles);
  cudaFree(d_err);
  return 0;
}
