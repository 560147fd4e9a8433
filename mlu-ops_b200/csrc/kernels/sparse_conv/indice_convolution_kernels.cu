// Sparse convolution forward kernels for sm_100a.
//
//   features_out[r,:] = sum_k sum_{(j,r) in pairs_k} features[j,:] * W_k
//
// (reference kernels/sparse_conv/indice_convolution_forward/
// indice_convolution_forward.cpp:171-571: per kernel offset a gather, a matmul,
// a scatter into a zeroed [N_out,Co] buffer and an add over the whole output.)
//
// Here the computation is output-stationary.  The pair lists are first turned
// into a neighbour table nbr[k][r] = input row feeding output row r at offset
// k (-1 if none; a rulebook holds at most one pair per (k, r)).  A thread block
// then owns a tile of output rows, walks the kernel offsets in ascending
// order, gathers the live input rows of the tile into shared memory, multiplies
// by W_k and keeps the running sum in registers in fp32.  Every output row is
// written exactly once, already summed, in a fixed order: the scatter of the
// reference becomes a deterministic in-order reduction with no atomics and no
// per-offset pass over the output.
//
// Kernels:
//   repackFilterKernel      any layout -> T[K][Co][Ci]
//   buildNeighbourKernel    pair lists -> nbr table
//   convMmaF16Kernel        half, Ci and Co in {16,32,64,128}: cp.async row
//                           gather into padded shared tiles, ldmatrix +
//                           mma.sync m16n8k16 with fp32 accumulators, multi-stage
//                           pipeline over the live offsets of the tile
//   convGenericKernel       float, and half with other channel counts: fp32 FMA
#include "kernels/sparse_conv/indice_convolution_kernels.h"

#include <cstdlib>
#include <cstring>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <string>

#include "core/trace.h"
#include "kernels/sparse_conv/get_indice_pairs_kernels.h"
#include "kernels/sparse_conv/indice_convolution_tcgen05.h"

namespace mluop {
namespace sparse_conv {

namespace {

inline size_t alignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

// a table emitted by the rulebook kernels is read by the convolution as its own
static_assert(kPairsTablePadRows == kConvPadRows, "one row padding for both producers of a neighbour table");

constexpr int kMaxCountsByValue = 128;
struct PairCounts {
  int32_t n[kMaxCountsByValue];
};

// ------------------------------------------------------------ preparation

// dst is [K][n_dst][c_dst]: n the produced channel, c the contracted channel of this
// direction (forward: n = Co, c = Ci; input gradient, `swap`: n = Ci, c = Co), zero where
// n >= n_real or c >= c_real (channel counts padded for the tensor-core kernel).
// Blocks [0, repack_blocks) of the grid repack; any further blocks fill `table` (table_vec
// 16-byte words, null when there is nothing to fill) with -1, so that a call that also builds
// its neighbour table needs one launch for both preparations.  Block 0 also clears the
// workspace's status words.
template <typename T>
__global__ void __launch_bounds__(256)
repackFilterKernel(const T *__restrict__ src, T *__restrict__ dst, int K, int ci, int co, int layout, int swap,
                   int n_dst, int c_dst, unsigned repack_blocks, int4 *__restrict__ table, int64_t table_vec,
                   int32_t *__restrict__ status_words, int image_row_bytes, int image_block_stride,
                   int image_bytes_per_offset) {
  // the 64 status words of the workspace start at zero for the kernels that follow
  if (blockIdx.x == 0 && threadIdx.x < 64) status_words[threadIdx.x] = 0;
  if (blockIdx.x >= repack_blocks) {
    const int4 none = make_int4(-1, -1, -1, -1);
    const int64_t stride = (int64_t)(gridDim.x - repack_blocks) * blockDim.x;
    for (int64_t i = (int64_t)(blockIdx.x - repack_blocks) * blockDim.x + threadIdx.x; i < table_vec; i += stride)
      table[i] = none;
    return;
  }
  const int64_t total = (int64_t)K * n_dst * c_dst;
  const int n_real = swap ? ci : co, c_real = swap ? co : ci;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)repack_blocks * blockDim.x) {
    const int c = (int)(i % c_dst);
    const int n = (int)((i / c_dst) % n_dst);
    const int k = (int)(i / ((int64_t)n_dst * c_dst));
    T v = T(0.f);
    if (n < n_real && c < c_real) {
      const int in_ch = swap ? n : c, out_ch = swap ? c : n;  // the caller's Ci and Co indices
      int64_t s;
      if (layout == kFilterArray) {
        s = ((int64_t)k * ci + in_ch) * co + out_ch;  // [K][Ci][Co]
      } else if (layout == kFilterNDHWC) {
        s = ((int64_t)out_ch * K + k) * ci + in_ch;  // [Co][K][Ci]
      } else {
        s = ((int64_t)out_ch * ci + in_ch) * K + k;  // [Co][Ci][K]
      }
      v = src[s];
    }
    if (image_row_bytes == 0) {
      dst[i] = v;
    } else {
      // the tensor-core kernel's shared-memory image of this offset (see Tcgen05FilterImage)
      const int block_k = image_row_bytes / (int)sizeof(T);
      unsigned off = (unsigned)(n * image_row_bytes + (c % block_k) * (int)sizeof(T));
      off ^= ((off >> 7) & (unsigned)(image_row_bytes / 16 - 1)) << 4;
      char *at = reinterpret_cast<char *>(dst) + (size_t)k * image_bytes_per_offset +
                 (size_t)(c / block_k) * image_block_stride + off;
      *reinterpret_cast<T *>(at) = v;
    }
  }
}

// Pairs handled by one thread (independent loads in flight before the stores).
constexpr int kBuildPairsPerThread = 4;

template <bool BY_VALUE>
__global__ void __launch_bounds__(256)
buildNeighbourKernel(const int32_t *__restrict__ pairs, int64_t pair_stride, int swap, int64_t L,
                     int64_t n_out, int64_t n_pad, PairCounts counts,
                     const int32_t *__restrict__ counts_dev, int32_t *__restrict__ nbr) {
  // pairs is [K][2][pair_stride]; row 0 of an offset holds the ids of the rows that
  // are gathered (L of them) and row 1 the ids of the rows that are produced (n_out),
  // the other way round when swap is set.
  const int k = blockIdx.y;
  const int64_t pk = BY_VALUE ? counts.n[k] : counts_dev[k];
  const int32_t *in_row = pairs + (size_t)k * 2 * pair_stride + (swap ? pair_stride : 0);
  const int32_t *out_row = pairs + (size_t)k * 2 * pair_stride + (swap ? 0 : pair_stride);
  int32_t *table = nbr + (size_t)k * n_pad;
  const int64_t span = (int64_t)blockDim.x * kBuildPairsPerThread;
  for (int64_t base = (int64_t)blockIdx.x * span; base < pk; base += (int64_t)gridDim.x * span) {
    int32_t src[kBuildPairsPerThread], dst[kBuildPairsPerThread];
#pragma unroll
    for (int i = 0; i < kBuildPairsPerThread; ++i) {
      const int64_t p = base + i * blockDim.x + threadIdx.x;
      src[i] = p < pk ? in_row[p] : -1;
      dst[i] = p < pk ? out_row[p] : -1;
    }
    // A rulebook holds one pair per (k, output row), so plain stores never collide.
#pragma unroll
    for (int i = 0; i < kBuildPairsPerThread; ++i)
      if (src[i] >= 0 && src[i] < L && dst[i] >= 0 && dst[i] < n_out) table[dst[i]] = src[i];
  }
}

// ------------------------------------------------------------ generic FMA

__device__ __forceinline__ float toFloat(float v) { return v; }
__device__ __forceinline__ float toFloat(__half v) { return __half2float(v); }
__device__ __forceinline__ void fromFloat(float v, float *dst) { *dst = v; }
__device__ __forceinline__ void fromFloat(float v, __half *dst) { *dst = __float2half_rn(v); }

constexpr int kGenRows = 32;      // output rows per block
constexpr int kGenLanes = 8;      // threads per row
constexpr int kGenCols = 128;     // output channels per block (blockIdx.y walks the rest)
constexpr int kGenCiChunk = 64;   // input channels staged per step
constexpr int kSmallFilterFloats = 8192;  // K*Ci*Co up to this many values stay resident in shared memory

// Thread (row, lane) owns output channels lane, lane+8, ... of its row.
template <typename T>
__global__ void __launch_bounds__(kGenRows *kGenLanes)
convGenericKernel(const T *__restrict__ features, const T *__restrict__ filter_kcoci,
                  const int32_t *__restrict__ nbr, int64_t n_out, int64_t n_pad, int K, int ci, int co,
                  T *__restrict__ out) {
  __shared__ float w_s[kGenCiChunk][kGenCols + 1];
  const int row_in_block = threadIdx.x / kGenLanes;
  const int lane = threadIdx.x % kGenLanes;
  const int64_t r = (int64_t)blockIdx.x * kGenRows + row_in_block;
  const int col0 = blockIdx.y * kGenCols;
  const int ncols = min(kGenCols, co - col0);
  float acc[kGenCols / kGenLanes];
#pragma unroll
  for (int i = 0; i < kGenCols / kGenLanes; ++i) acc[i] = 0.f;

  for (int k = 0; k < K; ++k) {
    const int idx = (r < n_out) ? nbr[(size_t)k * n_pad + r] : -1;
    if (!__syncthreads_or(idx >= 0)) continue;
    const T *wk = filter_kcoci + ((size_t)k * co + col0) * ci;
    for (int c0 = 0; c0 < ci; c0 += kGenCiChunk) {
      const int nc = min(kGenCiChunk, ci - c0);
      __syncthreads();
      for (int e = threadIdx.x; e < nc * ncols; e += blockDim.x) {
        const int c = e % nc, n = e / nc;
        w_s[c][n] = toFloat(wk[(size_t)n * ci + c0 + c]);
      }
      __syncthreads();
      if (idx >= 0) {
        const T *f = features + (size_t)idx * ci + c0;
        for (int c = 0; c < nc; ++c) {
          const float a = toFloat(f[c]);
#pragma unroll
          for (int i = 0; i < kGenCols / kGenLanes; ++i) {
            const int n = lane + i * kGenLanes;
            if (n < ncols) acc[i] = fmaf(a, w_s[c][n], acc[i]);
          }
        }
      }
    }
  }
  if (r < n_out) {
#pragma unroll
    for (int i = 0; i < kGenCols / kGenLanes; ++i) {
      const int n = lane + i * kGenLanes;
      if (n < ncols) fromFloat(acc[i], out + (size_t)r * co + col0 + n);
    }
  }
}

// Small filters (K*Ci*Co <= 8192 values, Co <= 32): the whole filter sits in
// shared memory as float [K][Ci][Co]; a thread owns NOUT consecutive output
// channels of one output row and walks the K offsets without block-wide
// synchronisation.  Same accumulation order as the general kernel.
template <typename T, int NOUT>
__global__ void __launch_bounds__(256)
convSmallFilterKernel(const T *__restrict__ features, const T *__restrict__ filter_kcoci,
                      const int32_t *__restrict__ nbr, int64_t n_out, int64_t n_pad, int K, int ci, int co,
                      T *__restrict__ out) {
  extern __shared__ float wf_s[];  // [K][ci][co]
  for (int e = threadIdx.x; e < K * ci * co; e += blockDim.x) {
    const int c = e % ci, n = (e / ci) % co, k = e / (ci * co);
    wf_s[((size_t)k * ci + c) * co + n] = toFloat(filter_kcoci[e]);
  }
  __syncthreads();
  const int groups = co / NOUT;  // threads per output row
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t r = t / groups;
  const int n0 = (int)(t % groups) * NOUT;
  if (r >= n_out) return;
  float acc[NOUT];
#pragma unroll
  for (int i = 0; i < NOUT; ++i) acc[i] = 0.f;
  for (int k = 0; k < K; ++k) {
    const int idx = nbr[(size_t)k * n_pad + r];
    if (idx < 0) continue;
    const T *f = features + (size_t)idx * ci;
    const float *w = wf_s + (size_t)k * ci * co + n0;
    for (int c = 0; c < ci; ++c) {
      const float a = toFloat(f[c]);
#pragma unroll
      for (int i = 0; i < NOUT; ++i) acc[i] = fmaf(a, w[c * co + i], acc[i]);
    }
  }
  T *dst = out + (size_t)r * co + n0;
#pragma unroll
  for (int i = 0; i < NOUT; ++i) fromFloat(acc[i], dst + i);
}

// ------------------------------------------------------------ tensor cores

constexpr int kMmaMaxOffsets = 32;  // kernel volumes up to 32 keep the tile's table in shared memory

__device__ __forceinline__ void cpAsync16(void *smem, const void *gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0: nothing is read, 16 zero bytes are written
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cpAsyncCommit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cpAsyncWait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrixX4(unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3,
                                           const void *smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(s));
}
__device__ __forceinline__ void mmaF16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int CI, int CO, int STAGES>
struct MmaConfig {
  static constexpr int kThreads = 256;
  static constexpr int kWarpsN = (CO >= 32) ? 2 : 1;
  static constexpr int kWarpsM = 8 / kWarpsN;
  static constexpr int kWarpRows = kConvTileRows / kWarpsM;  // 32 or 16
  static constexpr int kMI = kWarpRows / 16;
  static constexpr int kWarpCols = CO / kWarpsN;
  static constexpr int kNI = kWarpCols / 8;
  static constexpr int kRowHalfs = CI + 8;  // 16-byte pad: conflict-free ldmatrix
  static constexpr int kAStage = kConvTileRows * kRowHalfs;
  static constexpr int kBStage = CO * kRowHalfs;
  static constexpr size_t kStageBytes = (size_t)STAGES * (kAStage + kBStage) * sizeof(__half);
  // stages + live-offset list and masks + the tile's slice of the neighbour table for K offsets
  static size_t smemBytes(int K) { return kStageBytes + kMmaMaxOffsets * 8 + (size_t)K * kConvTileRows * 4; }
};

template <int CI, int CO, int STAGES>
__global__ void __launch_bounds__(256)
convMmaF16Kernel(const __half *__restrict__ features, const __half *__restrict__ filter_kcoci,
                 const int32_t *__restrict__ nbr, int64_t n_out, int64_t n_pad, int K,
                 __half *__restrict__ out) {
  using Cfg = MmaConfig<CI, CO, STAGES>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half *a_s = reinterpret_cast<__half *>(smem_raw);
  __half *b_s = a_s + STAGES * Cfg::kAStage;
  int32_t *klist_s = reinterpret_cast<int32_t *>(b_s + STAGES * Cfg::kBStage);  // live offsets
  int32_t *kmask_s = klist_s + kMmaMaxOffsets;                                 // 16-row group masks
  int32_t *nbr_s = kmask_s + kMmaMaxOffsets;                                   // [K][128]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t r0 = (int64_t)blockIdx.x * kConvTileRows;

  // Neighbour ids of the tile for every offset (the table is padded, so the
  // whole tile can be read), then which 16-row groups are live per offset.
  for (int e = tid; e < K * kConvTileRows; e += Cfg::kThreads) {
    const int k = e / kConvTileRows, r = e % kConvTileRows;
    nbr_s[e] = nbr[(size_t)k * n_pad + r0 + r];
  }
  __syncthreads();
  for (int k = warp; k < K; k += 8) {
    const int4 v = reinterpret_cast<const int4 *>(nbr_s + k * kConvTileRows)[lane];
    const unsigned any = __ballot_sync(0xffffffffu, (v.x & v.y & v.z & v.w) >= 0);
    if (lane == 0) {
      unsigned groups = 0;
      for (int g = 0; g < 8; ++g)
        if ((any >> (4 * g)) & 0xFu) groups |= 1u << g;
      kmask_s[k] = (int)groups;
    }
  }
  __syncthreads();
  __shared__ int n_live_s;
  if (tid == 0) {
    int n = 0;
    for (int k = 0; k < K; ++k)
      if (kmask_s[k]) klist_s[n++] = k;
    n_live_s = n;
  }
  __syncthreads();
  const int n_live = n_live_s;

  auto load_stage = [&](int stage, int k) {
    __half *a_dst = a_s + stage * Cfg::kAStage;
    __half *b_dst = b_s + stage * Cfg::kBStage;
    constexpr int kChunks = CI / 8;
    const int32_t *ids = nbr_s + k * kConvTileRows;
    for (int e = tid; e < kConvTileRows * kChunks; e += Cfg::kThreads) {
      const int r = e / kChunks, c = e % kChunks;
      const int idx = ids[r];
      const __half *src = features + (idx >= 0 ? (size_t)idx * CI + c * 8 : 0);
      cpAsync16(a_dst + r * Cfg::kRowHalfs + c * 8, src, idx >= 0);
    }
    const __half *wk = filter_kcoci + (size_t)k * CO * CI;
    for (int e = tid; e < CO * kChunks; e += Cfg::kThreads) {
      const int n = e / kChunks, c = e % kChunks;
      cpAsync16(b_dst + n * Cfg::kRowHalfs + c * 8, wk + (size_t)n * CI + c * 8, true);
    }
  };

  float acc[Cfg::kMI][Cfg::kNI][4];
#pragma unroll
  for (int mi = 0; mi < Cfg::kMI; ++mi)
#pragma unroll
    for (int ni = 0; ni < Cfg::kNI; ++ni)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[mi][ni][q] = 0.f;

  const int warp_m = warp / Cfg::kWarpsN, warp_n = warp % Cfg::kWarpsN;
  const int row_base = warp_m * Cfg::kWarpRows;
  const int col_base = warp_n * Cfg::kWarpCols;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < n_live) load_stage(s, klist_s[s]);
    cpAsyncCommit();
  }

  for (int it = 0; it < n_live; ++it) {
    cpAsyncWait<STAGES - 2>();
    __syncthreads();
    const int nxt = it + STAGES - 1;
    if (nxt < n_live) load_stage(nxt % STAGES, klist_s[nxt]);
    cpAsyncCommit();

    const int k = klist_s[it];
    const unsigned groups = (unsigned)kmask_s[k];
    // 16-row groups of this warp: bits row_base/16 ... (+kMI)
    const unsigned mine = (groups >> (row_base / 16)) & ((1u << Cfg::kMI) - 1u);
    if (mine == 0) continue;
    const __half *a_src = a_s + (it % STAGES) * Cfg::kAStage;
    const __half *b_src = b_s + (it % STAGES) * Cfg::kBStage;
#pragma unroll
    for (int kk = 0; kk < CI / 16; ++kk) {
      unsigned a[Cfg::kMI][4];
#pragma unroll
      for (int mi = 0; mi < Cfg::kMI; ++mi) {
        if ((mine >> mi) & 1u) {
          const int row = row_base + mi * 16 + (lane & 15);
          const int col = kk * 16 + (lane >> 4) * 8;
          ldmatrixX4(a[mi][0], a[mi][1], a[mi][2], a[mi][3], a_src + row * Cfg::kRowHalfs + col);
        }
      }
#pragma unroll
      for (int np = 0; np < Cfg::kNI / 2; ++np) {
        unsigned b[4];
        const int n = col_base + np * 16 + (lane >> 4) * 8 + (lane & 7);
        const int col = kk * 16 + ((lane >> 3) & 1) * 8;
        ldmatrixX4(b[0], b[1], b[2], b[3], b_src + n * Cfg::kRowHalfs + col);
#pragma unroll
        for (int mi = 0; mi < Cfg::kMI; ++mi) {
          if ((mine >> mi) & 1u) {
            mmaF16(acc[mi][np * 2], a[mi], b[0], b[1]);
            mmaF16(acc[mi][np * 2 + 1], a[mi], b[2], b[3]);
          }
        }
      }
    }
  }
  cpAsyncWait<0>();

  // Fragment layout of m16n8: rows lane/4 and lane/4+8, columns 2*(lane%4)+{0,1}.
#pragma unroll
  for (int mi = 0; mi < Cfg::kMI; ++mi) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int64_t r = r0 + row_base + mi * 16 + (lane >> 2) + half * 8;
      if (r >= n_out) continue;
      __half *dst = out + (size_t)r * CO + col_base + (lane & 3) * 2;
#pragma unroll
      for (int ni = 0; ni < Cfg::kNI; ++ni) {
        const __half2 v = __floats2half2_rn(acc[mi][ni][half * 2], acc[mi][ni][half * 2 + 1]);
        *reinterpret_cast<__half2 *>(dst + ni * 8) = v;
      }
    }
  }
}

template <int CI, int CO, int STAGES>
cudaError_t launchMma(const ConvProblem &p, const ConvWorkspacePlan &plan, const __half *features,
                      const __half *filter, const int32_t *nbr, __half *out, double algo_bytes,
                      double algo_flops, cudaStream_t stream) {
  using Cfg = MmaConfig<CI, CO, STAGES>;
  auto kernel = convMmaF16Kernel<CI, CO, STAGES>;
  const size_t smem = Cfg::smemBytes(p.K);
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) return err;
  const unsigned blocks = (unsigned)(plan.n_pad / kConvTileRows);
  static const std::string name =
      "convMmaF16Kernel<" + std::to_string(CI) + "," + std::to_string(CO) + ">";
  trace::Scope t(name.c_str(), stream, algo_bytes, algo_flops);
  kernel<<<blocks, Cfg::kThreads, smem, stream>>>(features, filter, nbr, p.n_out, plan.n_pad, p.K, out);
  return cudaGetLastError();
}

template <int CI>
cudaError_t dispatchMmaCo(const ConvProblem &p, const ConvWorkspacePlan &plan, const __half *features,
                          const __half *filter, const int32_t *nbr, __half *out, double algo_bytes,
                          double algo_flops, cudaStream_t stream) {
  constexpr int kStages = (CI >= 64) ? 3 : 4;
  switch (p.co) {
    case 16: return launchMma<CI, 16, kStages>(p, plan, features, filter, nbr, out, algo_bytes, algo_flops, stream);
    case 32: return launchMma<CI, 32, kStages>(p, plan, features, filter, nbr, out, algo_bytes, algo_flops, stream);
    case 64: return launchMma<CI, 64, kStages>(p, plan, features, filter, nbr, out, algo_bytes, algo_flops, stream);
    case 128: return launchMma<CI, 128, kStages>(p, plan, features, filter, nbr, out, algo_bytes, algo_flops, stream);
    default: return cudaErrorInvalidValue;
  }
}

bool mmaEligible(const ConvProblem &p, const void *features, const void *out) {
  auto pow2_16_128 = [](int c) { return c == 16 || c == 32 || c == 64 || c == 128; };
  return p.is_half && p.K <= kMmaMaxOffsets && pow2_16_128(p.ci) && pow2_16_128(p.co) &&
         (reinterpret_cast<size_t>(features) % 16 == 0) && (reinterpret_cast<size_t>(out) % 4 == 0);
}

}  // namespace

bool convRunsOnTensorMemory(const ConvProblem &caller, const void *rows_in, const void *rows_out) {
  static const char *forced = std::getenv("MLUOP_B200_CONV_KERNEL");
  if (forced && (std::strcmp(forced, "mma") == 0 || std::strcmp(forced, "fma") == 0)) return false;
  ConvProblem p = caller;
  if (caller.backward_data) {  // the rows that are gathered / produced, whichever direction runs
    p.L = caller.n_out;
    p.n_out = caller.L;
    p.ci = caller.co;
    p.co = caller.ci;
  }
  return tcgen05Eligible(p, rows_in, rows_out);
}

size_t neighbourTableBytes(const ConvProblem &p) {
  const int64_t rows_out = p.backward_data ? p.L : p.n_out;
  const int64_t n_pad = (rows_out + kConvPadRows - 1) / kConvPadRows * kConvPadRows;
  return (size_t)p.K * n_pad * sizeof(int32_t);
}

ConvWorkspacePlan planConvWorkspace(const ConvProblem &p, bool external_table) {
  ConvWorkspacePlan plan{};
  const size_t elem = p.is_half ? 2 : 4;
  const int64_t rows_out = p.backward_data ? p.L : p.n_out;
  plan.n_pad = (rows_out + kConvPadRows - 1) / kConvPadRows * kConvPadRows;
  size_t off = 0;
  plan.status = off;
  off = alignUp(off + 64 * sizeof(int32_t), 256);
  plan.filter = off;
  // room for the channel counts the tensor-core kernel pads to
  const size_t ci_room = p.is_half && tcgen05PaddedChannels(p.ci) ? tcgen05PaddedChannels(p.ci) : p.ci;
  const size_t co_room = p.is_half && tcgen05PaddedChannels(p.co) ? tcgen05PaddedChannels(p.co) : p.co;
  size_t filter_bytes = (size_t)p.K * ci_room * co_room * elem;
  if (p.is_half && tcgen05PaddedChannels(p.ci) && tcgen05PaddedChannels(p.co)) {
    // the tensor-core kernel's filter image (blocks padded to 1 KiB); the contracted channel is
    // Ci forward and Co in the input gradient, the image is as large either way round only when
    // both are taken into account
    const size_t fwd = (size_t)tcgen05FilterImage((int)ci_room, (int)co_room).bytes_per_offset;
    const size_t bwd = (size_t)tcgen05FilterImage((int)co_room, (int)ci_room).bytes_per_offset;
    const size_t image = (size_t)p.K * (fwd > bwd ? fwd : bwd);
    if (image > filter_bytes) filter_bytes = image;
  }
  off = alignUp(off + filter_bytes, 256);
  plan.neighbour = off;
  if (!external_table) off = alignUp(off + (size_t)p.K * plan.n_pad * sizeof(int32_t), 256);
  plan.counts = off;
  off = alignUp(off + (size_t)p.K * sizeof(int32_t), 256);
  plan.total = off + 256;
  return plan;
}

cudaError_t launchIndiceConvolution(const ConvProblem &caller, const ConvWorkspacePlan &plan,
                                    const void *features, const void *filters,
                                    const int32_t *indice_pairs, const int64_t *indice_num,
                                    void *workspace, void *features_out, int sm_count,
                                    cudaStream_t stream) {
  return launchIndiceConvolutionSteps(caller, plan, features, filters, indice_pairs, indice_num, workspace,
                                      features_out, sm_count, stream, nullptr, kTableBuildAndConvolve);
}

bool neighbourTableCountsFit(int32_t K) { return K <= kMaxCountsByValue; }

cudaError_t launchIndiceConvolutionSteps(const ConvProblem &caller, const ConvWorkspacePlan &plan,
                                         const void *features, const void *filters,
                                         const int32_t *indice_pairs, const int64_t *indice_num,
                                         void *workspace, void *features_out, int sm_count,
                                         cudaStream_t stream, int32_t *external_table, int steps) {
  const bool do_build = steps != kTableConvolveOnly, do_conv = steps != kTableBuildOnly;
  // From here on `p` describes the rows that are gathered (L of them, ci channels)
  // and the rows that are produced (n_out, co channels), whichever direction runs.
  ConvProblem p = caller;
  const int swap = caller.backward_data ? 1 : 0;
  if (swap) {
    p.L = caller.n_out;
    p.n_out = caller.L;
    p.ci = caller.co;
    p.co = caller.ci;
  }
  const int64_t pair_stride = caller.L;
  // Building a table alone needs no workspace (its counts travel by value).
  char *base = reinterpret_cast<char *>(alignUp(reinterpret_cast<size_t>(workspace), 256));
  void *filter_packed = workspace ? base + plan.filter : nullptr;
  int32_t *nbr = external_table ? external_table : reinterpret_cast<int32_t *>(base + plan.neighbour);
  int32_t *counts_dev = workspace ? reinterpret_cast<int32_t *>(base + plan.counts) : nullptr;
  int32_t *status = workspace ? reinterpret_cast<int32_t *>(base + plan.status) : nullptr;
  cudaError_t err;

  double pairs_total = 0;
  int64_t max_pairs = 0;
  for (int k = 0; k < p.K; ++k) {
    pairs_total += (double)indice_num[k];
    max_pairs = indice_num[k] > max_pairs ? indice_num[k] : max_pairs;
  }
  const double elem = p.is_half ? 2.0 : 4.0;
  // Algorithmic work of the convolution: per pair one gathered input row, one
  // scattered output row and two int32 ids; 2*Ci*Co flops.
  const double conv_bytes = pairs_total * ((p.ci + p.co) * elem + 8.0);
  const double conv_flops = 2.0 * pairs_total * p.ci * p.co;

  // Half with channel counts that are multiples of 8 up to 128 runs on the tcgen05 tensor
  // cores (odd counts at the next of 16/32/64/128, zero padded); MLUOP_B200_CONV_KERNEL=mma
  // selects the mma.sync variant instead (kept for cross-checking), =fma the plain FMA kernels.
  const bool use_tc = do_conv && convRunsOnTensorMemory(caller, features, features_out);
  static const char *forced = std::getenv("MLUOP_B200_CONV_KERNEL");
  const bool force_fma = forced && std::strcmp(forced, "fma") == 0;
  if (do_conv && caller.mirror_table && !use_tc) return cudaErrorNotSupported;

  // 1. filter -> [K][Co][Ci] (channel counts padded for the tensor-core kernel) and
  // 2. the neighbour table filled with -1; one launch does both when the call needs both
  const size_t table_bytes = (size_t)p.K * plan.n_pad * sizeof(int32_t);  // n_pad is a multiple of 512 rows
  if (do_conv) {
    const int n_dst = use_tc ? tcgen05PaddedChannels(p.co) : p.co;
    const int c_dst = use_tc ? tcgen05PaddedChannels(p.ci) : p.ci;
    const int64_t total = (int64_t)p.K * n_dst * c_dst;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    const int64_t table_vec = do_build ? (int64_t)(table_bytes / sizeof(int4)) : 0;
    // fill: 16 stores of 16 bytes per thread, at most 32 blocks per SM
    int64_t fill_blocks = (table_vec + 256 * 16 - 1) / (256 * 16);
    const int64_t fill_cap = (int64_t)(sm_count > 0 ? sm_count : 148) * 32;
    if (fill_blocks > fill_cap) fill_blocks = fill_cap;
    Tcgen05FilterImage image{0, 0, 0};
    if (use_tc) image = tcgen05FilterImage(c_dst, n_dst);
    trace::Scope t(do_build ? "repackFilterKernel+fill" : "repackFilterKernel", stream,
                   2.0 * total * elem + (double)(do_build ? table_bytes : 0));
    if (p.is_half) {
      repackFilterKernel<__half><<<blocks + (unsigned)fill_blocks, 256, 0, stream>>>(
          static_cast<const __half *>(filters), static_cast<__half *>(filter_packed), p.K, caller.ci, caller.co,
          p.filter_layout, swap, n_dst, c_dst, blocks, reinterpret_cast<int4 *>(nbr), table_vec, status,
          image.row_bytes, image.block_stride, image.bytes_per_offset);
    } else {
      repackFilterKernel<float><<<blocks + (unsigned)fill_blocks, 256, 0, stream>>>(
          static_cast<const float *>(filters), static_cast<float *>(filter_packed), p.K, caller.ci, caller.co,
          p.filter_layout, swap, n_dst, c_dst, blocks, reinterpret_cast<int4 *>(nbr), table_vec, status,
          image.row_bytes, image.block_stride, image.bytes_per_offset);
    }
  } else if (do_build) {
    trace::Scope t("memset:neighbour_table", stream, (double)table_bytes);
    if ((err = cudaMemsetAsync(nbr, 0xFF, table_bytes, stream)) != cudaSuccess) return err;
  }
  if (do_build && max_pairs > 0) {
    int64_t bx = (max_pairs + 256 * kBuildPairsPerThread - 1) / (256 * kBuildPairsPerThread);
    const int64_t cap = (int64_t)sm_count * 32;
    if (bx > cap) bx = cap;
    const dim3 grid((unsigned)bx, (unsigned)p.K);
    trace::Scope t("buildNeighbourKernel", stream, 12.0 * pairs_total);
    if (p.K <= kMaxCountsByValue) {
      PairCounts counts{};
      for (int k = 0; k < p.K; ++k) counts.n[k] = (int32_t)indice_num[k];
      buildNeighbourKernel<true><<<grid, 256, 0, stream>>>(indice_pairs, pair_stride, swap, p.L, p.n_out,
                                                           plan.n_pad, counts, nullptr, nbr);
    } else {
      // Large kernel volumes: counts travel through device memory.  The copy
      // from pageable host memory is staged by the runtime before it returns.
      int32_t *tmp = new int32_t[p.K];
      for (int k = 0; k < p.K; ++k) tmp[k] = (int32_t)indice_num[k];
      err = cudaMemcpyAsync(counts_dev, tmp, (size_t)p.K * sizeof(int32_t), cudaMemcpyHostToDevice, stream);
      delete[] tmp;
      if (err != cudaSuccess) return err;
      buildNeighbourKernel<false><<<grid, 256, 0, stream>>>(indice_pairs, pair_stride, swap, p.L, p.n_out,
                                                            plan.n_pad, PairCounts{}, counts_dev, nbr);
    }
  }
  if ((err = cudaGetLastError()) != cudaSuccess) return err;
  if (!do_conv) return cudaSuccess;

  // 3. convolution
  if (use_tc) {
    return launchConvTcgen05(p, plan, static_cast<const __half *>(features),
                             static_cast<const __half *>(filter_packed), nbr,
                             static_cast<__half *>(features_out), status, conv_bytes, conv_flops, stream);
  }
  if (!force_fma && mmaEligible(p, features, features_out)) {
    const __half *f = static_cast<const __half *>(features);
    const __half *w = static_cast<const __half *>(filter_packed);
    __half *o = static_cast<__half *>(features_out);
    switch (p.ci) {
      case 16: return dispatchMmaCo<16>(p, plan, f, w, nbr, o, conv_bytes, conv_flops, stream);
      case 32: return dispatchMmaCo<32>(p, plan, f, w, nbr, o, conv_bytes, conv_flops, stream);
      case 64: return dispatchMmaCo<64>(p, plan, f, w, nbr, o, conv_bytes, conv_flops, stream);
      default: return dispatchMmaCo<128>(p, plan, f, w, nbr, o, conv_bytes, conv_flops, stream);
    }
  }
  if ((int64_t)p.K * p.ci * p.co <= kSmallFilterFloats && p.co <= 32 && p.co % 4 == 0) {
    constexpr int kNout = 4;
    const int64_t threads = p.n_out * (p.co / kNout);
    const unsigned blocks = (unsigned)((threads + 255) / 256);
    const size_t smem = (size_t)p.K * p.ci * p.co * sizeof(float);
    if (p.is_half) {
      trace::Scope t("convSmallFilterKernel<half>", stream, conv_bytes, conv_flops);
      convSmallFilterKernel<__half, kNout><<<blocks, 256, smem, stream>>>(
          static_cast<const __half *>(features), static_cast<const __half *>(filter_packed), nbr, p.n_out,
          plan.n_pad, p.K, p.ci, p.co, static_cast<__half *>(features_out));
    } else {
      trace::Scope t("convSmallFilterKernel<float>", stream, conv_bytes, conv_flops);
      convSmallFilterKernel<float, kNout><<<blocks, 256, smem, stream>>>(
          static_cast<const float *>(features), static_cast<const float *>(filter_packed), nbr, p.n_out,
          plan.n_pad, p.K, p.ci, p.co, static_cast<float *>(features_out));
    }
    return cudaGetLastError();
  }
  const dim3 grid((unsigned)((p.n_out + kGenRows - 1) / kGenRows), (unsigned)((p.co + kGenCols - 1) / kGenCols));
  if (p.is_half) {
    trace::Scope t("convGenericKernel<half>", stream, conv_bytes, conv_flops);
    convGenericKernel<__half><<<grid, kGenRows * kGenLanes, 0, stream>>>(
        static_cast<const __half *>(features), static_cast<const __half *>(filter_packed), nbr, p.n_out,
        plan.n_pad, p.K, p.ci, p.co, static_cast<__half *>(features_out));
  } else {
    trace::Scope t("convGenericKernel<float>", stream, conv_bytes, conv_flops);
    convGenericKernel<float><<<grid, kGenRows * kGenLanes, 0, stream>>>(
        static_cast<const float *>(features), static_cast<const float *>(filter_packed), nbr, p.n_out,
        plan.n_pad, p.K, p.ci, p.co, static_cast<float *>(features_out));
  }
  return cudaGetLastError();
}

}  // namespace sparse_conv
}  // namespace mluop
