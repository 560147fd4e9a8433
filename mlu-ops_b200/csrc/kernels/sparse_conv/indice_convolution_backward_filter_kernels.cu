// Filter gradient of the sparse convolution for sm_100a.
//
//   filters_grad[k,c,n] = sum_{(i,o) in pairs_k} features[i,c] * output_grad[o,n]
//
// (reference kernels/sparse_conv/indice_convolution_backward_filter/
// indice_convolution_backward_filter.cpp:322-520: a fill of filters_grad, then
// per kernel offset two gathers into dense [P_k,Ci] / [P_k,Co] buffers and a
// transposed matmul.)
//
// Per kernel offset this is a [Ci x P_k] x [P_k x Co] product whose long axis is
// the pair list.  A thread block takes one segment of one pair list, gathers
// the two rows of every pair into shared memory (cp.async, 16 bytes at a time),
// and accumulates the [Ci x Co] product in float:
//   filterGradMmaKernel      half, Ci in {4,8,16,32,64,128}, Co in {16,32,64,128}: mma.sync m16n8k16;
//                            both operands lie pair-major in shared memory, so
//                            both fragments come from ldmatrix.trans
//   filterGradSmallKernel    Ci*Co <= 256 (a backbone's first layer): one thread per
//                            output element, pairs dealt round-robin to thread groups
//   filterGradGenericKernel  float, and half with other channel counts: FMA
// Every block writes its float partial; reduceFilterGradKernel adds the partials
// of an offset in ascending segment order and converts to the output type, so
// the result is reproducible.  Offsets without pairs give zeros.
#include "kernels/sparse_conv/indice_convolution_backward_filter_kernels.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <string>

#include "core/trace.h"
#include "kernels/sparse_conv/indice_convolution_backward_filter_tcgen05.h"

namespace mluop {
namespace sparse_conv {

namespace {

inline size_t alignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

__device__ __forceinline__ float toFloat(float v) { return v; }
__device__ __forceinline__ float toFloat(__half v) { return __half2float(v); }
__device__ __forceinline__ void fromFloat(float v, float *dst) { *dst = v; }
__device__ __forceinline__ void fromFloat(float v, __half *dst) { *dst = __float2half_rn(v); }

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
// Four 8x8 b16 matrices, each delivered transposed: lane (g = lane/4, t = lane%4)
// receives elements [2t][g] and [2t+1][g] of the matrix as it lies in memory.
__device__ __forceinline__ void ldmatrixX4Trans(unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3,
                                                const void *smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
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

// ------------------------------------------------------------ tensor cores

// 8 warps tile the [Ci x Co] product as kWarpsM x kWarpsN (up to 4 x 2); when the
// product is too small for eight tiles the remaining factor kWarpsK splits the
// pairs of a stage between warps (summed through shared memory at the end).
// (Wider warp tiles with a four-way pair split measured 35 % slower at 64 x 64.)
// CI_REAL < CI (4 or 8 channels, a backbone's first layer): feature rows are
// CI_REAL halves long and sit in the first columns of zero-filled 16-column rows.
template <int CI, int CO, int CI_REAL>
struct GradMmaConfig {
  static constexpr int kThreads = 256;
  static constexpr int kTilesM = CI / 16, kTilesN = CO / 8;
  static constexpr int kWarpsM = kTilesM < 4 ? kTilesM : 4;
  static constexpr int kWarpsN = (kTilesN / 2) < 2 ? (kTilesN / 2) : 2;
  static constexpr int kWarpsK = 8 / (kWarpsM * kWarpsN);
  static constexpr int kMI = kTilesM / kWarpsM;  // m16 tiles per warp
  static constexpr int kNI = kTilesN / kWarpsN;  // n8 tiles per warp (even)
  // about 16 KB of rows per stage: 64 pairs at 64+64 channels, up to 256 at 16+16;
  // every warp of a split needs a 16-pair slice per stage
  static constexpr int kByBytes = 8192 / (CI + CO);
  static constexpr int kByBytesPow2 = kByBytes >= 256 ? 256 : (kByBytes >= 128 ? 128 : 64);
  static constexpr int kStagePairs = kByBytesPow2 > 16 * kWarpsK ? kByBytesPow2 : 16 * kWarpsK;
  // two stages: shared memory then allows as many blocks per SM as the registers do (six at
  // 64 x 64), which measured faster than three or four stages with fewer blocks
  static constexpr int kStages = 2;
  static constexpr int kStrideA = CI + 8, kStrideB = CO + 8;  // halves; 16-byte pad: conflict-free ldmatrix
  static constexpr int kStageHalves = kStagePairs * (kStrideA + kStrideB);
  static constexpr size_t kPipeBytes = (size_t)kStages * kStageHalves * sizeof(__half);
  static constexpr size_t kSumBytes = (size_t)kWarpsK * CI * CO * sizeof(float);
  static constexpr size_t kRowsBytes = kPipeBytes > kSumBytes ? kPipeBytes : kSumBytes;
  // after the rows: two slots of pair ids (feature row, output_grad row) of one stage each
  static constexpr size_t kIdBytes = (size_t)2 * 2 * kStagePairs * sizeof(int32_t);
  static constexpr size_t kSmemBytes = kRowsBytes + kIdBytes;
};

__device__ __forceinline__ void cpAsync8(void *smem, const void *gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 8 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}

template <int CI, int CO, int CI_REAL>
__global__ void __launch_bounds__(256)
filterGradMmaKernel(const __half *__restrict__ features, const __half *__restrict__ output_grad,
                    const int32_t *__restrict__ pairs, const int32_t *__restrict__ counts, int64_t L,
                    int seg_pairs, int max_segments, float *__restrict__ partial) {
  using Cfg = GradMmaConfig<CI, CO, CI_REAL>;
  const int k = blockIdx.y, seg = blockIdx.x;
  const int64_t pk = counts[k];
  const int64_t begin = (int64_t)seg * seg_pairs;
  if (begin >= pk) return;
  const int64_t end = begin + seg_pairs < pk ? begin + seg_pairs : pk;
  const int32_t *in_row = pairs + (size_t)k * 2 * L;
  const int32_t *out_row = in_row + L;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half *stage_s = reinterpret_cast<__half *>(smem_raw);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wk = warp % Cfg::kWarpsK;
  const int wn = (warp / Cfg::kWarpsK) % Cfg::kWarpsN;
  const int wm = warp / (Cfg::kWarpsK * Cfg::kWarpsN);
  const int m_base = wm * Cfg::kMI * 16, n_base = wn * Cfg::kNI * 8;

  float acc[Cfg::kMI][Cfg::kNI][4];
#pragma unroll
  for (int mi = 0; mi < Cfg::kMI; ++mi)
#pragma unroll
    for (int ni = 0; ni < Cfg::kNI; ++ni)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[mi][ni][e] = 0.0f;

  const int n_stages = (int)((end - begin + Cfg::kStagePairs - 1) / Cfg::kStagePairs);

  // Pair ids reach shared memory one stage before the rows that they address are
  // requested, so that no cp.async waits for a dependent global load: they are
  // read into registers before a stage is computed and stored after it.
  int32_t *ids_s = reinterpret_cast<int32_t *>(smem_raw + Cfg::kRowsBytes);  // [2][2][kStagePairs]
  constexpr int kIdsPerThread = (2 * Cfg::kStagePairs + Cfg::kThreads - 1) / Cfg::kThreads;
  int32_t id_reg[kIdsPerThread];
  auto fetchIds = [&](int s) {
    const int64_t base = begin + (int64_t)s * Cfg::kStagePairs;
#pragma unroll
    for (int i = 0; i < kIdsPerThread; ++i) {
      const int r = tid + i * Cfg::kThreads;
      const int rr = r < Cfg::kStagePairs ? r : r - Cfg::kStagePairs;
      const int32_t *src = r < Cfg::kStagePairs ? in_row : out_row;
      id_reg[i] = (r < 2 * Cfg::kStagePairs && base + rr < end) ? src[base + rr] : -1;
    }
  };
  auto storeIds = [&](int s) {
    int32_t *slot = ids_s + (s & 1) * 2 * Cfg::kStagePairs;
#pragma unroll
    for (int i = 0; i < kIdsPerThread; ++i) {
      const int r = tid + i * Cfg::kThreads;
      if (r < 2 * Cfg::kStagePairs) slot[r] = id_reg[i];
    }
  };
  // 16-byte chunks of one stage: first the feature rows, then the output_grad rows
  constexpr int kChunksA = CI_REAL < 8 ? 1 : CI_REAL / 8, kChunksB = CO / 8;
  constexpr int kStageChunks = Cfg::kStagePairs * (kChunksA + kChunksB);
  auto issue = [&](int s, bool ids_in_smem) {
    __half *a_s = stage_s + (size_t)(s % Cfg::kStages) * Cfg::kStageHalves;
    __half *b_s = a_s + Cfg::kStagePairs * Cfg::kStrideA;
    const int32_t *slot = ids_s + (s & 1) * 2 * Cfg::kStagePairs;
    const int64_t base = begin + (int64_t)s * Cfg::kStagePairs;
    for (int c = tid; c < kStageChunks; c += Cfg::kThreads) {
      if (c < Cfg::kStagePairs * kChunksA) {
        const int r = c / kChunksA, ch = c % kChunksA;
        const int32_t id = ids_in_smem ? slot[r] : (base + r < end ? in_row[base + r] : -1);
        const __half *src = features + (int64_t)(id < 0 ? 0 : id) * CI_REAL + ch * 8;
        if (CI_REAL < 8) {
          cpAsync8(a_s + r * Cfg::kStrideA, src, id >= 0);
        } else {
          cpAsync16(a_s + r * Cfg::kStrideA + ch * 8, src, id >= 0);
        }
      } else {
        const int c2 = c - Cfg::kStagePairs * kChunksA;
        const int r = c2 / kChunksB, ch = c2 % kChunksB;
        const int32_t id =
            ids_in_smem ? slot[Cfg::kStagePairs + r] : (base + r < end ? out_row[base + r] : -1);
        cpAsync16(b_s + r * Cfg::kStrideB + ch * 8, output_grad + (int64_t)(id < 0 ? 0 : id) * CO + ch * 8, id >= 0);
      }
    }
  };

  if (CI_REAL < CI) {
    // columns CI_REAL.. of the feature rows are never copied to: zero them once
    for (int e = tid; e < Cfg::kStages * Cfg::kStageHalves / 8; e += Cfg::kThreads)
      reinterpret_cast<uint4 *>(stage_s)[e] = make_uint4(0, 0, 0, 0);
    __syncthreads();
  }
  // prologue: the first stages read their ids straight from global memory; the ids of
  // the stage that iteration 0 requests go to shared memory
#pragma unroll
  for (int s = 0; s < Cfg::kStages - 1; ++s) {
    if (s < n_stages) issue(s, false);
    cpAsyncCommit();
  }
  if (Cfg::kStages - 1 < n_stages) {
    fetchIds(Cfg::kStages - 1);
    storeIds(Cfg::kStages - 1);
  }
  const int j = lane >> 3, r8 = lane & 7;
  for (int s = 0; s < n_stages; ++s) {
    cpAsyncWait<Cfg::kStages - 2>();
    __syncthreads();
    if (s + Cfg::kStages - 1 < n_stages) issue(s + Cfg::kStages - 1, true);
    cpAsyncCommit();
    const bool more_ids = s + Cfg::kStages < n_stages;
    if (more_ids) fetchIds(s + Cfg::kStages);
    const __half *a_s = stage_s + (size_t)(s % Cfg::kStages) * Cfg::kStageHalves;
    const __half *b_s = a_s + Cfg::kStagePairs * Cfg::kStrideA;
#pragma unroll
    for (int ks = wk; ks < Cfg::kStagePairs / 16; ks += Cfg::kWarpsK) {
      const int k0 = ks * 16;
      unsigned a[Cfg::kMI][4];
#pragma unroll
      for (int mi = 0; mi < Cfg::kMI; ++mi) {
        // matrices: (pairs k0..+7, m..+7), (k0..+7, m+8..), (k0+8.., m..), (k0+8.., m+8..)
        const int m0 = m_base + mi * 16;
        ldmatrixX4Trans(a[mi][0], a[mi][1], a[mi][2], a[mi][3],
                        a_s + (k0 + (j >> 1) * 8 + r8) * Cfg::kStrideA + m0 + (j & 1) * 8);
      }
#pragma unroll
      for (int ni = 0; ni < Cfg::kNI; ni += 2) {
        // matrices: (k0..+7, n..+7), (k0+8.., n..+7), (k0..+7, n+8..), (k0+8.., n+8..)
        const int n0 = n_base + ni * 8;
        unsigned b[4];
        ldmatrixX4Trans(b[0], b[1], b[2], b[3],
                        b_s + (k0 + (j & 1) * 8 + r8) * Cfg::kStrideB + n0 + (j >> 1) * 8);
#pragma unroll
        for (int mi = 0; mi < Cfg::kMI; ++mi) {
          mmaF16(acc[mi][ni], a[mi], b[0], b[1]);
          mmaF16(acc[mi][ni + 1], a[mi], b[2], b[3]);
        }
      }
    }
    if (more_ids) storeIds(s + Cfg::kStages);
  }
  cpAsyncWait<0>();
  __syncthreads();

  // Sum over the warps that shared a tile (fixed order), then write the partial.
  float *sum_s = reinterpret_cast<float *>(smem_raw);  // [kWarpsK][CI][CO]
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int mi = 0; mi < Cfg::kMI; ++mi)
#pragma unroll
    for (int ni = 0; ni < Cfg::kNI; ++ni) {
      const int m = m_base + mi * 16 + g, n = n_base + ni * 8 + 2 * t;
      float *dst = sum_s + (size_t)wk * CI * CO;
      *reinterpret_cast<float2 *>(dst + m * CO + n) = make_float2(acc[mi][ni][0], acc[mi][ni][1]);
      *reinterpret_cast<float2 *>(dst + (m + 8) * CO + n) = make_float2(acc[mi][ni][2], acc[mi][ni][3]);
    }
  __syncthreads();
  float *dst = partial + ((size_t)k * max_segments + seg) * CI_REAL * CO;
  for (int e = tid; e < CI_REAL * CO; e += Cfg::kThreads) {
    float v = sum_s[e];
#pragma unroll
    for (int w = 1; w < Cfg::kWarpsK; ++w) v += sum_s[(size_t)w * CI * CO + e];
    dst[e] = v;
  }
}

// ------------------------------------------------------------ generic FMA

constexpr int kGenTile = 64;        // block computes a 64 x 64 tile of [Ci x Co]
constexpr int kGenStagePairs = 16;  // pairs staged per step

// Thread (ty, tx) of a 16 x 16 block owns the 4 x 4 outputs (4ty.., 4tx..) of the tile.
template <typename T>
__global__ void __launch_bounds__(256)
filterGradGenericKernel(const T *__restrict__ features, const T *__restrict__ output_grad,
                        const int32_t *__restrict__ pairs, const int32_t *__restrict__ counts, int64_t L,
                        int ci, int co, int seg_pairs, int max_segments, float *__restrict__ partial) {
  const int k = blockIdx.y, seg = blockIdx.x;
  const int tiles_n = (co + kGenTile - 1) / kGenTile;
  const int c0 = (blockIdx.z / tiles_n) * kGenTile, n0 = (blockIdx.z % tiles_n) * kGenTile;
  const int64_t pk = counts[k];
  const int64_t begin = (int64_t)seg * seg_pairs;
  if (begin >= pk) return;
  const int64_t end = begin + seg_pairs < pk ? begin + seg_pairs : pk;
  const int32_t *in_row = pairs + (size_t)k * 2 * L;
  const int32_t *out_row = in_row + L;

  __shared__ float a_s[kGenStagePairs][kGenTile];
  __shared__ float b_s[kGenStagePairs][kGenTile];
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  float acc[4][4] = {};
  for (int64_t base = begin; base < end; base += kGenStagePairs) {
    for (int e = tid; e < kGenStagePairs * kGenTile; e += 256) {
      const int r = e / kGenTile, c = e % kGenTile;
      const bool live = base + r < end;
      a_s[r][c] = (live && c0 + c < ci) ? toFloat(features[(int64_t)in_row[base + r] * ci + c0 + c]) : 0.0f;
      b_s[r][c] = (live && n0 + c < co) ? toFloat(output_grad[(int64_t)out_row[base + r] * co + n0 + c]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kGenStagePairs; ++r) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = a_s[r][4 * ty + i];
        b[i] = b_s[r][4 * tx + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[i][q] = fmaf(a[i], b[q], acc[i][q]);
    }
    __syncthreads();
  }
  float *dst = partial + ((size_t)k * max_segments + seg) * ci * co;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int c = c0 + 4 * ty + i, n = n0 + 4 * tx + q;
      if (c < ci && n < co) dst[(size_t)c * co + n] = acc[i][q];
    }
}

// ------------------------------------------------------------ narrow filters

constexpr int kSmallOutputs = 256;  // Ci*Co up to this: one thread per output element
constexpr int kSmallUnroll = 4;

// Ci*Co <= 256 (the first layer of a backbone: 4 -> 16 channels).  Thread t owns
// output element t % (Ci*Co) and, of its segment, the pairs g, g+G, ... with
// g = t / (Ci*Co) and G = 256 / (Ci*Co); the G sums are added in ascending g.
template <typename T>
__global__ void __launch_bounds__(256)
filterGradSmallKernel(const T *__restrict__ features, const T *__restrict__ output_grad,
                      const int32_t *__restrict__ pairs, const int32_t *__restrict__ counts, int64_t L,
                      int ci, int co, int seg_pairs, int max_segments, float *__restrict__ partial) {
  const int k = blockIdx.y, seg = blockIdx.x;
  const int64_t pk = counts[k];
  const int64_t begin = (int64_t)seg * seg_pairs;
  if (begin >= pk) return;
  const int64_t end = begin + seg_pairs < pk ? begin + seg_pairs : pk;
  const int32_t *in_row = pairs + (size_t)k * 2 * L;
  const int32_t *out_row = in_row + L;
  const int per = ci * co, groups = 256 / per;
  const int tid = threadIdx.x, g = tid / per, e = tid % per;
  const int c = e / co, n = e % co;
  __shared__ float sum_s[256];
  float acc = 0.0f;
  if (g < groups) {
    for (int64_t p = begin + g; p < end; p += (int64_t)kSmallUnroll * groups) {
      float a[kSmallUnroll], b[kSmallUnroll];
#pragma unroll
      for (int u = 0; u < kSmallUnroll; ++u) {
        const int64_t q = p + (int64_t)u * groups;
        const bool live = q < end;
        a[u] = live ? toFloat(features[(int64_t)in_row[q] * ci + c]) : 0.0f;
        b[u] = live ? toFloat(output_grad[(int64_t)out_row[q] * co + n]) : 0.0f;
      }
#pragma unroll
      for (int u = 0; u < kSmallUnroll; ++u) acc = fmaf(a[u], b[u], acc);
    }
  }
  sum_s[tid] = acc;
  __syncthreads();
  if (tid < per) {
    float v = sum_s[tid];
    for (int w = 1; w < groups; ++w) v += sum_s[w * per + tid];
    partial[((size_t)k * max_segments + seg) * per + tid] = v;
  }
}

// ------------------------------------------------------------ reduction

template <typename T>
__global__ void __launch_bounds__(256)
reduceFilterGradKernel(const float *__restrict__ partial, const int32_t *__restrict__ counts, int K,
                       int64_t cico, int seg_pairs, int max_segments, T *__restrict__ filters_grad) {
  const int64_t total = (int64_t)K * cico;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int k = (int)(i / cico);
    const int64_t e = i % cico;
    const int segs = (counts[k] + seg_pairs - 1) / seg_pairs;
    const float *src = partial + (size_t)k * max_segments * cico + e;
    float v = 0.0f;
    for (int s = 0; s < segs; ++s) v += src[(size_t)s * cico];
    fromFloat(v, filters_grad + i);
  }
}

template <int CI, int CO, int CI_REAL>
cudaError_t launchGradMma(const FilterGradProblem &p, const FilterGradWorkspacePlan &plan,
                          const __half *features, const __half *output_grad, const int32_t *pairs,
                          const int32_t *counts, float *partial, double bytes, double flops,
                          cudaStream_t stream) {
  using Cfg = GradMmaConfig<CI, CO, CI_REAL>;
  auto kernel = filterGradMmaKernel<CI, CO, CI_REAL>;
  cudaError_t err =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::kSmemBytes);
  if (err != cudaSuccess) return err;
  static const std::string name =
      "filterGradMmaKernel<" + std::to_string(CI_REAL) + "," + std::to_string(CO) + ">";
  trace::Scope t(name.c_str(), stream, bytes, flops);
  const dim3 grid((unsigned)plan.max_segments, (unsigned)p.K);
  kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(features, output_grad, pairs, counts, p.L,
                                                          plan.seg_pairs, plan.max_segments, partial);
  return cudaGetLastError();
}

template <int CI, int CI_REAL>
cudaError_t dispatchGradMmaCo(const FilterGradProblem &p, const FilterGradWorkspacePlan &plan,
                              const __half *f, const __half *g, const int32_t *pairs, const int32_t *counts,
                              float *partial, double bytes, double flops, cudaStream_t stream) {
  switch (p.co) {
    case 16: return launchGradMma<CI, 16, CI_REAL>(p, plan, f, g, pairs, counts, partial, bytes, flops, stream);
    case 32: return launchGradMma<CI, 32, CI_REAL>(p, plan, f, g, pairs, counts, partial, bytes, flops, stream);
    case 64: return launchGradMma<CI, 64, CI_REAL>(p, plan, f, g, pairs, counts, partial, bytes, flops, stream);
    case 128: return launchGradMma<CI, 128, CI_REAL>(p, plan, f, g, pairs, counts, partial, bytes, flops, stream);
    default: return cudaErrorInvalidValue;
  }
}

bool gradMmaEligible(const FilterGradProblem &p, const void *features, const void *output_grad) {
  auto ok_ci = [](int c) { return c == 4 || c == 8 || c == 16 || c == 32 || c == 64 || c == 128; };
  auto ok_co = [](int c) { return c == 16 || c == 32 || c == 64 || c == 128; };
  const size_t row_align = p.ci == 4 ? 8 : 16;
  return p.is_half && ok_ci(p.ci) && ok_co(p.co) && reinterpret_cast<size_t>(features) % row_align == 0 &&
         reinterpret_cast<size_t>(output_grad) % 16 == 0;
}

}  // namespace

FilterGradWorkspacePlan planFilterGradWorkspace(const FilterGradProblem &p, const int64_t *indice_num,
                                                int sm_count) {
  FilterGradWorkspacePlan plan{};
  int64_t max_pairs = 0, total_pairs = 0;
  for (int k = 0; k < p.K; ++k) {
    max_pairs = indice_num[k] > max_pairs ? indice_num[k] : max_pairs;
    total_pairs += indice_num[k];
  }
  // About sixteen blocks per SM (four waves at four resident blocks, so that the
  // last wave costs little); at least 1024 pairs per block so that the partials
  // stay small next to the gathered rows.
  const int64_t blocks = (int64_t)(sm_count > 0 ? sm_count : 148) * 16;
  int64_t seg = (total_pairs + blocks - 1) / blocks;
  if (seg < 1024) seg = 1024;
  seg = (seg + 127) / 128 * 128;
  // Wide filters: fewer, longer segments so that the partials stay below 128 MiB.
  const int64_t partial_cap = (int64_t)128 << 20;
  while ((max_pairs + seg - 1) / seg > 1 &&
         (int64_t)p.K * ((max_pairs + seg - 1) / seg) * p.ci * p.co * 4 > partial_cap) {
    seg *= 2;
  }
  plan.seg_pairs = (int32_t)seg;
  plan.max_segments = (int32_t)((max_pairs + seg - 1) / seg);
  if (plan.max_segments < 1) plan.max_segments = 1;
  size_t off = 0;
  plan.counts = off;
  off = alignUp(off + (size_t)p.K * sizeof(int32_t), 256);
  plan.partial = off;
  off = alignUp(off + (size_t)p.K * plan.max_segments * p.ci * p.co * sizeof(float), 256);
  // The tensor-memory kernel is chosen by shape; should the pointers of the call
  // turn out misaligned the pair-list kernels run in the same workspace.
  plan.use_tc = filterGradTcShapeEligible(p) ? 1 : 0;
  if (plan.use_tc) {
    const FilterGradTcPlan tc = planFilterGradTc(p, sm_count);
    size_t tc_off = plan.partial;
    plan.tc_status = tc_off;
    tc_off = alignUp(tc_off + 64 * sizeof(int32_t), 256);
    plan.tc_table = tc_off;
    tc_off = alignUp(tc_off + tc.table_bytes, 256);
    plan.tc_partial = tc_off;
    tc_off = alignUp(tc_off + tc.partial_bytes, 256);
    if (tc_off > off) off = tc_off;
  }
  plan.total = off + 256;
  return plan;
}

bool filterGradRunsFromTable(const FilterGradProblem &p, const FilterGradWorkspacePlan &plan, const void *features,
                             const void *output_grad) {
  (void)p;
  return plan.use_tc && reinterpret_cast<size_t>(features) % 16 == 0 && reinterpret_cast<size_t>(output_grad) % 16 == 0;
}

cudaError_t launchIndiceConvolutionBackwardFilter(const FilterGradProblem &p,
                                                  const FilterGradWorkspacePlan &plan,
                                                  const void *features, const void *output_grad,
                                                  const int32_t *indice_pairs,
                                                  const int64_t *indice_num, void *workspace,
                                                  void *filters_grad, int sm_count, cudaStream_t stream,
                                                  const int32_t *forward_table) {
  char *base = reinterpret_cast<char *>(alignUp(reinterpret_cast<size_t>(workspace), 256));
  int32_t *counts = reinterpret_cast<int32_t *>(base + plan.counts);
  float *partial = reinterpret_cast<float *>(base + plan.partial);
  cudaError_t err;

  // Pair counts travel through device memory.  The copy from pageable host
  // memory is staged by the runtime before it returns.
  double pairs_total = 0;
  {
    int32_t *tmp = new int32_t[p.K];
    for (int k = 0; k < p.K; ++k) {
      tmp[k] = (int32_t)indice_num[k];
      pairs_total += (double)indice_num[k];
    }
    err = cudaMemcpyAsync(counts, tmp, (size_t)p.K * sizeof(int32_t), cudaMemcpyHostToDevice, stream);
    delete[] tmp;
    if (err != cudaSuccess) return err;
  }
  const double elem = p.is_half ? 2.0 : 4.0;
  // Algorithmic work: per pair one feature row, one output_grad row and two ids;
  // the filter gradient written once; 2*Ci*Co flops per pair.
  const double bytes = pairs_total * ((p.ci + p.co) * elem + 8.0) + (double)p.K * p.ci * p.co * elem;
  const double flops = 2.0 * pairs_total * p.ci * p.co;

  if (filterGradRunsFromTable(p, plan, features, output_grad)) {
    return launchFilterGradTcgen05(p, planFilterGradTc(p, sm_count), features, output_grad, indice_pairs, indice_num,
                                   reinterpret_cast<int32_t *>(base + plan.tc_table),
                                   reinterpret_cast<float *>(base + plan.tc_partial),
                                   reinterpret_cast<int32_t *>(base + plan.tc_status), filters_grad, sm_count, bytes,
                                   flops, stream, forward_table);
  }
  if (forward_table != nullptr) return cudaErrorNotSupported;  // the pair-list kernels have no use for a table
  if (gradMmaEligible(p, features, output_grad)) {
    const __half *f = static_cast<const __half *>(features);
    const __half *g = static_cast<const __half *>(output_grad);
    switch (p.ci) {
      case 4: err = dispatchGradMmaCo<16, 4>(p, plan, f, g, indice_pairs, counts, partial, bytes, flops, stream); break;
      case 8: err = dispatchGradMmaCo<16, 8>(p, plan, f, g, indice_pairs, counts, partial, bytes, flops, stream); break;
      case 16: err = dispatchGradMmaCo<16, 16>(p, plan, f, g, indice_pairs, counts, partial, bytes, flops, stream); break;
      case 32: err = dispatchGradMmaCo<32, 32>(p, plan, f, g, indice_pairs, counts, partial, bytes, flops, stream); break;
      case 64: err = dispatchGradMmaCo<64, 64>(p, plan, f, g, indice_pairs, counts, partial, bytes, flops, stream); break;
      default: err = dispatchGradMmaCo<128, 128>(p, plan, f, g, indice_pairs, counts, partial, bytes, flops, stream); break;
    }
  } else if (p.ci * p.co <= kSmallOutputs) {
    const dim3 grid((unsigned)plan.max_segments, (unsigned)p.K);
    if (p.is_half) {
      trace::Scope t("filterGradSmallKernel<half>", stream, bytes, flops);
      filterGradSmallKernel<__half><<<grid, 256, 0, stream>>>(
          static_cast<const __half *>(features), static_cast<const __half *>(output_grad), indice_pairs, counts,
          p.L, p.ci, p.co, plan.seg_pairs, plan.max_segments, partial);
    } else {
      trace::Scope t("filterGradSmallKernel<float>", stream, bytes, flops);
      filterGradSmallKernel<float><<<grid, 256, 0, stream>>>(
          static_cast<const float *>(features), static_cast<const float *>(output_grad), indice_pairs, counts,
          p.L, p.ci, p.co, plan.seg_pairs, plan.max_segments, partial);
    }
    err = cudaGetLastError();
  } else {
    const int tiles = ((p.ci + kGenTile - 1) / kGenTile) * ((p.co + kGenTile - 1) / kGenTile);
    const dim3 grid((unsigned)plan.max_segments, (unsigned)p.K, (unsigned)tiles);
    if (p.is_half) {
      trace::Scope t("filterGradGenericKernel<half>", stream, bytes, flops);
      filterGradGenericKernel<__half><<<grid, 256, 0, stream>>>(
          static_cast<const __half *>(features), static_cast<const __half *>(output_grad), indice_pairs, counts,
          p.L, p.ci, p.co, plan.seg_pairs, plan.max_segments, partial);
    } else {
      trace::Scope t("filterGradGenericKernel<float>", stream, bytes, flops);
      filterGradGenericKernel<float><<<grid, 256, 0, stream>>>(
          static_cast<const float *>(features), static_cast<const float *>(output_grad), indice_pairs, counts,
          p.L, p.ci, p.co, plan.seg_pairs, plan.max_segments, partial);
    }
    err = cudaGetLastError();
  }
  if (err != cudaSuccess) return err;

  const int64_t cico = (int64_t)p.ci * p.co;
  const int64_t total = (int64_t)p.K * cico;
  const unsigned blocks = (unsigned)((total + 255) / 256 < 2048 ? (total + 255) / 256 : 2048);
  trace::Scope t("reduceFilterGradKernel", stream,
                 4.0 * p.K * plan.max_segments * (double)cico + elem * (double)total);
  if (p.is_half) {
    reduceFilterGradKernel<__half><<<blocks, 256, 0, stream>>>(partial, counts, p.K, cico, plan.seg_pairs,
                                                               plan.max_segments,
                                                               static_cast<__half *>(filters_grad));
  } else {
    reduceFilterGradKernel<float><<<blocks, 256, 0, stream>>>(partial, counts, p.K, cico, plan.seg_pairs,
                                                              plan.max_segments,
                                                              static_cast<float *>(filters_grad));
  }
  return cudaGetLastError();
}

}  // namespace sparse_conv
}  // namespace mluop
