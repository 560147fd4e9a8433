/*
 * CPU oracle for the sparse-convolution forward path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's CPU
 * implementation (the code its gtest harness compares the device against):
 *
 *   rulebook generation   test/mlu_op_gtest/pb_gtest/src/zoo/get_indice_pairs/get_indice_pairs.cpp
 *                         :177-232 (buffer initialisation), :234-286 (candidate
 *                         outputs of one input voxel), :288-406 (pair lists,
 *                         sort/unique/decode/remap in default mode)
 *   convolution           test/mlu_op_gtest/pb_gtest/src/zoo/indice_convolution_forward/indice_convolution_forward.cpp
 *                         :117-141 (filter re-layout), :143-146 (zero init),
 *                         :148-171 (accumulation order)
 *   float <-> half        test/mlu_op_gtest/pb_gtest/src/tools.cpp:460-505
 *   diff1 / diff2 / diff3 test/mlu_op_gtest/pb_gtest/include/evaluator.h:431-519
 *
 * Parity status: pinned.  The restatement is checked bit for bit against the
 * reference's own function bodies compiled from the reference tree (the
 * optional library built by oracle/build_ref.py) and against committed golden
 * vectors generated from that library (tests/golden/).
 *
 * Nothing in the shipped library links or calls this file; only tests, the
 * smoke check and the CPU-baseline leg of the benchmark do.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_NDIM 3

/* ------------------------------------------------------------------ */
/* Candidate outputs of one input voxel                                */
/* (get_indice_pairs.cpp:234-286).  For every spatial dim the set of   */
/* output coordinates o with  i + pad - o*stride = kk*dilation,        */
/* 0 <= kk < ksize, is the arithmetic progression uppers, uppers-dil,  */
/* ..., >= lowers.  Points are enumerated with the last dim fastest,   */
/* starting from the upper corner; the kernel offset of a point is     */
/* sum_d m_d * (i_d - o_d*stride_d + pad_d) / dil_d  with m_d the      */
/* row-major weight of dim d inside the kernel (w fastest).            */
/* A point outside [0, out_space) is dropped.                          */
/* out: rows of (o_0, o_1, o_2, offset).  Returns the kept count.      */
/* ------------------------------------------------------------------ */
static int32_t candidate_outputs(const int32_t *pos, const int32_t *ksize,
                                 const int32_t *pad, const int32_t *stride,
                                 const int32_t *dil, const int32_t *out_space,
                                 int32_t *out) {
  int32_t lo[ORACLE_NDIM], hi[ORACLE_NDIM], cnt[ORACLE_NDIM], ctr[ORACLE_NDIM];
  int32_t total = 1;
  for (int d = 0; d < ORACLE_NDIM; ++d) {
    /* C integer division (truncation toward zero), as in the reference. */
    lo[d] = (pos[d] - (ksize[d] - 1) * dil[d] - 1 + stride[d] + pad[d]) / stride[d];
    hi[d] = (pos[d] + pad[d]) / stride[d];
    cnt[d] = (hi[d] - lo[d]) / dil[d] + 1;
    total *= cnt[d];
    ctr[d] = 0;
  }
  int32_t kept = 0;
  for (int32_t p = 0; p < total; ++p) {
    int ok = 1;
    int32_t weight = 1, offset = 0;
    int32_t *row = out + (size_t)kept * (ORACLE_NDIM + 1);
    for (int d = ORACLE_NDIM - 1; d >= 0; --d) {
      int32_t o = hi[d] - ctr[d] * dil[d];
      row[d] = o;
      if (o < 0 || o > out_space[d] - 1) ok = 0;
      offset += weight * (pos[d] - o * stride[d] + pad[d]) / dil[d];
      weight *= ksize[d];
    }
    row[ORACLE_NDIM] = offset;
    if (ok) ++kept;
    ctr[ORACLE_NDIM - 1] += 1;
    for (int d = ORACLE_NDIM - 1; d > 0; --d) {
      if (ctr[d] == cnt[d]) {
        ctr[d - 1] += 1;
        ctr[d] = 0;
      }
    }
  }
  return kept;
}

static int32_t linear_index(const int32_t *coord, const int32_t *space) {
  int32_t idx = 0, w = 1;
  for (int d = ORACLE_NDIM - 1; d >= 0; --d) {
    idx += coord[d] * w;
    w *= space[d];
  }
  return idx;
}

static int cmp_i32(const void *a, const void *b) {
  int32_t x = *(const int32_t *)a, y = *(const int32_t *)b;
  return (x > y) - (x < y);
}

/*
 * Rulebook generation (get_indice_pairs.cpp:177-232 + :288-406).
 *
 *   indices       [L,4] int32 rows (b, z, y, x)
 *   indice_pairs  [K,2,L] int32, fully written (-1 beyond each list)
 *   out_indices   [out_rows,4] int32, fully written (-1 beyond num_act_out)
 *   indice_num    [K] int32
 *   num_act_out   number of active outputs (default mode); L in subm mode
 *   sentinel_quirk  non-zero reproduces the reference line
 *                   `num_act_out = unique.size() - 1` (:380), which assumes at
 *                   least one (k,j) slot is unused; zero uses the true count.
 *                   Both agree whenever an unused slot exists.
 * Returns 0, or -1 when memory cannot be had.
 */
int mluops_oracle_get_indice_pairs(
    const int32_t *indices, int32_t L, int32_t batch, const int32_t *pad,
    const int32_t *stride, const int32_t *dilation, const int32_t *filter_space,
    const int32_t *out_space, int32_t sub_m, int32_t *indice_pairs,
    int32_t *out_indices, int64_t out_rows, int32_t *indice_num,
    int32_t *num_act_out, int32_t sentinel_quirk) {
  const int32_t W = ORACLE_NDIM + 1;
  int32_t vol = 1, K = 1;
  for (int d = 0; d < ORACLE_NDIM; ++d) {
    vol *= out_space[d];
    K *= filter_space[d];
  }
  const int64_t grid_n = (int64_t)batch * vol;
  const int64_t slots = (int64_t)K * L;
  int32_t *grid = (int32_t *)malloc(sizeof(int32_t) * (size_t)(grid_n > 0 ? grid_n : 1));
  int32_t *cand = (int32_t *)malloc(sizeof(int32_t) * (size_t)K * W);
  int32_t *uniq = (int32_t *)malloc(sizeof(int32_t) * (size_t)(slots > 0 ? slots : 1));
  if (!grid || !cand || !uniq) {
    free(grid); free(cand); free(uniq);
    return -1;
  }
  for (int64_t i = 0; i < grid_n; ++i) grid[i] = -1;
  for (int64_t i = 0; i < 2 * slots; ++i) indice_pairs[i] = -1;
  for (int32_t k = 0; k < K; ++k) indice_num[k] = 0;
  for (int64_t i = 0; i < out_rows * W; ++i) out_indices[i] = -1;
  const int32_t sentinel = batch * vol + 1;
  for (int64_t i = 0; i < slots; ++i) uniq[i] = sentinel;

  if (sub_m) {
    /* Occupancy grid of the inputs; a repeated coordinate keeps the last row. */
    for (int32_t j = 0; j < L; ++j) {
      const int32_t *row = indices + (size_t)j * W;
      grid[linear_index(row + 1, out_space) + vol * row[0]] = j;
    }
    for (int64_t i = 0; i < (int64_t)L * W; ++i) out_indices[i] = indices[i];
  }

  for (int32_t j = 0; j < L; ++j) {
    const int32_t *row = indices + (size_t)j * W;
    const int32_t b = row[0];
    int32_t n = candidate_outputs(row + 1, filter_space, pad, stride, dilation,
                                  out_space, cand);
    for (int32_t c = 0; c < n; ++c) {
      const int32_t *pt = cand + (size_t)c * W;
      const int32_t k = pt[ORACLE_NDIM];
      const int32_t lin = linear_index(pt, out_space) + vol * b;
      int32_t *in_row = indice_pairs + (size_t)k * 2 * L;
      int32_t *out_row = in_row + L;
      if (sub_m) {
        if (grid[lin] > -1) {
          int32_t p = indice_num[k]++;
          in_row[p] = j;
          out_row[p] = grid[lin];
        }
      } else {
        int32_t p = indice_num[k]++;
        in_row[p] = j;
        out_row[p] = lin;
        uniq[(size_t)k * L + p] = lin;
      }
    }
  }

  if (!sub_m) {
    qsort(uniq, (size_t)slots, sizeof(int32_t), cmp_i32);
    int64_t n_unique = 0;
    for (int64_t i = 0; i < slots; ++i) {
      if (i == 0 || uniq[i] != uniq[i - 1]) uniq[n_unique++] = uniq[i];
    }
    int64_t n_out;
    if (sentinel_quirk) {
      n_out = n_unique - 1;
    } else {
      n_out = n_unique;
      if (n_unique > 0 && uniq[n_unique - 1] == sentinel) n_out -= 1;
    }
    if (n_out < 0) n_out = 0;
    const int32_t hw = out_space[2] * out_space[1];
    for (int64_t r = 0; r < n_out; ++r) {
      int32_t lin = uniq[r];
      grid[lin] = (int32_t)r;
      int32_t *o = out_indices + (size_t)r * W;
      o[0] = lin / vol;
      lin -= o[0] * vol;
      o[1] = lin / hw;
      lin -= o[1] * hw;
      o[2] = lin / out_space[2];
      lin -= o[2] * out_space[2];
      o[3] = lin;
    }
    for (int32_t j = 0; j < L; ++j) {
      for (int32_t k = 0; k < K; ++k) {
        int32_t *slot = indice_pairs + (size_t)k * 2 * L + L + j;
        if (*slot > -1) *slot = grid[*slot];
      }
    }
    *num_act_out = (int32_t)n_out;
  } else {
    *num_act_out = L;
  }
  free(grid); free(cand); free(uniq);
  return 0;
}

/*
 * Convolution (indice_convolution_forward.cpp:117-171).
 *   features   [L,Ci] float   (already rounded to half and widened when the
 *                              device dtype is half)
 *   filters    5-D float; filter_layout: 0 = [kd,kh,kw,Ci,Co] (ARRAY),
 *              1 = [Co,kd,kh,kw,Ci] (NDHWC), 2 = [Co,Ci,kd,kh,kw] (NCDHW)
 *   indice_pairs [K,2,L] int32, indice_num [K] int64 (host array in the API)
 *   features_out [num_act_out,Co] float, zeroed then accumulated in the
 *              reference order: kernel offset ascending, pair in list order,
 *              ci ascending, one float add per product.
 */
int mluops_oracle_indice_convolution_forward(
    const float *features, const float *filters, int32_t filter_layout,
    const int32_t *indice_pairs, const int64_t *indice_num, int64_t L,
    int64_t ci, int64_t co, int64_t K, int64_t num_act_out,
    float *features_out) {
  const float *w = filters;
  float *packed = NULL;
  if (filter_layout != 0) {
    int64_t s_k, s_ci, s_co;
    if (filter_layout == 2) {
      s_k = 1; s_ci = K; s_co = K * ci;
    } else {
      s_k = ci; s_ci = 1; s_co = ci * K;
    }
    packed = (float *)malloc(sizeof(float) * (size_t)(K * ci * co));
    if (!packed) return -1;
    for (int64_t k = 0; k < K; ++k)
      for (int64_t c = 0; c < ci; ++c)
        for (int64_t o = 0; o < co; ++o)
          packed[k * co * ci + c * co + o] = filters[k * s_k + c * s_ci + o * s_co];
    w = packed;
  }
  memset(features_out, 0, sizeof(float) * (size_t)(num_act_out * co));
  for (int64_t k = 0; k < K; ++k) {
    const int32_t *in_row = indice_pairs + k * 2 * L;
    const int32_t *out_row = in_row + L;
    for (int64_t p = 0; p < indice_num[k]; ++p) {
      const int64_t src = in_row[p], dst = out_row[p];
      if (dst < 0 || src < 0) continue;
      const float *f = features + src * ci;
      float *o = features_out + dst * co;
      for (int64_t c = 0; c < ci; ++c) {
        const float a = f[c];
        const float *wr = w + k * ci * co + c * co;
        for (int64_t n = 0; n < co; ++n) {
          /* product rounded to float, then one float add, as in the reference;
             the volatile keeps the compiler from contracting into an fma. */
          volatile float prod = a * wr[n];
          o[n] += prod;
        }
      }
    }
  }
  free(packed);
  return 0;
}

/* Same arithmetic without the anti-contraction barrier: used only as the
 * timed CPU baseline, where the compiler may vectorise the inner loop. */
int mluops_oracle_indice_convolution_forward_fast(
    const float *features, const float *filters_kcico,
    const int32_t *indice_pairs, const int64_t *indice_num, int64_t L,
    int64_t ci, int64_t co, int64_t K, int64_t num_act_out,
    float *features_out) {
  memset(features_out, 0, sizeof(float) * (size_t)(num_act_out * co));
  for (int64_t k = 0; k < K; ++k) {
    const int32_t *in_row = indice_pairs + k * 2 * L;
    const int32_t *out_row = in_row + L;
    for (int64_t p = 0; p < indice_num[k]; ++p) {
      const int64_t src = in_row[p], dst = out_row[p];
      if (dst < 0 || src < 0) continue;
      const float *f = features + src * ci;
      float *o = features_out + dst * co;
      for (int64_t c = 0; c < ci; ++c) {
        const float a = f[c];
        const float *wr = filters_kcico + k * ci * co + c * co;
        for (int64_t n = 0; n < co; ++n) o[n] += a * wr[n];
      }
    }
  }
  return 0;
}

/* The same loop nest with the pairs of one offset shared among OpenMP threads: a
 * rulebook holds at most one pair per (offset, output row), so the pairs of one
 * offset write disjoint rows and need no synchronisation; the offsets stay in
 * order.  Timed all-cores baseline only (compiled with -fopenmp into a library of
 * its own; without OpenMP the pragma is ignored). */
int mluops_oracle_indice_convolution_forward_threads(
    const float *features, const float *filters_kcico,
    const int32_t *indice_pairs, const int64_t *indice_num, int64_t L,
    int64_t ci, int64_t co, int64_t K, int64_t num_act_out,
    float *features_out) {
  memset(features_out, 0, sizeof(float) * (size_t)(num_act_out * co));
  for (int64_t k = 0; k < K; ++k) {
    const int32_t *in_row = indice_pairs + k * 2 * L;
    const int32_t *out_row = in_row + L;
    const int64_t pairs = indice_num[k];
    const float *wk = filters_kcico + k * ci * co;
#pragma omp parallel for schedule(static)
    for (int64_t p = 0; p < pairs; ++p) {
      const int64_t src = in_row[p], dst = out_row[p];
      if (dst < 0 || src < 0) continue;
      const float *f = features + src * ci;
      float *o = features_out + dst * co;
      for (int64_t c = 0; c < ci; ++c) {
        const float a = f[c];
        const float *wr = wk + c * co;
        for (int64_t n = 0; n < co; ++n) o[n] += a * wr[n];
      }
    }
  }
  return 0;
}

/* ------------------------------------------------------------------ */
/* float -> half bits (tools.cpp:460-505): round to nearest even in    */
/* the normal range, saturate finite overflow to 0x7bff, round-half-up */
/* on the discarded bit in the subnormal range.                        */
/* ------------------------------------------------------------------ */
uint16_t mluops_oracle_float_to_half_bits(float x) {
  int32_t in;
  memcpy(&in, &x, sizeof(in));
  int32_t sign = in >> 31; /* only bit 0 is used below */
  int32_t exp = ((in >> 23) & 0xff) - 127;
  int32_t frac = in & 0x7fffff;
  int32_t mant, round = 0, subnormal = 0;
  if (exp == 128 && frac) {
    exp = 0x1f - 15; mant = 0x200;
  } else if (exp == 128) {
    exp = 0x1f - 15; mant = 0;
  } else if (exp >= 16) {
    exp = 0xf; mant = 0x3ff;
  } else if (exp >= -14) {
    int32_t sticky = in & 0xfff, half_bit = (in >> 12) & 1, lsb = (in >> 13) & 1;
    round = (half_bit && sticky) || (half_bit && lsb);
    mant = (in >> 13) & 0x3ff;
  } else if (exp >= -24) {
    int32_t full = frac | 0x800000;
    round = (full >> (-exp - 2)) & 1;
    mant = (full >> (-exp - 1)) & 0x3ff;
    subnormal = 1; exp = 0;
  } else {
    subnormal = 1; exp = 0;
    mant = (in & 0x7fffffff) ? 1 : 0;
  }
  mant += round;
  if (!subnormal) exp += 15;
  int32_t r = ((sign & 1) << 15) + (exp << 10) + mant;
  return (uint16_t)r;
}

float mluops_oracle_half_bits_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h >> 15) << 31;
  int32_t exp = (h >> 10) & 0x1f;
  uint32_t mant = h & 0x3ff;
  uint32_t bits;
  if (exp == 0) {
    if (mant == 0) {
      bits = sign;
    } else {
      int shift = 0;
      while (!(mant & 0x400)) { mant <<= 1; ++shift; }
      mant &= 0x3ff;
      bits = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (mant << 13);
    }
  } else if (exp == 0x1f) {
    bits = sign | 0x7f800000u | (mant << 13);
  } else {
    bits = sign | ((uint32_t)(exp - 15 + 127) << 23) | (mant << 13);
  }
  float f;
  memcpy(&f, &bits, sizeof(f));
  return f;
}

/* dst[i] = widen(round_to_half(src[i])): the harness's conditioning of fp16
 * inputs and of the CPU result when the output dtype is half
 * (pb_gtest/src/executor.cpp:1863-1868, :2247-2275). */
void mluops_oracle_round_through_half(const float *src, float *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i)
    dst[i] = mluops_oracle_half_bits_to_float(mluops_oracle_float_to_half_bits(src[i]));
}

void mluops_oracle_float_to_half_array(const float *src, uint16_t *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = mluops_oracle_float_to_half_bits(src[i]);
}

void mluops_oracle_half_to_float_array(const uint16_t *src, float *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = mluops_oracle_half_bits_to_float(src[i]);
}

/* diff1, diff2, diff3 (evaluator.h:431-519); `test` is the device result,
 * `base` the CPU result.  is_half selects the diff3 small-value threshold. */
void mluops_oracle_diffs(const float *test, const float *base, int64_t n,
                         int32_t is_half, double *diff1, double *diff2,
                         double *diff3) {
  const double eps = 1e-9;
  const double small = is_half ? 1e-4 : 1e-6;
  double n1 = 0, d1 = 0, n2 = 0, d2 = 0, m3 = 0;
  for (int64_t i = 0; i < n; ++i) {
    double a = (double)test[i], b = (double)base[i];
    double e = fabs(a - b), mag = fabs(b);
    n1 += e; d1 += mag;
    n2 += e * e; d2 += b * b;
    double r = (mag < small) ? e : e / (mag + eps);
    if (r > m3) m3 = r;
  }
  *diff1 = n1 / (d1 + eps);
  *diff2 = sqrt(n2 / (d2 + eps));
  *diff3 = m3;
}
