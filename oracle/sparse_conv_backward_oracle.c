/*
 * CPU oracle for the two backward operators of the sparse convolution.
 * TEST INFRASTRUCTURE ONLY.
 *
 * Restates, in plain C, the arithmetic of the reference's CPU implementations:
 *
 *   input gradient   test/mlu_op_gtest/pb_gtest/src/zoo/indice_convolution_backward_data/
 *                    indice_convolution_backward_data.cpp:176-250 (filter re-layout to
 *                    [K,Ci,Co]), :252-339 (zero init and accumulation; for a half
 *                    device dtype every product and every running sum of one pair is
 *                    rounded through half, the sum over pairs stays in float)
 *   filter gradient  test/mlu_op_gtest/pb_gtest/src/zoo/indice_convolution_backward_filter/
 *                    indice_convolution_backward_filter.cpp:122-182 (per kernel offset,
 *                    per (ci, co): one float accumulator over the pair list, in list
 *                    order; output layout [K,Ci,Co])
 *
 * The reference rounds to half through its vendor runtime's cast routine
 * (tools.cpp:49-57, cnrtCastDataType_V2), which is not part of the reference
 * tree.  This file uses the reference's own software conversion
 * (tools.cpp:460-505, restated in sparse_conv_oracle.c) in its place; the two
 * can differ only where a value lies exactly half way between two halves.
 *
 * Parity status: pinned.  Checked against the reference's own function bodies
 * compiled from the reference tree (oracle/build_ref.py) bit for bit, and
 * against golden vectors generated from that build (tests/golden/).
 *
 * Nothing in the shipped library links or calls this file.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

uint16_t mluops_oracle_float_to_half_bits(float x);
float mluops_oracle_half_bits_to_float(uint16_t h);

static float through_half(float x) {
  return mluops_oracle_half_bits_to_float(mluops_oracle_float_to_half_bits(x));
}

/* filters in layout code 0 = [K,Ci,Co] (ARRAY / HWCN), 1 = [Co,K,Ci] (NDHWC / NHWC),
 * 2 = [Co,Ci,K] (NCDHW / NCHW) -> malloc'ed [K,Ci,Co], or NULL when already so. */
static float *to_k_ci_co(const float *filters, int32_t layout, int64_t K, int64_t ci, int64_t co) {
  if (layout == 0) return NULL;
  int64_t s_k, s_ci, s_co;
  if (layout == 2) {
    s_k = 1; s_ci = K; s_co = K * ci;
  } else {
    s_k = ci; s_ci = 1; s_co = ci * K;
  }
  float *packed = (float *)malloc(sizeof(float) * (size_t)(K * ci * co));
  if (!packed) return NULL;
  for (int64_t k = 0; k < K; ++k)
    for (int64_t c = 0; c < ci; ++c)
      for (int64_t o = 0; o < co; ++o)
        packed[(k * ci + c) * co + o] = filters[k * s_k + c * s_ci + o * s_co];
  return packed;
}

/*
 * input_grad[i,:] = sum_k sum_{(i,o) in pairs_k} output_grad[o,:] * W_k^T
 *   output_grad [n_out,Co] float, filters as above, indice_pairs [K,2,L] int32,
 *   input_grad [L,Ci] float.  is_half: emulate half arithmetic inside one pair
 *   as the reference does.
 */
int mluops_oracle_indice_convolution_backward_data(
    const float *output_grad, const float *filters, int32_t filter_layout,
    const int32_t *indice_pairs, const int64_t *indice_num, int64_t L, int64_t ci,
    int64_t co, int64_t K, int32_t is_half, float *input_grad) {
  float *packed = to_k_ci_co(filters, filter_layout, K, ci, co);
  if (filter_layout != 0 && !packed) return -1;
  const float *w = packed ? packed : filters;
  memset(input_grad, 0, sizeof(float) * (size_t)(L * ci));
  for (int64_t k = 0; k < K; ++k) {
    const int32_t *in_row = indice_pairs + k * 2 * L;
    const int32_t *out_row = in_row + L;
    const float *wk = w + k * ci * co;
    for (int64_t p = 0; p < indice_num[k]; ++p) {
      float *dx = input_grad + (int64_t)in_row[p] * ci;
      const float *dy = output_grad + (int64_t)out_row[p] * co;
      for (int64_t c = 0; c < ci; ++c) {
        float acc = 0.0f;
        for (int64_t n = 0; n < co; ++n) {
          if (is_half) {
            const float a = through_half(dy[n]);
            const float b = through_half(wk[c * co + n]);
            volatile float prod = a * b;
            const float pr = through_half(prod);
            volatile float sum = acc + pr;
            acc = through_half(sum);
          } else {
            volatile float prod = dy[n] * wk[c * co + n];
            acc += prod;
          }
        }
        dx[c] += acc;
      }
    }
  }
  free(packed);
  return 0;
}

/*
 * filters_grad[k,c,n] = sum_{(i,o) in pairs_k} features[i,c] * output_grad[o,n]
 *   one float accumulator per element, pairs in list order; offsets with no
 *   pairs give zeros.  filters_grad [K,Ci,Co] float.
 */
int mluops_oracle_indice_convolution_backward_filter(
    const float *features, const float *output_grad, const int32_t *indice_pairs,
    const int64_t *indice_num, int64_t L, int64_t ci, int64_t co, int64_t K,
    float *filters_grad) {
  for (int64_t k = 0; k < K; ++k) {
    const int32_t *in_row = indice_pairs + k * 2 * L;
    const int32_t *out_row = in_row + L;
    for (int64_t c = 0; c < ci; ++c) {
      for (int64_t n = 0; n < co; ++n) {
        float acc = 0.0f;
        for (int64_t p = 0; p < indice_num[k]; ++p) {
          volatile float prod = features[(int64_t)in_row[p] * ci + c] * output_grad[(int64_t)out_row[p] * co + n];
          acc += prod;
        }
        filters_grad[(k * ci + c) * co + n] = acc;
      }
    }
  }
  return 0;
}
