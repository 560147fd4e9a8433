// Parameter block of one sparse convolution (reference
// kernels/sparse_conv/get_indice_pairs/get_indice_pairs_structs.h:85-98).
// Arrays are in (D, H, W) order.  num_act_out is an output field written by
// mluOpGetIndicePairs.
#ifndef MLUOP_B200_KERNELS_SPARSE_CONV_DESC_H_
#define MLUOP_B200_KERNELS_SPARSE_CONV_DESC_H_

#include "mlu_op.h"

struct mluOpSparseConvolutionStruct {
  int dimNb = 0;
  int batch = 0;
  int pad[3] = {0, 0, 0};
  int stride[3] = {1, 1, 1};
  int dilation[3] = {1, 1, 1};
  int input_space[3] = {0, 0, 0};
  int filter_space[3] = {0, 0, 0};
  int output_space[3] = {0, 0, 0};
  int sub_m = 0;
  int transpose = 0;
  int inverse = 0;
  int num_act_out = 0;
};

#endif  // MLUOP_B200_KERNELS_SPARSE_CONV_DESC_H_
