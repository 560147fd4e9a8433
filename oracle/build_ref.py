"""Build the reference's own CPU code for the sparse-conv path into oracle/_ref/.

TEST INFRASTRUCTURE ONLY.  The reference's CPU implementation of this path lives
in gtest Executor classes that cannot be built as they are (they include vendor
runtime headers and protobuf-generated code that are not available).  The
arithmetic itself is self-contained C++, so this recipe compiles exactly those
function bodies, read from the reference tree where they lie, behind a small
stand-in for the members they touch:

  GetIndicePairsExecutor::getValidOutPos      zoo/get_indice_pairs/get_indice_pairs.cpp
  GetIndicePairsExecutor::cpuGetIndicePairs   zoo/get_indice_pairs/get_indice_pairs.cpp
  IndiceConvolutionForwardExecutor::cpuCompute
                                              zoo/indice_convolution_forward/indice_convolution_forward.cpp
  cvtFloatToHalf                              pb_gtest/src/tools.cpp
  IndiceConvolutionBackwardDataExecutor::getFilterDims / cpuTransposeFilter / cpuCompute
                                              zoo/indice_convolution_backward_data/indice_convolution_backward_data.cpp
  IndiceConvolutionBackwardFilterExecutor::cpuTranspose / cpuCompute
                                              zoo/indice_convolution_backward_filter/indice_convolution_backward_filter.cpp

  dynamicVoxelize / pointToVoxelidx / determinVoxelNum / assignPointToVoxel / assignVoxelCoors and
  VoxelizationExecutor::deterministic_hard_voxelize
                                              zoo/voxelization/voxelization.cpp

  DynamicPointToVoxelForwardExecutor::cpuCompute
                                              zoo/dynamic_point_to_voxel_forward/dynamic_point_to_voxel_forward.cpp

  DynamicPointToVoxelBackwardExecutor::cpuCompute
                                              zoo/dynamic_point_to_voxel_backward/dynamic_point_to_voxel_backward.cpp

The backward-data body rounds to half through wrapRtConvertFloatToHalf /
wrapRtConvertHalfToFloat, which forward to the vendor runtime's cast routine
(tools.cpp:49-57); that runtime is not part of the reference tree, so the
stand-in forwards the first to the reference's own software conversion from the
same file and writes the second (an exact conversion) out.

The generated translation unit lives only in a temporary directory; the single
output is oracle/_ref/libmluops_ref_cpu.so (git-ignored).  No reference source
is written into the repository.

Usage: python oracle/build_ref.py [reference_root]
"""
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT_LIB = os.path.join(OUT_DIR, "libmluops_ref_cpu.so")

ZOO = "test/mlu_op_gtest/pb_gtest/src/zoo"
SOURCES = {
    "pairs": ZOO + "/get_indice_pairs/get_indice_pairs.cpp",
    "conv": ZOO + "/indice_convolution_forward/indice_convolution_forward.cpp",
    "tools": "test/mlu_op_gtest/pb_gtest/src/tools.cpp",
    "bwd_data": ZOO + "/indice_convolution_backward_data/indice_convolution_backward_data.cpp",
    "bwd_filter": ZOO + "/indice_convolution_backward_filter/indice_convolution_backward_filter.cpp",
    "voxel": ZOO + "/voxelization/voxelization.cpp",
    "dpv": ZOO + "/dynamic_point_to_voxel_forward/dynamic_point_to_voxel_forward.cpp",
    "dpv_bwd": ZOO + "/dynamic_point_to_voxel_backward/dynamic_point_to_voxel_backward.cpp",
}

PRELUDE = r"""
#include <algorithm>
#include <cmath>
#include <numeric>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <vector>
using std::sort;
using std::unique;

#include <string>
enum mluOpTensorLayout_t {
  MLUOP_LAYOUT_NCHW = 0, MLUOP_LAYOUT_NHWC = 1, MLUOP_LAYOUT_HWCN = 2,
  MLUOP_LAYOUT_NDHWC = 3, MLUOP_LAYOUT_ARRAY = 4, MLUOP_LAYOUT_NCDHW = 5
};
enum mluOpDataType_t { MLUOP_DTYPE_HALF = 1, MLUOP_DTYPE_FLOAT = 2, MLUOP_DTYPE_INT32 = 6 };

struct StandInTensor {
  std::vector<int64_t> dims;
  mluOpTensorLayout_t layout = MLUOP_LAYOUT_ARRAY;
  mluOpDataType_t dtype = MLUOP_DTYPE_FLOAT;
  int64_t getDimIndex(int i) const { return dims[i]; }
  int getDim() const { return (int)dims.size(); }
  mluOpTensorLayout_t getLayout() const { return layout; }
  mluOpDataType_t getDtype() const { return dtype; }
  int64_t getTotalElementNum() const {
    int64_t n = 1;
    for (auto d : dims) n *= d;
    return n;
  }
};
typedef StandInTensor *mluOpTensorDescriptor_t;

static inline int64_t mluOpGetTensordimD(const mluOpTensorDescriptor_t d) {
  return d->layout == MLUOP_LAYOUT_NDHWC ? d->dims[1] : d->dims[2];
}
static inline int64_t mluOpGetTensordimH(const mluOpTensorDescriptor_t d) {
  if (d->layout == MLUOP_LAYOUT_HWCN) return d->dims[0];
  return d->layout == MLUOP_LAYOUT_NDHWC ? d->dims[2] : d->dims[3];
}
static inline int64_t mluOpGetTensordimW(const mluOpTensorDescriptor_t d) {
  return d->layout == MLUOP_LAYOUT_NDHWC ? d->dims[3] : d->dims[4];
}
static inline int mluOpDataTypeBytes(mluOpDataType_t t) {
  return t == MLUOP_DTYPE_HALF ? 2 : 4;
}

struct StandInRuntime {
  void *allocate(size_t n) { return malloc(n ? n : 1); }
  void deallocate(void *p) { free(p); }
};
struct StandInBackwardDataParam {
  std::vector<int64_t> num;
  int64_t indice_num(int k) const { return num[k]; }
  int64_t inverse() const { return 0; }
  int64_t sub_m() const { return 0; }
};
struct StandInProtoNode {
  StandInBackwardDataParam bwd_data;
  const StandInBackwardDataParam &indice_convolution_backward_data_param() const { return bwd_data; }
};
struct StandInParser {
  int64_t out_count = 0;
  int in_num = 0, out_num = 0;
  StandInProtoNode node;
  int64_t getOutputDataCount(int) { return out_count; }
  int getInputNum() const { return in_num; }
  int getOutputNum() const { return out_num; }
  StandInProtoNode *getProtoNode() { return &node; }
};
struct StandInDescHolder { StandInTensor *tensor = nullptr; };
#define GTEST_CHECK(cond, ...) do { if (!(cond)) { std::cerr << "check failed: " #cond << std::endl; abort(); } } while (0)
struct StandInBlock { void *host_ptr = nullptr; void *device_ptr = nullptr; };

#define ERROR 0
#define LOG(x) std::cerr
#define VLOG(x) if (false) std::cerr

namespace mluoptest {
struct GetIndicePairsExecutor {
  StandInRuntime cpu_runtime_;
  int32_t getValidOutPos(int32_t *input_pos, std::vector<int32_t> kernel_size,
                         std::vector<int32_t> pad, std::vector<int32_t> stride,
                         std::vector<int32_t> dilation,
                         std::vector<int32_t> out_spatail_shape, int32_t *out,
                         int32_t NDim);
  void cpuGetIndicePairs(int32_t *indice_in, int32_t *indice_pairs,
                         int32_t *indice_out, int32_t *indice_num,
                         int32_t *grid_out,
                         const mluOpTensorDescriptor_t indice_in_desc,
                         std::vector<int32_t> kernel_size,
                         std::vector<int32_t> pad, std::vector<int32_t> stride,
                         std::vector<int32_t> dilation,
                         std::vector<int32_t> out_spatail_shape,
                         const int32_t dimNb, const int32_t sub_m,
                         const int32_t batch_size);
};
struct IndiceConvolutionForwardExecutor {
  StandInRuntime cpu_runtime_;
  StandInParser parser_storage_;
  StandInParser *parser_ = &parser_storage_;
  std::vector<float *> cpu_fp32_input_;
  std::vector<float *> cpu_fp32_output_;
  std::vector<StandInBlock> data_vector_;
  mluOpTensorDescriptor_t features_desc_ = nullptr;
  mluOpTensorDescriptor_t filters_desc_ = nullptr;
  mluOpTensorDescriptor_t indice_pairs_desc_ = nullptr;
  mluOpTensorDescriptor_t features_out_desc_ = nullptr;
  std::vector<int64_t> indice_num_;
  void cpuCompute();
};
int16_t cvtFloatToHalf(float x);
// half -> float is exact; written out here because the reference's routine picks
// its implementation through test-harness globals.
static inline float standInHalfToFloat(uint16_t h) {
  const uint32_t sign = (uint32_t)(h >> 15) << 31;
  const int32_t exp = (h >> 10) & 0x1f;
  uint32_t man = h & 0x3ff;
  uint32_t bits;
  if (exp == 0x1f) {
    bits = sign | 0x7f800000u | (man << 13);
  } else if (exp != 0) {
    bits = sign | ((uint32_t)(exp + 112) << 23) | (man << 13);
  } else if (man == 0) {
    bits = sign;
  } else {
    int32_t e = 113;
    while (!(man & 0x400)) { man <<= 1; --e; }
    bits = sign | ((uint32_t)e << 23) | ((man & 0x3ff) << 13);
  }
  float f;
  memcpy(&f, &bits, sizeof(f));
  return f;
}
static inline int wrapRtConvertFloatToHalf(uint16_t *f16, float d) {
  *f16 = (uint16_t)cvtFloatToHalf(d);
  return 0;
}
static inline int wrapRtConvertHalfToFloat(float *d, uint16_t f16) {
  *d = standInHalfToFloat(f16);
  return 0;
}
struct IndiceConvolutionBackwardDataExecutor {
  StandInRuntime cpu_runtime_;
  StandInParser parser_storage_;
  StandInParser *parser_ = &parser_storage_;
  std::vector<float *> cpu_fp32_input_;
  std::vector<float *> cpu_fp32_output_;
  std::vector<StandInDescHolder> tensor_desc_;
  int64_t inverse_ = 0, sub_m_ = 0;
  int dyc, dxc, kd, kh, kw;
  bool filter_4d;
  void getFilterDims();
  void setSpconvdataParams() {}
  void cpuTransposeFilter(float *filter_transpose_cpu, mluOpTensorLayout_t origin_layout);
  void cpuCompute();
};
enum ReduceMode { REDUCE_MODE_SUM = 0, REDUCE_MODE_MEAN = 1, REDUCE_MODE_MAX = 2 };
struct StandInDpvParam {
  ReduceMode mode = REDUCE_MODE_MAX;
  ReduceMode reduce_type() const { return mode; }
};
struct StandInDpvNode {
  StandInDpvParam param;
  const StandInDpvParam &dynamic_point_to_voxel_forward_param() const { return param; }
};
struct StandInDpvParser {
  StandInDpvNode node;
  int64_t in_count[2] = {0, 0};
  StandInDpvNode *getProtoNode() { return &node; }
  int64_t getInputDataCount(int i) { return in_count[i]; }
};
struct DynamicPointToVoxelForwardExecutor {
  StandInDpvParser parser_storage_;
  StandInDpvParser *parser_ = &parser_storage_;
  std::vector<float *> cpu_fp32_input_;
  std::vector<float *> cpu_fp32_output_;
  std::vector<StandInDescHolder> tensor_desc_;
  int64_t theory_ops_ = 0;
  void cpuCompute();
};
struct DynamicPointToVoxelBackwardExecutor {
  StandInDpvParser parser_storage_;
  StandInDpvParser *parser_ = &parser_storage_;
  std::vector<float *> cpu_fp32_input_;
  std::vector<float *> cpu_fp32_output_;
  std::vector<StandInDescHolder> tensor_desc_;
  void cpuCompute();
};
struct VoxelizationExecutor {
  StandInRuntime cpu_runtime_;
  void deterministic_hard_voxelize(const float *points, const float *voxel_size, const float *coors_range,
                                   const int32_t num_points, const int32_t num_features,
                                   const int32_t max_points, const int32_t max_voxels, const int32_t NDim,
                                   float *voxels, float *coors, float *num_points_per_voxel,
                                   float *voxel_num);
};
struct IndiceConvolutionBackwardFilterExecutor {
  StandInRuntime cpu_runtime_;
  std::vector<float *> cpu_fp32_input_;
  std::vector<float *> cpu_fp32_output_;
  std::vector<StandInBlock> data_vector_;
  mluOpTensorDescriptor_t input_indice_desc_ = nullptr;
  mluOpTensorDescriptor_t diffy_indice_desc_ = nullptr;
  mluOpTensorDescriptor_t indice_pair_desc_ = nullptr;
  mluOpTensorDescriptor_t diffw_desc_ = nullptr;
  std::vector<int64_t> indice_num_;
  bool diffw_trans_ = false;
  void cpuTranspose(float *output, const float *input, const int64_t kernel_volume, const int64_t ci,
                    const int64_t co, const mluOpTensorLayout_t diffw_layout);
  void cpuCompute();
};
"""

EPILOGUE = r"""
}  // namespace mluoptest

extern "C" {

// Buffer initialisation as GetIndicePairsExecutor::cpuCompute does it before
// the call (pairs -1, counts 0, out_indices -1, grid -1).
int mluops_ref_get_indice_pairs(const int32_t *indices, int32_t L, int32_t batch,
                                const int32_t *pad, const int32_t *stride,
                                const int32_t *dilation, const int32_t *filter_space,
                                const int32_t *out_space, int32_t sub_m,
                                int32_t *indice_pairs, int32_t *out_indices,
                                int64_t out_rows, int32_t *indice_num) {
  int64_t K = 1, grid_n = batch;
  for (int i = 0; i < 3; ++i) { K *= filter_space[i]; grid_n *= out_space[i]; }
  std::vector<int32_t> grid((size_t)grid_n, -1);
  std::fill(indice_pairs, indice_pairs + K * 2 * (int64_t)L, -1);
  std::fill(indice_num, indice_num + K, 0);
  std::fill(out_indices, out_indices + out_rows * 4, -1);
  StandInTensor in_desc;
  in_desc.dims = {L, 4};
  mluoptest::GetIndicePairsExecutor ex;
  auto v = [](const int32_t *p) { return std::vector<int32_t>(p, p + 3); };
  ex.cpuGetIndicePairs(const_cast<int32_t *>(indices), indice_pairs, out_indices,
                       indice_num, grid.data(), &in_desc, v(filter_space), v(pad),
                       v(stride), v(dilation), v(out_space), 5, sub_m, batch);
  return 0;
}

// filter_layout: 0 ARRAY [kd,kh,kw,Ci,Co], 1 NDHWC [Co,kd,kh,kw,Ci], 2 NCDHW [Co,Ci,kd,kh,kw]
int mluops_ref_indice_convolution_forward(const float *features, const float *filters,
                                          int32_t filter_layout, const int32_t *kdhw,
                                          const int32_t *indice_pairs,
                                          const int64_t *indice_num, int64_t L,
                                          int64_t ci, int64_t co, int64_t num_act_out,
                                          float *features_out) {
  const int64_t kd = kdhw[0], kh = kdhw[1], kw = kdhw[2], K = kd * kh * kw;
  StandInTensor f, w, p, o;
  f.dims = {L, ci};
  o.dims = {num_act_out, co};
  p.dims = {K, 2, L};
  if (filter_layout == 0) { w.layout = MLUOP_LAYOUT_ARRAY; w.dims = {kd, kh, kw, ci, co}; }
  else if (filter_layout == 1) { w.layout = MLUOP_LAYOUT_NDHWC; w.dims = {co, kd, kh, kw, ci}; }
  else { w.layout = MLUOP_LAYOUT_NCDHW; w.dims = {co, ci, kd, kh, kw}; }
  mluoptest::IndiceConvolutionForwardExecutor ex;
  ex.features_desc_ = &f; ex.filters_desc_ = &w; ex.indice_pairs_desc_ = &p;
  ex.features_out_desc_ = &o;
  ex.cpu_fp32_input_ = {const_cast<float *>(features), const_cast<float *>(filters)};
  ex.cpu_fp32_output_ = {features_out};
  ex.data_vector_.resize(4);
  ex.data_vector_[2].host_ptr = const_cast<int32_t *>(indice_pairs);
  ex.indice_num_.assign(indice_num, indice_num + K);
  ex.parser_storage_.out_count = num_act_out * co;
  ex.cpuCompute();
  return 0;
}

// The reference's CPU path holds coors, num_points_per_voxel and voxel_num as float
// copies of integers and expects zero-initialised outputs; converted here.
int mluops_ref_voxelization(const float *points, int64_t num_points, int64_t num_features,
                            const float *voxel_size, const float *coors_range, int32_t max_points,
                            int32_t max_voxels, float *voxels, int32_t *coors,
                            int32_t *num_points_per_voxel, int32_t *voxel_num) {
  std::vector<float> coors_f((size_t)max_voxels * 3, 0.0f), npv_f((size_t)max_voxels, 0.0f);
  float num_f = 0.0f;
  std::fill(voxels, voxels + (size_t)max_voxels * max_points * num_features, 0.0f);
  mluoptest::VoxelizationExecutor ex;
  ex.deterministic_hard_voxelize(points, voxel_size, coors_range, (int32_t)num_points,
                                 (int32_t)num_features, max_points, max_voxels, 3, voxels,
                                 coors_f.data(), npv_f.data(), &num_f);
  for (size_t i = 0; i < coors_f.size(); ++i) coors[i] = (int32_t)coors_f[i];
  for (size_t i = 0; i < npv_f.size(); ++i) num_points_per_voxel[i] = (int32_t)npv_f[i];
  *voxel_num = (int32_t)num_f;
  return 0;
}

// The reference's CPU path holds every tensor, the coordinates included, as float.
int mluops_ref_dynamic_point_to_voxel_forward(const float *feats, int32_t *coors, int64_t n, int64_t c_num,
                                              int64_t voxel_rows, int32_t reduce_max, float *voxel_feats,
                                              int32_t *voxel_coors, int32_t *point2voxel_map,
                                              int32_t *voxel_points_count, int32_t *voxel_num) {
  std::vector<float> coors_f((size_t)n * 3), vc_f((size_t)voxel_rows * 3, 0.0f), map_f((size_t)n, 0.0f),
      cnt_f((size_t)voxel_rows, 0.0f);
  float num_f = 0.0f;
  for (size_t i = 0; i < coors_f.size(); ++i) coors_f[i] = (float)coors[i];
  StandInTensor d_feats, d_coors, d_vf;
  d_feats.dims = {n, c_num};
  d_coors.dims = {n, 3};
  d_vf.dims = {voxel_rows, c_num};
  mluoptest::DynamicPointToVoxelForwardExecutor ex;
  ex.parser_storage_.node.param.mode = reduce_max ? mluoptest::REDUCE_MODE_MAX : mluoptest::REDUCE_MODE_MEAN;
  ex.parser_storage_.in_count[0] = n * c_num;
  ex.parser_storage_.in_count[1] = n * 3;
  ex.tensor_desc_.resize(3);
  ex.tensor_desc_[0].tensor = &d_feats;
  ex.tensor_desc_[1].tensor = &d_coors;
  ex.tensor_desc_[2].tensor = &d_vf;
  ex.cpu_fp32_input_ = {const_cast<float *>(feats), coors_f.data()};
  ex.cpu_fp32_output_ = {voxel_feats, vc_f.data(), map_f.data(), cnt_f.data(), &num_f};
  ex.cpuCompute();
  for (size_t i = 0; i < coors_f.size(); ++i) coors[i] = (int32_t)coors_f[i];
  for (size_t i = 0; i < vc_f.size(); ++i) voxel_coors[i] = (int32_t)vc_f[i];
  for (size_t i = 0; i < map_f.size(); ++i) point2voxel_map[i] = (int32_t)map_f[i];
  for (size_t i = 0; i < cnt_f.size(); ++i) voxel_points_count[i] = (int32_t)cnt_f[i];
  *voxel_num = (int32_t)num_f;
  return 0;
}

int mluops_ref_dynamic_point_to_voxel_backward(const float *grad_voxel_feats, const float *feats,
                                               const float *voxel_feats, const int32_t *point2voxel_map,
                                               int32_t voxel_num, int64_t n, int64_t c_num, float *grad_feats) {
  std::vector<float> map_f((size_t)n), cnt_f((size_t)(voxel_num > 0 ? voxel_num : 1), 0.0f);
  for (size_t i = 0; i < map_f.size(); ++i) map_f[i] = (float)point2voxel_map[i];
  float num_f = (float)voxel_num;
  std::fill(grad_feats, grad_feats + n * c_num, 0.0f);  // the harness hands the body a zeroed output
  StandInTensor d_feats;
  d_feats.dims = {n, c_num};
  mluoptest::DynamicPointToVoxelBackwardExecutor ex;
  ex.parser_storage_.in_count[0] = (int64_t)voxel_num * c_num;
  ex.parser_storage_.in_count[1] = n * c_num;
  ex.tensor_desc_.resize(2);
  ex.tensor_desc_[1].tensor = &d_feats;
  ex.cpu_fp32_input_ = {const_cast<float *>(grad_voxel_feats), const_cast<float *>(feats),
                        const_cast<float *>(voxel_feats), map_f.data(), cnt_f.data(), &num_f};
  ex.cpu_fp32_output_ = {grad_feats};
  ex.cpuCompute();
  return 0;
}

uint16_t mluops_ref_float_to_half_bits(float x) { return (uint16_t)mluoptest::cvtFloatToHalf(x); }

// filter_layout: 0 [K,Ci,Co] (passed as a 4-D HWCN filter {K,1,Ci,Co}: the reference's
// re-layout routine leaves its strides unset for a 5-D ARRAY filter), 1 NDHWC, 2 NCDHW.
int mluops_ref_indice_convolution_backward_data(const float *output_grad, const float *filters,
                                                int32_t filter_layout, const int32_t *kdhw,
                                                const int32_t *indice_pairs,
                                                const int64_t *indice_num, int64_t L, int64_t ci,
                                                int64_t co, int64_t n_out, int32_t is_half,
                                                float *input_grad) {
  const int64_t kd = kdhw[0], kh = kdhw[1], kw = kdhw[2], K = kd * kh * kw;
  StandInTensor og, w, p, ig;
  og.dims = {n_out, co};
  ig.dims = {L, ci};
  p.dims = {K, 2, L};
  p.dtype = MLUOP_DTYPE_INT32;
  w.dtype = is_half ? MLUOP_DTYPE_HALF : MLUOP_DTYPE_FLOAT;
  if (filter_layout == 0) { w.layout = MLUOP_LAYOUT_HWCN; w.dims = {K, 1, ci, co}; }
  else if (filter_layout == 1) { w.layout = MLUOP_LAYOUT_NDHWC; w.dims = {co, kd, kh, kw, ci}; }
  else { w.layout = MLUOP_LAYOUT_NCDHW; w.dims = {co, ci, kd, kh, kw}; }
  // the reference reads the pairs from the float copy of its inputs
  std::vector<float> pairs_f((size_t)(K * 2 * L));
  for (size_t i = 0; i < pairs_f.size(); ++i) pairs_f[i] = (float)indice_pairs[i];
  mluoptest::IndiceConvolutionBackwardDataExecutor ex;
  ex.tensor_desc_.resize(4);
  ex.tensor_desc_[0].tensor = &og; ex.tensor_desc_[1].tensor = &w;
  ex.tensor_desc_[2].tensor = &p; ex.tensor_desc_[3].tensor = &ig;
  ex.cpu_fp32_input_ = {const_cast<float *>(output_grad), const_cast<float *>(filters), pairs_f.data()};
  ex.cpu_fp32_output_ = {input_grad};
  ex.parser_storage_.in_num = 3; ex.parser_storage_.out_num = 1;
  ex.parser_storage_.out_count = L * ci;
  ex.parser_storage_.node.bwd_data.num.assign(indice_num, indice_num + K);
  ex.cpuCompute();
  return 0;
}

// filters_grad [K,Ci,Co].  The reference reads kw with the H accessor, so kh must equal kw.
int mluops_ref_indice_convolution_backward_filter(const float *features, const float *output_grad,
                                                  const int32_t *kdhw, const int32_t *indice_pairs,
                                                  const int64_t *indice_num, int64_t L, int64_t ci,
                                                  int64_t co, int64_t n_out, float *filters_grad) {
  const int64_t kd = kdhw[0], kh = kdhw[1], kw = kdhw[2], K = kd * kh * kw;
  if (kh != kw) return -1;
  StandInTensor f, og, p, w;
  f.dims = {L, ci};
  og.dims = {n_out, co};
  p.dims = {K, 2, L};
  w.layout = MLUOP_LAYOUT_NDHWC;  // only the D and H accessors are read: kd = dims[1], kh = kw = dims[2]
  w.dims = {co, kd, kh, kw, ci};
  mluoptest::IndiceConvolutionBackwardFilterExecutor ex;
  ex.input_indice_desc_ = &f; ex.diffy_indice_desc_ = &og; ex.indice_pair_desc_ = &p; ex.diffw_desc_ = &w;
  ex.cpu_fp32_input_ = {const_cast<float *>(features), const_cast<float *>(output_grad)};
  ex.cpu_fp32_output_ = {filters_grad};
  ex.data_vector_.resize(4);
  ex.data_vector_[2].host_ptr = const_cast<int32_t *>(indice_pairs);
  ex.indice_num_.assign(indice_num, indice_num + K);
  ex.cpuCompute();
  return 0;
}

}  // extern "C"
"""


def extract(path, signature_start):
    """Return the text of the function whose definition starts on a line that
    begins with `signature_start`, up to its closing brace in column 0."""
    with open(path) as f:
        lines = f.read().split("\n")
    for i, line in enumerate(lines):
        if line.startswith(signature_start):
            for j in range(i, len(lines)):
                if lines[j] == "}":
                    return '#line %d "%s"\n' % (i + 1, path) + "\n".join(lines[i:j + 1]) + "\n"
    raise RuntimeError("definition not found: %s in %s" % (signature_start, path))


def default_reference_root():
    """MLUOPS_REFERENCE_ROOT, else the directory `reference` beside this repository."""
    return os.environ.get("MLUOPS_REFERENCE_ROOT",
                          os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def build(reference_root=None, quiet=False):
    """Compile the library; returns its path, or None when the reference tree is absent."""
    if reference_root is None:
        reference_root = default_reference_root()
    paths = {k: os.path.join(reference_root, v) for k, v in SOURCES.items()}
    if not all(os.path.isfile(p) for p in paths.values()):
        return None
    os.makedirs(OUT_DIR, exist_ok=True)
    parts = [PRELUDE]
    parts.append(extract(paths["pairs"], "int32_t GetIndicePairsExecutor::getValidOutPos("))
    parts.append(extract(paths["pairs"], "void GetIndicePairsExecutor::cpuGetIndicePairs("))
    parts.append(extract(paths["conv"], "void IndiceConvolutionForwardExecutor::cpuCompute("))
    parts.append(extract(paths["tools"], "int16_t cvtFloatToHalf("))
    parts.append(extract(paths["bwd_data"], "void IndiceConvolutionBackwardDataExecutor::getFilterDims("))
    parts.append(extract(paths["bwd_data"], "void IndiceConvolutionBackwardDataExecutor::cpuTransposeFilter("))
    parts.append(extract(paths["bwd_data"], "void IndiceConvolutionBackwardDataExecutor::cpuCompute("))
    parts.append(extract(paths["bwd_filter"], "void IndiceConvolutionBackwardFilterExecutor::cpuTranspose("))
    parts.append(extract(paths["bwd_filter"], "void IndiceConvolutionBackwardFilterExecutor::cpuCompute("))
    for fn in ("void dynamicVoxelize(", "void pointToVoxelidx(", "void determinVoxelNum(",
               "void assignPointToVoxel(", "void assignVoxelCoors(",
               "void VoxelizationExecutor::deterministic_hard_voxelize("):
        parts.append(extract(paths["voxel"], fn))
    parts.append(extract(paths["dpv"], "void DynamicPointToVoxelForwardExecutor::cpuCompute("))
    parts.append(extract(paths["dpv_bwd"], "void DynamicPointToVoxelBackwardExecutor::cpuCompute("))
    parts.append(EPILOGUE)
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "ref_cpu_unit.cpp")
        with open(src, "w") as f:
            f.write("\n".join(parts))
        cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-w", "-o", OUT_LIB, src]
        if not quiet:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    return OUT_LIB


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else default_reference_root()
    lib = build(root)
    print(lib if lib else "reference tree not found at %s; nothing built" % root)
