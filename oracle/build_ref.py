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
}

PRELUDE = r"""
#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <vector>
using std::sort;
using std::unique;

enum mluOpTensorLayout_t { MLUOP_LAYOUT_NDHWC = 3, MLUOP_LAYOUT_ARRAY = 4, MLUOP_LAYOUT_NCDHW = 5 };
enum mluOpDataType_t { MLUOP_DTYPE_HALF = 1, MLUOP_DTYPE_FLOAT = 2, MLUOP_DTYPE_INT32 = 6 };

struct StandInTensor {
  std::vector<int64_t> dims;
  mluOpTensorLayout_t layout = MLUOP_LAYOUT_ARRAY;
  mluOpDataType_t dtype = MLUOP_DTYPE_FLOAT;
  int64_t getDimIndex(int i) const { return dims[i]; }
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
struct StandInParser {
  int64_t out_count = 0;
  int64_t getOutputDataCount(int) { return out_count; }
};
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

uint16_t mluops_ref_float_to_half_bits(float x) { return (uint16_t)mluoptest::cvtFloatToHalf(x); }

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


def build(reference_root="/root/reference", quiet=False):
    """Compile the library; returns its path, or None when the reference tree is absent."""
    paths = {k: os.path.join(reference_root, v) for k, v in SOURCES.items()}
    if not all(os.path.isfile(p) for p in paths.values()):
        return None
    os.makedirs(OUT_DIR, exist_ok=True)
    parts = [PRELUDE]
    parts.append(extract(paths["pairs"], "int32_t GetIndicePairsExecutor::getValidOutPos("))
    parts.append(extract(paths["pairs"], "void GetIndicePairsExecutor::cpuGetIndicePairs("))
    parts.append(extract(paths["conv"], "void IndiceConvolutionForwardExecutor::cpuCompute("))
    parts.append(extract(paths["tools"], "int16_t cvtFloatToHalf("))
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
    root = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    lib = build(root)
    print(lib if lib else "reference tree not found at %s; nothing built" % root)
