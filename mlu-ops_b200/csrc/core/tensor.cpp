// Tensor-descriptor API (reference core/tensor.cpp:205-241 pool, :301-339 dims
// and contiguous strides, :560-857 entry points).
#include "core/tensor.h"

#include <algorithm>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

void mluOpTensorStruct::releaseHeapDims() {
  if (dims != inline_dims_) {
    delete[] dims;
    delete[] strides;
  }
  dims = inline_dims_;
  strides = inline_strides_;
}

void mluOpTensorStruct::resizeDims(int dimNb) {
  if (dimNb == dim) return;
  releaseHeapDims();
  if (dimNb > MLUOP_DIM_MAX) {
    dims = new int64_t[dimNb];
    strides = new int64_t[dimNb];
  }
  dim = dimNb;
}

void mluOpTensorStruct::reset() {
  dims = inline_dims_;
  strides = inline_strides_;
  dim = 0;
  dtype = MLUOP_DTYPE_FLOAT;
  layout = MLUOP_LAYOUT_ARRAY;
  total_element_num = 0;
  total_tensor_size = 0;
}

template <typename Int>
mluOpStatus_t mluOpTensorStruct::set(mluOpTensorLayout_t layout_, mluOpDataType_t dtype_, int dimNb,
                                     const Int *dimSize) {
  PARAM_CHECK("[mluOpSetTensorDescriptor]", layout_ >= 0);
  PARAM_CHECK("[mluOpSetTensorDescriptor]", dtype_ >= 0);
  dtype = dtype_;
  layout = layout_;
  if (dimNb == 0) {
    // A rank-0 descriptor only describes host scalars in the reference
    // (core/tensor.cpp:43-57); device tensors of this path never have rank 0.
    LOG(ERROR) << "[mluOpSetTensorDescriptor]: dimNb 0 is only valid for host-pointer "
                  "descriptors, which this build does not provide.";
    return MLUOP_STATUS_BAD_PARAM;
  }
  PARAM_CHECK("[mluOpSetTensorDescriptor]", dimNb > 0);
  PARAM_CHECK("[mluOpSetTensorDescriptor]", dimSize != NULL);
  resizeDims(dimNb);
  uint64_t running = 1;
  bool overflow = false;
  for (int i = dimNb - 1; i >= 0; --i) {
    dims[i] = (int64_t)dimSize[i];
    strides[i] = (int64_t)running;
    running *= (uint64_t)dimSize[i];
    overflow |= running >= LARGE_TENSOR_NUM;
  }
  total_element_num = running;
  total_tensor_size = running * mluop::getSizeOfDataType(dtype);
  if (overflow) {
    LOG(WARNING) << "[mluOpSetTensorDescriptor]: tensor has " << running
                 << " elements; operators accept fewer than 2^31.";
  }
  return MLUOP_STATUS_SUCCESS;
}

template <typename Int>
mluOpStatus_t mluOpTensorStruct::setEx(mluOpTensorLayout_t layout_, mluOpDataType_t dtype_, int dimNb,
                                       const Int *dimSize, const Int *dimStride) {
  PARAM_CHECK("[mluOpSetTensorDescriptorEx]", layout_ >= 0);
  PARAM_CHECK("[mluOpSetTensorDescriptorEx]", dtype_ >= 0);
  dtype = dtype_;
  layout = layout_;
  PARAM_CHECK("[mluOpSetTensorDescriptorEx]", dimSize != NULL);
  PARAM_CHECK("[mluOpSetTensorDescriptorEx]", dimStride != NULL);
  PARAM_CHECK("[mluOpSetTensorDescriptorEx]", dimNb > 0);
  resizeDims(dimNb);
  total_element_num = 1;
  for (int i = 0; i < dimNb; ++i) {
    dims[i] = (int64_t)dimSize[i];
    strides[i] = (int64_t)dimStride[i];
    total_element_num *= (uint64_t)dimSize[i];
  }
  total_tensor_size = total_element_num * mluop::getSizeOfDataType(dtype);
  return MLUOP_STATUS_SUCCESS;
}

namespace {

// Free list of descriptor storage: creating and destroying descriptors is on
// the per-call path of framework plugins, so storage is recycled instead of
// going through the allocator each time.  Guarded by a mutex; blocks are
// carved in growing chunks and live until process exit.
class DescriptorPool {
 public:
  mluOpTensorStruct *take() {
    std::lock_guard<std::mutex> guard(lock_);
    if (free_.empty()) grow();
    void *slot = free_.back();
    free_.pop_back();
    return ::new (slot) mluOpTensorStruct;
  }
  void give(mluOpTensorStruct *desc) {
    desc->~mluOpTensorStruct();
    std::lock_guard<std::mutex> guard(lock_);
    free_.push_back(desc);
  }

 private:
  void grow() {
    auto *block = static_cast<unsigned char *>(::operator new(chunk_ * sizeof(mluOpTensorStruct)));
    for (size_t i = 0; i < chunk_; ++i) free_.push_back(block + i * sizeof(mluOpTensorStruct));
    chunk_ *= 2;
  }
  std::mutex lock_;
  std::vector<void *> free_;
  size_t chunk_ = 64;
};

DescriptorPool &pool() {
  static DescriptorPool *p = new DescriptorPool;  // never destroyed: descriptors may outlive statics
  return *p;
}

template <typename Int>
mluOpStatus_t readBack(const mluOpTensorDescriptor_t desc, mluOpTensorLayout_t *layout,
                       mluOpDataType_t *dtype, int *dimNb, Int *dimSize, Int *dimStride) {
  if (layout) *layout = desc->layout;
  if (dtype) *dtype = desc->dtype;
  if (dimNb) *dimNb = desc->dim;
  for (int i = 0; i < desc->dim; ++i) {
    if (dimSize) dimSize[i] = (Int)desc->dims[i];
    if (dimStride) dimStride[i] = (Int)desc->strides[i];
  }
  return MLUOP_STATUS_SUCCESS;
}

}  // namespace

extern "C" {

mluOpStatus_t MLUOP_WIN_API mluOpCreateTensorDescriptor(mluOpTensorDescriptor_t *desc) {
  PARAM_CHECK("[mluOpCreateTensorDescriptor]", desc != NULL);
  *desc = pool().take();
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpDestroyTensorDescriptor(mluOpTensorDescriptor_t desc) {
  PARAM_CHECK("[mluOpDestroyTensorDescriptor]", desc != NULL);
  pool().give(desc);
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpSetTensorDescriptor(mluOpTensorDescriptor_t desc, mluOpTensorLayout_t layout,
                                                     mluOpDataType_t dtype, int dimNb, const int dimSize[]) {
  PARAM_CHECK("[mluOpSetTensorDescriptor]", desc != NULL);
  return desc->set<int>(layout, dtype, dimNb, dimSize);
}

mluOpStatus_t MLUOP_WIN_API mluOpSetTensorDescriptor_v2(mluOpTensorDescriptor_t desc,
                                                        mluOpTensorLayout_t layout, mluOpDataType_t dtype,
                                                        int dimNb, const int64_t dimSize[]) {
  PARAM_CHECK("[mluOpSetTensorDescriptor]", desc != NULL);
  return desc->set<int64_t>(layout, dtype, dimNb, dimSize);
}

mluOpStatus_t MLUOP_WIN_API mluOpSetTensorDescriptorEx(mluOpTensorDescriptor_t desc,
                                                       mluOpTensorLayout_t layout, mluOpDataType_t dtype,
                                                       int dimNb, const int dimSize[],
                                                       const int dimStride[]) {
  PARAM_CHECK("[mluOpSetTensorDescriptorEx]", desc != NULL);
  return desc->setEx<int>(layout, dtype, dimNb, dimSize, dimStride);
}

mluOpStatus_t MLUOP_WIN_API mluOpSetTensorDescriptorEx_v2(mluOpTensorDescriptor_t desc,
                                                          mluOpTensorLayout_t layout,
                                                          mluOpDataType_t dtype, int dimNb,
                                                          const int64_t dimSize[],
                                                          const int64_t dimStride[]) {
  PARAM_CHECK("[mluOpSetTensorDescriptorEx]", desc != NULL);
  return desc->setEx<int64_t>(layout, dtype, dimNb, dimSize, dimStride);
}

mluOpStatus_t MLUOP_WIN_API mluOpResetTensorDescriptor(mluOpTensorDescriptor_t desc) {
  PARAM_CHECK("[mluOpResetTensorDescriptor]", desc != NULL);
  desc->~mluOpTensorStruct();
  ::new (desc) mluOpTensorStruct;
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpGetTensorDescriptor(const mluOpTensorDescriptor_t desc,
                                                     mluOpTensorLayout_t *layout, mluOpDataType_t *dtype,
                                                     int *dimNb, int dimSize[]) {
  PARAM_CHECK("[mluOpGetTensorDescriptor]", desc != NULL);
  return readBack<int>(desc, layout, dtype, dimNb, dimSize, nullptr);
}

mluOpStatus_t MLUOP_WIN_API mluOpGetTensorDescriptor_v2(const mluOpTensorDescriptor_t desc,
                                                        mluOpTensorLayout_t *layout,
                                                        mluOpDataType_t *dtype, int *dimNb,
                                                        int64_t dimSize[]) {
  PARAM_CHECK("[mluOpGetTensorDescriptor]", desc != NULL);
  return readBack<int64_t>(desc, layout, dtype, dimNb, dimSize, nullptr);
}

mluOpStatus_t MLUOP_WIN_API mluOpGetTensorDescriptorEx(const mluOpTensorDescriptor_t desc,
                                                       mluOpTensorLayout_t *layout,
                                                       mluOpDataType_t *dtype, int *dimNb, int dimSize[],
                                                       int dimStride[]) {
  PARAM_CHECK("[mluOpGetTensorDescriptorEx]", desc != NULL);
  return readBack<int>(desc, layout, dtype, dimNb, dimSize, dimStride);
}

uint64_t MLUOP_WIN_API mluOpGetTensorElementNum(const mluOpTensorDescriptor_t desc) {
  if (desc == NULL) {
    LOG(ERROR) << "[mluOpGetTensorElementNum] Check failed: desc != NULL.";
    return 0;
  }
  return desc->getTotalElementNum();
}

}  // extern "C"

namespace {
int64_t dimByLayout(const mluOpTensorDescriptor_t desc, const char *which, const int index_of[11]) {
  int layout = (int)desc->getLayout();
  if (layout >= 0 && layout <= 10 && index_of[layout] >= 0) return desc->getDimIndex(index_of[layout]);
  LOG(ERROR) << "Failed to call dim" << which << ", illegal layout in TensorDescriptor.";
  return 0;
}
}  // namespace

// index of the wanted axis per layout, in enum order
// NCHW NHWC HWCN NDHWC ARRAY NCDHW TNC NTC NC NLC NCL
int64_t mluOpGetTensordimN(const mluOpTensorDescriptor_t d) {
  static const int at[11] = {0, 0, 3, 0, -1, 0, 1, -1, 0, 0, 0};
  return dimByLayout(d, "N", at);
}
int64_t mluOpGetTensordimD(const mluOpTensorDescriptor_t d) {
  static const int at[11] = {-1, -1, -1, 1, -1, 2, -1, -1, -1, -1, -1};
  return dimByLayout(d, "D", at);
}
int64_t mluOpGetTensordimC(const mluOpTensorDescriptor_t d) {
  static const int at[11] = {1, 3, 2, 4, -1, 1, 2, 2, 1, 2, 1};
  return dimByLayout(d, "C", at);
}
int64_t mluOpGetTensordimH(const mluOpTensorDescriptor_t d) {
  static const int at[11] = {2, 1, 0, 2, -1, 3, -1, -1, -1, -1, -1};
  return dimByLayout(d, "H", at);
}
int64_t mluOpGetTensordimW(const mluOpTensorDescriptor_t d) {
  static const int at[11] = {3, 2, 1, 3, -1, 4, -1, -1, -1, -1, -1};
  return dimByLayout(d, "W", at);
}
