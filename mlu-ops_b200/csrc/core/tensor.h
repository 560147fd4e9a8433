// Tensor descriptor: layout, dtype, dims and strides of one tensor
// (reference core/tensor.h:41-235; only the members the sparse-convolution
// path and its callers touch).  Up to MLUOP_DIM_MAX dims live inline, more go
// to the heap.
#ifndef MLUOP_B200_CORE_TENSOR_H_
#define MLUOP_B200_CORE_TENSOR_H_

#include <cstdint>

#include "core/logging.h"
#include "core/type.h"
#include "mlu_op.h"

struct mluOpTensorStruct {
  mluOpTensorStruct() { reset(); }
  ~mluOpTensorStruct() { releaseHeapDims(); }
  mluOpTensorStruct(const mluOpTensorStruct &) = delete;
  mluOpTensorStruct &operator=(const mluOpTensorStruct &) = delete;

  // Accessors with the reference's names.
  int getDim() const { return dim; }
  int64_t getDimIndex(int i) const { return dims[i]; }
  int64_t getStrideIndex(int i) const { return strides[i]; }
  const int64_t *getDims() const { return dims; }
  const int64_t *getStrides() const { return strides; }
  mluOpDataType_t getDtype() const { return dtype; }
  mluOpTensorLayout_t getLayout() const { return layout; }
  uint64_t getTotalElementNum() const { return total_element_num; }
  uint64_t getTotalTensorSize() const { return total_tensor_size; }

  void reset();
  // dims with contiguous strides
  template <typename Int>
  mluOpStatus_t set(mluOpTensorLayout_t layout, mluOpDataType_t dtype, int dimNb, const Int *dimSize);
  // dims with caller strides
  template <typename Int>
  mluOpStatus_t setEx(mluOpTensorLayout_t layout, mluOpDataType_t dtype, int dimNb, const Int *dimSize,
                      const Int *dimStride);

  int dim;
  int64_t *dims;
  int64_t *strides;
  mluOpDataType_t dtype;
  mluOpTensorLayout_t layout;
  uint64_t total_element_num;
  uint64_t total_tensor_size;

 private:
  void resizeDims(int dimNb);
  void releaseHeapDims();
  int64_t inline_dims_[MLUOP_DIM_MAX];
  int64_t inline_strides_[MLUOP_DIM_MAX];
};

// Layout-aware dimension getters (reference core/tensor.h:387-478).
int64_t mluOpGetTensordimN(const mluOpTensorDescriptor_t desc);
int64_t mluOpGetTensordimD(const mluOpTensorDescriptor_t desc);
int64_t mluOpGetTensordimC(const mluOpTensorDescriptor_t desc);
int64_t mluOpGetTensordimH(const mluOpTensorDescriptor_t desc);
int64_t mluOpGetTensordimW(const mluOpTensorDescriptor_t desc);

inline int mluOpDataTypeBytes(mluOpDataType_t dt) { return (int)mluop::getSizeOfDataType(dt); }

#endif  // MLUOP_B200_CORE_TENSOR_H_
