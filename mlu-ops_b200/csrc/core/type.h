// Data-type helpers (reference core/type.h:55, core/type.cpp:53).
#ifndef MLUOP_B200_CORE_TYPE_H_
#define MLUOP_B200_CORE_TYPE_H_

#include <cstddef>

#include "mlu_op.h"

namespace mluop {

inline size_t getSizeOfDataType(mluOpDataType_t dtype) {
  switch (dtype) {
    case MLUOP_DTYPE_BOOL:
    case MLUOP_DTYPE_INT8:
    case MLUOP_DTYPE_UINT8:
      return 1;
    case MLUOP_DTYPE_INT16:
    case MLUOP_DTYPE_UINT16:
    case MLUOP_DTYPE_HALF:
    case MLUOP_DTYPE_BFLOAT16:
      return 2;
    case MLUOP_DTYPE_INT31:
    case MLUOP_DTYPE_INT32:
    case MLUOP_DTYPE_UINT32:
    case MLUOP_DTYPE_FLOAT:
    case MLUOP_DTYPE_COMPLEX_HALF:
      return 4;
    case MLUOP_DTYPE_UINT64:
    case MLUOP_DTYPE_INT64:
    case MLUOP_DTYPE_DOUBLE:
    case MLUOP_DTYPE_COMPLEX_FLOAT:
      return 8;
    default:
      return 0;
  }
}

const char *getNameOfTensorLayout(mluOpTensorLayout_t layout);
const char *getNameOfDataType(mluOpDataType_t dtype);

}  // namespace mluop

#endif  // MLUOP_B200_CORE_TYPE_H_
