// Status strings and data-type sizes (reference core/type.cpp:53-80).
#include "core/type.h"

#include "core/logging.h"

extern "C" {

const char *MLUOP_WIN_API mluOpGetErrorString(mluOpStatus_t status) {
  switch (status) {
    case MLUOP_STATUS_SUCCESS: return "MLUOP_STATUS_SUCCESS";
    case MLUOP_STATUS_NOT_INITIALIZED: return "MLUOP_STATUS_NOT_INITIALIZED";
    case MLUOP_STATUS_ALLOC_FAILED: return "MLUOP_STATUS_ALLOC_FAILED";
    case MLUOP_STATUS_BAD_PARAM: return "MLUOP_STATUS_BAD_PARAM";
    case MLUOP_STATUS_INTERNAL_ERROR: return "MLUOP_STATUS_INTERNAL_ERROR";
    case MLUOP_STATUS_ARCH_MISMATCH: return "MLUOP_STATUS_ARCH_MISMATCH";
    case MLUOP_STATUS_EXECUTION_FAILED: return "MLUOP_STATUS_EXECUTION_FAILED";
    case MLUOP_STATUS_NOT_SUPPORTED: return "MLUOP_STATUS_NOT_SUPPORTED";
    case MLUOP_STATUS_NUMERICAL_OVERFLOW: return "MLUOP_STATUS_NUMERICAL_OVERFLOW";
  }
  return "MLUOP_STATUS_UNKNOWN";
}

mluOpStatus_t MLUOP_WIN_API mluOpGetSizeOfDataType(mluOpDataType_t data_type, size_t *size) {
  PARAM_CHECK("[mluOpGetSizeOfDataType]", size != NULL);
  if (data_type != MLUOP_DTYPE_INVALID) {
    *size = mluop::getSizeOfDataType(data_type);
    return MLUOP_STATUS_SUCCESS;
  }
  LOG(ERROR) << "[mluOpGetSizeOfDataType] does not support MLUOP_DTYPE_INVALID.";
  return MLUOP_STATUS_BAD_PARAM;
}

}  // extern "C"

namespace mluop {

const char *getNameOfTensorLayout(mluOpTensorLayout_t layout) {
  static const char *names[] = {"LAYOUT_NCHW", "LAYOUT_NHWC", "LAYOUT_HWCN", "LAYOUT_NDHWC",
                                "LAYOUT_ARRAY", "LAYOUT_NCDHW", "LAYOUT_TNC", "LAYOUT_NTC",
                                "LAYOUT_NC", "LAYOUT_NLC", "LAYOUT_NCL"};
  int i = static_cast<int>(layout);
  return (i >= 0 && i <= 10) ? names[i] : "LAYOUT_ARRAY";
}

const char *getNameOfDataType(mluOpDataType_t dtype) {
  switch (dtype) {
    case MLUOP_DTYPE_HALF: return "half";
    case MLUOP_DTYPE_FLOAT: return "float";
    case MLUOP_DTYPE_DOUBLE: return "double";
    case MLUOP_DTYPE_INT8: return "int8";
    case MLUOP_DTYPE_INT16: return "int16";
    case MLUOP_DTYPE_INT31: return "int31";
    case MLUOP_DTYPE_INT32: return "int32";
    case MLUOP_DTYPE_INT64: return "int64";
    case MLUOP_DTYPE_UINT8: return "uint8";
    case MLUOP_DTYPE_UINT16: return "uint16";
    case MLUOP_DTYPE_UINT32: return "uint32";
    case MLUOP_DTYPE_UINT64: return "uint64";
    case MLUOP_DTYPE_BOOL: return "bool";
    case MLUOP_DTYPE_COMPLEX_HALF: return "complex_half";
    case MLUOP_DTYPE_COMPLEX_FLOAT: return "complex_float";
    case MLUOP_DTYPE_BFLOAT16: return "bfloat16";
    default: return "invalid";
  }
}

}  // namespace mluop
