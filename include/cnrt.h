/*
 * cnrt.h -- stand-in for the vendor runtime header that the reference's
 * mlu_op.h includes (reference mlu_op.h:44).  On this build a queue is a CUDA
 * stream, so code that names cnrtQueue_t keeps compiling.  Only the types the
 * sparse-convolution API mentions are provided.
 */
#ifndef MLUOP_B200_CNRT_H_
#define MLUOP_B200_CNRT_H_

#if defined(__CUDACC__) || defined(MLUOP_B200_HAVE_CUDA_RUNTIME)
#include <cuda_runtime_api.h>
#else
/* Same opaque pointer type the CUDA runtime declares; lets plain C/C++ callers
 * include the API without the CUDA toolkit on their include path. */
typedef struct CUstream_st *cudaStream_t;
#endif

typedef cudaStream_t cnrtQueue_t;

#endif /* MLUOP_B200_CNRT_H_ */
