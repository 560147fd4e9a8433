/*
 * mlu_op.h -- C API of the B200 (sm_100a) build of the sparse-convolution
 * forward path of mlu-ops.
 *
 * This header declares the subset of the reference's public header that the
 * path needs, with identical names, argument lists, enum values and status
 * conventions, so that code written against the reference recompiles
 * unchanged.  The only type that differs is the queue: a cnrtQueue_t here is a
 * cudaStream_t (see the stand-in header cnrt.h next to this file).
 *
 * Every declaration cites the reference declaration it replaces as
 * mlu_op.h:<line> (the reference's single public header) and the reference
 * implementation as <file>:<line> inside the reference tree.
 *
 * All pointers named *_desc and handle are host objects of this library.
 * All data pointers (indices, features, filters, workspace, outputs) are
 * device pointers, except indice_num[] of the two convolution functions,
 * which is a host array (reference mlu_op.h:10357-10358).
 */
#ifndef MLUOP_B200_MLU_OP_H_
#define MLUOP_B200_MLU_OP_H_

#define MLUOP_MAJOR 1       /* reference mlu_op.h:30 */
#define MLUOP_MINOR 11      /* reference mlu_op.h:31 */
#define MLUOP_PATCHLEVEL 1  /* reference mlu_op.h:32 */
#define MLUOP_VERSION (MLUOP_MAJOR * 1000 + MLUOP_MINOR * 100 + MLUOP_PATCHLEVEL)
#define MLUOP_DIM_MAX 8     /* reference mlu_op.h:39 */

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#include "cn_api.h" /* stand-in: CNdev */
#include "cnrt.h"   /* stand-in: cnrtQueue_t = cudaStream_t */

#ifndef MLUOP_WIN_API
#define MLUOP_WIN_API
#endif

#if defined(__cplusplus)
extern "C" {
#endif

/* reference mlu_op.h:63-94 */
typedef enum {
  MLUOP_STATUS_SUCCESS = 0,
  MLUOP_STATUS_NOT_INITIALIZED = 1,
  MLUOP_STATUS_ALLOC_FAILED = 2,
  MLUOP_STATUS_BAD_PARAM = 3,
  MLUOP_STATUS_INTERNAL_ERROR = 4,
  MLUOP_STATUS_ARCH_MISMATCH = 5,
  MLUOP_STATUS_EXECUTION_FAILED = 6,
  MLUOP_STATUS_NOT_SUPPORTED = 7,
  MLUOP_STATUS_NUMERICAL_OVERFLOW = 8,
} mluOpStatus_t;

/* reference mlu_op.h:115-140 */
typedef enum {
  MLUOP_LAYOUT_NCHW = 0,
  MLUOP_LAYOUT_NHWC = 1,
  MLUOP_LAYOUT_HWCN = 2,
  MLUOP_LAYOUT_NDHWC = 3,
  MLUOP_LAYOUT_ARRAY = 4,
  MLUOP_LAYOUT_NCDHW = 5,
  MLUOP_LAYOUT_TNC = 6,
  MLUOP_LAYOUT_NTC = 7,
  MLUOP_LAYOUT_NC = 8,
  MLUOP_LAYOUT_NLC = 9,
  MLUOP_LAYOUT_NCL = 10,
} mluOpTensorLayout_t;

/* reference mlu_op.h:169-189 */
typedef enum {
  MLUOP_DTYPE_INVALID = 0,
  MLUOP_DTYPE_HALF = 1,
  MLUOP_DTYPE_FLOAT = 2,
  MLUOP_DTYPE_DOUBLE = 14,
  MLUOP_DTYPE_INT8 = 3,
  MLUOP_DTYPE_INT16 = 4,
  MLUOP_DTYPE_INT31 = 5,
  MLUOP_DTYPE_INT32 = 6,
  MLUOP_DTYPE_INT64 = 9,
  MLUOP_DTYPE_UINT8 = 7,
  MLUOP_DTYPE_UINT16 = 13,
  MLUOP_DTYPE_UINT32 = 11,
  MLUOP_DTYPE_UINT64 = 12,
  MLUOP_DTYPE_BOOL = 8,
  MLUOP_DTYPE_COMPLEX_HALF = 15,
  MLUOP_DTYPE_COMPLEX_FLOAT = 16,
  MLUOP_DTYPE_BFLOAT16 = 17,
} mluOpDataType_t;

/* reference mlu_op.h:214-220 */
typedef enum {
  MLUOP_ATOMICS_NOT_ALLOWED = 1,
  MLUOP_ATOMICS_ALLOWED = 2,
} mluOpAtomicsMode_t;

/* reference mlu_op.h:404, :889, :1161 */
typedef struct mluOpContext *mluOpHandle_t;
typedef struct mluOpTensorStruct *mluOpTensorDescriptor_t;
typedef struct mluOpSparseConvolutionStruct *mluOpSparseConvolutionDescriptor_t;

/* ---------------------------------------------------------------- handle */

/* reference mlu_op.h:456, core/context.cpp:158.  Binds the handle to the
 * current CUDA device; the queue starts as the NULL (default) stream.
 * MLUOP_STATUS_NOT_INITIALIZED when no CUDA device can be used. */
mluOpStatus_t MLUOP_WIN_API mluOpCreate(mluOpHandle_t *handle);

/* reference mlu_op.h:530, core/context.cpp:354 */
mluOpStatus_t MLUOP_WIN_API mluOpDestroy(mluOpHandle_t handle);

/* reference mlu_op.h:571, core/context.cpp:362.  queue may be NULL. */
mluOpStatus_t MLUOP_WIN_API mluOpSetQueue(mluOpHandle_t handle, cnrtQueue_t queue);

/* reference mlu_op.h:608, core/context.cpp:372 */
mluOpStatus_t MLUOP_WIN_API mluOpGetQueue(mluOpHandle_t handle, cnrtQueue_t *queue);

/* reference core/context.cpp:382 (mluOpGetDevice) */
mluOpStatus_t MLUOP_WIN_API mluOpGetDevice(mluOpHandle_t handle, CNdev *device);

/* reference mlu_op.h:646, core/type.cpp:53 */
const char *MLUOP_WIN_API mluOpGetErrorString(mluOpStatus_t status);

/* reference mlu_op.h:682, core/type.h:55 */
mluOpStatus_t MLUOP_WIN_API mluOpGetSizeOfDataType(mluOpDataType_t data_type, size_t *size);

/* reference mlu_op.h:722, core/context.cpp:462 */
void MLUOP_WIN_API mluOpGetLibVersion(int *major, int *minor, int *patch);

/* reference mlu_op.h:837 / :874, core/context.cpp.  The default mode,
 * MLUOP_ATOMICS_NOT_ALLOWED, is the only one this path uses: every kernel on
 * it is deterministic. */
mluOpStatus_t MLUOP_WIN_API mluOpSetAtomicsMode(mluOpHandle_t handle, mluOpAtomicsMode_t atomics_mode);
mluOpStatus_t MLUOP_WIN_API mluOpGetAtomicsMode(mluOpHandle_t handle, mluOpAtomicsMode_t *atomics_mode);

/* ---------------------------------------------------- tensor descriptors */

/* reference mlu_op.h:1233, core/tensor.cpp:560 */
mluOpStatus_t MLUOP_WIN_API mluOpCreateTensorDescriptor(mluOpTensorDescriptor_t *desc);

/* reference mlu_op.h:1406, core/tensor.cpp:602.  Contiguous strides are derived. */
mluOpStatus_t MLUOP_WIN_API mluOpSetTensorDescriptor(mluOpTensorDescriptor_t desc,
                                                     mluOpTensorLayout_t layout,
                                                     mluOpDataType_t dtype, int dimNb,
                                                     const int dimSize[]);

/* reference mlu_op.h:1511, core/tensor.cpp:609 */
mluOpStatus_t MLUOP_WIN_API mluOpSetTensorDescriptor_v2(mluOpTensorDescriptor_t desc,
                                                        mluOpTensorLayout_t layout,
                                                        mluOpDataType_t dtype, int dimNb,
                                                        const int64_t dimSize[]);

/* reference mlu_op.h:1815, core/tensor.cpp:680.  Explicit strides (elements). */
mluOpStatus_t MLUOP_WIN_API mluOpSetTensorDescriptorEx(mluOpTensorDescriptor_t desc,
                                                       mluOpTensorLayout_t layout,
                                                       mluOpDataType_t dtype, int dimNb,
                                                       const int dimSize[],
                                                       const int dimStride[]);

/* reference mlu_op.h:1874, core/tensor.cpp:688 */
mluOpStatus_t MLUOP_WIN_API mluOpSetTensorDescriptorEx_v2(mluOpTensorDescriptor_t desc,
                                                          mluOpTensorLayout_t layout,
                                                          mluOpDataType_t dtype, int dimNb,
                                                          const int64_t dimSize[],
                                                          const int64_t dimStride[]);

/* reference mlu_op.h:1761, core/tensor.cpp:675 */
mluOpStatus_t MLUOP_WIN_API mluOpResetTensorDescriptor(mluOpTensorDescriptor_t desc);

/* reference mlu_op.h:2173, core/tensor.cpp:751 */
mluOpStatus_t MLUOP_WIN_API mluOpGetTensorDescriptor(const mluOpTensorDescriptor_t desc,
                                                     mluOpTensorLayout_t *layout,
                                                     mluOpDataType_t *dtype, int *dimNb,
                                                     int dimSize[]);

/* reference mlu_op.h:2221, core/tensor.cpp:758 */
mluOpStatus_t MLUOP_WIN_API mluOpGetTensorDescriptor_v2(const mluOpTensorDescriptor_t desc,
                                                        mluOpTensorLayout_t *layout,
                                                        mluOpDataType_t *dtype, int *dimNb,
                                                        int64_t dimSize[]);

/* reference mlu_op.h:2274, core/tensor.cpp:736 */
mluOpStatus_t MLUOP_WIN_API mluOpGetTensorDescriptorEx(const mluOpTensorDescriptor_t desc,
                                                       mluOpTensorLayout_t *layout,
                                                       mluOpDataType_t *dtype, int *dimNb,
                                                       int dimSize[], int dimStride[]);

/* reference mlu_op.h:2377, core/tensor.cpp:854 */
uint64_t MLUOP_WIN_API mluOpGetTensorElementNum(const mluOpTensorDescriptor_t desc);

/* reference mlu_op.h:2573, core/tensor.cpp:817 */
mluOpStatus_t MLUOP_WIN_API mluOpDestroyTensorDescriptor(mluOpTensorDescriptor_t desc);

/* ------------------------------------------- sparse-convolution descriptor */

/* reference mlu_op.h:1272, get_indice_pairs_structs.cpp:31.
 * NULL argument -> MLUOP_STATUS_NOT_INITIALIZED. */
mluOpStatus_t MLUOP_WIN_API
mluOpCreateSparseConvolutionDescriptor(mluOpSparseConvolutionDescriptor_t *desc);

/* reference mlu_op.h:1311, get_indice_pairs_structs.cpp:125.
 * NULL argument -> MLUOP_STATUS_EXECUTION_FAILED. */
mluOpStatus_t MLUOP_WIN_API
mluOpDestroySparseConvolutionDescriptor(mluOpSparseConvolutionDescriptor_t desc);

/* reference mlu_op.h:1607, get_indice_pairs_structs.cpp:47.  dimNb must be 5,
 * batch > 0, transpose == 0, inverse == 0, pad >= 0, everything else >= 1.
 * The three-element arrays are in (D, H, W) order. */
mluOpStatus_t MLUOP_WIN_API mluOpSetSparseConvolutionDescriptor(
    mluOpSparseConvolutionDescriptor_t desc, int dimNb, int batch, const int pad[],
    const int stride[], const int dilation[], const int input_space[],
    const int filter_space[], const int output_space[], const int sub_m,
    const int transpose, const int inverse);

/* reference mlu_op.h:1654, get_indice_pairs_structs.cpp:111.  The value is
 * written by mluOpGetIndicePairs: the number of active output voxels in
 * default mode; in submanifold mode this library stores the number of input
 * voxels (the reference leaves the field untouched in that mode). */
mluOpStatus_t MLUOP_WIN_API
mluOpGetSparseConvolutionNumActOut(mluOpSparseConvolutionDescriptor_t desc, int *num_act_out);

/* ------------------------------------------------------------ the hot path */

/* reference mlu_op.h:8674, get_indice_pairs.cpp:251.  Bytes of device scratch
 * mluOpGetIndicePairs needs for these descriptors.  Upper bound: with an
 * occupancy table (default mode; submanifold mode on grids of at most 1024 cells
 * per voxel) cells / 4 + 16 * L + 1 MiB, where cells = batch * D * H * W of the
 * output space, i.e. at most 512 MiB at the 2^31-cell limit; with a hash table
 * (sparser submanifold grids) 40 * L + 1 MiB.  Kernel volumes above 32 add
 * 4 * K * L for the staged matches. */
mluOpStatus_t MLUOP_WIN_API mluOpGetIndicePairsWorkspaceSize(
    mluOpHandle_t handle, mluOpSparseConvolutionDescriptor_t sparse_conv_desc,
    const mluOpTensorDescriptor_t indices_desc,
    const mluOpTensorDescriptor_t indice_pairs_desc,
    const mluOpTensorDescriptor_t out_indices_desc,
    const mluOpTensorDescriptor_t indice_num_desc, size_t *workspace_size);

/* reference mlu_op.h:8598, get_indice_pairs.cpp:237 ->
 * normal_get_indice_pairs.cpp:831.  Rulebook generation:
 *   indices       [L,4]  int32 rows (b, z, y, x)
 *   indice_pairs  [K,2,L] int32: row [k,0,:] input ids ascending, row [k,1,:]
 *                 the matching output ids, -1 from position indice_num[k] on
 *   out_indices   [rows,4] int32: coordinates of the active outputs in
 *                 ascending linear order (default mode) or a copy of indices
 *                 (sub_m); rows past the active count are set to -1
 *   indice_num    [K] int32 (device)
 * indices and out_indices must be 16-byte aligned (a coordinate row is moved as
 * one 16-byte word); a pointer that is not is MLUOP_STATUS_BAD_PARAM.
 * Work is enqueued on the handle's queue.  In default mode the call blocks
 * once to read the number of active outputs into the descriptor. */
mluOpStatus_t MLUOP_WIN_API mluOpGetIndicePairs(
    mluOpHandle_t handle, mluOpSparseConvolutionDescriptor_t sparse_conv_desc,
    const mluOpTensorDescriptor_t indices_desc, const void *indices, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t indice_pairs_desc,
    void *indice_pairs, const mluOpTensorDescriptor_t out_indices_desc, void *out_indices,
    const mluOpTensorDescriptor_t indice_num_desc, void *indice_num);

/* reference mlu_op.h:10322, indice_convolution_forward.cpp:581 */
mluOpStatus_t MLUOP_WIN_API mluOpGetIndiceConvolutionForwardWorkspaceSize(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc,
    const mluOpTensorDescriptor_t filters_desc,
    const mluOpTensorDescriptor_t indice_pairs_desc,
    const mluOpTensorDescriptor_t features_out_desc, const int64_t indice_num[],
    const int64_t num_act_out, const int64_t inverse, const int64_t sub_m,
    size_t *workspace_size);

/* reference mlu_op.h:10434, indice_convolution_forward.cpp:621.
 *   features_out[r,:] = sum_k sum_{(j,r) in pairs_k} features[j,:] * W_k
 * features [L,Ci], filters 5-D (NDHWC [Co,kd,kh,kw,Ci], NCDHW [Co,Ci,kd,kh,kw]
 * or ARRAY [kd,kh,kw,Ci,Co]), features_out [num_act_out,Co]; half or float,
 * all three the same; accumulation is in float, kernel offset ascending.
 * Output rows without a pair are zero.  Asynchronous on the handle's queue. */
mluOpStatus_t MLUOP_WIN_API mluOpIndiceConvolutionForward(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc,
    const void *features, const mluOpTensorDescriptor_t filters_desc, const void *filters,
    const mluOpTensorDescriptor_t indice_pairs_desc, const void *indice_pairs,
    const int64_t indice_num[], const int64_t num_act_out, const int64_t inverse,
    const int64_t sub_m, void *workspace, const size_t workspace_size,
    const mluOpTensorDescriptor_t features_out_desc, void *features_out);

/* reference mlu_op.h:9626, indice_convolution_backward_data.cpp:358 */
mluOpStatus_t MLUOP_WIN_API mluOpGetIndiceConvolutionBackwardDataWorkspaceSize(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t output_grad_desc,
    const mluOpTensorDescriptor_t filters_desc,
    const mluOpTensorDescriptor_t indice_pairs_desc,
    const mluOpTensorDescriptor_t input_grad_desc, const int64_t indice_num[],
    const int64_t inverse, size_t *workspace_size);

/* reference mlu_op.h:9760, indice_convolution_backward_data.cpp:568.
 *   input_grad[i,:] = sum_k sum_{(i,o) in pairs_k} output_grad[o,:] * W_k^T
 * output_grad [N_out,Co], input_grad [L,Ci] (L = indice_pairs dims[2]); filters
 * 4-D (NHWC, NCHW, HWCN) or 5-D (NDHWC, NCDHW, ARRAY = [kd,kh,kw,Ci,Co]); half
 * or float, all three the same; accumulation in float, kernel offset ascending.
 * Input rows without a pair are zero.  Asynchronous on the handle's queue. */
mluOpStatus_t MLUOP_WIN_API mluOpIndiceConvolutionBackwardData(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t output_grad_desc,
    const void *output_grad, const mluOpTensorDescriptor_t filters_desc, const void *filters,
    const mluOpTensorDescriptor_t indice_pairs_desc, const void *indice_pairs,
    const int64_t indice_num[], const int64_t inverse, const int64_t sub_m, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t input_grad_desc,
    void *input_grad);

/* reference mlu_op.h:9838, indice_convolution_backward_filter.cpp:531 */
mluOpStatus_t MLUOP_WIN_API mluOpGetIndiceConvolutionBackwardFilterWorkspaceSize(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc,
    const mluOpTensorDescriptor_t output_grad_desc,
    const mluOpTensorDescriptor_t indice_pairs_desc,
    const mluOpTensorDescriptor_t filters_grad_desc, const int64_t indice_num[],
    const int64_t inverse, const int64_t sub_m, size_t *workspace_size);

/* reference mlu_op.h:9934, indice_convolution_backward_filter.cpp:570.
 *   filters_grad[k,c,n] = sum_{(i,o) in pairs_k} features[i,c] * output_grad[o,n]
 * features [L,Ci], output_grad [N_out,Co], filters_grad 4-D [kh,kw,Ci,Co] or 5-D
 * [kd,kh,kw,Ci,Co] (the reference writes this order whatever layout tag the
 * descriptor carries); half or float, all three the same; accumulation in
 * float in a fixed order (results are reproducible run to run).  Kernel offsets
 * without pairs give zeros.  Asynchronous on the handle's queue. */
mluOpStatus_t MLUOP_WIN_API mluOpIndiceConvolutionBackwardFilter(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc, const void *features,
    const mluOpTensorDescriptor_t output_grad_desc, const void *output_grad,
    const mluOpTensorDescriptor_t indice_pairs_desc, const void *indice_pairs,
    const int64_t indice_num[], const int64_t inverse, const int64_t sub_m, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t filters_grad_desc,
    void *filters_grad);

/* ------------------------------------------- neighbour-table fast path */

/* No counterpart in the reference (the four entry points below).
 * mluOpIndiceConvolutionForward converts indice_pairs into a neighbour table
 * (int32 [K][rows padded to 512]: the input row that feeds an output row at a
 * kernel offset, -1 if none) on every call.  Layers that share a rulebook can
 * build that table once and run every convolution from it:
 *   mluOpGetIndiceNeighbourTableSize  -> bytes of the table (caller allocates, 16-byte aligned)
 *   mluOpBuildIndiceNeighbourTable    -> fills it from indice_pairs / indice_num (kernel volume <= 128)
 *   mluOpGetIndiceConvolutionForwardFromTableWorkspaceSize / mluOpIndiceConvolutionForwardFromTable
 *       -> mluOpIndiceConvolutionForward with (table, table_size) in place of the
 *          indice_pairs pointer; same checks, same results bit for bit.
 *   mluOpGetIndicePairsWithNeighbourTable
 *       -> mluOpGetIndicePairs that also fills the table while it has every match
 *          in hand (no separate build).  Only for submanifold rulebooks with odd
 *          kernel sizes (volume <= 32), unit stride and dilation and pad = size / 2;
 *          any other rulebook is MLUOP_STATUS_NOT_SUPPORTED before anything is
 *          launched, and the caller builds the table from indice_pairs instead.
 * The table is valid as long as indice_pairs, indice_num and num_act_out are. */
mluOpStatus_t MLUOP_WIN_API mluOpGetIndiceNeighbourTableSize(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t indice_pairs_desc,
    const int64_t num_act_out, size_t *table_size);

mluOpStatus_t MLUOP_WIN_API mluOpBuildIndiceNeighbourTable(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t indice_pairs_desc,
    const void *indice_pairs, const int64_t indice_num[], const int64_t num_act_out,
    void *table, const size_t table_size);

mluOpStatus_t MLUOP_WIN_API mluOpGetIndicePairsWithNeighbourTable(
    mluOpHandle_t handle, mluOpSparseConvolutionDescriptor_t sparse_conv_desc,
    const mluOpTensorDescriptor_t indices_desc, const void *indices, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t indice_pairs_desc,
    void *indice_pairs, const mluOpTensorDescriptor_t out_indices_desc, void *out_indices,
    const mluOpTensorDescriptor_t indice_num_desc, void *indice_num, void *table,
    const size_t table_size);

mluOpStatus_t MLUOP_WIN_API mluOpGetIndiceConvolutionForwardFromTableWorkspaceSize(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc,
    const mluOpTensorDescriptor_t filters_desc,
    const mluOpTensorDescriptor_t indice_pairs_desc,
    const mluOpTensorDescriptor_t features_out_desc, const int64_t indice_num[],
    const int64_t num_act_out, const int64_t inverse, const int64_t sub_m,
    size_t *workspace_size);

mluOpStatus_t MLUOP_WIN_API mluOpIndiceConvolutionForwardFromTable(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc,
    const void *features, const mluOpTensorDescriptor_t filters_desc, const void *filters,
    const mluOpTensorDescriptor_t indice_pairs_desc, const void *table,
    const size_t table_size, const int64_t indice_num[], const int64_t num_act_out,
    const int64_t inverse, const int64_t sub_m, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t features_out_desc,
    void *features_out);

/* The same for the gradients (no counterpart in the reference either).
 *
 * Input gradient: mluOpIndiceConvolutionBackwardData works from the table of the
 * opposite direction (int32 [K][L padded to 512]: the OUTPUT row an input row
 * feeds at a kernel offset, -1 if none) and builds it from indice_pairs on every
 * call.  mluOpGetIndiceInputNeighbourTableSize / mluOpBuildIndiceInputNeighbourTable
 * build it once per rulebook; mluOpIndiceConvolutionBackwardDataFromTable is
 * mluOpIndiceConvolutionBackwardData with (table, table_size) in place of the
 * indice_pairs pointer, its workspace the size
 * mluOpGetIndiceConvolutionBackwardDataFromTableWorkspaceSize reports.  Bit-identical
 * to the reference-shaped call.
 *
 * Filter gradient: the tensor-memory kernel (half, 64 input channels, 64 or 128 output
 * channels, 16-byte aligned rows) works from the FORWARD table (the one
 * mluOpBuildIndiceNeighbourTable builds or mluOpGetIndicePairsWithNeighbourTable emits).
 * mluOpIndiceConvolutionBackwardFilterFromTable is mluOpIndiceConvolutionBackwardFilter
 * with (table, table_size) in place of the indice_pairs pointer and the workspace
 * mluOpGetIndiceConvolutionBackwardFilterWorkspaceSize reports; other shapes return
 * MLUOP_STATUS_NOT_SUPPORTED before anything is enqueued (the caller uses the
 * reference-shaped call).  Bit-identical to the reference-shaped call. */
mluOpStatus_t MLUOP_WIN_API mluOpGetIndiceInputNeighbourTableSize(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t indice_pairs_desc, size_t *table_size);

mluOpStatus_t MLUOP_WIN_API mluOpBuildIndiceInputNeighbourTable(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t indice_pairs_desc, const void *indice_pairs,
    const int64_t indice_num[], const int64_t num_act_out, void *table, const size_t table_size);

mluOpStatus_t MLUOP_WIN_API mluOpGetIndiceConvolutionBackwardDataFromTableWorkspaceSize(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t output_grad_desc,
    const mluOpTensorDescriptor_t filters_desc, const mluOpTensorDescriptor_t indice_pairs_desc,
    const mluOpTensorDescriptor_t input_grad_desc, const int64_t indice_num[], const int64_t inverse,
    size_t *workspace_size);

mluOpStatus_t MLUOP_WIN_API mluOpIndiceConvolutionBackwardDataFromTable(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t output_grad_desc, const void *output_grad,
    const mluOpTensorDescriptor_t filters_desc, const void *filters,
    const mluOpTensorDescriptor_t indice_pairs_desc, const void *table, const size_t table_size,
    const int64_t indice_num[], const int64_t inverse, const int64_t sub_m, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t input_grad_desc, void *input_grad);

/* The input gradient of a SUBMANIFOLD layer with centred padding (stride 1, dilation 1, odd
 * kernel extents, pad = extent / 2) straight from the rulebook's FORWARD table: such a rulebook is
 * symmetric, so the kernel reads the forward table with the offsets mirrored and no input table
 * is built at all.  The caller vouches for the geometry; sub_m must be 1 and input_grad has as
 * many rows as output_grad.  Only the tensor-memory kernel reads a table this way (half, channel
 * counts that are multiples of 8 up to 128, 16-byte aligned rows): anything else returns
 * MLUOP_STATUS_NOT_SUPPORTED before anything is enqueued and the caller uses
 * mluOpIndiceConvolutionBackwardDataFromTable.  Workspace as for that entry point.  Bit-identical
 * to the reference-shaped call.  No counterpart in the reference. */
mluOpStatus_t MLUOP_WIN_API mluOpIndiceConvolutionBackwardDataFromForwardTable(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t output_grad_desc, const void *output_grad,
    const mluOpTensorDescriptor_t filters_desc, const void *filters,
    const mluOpTensorDescriptor_t indice_pairs_desc, const void *table, const size_t table_size,
    const int64_t indice_num[], const int64_t inverse, const int64_t sub_m, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t input_grad_desc, void *input_grad);

mluOpStatus_t MLUOP_WIN_API mluOpIndiceConvolutionBackwardFilterFromTable(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc, const void *features,
    const mluOpTensorDescriptor_t output_grad_desc, const void *output_grad,
    const mluOpTensorDescriptor_t indice_pairs_desc, const void *table, const size_t table_size,
    const int64_t indice_num[], const int64_t inverse, const int64_t sub_m, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t filters_grad_desc, void *filters_grad);

/* ------------------------------------------------ the step before the path */

/* reference mlu_op.h:5942, kernels/voxelization/voxelization.cpp:178.  Bytes of
 * device scratch mluOpVoxelization needs (this implementation's own figure). */
mluOpStatus_t MLUOP_WIN_API mluOpGetVoxelizationWorkspaceSize(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t points_desc,
    const mluOpTensorDescriptor_t voxel_size_desc,
    const mluOpTensorDescriptor_t coors_range_desc, const int32_t max_points,
    const int32_t max_voxels, const int32_t NDim, const bool deterministic,
    const mluOpTensorDescriptor_t voxels_desc, const mluOpTensorDescriptor_t coors_desc,
    const mluOpTensorDescriptor_t num_points_per_voxel_desc,
    const mluOpTensorDescriptor_t voxel_num_desc, size_t *size);

/* reference mlu_op.h:6051, kernels/voxelization/voxelization.cpp:226.  Hard
 * voxelization, deterministic mode (the only mode the reference supports):
 *   points [N,F] float (x, y, z first), voxel_size [3], coors_range [6] =
 *   (x_min, y_min, z_min, x_max, y_max, z_max), all float, on the device
 *   voxels [max_voxels,max_points,F] float, coors [max_voxels,3] int32 (z, y, x),
 *   num_points_per_voxel [max_voxels] int32, voxel_num [1] int32
 * Voxels are numbered in the order of their first points; a voxel keeps its
 * first max_points points in index order; rows past voxel_num are zero.  The
 * grid (round((max - min) / voxel_size) per axis) must have fewer than 2^63 cells.
 * Asynchronous on the handle's queue. */
mluOpStatus_t MLUOP_WIN_API mluOpVoxelization(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t points_desc, const void *points,
    const mluOpTensorDescriptor_t voxel_size_desc, const void *voxel_size,
    const mluOpTensorDescriptor_t coors_range_desc, const void *coors_range,
    const int32_t max_points, const int32_t max_voxels, const int32_t NDim,
    const bool deterministic, void *workspace, size_t workspace_size,
    const mluOpTensorDescriptor_t voxels_desc, void *voxels,
    const mluOpTensorDescriptor_t coors_desc, void *coors,
    const mluOpTensorDescriptor_t num_points_per_voxel_desc, void *num_points_per_voxel,
    const mluOpTensorDescriptor_t voxel_num_desc, void *voxel_num);

/* reference mlu_op.h:361-365 */
typedef enum {
  MLUOP_REDUCE_DSUM = 0,
  MLUOP_REDUCE_DMEAN = 1,
  MLUOP_REDUCE_DMAX = 2,
} mluOpReduceMode_t;

/* reference mlu_op.h:3768, dynamic_point_to_voxel_forward.cpp:193.  Bytes of
 * device scratch mluOpDynamicPointToVoxelForward needs (this implementation's
 * own figure: 32 bytes per point for the sort records, plus counters). */
mluOpStatus_t MLUOP_WIN_API mluOpGetDynamicPointToVoxelForwardWorkspaceSize(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t feats_desc,
    const mluOpTensorDescriptor_t coors_desc, size_t *workspace_size);

/* reference mlu_op.h:3866, dynamic_point_to_voxel_forward.cpp:226.  Groups
 * points by their integer voxel coordinates and reduces their features:
 *   feats [N,C] float, coors [N,3] int32 (rows with a negative entry are set to
 *   (-1,-1,-1) in place and belong to no voxel)
 *   voxel_coors [M,3]: the distinct coordinates in ascending lexicographic order
 *   point2voxel_map [N]: row of voxel_coors of every point, -1 for none
 *   voxel_points_count [M], voxel_num [1], voxel_feats [M,C]: per voxel the
 *   maximum (MLUOP_REDUCE_DMAX) or the mean (MLUOP_REDUCE_DMEAN, summed as
 *   sum_i feats_i / count in point order) of its points' features
 * with M <= N rows allocated by the caller (N to be safe); rows past voxel_num
 * hold zeros (-inf in voxel_feats for the maximum).  Results are reproducible
 * run to run.  Asynchronous on the handle's queue. */
mluOpStatus_t MLUOP_WIN_API mluOpDynamicPointToVoxelForward(
    const mluOpHandle_t handle, const mluOpReduceMode_t reduce_type,
    const mluOpTensorDescriptor_t feats_desc, const void *feats,
    const mluOpTensorDescriptor_t coors_desc, void *coors, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t voxel_feats_desc,
    void *voxel_feats, const mluOpTensorDescriptor_t voxel_coors_desc, void *voxel_coors,
    const mluOpTensorDescriptor_t point2voxel_map_desc, void *point2voxel_map,
    const mluOpTensorDescriptor_t voxel_points_count_desc, void *voxel_points_count,
    const mluOpTensorDescriptor_t voxel_num_desc, void *voxel_num);

/* reference mlu_op.h:3598, dynamic_point_to_voxel_backward.cpp:342 */
mluOpStatus_t MLUOP_WIN_API mluOpGetDynamicPointToVoxelBackwardWorkspaceSize(
    const mluOpHandle_t handle, const mluOpReduceMode_t reduce_type,
    const mluOpTensorDescriptor_t grad_voxel_feats_desc,
    const mluOpTensorDescriptor_t feats_desc, const mluOpTensorDescriptor_t voxel_feats_desc,
    const mluOpTensorDescriptor_t point2voxel_map_desc,
    const mluOpTensorDescriptor_t voxel_points_count_desc,
    const mluOpTensorDescriptor_t voxel_num_desc, size_t *workspace_size);

/* reference mlu_op.h:3708, dynamic_point_to_voxel_backward.cpp:232.  Gradient of
 * mluOpDynamicPointToVoxelForward for MLUOP_REDUCE_DMAX (the only mode the
 * reference supports): per voxel and channel, the point with the smallest index
 * whose feature equals the voxel's maximum receives grad_voxel_feats; all other
 * entries of grad_feats [N,C] are zero.  Asynchronous on the handle's queue. */
mluOpStatus_t MLUOP_WIN_API mluOpDynamicPointToVoxelBackward(
    const mluOpHandle_t handle, const mluOpReduceMode_t reduce_type,
    const mluOpTensorDescriptor_t grad_voxel_feats_desc, const void *grad_voxel_feats,
    const mluOpTensorDescriptor_t feats_desc, const void *feats,
    const mluOpTensorDescriptor_t voxel_feats_desc, const void *voxel_feats,
    const mluOpTensorDescriptor_t point2voxel_map_desc, const void *point2voxel_map,
    const mluOpTensorDescriptor_t voxel_points_count_desc, const void *voxel_points_count,
    const mluOpTensorDescriptor_t voxel_num_desc, const void *voxel_num, void *workspace,
    const size_t workspace_size, const mluOpTensorDescriptor_t grad_feats_desc,
    void *grad_feats);

/* No counterpart in the reference.  Same computation and arguments as
 * mluOpIndiceConvolutionForward, without the workspace pair: the scratch is a
 * fixed array of MLUOP_BUILTIN_CONV_WORKSPACE_BYTES in device memory that
 * belongs to the library itself.  It exists for callers that cannot allocate
 * device memory where they call the library: inference loops that forbid
 * allocator calls once running (cudaMalloc synchronises the device and can fail
 * late), and plugins inside a process whose device memory is owned by another
 * component's pool.  The entry point allocates and frees nothing.
 *   - A problem whose workspace query exceeds the built-in size is refused with
 *     MLUOP_STATUS_NOT_SUPPORTED and a log line naming both sizes (with 3x3x3
 *     kernels and 64 channels that is about 300,000 output rows).
 *   - Every GPU on which the process loads the library holds the array from
 *     load until exit, used or not.
 *   - The first call on each device looks the array's device address up
 *     (cudaGetSymbolAddress, with that device current); make that first call
 *     outside any stream capture.
 *   - All calls on a device share the one array, which still holds what the
 *     previous call left there; the call itself resets what it needs reset.
 *     Two such calls whose GPU work overlaps (different streams or threads) race
 *     on it: serialise them. */
#define MLUOP_BUILTIN_CONV_WORKSPACE_BYTES (32u << 20)
mluOpStatus_t MLUOP_WIN_API mluOpIndiceConvolutionForwardBuiltinWorkspace(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc, const void *features,
    const mluOpTensorDescriptor_t filters_desc, const void *filters,
    const mluOpTensorDescriptor_t indice_pairs_desc, const void *indice_pairs,
    const int64_t indice_num[], const int64_t num_act_out, const int64_t inverse,
    const int64_t sub_m, const mluOpTensorDescriptor_t features_out_desc, void *features_out);

#if defined(__cplusplus)
}
#endif

#endif /* MLUOP_B200_MLU_OP_H_ */
