/*
 * mlu_op_trace.h -- per-kernel timing of the library's own launches.
 *
 * Counterpart of the reference's kernel tracing, which is switched on by the
 * environment variables MLUOP_TRACE_ENABLE_KERNEL / MLUOP_TRACE_DATA_DIR and
 * writes mlu_op_kernel.csv (reference core/mlu_op_trace.cpp:42-100,
 * core/kernel_tracing.cpp:321-356).  The same two variables work here; the
 * three functions below give a running process the same data without a file.
 *
 * When tracing is on, every kernel, memset and copy the library enqueues is
 * bracketed by two CUDA events on the launching stream.  Nothing is measured
 * while tracing is off (the default).
 */
#ifndef MLUOP_B200_MLU_OP_TRACE_H_
#define MLUOP_B200_MLU_OP_TRACE_H_

#include "mlu_op.h"

#if defined(__cplusplus)
extern "C" {
#endif

/* Replaces the reference's MLUOP_TRACE_ENABLE_KERNEL switch
 * (core/mlu_op_trace.cpp:52-100) for callers that cannot set the environment
 * before the library loads.  enable != 0 starts recording, 0 stops it. */
mluOpStatus_t MLUOP_WIN_API mluOpTraceKernelEnable(int enable);

/* Drops everything recorded so far. */
mluOpStatus_t MLUOP_WIN_API mluOpTraceKernelReset(void);

/* Waits for the recorded events and writes one CSV line per distinct name,
 * in first-launch order, with the header
 *   name,launches,total_ms,algorithmic_bytes,flops
 * (the columns of the reference's mlu_op_kernel.csv that apply, plus the
 * algorithmic bytes and flops the launch site states for the launch).  Names
 * starting with "memset:" or "memcpy:" are runtime operations, the rest are
 * kernels of this library.  The text is NUL terminated and truncated to
 * buffer_size; *needed (optional) receives the full length including the NUL.
 * The records are cleared once a call's buffer held the whole text: a call whose
 * buffer was too small (a size query) keeps it for the next call. */
mluOpStatus_t MLUOP_WIN_API mluOpTraceKernelReport(char *buffer, size_t buffer_size, size_t *needed);

#if defined(__cplusplus)
}
#endif

#endif /* MLUOP_B200_MLU_OP_TRACE_H_ */
