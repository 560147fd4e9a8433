// Library handle: one CUDA device, one stream, and the device facts kernels
// size their launches by (reference core/context.h:53-147, with the MLU
// cluster/NRAM fields replaced by their CUDA counterparts).
#ifndef MLUOP_B200_CORE_CONTEXT_H_
#define MLUOP_B200_CORE_CONTEXT_H_

#include <cuda_runtime_api.h>

#include <cstdint>

#include "mlu_op.h"

#define CONTEXT_DEVICENAME_BUFFER_SIZE 64

// handle->arch.  The reference's values are kept so that code comparing
// against them still compiles; MLUOP_UNKNOWN_DEVICE stays the wildcard.  Any
// GPU that is not compute capability 10.x reports MLUOP_UNKNOWN_DEVICE and is
// refused by the operators with MLUOP_STATUS_ARCH_MISMATCH.
typedef enum {
  MLUOP_UNKNOWN_DEVICE = 0,
  MLUOP_MLU220 = 220,
  MLUOP_MLU270 = 270,
  MLUOP_MLU290 = 290,
  MLUOP_MLU370 = 372,
  MLUOP_MLU590 = 592,
  MLUOP_MTP613 = 613,
  MLUOP_MTP617 = 617,
  MLUOP_B200 = 1000,
} mluOpDevType_t;

struct mluOpContext {
  CNdev device = -1;             // CUDA device ordinal; -1 for a host-only handle
  cnrtQueue_t queue = nullptr;   // cudaStream_t work is enqueued on
  mluOpDevType_t arch = MLUOP_UNKNOWN_DEVICE;
  char device_name[CONTEXT_DEVICENAME_BUFFER_SIZE] = "";
  int32_t sm_count = 0;              // streaming multiprocessors
  int32_t max_smem_per_block = 0;    // opt-in shared memory per block, bytes
  int32_t l2cache_size = 0;          // bytes
  int32_t clock_rate = 0;            // kHz
  double memory_band_width = 0;      // GB/s, from memory clock and bus width
  mluOpAtomicsMode_t atomics_mode = MLUOP_ATOMICS_NOT_ALLOWED;
  // Pinned, device-mapped host words that kernels store results into when the
  // host must read them ([0] error bits and [1] active-output count of the last
  // rulebook), and [kStickyWord]: error bits of asynchronous calls, which a
  // kernel's error path (a full hash table, a bounded wait that gave up) ORs
  // in and the next entry point on this handle reports and clears.
  int32_t *host_words = nullptr;
  static constexpr int kHostWords = 16;
  static constexpr int kStickyWord = 2;
  bool host_only = false;  // created without a device: argument checks only
};

namespace mluop {

// True when MLUOP_B200_CHECK_STATUS=1: entry points then wait for their work and
// report device error bits themselves (debugging and tests).
bool checkStatusRequested();

// Asynchronous entry points cannot report a device-side error of their own
// launch.  Such an error is recorded in the handle's sticky word; the next entry
// point called on the handle calls this, which logs the bits, clears the word
// and returns true (the caller returns MLUOP_STATUS_EXECUTION_FAILED).  No
// synchronisation: only errors that have already reached the host are seen.
bool takeStickyDeviceError(mluOpHandle_t handle, const char *api);

}  // namespace mluop

#endif  // MLUOP_B200_CORE_CONTEXT_H_
