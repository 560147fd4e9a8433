// Handle life cycle (reference core/context.cpp:158-307 mluOpCreate, :354
// mluOpDestroy, :362 mluOpSetQueue, :372 mluOpGetQueue, :382 mluOpGetDevice,
// :462 mluOpGetLibVersion, atomics mode).
#include "core/context.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include "core/logging.h"

namespace mluop {

bool checkStatusRequested() {
  const char *check = std::getenv("MLUOP_B200_CHECK_STATUS");
  return check && check[0] == '1';
}

bool takeStickyDeviceError(mluOpHandle_t handle, const char *api) {
  if (handle == nullptr || handle->host_words == nullptr) return false;
  volatile int32_t *word = handle->host_words + mluOpContext::kStickyWord;
  const int32_t bits = *word;
  if (bits == 0) return false;
  *word = 0;
  LOG(ERROR) << api << " an earlier asynchronous call on this handle reported device error bits " << bits
             << " (1: hash table full, 4: look-back wait gave up, 0x100 and up: a bounded wait of the "
             << "convolution kernel gave up); its outputs are not valid.";
  return true;
}

}  // namespace mluop

extern "C" {

mluOpStatus_t MLUOP_WIN_API mluOpCreate(mluOpHandle_t *handle) {
  PARAM_CHECK("[mluOpCreate]", handle != NULL);
  mluOpContext *ctx = new (std::nothrow) mluOpContext();
  if (ctx == nullptr) return MLUOP_STATUS_ALLOC_FAILED;

  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) {
    (void)cudaGetLastError();
    // Without a usable device the library cannot compute anything.  A
    // host-only handle can still be asked for explicitly: it runs the
    // argument checks of every entry point (which all precede the first
    // launch) and fails with MLUOP_STATUS_EXECUTION_FAILED at the first launch.
    const char *host_only = std::getenv("MLUOP_B200_HOST_ONLY_HANDLE");
    if (host_only && std::strcmp(host_only, "1") == 0) {
      ctx->host_only = true;
      ctx->arch = MLUOP_B200;
      std::snprintf(ctx->device_name, CONTEXT_DEVICENAME_BUFFER_SIZE, "%s", "host-only");
      ctx->host_words = new int32_t[mluOpContext::kHostWords]();
      *handle = ctx;
      return MLUOP_STATUS_SUCCESS;
    }
    LOG(ERROR) << "[mluOpCreate] no usable CUDA device: " << cudaGetErrorString(err);
    delete ctx;
    return MLUOP_STATUS_NOT_INITIALIZED;
  }
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    LOG(ERROR) << "[mluOpCreate] An internal error occured. cudaGetDeviceProperties";
    delete ctx;
    return MLUOP_STATUS_INTERNAL_ERROR;
  }
  ctx->device = dev;
  ctx->arch = (prop.major == 10) ? MLUOP_B200 : MLUOP_UNKNOWN_DEVICE;
  std::snprintf(ctx->device_name, CONTEXT_DEVICENAME_BUFFER_SIZE, "%.63s", prop.name);
  ctx->sm_count = prop.multiProcessorCount;
  ctx->max_smem_per_block = (int32_t)prop.sharedMemPerBlockOptin;
  ctx->l2cache_size = prop.l2CacheSize;
  int clock_khz = 0, mem_khz = 0, bus_bits = 0;
  cudaDeviceGetAttribute(&clock_khz, cudaDevAttrClockRate, dev);
  cudaDeviceGetAttribute(&mem_khz, cudaDevAttrMemoryClockRate, dev);
  cudaDeviceGetAttribute(&bus_bits, cudaDevAttrGlobalMemoryBusWidth, dev);
  (void)cudaGetLastError();
  ctx->clock_rate = clock_khz;
  ctx->memory_band_width = 2.0 * mem_khz * 1e3 * (bus_bits / 8.0) / 1e9;
  if (cudaHostAlloc((void **)&ctx->host_words, sizeof(int32_t) * mluOpContext::kHostWords,
                    cudaHostAllocMapped) != cudaSuccess) {
    (void)cudaGetLastError();
    LOG(ERROR) << "[mluOpCreate] pinned host allocation failed.";
    delete ctx;
    return MLUOP_STATUS_ALLOC_FAILED;
  }
  std::memset(ctx->host_words, 0, sizeof(int32_t) * mluOpContext::kHostWords);
  *handle = ctx;
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpDestroy(mluOpHandle_t handle) {
  PARAM_CHECK("[mluOpDestroy]", handle != NULL);
  // an error of the last asynchronous call would otherwise never be reported
  const bool pending_error = mluop::takeStickyDeviceError(handle, "[mluOpDestroy]");
  if (handle->host_words) {
    if (handle->host_only) {
      delete[] handle->host_words;
    } else {
      cudaFreeHost(handle->host_words);
      (void)cudaGetLastError();
    }
  }
  delete handle;
  return pending_error ? MLUOP_STATUS_EXECUTION_FAILED : MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpSetQueue(mluOpHandle_t handle, cnrtQueue_t queue) {
  PARAM_CHECK("[mluOpSetQueue]", handle != NULL);
  handle->queue = queue;  // NULL selects the default stream
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpGetQueue(mluOpHandle_t handle, cnrtQueue_t *queue) {
  PARAM_CHECK("[mluOpGetQueue]", handle != NULL);
  PARAM_CHECK("[mluOpGetQueue]", queue != NULL);
  *queue = handle->queue;
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpGetDevice(mluOpHandle_t handle, CNdev *device) {
  PARAM_CHECK("[mluOpGetDevice]", handle != NULL);
  PARAM_CHECK("[mluOpGetDevice]", device != NULL);
  *device = handle->device;
  return MLUOP_STATUS_SUCCESS;
}

void MLUOP_WIN_API mluOpGetLibVersion(int *major, int *minor, int *patch) {
  if (major) *major = MLUOP_MAJOR;
  if (minor) *minor = MLUOP_MINOR;
  if (patch) *patch = MLUOP_PATCHLEVEL;
}

mluOpStatus_t MLUOP_WIN_API mluOpSetAtomicsMode(mluOpHandle_t handle, mluOpAtomicsMode_t atomics_mode) {
  PARAM_CHECK("[mluOpSetAtomicsMode]", handle != NULL);
  PARAM_CHECK("[mluOpSetAtomicsMode]",
              atomics_mode == MLUOP_ATOMICS_ALLOWED || atomics_mode == MLUOP_ATOMICS_NOT_ALLOWED);
  handle->atomics_mode = atomics_mode;
  return MLUOP_STATUS_SUCCESS;
}

mluOpStatus_t MLUOP_WIN_API mluOpGetAtomicsMode(mluOpHandle_t handle, mluOpAtomicsMode_t *atomics_mode) {
  PARAM_CHECK("[mluOpGetAtomicsMode]", handle != NULL);
  PARAM_CHECK("[mluOpGetAtomicsMode]", atomics_mode != NULL);
  *atomics_mode = handle->atomics_mode;
  return MLUOP_STATUS_SUCCESS;
}

}  // extern "C"
