// mluOpIndiceConvolutionForwardBuiltinWorkspace: the sparse convolution for
// callers that have no way to hand the library a scratch buffer.
//
// Some hosts of this library cannot allocate device memory at the point where
// they call it: an inference loop that forbids allocator calls once it is
// running (cudaMalloc synchronises the device and may fail or fragment), or a
// plugin inside a process whose whole device memory belongs to another
// component's pool and that is only given the tensors it operates on.  For them
// the scratch lives inside the library: a fixed array in device memory that is
// part of the loaded module.  Every GPU the process uses with this library
// holds these kBuiltinWorkspaceBytes from module load until exit, whether or
// not this entry point is ever called.
//
// The entry point allocates and frees nothing, on the device or through any
// library.  It sizes the request with the ordinary workspace query, refuses
// requests that do not fit, and forwards to mluOpIndiceConvolutionForward with
// the array as the workspace, so results are those of the ordinary entry point.
#include <cuda_runtime.h>

#include <mutex>

#include "core/context.h"
#include "core/logging.h"
#include "mlu_op.h"

namespace {

constexpr size_t kBuiltinWorkspaceBytes = MLUOP_BUILTIN_CONV_WORKSPACE_BYTES;

// In host code this name is only a handle for the runtime's symbol table, not a
// device address; the address is looked up per device below.
static __device__ __align__(256) unsigned char g_builtin_conv_workspace[kBuiltinWorkspaceBytes];

constexpr int kMaxDevices = 64;
std::mutex g_lock;
void *g_address[kMaxDevices] = {};

// Device address of the array on the handle's device, looked up once per device
// with that device current.  The address is keyed by the handle's device, not by
// whatever device the calling thread has current: a caller whose current device
// differs from the handle's must still get the array of the GPU its stream runs on.
mluOpStatus_t builtinWorkspaceAddress(const char *api, int device, void **out) {
  if (device < 0 || device >= kMaxDevices) {
    LOG(ERROR) << api << " the handle's device ordinal " << device << " is out of range.";
    return MLUOP_STATUS_EXECUTION_FAILED;
  }
  std::lock_guard<std::mutex> guard(g_lock);
  if (g_address[device] == nullptr) {
    int current = -1;
    cudaError_t err = cudaGetDevice(&current);
    if (err == cudaSuccess && current != device) err = cudaSetDevice(device);
    void *ptr = nullptr;
    if (err == cudaSuccess) err = cudaGetSymbolAddress(&ptr, g_builtin_conv_workspace);
    if (current >= 0 && current != device) (void)cudaSetDevice(current);
    if (err != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();
      LOG(ERROR) << api << " cudaGetSymbolAddress failed on device " << device << ": " << cudaGetErrorString(err);
      return MLUOP_STATUS_EXECUTION_FAILED;
    }
    g_address[device] = ptr;
  }
  *out = g_address[device];
  return MLUOP_STATUS_SUCCESS;
}

}  // namespace

extern "C" {

mluOpStatus_t MLUOP_WIN_API mluOpIndiceConvolutionForwardBuiltinWorkspace(
    mluOpHandle_t handle, const mluOpTensorDescriptor_t features_desc, const void *features,
    const mluOpTensorDescriptor_t filters_desc, const void *filters,
    const mluOpTensorDescriptor_t indice_pairs_desc, const void *indice_pairs, const int64_t indice_num[],
    const int64_t num_act_out, const int64_t inverse, const int64_t sub_m,
    const mluOpTensorDescriptor_t features_out_desc, void *features_out) {
  const char *api = "[mluOpIndiceConvolutionForwardBuiltinWorkspace]";
  size_t needed = 0;
  mluOpStatus_t st = mluOpGetIndiceConvolutionForwardWorkspaceSize(handle, features_desc, filters_desc,
                                                                   indice_pairs_desc, features_out_desc,
                                                                   indice_num, num_act_out, inverse, sub_m, &needed);
  if (st != MLUOP_STATUS_SUCCESS) return st;
  if (needed > kBuiltinWorkspaceBytes) {
    LOG(ERROR) << api << " this problem needs " << needed << " bytes of scratch but the built-in workspace holds "
               << kBuiltinWorkspaceBytes << " bytes; use mluOpIndiceConvolutionForward with a caller-provided "
               << "workspace, or fewer output rows per call.";
    return MLUOP_STATUS_NOT_SUPPORTED;
  }
  void *workspace = nullptr;
  size_t workspace_size = 0;
  if (needed > 0 && !(handle != nullptr && handle->host_only)) {
    st = builtinWorkspaceAddress(api, handle->device, &workspace);
    if (st != MLUOP_STATUS_SUCCESS) return st;
    workspace_size = kBuiltinWorkspaceBytes;
  } else if (needed > 0) {
    // a handle without a device: let the ordinary entry point report it
    workspace = reinterpret_cast<void *>(256);
    workspace_size = kBuiltinWorkspaceBytes;
  }
  return mluOpIndiceConvolutionForward(handle, features_desc, features, filters_desc, filters, indice_pairs_desc,
                                       indice_pairs, indice_num, num_act_out, inverse, sub_m, workspace,
                                       workspace_size, features_out_desc, features_out);
}

}  // extern "C"
