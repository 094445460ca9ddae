// CUDA driver API reached through dlopen("libcuda.so.1"): the native library links against no CUDA
// library, so it imports on machines without a GPU (verifier, pool, fake-device backend) and binds
// the driver only when a device is first used.
// (The reference binds the driver the same way: examples/cpp/cuda_api.hpp, and cudarc's dynamic
// loading behind crates/kern-runtime.)
#pragma once
#include <cuda.h>
#include <dlfcn.h>

#include <mutex>
#include <stdexcept>
#include <string>

namespace kern {

#define KERN_STR_(x) #x
#define KERN_STR(x) KERN_STR_(x)

// name, as spelled in cuda.h (macros there map some names to their _v2/_v3 symbols)
#define KERN_CUDA_FUNCS(X)          \
  X(cuInit)                         \
  X(cuGetErrorString)               \
  X(cuDriverGetVersion)             \
  X(cuDeviceGet)                    \
  X(cuDeviceGetCount)               \
  X(cuDeviceGetAttribute)           \
  X(cuDeviceGetName)                \
  X(cuDeviceTotalMem)               \
  X(cuDevicePrimaryCtxRetain)       \
  X(cuDevicePrimaryCtxRelease)      \
  X(cuCtxSetCurrent)                \
  X(cuCtxGetCurrent)                \
  X(cuCtxSynchronize)               \
  X(cuModuleLoadData)               \
  X(cuModuleUnload)                 \
  X(cuModuleGetFunction)            \
  X(cuModuleGetGlobal)              \
  X(cuModuleGetFunctionCount)       \
  X(cuModuleEnumerateFunctions)     \
  X(cuFuncGetName)                  \
  X(cuFuncGetParamInfo)             \
  X(cuFuncSetAttribute)             \
  X(cuFuncGetAttribute)             \
  X(cuLaunchKernelEx)               \
  X(cuMemAlloc)                     \
  X(cuMemFree)                      \
  X(cuMemGetInfo)                   \
  X(cuMemsetD8Async)                \
  X(cuMemsetD32Async)               \
  X(cuMemcpyHtoDAsync)              \
  X(cuMemcpyDtoHAsync)              \
  X(cuMemcpyDtoDAsync)              \
  X(cuMemcpy2DAsync)                \
  X(cuMemHostAlloc)                 \
  X(cuMemFreeHost)                  \
  X(cuMemHostRegister)              \
  X(cuMemHostUnregister)            \
  X(cuStreamCreate)                 \
  X(cuStreamDestroy)                \
  X(cuStreamSynchronize)            \
  X(cuStreamWaitEvent)              \
  X(cuStreamBeginCapture)           \
  X(cuStreamEndCapture)             \
  X(cuStreamIsCapturing)            \
  X(cuEventCreate)                  \
  X(cuEventDestroy)                 \
  X(cuEventRecord)                  \
  X(cuEventSynchronize)             \
  X(cuEventQuery)                   \
  X(cuEventElapsedTime)             \
  X(cuGraphInstantiateWithFlags)    \
  X(cuGraphLaunch)                  \
  X(cuGraphDestroy)                 \
  X(cuGraphExecDestroy)             \
  X(cuGraphGetNodes)                \
  X(cuTensorMapEncodeTiled)         \
  X(cuIpcGetMemHandle)              \
  X(cuIpcOpenMemHandle)             \
  X(cuIpcCloseMemHandle)            \
  X(cuDeviceCanAccessPeer)          \
  X(cuCtxEnablePeerAccess)

struct Cuda {
#define X(name) decltype(&::name) name##_ = nullptr;
  KERN_CUDA_FUNCS(X)
#undef X
  void* lib = nullptr;

  static Cuda& get() {
    static Cuda api;
    static std::once_flag once;
    std::call_once(once, [] { api.open(); });
    if (!api.lib) throw std::runtime_error("CUDA driver (libcuda.so.1) is not available on this machine");
    return api;
  }
  static bool available() {
    try {
      get();
      return true;
    } catch (...) {
      return false;
    }
  }

 private:
  void open() {
    lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) return;
#define X(name)                                                                  \
  name##_ = reinterpret_cast<decltype(&::name)>(dlsym(lib, KERN_STR(name)));
    KERN_CUDA_FUNCS(X)
#undef X
    if (!cuInit_ || cuInit_(0) != CUDA_SUCCESS) {
      lib = nullptr;
    }
  }
};

inline void cu_check(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return;
  const char* msg = nullptr;
  auto& c = Cuda::get();
  if (c.cuGetErrorString_) c.cuGetErrorString_(r, &msg);
  throw std::runtime_error(std::string(what) + ": CUDA error " + std::to_string((int)r) + " (" +
                           (msg ? msg : "?") + ")");
}
#define KERN_CU(call) ::kern::cu_check(::kern::Cuda::get().call, #call)

}  // namespace kern
