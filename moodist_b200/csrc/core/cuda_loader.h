// Lazily loaded CUDA driver and NVML entry points.
//
// The library must import and run CPU collectives on machines with no GPU and no libcuda, so nothing
// links against the driver: the first CUDA-side call dlopen()s libcuda.so.1 (and libnvidia-ml.so.1
// for topology) and resolves the functions below. The reference does the same with its own type
// declarations (core/cuda_loader.cc:34-230); here the CUDA toolkit headers supply the types and the
// versioned symbol names.
#pragma once

#include <cuda.h>

#include <string>

namespace moodist {

#define MOODIST_CU_FUNCS(X)           \
  X(cuInit)                           \
  X(cuGetErrorString)                 \
  X(cuDriverGetVersion)               \
  X(cuDeviceGet)                      \
  X(cuDeviceGetCount)                 \
  X(cuDeviceGetAttribute)             \
  X(cuDeviceGetPCIBusId)              \
  X(cuDeviceCanAccessPeer)            \
  X(cuDevicePrimaryCtxRetain)         \
  X(cuDevicePrimaryCtxRelease)        \
  X(cuCtxGetCurrent)                  \
  X(cuCtxSetCurrent)                  \
  X(cuCtxGetDevice)                   \
  X(cuMemGetInfo)                     \
  X(cuMemAddressReserve)              \
  X(cuMemAddressFree)                 \
  X(cuMemCreate)                      \
  X(cuMemRelease)                     \
  X(cuMemMap)                         \
  X(cuMemUnmap)                       \
  X(cuMemSetAccess)                   \
  X(cuMemGetAllocationGranularity)    \
  X(cuMemExportToShareableHandle)     \
  X(cuMemImportFromShareableHandle)   \
  X(cuMulticastCreate)                \
  X(cuMulticastAddDevice)             \
  X(cuMulticastBindMem)               \
  X(cuMulticastUnbind)                \
  X(cuMulticastGetGranularity)        \
  X(cuMemsetD8)                       \
  X(cuMemsetD32Async)                 \
  X(cuMemcpyAsync)                    \
  X(cuMemcpyDtoH)                     \
  X(cuMemcpyHtoD)                     \
  X(cuMemHostRegister)                \
  X(cuMemHostUnregister)              \
  X(cuStreamSynchronize)              \
  X(cuStreamWriteValue32)             \
  X(cuStreamWaitValue32)              \
  X(cuLaunchHostFunc)                 \
  X(cuPointerGetAttribute)

struct CudaApi {
#define X(name) decltype(&::name) name = nullptr;
  MOODIST_CU_FUNCS(X)
#undef X
  bool loaded = false;
  std::string error;  // why loading failed
};

// Loads on first use. Returns an object with loaded == false (and `error` set) when no driver exists.
const CudaApi& cuda();
// Throws moodist::Error if the driver is unavailable.
const CudaApi& cuda_required();

std::string cu_error_string(CUresult r);
void cu_check(CUresult r, const char* what);

#define CU_CHECK(expr) ::moodist::cu_check((expr), #expr)

// ---- NVML (only what topology discovery needs; declared here so no NVML header is required) ----
struct NvmlApi {
  int (*nvmlInit_v2)() = nullptr;
  int (*nvmlShutdown)() = nullptr;
  int (*nvmlDeviceGetHandleByPciBusId_v2)(const char*, void**) = nullptr;
  int (*nvmlDeviceGetHandleByIndex_v2)(unsigned, void**) = nullptr;
  int (*nvmlDeviceGetP2PStatus)(void*, void*, int /*index*/, int* /*status*/) = nullptr;
  int (*nvmlDeviceGetNvLinkState)(void*, unsigned, int*) = nullptr;
  int (*nvmlDeviceGetNvLinkRemotePciInfo_v2)(void*, unsigned, void*) = nullptr;
  int (*nvmlDeviceGetNumaNodeId)(void*, unsigned*) = nullptr;
  int (*nvmlDeviceGetCount_v2)(unsigned*) = nullptr;
  int (*nvmlDeviceGetPciInfo_v3)(void*, void*) = nullptr;
  bool loaded = false;
};
const NvmlApi& nvml();

}  // namespace moodist
