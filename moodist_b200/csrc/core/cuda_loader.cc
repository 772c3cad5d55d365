#include "cuda_loader.h"

#include <dlfcn.h>

#include <mutex>

#include "log.h"

namespace moodist {

#define MOODIST_STR2(x) #x
#define MOODIST_STR(x) MOODIST_STR2(x)

static CudaApi g_cuda;
static NvmlApi g_nvml;

const CudaApi& cuda() {
  static std::once_flag once;
  std::call_once(once, [] {
    void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) lib = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) {
      g_cuda.error = std::string("cannot load libcuda.so.1: ") + (dlerror() ?: "?");
      return;
    }
    bool ok = true;
    // MOODIST_STR expands the toolkit's versioning macros, so e.g. cuMemGetInfo resolves cuMemGetInfo_v2
#define X(name)                                                             \
  g_cuda.name = reinterpret_cast<decltype(g_cuda.name)>(dlsym(lib, MOODIST_STR(name))); \
  if (!g_cuda.name) {                                                       \
    ok = false;                                                             \
    g_cuda.error += std::string(" missing ") + MOODIST_STR(name);           \
  }
    MOODIST_CU_FUNCS(X)
#undef X
    if (!ok) return;
    CUresult r = g_cuda.cuInit(0);
    if (r != CUDA_SUCCESS) {
      g_cuda.error = "cuInit failed: " + std::to_string((int)r);
      return;
    }
    g_cuda.loaded = true;
  });
  return g_cuda;
}

const CudaApi& cuda_required() {
  const CudaApi& c = cuda();
  if (!c.loaded) fail("CUDA driver is not available: " + c.error);
  return c;
}

std::string cu_error_string(CUresult r) {
  const char* s = nullptr;
  if (g_cuda.cuGetErrorString && g_cuda.cuGetErrorString(r, &s) == CUDA_SUCCESS && s) return s;
  return "CUDA error " + std::to_string((int)r);
}

void cu_check(CUresult r, const char* what) {
  if (r != CUDA_SUCCESS) fail(std::string(what) + " failed: " + cu_error_string(r));
}

const NvmlApi& nvml() {
  static std::once_flag once;
  std::call_once(once, [] {
    void* lib = dlopen("libnvidia-ml.so.1", RTLD_NOW);
    if (!lib) return;
#define N(name) g_nvml.name = reinterpret_cast<decltype(g_nvml.name)>(dlsym(lib, #name));
    N(nvmlInit_v2)
    N(nvmlShutdown)
    N(nvmlDeviceGetHandleByPciBusId_v2)
    N(nvmlDeviceGetHandleByIndex_v2)
    N(nvmlDeviceGetP2PStatus)
    N(nvmlDeviceGetNvLinkState)
    N(nvmlDeviceGetNvLinkRemotePciInfo_v2)
    N(nvmlDeviceGetNumaNodeId)
    N(nvmlDeviceGetCount_v2)
    N(nvmlDeviceGetPciInfo_v3)
#undef N
    if (g_nvml.nvmlInit_v2 && g_nvml.nvmlInit_v2() == 0) g_nvml.loaded = true;
  });
  return g_nvml;
}

}  // namespace moodist
