// Version, error reporting and the device status word of the C ABI (include/nf4ll.h).
#include <cstdarg>
#include <cstdio>

#include "nf4ll_common.cuh"

namespace nf4ll {

static thread_local char g_detail[512] = "";
static thread_local int64_t g_launches = 0;

void count_launch() { ++g_launches; }

void set_detail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_detail, sizeof(g_detail), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t err, const char* what) {
  set_detail("%s: %s", what, cudaGetErrorString(err));
  return NF4LL_ERR_CUDA;
}

int require_sm100() {
  int dev = 0, major = 0;
  NF4LL_CUDA(cudaGetDevice(&dev));
  NF4LL_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) {
    set_detail("device %d has compute capability %d.x; this library is built for sm_100a only", dev, major);
    return NF4LL_ERR_ARCH;
  }
  return NF4LL_OK;
}

}  // namespace nf4ll

extern "C" int nf4ll_version(void) { return NF4LL_VERSION; }

extern "C" const char* nf4ll_error_string(int code) {
  switch (code) {
    case NF4LL_OK: return "ok";
    case NF4LL_ERR_NULL: return "required pointer is null";
    case NF4LL_ERR_SHAPE: return "unsupported shape";
    case NF4LL_ERR_ALIGN: return "misaligned pointer or leading dimension";
    case NF4LL_ERR_RANK: return "unsupported LoRA rank (only 16)";
    case NF4LL_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case NF4LL_ERR_ARCH: return "device is not sm_100";
    case NF4LL_ERR_CUDA: return "CUDA call failed";
    case NF4LL_ERR_DEVICE_WAIT: return "a bounded wait inside a kernel expired";
    default: return "unknown nf4ll status";
  }
}

extern "C" const char* nf4ll_last_error_detail(void) { return nf4ll::g_detail; }

extern "C" int64_t nf4ll_launch_count(void) { return nf4ll::g_launches; }

extern "C" int nf4ll_read_status(const int32_t* status, void* stream) {
  using namespace nf4ll;
  if (!status) {
    set_detail("nf4ll_read_status: null status pointer");
    return NF4LL_ERR_NULL;
  }
  int32_t word = 0;
  NF4LL_CUDA(cudaMemcpyAsync(&word, status, sizeof(word), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  NF4LL_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  if (word != 0) {
    set_detail("device status word 0x%08x (role %d, site %d)", static_cast<unsigned>(word), (word >> 8) & 0xff, word & 0xff);
    return NF4LL_ERR_DEVICE_WAIT;
  }
  return NF4LL_OK;
}
