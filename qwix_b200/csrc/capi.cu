// Version and status strings of the C ABI.
#include <atomic>

#include "common.cuh"

namespace qwx {
namespace {
std::atomic<int> g_programmatic_launch{0};
}
bool programmatic_launch_enabled() { return g_programmatic_launch.load(std::memory_order_relaxed) != 0; }
}  // namespace qwx

extern "C" void qwx_set_programmatic_launch(int enabled) {
  qwx::g_programmatic_launch.store(enabled ? 1 : 0, std::memory_order_relaxed);
}
extern "C" int qwx_get_programmatic_launch(void) { return qwx::programmatic_launch_enabled() ? 1 : 0; }

extern "C" int qwx_version(void) { return 100; }

extern "C" const char* qwx_status_string(int status) {
  switch (status) {
    case QWX_OK: return "ok";
    case QWX_ERR_NULL: return "a required pointer is NULL";
    case QWX_ERR_SHAPE: return "inconsistent shape, tile or option";
    case QWX_ERR_ALIGN: return "pointer or row pitch is not 16-byte aligned";
    case QWX_ERR_DTYPE: return "unsupported dtype combination";
    case QWX_ERR_UNSUPPORTED: return "valid request that this build does not implement";
    case QWX_ERR_WORKSPACE: return "workspace missing or too small";
    case QWX_ERR_LAUNCH: return "CUDA launch or driver call failed";
    case QWX_ERR_DEVICE_WAIT: return "a bounded device-side wait ran out";
    case QWX_ERR_NO_DEVICE: return "no usable sm_100 device or driver entry point";
    default: return "unknown status";
  }
}
