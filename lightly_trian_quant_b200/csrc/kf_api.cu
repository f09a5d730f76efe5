// Status plumbing of the C-ABI: thread-local last-error text, CUDA error mapping, version, scale-tensor sizes.
#include <cstdarg>
#include <cstdio>

#include "kf_common.cuh"

namespace kf {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_status(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return KF_OK;
  set_error("%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
  return (int)e;
}

}  // namespace kf

extern "C" const char* kf_version(void) { return "kf_b200 0.1 sm_100a"; }

extern "C" const char* kf_last_error_string(void) { return kf::g_err; }

extern "C" int64_t kf_sf_bytes(int64_t R, int64_t K, int fmt) {
  if (R < 0 || K <= 0 || (fmt != KF_FMT_MX8 && fmt != KF_FMT_NV4 && fmt != KF_FMT_MX4)) {
    kf::set_error("kf_sf_bytes: bad argument R=%lld K=%lld fmt=%d", (long long)R, (long long)K, fmt);
    return KF_ERR_BAD_ARGUMENT;
  }
  int64_t nkb = K / kf::fmt_vec(fmt);
  return ((R + 127) / 128) * ((nkb + 3) / 4) * 512;
}
