#include <stdlib.h>
// Library-level entry points: error strings, ABI version, last rejected CUDA launch.
#include "rd_common.cuh"

static thread_local int g_last_cuda_error = 0;

int rd_pdl_enabled() {
  static int enabled = [] {
    const char* v = getenv("RD_PDL");
    return (v && v[0] == '0') ? 0 : 1;
  }();
  return enabled;
}

void rd_set_last_cuda_error(int e) {
  g_last_cuda_error = e;
  (void)cudaGetLastError();  // clear the sticky-free launch error so later calls start clean
}

extern "C" int rd_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" int rd_abi_version(void) { return 1; }

extern "C" const char* rd_strerror(int code) {
  switch (code) {
    case RD_OK: return "ok";
    case RD_ERR_ARG: return "invalid argument (null pointer or inconsistent option)";
    case RD_ERR_DTYPE: return "unsupported dtype";
    case RD_ERR_SIZE: return "size outside the supported range";
    case RD_ERR_LAUNCH: return "CUDA launch rejected (see rd_last_cuda_error)";
    case RD_ERR_ALIGN: return "pointer or leading dimension misaligned";
    case RD_ERR_UNSUPPORTED: return "combination not implemented";
    case RD_ERR_CAPACITY: return "request exceeds the fixed capacity of this entry point (it cannot allocate)";
    default: return "unknown error code";
  }
}
