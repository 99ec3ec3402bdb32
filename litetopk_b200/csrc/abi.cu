// ABI-level helpers of liblitedsa_b200.so: version, error strings.
#include "common.cuh"

extern "C" int litedsa_abi_version(void) { return 1; }

extern "C" const char* litedsa_error_string(int code) {
  switch (code) {
    case LITEDSA_OK: return "ok";
    case LITEDSA_ERR_ARG: return "bad argument (null pointer or inconsistent optional arguments)";
    case LITEDSA_ERR_SHAPE: return "shape rule of the operator violated";
    case LITEDSA_ERR_UNSUPPORTED: return "configuration not supported by this build";
    case LITEDSA_ERR_CUDA: return "CUDA runtime or driver call failed";
    case LITEDSA_ERR_TIMEOUT: return "device-side bounded wait expired";
    default: return "unknown litedsa error code";
  }
}
