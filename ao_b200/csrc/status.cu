// Status strings and ABI version of the C interface.
#include "common.cuh"

extern "C" const char* ao_status_string(int status) {
    switch (status) {
        case AO_OK: return "ok";
        case AO_ERR_SHAPE: return "shape or divisibility requirement not met";
        case AO_ERR_ALIGN: return "pointer not aligned as required";
        case AO_ERR_DTYPE: return "unsupported dtype or dtype combination";
        case AO_ERR_LAUNCH: return "CUDA launch failed";
        case AO_ERR_TIMEOUT: return "bounded device-side wait ran out";
        case AO_ERR_UNSUPPORTED: return "no kernel for this configuration";
        case AO_ERR_WORKSPACE: return "workspace missing or too small";
        case AO_ERR_ARG: return "invalid argument";
    }
    return "unknown status";
}

extern "C" int ao_abi_version(void) { return 1; }
