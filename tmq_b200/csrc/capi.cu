// Status strings and ABI version of the tmq_b200 C interface.
#include "common.cuh"

extern "C" const char *tmq_status_string(int status) {
    switch (status) {
        case TMQ_OK: return "ok";
        case TMQ_ERR_ARG: return "invalid argument";
        case TMQ_ERR_ALIGN: return "pointer alignment";
        case TMQ_ERR_LAUNCH: return "CUDA launch failed";
        case TMQ_ERR_TIMEOUT: return "bounded device wait ran out";
        case TMQ_ERR_SCRATCH: return "scratch buffer too small";
        case TMQ_ERR_UNSUPPORTED: return "unsupported shape";
        default: return "unknown status";
    }
}

extern "C" int tmq_last_cuda_error(void) { return tmq::g_last_cuda_error; }

extern "C" int tmq_abi_version(void) { return 1; }
