// ABI version and error strings of the C interface.
#include "exl3_common.cuh"

extern "C" int exl3_abi_version(void) { return EXL3_ABI_VERSION; }

extern "C" const char *exl3_strerror(int code) {
    switch (code) {
        case EXL3_OK: return "ok";
        case EXL3_E_SHAPE: return "bad shape: a dimension, row count or packed size is not allowed";
        case EXL3_E_ALIGN: return "misaligned pointer or leading dimension";
        case EXL3_E_UNSUPPORTED: return "unsupported bitrate, codebook flag or mode";
        case EXL3_E_LAUNCH: return "CUDA launch failed";
        case EXL3_E_WORKSPACE: return "workspace missing or too small";
        case EXL3_E_NULL: return "required pointer is NULL";
        case EXL3_E_DEVICE: return "a tensor does not live on the current device";
    }
    return "unknown error";
}
