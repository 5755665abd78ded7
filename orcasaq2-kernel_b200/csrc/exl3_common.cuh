// Host-side helpers shared by the C-ABI translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/exl3_b200.h"

namespace exl3 {

inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// integer K in 1..8 from k_times_2, or 0 if unsupported
inline int integer_k(int k_times_2) {
    if (k_times_2 < 2 || k_times_2 > 16 || (k_times_2 & 1)) return 0;
    return k_times_2 >> 1;
}

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? EXL3_OK : EXL3_E_LAUNCH; }

}  // namespace exl3
