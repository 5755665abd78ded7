// Host-side helpers shared by the C-ABI translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "../../include/exl3_b200.h"

namespace exl3 {

inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// integer K in 1..8 from k_times_2, or 0 if unsupported
inline int integer_k(int k_times_2) {
    if (k_times_2 < 2 || k_times_2 > 16 || (k_times_2 & 1)) return 0;
    return k_times_2 >> 1;
}

// Launch with programmatic stream serialization: the grid may be scheduled while its predecessor on
// the stream is still running; the kernel itself waits (griddepcontrol.wait) before it touches
// anything the predecessor produces.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? EXL3_OK : EXL3_E_LAUNCH; }

}  // namespace exl3
