// One-shot all-reduce of the row-parallel layers' partial outputs over peer memory (NVLink / NVSwitch).
//
// After a row-parallel projection every tensor-parallel rank holds a partial [rows][hidden] fp16 result; the
// reference plugin refuses tensor parallelism (orcasaq2/config.py:173-177) and the engine around it would sum the
// partials with a library all-reduce (vllm/model_executor/layers/linear.py:1556-1559).  At decode sizes (10 KB to
// 640 KB) that collective is pure latency, so this kernel does the whole exchange in one launch:
//
//   every rank owns a communication buffer that all ranks have mapped (CUDA IPC):
//       [status word][per-chunk generation counters (local use)][arrival flags: one per (source rank, chunk)]
//       [two data slots of `capacity` bytes]
//   a CTA handles one chunk of 4096 values end to end:
//     1. generation g = counter + 1; copy its chunk of the partial into data slot (g & 1) of the own buffer;
//     2. system-scope fence, then write g into flag (own rank, chunk) of EVERY rank's buffer (plain peer stores);
//     3. wait, with a bound, until the own buffer's flags of all source ranks show >= g;
//     4. read the chunk from every rank's slot (plain peer loads, own part from registers), add in fp32 in rank
//        order -- every rank computes bitwise the same sum -- round once, write the result (in place is fine);
//     5. counter = g.
//   Slot parity makes the data safe without a second handshake: a rank can overwrite slot (g & 1) only in
//   generation g + 2, which it cannot reach before every peer has signalled g + 1, i.e. finished reading g.
//
// Small messages (up to 32 Ki values) take a lower-latency form of the same exchange: instead of publishing the
// partial locally and letting the peers fetch it, every rank WRITES its partial into a region of every peer's
// buffer reserved for it, each 4-byte word paired with the generation number in one 8-byte store.  A receiver
// polls the words themselves until they carry the generation it expects, so no fence, no separate flag and no
// load across the link are needed: the exchange costs one store latency.  Sum order and slot parity as above.
//
// Nothing here uses multicast or TMA on peer memory.  A wait that runs out sets the status word, skips the
// chunk (the output keeps the partial) and returns; the generation counter is then left where it was.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "exl3_common.cuh"

namespace exl3 {

constexpr int kArChunk = 4096;                 // values per CTA
constexpr int kArThreads = 512;                // 8 values (16 bytes) per thread
constexpr int kArMaxChunks = 1024;             // 4 Mi values per call
constexpr size_t kArStatusBytes = 256;
constexpr size_t kArCounterBytes = (size_t)kArMaxChunks * 4;
constexpr size_t kArFlagBytes = (size_t)EXL3_AR_MAX_RANKS * kArMaxChunks * 4;
constexpr int kArLLMaxValues = 32768;          // messages up to this size take the word-with-flag form
constexpr size_t kArLLSrcBytes = (size_t)kArLLMaxValues * 4;                       // 8 bytes per 2 values
constexpr size_t kArLLBytes = 2 * (size_t)EXL3_AR_MAX_RANKS * kArLLSrcBytes;       // [slot][source rank]
constexpr size_t kArHeadBytes = kArStatusBytes + kArCounterBytes + kArFlagBytes + kArLLBytes;
constexpr size_t kArLLOffset = kArStatusBytes + kArCounterBytes + kArFlagBytes;

struct ArParams {
    unsigned char *peer[EXL3_AR_MAX_RANKS];    // every rank's communication buffer, own included
    const __half *in;
    __half *out;
    long long n;                               // values
    size_t capacity;                           // bytes of one data slot
    int rank, world, spin_limit;
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_peer_v4(const void *p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kArThreads) allreduce_oneshot_kernel(const __grid_constant__ ArParams P) {
    asm volatile("griddepcontrol.wait;" ::: "memory");      // the partial comes from the kernel before this one
    asm volatile("griddepcontrol.launch_dependents;");
    __shared__ unsigned s_ok;
    const int tid = threadIdx.x, chunk = blockIdx.x;
    unsigned char *mine = P.peer[P.rank];
    unsigned *status = reinterpret_cast<unsigned *>(mine);
    unsigned *counter = reinterpret_cast<unsigned *>(mine + kArStatusBytes) + chunk;
    const unsigned gen = *counter + 1u;
    const size_t slot_off = kArHeadBytes + (size_t)(gen & 1u) * P.capacity + (size_t)chunk * kArChunk * 2;
    const long long e0 = (long long)chunk * kArChunk + 8 * tid;      // this thread's eight values
    const bool live = e0 < P.n;                                      // n is a multiple of 8

    // 1. the own partial into the slot peers read
    uint4 own = make_uint4(0u, 0u, 0u, 0u);
    if (live) {
        own = *reinterpret_cast<const uint4 *>(P.in + e0);
        *reinterpret_cast<uint4 *>(mine + slot_off + 16 * tid) = own;
    }
    __threadfence_system();
    if (tid == 0) s_ok = 1u;
    __syncthreads();
    // 2. tell every rank (this one included), 3. wait for every rank
    if (tid < P.world) {
        unsigned *flag = reinterpret_cast<unsigned *>(P.peer[tid] + kArStatusBytes + kArCounterBytes) +
                         (size_t)P.rank * kArMaxChunks + chunk;
        st_release_sys(flag, gen);
        const unsigned *wait_on = reinterpret_cast<const unsigned *>(mine + kArStatusBytes + kArCounterBytes) +
                                  (size_t)tid * kArMaxChunks + chunk;
        bool there = false;
        for (int it = 0; it < P.spin_limit && !there; ++it) there = (int)(ld_acquire_sys(wait_on) - gen) >= 0;
        if (!there) {
            atomicOr(status, 1u);
            s_ok = 0u;
        }
    }
    __syncthreads();
    if (!s_ok) return;                                               // the output keeps the partial; counter unchanged
    // 4. sum in rank order
    if (live) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        uint4 v[EXL3_AR_MAX_RANKS];
#pragma unroll
        for (int r = 0; r < EXL3_AR_MAX_RANKS; ++r)
            if (r < P.world) v[r] = r == P.rank ? own : ld_peer_v4(P.peer[r] + slot_off + 16 * tid);
#pragma unroll
        for (int r = 0; r < EXL3_AR_MAX_RANKS; ++r)
            if (r < P.world) {
                const __half2 *h = reinterpret_cast<const __half2 *>(&v[r]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(h[j]);
                    acc[2 * j] += f.x;
                    acc[2 * j + 1] += f.y;
                }
            }
        uint4 o;
        __half2 *oh = reinterpret_cast<__half2 *>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
        *reinterpret_cast<uint4 *>(P.out + e0) = o;
    }
    // 5.
    if (tid == 0) *counter = gen;
}

__device__ __forceinline__ void st_ll(void *p, uint32_t data, uint32_t flag) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(data), "r"(flag) : "memory");
}
__device__ __forceinline__ uint2 ld_ll(const void *p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

// The word-with-flag form: see the head of this file.
__global__ void __launch_bounds__(kArThreads) allreduce_ll_kernel(const __grid_constant__ ArParams P) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const int tid = threadIdx.x, chunk = blockIdx.x;
    unsigned char *mine = P.peer[P.rank];
    unsigned *status = reinterpret_cast<unsigned *>(mine);
    unsigned *counter = reinterpret_cast<unsigned *>(mine + kArStatusBytes) + chunk;
    const unsigned gen = *counter + 1u;
    const long long e0 = (long long)chunk * kArChunk + 8 * tid;
    const bool live = e0 < P.n;
    // this thread's four words inside a (slot, source) region: 8 bytes per word
    const size_t word_off = kArLLOffset + (size_t)(gen & 1u) * EXL3_AR_MAX_RANKS * kArLLSrcBytes + (size_t)(e0 / 2) * 8;
    bool ok = true;
    uint4 own = make_uint4(0u, 0u, 0u, 0u);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (live) {
        own = *reinterpret_cast<const uint4 *>(P.in + e0);
        const uint32_t w[4] = {own.x, own.y, own.z, own.w};
#pragma unroll
        for (int r = 0; r < EXL3_AR_MAX_RANKS; ++r)
            if (r < P.world && r != P.rank) {
                unsigned char *dst = P.peer[r] + word_off + (size_t)P.rank * kArLLSrcBytes;
#pragma unroll
                for (int j = 0; j < 4; ++j) st_ll(dst + 8 * j, w[j], gen);
            }
#pragma unroll
        for (int r = 0; r < EXL3_AR_MAX_RANKS; ++r)
            if (r < P.world) {
                uint32_t v[4] = {own.x, own.y, own.z, own.w};
                if (r != P.rank) {
                    const unsigned char *src = mine + word_off + (size_t)r * kArLLSrcBytes;
                    uint2 q[4];
                    bool there = false;
                    for (int it = 0; it < P.spin_limit && !there; ++it) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) q[j] = ld_ll(src + 8 * j);
                        there = q[0].y == gen && q[1].y == gen && q[2].y == gen && q[3].y == gen;
                    }
                    ok = ok && there;
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] = q[j].x;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&v[j]));
                    acc[2 * j] += f.x;
                    acc[2 * j + 1] += f.y;
                }
            }
    }
    // all or nothing per chunk
    if (!__syncthreads_and(ok ? 1 : 0)) {
        if (tid == 0) atomicOr(status, 1u);
        return;
    }
    if (live) {
        uint4 o;
        __half2 *oh = reinterpret_cast<__half2 *>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
        *reinterpret_cast<uint4 *>(P.out + e0) = o;
    }
    if (tid == 0) *counter = gen;
}

}  // namespace exl3

extern "C" size_t exl3_allreduce_buffer_bytes(size_t max_values) {
    const size_t cap = ((max_values * 2 + 255) / 256) * 256;
    return exl3::kArHeadBytes + 2 * cap;
}

extern "C" int exl3_allreduce_oneshot(void *const *peer_buffers, int rank, int world, size_t buffer_bytes, const void *in,
                                      void *out, long long n_values, int spin_limit, void *stream) {
    using namespace exl3;
    if (!peer_buffers || !in || !out) return EXL3_E_NULL;
    if (world < 1 || world > EXL3_AR_MAX_RANKS || rank < 0 || rank >= world || n_values <= 0 || (n_values & 7))
        return EXL3_E_SHAPE;
    if (buffer_bytes < kArHeadBytes + 512 || ((buffer_bytes - kArHeadBytes) & 511)) return EXL3_E_WORKSPACE;
    const size_t cap = (buffer_bytes - kArHeadBytes) / 2;
    const long long chunks = (n_values + kArChunk - 1) / kArChunk;
    if ((size_t)n_values * 2 > cap || chunks > kArMaxChunks) return EXL3_E_WORKSPACE;
    if (!aligned(in, 16) || !aligned(out, 16)) return EXL3_E_ALIGN;
    ArParams P;
    for (int r = 0; r < EXL3_AR_MAX_RANKS; ++r) {
        P.peer[r] = r < world ? static_cast<unsigned char *>(peer_buffers[r]) : nullptr;
        if (r < world && (!P.peer[r] || !aligned(P.peer[r], 256))) return P.peer[r] ? EXL3_E_ALIGN : EXL3_E_NULL;
    }
    P.in = static_cast<const __half *>(in);
    P.out = static_cast<__half *>(out);
    P.n = n_values;
    P.capacity = cap;
    P.rank = rank;
    P.world = world;
    P.spin_limit = spin_limit > 0 ? spin_limit : (1 << 19);       // a fraction of a second of polling
    const cudaError_t e = launch_pdl(n_values <= kArLLMaxValues ? allreduce_ll_kernel : allreduce_oneshot_kernel,
                                     dim3((unsigned)chunks), dim3(kArThreads), 0, static_cast<cudaStream_t>(stream), P);
    if (e != cudaSuccess) { cudaGetLastError(); return EXL3_E_LAUNCH; }
    return launch_status();
}

// ---- the communication buffer: device memory that other processes on the node can map
extern "C" int exl3_comm_alloc(size_t bytes, void **ptr_out, void *ipc_handle_out64) {
    if (!ptr_out || !ipc_handle_out64 || !bytes) return EXL3_E_NULL;
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return EXL3_E_WORKSPACE; }
    if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) { cudaGetLastError(); cudaFree(p); return EXL3_E_LAUNCH; }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaGetLastError(); cudaFree(p); return EXL3_E_LAUNCH; }
    static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
    memcpy(ipc_handle_out64, &h, sizeof(h));
    *ptr_out = p;
    return EXL3_OK;
}
extern "C" int exl3_comm_open(const void *ipc_handle64, void **ptr_out) {
    if (!ipc_handle64 || !ptr_out) return EXL3_E_NULL;
    cudaIpcMemHandle_t h;
    memcpy(&h, ipc_handle64, sizeof(h));
    void *p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return EXL3_E_LAUNCH; }
    *ptr_out = p;
    return EXL3_OK;
}
extern "C" int exl3_comm_close(void *ptr) {
    if (ptr && cudaIpcCloseMemHandle(ptr) != cudaSuccess) { cudaGetLastError(); return EXL3_E_LAUNCH; }
    return EXL3_OK;
}
extern "C" int exl3_comm_free(void *ptr) {
    if (ptr && cudaFree(ptr) != cudaSuccess) { cudaGetLastError(); return EXL3_E_LAUNCH; }
    return EXL3_OK;
}
extern "C" int exl3_comm_status(const void *own_buffer, unsigned *status_out) {
    if (!own_buffer || !status_out) return EXL3_E_NULL;
    if (cudaMemcpy(status_out, own_buffer, 4, cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); return EXL3_E_LAUNCH; }
    return EXL3_OK;
}
