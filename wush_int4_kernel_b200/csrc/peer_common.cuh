// Device-side pieces shared by the kernels that exchange data through the peer-mapped buffers of
// a communicator (peer_reduce.cu, and the decode GEMV when it pushes its result to the peers).
//
// Buffer of one rank (cudaMalloc'ed, mapped by every peer through CUDA IPC):
//   slots[2][world][slot_bytes]   slot (s & 1, r) holds rank r's contribution of step s
//   flags[world]                  flags[r] = number of steps rank r has published
//   state                         CommState
// A contribution is either written by its owner into its OWN buffer and read by the peers
// (pull), or written by its owner into EVERY rank's buffer and read locally (push).
#pragma once
#include <stdint.h>

namespace wush {

constexpr int PR_MAX_WORLD = 8;                      // the GPUs of one NVSwitch node
constexpr size_t PR_FLAG_BYTES = 256, PR_STATE_BYTES = 256;

struct CommState {                                   // device resident
    unsigned int step;                               // steps completed so far
    unsigned int copied;                             // CTAs that finished writing the current step's contribution
    unsigned int done;                               // CTAs that finished the reduction of the current step
    int error;                                       // 1 = a wait ran out
    unsigned int poll_limit;                         // polls after which a wait gives up
    unsigned int copied2;                            // CTAs that finished the second phase of a two-phase step
};

struct PeerTable {                                   // kernel argument: the buffers of all ranks
    uint8_t* base[PR_MAX_WORLD];
    unsigned int* flags[PR_MAX_WORLD];
    CommState* state;                                // this rank's
    size_t slot_bytes;
    int rank, world;
};

__device__ __forceinline__ size_t slot_offset(const PeerTable& t, unsigned int step, int src) {
    return ((size_t)(step & 1u) * t.world + src) * t.slot_bytes;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_sys_v4(const void* p) {            // system-scope load, not served from L1
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

// Called by one full warp of every CTA once the CTA's share of the contribution is written and
// fenced to system scope: counts the CTA, and the last one publishes step + 1 to all ranks
// (lane r stores into rank r's flag array, so the remote stores overlap).
__device__ __forceinline__ void comm_count_and_publish(const PeerTable& t, unsigned int step, int lane,
                                                       unsigned int* counter = nullptr) {
    unsigned int arrived = 0;
    if (lane == 0) arrived = atomicAdd(counter ? counter : &t.state->copied, 1u);
    arrived = __shfl_sync(0xffffffffu, arrived, 0);
    if (arrived == gridDim.x - 1) {
        __threadfence_system();
        if (lane < t.world) st_release_sys(t.flags[lane] + t.rank, step + 1u);
    }
}

}  // namespace wush
