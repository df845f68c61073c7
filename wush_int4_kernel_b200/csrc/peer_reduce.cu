// One-shot all-reduce (sum) of small fp16 partial products over NVLink peer memory
// (C-ABI wush_comm_*).  No counterpart in the reference, which is single-GPU; this is the
// exchange step of the row-parallel down projection when the FFN block is sharded over the
// GPUs of one NVSwitch node.
//
// Decode-size results (M * N * 2 bytes: 16 KB .. a few MB) are latency-bound: a library
// all-reduce costs tens of microseconds there, several times the sharded GEMV it follows.
// Here every rank owns a buffer that all peers have mapped (CUDA IPC):
//
//   slots[2][world][slot_bytes]   slot (s & 1, r) holds rank r's partial result of step s
//   flags[world]                  flags[r] = number of steps rank r has published
//   state                         {step counter, arrival counters, error word, wait bound}
//
// and one kernel per step does
//   1. copy the local partial into this rank's slot (all CTAs, grid-stride), fence to system scope;
//   2. the last CTA to finish the copy publishes: it stores step + 1 into flags[rank] of EVERY
//      rank (remote stores with release semantics at system scope);
//   3. every CTA polls its OWN flags (local memory) until all ranks have published this step
//      -- bounded: after ~1 s it records an error and leaves;
//   4. every CTA sums its share of the world's slots in rank order (peer loads that bypass L1),
//      fp32 accumulation, and writes fp16; the last CTA to finish advances the step counter.
// The result is bit-identical on all ranks (fixed summation order).  Two slots suffice: a rank
// can only publish step s + 2 after its step s + 1 kernel has finished, which needed every
// peer's step s + 1 flag, which a peer sends only after its own step s kernel -- the last reader
// of slot s & 1 -- has completed.  All state lives in device memory, so the launch is the same
// every step and can be captured in a CUDA Graph.
//
// The grid never exceeds the number of multiprocessors: every CTA must be resident while it waits.
//
// Pushed form (wush_comm_gemv_allreduce): the decode GEMV writes its result straight into slot
// (s & 1, rank) of EVERY rank's buffer from its epilogue and publishes when its last CTA is done;
// the kernel here then skips steps 1 and 2 and sums the slots of its OWN buffer -- no copy, and no
// NVLink round trip after the flags have arrived.
#include <cstddef>
#include <cstring>

#include "common.cuh"
#include "peer_common.cuh"

namespace wush {
namespace {

constexpr int PR_THREADS = 256;
constexpr uint32_t PR_POLL_LIMIT = 1u << 21;        // default bound of a wait: x ~0.5 us of back-off per poll

// Steps 1-3 of an exchange, shared by the sum and the gather: write the contribution (unless the
// producer kernel pushed it), publish, wait -- bounded -- until every rank has published this step.
// Called by all threads of every CTA; returns the step number and whether the wait succeeded.
__device__ __forceinline__ bool exchange_begin(const uint4* __restrict__ local, long long n_vec, const PeerTable& peers,
                                               int pushed, unsigned int* step_out)
{
    __shared__ unsigned int s_step, s_ok;
    CommState* state = peers.state;
    const int rank = peers.rank, world = peers.world;
    pdl_wait();                                                        // the partial may come from the kernel just before
    if (threadIdx.x == 0) s_step = *reinterpret_cast<volatile unsigned int*>(&state->step);
    __syncthreads();
    const unsigned int step = s_step;
    const unsigned int poll_limit = *reinterpret_cast<volatile unsigned int*>(&state->poll_limit);
    const long long stride = (long long)gridDim.x * PR_THREADS;
    const long long first = (long long)blockIdx.x * PR_THREADS + threadIdx.x;

    if (!pushed) {
        // 1. publish the data: this rank's slot of its own buffer
        uint4* mine = reinterpret_cast<uint4*>(peers.base[rank] + slot_offset(peers, step, rank));
        for (long long i = first; i < n_vec; i += stride) mine[i] = local[i];
        __threadfence_system();
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        // warp 0: lane r talks to rank r, so the remote stores and the polls of all ranks overlap
        const int lane = threadIdx.x;
        // 2. every CTA's part is written and fenced: the last one tells everybody (this rank included)
        if (!pushed) comm_count_and_publish(peers, step, lane);
        // 3. wait until every rank has published this step (flags only ever grow)
        bool ok = true;
        if (lane < world) {
            uint32_t polls = 0;
            while ((int)(ld_acquire_sys(peers.flags[rank] + lane) - (step + 1u)) < 0) {
                if (++polls > poll_limit) { ok = false; break; }
                __nanosleep(polls < 64 ? 20 : 500);
            }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (lane == 0) {
            if (!ok) atomicExch(&state->error, 1);
            s_ok = ok ? 1u : 0u;
        }
    }
    __syncthreads();
    *step_out = step;
    return s_ok != 0;
}

// The last CTA out advances the step counter and clears the arrival counters.
__device__ __forceinline__ void exchange_end(const PeerTable& peers, unsigned int step)
{
    CommState* state = peers.state;
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int finished = atomicAdd(&state->done, 1u);
        if (finished == gridDim.x - 1) {
            state->copied = 0;
            state->copied2 = 0;
            state->done = 0;
            __threadfence();
            state->step = step + 1u;
        }
    }
}

// Bounded wait of warp 0 until every rank has published `target` steps; all threads get the outcome.
__device__ __forceinline__ bool wait_all_published(const PeerTable& peers, unsigned int target)
{
    __shared__ unsigned int s_ok2;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        const unsigned int poll_limit = *reinterpret_cast<volatile unsigned int*>(&peers.state->poll_limit);
        bool ok = true;
        if (lane < peers.world) {
            uint32_t polls = 0;
            while ((int)(ld_acquire_sys(peers.flags[peers.rank] + lane) - target) < 0) {
                if (++polls > poll_limit) { ok = false; break; }
                __nanosleep(polls < 64 ? 20 : 500);
            }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (lane == 0) {
            if (!ok) atomicExch(&peers.state->error, 1);
            s_ok2 = ok ? 1u : 0u;
        }
    }
    __syncthreads();
    return s_ok2 != 0;
}

// Two-phase sum for results of megabytes (prefill): a reduce-scatter and an all-gather over peer memory in ONE
// kernel, two steps of the communicator.  Step s: every rank puts its partial into its own slot (s & 1, rank)
// and publishes; rank r then sums vectors [r n/world, (r+1) n/world) of all ranks' slots in rank order (peer
// loads, fp32) and stores the fp16 result into slot ((s+1) & 1, p) of EVERY rank p (remote stores).  Step
// s + 1: publish, wait, copy the own slot ((s+1) & 1, rank) to the output.  Per rank (world-1)/world of the
// data crosses NVLink in each direction, against (world-1) times the data read by the one-phase kernel; the
// result is the same bit for bit (same summation order).
__global__ void __launch_bounds__(PR_THREADS)
peer_allreduce_two_phase_f16_kernel(const uint4* __restrict__ local, uint4* __restrict__ out, long long n_vec, const PeerTable peers)
{
    const int rank = peers.rank, world = peers.world;
    const long long stride = (long long)gridDim.x * PR_THREADS;
    const long long first = (long long)blockIdx.x * PR_THREADS + threadIdx.x;
    unsigned int step;
    bool ok = exchange_begin(local, n_vec, peers, 0, &step);

    if (ok) {                                                          // reduce-scatter: this rank's share
        const long long c0 = n_vec * rank / world, c1 = n_vec * (rank + 1) / world;
        for (long long i = c0 + first; i < c1; i += stride) {
            uint4 v[PR_MAX_WORLD];
#pragma unroll
            for (int r = 0; r < PR_MAX_WORLD; ++r) {
                const int src = r < world ? r : rank;
                v[r] = ld_sys_v4(reinterpret_cast<const uint4*>(peers.base[src] + slot_offset(peers, step, src)) + i);
            }
            float acc[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
            for (int r = 0; r < PR_MAX_WORLD; ++r) {
                if (r < world) {
                    const uint32_t w[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[p]));
                        acc[2 * p] += f.x;
                        acc[2 * p + 1] += f.y;
                    }
                }
            }
            uint32_t o[4];
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                __half2 h = __floats2half2_rn(acc[2 * p], acc[2 * p + 1]);
                o[p] = *reinterpret_cast<uint32_t*>(&h);
            }
            const uint4 res = make_uint4(o[0], o[1], o[2], o[3]);
#pragma unroll
            for (int p = 0; p < PR_MAX_WORLD; ++p)
                if (p < world) reinterpret_cast<uint4*>(peers.base[p] + slot_offset(peers, step + 1u, p))[i] = res;
        }
    }
    // second step: this rank's share is in every rank's buffer -> publish, wait for everybody's
    __threadfence_system();
    __syncthreads();
    if (ok && threadIdx.x < 32) comm_count_and_publish(peers, step + 1u, threadIdx.x, &peers.state->copied2);   // a rank that did not see every partial delivers nothing
    ok = wait_all_published(peers, step + 2u) && ok;
    if (ok) {
        const uint4* mine = reinterpret_cast<const uint4*>(peers.base[rank] + slot_offset(peers, step + 1u, rank));
        for (long long i = first; i < n_vec; i += stride) out[i] = ld_sys_v4(mine + i);
    }
    exchange_end(peers, step + 1u);
}

__global__ void __launch_bounds__(PR_THREADS)
peer_allreduce_f16_kernel(const uint4* __restrict__ local, uint4* __restrict__ out, long long n_vec,   // 8 halves per vector
                          const PeerTable peers, int pushed)
{
    const int rank = peers.rank, world = peers.world;
    const long long stride = (long long)gridDim.x * PR_THREADS;
    const long long first = (long long)blockIdx.x * PR_THREADS + threadIdx.x;
    unsigned int step;
    const bool ok = exchange_begin(local, n_vec, peers, pushed, &step);

    // 4. reduce in rank order
    if (ok) {
        for (long long i = first; i < n_vec; i += stride) {
            // all peers' vectors are requested before the first one is used: one NVLink round trip, not `world`
            uint4 v[PR_MAX_WORLD];
#pragma unroll
            for (int r = 0; r < PR_MAX_WORLD; ++r) {           // ranks beyond the world re-read this rank's slot (ignored below)
                const int src = r < world ? r : rank;
                v[r] = ld_sys_v4(reinterpret_cast<const uint4*>(peers.base[pushed ? rank : src] + slot_offset(peers, step, src)) + i);
            }
            float acc[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
            for (int r = 0; r < PR_MAX_WORLD; ++r) {
                if (r < world) {
                    const uint32_t w[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[p]));
                        acc[2 * p] += f.x;
                        acc[2 * p + 1] += f.y;
                    }
                }
            }
            uint32_t o[4];
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                __half2 h = __floats2half2_rn(acc[2 * p], acc[2 * p + 1]);
                o[p] = *reinterpret_cast<uint32_t*>(&h);
            }
            out[i] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
    exchange_end(peers, step);
}

// All-gather of column blocks: rank r contributes a (rows, width[r]) fp16 block (row-major in its slot), the
// result is the (rows, sum of widths) matrix with the blocks side by side in rank order.  Widths and offsets
// are in 16-byte vectors (8 halves).
struct GatherShape {
    int width[PR_MAX_WORLD];
    int offset[PR_MAX_WORLD];
    int total;
};

__global__ void __launch_bounds__(PR_THREADS)
peer_allgather_f16_kernel(const uint4* __restrict__ local, uint4* __restrict__ out, int rows, const GatherShape shape,
                          const PeerTable peers, int pushed)
{
    const int rank = peers.rank, world = peers.world;
    const long long stride = (long long)gridDim.x * PR_THREADS;
    const long long first = (long long)blockIdx.x * PR_THREADS + threadIdx.x;
    unsigned int step;
    const bool ok = exchange_begin(local, (long long)rows * shape.width[rank], peers, pushed, &step);

    // 4. copy: the output is walked in its own order (coalesced stores), the source slot found per vector
    if (ok) {
        const long long n_out = (long long)rows * shape.total;
        for (long long j = first; j < n_out; j += stride) {
            const int row = (int)(j / shape.total), c = (int)(j - (long long)row * shape.total);
            int src = 0;
#pragma unroll
            for (int r = 1; r < PR_MAX_WORLD; ++r)
                if (r < world && c >= shape.offset[r]) src = r;
            const uint4* slot = reinterpret_cast<const uint4*>(peers.base[pushed ? rank : src] + slot_offset(peers, step, src));
            out[j] = ld_sys_v4(slot + (long long)row * shape.width[src] + (c - shape.offset[src]));
        }
    }
    exchange_end(peers, step);
}

struct Comm {
    int rank, world, device;
    size_t slot_bytes;
    uint8_t* base;                 // own allocation: slots | flags | state
    uint8_t* peer_base[PR_MAX_WORLD];
    bool connected[PR_MAX_WORLD];
    bool borrowed[PR_MAX_WORLD];   // mapped by pointer (same process), not through an IPC handle
};

size_t slots_bytes(const Comm* c) { return 2 * (size_t)c->world * c->slot_bytes; }
size_t comm_bytes(const Comm* c) { return slots_bytes(c) + PR_FLAG_BYTES + PR_STATE_BYTES; }

int fill_table(const Comm* c, PeerTable* t, const char* what)
{
    for (int r = 0; r < PR_MAX_WORLD; ++r) { t->base[r] = nullptr; t->flags[r] = nullptr; }
    for (int r = 0; r < c->world; ++r) {
        if (!c->connected[r]) return fail(WUSH_ERR_INVALID_ARGUMENT, "%s: rank %d is not connected", what, r);
        t->base[r] = c->peer_base[r];
        t->flags[r] = reinterpret_cast<unsigned int*>(c->peer_base[r] + slots_bytes(c));
    }
    t->state = reinterpret_cast<CommState*>(c->base + slots_bytes(c) + PR_FLAG_BYTES);
    t->slot_bytes = c->slot_bytes;
    t->rank = c->rank;
    t->world = c->world;
    return WUSH_OK;
}

int launch_reduce(const Comm* c, const PeerTable& t, const void* partial, void* out, int64_t n, int pushed, cudaStream_t st)
{
    const long long n_vec = n / 8;
    long long blocks = (n_vec + PR_THREADS - 1) / PR_THREADS;
    if (blocks > sm_count()) blocks = sm_count();                       // every CTA resident while it waits
    cudaError_t e = launch_dependent(peer_allreduce_f16_kernel, dim3((unsigned)blocks), dim3(PR_THREADS), (size_t)0, st,
                                     (const uint4*)partial, (uint4*)out, n_vec, t, pushed);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "comm_allreduce launch: %s", cudaGetErrorString(e));
    return WUSH_OK;
}

int launch_reduce_two_phase(const Comm* c, const PeerTable& t, const void* partial, void* out, int64_t n, cudaStream_t st)
{
    const long long n_vec = n / 8;
    long long blocks = (n_vec + PR_THREADS - 1) / PR_THREADS;
    if (blocks > sm_count()) blocks = sm_count();                       // every CTA resident while it waits
    cudaError_t e = launch_dependent(peer_allreduce_two_phase_f16_kernel, dim3((unsigned)blocks), dim3(PR_THREADS), (size_t)0, st,
                                     (const uint4*)partial, (uint4*)out, n_vec, t);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "comm_allreduce (two-phase) launch: %s", cudaGetErrorString(e));
    return WUSH_OK;
}

int gather_shape(const Comm* c, const int64_t* widths, int64_t rows, GatherShape* g, const char* what)
{
    if (!widths) return fail(WUSH_ERR_INVALID_ARGUMENT, "%s: null widths", what);
    int64_t off = 0;
    for (int r = 0; r < PR_MAX_WORLD; ++r) { g->width[r] = 0; g->offset[r] = 0; }
    for (int r = 0; r < c->world; ++r) {
        const int64_t w = widths[r];
        if (w <= 0 || w % 8 != 0) return fail(WUSH_ERR_INVALID_ARGUMENT, "%s: width of rank %d (%lld) must be a positive multiple of 8", what, r, (long long)w);
        if ((size_t)(rows * w) * 2 > c->slot_bytes)
            return fail(WUSH_ERR_INVALID_ARGUMENT, "%s: %lld x %lld halves do not fit the slot of %zu bytes", what, (long long)rows, (long long)w, c->slot_bytes);
        g->width[r] = (int)(w / 8);
        g->offset[r] = (int)(off / 8);
        off += w;
    }
    if (off / 8 > INT32_MAX / 2 || rows > INT32_MAX / 2) return fail(WUSH_ERR_INVALID_ARGUMENT, "%s: result too large", what);
    g->total = (int)(off / 8);
    return WUSH_OK;
}

int launch_gather(const Comm* c, const PeerTable& t, const void* local, void* out, int64_t rows, const GatherShape& g, int pushed,
                  cudaStream_t st)
{
    long long blocks = ((long long)rows * g.total + PR_THREADS - 1) / PR_THREADS;
    if (blocks > sm_count()) blocks = sm_count();                       // every CTA resident while it waits
    cudaError_t e = launch_dependent(peer_allgather_f16_kernel, dim3((unsigned)blocks), dim3(PR_THREADS), (size_t)0, st,
                                     (const uint4*)local, (uint4*)out, (int)rows, g, t, pushed);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "comm_allgather launch: %s", cudaGetErrorString(e));
    return WUSH_OK;
}

}  // namespace
}  // namespace wush

WUSH_API int wush_comm_create(int rank, int world, size_t slot_bytes, void** comm_out)
{
    using namespace wush;
    if (int e = ensure_init()) return e;
    WUSH_REQUIRE(comm_out, "comm_create: null pointer");
    WUSH_REQUIRE(world >= 1 && world <= PR_MAX_WORLD && rank >= 0 && rank < world, "comm_create: bad rank %d of %d", rank, world);
    WUSH_REQUIRE(slot_bytes > 0 && slot_bytes % 256 == 0, "comm_create: slot size must be a positive multiple of 256 bytes");
    Comm* c = new Comm();
    c->rank = rank;
    c->world = world;
    c->slot_bytes = slot_bytes;
    cudaGetDevice(&c->device);
    for (int r = 0; r < PR_MAX_WORLD; ++r) { c->peer_base[r] = nullptr; c->connected[r] = false; c->borrowed[r] = false; }
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&c->base), comm_bytes(c));
    if (e == cudaSuccess) e = cudaMemset(c->base, 0, comm_bytes(c));
    if (e == cudaSuccess) {
        CommState init = {0, 0, 0, 0, PR_POLL_LIMIT, 0};
        e = cudaMemcpy(c->base + slots_bytes(c) + PR_FLAG_BYTES, &init, sizeof(init), cudaMemcpyHostToDevice);
    }
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        delete c;
        return fail(WUSH_ERR_CUDA, "comm_create: %s", cudaGetErrorString(e));
    }
    c->peer_base[rank] = c->base;
    c->connected[rank] = true;
    *comm_out = c;
    return WUSH_OK;
}

WUSH_API int wush_comm_export(void* comm, void* handle64)
{
    using namespace wush;
    WUSH_REQUIRE(comm && handle64, "comm_export: null pointer");
    Comm* c = static_cast<Comm*>(comm);
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, c->base);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "comm_export: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
    memcpy(handle64, &h, 64);
    return WUSH_OK;
}

WUSH_API int wush_comm_connect(void* comm, int peer_rank, const void* handle64)
{
    using namespace wush;
    WUSH_REQUIRE(comm && handle64, "comm_connect: null pointer");
    Comm* c = static_cast<Comm*>(comm);
    WUSH_REQUIRE(peer_rank >= 0 && peer_rank < c->world && peer_rank != c->rank, "comm_connect: bad peer rank %d", peer_rank);
    WUSH_REQUIRE(!c->connected[peer_rank], "comm_connect: rank %d is already connected", peer_rank);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "comm_connect: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
    c->peer_base[peer_rank] = static_cast<uint8_t*>(p);
    c->connected[peer_rank] = true;
    return WUSH_OK;
}

WUSH_API int wush_comm_connect_pointer(void* comm, int peer_rank, void* peer_base)
{
    using namespace wush;
    WUSH_REQUIRE(comm && peer_base, "comm_connect_pointer: null pointer");
    Comm* c = static_cast<Comm*>(comm);
    WUSH_REQUIRE(peer_rank >= 0 && peer_rank < c->world && peer_rank != c->rank, "comm_connect_pointer: bad peer rank %d", peer_rank);
    WUSH_REQUIRE(!c->connected[peer_rank], "comm_connect_pointer: rank %d is already connected", peer_rank);
    c->peer_base[peer_rank] = static_cast<uint8_t*>(peer_base);
    c->connected[peer_rank] = true;
    c->borrowed[peer_rank] = true;
    return WUSH_OK;
}

WUSH_API int wush_comm_base(void* comm, void** base)
{
    using namespace wush;
    WUSH_REQUIRE(comm && base, "comm_base: null pointer");
    *base = static_cast<Comm*>(comm)->base;
    return WUSH_OK;
}

WUSH_API int wush_comm_set_poll_limit(void* comm, unsigned int polls)
{
    using namespace wush;
    WUSH_REQUIRE(comm && polls > 0, "comm_set_poll_limit: bad argument");
    Comm* c = static_cast<Comm*>(comm);
    cudaError_t e = cudaMemcpy(c->base + slots_bytes(c) + PR_FLAG_BYTES + offsetof(CommState, poll_limit), &polls,
                               sizeof(polls), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "comm_set_poll_limit: %s", cudaGetErrorString(e));
    return WUSH_OK;
}

WUSH_API int wush_comm_allreduce_f16(void* comm, const void* partial, void* out, int64_t n, void* stream)
{
    using namespace wush;
    WUSH_REQUIRE(comm, "comm_allreduce: null communicator");
    Comm* c = static_cast<Comm*>(comm);
    WUSH_REQUIRE(n >= 0 && n % 8 == 0, "comm_allreduce: element count must be a multiple of 8");
    if (n == 0) return WUSH_OK;
    WUSH_REQUIRE(partial && out && aligned16(partial) && aligned16(out), "comm_allreduce: pointers must be 16-byte aligned");
    WUSH_REQUIRE((size_t)n * 2 <= c->slot_bytes, "comm_allreduce: %lld halves do not fit the slot of %zu bytes", (long long)n,
                 c->slot_bytes);
    PeerTable t;
    if (int s = fill_table(c, &t, "comm_allreduce")) return s;
    return launch_reduce(c, t, partial, out, n, 0, (cudaStream_t)stream);
}

// The same sum as reduce-scatter + all-gather in one kernel (two steps of the communicator): for results of a
// megabyte and more, where the one-phase kernel's (world - 1) reads of everything cost more than a second wait.
WUSH_API int wush_comm_allreduce_two_phase_f16(void* comm, const void* partial, void* out, int64_t n, void* stream)
{
    using namespace wush;
    WUSH_REQUIRE(comm, "comm_allreduce_two_phase: null communicator");
    Comm* c = static_cast<Comm*>(comm);
    WUSH_REQUIRE(n >= 0 && n % 8 == 0, "comm_allreduce_two_phase: element count must be a multiple of 8");
    if (n == 0) return WUSH_OK;
    WUSH_REQUIRE(partial && out && aligned16(partial) && aligned16(out), "comm_allreduce_two_phase: pointers must be 16-byte aligned");
    WUSH_REQUIRE((size_t)n * 2 <= c->slot_bytes, "comm_allreduce_two_phase: %lld halves do not fit the slot of %zu bytes", (long long)n,
                 c->slot_bytes);
    PeerTable t;
    if (int s = fill_table(c, &t, "comm_allreduce_two_phase")) return s;
    return launch_reduce_two_phase(c, t, partial, out, n, (cudaStream_t)stream);
}

// Decode product and the sum over ranks as one chain of two kernels that share the exchange: the
// product's epilogue stores into every rank's slot, its last CTA publishes, the reduction reads
// only local memory.  M <= 2 runs the CUDA-core GEMV, 3 <= M <= 32 (and M <= 2 with a K the GEMV
// does not hold in shared memory) the tensor-core streaming kernel (K % 256 == 0).
// WUSH_ERR_UNSUPPORTED for other shapes or results that do not fit a slot: use wush_w4a4_gemm +
// wush_comm_allreduce_f16.
namespace wush {
int gemv_dispatch_push(const uint8_t*, const void*, const uint8_t*, const void*, int64_t, int64_t, int64_t, const PeerTable&,
                       cudaStream_t);
size_t gemv_smem_bytes(int M, int64_t K);
int stream_dispatch_push(const uint8_t*, const void*, const uint8_t*, const void*, int64_t, int64_t, int64_t, const PeerTable&,
                         cudaStream_t);
bool stream_supported(int64_t K, const void* xs, const void* ws);
}

WUSH_API int wush_comm_gemv_allreduce(void* comm, const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws,
                                      int64_t M, int64_t N, int64_t K, void* out, void* stream)
{
    using namespace wush;
    WUSH_REQUIRE(comm, "comm_gemv_allreduce: null communicator");
    Comm* c = static_cast<Comm*>(comm);
    WUSH_REQUIRE(M >= 1 && N >= 1 && K > 0 && K % 32 == 0, "comm_gemv_allreduce: bad shape");
    WUSH_REQUIRE(xq && xs && wq && ws && out, "comm_gemv_allreduce: null pointer");
    WUSH_REQUIRE(aligned16(xq) && aligned16(wq) && aligned16(out), "comm_gemv_allreduce: pointers must be 16-byte aligned");
    const bool by_gemv = M <= 2 && gemv_smem_bytes((int)M, K) <= 200 * 1024;
    const bool by_stream = M <= 32 && stream_supported(K, xs, ws);
    if ((!by_gemv && !by_stream) || (M * N) % 8 != 0 || (size_t)(M * N) * 2 > c->slot_bytes)
        return fail(WUSH_ERR_UNSUPPORTED, "comm_gemv_allreduce: M=%lld N=%lld K=%lld is outside the pushed kernels' range",
                    (long long)M, (long long)N, (long long)K);
    PeerTable t;
    if (int s = fill_table(c, &t, "comm_gemv_allreduce")) return s;
    if (int s = by_gemv ? gemv_dispatch_push(xq, xs, wq, ws, M, N, K, t, (cudaStream_t)stream)
                        : stream_dispatch_push(xq, xs, wq, ws, M, N, K, t, (cudaStream_t)stream))
        return s;
    return launch_reduce(c, t, nullptr, out, M * N, 1, (cudaStream_t)stream);
}

// All-gather of the column blocks of a column-parallel product: out (rows, sum of widths) receives rank r's
// (rows, widths[r]) block at column offset widths[0] + .. + widths[r-1].
WUSH_API int wush_comm_allgather_f16(void* comm, const void* local, void* out, int64_t rows, const int64_t* widths, void* stream)
{
    using namespace wush;
    WUSH_REQUIRE(comm, "comm_allgather: null communicator");
    Comm* c = static_cast<Comm*>(comm);
    WUSH_REQUIRE(rows >= 0, "comm_allgather: bad row count");
    GatherShape g;
    if (int s = gather_shape(c, widths, rows, &g, "comm_allgather")) return s;
    if (rows == 0) return WUSH_OK;
    WUSH_REQUIRE(local && out && aligned16(local) && aligned16(out), "comm_allgather: pointers must be 16-byte aligned");
    PeerTable t;
    if (int s = fill_table(c, &t, "comm_allgather")) return s;
    return launch_gather(c, t, local, out, rows, g, 0, (cudaStream_t)stream);
}

// Column-parallel decode product and the all-gather of its column blocks as one chain: the product's
// epilogue stores this rank's (M, widths[rank]) block into its slot of EVERY rank's buffer, the gather
// that follows reads only local memory.  Shapes as for wush_comm_gemv_allreduce (N = widths[rank]).
WUSH_API int wush_comm_gemv_allgather(void* comm, const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws,
                                      int64_t M, int64_t K, const int64_t* widths, void* out, void* stream)
{
    using namespace wush;
    WUSH_REQUIRE(comm, "comm_gemv_allgather: null communicator");
    Comm* c = static_cast<Comm*>(comm);
    WUSH_REQUIRE(M >= 1 && K > 0 && K % 32 == 0, "comm_gemv_allgather: bad shape");
    WUSH_REQUIRE(xq && xs && wq && ws && out, "comm_gemv_allgather: null pointer");
    WUSH_REQUIRE(aligned16(xq) && aligned16(wq) && aligned16(out), "comm_gemv_allgather: pointers must be 16-byte aligned");
    GatherShape g;
    if (int s = gather_shape(c, widths, M, &g, "comm_gemv_allgather")) return s;
    const int64_t N = widths[c->rank];
    const bool by_gemv = M <= 2 && gemv_smem_bytes((int)M, K) <= 200 * 1024;
    const bool by_stream = M <= 32 && stream_supported(K, xs, ws);
    if (!by_gemv && !by_stream)
        return fail(WUSH_ERR_UNSUPPORTED, "comm_gemv_allgather: M=%lld K=%lld is outside the pushed kernels' range", (long long)M,
                    (long long)K);
    PeerTable t;
    if (int s = fill_table(c, &t, "comm_gemv_allgather")) return s;
    if (int s = by_gemv ? gemv_dispatch_push(xq, xs, wq, ws, M, N, K, t, (cudaStream_t)stream)
                        : stream_dispatch_push(xq, xs, wq, ws, M, N, K, t, (cudaStream_t)stream))
        return s;
    return launch_gather(c, t, nullptr, out, M, g, 1, (cudaStream_t)stream);
}

WUSH_API int wush_comm_error(void* comm, int* error)
{
    using namespace wush;
    WUSH_REQUIRE(comm && error, "comm_error: null pointer");
    Comm* c = static_cast<Comm*>(comm);
    CommState st;
    cudaError_t e = cudaMemcpy(&st, c->base + slots_bytes(c) + PR_FLAG_BYTES, sizeof(st), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "comm_error: %s", cudaGetErrorString(e));
    *error = st.error;
    return WUSH_OK;
}

WUSH_API int wush_comm_destroy(void* comm)
{
    using namespace wush;
    if (!comm) return WUSH_OK;
    Comm* c = static_cast<Comm*>(comm);
    cudaDeviceSynchronize();
    for (int r = 0; r < c->world; ++r)
        if (r != c->rank && c->connected[r] && !c->borrowed[r]) cudaIpcCloseMemHandle(c->peer_base[r]);
    cudaFree(c->base);
    delete c;
    return WUSH_OK;
}
