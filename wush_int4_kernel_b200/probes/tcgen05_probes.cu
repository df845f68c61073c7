// Micro-probes of the Blackwell (sm_100a) facts the tcgen05 kernels of this package are designed around.
// Not part of the library: a stand-alone program that prints the figures quoted in the kernels' comments.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o tcgen05_probes wush_int4_kernel_b200/probes/tcgen05_probes.cu
//   ./tcgen05_probes            (a few seconds on one B200; every wait in it is bounded)
//
// 1. issue:   cycles per tcgen05.mma (M = 128; N = 16..256; kind::i8 K = 32 and kind::f16 K = 16; both operand
//             layouts) when ONE thread issues them with precomputed descriptors over 1..16 independent accumulators;
// 2. sync:    mbarrier hop between two warps, tcgen05.commit -> barrier, MMA with A from tensor memory, tcgen05.st,
//             and what a wait on an already-completed barrier costs (try_wait against test_wait);
// 3. contend: the MMA rate and the tcgen05.ld / st round trips while 4..16 other warps hammer tensor memory.
#include <cstdio>
#include <cuda_runtime.h>
#include "../csrc/tc_common.cuh"
using namespace wush::tc;
namespace issue {
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
    uint64_t d = 0; d |= (uint64_t)((saddr & 0x3FFFFu) >> 4); d |= (uint64_t)1 << 16; d |= (uint64_t)(1024 >> 4) << 32; d |= 1ull << 46; d |= 2ull << 61; return d;
}
__device__ __forceinline__ void mma_f16_1(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" :: "r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
// KIND 0 = i8 (K=32), 1 = f16 (K=16); LAYOUT 0 = no swizzle, 1 = SW128; NBUF accumulators; ATILES distinct A tiles
template <int KIND, int LAYOUT, int N, int NBUF, int ATILES>
__global__ void __launch_bounds__(128) probe(int rounds, long long* clk, int* status) {
    extern __shared__ uint8_t raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint32_t slot; __shared__ __align__(8) uint64_t bar;
    for (int i = threadIdx.x; i < 160 * 1024 / 4; i += 128) ((uint32_t*)smem)[i] = KIND == 0 ? 0x01010101u : 0x3c003c00u;
    fence_proxy_async();
    if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
    if (threadIdx.x < 32) { tmem_alloc(&slot, 512); tmem_relinquish(); }
    tc_fence_before(); __syncthreads(); tc_fence_after();
    uint32_t tm = slot;
    if (threadIdx.x == 0) {
        const uint32_t base = smem_u32(smem), bbase = base + 128 * 1024;
        constexpr uint32_t idesc = KIND == 0 ? idesc_i8(N) : idesc_f16(N);
        constexpr int U = NBUF > ATILES ? NBUF : ATILES;          // unroll: one pass over max(bufs, tiles)
        uint64_t ad[ATILES], bd;
#pragma unroll
        for (int t = 0; t < ATILES; ++t)
            ad[t] = LAYOUT == 0 ? smem_desc_kmajor(base + t * 16384, 128 * 16, 128) : desc_sw128(base + t * 16384);
        bd = LAYOUT == 0 ? smem_desc_kmajor(bbase, N * 16, 128) : desc_sw128(bbase);
        long long t0 = clock64();
#pragma unroll 1
        for (int r = 0; r < rounds; ++r) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (KIND == 0) mma_i8(tm + (u % NBUF) * N, ad[u % ATILES], bd, idesc, r > 0);
                else mma_f16_1(tm + (u % NBUF) * N, ad[u % ATILES], bd, idesc, r > 0);
            }
        }
        mma_commit(&bar);
        if (!mbar_wait(&bar, 0)) atomicExch(status, 1);
        long long t1 = clock64();
        if (blockIdx.x == 0) *clk = t1 - t0;
    }
    tc_fence_before(); __syncthreads();
    if (threadIdx.x < 32) tmem_dealloc(tm, 512);
}
static int* status; static long long* clk;
template <int KIND, int LAYOUT, int N, int NBUF, int ATILES> void run() {
    constexpr int U = NBUF > ATILES ? NBUF : ATILES;
    const int rounds = 16384 / U;
    cudaFuncSetAttribute(probe<KIND, LAYOUT, N, NBUF, ATILES>, cudaFuncAttributeMaxDynamicSharedMemorySize, 170 * 1024);
    long long c = 0; float ms = 0;
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    for (int rep = 0; rep < 2; ++rep) {
        cudaEventRecord(e0);
        probe<KIND, LAYOUT, N, NBUF, ATILES><<<148, 128, 165 * 1024>>>(rounds, clk, status);
        cudaEventRecord(e1);
        cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) { printf("CUDA error: %s\n", cudaGetErrorString(e)); exit(1); }
        cudaEventElapsedTime(&ms, e0, e1);
        cudaMemcpy(&c, clk, 8, cudaMemcpyDeviceToHost);
    }
    int st = 0; cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
    const int k = KIND == 0 ? 32 : 16; const double iters = (double)rounds * U;
    printf("%-8s %-5s N=%3d bufs=%2d atiles=%d: %7.1f clk/MMA  %6.0f MAC/clk/SM  %7.1f ns/MMA (%.2f P(FL)OPS)  status %d\n", KIND == 0 ? "i8 K=32" : "f16 K=16",
           LAYOUT == 0 ? "noswz" : "sw128", N, NBUF, ATILES, (double)c / iters, 128.0 * N * k * iters / (double)c, ms * 1e6 / iters,
           2.0 * 148 * 128.0 * N * k * iters / (ms * 1e-3) / 1e15, st);
    fflush(stdout);
}
template <int KIND, int LAYOUT> void sweep() {
    run<KIND, LAYOUT, 16, 1, 1>(); run<KIND, LAYOUT, 16, 4, 1>(); run<KIND, LAYOUT, 16, 16, 1>(); run<KIND, LAYOUT, 16, 16, 8>();
    run<KIND, LAYOUT, 32, 1, 1>(); run<KIND, LAYOUT, 32, 4, 1>(); run<KIND, LAYOUT, 32, 16, 1>(); run<KIND, LAYOUT, 32, 16, 8>();
    run<KIND, LAYOUT, 64, 1, 1>(); run<KIND, LAYOUT, 64, 4, 1>(); run<KIND, LAYOUT, 64, 8, 1>(); run<KIND, LAYOUT, 64, 8, 8>();
    run<KIND, LAYOUT, 128, 1, 1>(); run<KIND, LAYOUT, 128, 4, 1>(); run<KIND, LAYOUT, 128, 4, 8>();
    run<KIND, LAYOUT, 256, 1, 1>(); run<KIND, LAYOUT, 256, 2, 1>(); run<KIND, LAYOUT, 256, 2, 8>();
}
int probe_main() {
    cudaMalloc(&status, 4); cudaMemset(status, 0, 4); cudaMalloc(&clk, 8);
    sweep<0, 0>(); sweep<0, 1>(); sweep<1, 0>(); sweep<1, 1>();
    return 0;
}

}  // namespace issue
namespace sync_lat {
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, 1, 0; tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p; }" :: "r"(d), "r"(a), "l"(b), "r"(idesc) : "memory");
}
__global__ void __launch_bounds__(128) probe(long long* out) {
    extern __shared__ uint8_t raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint32_t slot; __shared__ __align__(8) uint64_t bar[4];
    for (int i = threadIdx.x; i < 16 * 1024 / 4; i += 128) ((uint32_t*)smem)[i] = 0x01010101u;
    fence_proxy_async();
    if (threadIdx.x == 0) { for (int i = 0; i < 4; ++i) mbar_init(&bar[i], 1); mbar_fence_init(); }
    if (threadIdx.x < 32) { tmem_alloc(&slot, 512); tmem_relinquish(); }
    tc_fence_before(); __syncthreads(); tc_fence_after();
    const uint32_t tm = slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int N = 2000;
    // (1) ping-pong: warp 0 lane 0 <-> warp 1 lane 0
    if (lane == 0 && warp < 2) {
        long long t0 = clock64();
        for (int i = 0; i < N; ++i) {
            if (warp == 0) { mbar_arrive(&bar[0]); while (!mbar_try_wait(&bar[1], i & 1)) {} }
            else { while (!mbar_try_wait(&bar[0], i & 1)) {} mbar_arrive(&bar[1]); }
        }
        if (warp == 0) out[0] = (clock64() - t0) / N;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // (2a) commit alone -> wait
        long long t0 = clock64();
        for (int i = 0; i < N; ++i) { mma_commit(&bar[2]); while (!mbar_try_wait(&bar[2], i & 1)) {} }
        out[1] = (clock64() - t0) / N;
        // (2b) one MMA (A in TMEM cols 0..7, D cols 64..79, N=16) + commit -> wait
        const uint64_t bd = smem_desc_kmajor(smem_u32(smem), 16 * 16, 128);
        t0 = clock64();
        for (int i = 0; i < N; ++i) { mma_ts(tm + 64, tm, bd, idesc_i8(16)); mma_commit(&bar[3]); while (!mbar_try_wait(&bar[3], i & 1)) {} }
        out[2] = (clock64() - t0) / N;
        // (2c) four MMAs + commit -> wait
        uint32_t ph = N & 1;
        t0 = clock64();
        for (int i = 0; i < N; ++i) {
            for (int j = 0; j < 4; ++j) mma_ts(tm + 64 + j * 16, tm + j * 8, bd, idesc_i8(16));
            mma_commit(&bar[3]); while (!mbar_try_wait(&bar[3], ph)) {} ph ^= 1;
        }
        out[3] = (clock64() - t0) / N;
        // (2d) back-to-back MMAs from TMEM A, 8 independent accumulators, one commit at the end
        t0 = clock64();
        for (int i = 0; i < N; ++i) for (int j = 0; j < 8; ++j) mma_ts(tm + 64 + j * 16, tm + (j & 3) * 8, bd, idesc_i8(16));
        mma_commit(&bar[3]); while (!mbar_try_wait(&bar[3], ph)) {} ph ^= 1;
        out[4] = (clock64() - t0) / (N * 8);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // (5) issue cost of a wait on an already completed barrier (parity of the previous phase), and of commits
        mbar_init(&bar[0], 1); mbar_fence_init();
        volatile int* flag = (volatile int*)(smem + 8192);
        long long t0 = clock64();
        int acc = 0;
        for (int i = 0; i < N; ++i) {
            for (uint32_t k = 0; k < (1u << 22); ++k) { if (mbar_try_wait(&bar[0], 1)) break; if ((k & 255u) == 255u && *flag) { acc++; break; } }
        }
        out[8] = (clock64() - t0) / N + acc;
        {
            long long t1 = clock64(); int hits = 0;
            for (int i = 0; i < N; ++i) {
                uint32_t ok;
                asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.b32 %0, 1, 0, p; }" : "=r"(ok) : "r"(smem_u32(&bar[0])), "r"(1u) : "memory");
                hits += ok;
            }
            out[11] = (clock64() - t1) / N; out[12] = hits;
            t1 = clock64(); hits = 0;
            for (int i = 0; i < N; ++i) {     // try_wait with a zero suspend-time hint
                uint32_t ok;
                asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3; selp.b32 %0, 1, 0, p; }" : "=r"(ok) : "r"(smem_u32(&bar[0])), "r"(1u), "r"(0u) : "memory");
                hits += ok;
            }
            out[13] = (clock64() - t1) / N; out[14] = hits;
        }
        mbar_init(&bar[1], 1 << 20); mbar_fence_init();
        t0 = clock64();
        for (int i = 0; i < N; ++i) mma_commit(&bar[1]);
        out[9] = (clock64() - t0) / N;
        t0 = clock64();
        for (int i = 0; i < N; ++i) { tc_fence_after(); }
        out[10] = (clock64() - t0) / N;
    }
    __syncthreads();
    // (3) tcgen05.st x8 + wait::st by a full warp
    if (warp == 0) {
        long long t0 = clock64();
        for (int i = 0; i < N; ++i) {
            asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1};" :: "r"(tm + 256), "r"(i) : "memory");
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
        if (lane == 0) out[5] = (clock64() - t0) / N;
        t0 = clock64();
        for (int i = 0; i < N; ++i) {
            for (int j = 0; j < 4; ++j) asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1};" :: "r"(tm + 256 + j * 8), "r"(i) : "memory");
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
        if (lane == 0) out[6] = (clock64() - t0) / N;
        // fence.proxy.async cost after smem stores
        t0 = clock64();
        for (int i = 0; i < N; ++i) { ((volatile uint32_t*)smem)[lane + 32 * (i & 7)] = i; fence_proxy_async(); }
        if (lane == 0) out[7] = (clock64() - t0) / N;
    }
    tc_fence_before(); __syncthreads();
    if (threadIdx.x < 32) tmem_dealloc(tm, 512);
}
int probe_main() {
    long long* out; cudaMalloc(&out, 128); cudaMemset(out, 0, 128);
    cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * 1024);
    for (int rep = 0; rep < 2; ++rep) { probe<<<1, 128, 20 * 1024>>>(out); cudaError_t e = cudaDeviceSynchronize(); if (e != cudaSuccess) { printf("CUDA error %s\n", cudaGetErrorString(e)); return 1; } }
    long long h[16]; cudaMemcpy(h, out, 128, cudaMemcpyDeviceToHost);
    printf("mbarrier ping-pong round trip (2 hops): %lld clk\n", h[0]);
    printf("commit alone -> barrier seen: %lld clk\n", h[1]);
    printf("1 MMA(TS,N=16) + commit -> seen: %lld clk\n", h[2]);
    printf("4 MMAs + commit -> seen: %lld clk\n", h[3]);
    printf("MMA(TS,N=16) issue rate, 8 accumulators: %lld clk/MMA\n", h[4]);
    printf("tcgen05.st.x8 + wait::st: %lld clk;  4 x st.x8 + wait: %lld clk\n", h[5], h[6]);
    printf("st.shared + fence.proxy.async: %lld clk\n", h[7]);
    printf("test_wait on a completed barrier: %lld clk (hits %lld); try_wait with hint 0: %lld clk (hits %lld)\n", h[11], h[12], h[13], h[14]);
    printf("bounded wait on a completed barrier: %lld clk; commit issue: %lld clk; fence::after: %lld clk\n", h[8], h[9], h[10]);
    return 0;
}

}  // namespace sync_lat
namespace contend {
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, 1, 0; tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p; }" :: "r"(d), "r"(a), "l"(b), "r"(idesc) : "memory");
}
__global__ void __launch_bounds__(640) probe(int nld, int nst, int mma_on, long long* out) {
    extern __shared__ uint8_t raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint32_t slot; __shared__ __align__(8) uint64_t bar; __shared__ volatile int stop;
    for (int i = threadIdx.x; i < 16 * 1024 / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0x01010101u;
    fence_proxy_async();
    if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_fence_init(); stop = 0; }
    if (threadIdx.x < 32) { tmem_alloc(&slot, 512); tmem_relinquish(); }
    tc_fence_before(); __syncthreads(); tc_fence_after();
    const uint32_t tm = slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const int N = 4000;
    if (warp == 0) {
        if (lane == 0) {
            const uint64_t bd = smem_desc_kmajor(smem_u32(smem), 16 * 16, 128);
            long long t0 = clock64();
            if (mma_on) {
                for (int i = 0; i < N; ++i) for (int j = 0; j < 8; ++j) mma_ts(tm + 256 + j * 16, tm + (j & 3) * 8, bd, idesc_i8(16));
                mma_commit(&bar); while (!mbar_try_wait(&bar, 0)) {}
            } else { for (int i = 0; i < 2000; ++i) __nanosleep(100); }
            out[0] = (clock64() - t0) / (N * 8);
            stop = 1;
        }
    } else if (warp >= 4 && warp < 4 + nld) {
        long long t0 = clock64(); long long n = 0; uint32_t v[16];
        while (!stop) {
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]) : "r"(tm + lane_base + 384 + ((warp >> 2) & 3) * 16) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" :: "r"(tm + lane_base + 384 + ((warp >> 2) & 3) * 16), "r"(v[0]) : "memory");
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            ++n;
        }
        if (lane == 0 && warp == 4) { out[1] = (clock64() - t0) / (n ? n : 1); }
    } else if (warp >= 12 && warp < 12 + nst) {
        long long t0 = clock64(); long long n = 0;
        while (!stop) {
            for (int j = 0; j < 4; ++j) asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1};" :: "r"(tm + lane_base + 64 + ((warp >> 2) & 1) * 32 + j * 8), "r"((int)n) : "memory");
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            ++n;
        }
        if (lane == 0 && warp == 12) { out[2] = (clock64() - t0) / (n ? n : 1); }
    }
    tc_fence_before(); __syncthreads();
    if (threadIdx.x < 32) tmem_dealloc(tm, 512);
}
int probe_main() {
    long long* out; cudaMalloc(&out, 64);
    cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * 1024);
    int cfg[][3] = {{0, 0, 1}, {8, 0, 1}, {0, 8, 1}, {8, 8, 1}, {8, 8, 0}, {4, 4, 1}};
    for (auto& c : cfg) {
        cudaMemset(out, 0, 64);
        probe<<<148, 640, 20 * 1024>>>(c[0], c[1], c[2], out);
        cudaError_t e = cudaDeviceSynchronize(); if (e != cudaSuccess) { printf("CUDA error %s\n", cudaGetErrorString(e)); return 1; }
        long long h[3]; cudaMemcpy(h, out, 24, cudaMemcpyDeviceToHost);
        printf("ld/st warps %d, st warps %d, mma %d: %lld clk/MMA; ld16+st16 round %lld clk; 4xst8 round %lld clk\n", c[0], c[1], c[2], h[0], h[1], h[2]);
    }
    return 0;
}

}  // namespace contend

int main() {
    printf("== 1. tcgen05.mma issue rate ==\n");
    if (int r = issue::probe_main()) return r;
    printf("== 2. synchronisation latencies ==\n");
    if (int r = sync_lat::probe_main()) return r;
    printf("== 3. tensor-memory contention ==\n");
    return contend::probe_main();
}
