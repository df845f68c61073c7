// Helpers around the tensor-core product kernels (the streaming kernel lives in
// gemm_stream.cu, the tcgen05 tile kernel in gemm_tc.cu):
//   * a plain CUDA-core kernel for shapes neither takes (K not a multiple of 256),
//   * the exact-partial-sum test op wush_group_partials, which runs the SAME tensor-core
//     kernels in a mode that writes the int32 group sums instead of scaling them,
//   * the one-atom int8 MMA self-test (reference s4_atom_selftest, csrc/gemm_s4.cu:50-82).
#include "common.cuh"

namespace wush {

bool tc_supported(int64_t M, int64_t N, int64_t K);
int tc_partials(const uint8_t* xq, const uint8_t* wq, int64_t M, int64_t N, int64_t K, int32_t* P, int* err, cudaStream_t st);
bool stream_supported(int64_t K, const void* xs, const void* ws);
int stream_dispatch(const uint8_t*, const void*, const uint8_t*, const void*, int64_t, int64_t, int64_t, void*, cudaStream_t);
int stream_partials(const uint8_t* xq, const uint8_t* wq, int64_t M, int64_t N, int64_t K, int32_t* P, cudaStream_t st);
__device__ int g_partials_err;

__device__ __forceinline__ void mma_s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Plain CUDA-core kernel for any K % 32 == 0 (used when K % 256 != 0): one thread per output,
// exact integer dot per group via dp4a, fp32 accumulation.  PARTIALS as above.
template <bool PARTIALS>
__global__ void __launch_bounds__(256)
w4a4_simple_kernel(const uint8_t* __restrict__ xq, const __nv_bfloat16* __restrict__ xs,
                   const uint8_t* __restrict__ wq, const __nv_bfloat16* __restrict__ ws,
                   __half* __restrict__ y, int32_t* __restrict__ part, int M, int N, int K)
{
    const int n = blockIdx.x * 32 + (threadIdx.x & 31);
    const int m = blockIdx.y * 8 + (threadIdx.x >> 5);
    if (n >= N || m >= M) return;
    const int G = K >> 5;
    const uint4* xr = reinterpret_cast<const uint4*>(xq + (size_t)m * (K >> 1));
    const uint4* wr = reinterpret_cast<const uint4*>(wq + (size_t)n * (K >> 1));
    float acc = 0.f;
    for (int g = 0; g < G; ++g) {
        uint4 a = xr[g], b = wr[g];
        uint32_t ae, ao, be, bo;
        int d = 0;
        unpack_x16(a.x, ae, ao); unpack_x16(b.x, be, bo); d = dp4a_s8(ae, be, d); d = dp4a_s8(ao, bo, d);
        unpack_x16(a.y, ae, ao); unpack_x16(b.y, be, bo); d = dp4a_s8(ae, be, d); d = dp4a_s8(ao, bo, d);
        unpack_x16(a.z, ae, ao); unpack_x16(b.z, be, bo); d = dp4a_s8(ae, be, d); d = dp4a_s8(ao, bo, d);
        unpack_x16(a.w, ae, ao); unpack_x16(b.w, be, bo); d = dp4a_s8(ae, be, d); d = dp4a_s8(ao, bo, d);
        if constexpr (PARTIALS) {
            part[((size_t)m * N + n) * G + g] = d >> 8;
        } else {
            float s = __bfloat162float(xs[(size_t)m * G + g]) * __bfloat162float(ws[(size_t)n * G + g]);
            acc = fmaf((float)d, s * (1.0f / 256.0f), acc);
        }
    }
    if constexpr (!PARTIALS) y[(size_t)m * N + n] = __float2half_rn(acc);
}

// One int8 MMA atom: a (8,32) row-major, b (32,8) row-major (b[k*8+n]) -> c (8,8) int32.
__global__ void i8_atom_kernel(const int8_t* __restrict__ a, const int8_t* __restrict__ b, int32_t* __restrict__ c)
{
    const int lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    auto pack4 = [](int v0, int v1, int v2, int v3) {
        return (uint32_t)(v0 & 0xff) | ((uint32_t)(v1 & 0xff) << 8) | ((uint32_t)(v2 & 0xff) << 16) | ((uint32_t)(v3 & 0xff) << 24);
    };
    const int8_t* ar = a + gid * 32;
    uint32_t a0 = pack4(ar[tig * 4], ar[tig * 4 + 1], ar[tig * 4 + 2], ar[tig * 4 + 3]);
    uint32_t a2 = pack4(ar[16 + tig * 4], ar[16 + tig * 4 + 1], ar[16 + tig * 4 + 2], ar[16 + tig * 4 + 3]);
    uint32_t b0 = pack4(b[(tig * 4) * 8 + gid], b[(tig * 4 + 1) * 8 + gid], b[(tig * 4 + 2) * 8 + gid], b[(tig * 4 + 3) * 8 + gid]);
    uint32_t b1 = pack4(b[(16 + tig * 4) * 8 + gid], b[(17 + tig * 4) * 8 + gid], b[(18 + tig * 4) * 8 + gid], b[(19 + tig * 4) * 8 + gid]);
    int d[4];
    mma_s8_16832(d, a0, 0u, a2, 0u, b0, b1);       // rows 8..15 of the atom are zero
    c[gid * 8 + tig * 2] = d[0];
    c[gid * 8 + tig * 2 + 1] = d[1];
}

int mma_set_attributes() { return WUSH_OK; }

// Any M.  Streaming tensor-core kernel when the shape allows whole TMA stages, else CUDA cores.
int mma_dispatch(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N,
                 int64_t K, void* y, cudaStream_t st)
{
    if (stream_supported(K, xs, ws)) return stream_dispatch(xq, xs, wq, ws, M, N, K, y, st);
    dim3 grid((unsigned)((N + 31) / 32), (unsigned)((M + 7) / 8));
    if (grid.y > 65535) return fail(WUSH_ERR_UNSUPPORTED, "w4a4_gemm: M too large for the fallback kernel");
    w4a4_simple_kernel<false><<<grid, 256, 0, st>>>(xq, (const __nv_bfloat16*)xs, wq, (const __nv_bfloat16*)ws,
                                                    (__half*)y, nullptr, (int)M, (int)N, (int)K);
    return check_launch("w4a4_simple");
}

}  // namespace wush

WUSH_API int wush_group_partials(const uint8_t* xq, const uint8_t* wq, int64_t M, int64_t N, int64_t K,
                                 int32_t* P, void* stream)
{
    using namespace wush;
    if (int e = ensure_init()) return e;
    WUSH_REQUIRE(M > 0 && N > 0 && K > 0 && K % 32 == 0, "group_partials: bad shape");
    WUSH_REQUIRE(xq && wq && P, "group_partials: null pointer");
    WUSH_REQUIRE(aligned16(xq) && aligned16(wq), "group_partials: codes must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    if (M > 32 && tc_supported(M, N, K)) {
        // same tcgen05 path as the tile GEMM; its bounded-wait error word lives in a
        // library-owned device int (this is a test op, the GEMM itself takes caller scratch)
        int* err = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&err, g_partials_err);
        if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        cudaMemsetAsync(err, 0, sizeof(int), st);
        return tc_partials(xq, wq, M, N, K, P, err, st);
    }
    if (K % 256 != 0) {
        dim3 grid((unsigned)((N + 31) / 32), (unsigned)((M + 7) / 8));
        w4a4_simple_kernel<true><<<grid, 256, 0, st>>>(xq, nullptr, wq, nullptr, nullptr, P, (int)M, (int)N, (int)K);
        return check_launch("group_partials(simple)");
    }
    return stream_partials(xq, wq, M, N, K, P, st);
}

WUSH_API int wush_i8_atom_selftest(const int8_t* a, const int8_t* b, int32_t* c, void* stream)
{
    using namespace wush;
    if (int e = ensure_init()) return e;
    WUSH_REQUIRE(a && b && c, "i8_atom_selftest: null pointer");
    i8_atom_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(a, b, c);
    return check_launch("i8_atom_selftest");
}
