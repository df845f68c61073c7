// One tcgen05.mma kind::i8 tile through the same plumbing the tile GEMM uses (C-ABI
// wush_i8_tile_selftest): a (128, 32) int8, b (n, 32) int8, d (128, n) int32 = a . b^T.
//
// It exists to pin, on the device, the pieces no compiler checks: the shared-memory matrix
// descriptor (K-major, no swizzle: 8x16-byte core matrices, leading/stride byte offsets), the
// instruction descriptor, TMEM allocation, tcgen05.commit -> mbarrier, and the lane/column
// mapping of tcgen05.ld.  Takes the place of the reference's one-atom check
// (csrc/gemm_s4.cu:50-82), at the granularity of the Blackwell instruction.
#include "common.cuh"
#include "tc_common.cuh"

namespace wush {

// layout_mode 0: leading offset = K-piece stride, stride offset = 8-row-block stride (the
// documented meaning); 1: the two swapped (kept only so a wrong reading of the descriptor
// shows up as "mode 1 passes, mode 0 fails" instead of as garbage in the GEMM).
__global__ void __launch_bounds__(128)
i8_tile_selftest_kernel(const int8_t* __restrict__ a, const int8_t* __restrict__ b, int32_t* __restrict__ d, int n,
                        int layout_mode, int* __restrict__ status)
{
    __shared__ __align__(128) uint8_t a_s[32 * 1024 + 256];   // oversized: every address either layout reading can form stays inside
    __shared__ __align__(128) uint8_t b_s[256 * 32];
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_slot;

    const int tid = threadIdx.x, warp = tid >> 5;
    // canonical K-major layout: 16-byte piece c of row r -> c * (rows*16) + (r/8)*128 + (r%8)*16
    {
        const uint4* src = reinterpret_cast<const uint4*>(a + tid * 32);
        *reinterpret_cast<uint4*>(a_s + 0 * (128 * 16) + (tid >> 3) * 128 + (tid & 7) * 16) = src[0];
        *reinterpret_cast<uint4*>(a_s + 1 * (128 * 16) + (tid >> 3) * 128 + (tid & 7) * 16) = src[1];
    }
    for (int r = tid; r < n; r += 128) {
        const uint4* src = reinterpret_cast<const uint4*>(b + r * 32);
        *reinterpret_cast<uint4*>(b_s + 0 * (n * 16) + (r >> 3) * 128 + (r & 7) * 16) = src[0];
        *reinterpret_cast<uint4*>(b_s + 1 * (n * 16) + (r >> 3) * 128 + (r & 7) * 16) = src[1];
    }
    tc::fence_proxy_async();                              // my generic writes -> async proxy
    if (tid == 0) {
        tc::mbar_init(&bar, 1);
        tc::mbar_fence_init();
    }
    uint32_t ncols = 32;
    while ((int)ncols < n) ncols <<= 1;
    if (warp == 0) {
        tc::tmem_alloc(&tmem_slot, ncols);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = tmem_slot;

    if (tid == 0) {
        uint32_t lbo_a = 128 * 16, sbo_a = 128, lbo_b = (uint32_t)n * 16, sbo_b = 128;
        if (layout_mode == 1) {
            uint32_t t = lbo_a; lbo_a = sbo_a; sbo_a = t;
            t = lbo_b; lbo_b = sbo_b; sbo_b = t;
        }
        const uint64_t adesc = tc::smem_desc_kmajor(tc::smem_u32(a_s), lbo_a, sbo_a);
        const uint64_t bdesc = tc::smem_desc_kmajor(tc::smem_u32(b_s), lbo_b, sbo_b);
        tc::mma_i8(tmem, adesc, bdesc, tc::idesc_i8(n), 0u);
        tc::mma_commit(&bar);
    }
    const bool ok = tc::mbar_wait(&bar, 0);
    if (!ok && tid == 0) atomicExch(status, 1);
    tc::tc_fence_after();
    if (ok) {
        for (int c0 = 0; c0 < n; c0 += 32) {
            uint32_t r[32];
            tc::tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
            tc::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (c0 + j < n) d[(size_t)tid * n + c0 + j] = (int32_t)r[j];
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem, ncols);
}

}  // namespace wush

WUSH_API int wush_i8_tile_selftest(const int8_t* a, const int8_t* b, int32_t* d, int n, int layout_mode, int* status,
                                   void* stream)
{
    using namespace wush;
    if (int e = ensure_init()) return e;
    WUSH_REQUIRE(a && b && d && status, "i8_tile_selftest: null pointer");
    WUSH_REQUIRE(n >= 16 && n <= 256 && n % 16 == 0, "i8_tile_selftest: n must be a multiple of 16 in [16, 256]");
    WUSH_REQUIRE(aligned16(a) && aligned16(b), "i8_tile_selftest: operands must be 16-byte aligned");
    WUSH_REQUIRE(layout_mode == 0 || (layout_mode == 1 && n <= 64),
                 "i8_tile_selftest: layout_mode is 0, or 1 with n <= 64");
    i8_tile_selftest_kernel<<<1, 128, 0, (cudaStream_t)stream>>>(a, b, d, n, layout_mode, status);
    return check_launch("i8_tile_selftest");
}
