// Per-tensor-scale route (C-ABI wush_quant_int4_tensor_scale, wush_w4a4_gemm_tensor_scale).
//
// Replaces quant_int4_tensor_scale{,_dev} (csrc/fast_path.cu:17-109) and
// w4a4_gemm_cutlass{,_dev} (csrc/gemm_cutlass_int4.cu:39-188) of the reference:
//   q = clamp(rint(x * inv_scale), -7, 7)           (fp32 multiply, no division)
//   y = fp16(alpha * sum_k qa*qw)                    (int32 accumulation over the whole K)
// The scalar may live in device memory so a captured graph can recompute it every replay.
#include "common.cuh"

namespace wush {

bool i8_tile_supported(int64_t M, int64_t N, int64_t K);
size_t i8_tile_workspace_bytes(int64_t M, int64_t N, int64_t K);
int i8_tile_dispatch(const uint8_t*, const uint8_t*, int64_t, int64_t, int64_t, float, const float*, void*, void*, size_t,
                     cudaStream_t);

__global__ void __launch_bounds__(256)
quant_ts_kernel(const uint4* __restrict__ x, uint32_t* __restrict__ q, float inv_host,
                const float* __restrict__ inv_dev, long long n_chunks)   // chunk = 8 bf16 -> 4 bytes
{
    const float inv = inv_dev ? __ldg(inv_dev) : inv_host;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < n_chunks; c += stride) {
        uint4 v = ldg_nc_v4(x + c);
        float f[8] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y),
                      bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w)};
        uint32_t w = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            int qi = __float2int_rn(__fmul_rn(f[e], inv));
            qi = max(-7, min(7, qi));
            w |= ((uint32_t)qi & 0xFu) << (4 * e);
        }
        q[c] = w;
    }
}

// Small shapes and callers without scratch: one thread per output with 16-byte loads and dp4a
// (exact int32).  Large M with scratch goes to the tcgen05 tile kernel (gemm_f16.cu).
__global__ void __launch_bounds__(256)
gemm_ts_kernel(const uint8_t* __restrict__ xq, const uint8_t* __restrict__ wq, __half* __restrict__ y,
               float alpha_host, const float* __restrict__ alpha_dev, int M, int N, int K)
{
    const int n = blockIdx.x * 32 + (threadIdx.x & 31);
    const int m = blockIdx.y * 8 + (threadIdx.x >> 5);
    if (n >= N || m >= M) return;
    const float alpha = alpha_dev ? __ldg(alpha_dev) : alpha_host;
    const uint4* xr = reinterpret_cast<const uint4*>(xq + (size_t)m * (K >> 1));
    const uint4* wr = reinterpret_cast<const uint4*>(wq + (size_t)n * (K >> 1));
    int acc = 0;                                        // holds 256 * sum: |sum| <= 64*K, fine for K < 2^17
    long long wide = 0;
    const int G = K >> 5;
    for (int g = 0; g < G; ++g) {
        uint4 a = xr[g], b = wr[g];
        uint32_t ae, ao, be, bo;
        int d = 0;
        unpack_x16(a.x, ae, ao); unpack_x16(b.x, be, bo); d = dp4a_s8(ae, be, d); d = dp4a_s8(ao, bo, d);
        unpack_x16(a.y, ae, ao); unpack_x16(b.y, be, bo); d = dp4a_s8(ae, be, d); d = dp4a_s8(ao, bo, d);
        unpack_x16(a.z, ae, ao); unpack_x16(b.z, be, bo); d = dp4a_s8(ae, be, d); d = dp4a_s8(ao, bo, d);
        unpack_x16(a.w, ae, ao); unpack_x16(b.w, be, bo); d = dp4a_s8(ae, be, d); d = dp4a_s8(ao, bo, d);
        acc += d >> 8;
        if ((g & 1023) == 1023) { wide += acc; acc = 0; }
    }
    wide += acc;
    y[(size_t)m * N + n] = __float2half_rn(__fmul_rn(alpha, (float)(int)wide));
}

}  // namespace wush

WUSH_API int wush_quant_int4_tensor_scale(const void* x, int64_t n, float inv_scale, const float* inv_scale_dev,
                                          uint8_t* q, void* stream)
{
    using namespace wush;
    if (int e = ensure_init()) return e;
    WUSH_REQUIRE(n >= 0 && n % 32 == 0, "quant_int4_tensor_scale: element count must be a multiple of 32");
    if (n == 0) return WUSH_OK;
    WUSH_REQUIRE(x && q, "quant_int4_tensor_scale: null pointer");
    WUSH_REQUIRE(aligned16(x) && (reinterpret_cast<uintptr_t>(q) & 3u) == 0, "quant_int4_tensor_scale: misaligned pointer");
    const long long chunks = n / 8;
    long long blocks = (chunks + 255) / 256;
    const long long cap = (long long)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    quant_ts_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const uint4*)x, (uint32_t*)q, inv_scale,
                                                                        inv_scale_dev, chunks);
    return check_launch("quant_int4_tensor_scale");
}

WUSH_API int wush_w4a4_gemm_tensor_scale(const uint8_t* xq, const uint8_t* wq, int64_t M, int64_t N, int64_t K,
                                         float alpha, const float* alpha_dev, void* y, void* stream)
{
    using namespace wush;
    if (int e = ensure_init()) return e;
    WUSH_REQUIRE(M >= 0 && N >= 0 && K > 0 && K % 32 == 0, "gemm_tensor_scale: bad shape");
    if (M == 0 || N == 0) return WUSH_OK;
    WUSH_REQUIRE(xq && wq && y, "gemm_tensor_scale: null pointer");
    WUSH_REQUIRE(aligned16(xq) && aligned16(wq), "gemm_tensor_scale: codes must be 16-byte aligned");
    WUSH_REQUIRE(K <= (1 << 24), "gemm_tensor_scale: K too large");
    dim3 grid((unsigned)((N + 31) / 32), (unsigned)((M + 7) / 8));
    WUSH_REQUIRE(grid.y <= 65535, "gemm_tensor_scale: M too large");
    gemm_ts_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(xq, wq, (__half*)y, alpha, alpha_dev, (int)M, (int)N, (int)K);
    return check_launch("gemm_tensor_scale");
}

// Rows from which the tensor-core tile route pays for its widening pre-pass.
static const int64_t TS_TILE_MIN_ROWS = 128;

WUSH_API size_t wush_w4a4_gemm_tensor_scale_workspace_bytes(int64_t M, int64_t N, int64_t K)
{
    using namespace wush;
    if (M < TS_TILE_MIN_ROWS || N <= 0 || K <= 0 || K > (1 << 18) || !i8_tile_supported(M, N, K)) return 0;
    return i8_tile_workspace_bytes(M, N, K);
}

WUSH_API int wush_w4a4_gemm_tensor_scale_ws(const uint8_t* xq, const uint8_t* wq, int64_t M, int64_t N, int64_t K, float alpha,
                                            const float* alpha_dev, void* y, void* workspace, size_t workspace_bytes,
                                            void* stream)
{
    using namespace wush;
    if (int e = ensure_init()) return e;
    const size_t need = wush_w4a4_gemm_tensor_scale_workspace_bytes(M, N, K);
    if (need == 0 || !workspace || workspace_bytes == 0)
        return wush_w4a4_gemm_tensor_scale(xq, wq, M, N, K, alpha, alpha_dev, y, stream);
    WUSH_REQUIRE(xq && wq && y, "gemm_tensor_scale: null pointer");
    WUSH_REQUIRE(aligned16(xq) && aligned16(wq), "gemm_tensor_scale: codes must be 16-byte aligned");
    return i8_tile_dispatch(xq, wq, M, N, K, alpha, alpha_dev, y, workspace, workspace_bytes, (cudaStream_t)stream);
}
