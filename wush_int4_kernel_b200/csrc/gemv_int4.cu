// Decode GEMV family, M <= 4 rows of activations (part of C-ABI wush_w4a4_gemm).
//
//   y[m][n] = sum_g sx[m][g] * sw[n][g] * P_g,   P_g = sum_{k in g} qa[m][k] * qw[n][k]
//
// Replaces w4a4_gemv_kernel / w4a4_gemv_multi_kernel of the reference
// (csrc/gemv_int4.cu:23-72, 78-143).  The job is to stream the packed weights and their
// scales exactly once at HBM rate; the arithmetic rides along on the CUDA cores:
//
//   * a CTA first expands the M activation rows into shared memory as signed bytes
//     (16 * code, even and odd codes of a group in separate 16-byte vectors, so lanes read
//     consecutive vectors without bank conflicts) and their scales as fp32 / 256;
//   * each warp owns one weight row per trip; lane l takes groups l, l+32, ...: one 16-byte
//     load of codes and one 2-byte load of the scale per group, eight groups (144 B per lane)
//     in flight before the first use; the next row's loads are issued before the reduction
//     of the current one, and the very first ones before the activation prologue;
//   * a word of 8 nibbles becomes two words of 4 signed bytes with one shift and two ANDs
//     (byte = 16 * code, no sign extension needed), then dp4a against the activation bytes:
//     the exact group sum comes out multiplied by 256, which the pre-scaled sx undoes;
//   * fp32 accumulation over groups per lane, xor-shuffle tree over lanes, fp16 store.
//
// The grid is persistent and sized by the occupancy calculator (every CTA resident), rows are
// dealt round-robin to the warps: with ~40 warps per SM the last round is ~97 % full.
// Algorithmic HBM bytes per call: 9*N*K/16 (codes + scales of W) + 9*M*K/16 + 2*M*N.
#include "common.cuh"

namespace wush {

constexpr int GV_THREADS = 256;
constexpr int GV_WARPS = GV_THREADS / 32;

// One weight row per warp and trip: lane l owns groups l, l+32, ... (8 per lane and trip, i.e.
// 144 B of loads in flight per lane).  FIRST is issued before the activation prologue so the
// weight stream starts while the CTA is still expanding x.
struct RowLoads {
    uint4 w[8];
    unsigned short s[8];
};

__device__ __forceinline__ void issue_row_loads(RowLoads& r, const uint8_t* __restrict__ wrow,
                                                const unsigned short* __restrict__ srow, int gb, int lane, int G)
{
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int g = gb + u * 32 + lane;
        if (g < G) {
            r.w[u] = ldg_nc_v4(wrow + (size_t)g * 16);
            r.s[u] = __ldg(srow + g);
        } else {
            r.w[u] = make_uint4(0, 0, 0, 0);
            r.s[u] = 0;
        }
    }
}

template <int MB>
__global__ void __launch_bounds__(GV_THREADS)
gemv_dp4a_kernel(const uint32_t* __restrict__ xq,          // (MB, K/8) words
                 const __nv_bfloat16* __restrict__ xs,     // (MB, G)
                 const uint8_t* __restrict__ wq,           // (N, K/2)
                 const __nv_bfloat16* __restrict__ ws,     // (N, G)
                 __half* __restrict__ y,                   // (MB, N)
                 int N, int K)
{
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int G = K >> 5;
    uint4* xe = reinterpret_cast<uint4*>(smem_raw);                    // [MB][G] even codes * 16
    uint4* xo = xe + (size_t)MB * G;                                   // [MB][G] odd codes * 16
    float* sxf = reinterpret_cast<float*>(xo + (size_t)MB * G);        // [MB][G] sx / 256

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t K2 = (size_t)K >> 1;
    const int stride = gridDim.x * GV_WARPS;
    int n = blockIdx.x * GV_WARPS + warp;
    const unsigned short* ws16 = reinterpret_cast<const unsigned short*>(ws);

    // start the weight stream first: it does not depend on x
    RowLoads cur;
    if (n < N) issue_row_loads(cur, wq + (size_t)n * K2, ws16 + (size_t)n * G, 0, lane, G);

    for (int idx = threadIdx.x; idx < MB * G; idx += GV_THREADS) {
        uint4 w = *reinterpret_cast<const uint4*>(xq + (size_t)idx * 4);
        uint4 e, o;
        unpack_x16(w.x, e.x, o.x); unpack_x16(w.y, e.y, o.y);
        unpack_x16(w.z, e.z, o.z); unpack_x16(w.w, e.w, o.w);
        xe[idx] = e; xo[idx] = o;
        sxf[idx] = __bfloat162float(xs[idx]) * (1.0f / 256.0f);
    }
    __syncthreads();

    for (; n < N; n += stride) {
        const uint8_t* wrow = wq + (size_t)n * K2;
        const unsigned short* srow = ws16 + (size_t)n * G;
        float acc[MB];
#pragma unroll
        for (int m = 0; m < MB; ++m) acc[m] = 0.f;
        for (int gb = 0; gb < G; gb += 256) {
            if (gb) issue_row_loads(cur, wrow, srow, gb, lane, G);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int g = min(gb + u * 32 + lane, G - 1);          // lanes past the end carry zero weights
                uint4 ae, ao;
                unpack_x16(cur.w[u].x, ae.x, ao.x); unpack_x16(cur.w[u].y, ae.y, ao.y);
                unpack_x16(cur.w[u].z, ae.z, ao.z); unpack_x16(cur.w[u].w, ae.w, ao.w);
                const float sw = bf16_bits_to_f32(cur.s[u]);
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    const uint4 ve = xe[m * G + g], vo = xo[m * G + g];
                    int d = dp4a_s8(ae.x, ve.x, 0); d = dp4a_s8(ao.x, vo.x, d);
                    d = dp4a_s8(ae.y, ve.y, d); d = dp4a_s8(ao.y, vo.y, d);
                    d = dp4a_s8(ae.z, ve.z, d); d = dp4a_s8(ao.z, vo.z, d);
                    d = dp4a_s8(ae.w, ve.w, d); d = dp4a_s8(ao.w, vo.w, d);
                    acc[m] = fmaf((float)d, sxf[m * G + g] * sw, acc[m]);
                }
            }
        }
        // next row's first trip goes out before the reduction of this one
        const int nn = n + stride;
        if (nn < N) issue_row_loads(cur, wq + (size_t)nn * K2, ws16 + (size_t)nn * G, 0, lane, G);
#pragma unroll
        for (int m = 0; m < MB; ++m) {
#pragma unroll
            for (int off = 16; off; off >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], off);
        }
        if (lane == 0) {
#pragma unroll
            for (int m = 0; m < MB; ++m) y[(size_t)m * N + n] = __float2half_rn(acc[m]);
        }
    }
}

size_t gemv_smem_bytes(int M, int64_t K) { return (size_t)M * (K / 32) * (16 + 16 + 4); }

template <int MB>
static int launch_gemv(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t N,
                       int64_t K, void* y, cudaStream_t st)
{
    const size_t smem = gemv_smem_bytes(MB, K);
    // resident CTAs per SM for this shared-memory size (a host-side query, cached per size)
    static thread_local size_t cached_smem = ~size_t(0);
    static thread_local int cached_per_sm = 1;
    if (cached_smem != smem) {
        int q = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&q, gemv_dp4a_kernel<MB>, GV_THREADS, smem) != cudaSuccess || q < 1) q = 1;
        cached_smem = smem;
        cached_per_sm = q;
    }
    const int per_sm = cached_per_sm;
    // persistent grid: every CTA resident at once, rows dealt round-robin to the warps
    long long ctas = (long long)sm_count() * per_sm;
    const long long needed = (N + GV_WARPS - 1) / GV_WARPS;
    if (ctas > needed) ctas = needed;
    gemv_dp4a_kernel<MB><<<(unsigned)ctas, GV_THREADS, smem, st>>>((const uint32_t*)xq, (const __nv_bfloat16*)xs, wq,
                                                                   (const __nv_bfloat16*)ws, (__half*)y, (int)N, (int)K);
    return check_launch("gemv_dp4a");
}

int gemv_set_attributes()
{
    const int max_smem = 200 * 1024;
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(gemv_dp4a_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem)) != cudaSuccess ||
        (e = cudaFuncSetAttribute(gemv_dp4a_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem)) != cudaSuccess ||
        (e = cudaFuncSetAttribute(gemv_dp4a_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem)) != cudaSuccess ||
        (e = cudaFuncSetAttribute(gemv_dp4a_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem)) != cudaSuccess)
        return fail(WUSH_ERR_CUDA, "gemv: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    return WUSH_OK;
}

// M in 1..4, shared memory must fit (checked by the dispatcher).
int gemv_dispatch(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N,
                  int64_t K, void* y, cudaStream_t st)
{
    switch (M) {
        case 1: return launch_gemv<1>(xq, xs, wq, ws, N, K, y, st);
        case 2: return launch_gemv<2>(xq, xs, wq, ws, N, K, y, st);
        case 3: return launch_gemv<3>(xq, xs, wq, ws, N, K, y, st);
        case 4: return launch_gemv<4>(xq, xs, wq, ws, N, K, y, st);
    }
    return fail(WUSH_ERR_INVALID_ARGUMENT, "gemv: M=%lld outside 1..4", (long long)M);
}

}  // namespace wush
