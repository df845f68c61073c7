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
//   * each warp owns TWO weight rows at a time; lane l takes groups l, l+32, ...:
//     one 16-byte load of codes and one 2-byte load of the scale per row and group, four
//     groups in flight per lane before the first use (>= 128 B per lane outstanding);
//   * a word of 8 nibbles becomes two words of 4 signed bytes with one shift and two ANDs
//     (byte = 16 * code, no sign extension needed), then dp4a against the activation bytes:
//     the exact group sum comes out multiplied by 256, which the pre-scaled sx undoes;
//   * fp32 accumulation over groups per lane, xor-shuffle tree over lanes, fp16 store.
//
// The grid is persistent: a whole number of CTAs per SM, each looping over row pairs, so the
// activation expansion is paid once per CTA.
// Algorithmic HBM bytes per call: 9*N*K/16 (codes + scales of W) + 9*M*K/16 + 2*M*N.
#include "common.cuh"

namespace wush {

constexpr int GV_THREADS = 256;
constexpr int GV_WARPS = GV_THREADS / 32;

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

    for (int idx = threadIdx.x; idx < MB * G; idx += GV_THREADS) {
        uint4 w = *reinterpret_cast<const uint4*>(xq + (size_t)idx * 4);
        uint4 e, o;
        unpack_x16(w.x, e.x, o.x); unpack_x16(w.y, e.y, o.y);
        unpack_x16(w.z, e.z, o.z); unpack_x16(w.w, e.w, o.w);
        xe[idx] = e; xo[idx] = o;
        sxf[idx] = __bfloat162float(xs[idx]) * (1.0f / 256.0f);
    }
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_pairs = (N + 1) >> 1;
    const size_t K2 = (size_t)K >> 1;

    for (int pair = blockIdx.x * GV_WARPS + warp; pair < n_pairs; pair += gridDim.x * GV_WARPS) {
        const int n0 = pair * 2;
        const int n1 = min(n0 + 1, N - 1);
        const uint8_t* w0 = wq + (size_t)n0 * K2;
        const uint8_t* w1 = wq + (size_t)n1 * K2;
        const unsigned short* s0 = reinterpret_cast<const unsigned short*>(ws) + (size_t)n0 * G;
        const unsigned short* s1 = reinterpret_cast<const unsigned short*>(ws) + (size_t)n1 * G;
        float acc0[MB], acc1[MB];
#pragma unroll
        for (int m = 0; m < MB; ++m) acc0[m] = acc1[m] = 0.f;

        for (int gb = 0; gb < G; gb += 128) {               // 4 groups per lane per trip
            uint4 wa[4], wb[4];
            float sa[4], sb[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int g = gb + u * 32 + lane;
                if (g < G) {
                    wa[u] = ldg_nc_v4(w0 + (size_t)g * 16);
                    wb[u] = ldg_nc_v4(w1 + (size_t)g * 16);
                    sa[u] = bf16_bits_to_f32(__ldg(s0 + g));
                    sb[u] = bf16_bits_to_f32(__ldg(s1 + g));
                } else {
                    wa[u] = wb[u] = make_uint4(0, 0, 0, 0);
                    sa[u] = sb[u] = 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int g = min(gb + u * 32 + lane, G - 1);   // clamped lanes carry zero weights
                uint4 ae, ao, be, bo;
                unpack_x16(wa[u].x, ae.x, ao.x); unpack_x16(wa[u].y, ae.y, ao.y);
                unpack_x16(wa[u].z, ae.z, ao.z); unpack_x16(wa[u].w, ae.w, ao.w);
                unpack_x16(wb[u].x, be.x, bo.x); unpack_x16(wb[u].y, be.y, bo.y);
                unpack_x16(wb[u].z, be.z, bo.z); unpack_x16(wb[u].w, be.w, bo.w);
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    const uint4 ve = xe[m * G + g], vo = xo[m * G + g];
                    int d0 = dp4a_s8(ae.x, ve.x, 0); d0 = dp4a_s8(ao.x, vo.x, d0);
                    d0 = dp4a_s8(ae.y, ve.y, d0); d0 = dp4a_s8(ao.y, vo.y, d0);
                    d0 = dp4a_s8(ae.z, ve.z, d0); d0 = dp4a_s8(ao.z, vo.z, d0);
                    d0 = dp4a_s8(ae.w, ve.w, d0); d0 = dp4a_s8(ao.w, vo.w, d0);
                    int d1 = dp4a_s8(be.x, ve.x, 0); d1 = dp4a_s8(bo.x, vo.x, d1);
                    d1 = dp4a_s8(be.y, ve.y, d1); d1 = dp4a_s8(bo.y, vo.y, d1);
                    d1 = dp4a_s8(be.z, ve.z, d1); d1 = dp4a_s8(bo.z, vo.z, d1);
                    d1 = dp4a_s8(be.w, ve.w, d1); d1 = dp4a_s8(bo.w, vo.w, d1);
                    const float sx = sxf[m * G + g];
                    acc0[m] = fmaf((float)d0, sx * sa[u], acc0[m]);
                    acc1[m] = fmaf((float)d1, sx * sb[u], acc1[m]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MB; ++m) {
#pragma unroll
            for (int off = 16; off; off >>= 1) {
                acc0[m] += __shfl_xor_sync(0xffffffffu, acc0[m], off);
                acc1[m] += __shfl_xor_sync(0xffffffffu, acc1[m], off);
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                y[(size_t)m * N + n0] = __float2half_rn(acc0[m]);
                if (n0 + 1 < N) y[(size_t)m * N + n0 + 1] = __float2half_rn(acc1[m]);
            }
        }
    }
}

size_t gemv_smem_bytes(int M, int64_t K) { return (size_t)M * (K / 32) * (16 + 16 + 4); }

template <int MB>
static int launch_gemv(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t N,
                       int64_t K, void* y, cudaStream_t st)
{
    const size_t smem = gemv_smem_bytes(MB, K);
    const int n_pairs = (int)((N + 1) / 2);
    int ctas = (n_pairs + GV_WARPS - 1) / GV_WARPS;
    const int resident = sm_count() * (smem > 64 * 1024 ? 1 : (smem > 24 * 1024 ? 2 : 4));
    if (ctas > resident) ctas = resident;
    gemv_dp4a_kernel<MB><<<ctas, GV_THREADS, smem, st>>>((const uint32_t*)xq, (const __nv_bfloat16*)xs, wq,
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
