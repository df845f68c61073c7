// Tensor-core streaming kernel for small batches (part of C-ABI wush_w4a4_gemm, variant
// DECODE; also the generic fallback for shapes the tcgen05 tile kernel does not take).
//
//   y[m][n] = sum_g sx[m][g] * sw[n][g] * P_g,   P_g exact int32 per 32-wide group
//
// Replaces the small-M branch of w4a4_gemm_s4 (csrc/gemm_s4.cu:346-347, TM=32 + split-K)
// and w4a4_gemv_multi for M > 4 (csrc/gemv_int4.cu:78-143) of the reference.
//
// Orientation: the WEIGHTS are the wide MMA operand.  A CTA of 8 warps owns 128 weight
// rows; each warp owns 16 of them (the M=16 side of mma.m16n8k32.s8) and all of the batch
// (1, 2 or 4 n-tiles of 8 activation rows).  K is walked in chunks of 16 groups:
//   * cp.async copies 16-byte pieces of packed codes and scales into a 4-deep ring of
//     shared-memory stages (rows padded to 272 B so that ldmatrix is conflict free);
//   * ldmatrix hands every lane the one 4-byte word of 8 nibbles it needs per row; one
//     shift and two ANDs turn it into two MMA registers of signed bytes (16 * code).  The
//     k order inside a group is permuted identically for both operands, which the dot
//     product does not see;
//   * one MMA per (group, n-tile) starts from zero, so its int32 result is 256 * P_g exactly;
//     it is scaled by sx*sw/256 and accumulated in fp32 registers.
// The weights are read from HBM once (M <= 32) in fully used 32-byte sectors.
//
// Also here: the exact-partial-sum test op (same kernel, PARTIALS mode), the one-atom
// self-test and a plain CUDA-core kernel for K that is not a multiple of 256.
#include "common.cuh"

namespace wush {

constexpr int MM_THREADS = 256;
constexpr int MM_ROWS = 128;           // weight rows per CTA
constexpr int MM_KC = 16;              // groups per stage
constexpr int MM_STAGES = 4;
constexpr int MM_PITCH = MM_KC * 16 + 16;   // bytes per staged row of codes

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    int bytes = valid ? 16 : 0;          // 0 -> the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(s));
}

__device__ __forceinline__ void mma_s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

template <int MT>
struct MmaSmem {
    static constexpr int XROWS = MT * 8;
    static constexpr int W_CODES = MM_ROWS * MM_PITCH;
    static constexpr int X_CODES = XROWS * MM_PITCH;
    static constexpr int W_SCALES = MM_ROWS * MM_KC * 2;
    static constexpr int X_SCALES = XROWS * MM_KC * 2;
    static constexpr int STAGE = W_CODES + X_CODES + W_SCALES + X_SCALES;
    static constexpr int TOTAL = STAGE * MM_STAGES;
};

// MT = number of 8-row activation tiles per CTA.  PARTIALS: write 256*P_g / 256 to `part`
// ([M][N][G] int32) instead of the scaled sum.
template <int MT, bool PARTIALS>
__global__ void __launch_bounds__(MM_THREADS, 1)
w4a4_mma_kernel(const uint8_t* __restrict__ xq, const __nv_bfloat16* __restrict__ xs,
                const uint8_t* __restrict__ wq, const __nv_bfloat16* __restrict__ ws,
                __half* __restrict__ y, int32_t* __restrict__ part, int M, int N, int K)
{
    using L = MmaSmem<MT>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gid = lane >> 2, tig = lane & 3;
    const int G = K >> 5;
    const size_t K2 = (size_t)K >> 1;
    const int n_chunks = (G + MM_KC - 1) / MM_KC;
    const int m_base = blockIdx.y * L::XROWS;
    const int n_blocks = (N + MM_ROWS - 1) / MM_ROWS;

    for (int nb = blockIdx.x; nb < n_blocks; nb += gridDim.x) {
        const int n_base = nb * MM_ROWS;

        auto load_stage = [&](int kc, int slot) {
            uint8_t* st = smem + (size_t)slot * L::STAGE;
            const int g0 = kc * MM_KC;
            // weight codes: 128 rows x 16 pieces
#pragma unroll
            for (int it = 0; it < MM_ROWS * MM_KC / MM_THREADS; ++it) {
                int c = it * MM_THREADS + tid, row = c >> 4, col = c & 15;
                int n = min(n_base + row, N - 1);
                bool ok = (g0 + col) < G;
                cp_async16(st + row * MM_PITCH + col * 16, wq + (size_t)n * K2 + (size_t)(ok ? g0 + col : 0) * 16, ok);
            }
            // activation codes: XROWS rows x 16 pieces
            for (int c = tid; c < L::XROWS * MM_KC; c += MM_THREADS) {
                int row = c >> 4, col = c & 15;
                int m = min(m_base + row, M - 1);
                bool ok = (g0 + col) < G;
                cp_async16(st + L::W_CODES + row * MM_PITCH + col * 16,
                           xq + (size_t)m * K2 + (size_t)(ok ? g0 + col : 0) * 16, ok);
            }
            // scales: rows of 16 bf16 = two 16-byte pieces (G % 8 == 0 is guaranteed by the host)
            {
                int row = tid >> 1, half = tid & 1;
                int n = min(n_base + row, N - 1);
                bool ok = (g0 + half * 8) < G;
                cp_async16(st + L::W_CODES + L::X_CODES + row * 32 + half * 16,
                           ws + (size_t)n * G + (ok ? g0 + half * 8 : 0), ok);
            }
            if (tid < L::XROWS * 2) {
                int row = tid >> 1, half = tid & 1;
                int m = min(m_base + row, M - 1);
                bool ok = (g0 + half * 8) < G;
                cp_async16(st + L::W_CODES + L::X_CODES + L::W_SCALES + row * 32 + half * 16,
                           xs + (size_t)m * G + (ok ? g0 + half * 8 : 0), ok);
            }
        };

        float acc[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;

#pragma unroll
        for (int s = 0; s < MM_STAGES - 1; ++s) {
            if (s < n_chunks) load_stage(s, s);
            cp_async_commit();
        }

        for (int kc = 0; kc < n_chunks; ++kc) {
            cp_async_wait<MM_STAGES - 2>();
            __syncthreads();                        // stage kc landed; stage kc-1 is free again
            {
                int nk = kc + MM_STAGES - 1;
                if (nk < n_chunks) load_stage(nk, nk % MM_STAGES);
                cp_async_commit();
            }
            const uint8_t* st = smem + (size_t)(kc % MM_STAGES) * L::STAGE;
            const uint8_t* wc = st + (warp * 16) * MM_PITCH;
            const uint8_t* xc = st + L::W_CODES;
            const unsigned short* wsc = reinterpret_cast<const unsigned short*>(st + L::W_CODES + L::X_CODES) + (warp * 16) * MM_KC;
            const unsigned short* xsc = reinterpret_cast<const unsigned short*>(st + L::W_CODES + L::X_CODES + L::W_SCALES);
            const int g_left = min(MM_KC, G - kc * MM_KC);

#pragma unroll
            for (int gb = 0; gb < MM_KC; gb += 4) {
                if (gb >= g_left) break;
                // A operand source words: [pair][r] -> pair p covers groups gb+2p, gb+2p+1
                uint32_t wa[2][4];
#pragma unroll
                for (int p = 0; p < 2; ++p)
                    ldmatrix_x4(wa[p], wc + ((lane & 7) + 8 * ((lane >> 3) & 1)) * MM_PITCH + (gb + 2 * p + (lane >> 4)) * 16);
                // B operand source words xb[gg][mt]
                uint32_t xb[4][MT];
                if constexpr (MT == 4) {
#pragma unroll
                    for (int gg = 0; gg < 4; ++gg) {
                        uint32_t r[4];
                        ldmatrix_x4(r, xc + lane * MM_PITCH + (gb + gg) * 16);
#pragma unroll
                        for (int mt = 0; mt < 4; ++mt) xb[gg][mt] = r[mt];
                    }
                } else if constexpr (MT == 2) {
#pragma unroll
                    for (int p = 0; p < 2; ++p) {
                        uint32_t r[4];
                        ldmatrix_x4(r, xc + (lane & 15) * MM_PITCH + (gb + 2 * p + (lane >> 4)) * 16);
                        xb[2 * p][0] = r[0]; xb[2 * p][1] = r[1];
                        xb[2 * p + 1][0] = r[2]; xb[2 * p + 1][1] = r[3];
                    }
                } else {
                    uint32_t r[4];
                    ldmatrix_x4(r, xc + (lane & 7) * MM_PITCH + (gb + (lane >> 3)) * 16);
#pragma unroll
                    for (int gg = 0; gg < 4; ++gg) xb[gg][0] = r[gg];
                }
#pragma unroll
                for (int gg = 0; gg < 4; ++gg) {
                    const int gl = gb + gg;                 // group inside the stage
                    if (gl < g_left) {
                        const uint32_t w_lo = wa[gg >> 1][(gg & 1) * 2 + 0];   // row gid
                        const uint32_t w_hi = wa[gg >> 1][(gg & 1) * 2 + 1];   // row gid + 8
                        uint32_t a0, a1, a2, a3;
                        unpack_x16(w_lo, a0, a2);
                        unpack_x16(w_hi, a1, a3);
                        const float swa = bf16_bits_to_f32(wsc[gid * MM_KC + gl]) * (1.0f / 256.0f);
                        const float swb = bf16_bits_to_f32(wsc[(gid + 8) * MM_KC + gl]) * (1.0f / 256.0f);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            uint32_t b0, b1;
                            unpack_x16(xb[gg][mt], b0, b1);
                            int c[4];
                            mma_s8_16832(c, a0, a1, a2, a3, b0, b1);
                            if constexpr (PARTIALS) {
                                const int g = kc * MM_KC + gl;
                                const int na = n_base + warp * 16 + gid, nbb = na + 8;
                                const int m0 = m_base + mt * 8 + tig * 2, m1 = m0 + 1;
                                if (m0 < M && na < N) part[((size_t)m0 * N + na) * G + g] = c[0] >> 8;
                                if (m1 < M && na < N) part[((size_t)m1 * N + na) * G + g] = c[1] >> 8;
                                if (m0 < M && nbb < N) part[((size_t)m0 * N + nbb) * G + g] = c[2] >> 8;
                                if (m1 < M && nbb < N) part[((size_t)m1 * N + nbb) * G + g] = c[3] >> 8;
                            } else {
                                const float sx0 = bf16_bits_to_f32(xsc[(mt * 8 + tig * 2) * MM_KC + gl]);
                                const float sx1 = bf16_bits_to_f32(xsc[(mt * 8 + tig * 2 + 1) * MM_KC + gl]);
                                acc[mt][0] = fmaf((float)c[0], swa * sx0, acc[mt][0]);
                                acc[mt][1] = fmaf((float)c[1], swa * sx1, acc[mt][1]);
                                acc[mt][2] = fmaf((float)c[2], swb * sx0, acc[mt][2]);
                                acc[mt][3] = fmaf((float)c[3], swb * sx1, acc[mt][3]);
                            }
                        }
                    }
                }
            }
        }
        cp_async_wait<0>();
        __syncthreads();                            // ring is idle before the next row block refills it

        if constexpr (!PARTIALS) {
            const int na = n_base + warp * 16 + gid, nbb = na + 8;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int m0 = m_base + mt * 8 + tig * 2, m1 = m0 + 1;
                if (m0 < M && na < N) y[(size_t)m0 * N + na] = __float2half_rn(acc[mt][0]);
                if (m1 < M && na < N) y[(size_t)m1 * N + na] = __float2half_rn(acc[mt][1]);
                if (m0 < M && nbb < N) y[(size_t)m0 * N + nbb] = __float2half_rn(acc[mt][2]);
                if (m1 < M && nbb < N) y[(size_t)m1 * N + nbb] = __float2half_rn(acc[mt][3]);
            }
        }
    }
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

template <int MT, bool PARTIALS>
static int launch_mma(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N,
                      int64_t K, void* y, int32_t* part, cudaStream_t st)
{
    using L = MmaSmem<MT>;
    const int n_blocks = (int)((N + MM_ROWS - 1) / MM_ROWS);
    const int m_blocks = (int)((M + L::XROWS - 1) / L::XROWS);
    int gx = n_blocks;
    if (m_blocks == 1 && gx > sm_count()) gx = sm_count();      // persistent over row blocks
    dim3 grid((unsigned)gx, (unsigned)m_blocks);
    w4a4_mma_kernel<MT, PARTIALS><<<grid, MM_THREADS, L::TOTAL, st>>>(
        xq, (const __nv_bfloat16*)xs, wq, (const __nv_bfloat16*)ws, (__half*)y, part, (int)M, (int)N, (int)K);
    return check_launch("w4a4_mma");
}

template <int MT, bool P>
static cudaError_t set_attr_one() {
    return cudaFuncSetAttribute(w4a4_mma_kernel<MT, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, MmaSmem<MT>::TOTAL);
}

int mma_set_attributes()
{
    cudaError_t e;
    if ((e = set_attr_one<1, false>()) != cudaSuccess || (e = set_attr_one<2, false>()) != cudaSuccess ||
        (e = set_attr_one<4, false>()) != cudaSuccess || (e = set_attr_one<4, true>()) != cudaSuccess)
        return fail(WUSH_ERR_CUDA, "mma: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    return WUSH_OK;
}

// Any M (grid.y walks blocks of 32 rows above 32).  K % 32 == 0.
int mma_dispatch(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N,
                 int64_t K, void* y, cudaStream_t st)
{
    if (K % 256 != 0 || M > 65535LL * 32) {
        dim3 grid((unsigned)((N + 31) / 32), (unsigned)((M + 7) / 8));
        if (grid.y > 65535) return fail(WUSH_ERR_UNSUPPORTED, "w4a4_gemm: M too large for the fallback kernel");
        w4a4_simple_kernel<false><<<grid, 256, 0, st>>>(xq, (const __nv_bfloat16*)xs, wq, (const __nv_bfloat16*)ws,
                                                        (__half*)y, nullptr, (int)M, (int)N, (int)K);
        return check_launch("w4a4_simple");
    }
    if (M <= 8) return launch_mma<1, false>(xq, xs, wq, ws, M, N, K, y, nullptr, st);
    if (M <= 16) return launch_mma<2, false>(xq, xs, wq, ws, M, N, K, y, nullptr, st);
    return launch_mma<4, false>(xq, xs, wq, ws, M, N, K, y, nullptr, st);
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
    if (K % 256 != 0) {
        dim3 grid((unsigned)((N + 31) / 32), (unsigned)((M + 7) / 8));
        w4a4_simple_kernel<true><<<grid, 256, 0, st>>>(xq, nullptr, wq, nullptr, nullptr, P, (int)M, (int)N, (int)K);
        return check_launch("group_partials(simple)");
    }
    // the scale pointers are still staged by the kernel: point them at the codes (16-byte
    // aligned, large enough: G*2 <= K/2 bytes per row) -- their values are never used here.
    return launch_mma<4, true>(xq, xq, wq, wq, M, N, K, nullptr, P, st);
}

WUSH_API int wush_i8_atom_selftest(const int8_t* a, const int8_t* b, int32_t* c, void* stream)
{
    using namespace wush;
    if (int e = ensure_init()) return e;
    WUSH_REQUIRE(a && b && c, "i8_atom_selftest: null pointer");
    i8_atom_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(a, b, c);
    return check_launch("i8_atom_selftest");
}
