// Weight-streaming tensor-core kernel for decode batches (C-ABI wush_w4a4_gemm, variant
// DECODE; also the fallback for large M when the tile GEMM does not take the shape).
//
//   y[m][n] = sum_g sx[m][g] * sw[n][g] * P_g,   P_g exact int32 per 32-wide group
//
// Replaces w4a4_gemv / w4a4_gemv_multi (csrc/gemv_int4.cu:23-143) and the small-M, split-K
// branch of w4a4_gemm_s4 (csrc/gemm_s4.cu:346-347) of the reference.  The job is to pull
// 9/16 byte per weight element out of HBM exactly once, at HBM rate, for 1..32 activation
// rows; the arithmetic must fit in the shadow of that stream.
//
//   * The WEIGHTS are the wide MMA operand: a CTA owns 128 weight rows, each of its 8 compute
//     warps 16 of them (the M=16 side of mma.m16n8k32.s8) against 1, 2 or 4 tiles of 8
//     activation rows.
//   * A ninth warp is the producer: per stage of 8 groups it issues four TMA tile loads
//     (packed weight codes and activation codes with 128-byte swizzle, the two bf16 scale
//     tiles) into a 4-deep ring; full/empty mbarriers, bounded waits.  Two CTAs fit per SM,
//     so ~150 KB of loads are in flight per SM and the grid needs no persistence.
//   * ldmatrix on the swizzled tile hands every lane the one 4-byte word of 8 nibbles it
//     needs per row (conflict free); one shift and two ANDs make two MMA registers of
//     signed bytes (16 * code).  The k order inside a group is permuted identically for both
//     operands.
//   * No integer->float conversion is executed: the MMA accumulates onto the bit pattern of
//     1.5 * 2^23, so its int32 result read as fp32 is 12582912 + 256 * P_g, and
//         t = fma(f, sw, -12582912 * sw)   (exact, = 256 * P_g * sw)
//         acc = fma(t, sx, acc)
//     applies both scales with two FMAs per output and group; 1/256 is applied once at the end.
//
// Algorithmic HBM bytes: 9*N*K/16 (weights) + 9*M*K/16 (activations, L2 resident) + 2*M*N.
#include "common.cuh"
#include "tc_common.cuh"
#include "tc_host.cuh"

namespace wush {

__device__ int g_device_flag;                       // library-owned error word of the streaming kernels

namespace {

constexpr int ST_ROWS = 128, ST_KS = 8, ST_STAGES = 4;
constexpr int ST_COMPUTE_WARPS = 8, ST_THREADS = (ST_COMPUTE_WARPS + 1) * 32;
constexpr uint32_t MAGIC_BITS = 0x4B400000u;
constexpr float MAGIC = 12582912.0f;

template <int MT>
struct StreamSmem {
    static constexpr int XROWS = MT * 8;
    static constexpr int WC = 0;                                   // 128 rows x 128 B, swizzled
    static constexpr int XC = WC + ST_ROWS * 128;                  // XROWS x 128 B, swizzled
    static constexpr int WS = XC + 4096;                           // 128 rows x 8 bf16
    static constexpr int XS = WS + ST_ROWS * 16;                   // XROWS x 8 bf16
    static constexpr int STAGE = ((XS + XROWS * 16 + 1023) / 1024) * 1024;
    static constexpr int TX = ST_ROWS * 128 + XROWS * 128 + ST_ROWS * 16 + XROWS * 16;
    static constexpr int BARS = ST_STAGES * STAGE;
    static constexpr int TOTAL = BARS + 2 * ST_STAGES * 8 + 1024;  // + alignment slack
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(tc::smem_u32(smem)));
}

// D = A * B + bias pattern (all four accumulators start at the bits of 1.5 * 2^23)
__device__ __forceinline__ void mma_s8_biased(uint32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(MAGIC_BITS));
}

// bf16 element e (0..7) of a 16-byte vector of scales, as fp32
__device__ __forceinline__ float scale_of(const uint4& v, int e) {
    const uint32_t w = (e < 2) ? v.x : (e < 4) ? v.y : (e < 6) ? v.z : v.w;
    return (e & 1) ? bf16_hi(w) : bf16_lo(w);
}

template <int MT, bool PARTIALS>
__global__ void __launch_bounds__(ST_THREADS, 2)
w4a4_stream_kernel(const __grid_constant__ CUtensorMap map_wq, const __grid_constant__ CUtensorMap map_xq,
                   const __grid_constant__ CUtensorMap map_ws, const __grid_constant__ CUtensorMap map_xs,
                   __half* __restrict__ y, int32_t* __restrict__ part, int M, int N, int K)
{
    using L = StreamSmem<MT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BARS);
    uint64_t* empty = full + ST_STAGES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = K >> 5, n_chunks = G / ST_KS;
    const int n_base = blockIdx.x * ST_ROWS, m_base = blockIdx.y * L::XROWS;

    if (tid == 0) {
        for (int i = 0; i < ST_STAGES; ++i) { tc::mbar_init(&full[i], 1); tc::mbar_init(&empty[i], ST_COMPUTE_WARPS); }
        tc::mbar_fence_init();
    }
    __syncthreads();

    if (warp == ST_COMPUTE_WARPS) {
        // ------------------------------ producer ----------------------------------------------
        if (lane == 0) {
            tc::prefetch_tensormap(&map_wq); tc::prefetch_tensormap(&map_xq);
            tc::prefetch_tensormap(&map_ws); tc::prefetch_tensormap(&map_xs);
            uint32_t slot = 0, phase = 0;
            int issued = 0;
            bool ok = true;
            for (int kc = 0; kc < n_chunks; ++kc) {
                if (!tc::mbar_wait(&empty[slot], phase ^ 1)) { ok = false; break; }
                uint8_t* st = smem + slot * L::STAGE;
                tc::mbar_expect_tx(&full[slot], L::TX);
                tc::tma_load_2d(st + L::WC, &map_wq, &full[slot], kc * 128, n_base);
                tc::tma_load_2d(st + L::XC, &map_xq, &full[slot], kc * 128, m_base);
                tc::tma_load_2d(st + L::WS, &map_ws, &full[slot], kc * ST_KS, n_base);
                tc::tma_load_2d(st + L::XS, &map_xs, &full[slot], kc * ST_KS, m_base);
                ++issued;
                if (++slot == ST_STAGES) { slot = 0; phase ^= 1; }
            }
            if (!ok) {
                atomicExch(&g_device_flag, 1);
                // copies already issued must land before the CTA's memory is given back
                for (int i = 0; i < (issued < ST_STAGES ? issued : ST_STAGES); ++i)
                    for (uint32_t spin = 0; spin < (1u << 16); ++spin)
                        if (tc::mbar_try_wait(&full[i], 0) || tc::mbar_try_wait(&full[i], 1)) break;
            }
        }
        return;
    }

    // ---------------------------------- compute warps -------------------------------------------
    const int gid = lane >> 2, tig = lane & 3;
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;

    // ldmatrix row addresses (the 128-byte swizzle XORs the 16-byte piece index with row & 7)
    const int w_row = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);        // matrices 0/2: rows 0-7, 1/3: rows 8-15
    const int w_gsel = lane >> 4;                                             // matrices 2,3 take the next group
    uint32_t slot = 0, phase = 0;
    bool ok = true;
    for (int kc = 0; kc < n_chunks; ++kc) {
        if (!tc::mbar_wait(&full[slot], phase)) { ok = false; break; }
        const uint8_t* st = smem + slot * L::STAGE;
        const uint8_t* wc = st + L::WC + w_row * 128;
        const uint8_t* xc = st + L::XC;
        // scales of the whole stage: 8 groups = one 16-byte vector per row
        const uint4 swa = *reinterpret_cast<const uint4*>(st + L::WS + (warp * 16 + gid) * 16);
        const uint4 swb = *reinterpret_cast<const uint4*>(st + L::WS + (warp * 16 + gid + 8) * 16);
        uint4 sx0[MT], sx1[MT];
        if constexpr (!PARTIALS) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                sx0[mt] = *reinterpret_cast<const uint4*>(st + L::XS + (mt * 8 + tig * 2) * 16);
                sx1[mt] = *reinterpret_cast<const uint4*>(st + L::XS + (mt * 8 + tig * 2 + 1) * 16);
            }
        }
#pragma unroll
        for (int gq = 0; gq < ST_KS; gq += 4) {
            // activation words for 4 groups: xb[group][m-tile]
            uint32_t xb[4][MT];
            if constexpr (MT == 4) {
#pragma unroll
                for (int gg = 0; gg < 4; ++gg) {
                    uint32_t r[4];
                    ldsm_x4(r, xc + lane * 128 + (((gq + gg) ^ (lane & 7)) << 4));
#pragma unroll
                    for (int mt = 0; mt < 4; ++mt) xb[gg][mt] = r[mt];
                }
            } else if constexpr (MT == 2) {
#pragma unroll
                for (int p = 0; p < 2; ++p) {
                    uint32_t r[4];
                    ldsm_x4(r, xc + (lane & 15) * 128 + (((gq + 2 * p + (lane >> 4)) ^ (lane & 7)) << 4));
                    xb[2 * p][0] = r[0]; xb[2 * p][1] = r[1];
                    xb[2 * p + 1][0] = r[2]; xb[2 * p + 1][1] = r[3];
                }
            } else {
                uint32_t r[4];
                ldsm_x4(r, xc + (lane & 7) * 128 + (((gq + (lane >> 3)) ^ (lane & 7)) << 4));
#pragma unroll
                for (int gg = 0; gg < 4; ++gg) xb[gg][0] = r[gg];
            }
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                uint32_t wa[4];
                ldsm_x4(wa, wc + (((gq + 2 * p + w_gsel) ^ (lane & 7)) << 4));
#pragma unroll
                for (int gg2 = 0; gg2 < 2; ++gg2) {
                    const int gl = gq + 2 * p + gg2;              // group inside the stage (compile-time)
                    uint32_t a0, a1, a2, a3;
                    unpack_x16(wa[gg2 * 2 + 0], a0, a2);          // row gid:     even codes, odd codes
                    unpack_x16(wa[gg2 * 2 + 1], a1, a3);          // row gid + 8
                    float s_a, s_b, c_a, c_b;
                    if constexpr (!PARTIALS) {
                        s_a = scale_of(swa, gl); s_b = scale_of(swb, gl);
                        c_a = -MAGIC * s_a; c_b = -MAGIC * s_b;   // exact: 2 x 8 significant bits
                    }
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        uint32_t b0, b1, d[4];
                        unpack_x16(xb[2 * p + gg2][mt], b0, b1);
                        mma_s8_biased(d, a0, a1, a2, a3, b0, b1);
                        if constexpr (PARTIALS) {
                            const int g = kc * ST_KS + gl;
                            const int na = n_base + warp * 16 + gid, nb = na + 8;
                            const int m0 = m_base + mt * 8 + tig * 2, m1 = m0 + 1;
                            if (m0 < M && na < N) part[((size_t)m0 * N + na) * G + g] = (int32_t)(d[0] - MAGIC_BITS) >> 8;
                            if (m1 < M && na < N) part[((size_t)m1 * N + na) * G + g] = (int32_t)(d[1] - MAGIC_BITS) >> 8;
                            if (m0 < M && nb < N) part[((size_t)m0 * N + nb) * G + g] = (int32_t)(d[2] - MAGIC_BITS) >> 8;
                            if (m1 < M && nb < N) part[((size_t)m1 * N + nb) * G + g] = (int32_t)(d[3] - MAGIC_BITS) >> 8;
                        } else {
                            const float x0 = scale_of(sx0[mt], gl), x1 = scale_of(sx1[mt], gl);
                            acc[mt][0] = fmaf(fmaf(__uint_as_float(d[0]), s_a, c_a), x0, acc[mt][0]);
                            acc[mt][1] = fmaf(fmaf(__uint_as_float(d[1]), s_a, c_a), x1, acc[mt][1]);
                            acc[mt][2] = fmaf(fmaf(__uint_as_float(d[2]), s_b, c_b), x0, acc[mt][2]);
                            acc[mt][3] = fmaf(fmaf(__uint_as_float(d[3]), s_b, c_b), x1, acc[mt][3]);
                        }
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&empty[slot]);
        if (++slot == ST_STAGES) { slot = 0; phase ^= 1; }
    }
    if (!ok) {
        if (lane == 0) atomicExch(&g_device_flag, 2);
        return;
    }
    if constexpr (!PARTIALS) {
        const int na = n_base + warp * 16 + gid, nb = na + 8;
        const float k = 1.0f / 256.0f;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int m0 = m_base + mt * 8 + tig * 2, m1 = m0 + 1;
            if (m0 < M && na < N) y[(size_t)m0 * N + na] = __float2half_rn(acc[mt][0] * k);
            if (m1 < M && na < N) y[(size_t)m1 * N + na] = __float2half_rn(acc[mt][1] * k);
            if (m0 < M && nb < N) y[(size_t)m0 * N + nb] = __float2half_rn(acc[mt][2] * k);
            if (m1 < M && nb < N) y[(size_t)m1 * N + nb] = __float2half_rn(acc[mt][3] * k);
        }
    }
}

template <int MT, bool PARTIALS>
int launch_stream(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N, int64_t K,
                  void* y, int32_t* part, cudaStream_t st)
{
    using L = StreamSmem<MT>;
    CUtensorMap mwq, mxq, mws, mxs;
    int s;
    if ((s = make_map_2d(&mwq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, K / 2, N, 128, ST_ROWS, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
    if ((s = make_map_2d(&mxq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, K / 2, M, 128, L::XROWS, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
    if ((s = make_map_2d(&mws, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ws, K / 32, N, ST_KS, ST_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE))) return s;
    if ((s = make_map_2d(&mxs, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, xs, K / 32, M, ST_KS, L::XROWS, CU_TENSOR_MAP_SWIZZLE_NONE))) return s;
    dim3 grid((unsigned)((N + ST_ROWS - 1) / ST_ROWS), (unsigned)((M + L::XROWS - 1) / L::XROWS));
    if (grid.y > 65535) return fail(WUSH_ERR_UNSUPPORTED, "w4a4_gemm(decode): M too large");
    w4a4_stream_kernel<MT, PARTIALS><<<grid, ST_THREADS, L::TOTAL, st>>>(mwq, mxq, mws, mxs, (__half*)y, part, (int)M,
                                                                         (int)N, (int)K);
    return check_launch("w4a4_stream");
}

template <int MT, bool P>
cudaError_t set_attr() {
    return cudaFuncSetAttribute(w4a4_stream_kernel<MT, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, StreamSmem<MT>::TOTAL);
}

}  // namespace

int stream_set_attributes()
{
    if (int s = resolve_tensor_map_encoder()) return s;
    cudaError_t e;
    if ((e = set_attr<1, false>()) != cudaSuccess || (e = set_attr<2, false>()) != cudaSuccess ||
        (e = set_attr<4, false>()) != cudaSuccess || (e = set_attr<4, true>()) != cudaSuccess)
        return fail(WUSH_ERR_CUDA, "decode kernel: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    return WUSH_OK;
}

// Whole TMA stages only (K % 256 == 0) and 16-byte aligned scale rows/pointers.
bool stream_supported(int64_t K, const void* xs, const void* ws)
{
    return K % 256 == 0 && aligned16(xs) && aligned16(ws);
}

int stream_dispatch(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N, int64_t K,
                    void* y, cudaStream_t st)
{
    if (M <= 8) return launch_stream<1, false>(xq, xs, wq, ws, M, N, K, y, nullptr, st);
    if (M <= 16) return launch_stream<2, false>(xq, xs, wq, ws, M, N, K, y, nullptr, st);
    return launch_stream<4, false>(xq, xs, wq, ws, M, N, K, y, nullptr, st);
}

int stream_partials(const uint8_t* xq, const uint8_t* wq, int64_t M, int64_t N, int64_t K, int32_t* P, cudaStream_t st)
{
    // the scale tiles are still fetched; the codes are readable, aligned and large enough
    return launch_stream<4, true>(xq, xq, wq, wq, M, N, K, nullptr, P, st);
}

}  // namespace wush

WUSH_API int wush_device_flag(int* flag)
{
    using namespace wush;
    if (int e = ensure_init()) return e;
    WUSH_REQUIRE(flag, "device_flag: null pointer");
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(flag, g_device_flag, sizeof(int));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_device_flag, &zero, sizeof(int));
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "device_flag: %s", cudaGetErrorString(e));
    return WUSH_OK;
}
