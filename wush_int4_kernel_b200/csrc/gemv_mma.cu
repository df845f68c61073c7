// Decode product for a few activation rows with the weights streamed from global memory straight
// into tensor-core fragments (part of C-ABI wush_w4a4_gemm, variant GEMV_MMA; 2 < M <= 16).
//
//   y[m][n] = sum_g sx[m][g] * sw[n][g] * P_g,   P_g = sum_{k in g} qa[m][k] * qw[n][k]   (exact int32)
//
// Replaces w4a4_gemv_multi_kernel of the reference (csrc/gemv_int4.cu:78-143) for these M.  Like the
// CUDA-core GEMV the kernel has no shared-memory staging of the weights, no barriers and no producer
// warp: a warp owns 16 weight rows, every lane keeps a ring of 16-byte loads in flight and reloads a
// slot as soon as it is consumed.  What differs is who does the dot products:
//
//   * A lane's 16-byte load is ONE GROUP of one row (32 codes): lane (gid, tig) holds group 4s + tig of
//     row gid (and of row gid + 8) in step s.  An mma.m16n8k32.s8 takes its 32 k-slots from the four
//     lanes of a quad, eight from each -- so one MMA sees eight codes of FOUR different groups.  The
//     groups are kept apart on the other operand: the 8 columns of an MMA are 2 activation rows x 4
//     groups, and column (m, t) carries activation codes only in the k-slots that lane tig = t feeds
//     (zeros elsewhere).  Four MMAs (one per 32-bit word of the 16 bytes) chained through the
//     accumulator give the exact sums of 16 rows x 4 groups x 2 activation rows; three quarters of the
//     multiplies hit zeros, which the tensor pipe has to spare at these sizes (M = 8: 16 MMAs per
//     kilobyte of weights, 26 us of tensor time against 39 us of HBM time on the 70B layer).
//   * No transposition, no ldmatrix, no widening of the activations in the loop: a CTA expands the
//     activations once into shared memory in exactly the layout the column fragments need
//     ([step][row][group][word] -> (even codes, odd codes) x 16); only the 8 lanes of a warp whose column
//     is theirs read it (64 contiguous bytes), the other 24 read one zero word in other banks.
//   * The accumulator chain starts from the bit pattern of 1.5 * 2^23, so the sums arrive as fp32
//     12582912 + 256 * P and t = fma(f, sw, -12582912 * sw), acc = fma(t, sx, acc) apply both scales
//     without any conversion.  A lane's output pair is (group t, group t + 1) of one row and one
//     activation row: weight scales and activation scales are natural register pairs for the packed
//     fp32x2 FMAs (one 4-byte load of two bf16 weight scales per row and step).
//
//   * The ring of loads lives in shared memory, not in registers: every lane copies its own 16-byte pieces
//     with cp.async into slots only it reads (no barrier, no other lane involved), eight steps = 320 B per
//     lane ahead.  In registers such a ring allows four steps at 16 warps, and the kernel then waits on
//     memory latency: 13 warps x 5 KB in flight per multiprocessor are not enough for the HBM rate.
//
// Needs K % 128 == 0 (whole steps of four groups) and the activation table (M' * K * 17/16 bytes, M' = M
// rounded up to even) plus 10 KB per warp in shared memory.
// Algorithmic HBM bytes per call: 9*N*K/16 (codes + scales of W) + 9*M*K/16 + 2*M*N.
#include "common.cuh"

namespace wush {

namespace {

constexpr int GM_MAX_WARPS = 16;
constexpr int GM_DEPTH = 8;                        // steps (of 4 groups = 64 B per row) in flight per lane
constexpr int GM_RING_BYTES = GM_DEPTH * (1024 + 256);   // per warp: the lanes' own slots in shared memory
constexpr int GM_ROW = 136;                        // bytes of one activation row of a step: 4 groups x 32 B, + 8 so that two rows miss each other's banks
constexpr uint32_t GM_MAGIC_BITS = 0x4B400000u;    // 1.5 * 2^23 as fp32
constexpr float GM_MAGIC = 12582912.0f;

// Bytes of one step's block of the activation table: MP rows, rounded to 32 bytes so that every block (and the zero
// words behind the tables) starts on the same bank modulo 8 -- the bank argument at the reads relies on it.
__host__ __device__ constexpr int gm_block(int mp) { return (mp * GM_ROW + 31) / 32 * 32; }

__device__ __forceinline__ void mma_s8_acc(uint32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Asynchronous copies global -> shared of this thread's own bytes.  `after` is a value the copy must not overtake:
// the slot it overwrites was read into registers by this thread, and a use of those registers as an operand keeps
// the copy behind the arrival of that read.
__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, uint32_t after) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem), "r"(after) : "memory");
}
__device__ __forceinline__ void cp_async_4(void* smem, const void* gmem, uint32_t after) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem), "r"(after) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory"); }

// Where this lane's loads of a step come from: its group of rows gid and gid + 8 of a unit and its pair of scales.
struct LoadCursor {
    const uint8_t *wa, *wb;
    const uint32_t *sa, *sb;
    int unit, step;
};

__device__ __forceinline__ void cursor_to_unit(LoadCursor& c, const uint8_t* __restrict__ wq, const unsigned short* __restrict__ ws16,
                                               int unit, int gid, int tig, int N, int G, size_t K2, int units)
{
    c.unit = unit;
    c.step = 0;
    // rows past the end are read from the last row (valid memory) and never stored
    const int u = unit < units ? unit : 0;
    const int ra = min(u * 16 + gid, N - 1), rb = min(u * 16 + gid + 8, N - 1);
    c.wa = wq + (size_t)ra * K2 + tig * 16;
    c.wb = wq + (size_t)rb * K2 + tig * 16;
    c.sa = reinterpret_cast<const uint32_t*>(ws16 + (size_t)ra * G + 2 * (tig & 1));
    c.sb = reinterpret_cast<const uint32_t*>(ws16 + (size_t)rb * G + 2 * (tig & 1));
}

// Q chains of MMAs per step: activation rows 2q and 2q + 1.
template <int Q>
__global__ void __launch_bounds__(GM_MAX_WARPS * 32, 1)
gemv_mma_kernel(const uint32_t* __restrict__ xq,          // (M, K/8) words
                const __nv_bfloat16* __restrict__ xs,     // (M, G)
                const uint8_t* __restrict__ wq,           // (N, K/2)
                const __nv_bfloat16* __restrict__ ws,     // (N, G)
                __half* __restrict__ y,                   // (M, N)
                int M, int N, int K)
{
    constexpr int MP = 2 * Q, BLK = gm_block(MP), SXB = MP * 16;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int G = K >> 5, S = G >> 2;
    uint8_t* tbl = smem_raw;                               // [S][MP rows of GM_ROW]: (even, odd) words of 4 groups x 4 words
    uint8_t* sxt = tbl + (size_t)S * BLK;                  // [S][MP][4] fp32: sx / 256
    uint8_t* zero = sxt + (size_t)S * SXB;                 // BLK + 32 bytes of zeros
    uint8_t* rings = zero + BLK + 32;                      // per warp: [GM_DEPTH][2][32] 16 B of codes, [GM_DEPTH][32] 2 x 4 B of scales

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int gid = lane >> 2, tig = lane & 3;
    const size_t K2 = (size_t)K >> 1;
    const int units = (N + 15) >> 4;
    const int stride = gridDim.x * warps;
    int unit = blockIdx.x * warps + warp;
    const unsigned short* ws16 = reinterpret_cast<const unsigned short*>(ws);
    uint4* ring_w = reinterpret_cast<uint4*>(rings + (size_t)warp * GM_RING_BYTES) + lane;
    uint2* ring_s = reinterpret_cast<uint2*>(rings + (size_t)warp * GM_RING_BYTES + GM_DEPTH * 1024) + lane;

    pdl_wait();

    // start the weight stream first: it does not depend on the shared-memory prologue.  One commit group per step,
    // also for steps past the end of the warp's work, so that "all but the newest GM_DEPTH - 1 groups" is always the
    // step about to be consumed.
    LoadCursor lc;
    cursor_to_unit(lc, wq, ws16, unit, gid, tig, N, G, K2, units);
    const auto load_next = [&](int d, uint32_t after) {
        if (lc.unit < units) {
            cp_async_16(ring_w + (d * 2 + 0) * 32, lc.wa + (size_t)lc.step * 64, after);
            cp_async_16(ring_w + (d * 2 + 1) * 32, lc.wb + (size_t)lc.step * 64, after);
            cp_async_4(&ring_s[d * 32].x, lc.sa + lc.step * 2, after);
            cp_async_4(&ring_s[d * 32].y, lc.sb + lc.step * 2, after);
            if (++lc.step == S) cursor_to_unit(lc, wq, ws16, lc.unit + stride, gid, tig, N, G, K2, units);
        }
        cp_async_commit();
    };
#pragma unroll
    for (int d = 0; d < GM_DEPTH; ++d) load_next(d, 0u);

    // ---- activations into fragment order -------------------------------------------------------
    for (int idx = threadIdx.x; idx < MP * G; idx += blockDim.x) {
        const int m = idx / G, g = idx - m * G;
        uint4 w = make_uint4(0, 0, 0, 0);
        float sx = 0.f;
        if (m < M) {
            w = *reinterpret_cast<const uint4*>(xq + ((size_t)m * G + g) * 4);
            sx = __bfloat162float(xs[(size_t)m * G + g]) * (1.0f / 256.0f);
        }
        uint2* dst = reinterpret_cast<uint2*>(tbl + (size_t)(g >> 2) * BLK + m * GM_ROW + (g & 3) * 32);
        uint2 v;
        unpack_x16(w.x, v.x, v.y); dst[0] = v;
        unpack_x16(w.y, v.x, v.y); dst[1] = v;
        unpack_x16(w.z, v.x, v.y); dst[2] = v;
        unpack_x16(w.w, v.x, v.y); dst[3] = v;
        reinterpret_cast<float*>(sxt + (size_t)(g >> 2) * SXB + m * 16)[g & 3] = sx;
    }
    for (int idx = threadIdx.x; idx < (BLK + 32) / 4; idx += blockDim.x) reinterpret_cast<uint32_t*>(zero)[idx] = 0u;
    __syncthreads();
    pdl_launch_dependents();            // a dependent may become resident as this grid drains; it waits before reading y

    // the column of this lane in every MMA is (activation row gid >> 2 of the chain, group gid & 3 of the step): its
    // k-slots carry codes only if they are the slots this lane's own group feeds on the weight side
    const bool mine = tig == (gid & 3);
    const int col_off = (gid >> 2) * GM_ROW + tig * 32;
    const uint8_t* const zero_at = zero + 16;              // 4 banks away from what the 8 reading lanes touch
    const uint8_t* const sx_at = sxt + (tig >> 1) * 16 + (tig & 1) * 8;

    float2 acc[Q][2];
#pragma unroll
    for (int q = 0; q < Q; ++q) acc[q][0] = acc[q][1] = make_float2(0.f, 0.f);
    int step = 0;
    while (unit < units) {
#pragma unroll
        for (int d = 0; d < GM_DEPTH; ++d) {
            if (unit >= units) break;
            cp_async_wait<GM_DEPTH - 1>();
            const uint4 wa = ring_w[(d * 2 + 0) * 32], wb = ring_w[(d * 2 + 1) * 32];
            const uint2 sc = ring_s[d * 32];
            uint32_t ea[4], oa[4], eb[4], ob[4];
            unpack_x16(wa.x, ea[0], oa[0]); unpack_x16(wa.y, ea[1], oa[1]);
            unpack_x16(wa.z, ea[2], oa[2]); unpack_x16(wa.w, ea[3], oa[3]);
            unpack_x16(wb.x, eb[0], ob[0]); unpack_x16(wb.y, eb[1], ob[1]);
            unpack_x16(wb.z, eb[2], ob[2]); unpack_x16(wb.w, eb[3], ob[3]);
            const float2 swa = make_float2(bf16_lo(sc.x), bf16_hi(sc.x));
            const float2 swb = make_float2(bf16_lo(sc.y), bf16_hi(sc.y));
            // the slot has been read: it takes the step GM_DEPTH ahead, in this unit or one of the warp's next
            load_next(d, ea[0] ^ eb[0] ^ sc.x ^ sc.y);
            const float2 ca = make_float2(-GM_MAGIC * swa.x, -GM_MAGIC * swa.y);         // exact: 2 x 8 significant bits
            const float2 cb = make_float2(-GM_MAGIC * swb.x, -GM_MAGIC * swb.y);
            const uint8_t* bp = mine ? tbl + (size_t)step * BLK + col_off : zero_at;
            const uint8_t* sp = sx_at + (size_t)step * SXB;
            // the Q chains advance together, word by word: Q independent accumulators hide the MMA latency
            uint32_t dd[Q][4];
#pragma unroll
            for (int q = 0; q < Q; ++q) dd[q][0] = dd[q][1] = dd[q][2] = dd[q][3] = GM_MAGIC_BITS;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
                for (int q = 0; q < Q; ++q) {
                    const uint2 b = *reinterpret_cast<const uint2*>(bp + q * 2 * GM_ROW + c * 8);
                    mma_s8_acc(dd[q], ea[c], eb[c], oa[c], ob[c], b.x, b.y);
                }
            }
#pragma unroll
            for (int q = 0; q < Q; ++q) {
                const float2 x = *reinterpret_cast<const float2*>(sp + q * 32);
                const float2 fa = make_float2(__uint_as_float(dd[q][0]), __uint_as_float(dd[q][1]));
                const float2 fb = make_float2(__uint_as_float(dd[q][2]), __uint_as_float(dd[q][3]));
                acc[q][0] = __ffma2_rn(__ffma2_rn(fa, swa, ca), x, acc[q][0]);
                acc[q][1] = __ffma2_rn(__ffma2_rn(fb, swb, cb), x, acc[q][1]);
            }
            if (++step == S) {
                // the unit is complete.  A lane holds, for activation row 2q + (tig >> 1), the sums over the groups
                // = 2 (tig & 1) and + 1 (mod 4) of rows gid and gid + 8; its neighbour tig ^ 1 holds the other two
                const int na = unit * 16 + gid, nb = na + 8;
#pragma unroll
                for (int q = 0; q < Q; ++q) {
                    float va = acc[q][0].x + acc[q][0].y, vb = acc[q][1].x + acc[q][1].y;
                    va += __shfl_xor_sync(0xffffffffu, va, 1);     // two addends: the same sum in both lanes of the pair
                    vb += __shfl_xor_sync(0xffffffffu, vb, 1);
                    const int m = 2 * q + (tig >> 1);
                    if ((tig & 1) == 0 && m < M) {
                        if (na < N) y[(size_t)m * N + na] = __float2half_rn(va);
                        if (nb < N) y[(size_t)m * N + nb] = __float2half_rn(vb);
                    }
                    acc[q][0] = acc[q][1] = make_float2(0.f, 0.f);
                }
                step = 0;
                unit += stride;
            }
        }
    }
    cp_async_wait<0>();                                    // nothing of this thread is in flight when the CTA's memory goes back
}

constexpr size_t GM_SMEM_MAX = 227 * 1024;

size_t table_bytes(int Q, int64_t K)                      // activation codes, activation scales, zero words
{
    const int64_t S = K / 128, MP = 2 * Q, blk = gm_block((int)MP);
    return (size_t)(S * blk + S * MP * 16 + blk + 32);
}

int warps_that_fit(int Q, int64_t K)
{
    const size_t t = table_bytes(Q, K);
    if (t + GM_RING_BYTES > GM_SMEM_MAX) return 0;
    const size_t w = (GM_SMEM_MAX - t) / GM_RING_BYTES;
    return w > GM_MAX_WARPS ? GM_MAX_WARPS : (int)w;
}

// Warps per CTA (one CTA per multiprocessor), at most `limit`.  A layer of at most one round of units is spread
// over all multiprocessors; a longer one gets the warp count whose rounds, dealt round-robin, come out fullest.
int pick_warps(int64_t units, int limit)
{
    const int sms = sm_count();
    if (units <= (int64_t)sms * limit) return (int)((units + sms - 1) / sms);
    int best = limit;
    double best_score = -1.0;
    for (int w = limit < 8 ? limit : 8; w <= limit; ++w) {
        const double rounds = (double)units / ((double)sms * w);
        const double whole = (double)(long long)(rounds + 0.999999);
        const double score = rounds / whole + 0.003 * w;
        if (score > best_score) { best_score = score; best = w; }
    }
    return best;
}

constexpr int chains_for(int64_t M) { return M <= 8 ? (int)((M + 1) / 2) : M <= 12 ? 6 : 8; }

template <int Q>
int launch(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N, int64_t K, void* y,
           cudaStream_t st)
{
    const int64_t units = (N + 15) / 16;
    const int warps = pick_warps(units, warps_that_fit(Q, K));
    int64_t ctas = (units + warps - 1) / warps;
    if (ctas > sm_count()) ctas = sm_count();
    cudaError_t e = launch_dependent(gemv_mma_kernel<Q>, dim3((unsigned)ctas), dim3(warps * 32),
                                     table_bytes(Q, K) + (size_t)warps * GM_RING_BYTES, st,
                                     (const uint32_t*)xq, (const __nv_bfloat16*)xs, wq, (const __nv_bfloat16*)ws, (__half*)y,
                                     (int)M, (int)N, (int)K);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "gemv_mma launch: %s", cudaGetErrorString(e));
    return WUSH_OK;
}

template <int Q>
cudaError_t set_attr() {
    return cudaFuncSetAttribute(gemv_mma_kernel<Q>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GM_SMEM_MAX);
}

}  // namespace

int gemv_mma_set_attributes()
{
    cudaError_t e;
    if ((e = set_attr<1>()) != cudaSuccess || (e = set_attr<2>()) != cudaSuccess || (e = set_attr<3>()) != cudaSuccess ||
        (e = set_attr<4>()) != cudaSuccess || (e = set_attr<6>()) != cudaSuccess || (e = set_attr<8>()) != cudaSuccess)
        return fail(WUSH_ERR_CUDA, "gemv_mma: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    return WUSH_OK;
}

// 1 <= M <= 16, whole steps of four groups, the activation table and at least four warps' rings in shared memory,
// 4-byte aligned scale pairs.
bool gemv_mma_supported(int64_t M, int64_t N, int64_t K, const void* xs, const void* ws)
{
    if (M < 1 || M > 16 || N < 1 || K % 128 != 0) return false;
    return warps_that_fit(chains_for(M), K) >= 4 && (reinterpret_cast<uintptr_t>(ws) & 3) == 0 && xs != nullptr;
}

int gemv_mma_dispatch(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N, int64_t K,
                      void* y, cudaStream_t st)
{
    switch (chains_for(M)) {
        case 1: return launch<1>(xq, xs, wq, ws, M, N, K, y, st);
        case 2: return launch<2>(xq, xs, wq, ws, M, N, K, y, st);
        case 3: return launch<3>(xq, xs, wq, ws, M, N, K, y, st);
        case 4: return launch<4>(xq, xs, wq, ws, M, N, K, y, st);
        case 6: return launch<6>(xq, xs, wq, ws, M, N, K, y, st);
        case 8: return launch<8>(xq, xs, wq, ws, M, N, K, y, st);
    }
    return fail(WUSH_ERR_INVALID_ARGUMENT, "gemv_mma: M=%lld outside 1..16", (long long)M);
}

}  // namespace wush
