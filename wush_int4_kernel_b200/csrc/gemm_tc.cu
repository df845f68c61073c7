// Prefill tile GEMM on the 5th-generation tensor cores (C-ABI wush_w4a4_gemm, variant TILE).
//
//   Y[m][n] = sum_g sx[m][g] * sw[n][g] * P_g[m][n],   P_g = sum_{k in group g} qa * qw
//
// Replaces w4a4_gemm_s4_kernel<TM> of the reference (csrc/gemm_s4.cu:106-318), whose
// mma.m8n8k32.s4 atom exists on sm_75 only.  sm_100 has no 4-bit integer MMA, so the codes
// are widened to signed bytes in shared memory and every 32-wide group is one
// tcgen05.mma kind::i8 instruction (M=128, N=128, K=32).  Bytes hold 16 * code, so the exact
// group sum arrives as 256 * P_g.  TMEM holds four 128x128 int32 accumulators in rotation, so
// the tensor core runs up to four groups ahead of the epilogue.
//
// Integer -> float conversion runs on the XU pipe at 1/8 rate on this architecture and would
// be the bottleneck, so it is never executed: each accumulator buffer is pre-loaded with the
// bit pattern of 1.5 * 2^23 and the MMA ACCUMULATES onto it.  The int32 result
// 0x4B400000 + 256*P is, read as fp32, exactly 12582912 + 256*P, and
//     t   = fma(f, sw, -12582912 * sw)              (exact: equals 256 * P * sw, <= 20 significant bits)
//     sum = fma(t, sx/256, sum)
// gives the scaled contribution with two FMAs, issued as packed fp32x2 instructions.  The
// epilogue stores the bias pattern back (tcgen05.st) right after reading a buffer.
//
// One persistent CTA per SM, four warpgroups with fixed roles (registers are re-balanced
// between them with setmaxnreg; warps 2-3 only donate theirs):
//   warp 0      TMA producer: per stage of 8 groups, four tile loads (packed activation and
//               weight codes with 128-byte swizzle, the two bf16 scale tiles) -> mbarrier tx
//   warps 4-7   widen: packed nibbles -> signed bytes in the canonical K-major core-matrix
//               layout (one shift, two ANDs per 8 codes; even codes form the first 16-byte
//               K piece, odd codes the second -- the same permutation on both operands);
//               they also lay the weight scales out as bf16 [group][n] and the activation
//               scales as fp32 / 256
//   warp 1      issues the MMAs (one thread), owns TMEM; tcgen05.commit frees the byte slot
//               and publishes the accumulator
//   warps 8-15  epilogue: tcgen05.ld 16 columns at a time (next load in flight while the
//               current one is scaled), re-arm with tcgen05.st, packed FMAs, fp16 stores at the end.
//               Thread = output row m, so sx is a per-thread scalar and sw a broadcast vector.
// Every wait is bounded; a timeout sets an error word, aborts the CTA's loops and still
// frees TMEM.
//
// The CUDA cores still do two FMAs per (m, n, group) against 32 tensor-core MACs, so this
// kernel is bound by the scaling epilogue (fp32 pipe), not by the MMA rate:
// that is the price of exact per-group bf16 scales on an architecture without a
// group-scaled integer MMA.
#include "common.cuh"
#include "tc_common.cuh"
#include "tc_host.cuh"

namespace wush {
namespace {

constexpr int BM = 128, BN = 128, KS = 8;                 // tile, groups per TMA stage
constexpr int PK_STAGES = 3, UNP_SLOTS = 8, ACC_BUFS = 4, SC_SLOTS = 4;
constexpr int TC_THREADS = 512;                           // four warpgroups: control, widen, epilogue x2
constexpr int CONV_WARP0 = 4, CONV_WARPS = 4, EPI_WARP0 = 8, EPI_WARPS = 8;
// registers per thread after the warpgroups trade them: 128 * (32 + 80 + 200 + 200) = 65536
constexpr int REGS_CTRL = 32, REGS_CONV = 80, REGS_EPI = 200;

constexpr int PKA_BYTES = BM * 128, PKB_BYTES = BN * 128, PKSX_BYTES = BM * 16, PKSW_BYTES = BN * 16;
constexpr int STAGE_TX = PKA_BYTES + PKB_BYTES + PKSX_BYTES + PKSW_BYTES;
constexpr int UNA_BYTES = BM * 32, UNB_BYTES = BN * 32;
constexpr int SCX_BYTES = BM * KS * 4, SCW_BYTES = KS * BN * 2;       // SCX: fp32 [row][group]/256, SCW: bf16 [group][n]
constexpr uint32_t MAGIC_BITS = 0x4B400000u;                         // fp32 12582912.0 = 1.5 * 2^23
constexpr float MAGIC = 12582912.0f;

struct SmemLayout {
    static constexpr int PKA = 0;
    static constexpr int PKB = PKA + PK_STAGES * PKA_BYTES;
    static constexpr int PKSX = PKB + PK_STAGES * PKB_BYTES;
    static constexpr int PKSW = PKSX + PK_STAGES * PKSX_BYTES;
    static constexpr int UNA = PKSW + PK_STAGES * PKSW_BYTES;
    static constexpr int UNB = UNA + UNP_SLOTS * UNA_BYTES;
    static constexpr int SCX = UNB + UNP_SLOTS * UNB_BYTES;
    static constexpr int SCW = SCX + SC_SLOTS * SCX_BYTES;
    static constexpr int BARS = SCW + SC_SLOTS * SCW_BYTES;
    static constexpr int NBARS = 2 * PK_STAGES + 2 * UNP_SLOTS + 2 * ACC_BUFS + 2 * SC_SLOTS + 1;
    static constexpr int MISC = BARS + NBARS * 8;
    static constexpr int TOTAL = MISC + 16 + 1024;        // + slack for the 1024-byte alignment
};

struct Ring {                      // running position in a ring of `n` slots
    uint32_t idx = 0, phase = 0;
    __device__ __forceinline__ void next(uint32_t n) { if (++idx == n) { idx = 0; phase ^= 1; } }
};

// bounded wait that also gives up when another role has already aborted
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < WUSH_SPIN_LIMIT; ++i) {
        if (tc::mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    return false;
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_st16_const(uint32_t taddr, uint32_t v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr), "r"(v)
        : "memory");
}
template <int N> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <bool PARTIALS>
__global__ void __launch_bounds__(TC_THREADS, 1)
w4a4_tc_kernel(const __grid_constant__ CUtensorMap map_xq, const __grid_constant__ CUtensorMap map_wq,
               const __grid_constant__ CUtensorMap map_xs, const __grid_constant__ CUtensorMap map_ws,
               __half* __restrict__ y, int32_t* __restrict__ part, int M, int N, int K, int* __restrict__ err)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    using L = SmemLayout;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);
    uint64_t* pk_full = bars;
    uint64_t* pk_empty = pk_full + PK_STAGES;
    uint64_t* un_full = pk_empty + PK_STAGES;
    uint64_t* un_empty = un_full + UNP_SLOTS;
    uint64_t* acc_full = un_empty + UNP_SLOTS;
    uint64_t* acc_empty = acc_full + ACC_BUFS;
    uint64_t* sc_full = acc_empty + ACC_BUFS;
    uint64_t* sc_empty = sc_full + SC_SLOTS;
    uint64_t* done_bar = sc_empty + SC_SLOTS;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::MISC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::MISC + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = K >> 5, n_stages = G / KS;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN, n_tiles = tiles_m * tiles_n;

    if (tid == 0) {
        for (int i = 0; i < PK_STAGES; ++i) { tc::mbar_init(&pk_full[i], 1); tc::mbar_init(&pk_empty[i], CONV_WARPS); }
        for (int i = 0; i < UNP_SLOTS; ++i) { tc::mbar_init(&un_full[i], CONV_WARPS); tc::mbar_init(&un_empty[i], 1); }
        for (int i = 0; i < ACC_BUFS; ++i) { tc::mbar_init(&acc_full[i], 1); tc::mbar_init(&acc_empty[i], EPI_WARPS); }
        for (int i = 0; i < SC_SLOTS; ++i) { tc::mbar_init(&sc_full[i], CONV_WARPS); tc::mbar_init(&sc_empty[i], EPI_WARPS); }
        tc::mbar_init(done_bar, 1);
        *abort_flag = 0;
        tc::mbar_fence_init();
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, ACC_BUFS * BN);          // 512 columns: the whole TMEM of the SM
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------------------
        reg_dec<REGS_CTRL>();
        if (lane == 0) {
            tc::prefetch_tensormap(&map_xq); tc::prefetch_tensormap(&map_wq);
            tc::prefetch_tensormap(&map_xs); tc::prefetch_tensormap(&map_ws);
            Ring pk;
            uint32_t issued = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
                for (int ks = 0; ks < n_stages; ++ks) {
                    if (!wait_bar(&pk_empty[pk.idx], pk.phase ^ 1, abort_flag)) { ok = false; break; }
                    tc::mbar_expect_tx(&pk_full[pk.idx], STAGE_TX);
                    tc::tma_load_2d(smem + L::PKA + pk.idx * PKA_BYTES, &map_xq, &pk_full[pk.idx], ks * 128, m0);
                    tc::tma_load_2d(smem + L::PKB + pk.idx * PKB_BYTES, &map_wq, &pk_full[pk.idx], ks * 128, n0);
                    tc::tma_load_2d(smem + L::PKSX + pk.idx * PKSX_BYTES, &map_xs, &pk_full[pk.idx], ks * KS, m0);
                    tc::tma_load_2d(smem + L::PKSW + pk.idx * PKSW_BYTES, &map_ws, &pk_full[pk.idx], ks * KS, n0);
                    ++issued;
                    pk.next(PK_STAGES);
                }
            }
            if (!ok) {
                *abort_flag = 1;
                atomicExch(err, 1);
                // let the copies already in flight land before this CTA gives its memory back
                Ring q = pk;
                for (uint32_t i = 0; i < (issued < (uint32_t)PK_STAGES ? issued : (uint32_t)PK_STAGES); ++i) {
                    q.idx = (q.idx + PK_STAGES - 1) % PK_STAGES;
                    for (uint32_t spin = 0; spin < (1u << 16); ++spin)
                        if (tc::mbar_try_wait(&pk_full[q.idx], 0) || tc::mbar_try_wait(&pk_full[q.idx], 1)) break;
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ----------------------------------------------
        reg_dec<REGS_CTRL>();
        if (lane == 0) {
            Ring un, acc;
            bool ok = true;
            const uint32_t idesc = tc::idesc_i8(BN);
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                for (int g = 0; g < G; ++g) {
                    if (!wait_bar(&un_full[un.idx], un.phase, abort_flag) ||
                        !wait_bar(&acc_empty[acc.idx], acc.phase, abort_flag)) { ok = false; break; }
                    tc::tc_fence_after();
                    const uint64_t adesc = tc::smem_desc_kmajor(tc::smem_u32(smem + L::UNA + un.idx * UNA_BYTES), BM * 16, 128);
                    const uint64_t bdesc = tc::smem_desc_kmajor(tc::smem_u32(smem + L::UNB + un.idx * UNB_BYTES), BN * 16, 128);
                    tc::mma_i8(tmem + acc.idx * BN, adesc, bdesc, idesc, 1u);   // onto the bias pattern
                    tc::mma_commit(&un_empty[un.idx]);
                    tc::mma_commit(&acc_full[acc.idx]);
                    un.next(UNP_SLOTS);
                    acc.next(ACC_BUFS);
                }
            }
            if (!ok) { *abort_flag = 1; atomicExch(err, 2); }
            tc::mma_commit(done_bar);                       // everything issued so far has retired
            for (uint32_t spin = 0; spin < WUSH_SPIN_LIMIT; ++spin)
                if (tc::mbar_try_wait(done_bar, 0)) break;
        }
    } else if (warp < CONV_WARP0) {
        reg_dec<REGS_CTRL>();                               // warps 2 and 3 only donate their registers
    } else if (warp < EPI_WARP0) {
        // ------------------------------ widen nibbles -> bytes ------------------------------------
        reg_dec<REGS_CONV>();
        const int row = (warp - CONV_WARP0) * 32 + lane;    // 0..127: one activation row and one weight row
        Ring pk, un, sc;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
            for (int ks = 0; ks < n_stages && ok; ++ks) {
                if (!wait_bar(&pk_full[pk.idx], pk.phase, abort_flag) ||
                    !wait_bar(&sc_empty[sc.idx], sc.phase ^ 1, abort_flag)) { ok = false; break; }
                {   // scales of this stage: activations as fp32 [row][8], weights as fp32/256 [group][n]
                    const uint4 vx = *reinterpret_cast<const uint4*>(smem + L::PKSX + pk.idx * PKSX_BYTES + row * 16);
                    float4* dx = reinterpret_cast<float4*>(smem + L::SCX + sc.idx * SCX_BYTES + row * 32);
                    const float k = 1.0f / 256.0f;           // undoes the 16 x 16 of the widened codes
                    dx[0] = make_float4(bf16_lo(vx.x) * k, bf16_hi(vx.x) * k, bf16_lo(vx.y) * k, bf16_hi(vx.y) * k);
                    dx[1] = make_float4(bf16_lo(vx.z) * k, bf16_hi(vx.z) * k, bf16_lo(vx.w) * k, bf16_hi(vx.w) * k);
                    const uint4 vw = *reinterpret_cast<const uint4*>(smem + L::PKSW + pk.idx * PKSW_BYTES + row * 16);
                    unsigned short* dw = reinterpret_cast<unsigned short*>(smem + L::SCW + sc.idx * SCW_BYTES) + row;
                    dw[0 * BN] = (unsigned short)(vw.x & 0xffffu); dw[1 * BN] = (unsigned short)(vw.x >> 16);
                    dw[2 * BN] = (unsigned short)(vw.y & 0xffffu); dw[3 * BN] = (unsigned short)(vw.y >> 16);
                    dw[4 * BN] = (unsigned short)(vw.z & 0xffffu); dw[5 * BN] = (unsigned short)(vw.z >> 16);
                    dw[6 * BN] = (unsigned short)(vw.w & 0xffffu); dw[7 * BN] = (unsigned short)(vw.w >> 16);
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(&sc_full[sc.idx]);
                    sc.next(SC_SLOTS);
                }
                const uint8_t* pa = smem + L::PKA + pk.idx * PKA_BYTES + row * 128;
                const uint8_t* pb = smem + L::PKB + pk.idx * PKB_BYTES + row * 128;
                const int dst_off = (row >> 3) * 128 + (row & 7) * 16;
#pragma unroll 1
                for (int j = 0; j < KS; ++j) {
                    if (!wait_bar(&un_empty[un.idx], un.phase ^ 1, abort_flag)) { ok = false; break; }
                    const int chunk = (j ^ (row & 7)) << 4;                 // 128-byte swizzle of the TMA tile
                    const uint4 a = *reinterpret_cast<const uint4*>(pa + chunk);
                    const uint4 b = *reinterpret_cast<const uint4*>(pb + chunk);
                    uint4 ae, ao, be, bo;
                    unpack_x16(a.x, ae.x, ao.x); unpack_x16(a.y, ae.y, ao.y);
                    unpack_x16(a.z, ae.z, ao.z); unpack_x16(a.w, ae.w, ao.w);
                    unpack_x16(b.x, be.x, bo.x); unpack_x16(b.y, be.y, bo.y);
                    unpack_x16(b.z, be.z, bo.z); unpack_x16(b.w, be.w, bo.w);
                    uint8_t* ua = smem + L::UNA + un.idx * UNA_BYTES + dst_off;
                    uint8_t* ub = smem + L::UNB + un.idx * UNB_BYTES + dst_off;
                    *reinterpret_cast<uint4*>(ua) = ae;
                    *reinterpret_cast<uint4*>(ua + BM * 16) = ao;
                    *reinterpret_cast<uint4*>(ub) = be;
                    *reinterpret_cast<uint4*>(ub + BN * 16) = bo;
                    tc::fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(&un_full[un.idx]);
                    un.next(UNP_SLOTS);
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&pk_empty[pk.idx]);
                pk.next(PK_STAGES);
            }
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(err, 3); }
    } else {
        // ------------------------------ epilogue --------------------------------------------------
        reg_inc<REGS_EPI>();
        const int e = warp - EPI_WARP0;                     // 0..7
        const int quarter = warp & 3;                       // TMEM lanes this warp may read
        const int half = e >> 2;                            // which 64 of the 128 columns
        const int row = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        Ring acc, sc;
        bool ok = true;
        // arm every accumulator buffer with the bias pattern, then hand them to the MMA warp
        for (int b = 0; b < ACC_BUFS; ++b)
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_st16_const(tmem + lane_base + b * BN + half * 64 + c * 16, MAGIC_BITS);
        tmem_st_wait();
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0)
            for (int b = 0; b < ACC_BUFS; ++b) tc::mbar_arrive(&acc_empty[b]);
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
            const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
            float2 sum[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) sum[i] = make_float2(0.f, 0.f);
            for (int ks = 0; ks < n_stages && ok; ++ks) {
                if (!wait_bar(&sc_full[sc.idx], sc.phase, abort_flag)) { ok = false; break; }
                const float4* sxp = reinterpret_cast<const float4*>(smem + L::SCX + sc.idx * SCX_BYTES + row * 32);
                const float* sxr = reinterpret_cast<const float*>(sxp);
                const unsigned short* swt = reinterpret_cast<const unsigned short*>(smem + L::SCW + sc.idx * SCW_BYTES) + half * 64;
#pragma unroll 1
                for (int j = 0; j < KS; ++j) {
                    if (!wait_bar(&acc_full[acc.idx], acc.phase, abort_flag)) { ok = false; break; }
                    tc::tc_fence_after();
                    const uint32_t taddr = tmem + lane_base + acc.idx * BN + half * 64;
                    const float sxj = sxr[j];
                    const float2 sx2 = make_float2(sxj, sxj);
                    const uint4* swg = reinterpret_cast<const uint4*>(swt + j * BN);   // 8 bf16 scales per vector
                    const float2 neg_magic = make_float2(-MAGIC, -MAGIC);
                    uint32_t ra[16], rb[16];
                    tmem_ld16(taddr, ra);
                    tc::tmem_ld_wait();
                    tmem_st16_const(taddr, MAGIC_BITS);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t (&cur)[16] = (c & 1) ? rb : ra;
                        uint32_t (&nxt)[16] = (c & 1) ? ra : rb;
                        if (c < 3) tmem_ld16(taddr + (c + 1) * 16, nxt);
                        if constexpr (PARTIALS) {
                            const int g = ks * KS + j, m = m0 + row;
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const int n = n0 + half * 64 + c * 16 + i;
                                if (m < M && n < N) part[((size_t)m * N + n) * G + g] = ((int32_t)(cur[i] - MAGIC_BITS)) >> 8;
                            }
                        } else {
#pragma unroll
                            for (int q8 = 0; q8 < 2; ++q8) {
                                const uint4 w8 = swg[c * 2 + q8];
                                const uint32_t ww[4] = {w8.x, w8.y, w8.z, w8.w};
#pragma unroll
                                for (int p = 0; p < 4; ++p) {
                                    // t = f*s - MAGIC*s = 256 * P * s exactly; the 1/256 rides on sx
                                    const float2 s2 = make_float2(bf16_lo(ww[p]), bf16_hi(ww[p]));
                                    const float2 c2 = __fmul2_rn(s2, neg_magic);
                                    const float2 f2 = make_float2(__uint_as_float(cur[q8 * 8 + p * 2]), __uint_as_float(cur[q8 * 8 + p * 2 + 1]));
                                    const float2 t2 = __ffma2_rn(f2, s2, c2);
                                    sum[c * 8 + q8 * 4 + p] = __ffma2_rn(t2, sx2, sum[c * 8 + q8 * 4 + p]);
                                }
                            }
                        }
                        if (c < 3) {
                            tc::tmem_ld_wait();
                            tmem_st16_const(taddr + (c + 1) * 16, MAGIC_BITS);   // re-arm what was just read
                        }
                        if (c == 2) {                        // buffer fully read and re-armed
                            tmem_st_wait();
                            tc::tc_fence_before();
                            __syncwarp();
                            if (lane == 0) tc::mbar_arrive(&acc_empty[acc.idx]);
                        }
                    }
                    acc.next(ACC_BUFS);
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&sc_empty[sc.idx]);
                sc.next(SC_SLOTS);
            }
            if constexpr (!PARTIALS) {
                const int m = m0 + row;
                if (ok && m < M) {
                    __half* yr = y + (size_t)m * N + n0 + half * 64;
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        if (n0 + half * 64 + v * 8 + 8 <= N) {
                            __half2 h0 = __floats2half2_rn(sum[v * 4 + 0].x, sum[v * 4 + 0].y);
                            __half2 h1 = __floats2half2_rn(sum[v * 4 + 1].x, sum[v * 4 + 1].y);
                            __half2 h2 = __floats2half2_rn(sum[v * 4 + 2].x, sum[v * 4 + 2].y);
                            __half2 h3 = __floats2half2_rn(sum[v * 4 + 3].x, sum[v * 4 + 3].y);
                            uint4 pack;
                            pack.x = *reinterpret_cast<uint32_t*>(&h0); pack.y = *reinterpret_cast<uint32_t*>(&h1);
                            pack.z = *reinterpret_cast<uint32_t*>(&h2); pack.w = *reinterpret_cast<uint32_t*>(&h3);
                            *reinterpret_cast<uint4*>(yr + v * 8) = pack;
                        }
                    }
                }
            }
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(err, 4); }
    }

    tc::tc_fence_before();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem, ACC_BUFS * BN);
}

// ---- host ---------------------------------------------------------------------------------------
template <bool PARTIALS>
int launch_tc(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N, int64_t K,
              void* y, int32_t* part, int* err, cudaStream_t st)
{
    CUtensorMap mxq, mwq, mxs, mws;
    int s;
    if ((s = make_map_2d(&mxq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, K / 2, M, 128, BM, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
    if ((s = make_map_2d(&mwq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, K / 2, N, 128, BN, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
    if ((s = make_map_2d(&mxs, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, xs, K / 32, M, KS, BM, CU_TENSOR_MAP_SWIZZLE_NONE))) return s;
    if ((s = make_map_2d(&mws, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ws, K / 32, N, KS, BN, CU_TENSOR_MAP_SWIZZLE_NONE))) return s;
    const int64_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    w4a4_tc_kernel<PARTIALS><<<grid, TC_THREADS, SmemLayout::TOTAL, st>>>(mxq, mwq, mxs, mws, (__half*)y, part, (int)M,
                                                                        (int)N, (int)K, err);
    return check_launch("w4a4_tc");
}

}  // namespace

EncodeTiledFn g_encode_tiled = nullptr;

int resolve_tensor_map_encoder()
{
    if (g_encode_tiled) return WUSH_OK;
    cudaDriverEntryPointQueryResult q;
    void* fn = nullptr;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
        return fail(WUSH_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available: %s", cudaGetErrorString(e));
    g_encode_tiled = (EncodeTiledFn)fn;
    return WUSH_OK;
}

int tc_set_attributes()
{
    if (int s = resolve_tensor_map_encoder()) return s;
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(w4a4_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout::TOTAL)) != cudaSuccess ||
        (e = cudaFuncSetAttribute(w4a4_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout::TOTAL)) != cudaSuccess)
        return fail(WUSH_ERR_CUDA, "tile GEMM: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    return WUSH_OK;
}

// Shapes the tile kernel takes: whole TMA stages (K % 256 == 0) and 16-byte output vectors.
bool tc_supported(int64_t M, int64_t N, int64_t K) { return M >= 1 && K % 256 == 0 && N % 8 == 0; }

// The only scratch is the 4-byte error word the bounded waits report through.
size_t tc_workspace_bytes(int64_t, int64_t, int64_t) { return 256; }

int tc_dispatch(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N, int64_t K,
                void* y, void* workspace, size_t workspace_bytes, cudaStream_t st)
{
    if (!aligned16(xs) || !aligned16(ws) || !aligned16(y))
        return fail(WUSH_ERR_INVALID_ARGUMENT, "w4a4_gemm(tile): scales and output must be 16-byte aligned");
    if (workspace_bytes < sizeof(int)) return fail(WUSH_ERR_WORKSPACE, "w4a4_gemm(tile): workspace too small");
    int* err = reinterpret_cast<int*>(workspace);
    cudaError_t e = cudaMemsetAsync(err, 0, sizeof(int), st);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    return launch_tc<false>(xq, xs, wq, ws, M, N, K, y, nullptr, err, st);
}

int tc_partials(const uint8_t* xq, const uint8_t* wq, int64_t M, int64_t N, int64_t K, int32_t* P, int* err, cudaStream_t st)
{
    // the scale tiles are still fetched; any readable, 16-byte aligned memory of the right
    // extent will do and the codes qualify (G*2 <= K/2 bytes per row)
    return launch_tc<true>(xq, xq, wq, wq, M, N, K, nullptr, P, err, st);
}

}  // namespace wush
