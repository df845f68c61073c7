// Prefill tile GEMM on the 5th-generation tensor cores (C-ABI wush_w4a4_gemm, variant TILE).
//
//   Y[m][n] = sum_g sx[m][g] * sw[n][g] * P_g[m][n],   P_g = sum_{k in group g} qa * qw
//
// Replaces w4a4_gemm_s4_kernel<TM> of the reference (csrc/gemm_s4.cu:106-318), whose
// mma.m8n8k32.s4 atom exists on sm_75 only.  sm_100 has no 4-bit integer MMA (the s4 shapes of
// mma.sync are emulated at ~1/24 of the int8 rate), so the codes are widened to signed bytes
// in shared memory and every 32-wide group is a tcgen05.mma kind::i8 instruction (M=128, N=64,
// K=32).  Bytes hold 16 * code, so the exact group sum arrives as 256 * P_g.
//
// CTA tile: R x 128 activation rows (R = 2, or 1 for M <= 128) by 64 weight rows.  Per group the
// R blocks are R MMAs into adjacent 64-column ranges of one TMEM accumulator buffer; four
// buffers rotate, so the tensor core runs up to four groups ahead of the epilogue.  A thread
// of the epilogue owns TMEM lane l = rows l and l+128: the per-column work (fetching the
// weight scale, forming its bias term) is shared by both rows.
//
// Integer -> float conversion is never executed: each accumulator buffer is pre-loaded with the
// bit pattern of 1.5 * 2^23 and the MMA ACCUMULATES onto it.  The int32 result
// 0x4B400000 + 256*P is, read as fp32, exactly 12582912 + 256*P, and
//     t   = fma(f, sw, -12582912 * sw)              (exact: equals 256 * P * sw, <= 20 significant bits)
//     sum = fma(t, sx/256, sum)
// gives the scaled contribution with two FMAs, issued as packed fp32x2 instructions.  The
// epilogue stores the bias pattern back (tcgen05.st) right after reading a buffer.
//
// One persistent CTA per SM, four warpgroups with fixed roles (registers are re-balanced between
// them with setmaxnreg; warps 2-3 only donate theirs):
//   warp 0      TMA producer: per stage of 8 groups, tile loads of the packed activation and
//               weight codes (128-byte swizzle) and of the two bf16 scale tiles -> mbarrier tx
//   warps 4-7   widen: packed nibbles -> signed bytes in the canonical K-major core-matrix
//               layout (one shift, two ANDs per 8 codes; even codes form the first 16-byte K
//               piece, odd codes the second -- the same permutation on both operands); they
//               also lay the weight scales out as fp32 [group][n] and the activation scales as
//               fp32 / 256 [row][group]
//   warp 1      issues the MMAs (one thread), owns TMEM; tcgen05.commit frees the byte slot and
//               publishes the accumulator
//   warps 8-15  epilogue: tcgen05.ld 16 columns of both rows at a time, re-arm with
//               tcgen05.st, packed FMAs, fp16 stores at the end.  Thread = output rows, so sx is
//               a per-thread scalar and sw a vector read from shared memory.
// Every wait is bounded; a timeout sets an error word, aborts the CTA's loops and still frees
// TMEM.
//
// The CUDA cores do two FMAs per (m, n, group) against 32 tensor-core MACs, so this kernel is
// bound by the scaling epilogue (issue slots of the fp32 pipe), not by the MMA rate: that is the
// price of exact per-group bf16 scales on an architecture without a group-scaled integer MMA.
#include "common.cuh"
#include "tc_common.cuh"
#include "tc_host.cuh"

namespace wush {
namespace {

constexpr int BLK = 128;                                  // rows per MMA block (TMEM lanes)
constexpr int BN = 64;                                    // weight rows per tile (MMA N)
constexpr int KS = 8;                                     // groups per TMA stage
constexpr int PK_STAGES = 2, UNP_SLOTS = 6, ACC_BUFS = 4, SC_SLOTS = 3;
constexpr int TC_THREADS = 512;                           // four warpgroups: control, widen, epilogue x2
constexpr int CONV_WARP0 = 4, CONV_WARPS = 4, EPI_WARP0 = 8, EPI_WARPS = 8;
// registers per thread after the warpgroups trade them: 128 * (32 + 80 + 200 + 200) = 65536
constexpr int REGS_CTRL = 32, REGS_CONV = 80, REGS_EPI = 200;
constexpr uint32_t MAGIC_BITS = 0x4B400000u;              // fp32 12582912.0 = 1.5 * 2^23
constexpr float MAGIC = 12582912.0f;

template <int R>
struct Smem {
    static constexpr int ROWS = R * BLK;
    static constexpr int PKA_BYTES = ROWS * 128, PKB_BYTES = BN * 128, PKSX_BYTES = ROWS * 16, PKSW_BYTES = BN * 16;
    static constexpr int STAGE_TX = PKA_BYTES + PKB_BYTES + PKSX_BYTES + PKSW_BYTES;
    static constexpr int UNA_BYTES = ROWS * 32, UNB_BYTES = BN * 32;
    static constexpr int SCX_BYTES = ROWS * KS * 4;       // fp32 [row][group] / 256
    static constexpr int SCW_BYTES = KS * BN * 4;         // fp32 [group][n]
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
    if (tc::mbar_test_wait(bar, parity)) return true;      // the common case once the rings are full: 16 cycles instead of ~190
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

template <int R, bool PARTIALS>
__global__ void __launch_bounds__(TC_THREADS, 1)
w4a4_tc_kernel(const __grid_constant__ CUtensorMap map_xq, const __grid_constant__ CUtensorMap map_wq,
               const __grid_constant__ CUtensorMap map_xs, const __grid_constant__ CUtensorMap map_ws,
               __half* __restrict__ y, int32_t* __restrict__ part, int M, int N, int K, int* __restrict__ err)
{
    using L = Smem<R>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
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
    const int tiles_m = (M + L::ROWS - 1) / L::ROWS, tiles_n = (N + BN - 1) / BN, n_tiles = tiles_m * tiles_n;
    constexpr int ACC_COLS = R * BN;                       // TMEM columns of one accumulator buffer
    constexpr int TMEM_COLS = (ACC_BUFS * ACC_COLS <= 256) ? 256 : 512;

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
        tc::tmem_alloc(tmem_slot, TMEM_COLS);
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
                const int m0 = (t % tiles_m) * L::ROWS, n0 = (t / tiles_m) * BN;
                for (int ks = 0; ks < n_stages; ++ks) {
                    if (!wait_bar(&pk_empty[pk.idx], pk.phase ^ 1, abort_flag)) { ok = false; break; }
                    tc::mbar_expect_tx(&pk_full[pk.idx], L::STAGE_TX);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        tc::tma_load_2d(smem + L::PKA + pk.idx * L::PKA_BYTES + r * BLK * 128, &map_xq, &pk_full[pk.idx], ks * 128, m0 + r * BLK);
                        tc::tma_load_2d(smem + L::PKSX + pk.idx * L::PKSX_BYTES + r * BLK * 16, &map_xs, &pk_full[pk.idx], ks * KS, m0 + r * BLK);
                    }
                    tc::tma_load_2d(smem + L::PKB + pk.idx * L::PKB_BYTES, &map_wq, &pk_full[pk.idx], ks * 128, n0);
                    tc::tma_load_2d(smem + L::PKSW + pk.idx * L::PKSW_BYTES, &map_ws, &pk_full[pk.idx], ks * KS, n0);
                    ++issued;
                    pk.next(PK_STAGES);
                }
            }
            if (!ok) {
                *abort_flag = 1;
                atomicExch(err, 1);
                // let the copies already in flight land before this CTA gives its memory back
                for (uint32_t i = 0; i < (issued < (uint32_t)PK_STAGES ? issued : (uint32_t)PK_STAGES); ++i)
                    for (uint32_t spin = 0; spin < (1u << 16); ++spin)
                        if (tc::mbar_try_wait(&pk_full[i], 0) || tc::mbar_try_wait(&pk_full[i], 1)) break;
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
                    const uint64_t bdesc = tc::smem_desc_kmajor(tc::smem_u32(smem + L::UNB + un.idx * L::UNB_BYTES), BN * 16, 128);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const uint64_t adesc = tc::smem_desc_kmajor(
                            tc::smem_u32(smem + L::UNA + un.idx * L::UNA_BYTES + r * BLK * 32), BLK * 16, 128);
                        tc::mma_i8(tmem + acc.idx * ACC_COLS + r * BN, adesc, bdesc, idesc, 1u);   // onto the bias pattern
                    }
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
        const int ct = (warp - CONV_WARP0) * 32 + lane;     // 0..127
        Ring pk, un, sc;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
            for (int ks = 0; ks < n_stages && ok; ++ks) {
                if (!wait_bar(&pk_full[pk.idx], pk.phase, abort_flag) ||
                    !wait_bar(&sc_empty[sc.idx], sc.phase ^ 1, abort_flag)) { ok = false; break; }
                {   // scales of this stage
                    const float k = 1.0f / 256.0f;          // undoes the 16 x 16 of the widened codes
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const int row = r * BLK + ct;
                        const uint4 vx = *reinterpret_cast<const uint4*>(smem + L::PKSX + pk.idx * L::PKSX_BYTES + row * 16);
                        float4* dx = reinterpret_cast<float4*>(smem + L::SCX + sc.idx * L::SCX_BYTES + row * 32);
                        dx[0] = make_float4(bf16_lo(vx.x) * k, bf16_hi(vx.x) * k, bf16_lo(vx.y) * k, bf16_hi(vx.y) * k);
                        dx[1] = make_float4(bf16_lo(vx.z) * k, bf16_hi(vx.z) * k, bf16_lo(vx.w) * k, bf16_hi(vx.w) * k);
                    }
                    if (ct < BN) {
                        const uint4 vw = *reinterpret_cast<const uint4*>(smem + L::PKSW + pk.idx * L::PKSW_BYTES + ct * 16);
                        float* dw = reinterpret_cast<float*>(smem + L::SCW + sc.idx * L::SCW_BYTES) + ct;
                        dw[0 * BN] = bf16_lo(vw.x); dw[1 * BN] = bf16_hi(vw.x);
                        dw[2 * BN] = bf16_lo(vw.y); dw[3 * BN] = bf16_hi(vw.y);
                        dw[4 * BN] = bf16_lo(vw.z); dw[5 * BN] = bf16_hi(vw.z);
                        dw[6 * BN] = bf16_lo(vw.w); dw[7 * BN] = bf16_hi(vw.w);
                    }
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(&sc_full[sc.idx]);
                    sc.next(SC_SLOTS);
                }
                const uint8_t* pa = smem + L::PKA + pk.idx * L::PKA_BYTES + ct * 128;
                const uint8_t* pb = smem + L::PKB + pk.idx * L::PKB_BYTES + ct * 128;
                const int dst_off = (ct >> 3) * 128 + (ct & 7) * 16;        // inside one 128-row block
#pragma unroll 1
                for (int j = 0; j < KS; ++j) {
                    if (!wait_bar(&un_empty[un.idx], un.phase ^ 1, abort_flag)) { ok = false; break; }
                    const int chunk = (j ^ (ct & 7)) << 4;                  // 128-byte swizzle of the TMA tile
                    uint8_t* ua = smem + L::UNA + un.idx * L::UNA_BYTES + dst_off;
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const uint4 a = *reinterpret_cast<const uint4*>(pa + r * BLK * 128 + chunk);
                        uint4 ae, ao;
                        unpack_x16(a.x, ae.x, ao.x); unpack_x16(a.y, ae.y, ao.y);
                        unpack_x16(a.z, ae.z, ao.z); unpack_x16(a.w, ae.w, ao.w);
                        *reinterpret_cast<uint4*>(ua + r * BLK * 32) = ae;
                        *reinterpret_cast<uint4*>(ua + r * BLK * 32 + BLK * 16) = ao;
                    }
                    if (ct < BN) {
                        const uint4 b = *reinterpret_cast<const uint4*>(pb + chunk);
                        uint4 be, bo;
                        unpack_x16(b.x, be.x, bo.x); unpack_x16(b.y, be.y, bo.y);
                        unpack_x16(b.z, be.z, bo.z); unpack_x16(b.w, be.w, bo.w);
                        uint8_t* ub = smem + L::UNB + un.idx * L::UNB_BYTES + dst_off;
                        *reinterpret_cast<uint4*>(ub) = be;
                        *reinterpret_cast<uint4*>(ub + BN * 16) = bo;
                    }
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
        const int half = e >> 2;                            // which 32 of the 64 columns
        const int row = quarter * 32 + lane;                // lane of the block = row inside each 128-row block
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        Ring acc, sc;
        bool ok = true;
        // arm every accumulator buffer with the bias pattern, then hand them to the MMA warp
        for (int b = 0; b < ACC_BUFS; ++b)
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int c = 0; c < 2; ++c)
                    tmem_st16_const(tmem + lane_base + b * ACC_COLS + r * BN + half * 32 + c * 16, MAGIC_BITS);
        tmem_st_wait();
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0)
            for (int b = 0; b < ACC_BUFS; ++b) tc::mbar_arrive(&acc_empty[b]);
        const float2 neg_magic = make_float2(-MAGIC, -MAGIC);
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
            const int m0 = (t % tiles_m) * L::ROWS, n0 = (t / tiles_m) * BN;
            float2 sum[R][16];                              // [row block][column pair]
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int i = 0; i < 16; ++i) sum[r][i] = make_float2(0.f, 0.f);
            for (int ks = 0; ks < n_stages && ok; ++ks) {
                if (!wait_bar(&sc_full[sc.idx], sc.phase, abort_flag)) { ok = false; break; }
                const float* sxr = reinterpret_cast<const float*>(smem + L::SCX + sc.idx * L::SCX_BYTES) + row * KS;
                const float* swt = reinterpret_cast<const float*>(smem + L::SCW + sc.idx * L::SCW_BYTES) + half * 32;
#pragma unroll 1
                for (int j = 0; j < KS; ++j) {
                    if (!wait_bar(&acc_full[acc.idx], acc.phase, abort_flag)) { ok = false; break; }
                    tc::tc_fence_after();
                    const uint32_t taddr = tmem + lane_base + acc.idx * ACC_COLS + half * 32;
                    float2 sx2[R];
#pragma unroll
                    for (int r = 0; r < R; ++r) { const float v = sxr[r * BLK * KS + j]; sx2[r] = make_float2(v, v); }
                    const float4* swg = reinterpret_cast<const float4*>(swt + j * BN);
#pragma unroll
                    for (int c = 0; c < 2; ++c) {            // 16 columns at a time, all R rows
                        uint32_t v[R][16];
#pragma unroll
                        for (int r = 0; r < R; ++r) tmem_ld16(taddr + r * BN + c * 16, v[r]);
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int r = 0; r < R; ++r) tmem_st16_const(taddr + r * BN + c * 16, MAGIC_BITS);   // re-arm
                        if (c == 1) {                        // buffer fully read and re-armed
                            tmem_st_wait();
                            tc::tc_fence_before();
                            __syncwarp();
                            if (lane == 0) tc::mbar_arrive(&acc_empty[acc.idx]);
                        }
                        if constexpr (PARTIALS) {
                            const int g = ks * KS + j;
#pragma unroll
                            for (int r = 0; r < R; ++r) {
                                const int m = m0 + r * BLK + row;
#pragma unroll
                                for (int i = 0; i < 16; ++i) {
                                    const int n = n0 + half * 32 + c * 16 + i;
                                    if (m < M && n < N) part[((size_t)m * N + n) * G + g] = ((int32_t)(v[r][i] - MAGIC_BITS)) >> 8;
                                }
                            }
                        } else {
#pragma unroll
                            for (int q4 = 0; q4 < 4; ++q4) {
                                const float4 w4 = swg[c * 4 + q4];
                                const float2 s01 = make_float2(w4.x, w4.y), s23 = make_float2(w4.z, w4.w);
                                const float2 c01 = __fmul2_rn(s01, neg_magic), c23 = __fmul2_rn(s23, neg_magic);
#pragma unroll
                                for (int r = 0; r < R; ++r) {
                                    // t = f*s - MAGIC*s = 256 * P * s exactly; the 1/256 rides on sx
                                    const float2 f01 = make_float2(__uint_as_float(v[r][q4 * 4 + 0]), __uint_as_float(v[r][q4 * 4 + 1]));
                                    const float2 f23 = make_float2(__uint_as_float(v[r][q4 * 4 + 2]), __uint_as_float(v[r][q4 * 4 + 3]));
                                    sum[r][c * 8 + q4 * 2 + 0] = __ffma2_rn(__ffma2_rn(f01, s01, c01), sx2[r], sum[r][c * 8 + q4 * 2 + 0]);
                                    sum[r][c * 8 + q4 * 2 + 1] = __ffma2_rn(__ffma2_rn(f23, s23, c23), sx2[r], sum[r][c * 8 + q4 * 2 + 1]);
                                }
                            }
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
                if (ok) {
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const int m = m0 + r * BLK + row;
                        if (m >= M) continue;
                        __half* yr = y + (size_t)m * N + n0 + half * 32;
#pragma unroll
                        for (int v8 = 0; v8 < 4; ++v8) {
                            if (n0 + half * 32 + v8 * 8 + 8 <= N) {
                                __half2 h0 = __floats2half2_rn(sum[r][v8 * 4 + 0].x, sum[r][v8 * 4 + 0].y);
                                __half2 h1 = __floats2half2_rn(sum[r][v8 * 4 + 1].x, sum[r][v8 * 4 + 1].y);
                                __half2 h2 = __floats2half2_rn(sum[r][v8 * 4 + 2].x, sum[r][v8 * 4 + 2].y);
                                __half2 h3 = __floats2half2_rn(sum[r][v8 * 4 + 3].x, sum[r][v8 * 4 + 3].y);
                                uint4 pack;
                                pack.x = *reinterpret_cast<uint32_t*>(&h0); pack.y = *reinterpret_cast<uint32_t*>(&h1);
                                pack.z = *reinterpret_cast<uint32_t*>(&h2); pack.w = *reinterpret_cast<uint32_t*>(&h3);
                                *reinterpret_cast<uint4*>(yr + v8 * 8) = pack;
                            }
                        }
                    }
                }
            }
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(err, 4); }
    }

    tc::tc_fence_before();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem, TMEM_COLS);
}

// ---- host ---------------------------------------------------------------------------------------
template <int R, bool PARTIALS>
int launch_tc(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N, int64_t K,
              void* y, int32_t* part, int* err, cudaStream_t st)
{
    using L = Smem<R>;
    CUtensorMap mxq, mwq, mxs, mws;
    int s;
    if ((s = make_map_2d(&mxq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, K / 2, M, 128, BLK, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
    if ((s = make_map_2d(&mwq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, K / 2, N, 128, BN, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
    if ((s = make_map_2d(&mxs, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, xs, K / 32, M, KS, BLK, CU_TENSOR_MAP_SWIZZLE_NONE))) return s;
    if ((s = make_map_2d(&mws, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ws, K / 32, N, KS, BN, CU_TENSOR_MAP_SWIZZLE_NONE))) return s;
    const int64_t tiles = ((M + L::ROWS - 1) / L::ROWS) * ((N + BN - 1) / BN);
    int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    w4a4_tc_kernel<R, PARTIALS><<<grid, TC_THREADS, L::TOTAL, st>>>(mxq, mwq, mxs, mws, (__half*)y, part, (int)M, (int)N,
                                                                   (int)K, err);
    return check_launch("w4a4_tc");
}

template <int R, bool P>
cudaError_t set_attr() {
    return cudaFuncSetAttribute(w4a4_tc_kernel<R, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<R>::TOTAL);
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
    if ((e = set_attr<1, false>()) != cudaSuccess || (e = set_attr<2, false>()) != cudaSuccess ||
        (e = set_attr<1, true>()) != cudaSuccess || (e = set_attr<2, true>()) != cudaSuccess)
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
    if (M <= BLK) return launch_tc<1, false>(xq, xs, wq, ws, M, N, K, y, nullptr, err, st);
    return launch_tc<2, false>(xq, xs, wq, ws, M, N, K, y, nullptr, err, st);
}

int tc_partials(const uint8_t* xq, const uint8_t* wq, int64_t M, int64_t N, int64_t K, int32_t* P, int* err, cudaStream_t st)
{
    // the scale tiles are still fetched; any readable, 16-byte aligned memory of the right
    // extent will do and the codes qualify (G*2 <= K/2 bytes per row)
    if (M <= BLK) return launch_tc<1, true>(xq, xq, wq, wq, M, N, K, nullptr, P, err, st);
    return launch_tc<2, true>(xq, xq, wq, wq, M, N, K, nullptr, P, err, st);
}

}  // namespace wush
