// Decode product on the 5th-generation tensor cores with the operands SWAPPED (C-ABI wush_w4a4_gemm,
// variant DECODE_TC; what AUTO picks for 5..32 activation rows when the caller brings the scratch).
//
//   Y[m][n] = sum_g sx[m][g] * sw[n][g] * P_g[m][n],   P_g = sum_{k in group g} qa * qw   (exact, int32)
//
// Same contract as the reference's decode family (w4a4_gemv_multi, csrc/gemv_int4.cu:78-143, and the
// small-M branch of w4a4_gemm_s4, csrc/gemm_s4.cu:346-347).  With a handful of activation rows the product
// is one pass over the packed weights, so the kernel is organised around that stream:
//
//   * the WEIGHTS are the 128-row operand of tcgen05.mma kind::i8 (one TMEM lane per weight row), the
//     NB = 16 / 32 (padded) activation rows are its N; one K = 32 instruction per group, so every group sum
//     is exact.  Measured issue cost of such an instruction with independent accumulators: ~46 cycles
//     whatever N <= 64 is -- 775 of them per multiprocessor for the 70B gate+up layer;
//   * the widened weights never touch shared memory: TMA streams stages of 8 groups of packed codes (16 KB
//     for 128 rows), eight warps widen nibbles to bytes holding 16 * code in registers (one shift, two ANDs
//     per 8 codes) and store them with tcgen05.st into tensor memory, from where the MMA takes its A operand
//     (a thread = a weight row = a TMEM lane, 8 columns per group).  Per stage the shared memory carries
//     ~60 KB instead of the ~115 KB of a widened copy written to and read back from it;
//   * the few activation rows are widened once per stage by two otherwise idle warps into the canonical
//     K-major core-matrix layout (even codes first, odd codes second -- the same order as the weights'
//     columns), the MMA's B operand;
//   * a thread of the epilogue owns one weight row: its scale sw[n][g] is a per-thread scalar read as bf16
//     straight from the TMA tile, the activation scales a small fp32 vector broadcast from shared memory.
//     No integer -> float conversion: the accumulators are pre-loaded with the bits of 1.5 * 2^23 and
//     re-armed after every read, so
//         t = fma(f, sw, -1.5 * 2^23 * sw)  ( = 256 * P * sw exactly ),   sum = fma(t, sx / 256, sum)
//     as packed fp32x2 instructions: two FMAs per output and group, which is what bounds M = 32;
//   * work is dealt in STAGES, not tiles: the (tile, stage) sequence is cut into equal contiguous ranges,
//     one per multiprocessor (57344 rows are 448 tiles = 3.03 per multiprocessor; whole tiles would leave a
//     fourth round for four of them, and narrow layers would leave most of the part idle).  A range that
//     covers a tile completely writes fp16 results; the at most two partial pieces per CTA go to the scratch
//     as fp32 and a second small kernel adds the pieces of each split tile in K order (deterministic).
//
// Roles (640 threads): warp 0 TMA producer, warp 1 MMA issuer and owner of the tensor memory, warps 2-3
// activation preparation, warps 4-11 weight widening (warps w and w + 4 share a lane quarter and take the
// two halves of a stage), warps 12-19 epilogue (two column halves per lane quarter).  Every wait is
// bounded; a wait that gives up sets an error word, aborts the CTA's loops and still frees the tensor memory.
#include <algorithm>

#include "common.cuh"
#include "tc_common.cuh"
#include "tc_host.cuh"

namespace wush {
namespace {

constexpr int DROWS = 128;                                // weight rows per tile (MMA M)
constexpr int DKS = 8;                                    // groups per TMA stage (128 bytes of packed codes per row)
constexpr int DGP = 4;                                    // groups per half stage: one A slot, one accumulator buffer
constexpr int D_PW_STAGES = 6, D_PX_STAGES = 4, D_PS_STAGES = 8, D_BX_SLOTS = 6, D_SC_SLOTS = 6;
constexpr int D_THREADS = 640;
constexpr int D_PREP_WARP0 = 2, D_PREP_WARPS = 2, D_CONV_WARP0 = 4, D_CONV_WARPS = 8, D_EPI_WARP0 = 12, D_EPI_WARPS = 8;
constexpr uint32_t D_MAGIC_BITS = 0x4B400000u;            // fp32 12582912.0 = 1.5 * 2^23
constexpr float D_MAGIC = 12582912.0f;
// Registers move between the five warpgroups.  What can be handed out is what the CTA was LAUNCHED with -- 640 threads
// of 96 registers (the compiler's figure under __launch_bounds__(640, 1)), not the whole register file: a
// setmaxnreg.inc that asks for more than the others have released never returns.
constexpr int D_REGS_LAUNCH = 96;
constexpr int D_REGS_CTRL = 72, D_REGS_CONV = 64, D_REGS_EPI = 136;
static_assert(D_REGS_CTRL + 2 * D_REGS_CONV + 2 * D_REGS_EPI <= 5 * D_REGS_LAUNCH, "setmaxnreg budget exceeds the launch allocation");

template <int NB>
struct DSmem {
    // Tensor memory: half of it (NB = 16) or a quarter (NB = 32) holds widened weights -- 8 / 4 slots of DGP groups x 8
    // columns --, the rest the accumulator buffers of DGP groups x NB columns.  A cross-warp mbarrier hop costs ~200
    // cycles and a commit after four MMAs ~400 (measured), so every ring must cover about a thousand cycles.
    static constexpr int A_SLOTS = NB <= 16 ? 8 : 4;
    static constexpr int A_COLS = A_SLOTS * DGP * 8;
    static constexpr int ACC_BUFS = (512 - A_COLS) / (DGP * NB) < 4 ? (512 - A_COLS) / (DGP * NB) : 4;
    static constexpr int TMEM_COLS = 512;
    static constexpr int PW_BYTES = DROWS * 128, PX_BYTES = NB * 128, PSX_BYTES = NB * 16, PS_BYTES = DROWS * 16;
    static constexpr int BX_BYTES = DKS * NB * 32;        // widened activations of one stage
    static constexpr int SCX_BYTES = DKS * NB * 4;        // fp32 [group][activation row] / 256
    static constexpr int PW = 0;
    static constexpr int PX = PW + D_PW_STAGES * PW_BYTES;
    static constexpr int PSX = PX + D_PX_STAGES * PX_BYTES;
    static constexpr int PS = PSX + D_PX_STAGES * PSX_BYTES;
    static constexpr int BX = PS + D_PS_STAGES * PS_BYTES;
    static constexpr int SCX = BX + D_BX_SLOTS * BX_BYTES;
    static constexpr int XCH = SCX + D_SC_SLOTS * SCX_BYTES;   // 4 quarters x 32 rows x NB fp32: sums of half 1 on their way to half 0
    static constexpr int BARS = XCH + 4 * 32 * NB * 4;
    static constexpr int NBARS = 2 * (D_PW_STAGES + D_PX_STAGES + D_PS_STAGES + D_BX_SLOTS + D_SC_SLOTS + A_SLOTS + ACC_BUFS + 4) + 1;
    static constexpr int MISC = BARS + NBARS * 8;
    static constexpr int TOTAL = MISC + 16 + 1024;        // + slack for the 1024-byte alignment
    static constexpr int PART_FLOATS = NB * DROWS;        // one partial piece in the scratch
};

struct DRing {
    uint32_t idx = 0, phase = 0;
    __device__ __forceinline__ void next(uint32_t n) { if (++idx == n) { idx = 0; phase ^= 1; } }
};

__device__ __forceinline__ bool d_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (tc::mbar_test_wait(bar, parity)) return true;      // the common case once the rings are full: 16 cycles instead of ~190
    for (uint32_t i = 0; i < WUSH_SPIN_LIMIT; ++i) {
        if (tc::mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    return false;
}

template <int NC> __device__ __forceinline__ void d_tmem_ld(uint32_t taddr, uint32_t (&r)[NC]);
template <> __device__ __forceinline__ void d_tmem_ld<8>(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
template <> __device__ __forceinline__ void d_tmem_ld<16>(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
template <int NC> __device__ __forceinline__ void d_tmem_arm(uint32_t taddr);
template <> __device__ __forceinline__ void d_tmem_arm<8>(uint32_t taddr) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr), "r"(D_MAGIC_BITS)
                 : "memory");
}
template <> __device__ __forceinline__ void d_tmem_arm<16>(uint32_t taddr) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr), "r"(D_MAGIC_BITS)
        : "memory");
}
// eight widened words of one group (32 bytes of one weight row) -> 8 columns of this thread's TMEM lane
__device__ __forceinline__ void d_tmem_st8(uint32_t taddr, const uint4& lo, const uint4& hi) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(lo.x), "r"(lo.y),
                 "r"(lo.z), "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
                 : "memory");
}
__device__ __forceinline__ void d_tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// A operand from tensor memory (row i in lane i, four int8 per 32-bit column), B from shared memory
__device__ __forceinline__ void d_mma_i8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
template <int R> __device__ __forceinline__ void d_reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(R)); }
template <int R> __device__ __forceinline__ void d_reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(R)); }

// Range of stage units of CTA `c` out of `C`: [c*S/C, (c+1)*S/C)
__host__ __device__ __forceinline__ long long unit_start(long long c, long long C, long long S) { return c * S / C; }
// the CTA whose range holds unit u
__host__ __device__ __forceinline__ int unit_owner(long long u, long long C, long long S) { return (int)(((u + 1) * C - 1) / S); }

template <int NB>
__global__ void __launch_bounds__(D_THREADS, 1)
w4a4_decode_tc_kernel(const __grid_constant__ CUtensorMap map_wq, const __grid_constant__ CUtensorMap map_xq,
                      const __grid_constant__ CUtensorMap map_ws, const __grid_constant__ CUtensorMap map_xs,
                      __half* __restrict__ y, float* __restrict__ part, int M, int N, int K, int* __restrict__ err)
{
    using L = DSmem<NB>;
    constexpr int ACC_COLS = DGP * NB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);
    uint64_t* pw_full = bars;                              // packed weight codes landed (TMA)
    uint64_t* pw_empty = pw_full + D_PW_STAGES;            // ... and are in the widening warps' registers
    uint64_t* px_full = pw_empty + D_PW_STAGES;            // packed activation codes + activation scales landed
    uint64_t* px_empty = px_full + D_PX_STAGES;
    uint64_t* ps_full = px_empty + D_PX_STAGES;            // weight scales landed
    uint64_t* ps_empty = ps_full + D_PS_STAGES;            // ... and are in the epilogue's registers
    uint64_t* bx_full = ps_empty + D_PS_STAGES;            // widened activations of a stage written
    uint64_t* bx_empty = bx_full + D_BX_SLOTS;             // ... and read by the stage's MMAs
    uint64_t* sc_full = bx_empty + D_BX_SLOTS;             // activation scales as fp32 written
    uint64_t* sc_empty = sc_full + D_SC_SLOTS;
    uint64_t* at_full = sc_empty + D_SC_SLOTS;             // widened weights of a half stage are in tensor memory
    uint64_t* mma_done = at_full + L::A_SLOTS;             // the MMAs of a half stage have retired: its A slot is free
    uint64_t* acc_full = mma_done + L::A_SLOTS;            // ... and its sums can be read.  (Two barriers although one event: a
                                                           // barrier may only be shared by waiters that cannot fall a whole ring
                                                           // behind it, and the epilogue's ring is the accumulator buffers, not the A slots.)
    uint64_t* acc_empty = acc_full + L::ACC_BUFS;          // an accumulator buffer has been read into registers
    uint64_t* xch_full = acc_empty + L::ACC_BUFS;          // per lane quarter: half 1's sums of a finished piece are in shared memory
    uint64_t* xch_empty = xch_full + 4;
    uint64_t* done_bar = xch_empty + 4;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::MISC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::MISC + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int spt = K >> 8;                                // stages per tile (8 groups = 256 codes each)
    const int units = ((N + DROWS - 1) / DROWS) * spt;      // < 2^30 (checked by the host)
    const int u0 = (int)unit_start(blockIdx.x, gridDim.x, units), u1 = (int)unit_start(blockIdx.x + 1, gridDim.x, units);

    // The error word is cleared here rather than by a memset node in front of the kernel (which would turn the
    // programmatic launch edge from the preceding kernel into a full one).  A wait can only give up after
    // seconds of polling, long after block 0 has passed this line.
    if (tid == 0 && blockIdx.x == 0) *err = 0;
    if (tid == 0) {
        for (int i = 0; i < D_PW_STAGES; ++i) { tc::mbar_init(&pw_full[i], 1); tc::mbar_init(&pw_empty[i], D_CONV_WARPS); }
        for (int i = 0; i < D_PX_STAGES; ++i) { tc::mbar_init(&px_full[i], 1); tc::mbar_init(&px_empty[i], D_PREP_WARPS); }
        for (int i = 0; i < D_PS_STAGES; ++i) { tc::mbar_init(&ps_full[i], 1); tc::mbar_init(&ps_empty[i], D_EPI_WARPS); }
        for (int i = 0; i < D_BX_SLOTS; ++i) { tc::mbar_init(&bx_full[i], D_PREP_WARPS); tc::mbar_init(&bx_empty[i], 1); }
        for (int i = 0; i < D_SC_SLOTS; ++i) { tc::mbar_init(&sc_full[i], D_PREP_WARPS); tc::mbar_init(&sc_empty[i], D_EPI_WARPS); }
        for (int i = 0; i < L::A_SLOTS; ++i) { tc::mbar_init(&at_full[i], 4); tc::mbar_init(&mma_done[i], 1); }
        for (int i = 0; i < L::ACC_BUFS; ++i) { tc::mbar_init(&acc_full[i], 1); tc::mbar_init(&acc_empty[i], 4); }
        for (int i = 0; i < 4; ++i) { tc::mbar_init(&xch_full[i], 1); tc::mbar_init(&xch_empty[i], 1); }
        tc::mbar_init(done_bar, 1);
        *abort_flag = 0;
        tc::mbar_fence_init();
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, L::TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_a = tmem, tmem_d = tmem + L::A_COLS;
    pdl_launch_dependents();                               // the piece-adding kernel may get resident; it waits for this grid

    if (warp < D_CONV_WARP0) {
        d_reg_dec<D_REGS_CTRL>();
        if (warp == 0) {
            // ------------------------------ TMA producer ------------------------------------------
            if (lane == 0) {
                tc::prefetch_tensormap(&map_wq); tc::prefetch_tensormap(&map_xq);
                tc::prefetch_tensormap(&map_ws); tc::prefetch_tensormap(&map_xs);
                DRing pw, ps;                              // weights and their scales do not depend on the kernel before: no wait
                bool ok = true;
                int tile = u0 / spt, st = u0 - tile * spt;
                for (int u = u0; u < u1; ++u) {
                    if (!d_wait(&ps_empty[ps.idx], ps.phase ^ 1, abort_flag)) { ok = false; break; }
                    tc::mbar_expect_tx(&ps_full[ps.idx], L::PS_BYTES);
                    tc::tma_load_2d(smem + L::PS + ps.idx * L::PS_BYTES, &map_ws, &ps_full[ps.idx], st * DKS, tile * DROWS);
                    if (!d_wait(&pw_empty[pw.idx], pw.phase ^ 1, abort_flag)) { ok = false; break; }
                    tc::mbar_expect_tx(&pw_full[pw.idx], L::PW_BYTES);
                    tc::tma_load_2d(smem + L::PW + pw.idx * L::PW_BYTES, &map_wq, &pw_full[pw.idx], st * 128, tile * DROWS);
                    pw.next(D_PW_STAGES); ps.next(D_PS_STAGES);
                    if (++st == spt) { st = 0; ++tile; }
                }
                if (!ok) { *abort_flag = 1; atomicCAS(err, 0, 1); }
                // Copies in flight land in this CTA's shared memory: on the normal path every one of them is consumed
                // before its consumers leave; after an abort give them a bounded time.
                if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(20000);
            }
        } else if (warp == 1) {
            // ------------------------------ MMA issuer ----------------------------------------------
            if (lane == 0) {
                DRing at, bx, acc;
                bool ok = true;
                const uint32_t idesc = tc::idesc_i8(NB);
                // The B descriptors differ only in their address field (bits 0-13, units of 16 bytes): one 32-bit add
                // per instruction on the low word.  This thread's instruction count is on the critical path.
                const uint64_t bdesc0 = tc::smem_desc_kmajor(tc::smem_u32(smem + L::BX), NB * 16, 128);
                const uint32_t b_hi = (uint32_t)(bdesc0 >> 32), b_lo0 = (uint32_t)bdesc0;
                for (int u = u0; u < u1 && ok; ++u) {
                    if (!d_wait(&bx_full[bx.idx], bx.phase, abort_flag)) { ok = false; break; }
                    const uint32_t b_lo = b_lo0 + bx.idx * (L::BX_BYTES >> 4);
#pragma unroll
                    for (int h = 0; h < DKS / DGP; ++h) {
                        if (!d_wait(&at_full[at.idx], at.phase, abort_flag) ||
                            !d_wait(&acc_empty[acc.idx], acc.phase ^ 1, abort_flag)) { ok = false; break; }
                        tc::tc_fence_after();
                        const uint32_t d0 = tmem_d + acc.idx * ACC_COLS, a0 = tmem_a + at.idx * (DGP * 8);
#pragma unroll
                        for (int jj = 0; jj < DGP; ++jj) {
                            const uint64_t bdesc = ((uint64_t)b_hi << 32) | (b_lo + (uint32_t)(((h * DGP + jj) * NB * 32) >> 4));
                            d_mma_i8_ts(d0 + jj * NB, a0 + jj * 8, bdesc, idesc, 0u);   // a fresh sum per group
                        }
                        tc::mma_commit(&mma_done[at.idx]);
                        tc::mma_commit(&acc_full[acc.idx]);
                        at.next(L::A_SLOTS);
                        acc.next(L::ACC_BUFS);
                    }
                    if (!ok) break;
                    tc::mma_commit(&bx_empty[bx.idx]);
                    bx.next(D_BX_SLOTS);
                }
                if (!ok) { *abort_flag = 1; atomicCAS(err, 0, 2); }
                tc::mma_commit(done_bar);                   // everything issued so far has retired
                for (uint32_t spin = 0; spin < WUSH_SPIN_LIMIT; ++spin)
                    if (tc::mbar_try_wait(done_bar, 0)) break;
            }
        } else {
            // ------------------------------ activation preparation (warps 2-3) ---------------------------
            // These warps also fetch their own input: thread 0 issues the TMA loads of the activation slice (codes and
            // scales) PX_STAGES stages ahead -- it knows when a slot is free, so the weight stream of warp 0 never waits
            // for this ring.
            const int t = (warp - D_PREP_WARP0) * 32 + lane;         // 0..63
            DRing px, bx, sc;
            bool ok = true;
            int st_load = (u0 % spt), u_load = u0;                   // next stage to fetch
            uint32_t ld_idx = 0, ld_phase = 0;
            if (t == 0) {
                pdl_wait();                                           // the activations may come from the kernel just before
                for (; u_load < u1 && u_load < u0 + D_PX_STAGES; ++u_load) {
                    tc::mbar_expect_tx(&px_full[ld_idx], L::PX_BYTES + L::PSX_BYTES);
                    tc::tma_load_2d(smem + L::PX + ld_idx * L::PX_BYTES, &map_xq, &px_full[ld_idx], st_load * 128, 0);
                    tc::tma_load_2d(smem + L::PSX + ld_idx * L::PSX_BYTES, &map_xs, &px_full[ld_idx], st_load * DKS, 0);
                    if (++st_load == spt) st_load = 0;
                    ++ld_idx;
                }
                ld_idx = 0;                                           // refills start over at slot 0 and wait for its first release
            }
            for (int u = u0; u < u1 && ok; ++u) {
                if (!d_wait(&px_full[px.idx], px.phase, abort_flag) || !d_wait(&bx_empty[bx.idx], bx.phase ^ 1, abort_flag) ||
                    !d_wait(&sc_empty[sc.idx], sc.phase ^ 1, abort_flag)) { ok = false; break; }
                const uint8_t* pxs = smem + L::PX + px.idx * L::PX_BYTES;
                uint8_t* bxs = smem + L::BX + bx.idx * L::BX_BYTES;
#pragma unroll
                for (int task = t; task < NB * DKS; task += 32 * D_PREP_WARPS) {
                    const int row = task % NB, j = task / NB;
                    const uint4 b = *reinterpret_cast<const uint4*>(pxs + row * 128 + ((j ^ (row & 7)) << 4));   // 128-byte swizzle of the TMA tile
                    uint4 be, bo;
                    unpack_x16(b.x, be.x, bo.x); unpack_x16(b.y, be.y, bo.y);
                    unpack_x16(b.z, be.z, bo.z); unpack_x16(b.w, be.w, bo.w);
                    uint8_t* ux = bxs + j * NB * 32 + (row >> 3) * 128 + (row & 7) * 16;
                    *reinterpret_cast<uint4*>(ux) = be;
                    *reinterpret_cast<uint4*>(ux + NB * 16) = bo;
                }
                if (t < NB) {
                    const float k = 1.0f / 256.0f;          // undoes the 16 x 16 of the widened codes
                    const uint4 vx = *reinterpret_cast<const uint4*>(smem + L::PSX + px.idx * L::PSX_BYTES + t * 16);
                    float* dx = reinterpret_cast<float*>(smem + L::SCX + sc.idx * L::SCX_BYTES) + t;
                    dx[0 * NB] = bf16_lo(vx.x) * k; dx[1 * NB] = bf16_hi(vx.x) * k;
                    dx[2 * NB] = bf16_lo(vx.y) * k; dx[3 * NB] = bf16_hi(vx.y) * k;
                    dx[4 * NB] = bf16_lo(vx.z) * k; dx[5 * NB] = bf16_hi(vx.z) * k;
                    dx[6 * NB] = bf16_lo(vx.w) * k; dx[7 * NB] = bf16_hi(vx.w) * k;
                }
                tc::fence_proxy_async();                    // the widened tile is read by the MMA (async proxy)
                __syncwarp();
                if (lane == 0) {
                    tc::mbar_arrive(&bx_full[bx.idx]);
                    tc::mbar_arrive(&sc_full[sc.idx]);
                    tc::mbar_arrive(&px_empty[px.idx]);
                }
                if (t == 0 && u_load < u1) {                          // refill the slot both warps have just left
                    if (!d_wait(&px_empty[ld_idx], ld_phase, abort_flag)) { ok = false; break; }
                    tc::mbar_expect_tx(&px_full[ld_idx], L::PX_BYTES + L::PSX_BYTES);
                    tc::tma_load_2d(smem + L::PX + ld_idx * L::PX_BYTES, &map_xq, &px_full[ld_idx], st_load * 128, 0);
                    tc::tma_load_2d(smem + L::PSX + ld_idx * L::PSX_BYTES, &map_xs, &px_full[ld_idx], st_load * DKS, 0);
                    if (++st_load == spt) st_load = 0;
                    if (++ld_idx == D_PX_STAGES) { ld_idx = 0; ld_phase ^= 1; }
                    ++u_load;
                }
                px.next(D_PX_STAGES); bx.next(D_BX_SLOTS); sc.next(D_SC_SLOTS);
            }
            if (!ok && lane == 0) { *abort_flag = 1; atomicCAS(err, 0, 5); }
        }
    } else if (warp < D_EPI_WARP0) {
        // ------------------------------ widen the weights into tensor memory ------------------------
        d_reg_dec<D_REGS_CONV>();
        const int quarter = warp & 3, h = (warp - D_CONV_WARP0) >> 2;   // lane quarter; which half of every stage
        const int row = quarter * 32 + lane;                // weight row of the tile = TMEM lane
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        DRing pw;
        uint32_t a_idx = (uint32_t)h, a_phase = 0;          // this half's A slots: h, h + 2, h, ...
        bool ok = true;
        for (int u = u0; u < u1 && ok; ++u) {
            if (!d_wait(&pw_full[pw.idx], pw.phase, abort_flag)) { ok = false; break; }
            const uint8_t* p = smem + L::PW + pw.idx * L::PW_BYTES + row * 128;
            uint4 a[DGP];
#pragma unroll
            for (int jj = 0; jj < DGP; ++jj) a[jj] = *reinterpret_cast<const uint4*>(p + (((h * DGP + jj) ^ (row & 7)) << 4));
            if (!d_wait(&mma_done[a_idx], a_phase ^ 1, abort_flag)) { ok = false; break; }
            tc::tc_fence_after();
#pragma unroll
            for (int jj = 0; jj < DGP; ++jj) {
                uint4 ae, ao;
                unpack_x16(a[jj].x, ae.x, ao.x); unpack_x16(a[jj].y, ae.y, ao.y);
                unpack_x16(a[jj].z, ae.z, ao.z); unpack_x16(a[jj].w, ae.w, ao.w);
                d_tmem_st8(tmem_a + lane_base + a_idx * (DGP * 8) + jj * 8, ae, ao);
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&pw_empty[pw.idx]);        // the packed words of this warp are in registers
            d_tmem_st_wait();
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&at_full[a_idx]);
            pw.next(D_PW_STAGES);
            a_idx += 2;
            if (a_idx >= (uint32_t)L::A_SLOTS) { a_idx -= L::A_SLOTS; a_phase ^= 1; }
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicCAS(err, 0, 3); }
    } else {
        // ------------------------------ epilogue --------------------------------------------------
        // Warp (quarter, eh): the 32 weight rows of its lane quarter, ALL NB activation columns, and the half eh of
        // every stage (its 4 groups = every second accumulator buffer).  Both halves of a row are added at the end.
        d_reg_inc<D_REGS_EPI>();
        const int quarter = warp & 3, eh = (warp - D_EPI_WARP0) >> 2;
        const int row = quarter * 32 + lane;                // weight row inside the tile
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        constexpr int GB = NB <= 16 ? 2 : 1;                // groups read from tensor memory at a time (32 registers)
        DRing sc, ps;
        uint32_t acc_idx = (uint32_t)eh % L::ACC_BUFS;      // this half's accumulator buffers: uses eh, eh + 2, ... (mod ACC_BUFS)
        uint32_t use = (uint32_t)eh;                        // use counter: buffer use % ACC_BUFS, wait parity (use / ACC_BUFS) & 1
        uint32_t xphase = 0;
        bool ok = true;

        float2 sum[NB / 2];
#pragma unroll
        for (int i = 0; i < NB / 2; ++i) sum[i] = make_float2(0.f, 0.f);
        int tile = u0 / spt, st = u0 - tile * spt;
        const int head_tile = tile;                         // a piece in this tile goes to slot 0 of the scratch
        bool from_start = (st == 0);                        // the running piece began at stage 0 of its tile
        float* exch = reinterpret_cast<float*>(smem + L::XCH) + (size_t)quarter * 32 * NB;   // half 1 -> half 0, this quarter
        for (int u = u0; u < u1 && ok; ++u, ++st) {
            if (st == spt) { st = 0; ++tile; }
            if (!d_wait(&ps_full[ps.idx], ps.phase, abort_flag)) { ok = false; break; }
            const uint2 vw = *reinterpret_cast<const uint2*>(smem + L::PS + ps.idx * L::PS_BYTES + row * 16 + eh * 8);   // this half's 4 bf16 scales
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&ps_empty[ps.idx]);
            ps.next(D_PS_STAGES);
            const float sw4[4] = {bf16_lo(vw.x), bf16_hi(vw.x), bf16_lo(vw.y), bf16_hi(vw.y)};
            if (!d_wait(&sc_full[sc.idx], sc.phase, abort_flag)) { ok = false; break; }
            const float* sxs = reinterpret_cast<const float*>(smem + L::SCX + sc.idx * L::SCX_BYTES) + eh * DGP * NB;
            if (!d_wait(&acc_full[acc_idx], (use / L::ACC_BUFS) & 1, abort_flag)) { ok = false; break; }
            tc::tc_fence_after();
            const uint32_t taddr = tmem_d + lane_base + acc_idx * ACC_COLS;
#pragma unroll
            for (int g0 = 0; g0 < DGP; g0 += GB) {
                uint32_t v[GB][NB];
#pragma unroll
                for (int jj = 0; jj < GB; ++jj)
#pragma unroll
                    for (int c = 0; c < NB; c += 16) d_tmem_ld<16>(taddr + (g0 + jj) * NB + c, *reinterpret_cast<uint32_t(*)[16]>(&v[jj][c]));
                tc::tmem_ld_wait();
                if (g0 + GB == DGP) {                                       // the sums are in registers: the buffer is free
                    tc::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(&acc_empty[acc_idx]);
                }
#pragma unroll
                for (int jj = 0; jj < GB; ++jj) {
                    const float sw = sw4[g0 + jj];
                    const float2 sw2 = make_float2(sw, sw);
                    const float cneg = -D_MAGIC * sw;                       // exact: 3 * 2^22 * (8-bit mantissa)
                    const float2 c2 = make_float2(cneg, cneg);
                    const float4* sx4 = reinterpret_cast<const float4*>(sxs + (g0 + jj) * NB);
#pragma unroll
                    for (int i4 = 0; i4 < NB / 4; ++i4) {
                        const float4 sx = sx4[i4];
                        // int32 sum 256 * P (|.| < 2^22) -> the float 1.5 * 2^23 + 256 * P by one integer add on its bits
                        const float2 f01 = make_float2(__uint_as_float(v[jj][i4 * 4 + 0] + D_MAGIC_BITS), __uint_as_float(v[jj][i4 * 4 + 1] + D_MAGIC_BITS));
                        const float2 f23 = make_float2(__uint_as_float(v[jj][i4 * 4 + 2] + D_MAGIC_BITS), __uint_as_float(v[jj][i4 * 4 + 3] + D_MAGIC_BITS));
                        // t = f*sw - MAGIC*sw = 256 * P * sw exactly; the 1/256 rides on sx
                        sum[i4 * 2 + 0] = __ffma2_rn(__ffma2_rn(f01, sw2, c2), make_float2(sx.x, sx.y), sum[i4 * 2 + 0]);
                        sum[i4 * 2 + 1] = __ffma2_rn(__ffma2_rn(f23, sw2, c2), make_float2(sx.z, sx.w), sum[i4 * 2 + 1]);
                    }
                }
            }
            // this half's next use: two further on
            acc_idx += 2;
            if (acc_idx >= (uint32_t)L::ACC_BUFS) acc_idx -= L::ACC_BUFS;
            use += 2;
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&sc_empty[sc.idx]);
            sc.next(D_SC_SLOTS);
            if (st == spt - 1 || u == u1 - 1) {
                // End of this CTA's piece of the tile: half 1 hands its sums to half 0 of the same lane quarter through
                // shared memory (a pair of mbarriers, bounded waits like everywhere else), half 0 adds them and stores.
                if (eh == 1) {
                    if (!d_wait(&xch_empty[quarter], xphase ^ 1, abort_flag)) { ok = false; break; }
#pragma unroll
                    for (int i = 0; i < NB / 2; ++i) *reinterpret_cast<float2*>(exch + (size_t)(2 * i) * 32 + 2 * lane) = sum[i];
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(&xch_full[quarter]);
                } else {
                    if (!d_wait(&xch_full[quarter], xphase, abort_flag)) { ok = false; break; }
#pragma unroll
                    for (int i = 0; i < NB / 2; ++i) {
                        const float2 o = *reinterpret_cast<const float2*>(exch + (size_t)(2 * i) * 32 + 2 * lane);
                        sum[i].x += o.x;
                        sum[i].y += o.y;
                    }
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(&xch_empty[quarter]);
                    const int n = tile * DROWS + row;
                    if (from_start && st == spt - 1) {                      // the whole tile: final fp16 results
                        if (n < N) {
#pragma unroll
                            for (int i = 0; i < NB / 2; ++i) {
                                const int m = 2 * i;
                                if (m < M) y[(size_t)m * N + n] = __float2half_rn(sum[i].x);
                                if (m + 1 < M) y[(size_t)(m + 1) * N + n] = __float2half_rn(sum[i].y);
                            }
                        }
                    } else {                                                // a piece: fp32 to the scratch, slot 0 = the piece at the head of the range
                        const int slot = (tile == head_tile) ? 0 : 1;
                        float* dst = part + ((size_t)blockIdx.x * 2 + slot) * L::PART_FLOATS + row;
#pragma unroll
                        for (int i = 0; i < NB / 2; ++i) {
                            dst[(2 * i) * DROWS] = sum[i].x;
                            dst[(2 * i + 1) * DROWS] = sum[i].y;
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < NB / 2; ++i) sum[i] = make_float2(0.f, 0.f);
                from_start = true;                                          // the next piece begins at stage 0 of the next tile
                xphase ^= 1;
            }
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicCAS(err, 0, 4); }
    }

    tc::tc_fence_before();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem, L::TMEM_COLS);
}

// Adds the pieces of every tile that was split over several CTAs, in K order, and rounds to fp16 once.
// One block per (tile, 8 activation rows): a thread adds the two or three pieces of ONE output, so the loads of
// a block are all in flight together.  Blocks of unsplit tiles leave at once.
template <int NB>
__global__ void __launch_bounds__(DROWS * 8)
decode_tc_join_kernel(const float* __restrict__ part, __half* __restrict__ y, int M, int N, int spt, int ctas)
{
    pdl_wait();                                            // the pieces come from the kernel just before
    const int tile = blockIdx.x, row = threadIdx.x, n = tile * DROWS + row, m = blockIdx.y * 8 + threadIdx.y;
    const long long units = (long long)gridDim.x * spt;
    const long long first_unit = (long long)tile * spt, last_unit = first_unit + spt - 1;
    const int c_first = unit_owner(first_unit, ctas, units), c_last = unit_owner(last_unit, ctas, units);
    if (c_first == c_last || n >= N || m >= M) return;     // written as a whole by one CTA
    constexpr int PART = NB * DROWS;
    float acc = 0.f;
    for (int c = c_first; c <= c_last; ++c) {
        const int slot = (unit_start(c, ctas, units) / spt == tile) ? 0 : 1;
        acc += part[((size_t)c * 2 + slot) * PART + m * DROWS + row];
    }
    y[(size_t)m * N + n] = __float2half_rn(acc);
}

template <int NB>
int launch_decode_tc(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N, int64_t K,
                     void* y, void* workspace, cudaStream_t st)
{
    using L = DSmem<NB>;
    CUtensorMap mwq, mxq, mws, mxs;
    int s;
    if ((s = make_map_2d(&mwq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, K / 2, N, 128, DROWS, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
    if ((s = make_map_2d(&mxq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, K / 2, M, 128, NB, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
    if ((s = make_map_2d(&mws, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ws, K / 32, N, DKS, DROWS, CU_TENSOR_MAP_SWIZZLE_NONE))) return s;
    if ((s = make_map_2d(&mxs, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, xs, K / 32, M, DKS, NB, CU_TENSOR_MAP_SWIZZLE_NONE))) return s;
    const int spt = (int)(K / 256), tiles = (int)((N + DROWS - 1) / DROWS);
    const long long units = (long long)tiles * spt;
    const int ctas = (int)std::min<long long>(units, sm_count());
    int* err = reinterpret_cast<int*>(workspace);
    float* part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + 256);
    cudaError_t e = launch_dependent(w4a4_decode_tc_kernel<NB>, dim3((unsigned)ctas), dim3(D_THREADS), (size_t)L::TOTAL, st, mwq, mxq, mws, mxs,
                                     (__half*)y, part, (int)M, (int)N, (int)K, err);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "w4a4_decode_tc: %s", cudaGetErrorString(e));
    if (units % ctas != 0 || (units / ctas) % spt != 0) {   // some tile is split
        e = launch_dependent(decode_tc_join_kernel<NB>, dim3((unsigned)tiles, (unsigned)((M + 7) / 8)), dim3(DROWS, 8), (size_t)0, st,
                             (const float*)part, (__half*)y, (int)M, (int)N, spt, ctas);
        if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "decode_tc_join: %s", cudaGetErrorString(e));
    }
    return check_launch("w4a4_decode_tc");
}

}  // namespace

int decode_tc_set_attributes()
{
    if (int s = resolve_tensor_map_encoder()) return s;
    cudaError_t e = cudaFuncSetAttribute(w4a4_decode_tc_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, DSmem<16>::TOTAL);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(w4a4_decode_tc_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, DSmem<32>::TOTAL);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "decode (tcgen05): cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    return WUSH_OK;
}

// At most 32 activation rows and whole TMA stages of 8 groups.
bool decode_tc_supported(int64_t M, int64_t N, int64_t K)
{
    return M >= 1 && M <= 32 && N >= 1 && K % 256 == 0 && ((N + DROWS - 1) / DROWS) * (K / 256) < (1ll << 30);
}

// scratch: error word | two fp32 pieces of 128 x NB per CTA
size_t decode_tc_workspace_bytes(int64_t M, int64_t N, int64_t K)
{
    const int nb = M <= 16 ? 16 : 32;
    return 256 + (size_t)sm_count() * 2 * nb * DROWS * sizeof(float);
}

int decode_tc_dispatch(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N, int64_t K,
                       void* y, void* workspace, size_t workspace_bytes, cudaStream_t st)
{
    if (!decode_tc_supported(M, N, K))
        return fail(WUSH_ERR_UNSUPPORTED, "w4a4_gemm(decode_tc): needs 1 <= M <= 32 and K %% 256 == 0 (got M=%lld, K=%lld)",
                    (long long)M, (long long)K);
    if (!aligned16(xs) || !aligned16(ws) || !aligned16(workspace))
        return fail(WUSH_ERR_INVALID_ARGUMENT, "w4a4_gemm(decode_tc): scales and workspace must be 16-byte aligned");
    if (!workspace || workspace_bytes < decode_tc_workspace_bytes(M, N, K))
        return fail(WUSH_ERR_WORKSPACE, "w4a4_gemm(decode_tc): workspace of %zu bytes needed, %zu given",
                    decode_tc_workspace_bytes(M, N, K), workspace_bytes);
    if (M <= 16) return launch_decode_tc<16>(xq, xs, wq, ws, M, N, K, y, workspace, st);
    return launch_decode_tc<32>(xq, xs, wq, ws, M, N, K, y, workspace, st);
}

}  // namespace wush
