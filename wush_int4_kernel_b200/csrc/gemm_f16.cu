// Large-M product with the scales folded into fp16 operands (C-ABI wush_w4a4_gemm, variant
// TILE_F16; what AUTO picks for M >= 128 when the caller provides the scratch).
//
//   Y[m][n] = sum_k (qa[m][k] * sx[m][g(k)]) * (qw[n][k] * sw[n][g(k)])
//
// Same contract as the reference's w4a4_gemm_s4 (csrc/gemm_s4.cu:320-379).  The exact
// per-group route (gemm_tc.cu) must run two CUDA-core FMAs per output and group, which caps it
// near 0.9 POPS on this part whatever the tensor cores do.  Here the per-group scales are
// multiplied into the operands instead:
//   * code * scale has at most 3 + 8 significant bits, so it is EXACTLY representable in fp16
//     once each row is shifted by a power of two (2^-e, e = exponent of the row's largest
//     scale; groups more than 2^13 below the row maximum lose low bits, a relative
//     contribution < 1e-6);
//   * products of two such values have <= 22 significant bits: exact in the tensor core's fp32
//     accumulation, which then runs over the whole K without any per-group epilogue;
//   * the two row shifts come back as one exact power-of-two factor in the epilogue.
// Results agree with the fp64 arbiter to ~1e-6 before the fp16 output rounding; what this
// route cannot do is expose the integer group sums (the i8 kernels do that).
//
// Kernels:
//   dequant_f16_kernel     one warp per row: codes + bf16 scales -> fp16 row (scratch) + 2^e
//   gemm_tile2_kernel  M > 2048, both operands pre-widened: persistent 256 x 256 tiles, TMA (128-byte
//                          swizzle) -> 3-stage ring -> tcgen05.mma kind::f16 (M=128, N=256, K=16), two MMA
//                          groups per weight tile -> TMEM -> epilogue warps tcgen05.ld, scale by
//                          2^(e_m+e_n), fp16 store
//                          (instantiated for kind::i8 as well: the per-tensor-scale product)
//   gemm_f16_fused_kernel  M <= 128: only the activations are pre-widened, the packed weight tile is
//   gemm_f16_fused2_kernel 128 < M <= 2048 (256 x 256 tiles): widened to fp16 inside the kernel
// Algorithmic traffic: the pre-pass reads 9/16 B and writes 2 B per operand element; the GEMM
// reads fp16 operands (L2-resident across the M tiles that share a weight tile); with in-kernel
// widening the weights are read once, packed.
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "tc_common.cuh"
#include "tc_host.cuh"

namespace wush {
namespace {

// ------------------------------------------------------------------------------------------------
// pre-pass
// ------------------------------------------------------------------------------------------------
// PERM: inside every octet of codes the output order is 0,4,1,5,2,6,3,7 -- the order in which the
// fused kernel below produces the other operand (a sum over k does not care, as long as both agree).
template <bool PERM>
__device__ __forceinline__ void dequant_f16_row(const uint8_t* __restrict__ q, const __nv_bfloat16* __restrict__ s,
                                                __half* __restrict__ out, float* __restrict__ row_factor, long long row, int K,
                                                int lane)
{
    const int G = K >> 5;
    const unsigned short* sr = reinterpret_cast<const unsigned short*>(s) + row * G;
    // largest scale of the row (bf16 bit patterns of non-negative values order like integers)
    unsigned mx = 0;
    for (int g = lane; g < G; g += 32) mx = max(mx, (unsigned)(sr[g] & 0x7fffu));
#pragma unroll
    for (int off = 16; off; off >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    int e = (int)(mx >> 7) - 127;                               // exponent of the largest scale
    e = max(-100, min(100, e));
    const float down = __uint_as_float((uint32_t)(127 - e) << 23);      // 2^-e
    if (lane == 0) row_factor[row] = __uint_as_float((uint32_t)(127 + e) << 23);
    const uint4* qr = reinterpret_cast<const uint4*>(q + row * (K >> 1));
    uint4* orow = reinterpret_cast<uint4*>(out + row * K);
    const bool wide = (reinterpret_cast<uintptr_t>(out) & 31) == 0;     // rows are multiples of 128 bytes: a scratch on a 32-byte boundary allows 32-byte stores
#pragma unroll 1
    for (int g = lane; g < G; g += 32) {
        const float sc = bf16_bits_to_f32(sr[g]) * down;        // exact: power-of-two shift
        const uint4 w = qr[g];
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
        uint4 o[4];
        uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const int lo = PERM ? ((int)(ww[i] << (28 - 4 * p))) >> 28      // nibble p
                                    : ((int)(ww[i] << (28 - 8 * p))) >> 28;    // nibble 2p, sign extended
                const int hi = PERM ? ((int)(ww[i] << (12 - 4 * p))) >> 28      // nibble p + 4
                                    : ((int)(ww[i] << (24 - 8 * p))) >> 28;    // nibble 2p + 1
                __half2 h = __floats2half2_rn((float)lo * sc, (float)hi * sc);  // exact products
                ow[i * 4 + p] = *reinterpret_cast<uint32_t*>(&h);
            }
        }
        if (wide) {                                             // whole 32-byte sectors per store instruction
            st_global_v8(orow + g * 4, o[0], o[1]);
            st_global_v8(orow + g * 4 + 2, o[2], o[3]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) orow[g * 4 + i] = o[i];
        }
    }
}

template <bool PERM>
__global__ void __launch_bounds__(256)
dequant_f16_kernel(const uint8_t* __restrict__ q, const __nv_bfloat16* __restrict__ s, __half* __restrict__ out,
                   float* __restrict__ row_factor, long long rows, int K)
{
    const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    dequant_f16_row<PERM>(q, s, out, row_factor, row, K, threadIdx.x & 31);
}

// The same as a grid that is resident as a whole and walks the rows, launched as a programmatic dependent of a
// kernel it does NOT depend on (it widens the weights of later column tiles while that kernel multiplies the
// first ones).  It must not COMPLETE before that kernel has, because whatever follows in the stream is ordered
// behind this grid only: hence the wait at the end.  (Kept apart from the kernel above: with the row loop around
// it the compiler schedules the inner loop less aggressively, 49.6 against 38.9 us for 7168 rows of K = 8192.)
__global__ void __launch_bounds__(256)
dequant_f16_resident_kernel(const uint8_t* __restrict__ q, const __nv_bfloat16* __restrict__ s, __half* __restrict__ out,
                            float* __restrict__ row_factor, long long rows, int K)
{
    for (long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); row < rows; row += (long long)gridDim.x * 8)
        dequant_f16_row<false>(q, s, out, row_factor, row, K, threadIdx.x & 31);
    pdl_wait();
}

// ------------------------------------------------------------------------------------------------
// GEMM
// ------------------------------------------------------------------------------------------------
constexpr int FM = 128, FN = 256;                               // tile; a stage holds 128 bytes of K per row
constexpr int F_ACC = 2;                                        // TMEM accumulators in rotation (128-row tiles)

// How the tiles of a persistent tile kernel's launch become units of work.  Tiles [0, full_tiles) run over the
// whole K and write y.  The others leave raw fp32 accumulators of K ranges in 256 x 256 slots of a scratch area and
// tail_sum_kernel adds a tile's ranges in a fixed order:
//   mode 1  every other tile in `split` equal ranges (slot = unit index behind the whole tiles);
//   mode 2  the other tiles' stages, laid end to end, are dealt to the `ctas` CTAs of the grid as contiguous runs
//           whose bounds are multiples of `gran` stages.  A run is at most one tile long, so it covers the end of one
//           tile (first piece, slot = CTA index) and possibly the start of the next (second piece, slot = ctas +
//           that tile's index among the cut tiles); either piece may be empty.  full_tiles is a multiple of ctas and
//           the grid has exactly `ctas` CTAs, so that CTA c meets the units of run c.
struct UnitPlan { int n_tiles, k_steps, full_tiles, mode, split, ctas, gran; };
struct Unit { int tile, ks0, len, slot; };                        // slot < 0: a whole tile

__host__ __device__ __forceinline__ int unit_count(const UnitPlan& p) {
    return p.full_tiles + (p.mode == 1 ? (p.n_tiles - p.full_tiles) * p.split : p.mode == 2 ? 2 * p.ctas : 0);
}
__host__ __device__ __forceinline__ int run_bound(const UnitPlan& p, int c) {  // first stage of CTA c's run (c = ctas: the end)
    const long long wg = (long long)(p.n_tiles - p.full_tiles) * p.k_steps / p.gran;
    return (int)(wg * c / p.ctas) * p.gran;
}
__host__ __device__ __forceinline__ Unit decode_unit(const UnitPlan& p, int u) {
    if (u < p.full_tiles) return {u, 0, p.k_steps, -1};
    const int v = u - p.full_tiles;
    if (p.mode == 1) {
        const int rs = p.k_steps / p.split;
        return {p.full_tiles + v / p.split, (v % p.split) * rs, rs, v};
    }
    const int j = v / p.ctas, c = v - j * p.ctas;
    const int lo = run_bound(p, c), hi = run_bound(p, c + 1);
    const int tt = lo / p.k_steps, first_end = hi < (tt + 1) * p.k_steps ? hi : (tt + 1) * p.k_steps;
    if (j == 0) return {p.full_tiles + tt, lo - tt * p.k_steps, first_end - lo, c};
    return {p.full_tiles + tt + 1, 0, hi - first_end, p.ctas + tt + 1};
}

// The slots that hold the pieces of cut tile `tt` (index among the cut tiles), in the order in which they are added:
// calls add(slot) for each.  The counterpart of decode_unit for tail_sum_kernel.
template <typename F>
__host__ __device__ __forceinline__ void pieces_of_tile(const UnitPlan& plan, int tt, F&& add) {
    if (plan.mode == 1) {
        for (int r = 0; r < plan.split; ++r) add(tt * plan.split + r);
        return;
    }
    // mode 2: the run that contains the tile's first stage, then every run that starts inside the tile
    const int tb = tt * plan.k_steps, te = tb + plan.k_steps;
    const long long wg = (long long)(plan.n_tiles - plan.full_tiles) * plan.k_steps / plan.gran;
    int c = (int)((long long)(tb / plan.gran) * plan.ctas / wg);
    while (c > 0 && run_bound(plan, c) > tb) --c;
    while (c + 1 < plan.ctas && run_bound(plan, c + 1) <= tb) ++c;          // now bound(c) <= tb < bound(c + 1), or c is the last run
    if (run_bound(plan, c) < tb) {
        if (run_bound(plan, c + 1) > tb) add(plan.ctas + tt);               // second piece of run c: the start of this tile
        ++c;
    }
    for (; c < plan.ctas && run_bound(plan, c) < te; ++c)
        if (run_bound(plan, c + 1) > run_bound(plan, c)) add(c);            // first piece of run c
}

// K-major operand in the 128-byte-swizzled layout TMA writes: rows of 128 B, 8-row groups 1 KB apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;                                     // leading byte offset: unused with swizzle
    d |= (uint64_t)(1024 >> 4) << 32;                           // stride byte offset between 8-row groups
    d |= 1ull << 46;                                            // descriptor version of sm_100
    d |= 2ull << 61;                                            // 128-byte swizzle
    return d;
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Epilogue constants of the two operand kinds the tile kernel serves.
//   fp16-folded operands: y = acc * 2^(e_m + e_n), one factor per row of each operand;
//   int8 codes (per-tensor scale): y = alpha * acc, alpha a host value or a device scalar.
struct TileScale {
    const float* fa;
    const float* fb;
    float alpha;
    const float* alpha_dev;
};

// ------------------------------------------------------------------------------------------------
// The same product with the weights widened INSIDE the kernel (M up to a few thousand rows)
// ------------------------------------------------------------------------------------------------
// The pre-pass over the weights above costs a read of the packed matrix, a write of four times
// as many bytes and their re-read by the GEMM: more than the GEMM itself below M ~ 1000.  Here
// only the activations are widened beforehand; the weight tile arrives packed (TMA, 32 bytes per
// row and stage) and eight warps turn it into the fp16 B operand in shared memory, in exactly the
// 128-byte-swizzled K-major layout a TMA load of fp16 would have produced:
//   nibble -> fp16: (w ^ 0x88888888) puts code + 8 into every nibble; (x >> 4j) & 0x000F000F |
//   0x64006400 is the half2 (1024 + code_j + 8, 1024 + code_{j+4} + 8); minus 1032 gives the codes,
//   times the row-shifted scale gives code * scale, both exact in fp16.
// The octet order 0,4,1,5,2,6,3,7 that falls out is mirrored by the activation pre-pass.
//   warp 0      TMA: fp16 activation tile (128 x 64) + packed weight tile (256 rows x 32 B) per stage
//   warp 1      tcgen05.mma issue (as above)
//   warps 4-7   epilogue (as above)
//   warps 8-23  widening: thread (d, g) owns group g (32 codes) of weight row d of the tile in every stage
constexpr int Q_STAGES = 5;                                       // ring of TMA stages: activation tile + packed weight tile
constexpr int Q_BUFS = 3;                                         // ring of widened (fp16) weight tiles
constexpr int Q_THREADS = 768;
constexpr int QA_BYTES = FM * 128, QB_BYTES = FN * 128, QP_BYTES = FN * 32;
constexpr int Q_STAGE = QA_BYTES + QP_BYTES;                     // 24 KB
constexpr int Q_BOFF = Q_STAGES * Q_STAGE;                       // widened tiles after the TMA ring (1 KB aligned)
constexpr int Q_BARS = Q_BOFF + Q_BUFS * QB_BYTES;
constexpr int Q_TOTAL = Q_BARS + (2 * Q_STAGES + 2 * Q_BUFS + 2 * F_ACC + 1) * 8 + 16 + 1024;

// one word of eight nibbles -> eight fp16 (code * scale), octet order 0,4,1,5,2,6,3,7
__device__ __forceinline__ uint4 widen_word_f16(uint32_t w, __half2 s2) {
    const uint32_t x = w ^ 0x88888888u;
    const __half2 off = __half2half2(__ushort_as_half((unsigned short)0x6408));        // 1032
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t h = ((x >> (4 * j)) & 0x000F000Fu) | 0x64006400u;
        __half2 v = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&h), off), s2);
        o[j] = *reinterpret_cast<uint32_t*>(&v);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// per weight row: 2^e (for the epilogue) and 2^-e (for the widening), e = exponent of its largest scale
__global__ void __launch_bounds__(256)
row_shift_kernel(const __nv_bfloat16* __restrict__ s, float* __restrict__ up, float* __restrict__ down, long long rows, int G)
{
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const unsigned short* sr = reinterpret_cast<const unsigned short*>(s) + row * G;
    unsigned mx = 0;
    for (int g = lane; g < G; g += 32) mx = max(mx, (unsigned)(sr[g] & 0x7fffu));
#pragma unroll
    for (int off = 16; off; off >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    int e = (int)(mx >> 7) - 127;
    e = max(-100, min(100, e));
    if (lane == 0) {
        up[row] = __uint_as_float((uint32_t)(127 + e) << 23);
        down[row] = __uint_as_float((uint32_t)(127 - e) << 23);
    }
}

__global__ void __launch_bounds__(Q_THREADS, 1)
gemm_f16_fused_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_p,
                      const unsigned short* __restrict__ ws, const float* __restrict__ down, const TileScale sc,
                      __half* __restrict__ y, int M, int N, int K, int* __restrict__ err, const UnitPlan plan,
                      float* __restrict__ part)                      // units of work as in the 256-row kernel below; slots of 128 x 256
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + Q_BARS);     // TMA stage landed
    uint64_t* empty = full + Q_STAGES;                               // TMA stage consumed: MMA (A) + 16 widening warps (packed B)
    uint64_t* widened = empty + Q_STAGES;                            // fp16 weight tile written
    uint64_t* bfree = widened + Q_BUFS;                              // fp16 weight tile consumed by the MMA
    uint64_t* acc_full = bfree + Q_BUFS;
    uint64_t* acc_empty = acc_full + F_ACC;
    uint64_t* done_bar = acc_empty + F_ACC;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles_m = (M + FM - 1) / FM, n_units = unit_count(plan);
    const int G = K >> 5;

    if (tid == 0) {
        for (int i = 0; i < Q_STAGES; ++i) { tc::mbar_init(&full[i], 1); tc::mbar_init(&empty[i], 17); }
        for (int i = 0; i < Q_BUFS; ++i) { tc::mbar_init(&widened[i], 16); tc::mbar_init(&bfree[i], 1); }
        for (int i = 0; i < F_ACC; ++i) { tc::mbar_init(&acc_full[i], 1); tc::mbar_init(&acc_empty[i], 4); }
        tc::mbar_init(done_bar, 1);
        tc::mbar_fence_init();
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, 512);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            tc::prefetch_tensormap(&map_a); tc::prefetch_tensormap(&map_p);
            uint32_t slot = 0, phase = 0;
            int issued = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
                const Unit un = decode_unit(plan, u);
                const int t = un.tile;
                const int m0 = (t % tiles_m) * FM, n0 = (t / tiles_m) * FN;
                for (int ks = un.ks0; ks < un.ks0 + un.len; ++ks) {
                    if (!tc::mbar_wait(&empty[slot], phase ^ 1)) { ok = false; break; }
                    uint8_t* st = smem + slot * Q_STAGE;
                    tc::mbar_expect_tx(&full[slot], QA_BYTES + QP_BYTES);
                    tc::tma_load_2d(st, &map_a, &full[slot], ks * 64, m0);
                    tc::tma_load_2d(st + QA_BYTES, &map_p, &full[slot], ks * 32, n0);
                    ++issued;
                    if (++slot == Q_STAGES) { slot = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                atomicExch(err, 1);
                for (int i = 0; i < (issued < Q_STAGES ? issued : Q_STAGES); ++i)
                    for (uint32_t spin = 0; spin < (1u << 16); ++spin)
                        if (tc::mbar_try_wait(&full[i], 0) || tc::mbar_try_wait(&full[i], 1)) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t slot = 0, phase = 0, buf = 0, bphase = 0, ab = 0, aphase = 0;
            const uint32_t idesc = tc::idesc_f16(FN);
            bool ok = true;
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
                const int k_steps = decode_unit(plan, u).len;
                if (k_steps == 0) continue;                                    // an empty piece of a run
                if (!tc::mbar_wait(&acc_empty[ab], aphase ^ 1)) { ok = false; break; }
                tc::tc_fence_after();
                for (int ks = 0; ks < k_steps; ++ks) {
                    if (!tc::mbar_wait(&full[slot], phase) || !tc::mbar_wait(&widened[buf], bphase)) { ok = false; break; }
                    tc::tc_fence_after();
                    const uint32_t sa = tc::smem_u32(smem + slot * Q_STAGE), sb = tc::smem_u32(smem + Q_BOFF + buf * QB_BYTES);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        mma_f16(tmem + ab * FN, smem_desc_sw128(sa + kk * 32), smem_desc_sw128(sb + kk * 32), idesc,
                                (ks | kk) ? 1u : 0u);
                    tc::mma_commit(&empty[slot]);                              // the activation tile of this stage
                    tc::mma_commit(&bfree[buf]);                               // and the widened weight tile are free again
                    if (++slot == Q_STAGES) { slot = 0; phase ^= 1; }
                    if (++buf == Q_BUFS) { buf = 0; bphase ^= 1; }
                }
                if (!ok) break;
                tc::mma_commit(&acc_full[ab]);
                if (++ab == F_ACC) { ab = 0; aphase ^= 1; }
            }
            if (!ok) atomicExch(err, 2);
            tc::mma_commit(done_bar);
            for (uint32_t spin = 0; spin < WUSH_SPIN_LIMIT; ++spin)
                if (tc::mbar_try_wait(done_bar, 0)) break;
        }
    } else if (warp >= 8) {
        // ------------------------------ widening warps -------------------------------------------
        const int d = (tid - 256) & 255, g = (tid - 256) >> 8;     // weight row of the tile, group of the stage
        uint32_t slot = 0, phase = 0, buf = 0, bphase = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
            const Unit un = decode_unit(plan, u);
            const int t = un.tile, ks0 = un.ks0, ks1 = un.ks0 + un.len;          // ks0 is a multiple of 4
            const int n = (t / tiles_m) * FN + d;
            const bool live = n < N;
            const float dn = live ? down[n] : 0.f;
            // scales: one 16-byte load covers this row's 8 groups = 4 stages; the next one is in flight meanwhile
            const uint4* srow = reinterpret_cast<const uint4*>(ws + (size_t)(live ? n : 0) * G);
            const uint4 zero4 = make_uint4(0, 0, 0, 0);
            uint4 s_cur = zero4, s_nxt = live ? __ldg(srow + (ks0 >> 2)) : zero4;
            for (int ks = ks0; ks < ks1; ++ks) {
                if ((ks & 3) == 0) {
                    s_cur = s_nxt;
                    if (live && ks + 4 < ks1) s_nxt = __ldg(srow + (ks >> 2) + 1);
                }
                const uint32_t pair = (ks & 2) ? ((ks & 1) ? s_cur.w : s_cur.z) : ((ks & 1) ? s_cur.y : s_cur.x);   // groups 2ks, 2ks+1
                const float s_f = g ? bf16_hi(pair) : bf16_lo(pair);
                if (!tc::mbar_wait(&full[slot], phase)) { ok = false; break; }
                const uint4 w = *reinterpret_cast<const uint4*>(smem + slot * Q_STAGE + QA_BYTES + d * 32 + g * 16);
                const __half2 s2 = __float2half2_rn(__fmul_rn(s_f, dn));                           // exact shift
                const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
                uint4 o[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) o[c] = widen_word_f16(ww[c], s2);
                __syncwarp();                                      // the packed words of this warp are in registers
                if (lane == 0) tc::mbar_arrive(&empty[slot]);
                if (!tc::mbar_wait(&bfree[buf], bphase ^ 1)) { ok = false; break; }
                uint8_t* brow = smem + Q_BOFF + buf * QB_BYTES + d * 128;
#pragma unroll
                for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(brow + (((g * 4 + c) ^ (d & 7)) << 4)) = o[c];
                tc::fence_proxy_async();                           // generic-proxy writes -> visible to tcgen05.mma
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&widened[buf]);
                if (++slot == Q_STAGES) { slot = 0; phase ^= 1; }
                if (++buf == Q_BUFS) { buf = 0; bphase ^= 1; }
            }
        }
        if (!ok && lane == 0) atomicExch(err, 8);
    } else if (warp >= 4) {
        const int quarter = warp & 3, row = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        uint32_t ab = 0, aphase = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
            const Unit un = decode_unit(plan, u);
            if (un.len == 0) continue;
            const int t = un.tile;
            const int m0 = (t % tiles_m) * FM, n0 = (t / tiles_m) * FN;
            float* prow = un.slot < 0 ? nullptr : part + ((size_t)un.slot * FM + row) * FN;
            if (!tc::mbar_wait(&acc_full[ab], aphase)) { ok = false; break; }
            tc::tc_fence_after();
            const int m = m0 + row;
            const float fm = (m < M) ? sc.fa[m] : 0.f;
#pragma unroll 1
            for (int c = 0; c < FN / 32; ++c) {
                uint32_t v[32];
                tc::tmem_ld32(tmem + lane_base + ab * FN + c * 32, v);
                tc::tmem_ld_wait();
                if (c == FN / 32 - 1) {
                    tc::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(&acc_empty[ab]);
                }
                const int n = n0 + c * 32;
                if (prow) {                                     // 128 bytes per lane: four 32-byte stores
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        st_global_v8(prow + c * 32 + q * 8, make_uint4(v[q * 8], v[q * 8 + 1], v[q * 8 + 2], v[q * 8 + 3]),
                                     make_uint4(v[q * 8 + 4], v[q * 8 + 5], v[q * 8 + 6], v[q * 8 + 7]));
                } else if (m < M && n < N) {
                    __half* yr = y + (size_t)m * N + n;
                    const bool wide = ((reinterpret_cast<uintptr_t>(y) & 31) == 0) && (N & 15) == 0;   // 32-byte stores possible
                    uint4 prev = make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int v8 = 0; v8 < 4; ++v8) {
                        if (n + v8 * 8 + 8 <= N) {
                            const float4 f0 = *reinterpret_cast<const float4*>(sc.fb + n + v8 * 8);
                            const float4 f1 = *reinterpret_cast<const float4*>(sc.fb + n + v8 * 8 + 4);
                            const float fs[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
                            uint32_t o[4];
#pragma unroll
                            for (int p = 0; p < 4; ++p) {
                                __half2 h = __floats2half2_rn(__uint_as_float(v[v8 * 8 + 2 * p]) * (fm * fs[2 * p]),
                                                              __uint_as_float(v[v8 * 8 + 2 * p + 1]) * (fm * fs[2 * p + 1]));
                                o[p] = *reinterpret_cast<uint32_t*>(&h);
                            }
                            const uint4 cur = make_uint4(o[0], o[1], o[2], o[3]);
                            if (!wide) *reinterpret_cast<uint4*>(yr + v8 * 8) = cur;
                            else if (v8 & 1) st_global_v8(yr + (v8 - 1) * 8, prev, cur);
                            else prev = cur;
                        }
                    }
                }
            }
            if (++ab == F_ACC) { ab = 0; aphase ^= 1; }
        }
        if (!ok && lane == 0) atomicExch(err, 4);
    }

    tc::tc_fence_before();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem, 512);
}

// The same kernel on 256 x 256 tiles: every widened weight tile feeds TWO MMAs (activation rows 0-127 and
// 128-255, accumulators in TMEM columns 0-255 and 256-511), which doubles the instruction budget of the
// widening warps per MMA cycle.  The two accumulators fill the whole TMEM, so a tile's epilogue (eight warps)
// does not overlap the next tile's MMAs.
constexpr int R_STAGES = 3, R_BUFS = 3;
constexpr int R_THREADS = 896;                                    // + warps 24-27: epilogue of the upper 128 rows
constexpr int RA_BYTES = 2 * FM * 128;
constexpr int R_STAGE = RA_BYTES + QP_BYTES;                     // 40 KB
constexpr int R_BOFF = R_STAGES * R_STAGE;
constexpr int R_BARS = R_BOFF + R_BUFS * QB_BYTES;
constexpr int R_TOTAL = R_BARS + (2 * R_STAGES + 2 * R_BUFS + 2 * F_ACC + 1) * 8 + 16 + 1024;

//
// Units of work: the first `full_tiles` tiles run over the whole K and write y; every other tile is cut into
// `ksplit` K ranges (few tiles on many multiprocessors: all tiles, full_tiles = 0; many tiles: only those of the
// last, partly filled wave).  A range leaves its raw fp32 accumulators in part[unit - full_tiles][256][256] and
// tail_sum_kernel adds the ranges of a tile in order.  A range is a whole number of 16-byte scale vectors
// (4 stages).
__global__ void __launch_bounds__(R_THREADS, 1)
gemm_f16_fused2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_p,
                      const unsigned short* __restrict__ ws, const float* __restrict__ down, const TileScale sc,
                      __half* __restrict__ y, int M, int N, int K, int* __restrict__ err, const UnitPlan plan,
                      float* __restrict__ part)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + R_BARS);     // TMA stage landed
    uint64_t* empty = full + R_STAGES;                               // TMA stage consumed: MMA (A) + 16 widening warps (packed B)
    uint64_t* widened = empty + R_STAGES;                            // fp16 weight tile written
    uint64_t* bfree = widened + R_BUFS;                              // fp16 weight tile consumed by the MMA
    uint64_t* acc_full = bfree + R_BUFS;
    uint64_t* acc_empty = acc_full + F_ACC;
    uint64_t* done_bar = acc_empty + F_ACC;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles_m = (M + 2 * FM - 1) / (2 * FM), tiles_n = (N + FN - 1) / FN;
    const int n_units = unit_count(plan), G = K >> 5;

    if (tid == 0) {
        for (int i = 0; i < R_STAGES; ++i) { tc::mbar_init(&full[i], 1); tc::mbar_init(&empty[i], 17); }
        for (int i = 0; i < R_BUFS; ++i) { tc::mbar_init(&widened[i], 16); tc::mbar_init(&bfree[i], 1); }
        for (int i = 0; i < F_ACC; ++i) { tc::mbar_init(&acc_full[i], 1); tc::mbar_init(&acc_empty[i], 8); }
        tc::mbar_init(done_bar, 1);
        tc::mbar_fence_init();
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, 512);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            tc::prefetch_tensormap(&map_a); tc::prefetch_tensormap(&map_p);
            uint32_t slot = 0, phase = 0;
            int issued = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
                const Unit un = decode_unit(plan, u);
                const int t = un.tile, ks0 = un.ks0, k_steps = un.len;
                const int m0 = (t % tiles_m) * 2 * FM, n0 = (t / tiles_m) * FN;
                for (int ks = ks0; ks < ks0 + k_steps; ++ks) {
                    if (!tc::mbar_wait(&empty[slot], phase ^ 1)) { ok = false; break; }
                    uint8_t* st = smem + slot * R_STAGE;
                    tc::mbar_expect_tx(&full[slot], RA_BYTES + QP_BYTES);
                    tc::tma_load_2d(st, &map_a, &full[slot], ks * 64, m0);
                    tc::tma_load_2d(st + RA_BYTES, &map_p, &full[slot], ks * 32, n0);
                    ++issued;
                    if (++slot == R_STAGES) { slot = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                atomicExch(err, 1);
                for (int i = 0; i < (issued < R_STAGES ? issued : R_STAGES); ++i)
                    for (uint32_t spin = 0; spin < (1u << 16); ++spin)
                        if (tc::mbar_try_wait(&full[i], 0) || tc::mbar_try_wait(&full[i], 1)) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t slot = 0, phase = 0, buf = 0, bphase = 0, aphase = 0;
            const uint32_t idesc = tc::idesc_f16(FN);
            bool ok = true;
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
                const int k_steps = decode_unit(plan, u).len;
                if (k_steps == 0) continue;                                    // an empty piece of a run
                if (!tc::mbar_wait(&acc_empty[0], aphase ^ 1)) { ok = false; break; }
                tc::tc_fence_after();
                for (int ks = 0; ks < k_steps; ++ks) {
                    if (!tc::mbar_wait(&full[slot], phase) || !tc::mbar_wait(&widened[buf], bphase)) { ok = false; break; }
                    tc::tc_fence_after();
                    const uint32_t sa = tc::smem_u32(smem + slot * R_STAGE), sb = tc::smem_u32(smem + R_BOFF + buf * QB_BYTES);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {                           // rows 0-127 -> columns 0-255, rows 128-255 -> 256-511
                        const uint64_t bdesc = smem_desc_sw128(sb + kk * 32);
                        mma_f16(tmem, smem_desc_sw128(sa + kk * 32), bdesc, idesc, (ks | kk) ? 1u : 0u);
                        mma_f16(tmem + FN, smem_desc_sw128(sa + FM * 128 + kk * 32), bdesc, idesc, (ks | kk) ? 1u : 0u);
                    }
                    tc::mma_commit(&empty[slot]);                              // the activation tile of this stage
                    tc::mma_commit(&bfree[buf]);                               // and the widened weight tile are free again
                    if (++slot == R_STAGES) { slot = 0; phase ^= 1; }
                    if (++buf == R_BUFS) { buf = 0; bphase ^= 1; }
                }
                if (!ok) break;
                tc::mma_commit(&acc_full[0]);
                aphase ^= 1;
            }
            if (!ok) atomicExch(err, 2);
            tc::mma_commit(done_bar);
            for (uint32_t spin = 0; spin < WUSH_SPIN_LIMIT; ++spin)
                if (tc::mbar_try_wait(done_bar, 0)) break;
        }
    } else if (warp >= 8 && warp < 24) {
        // ------------------------------ widening warps -------------------------------------------
        const int d = (tid - 256) & 255, g = (tid - 256) >> 8;     // weight row of the tile, group of the stage
        uint32_t slot = 0, phase = 0, buf = 0, bphase = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
            const Unit un = decode_unit(plan, u);
            const int t = un.tile, ks0 = un.ks0, ks1 = un.ks0 + un.len;          // ks0 is a multiple of 4
            const int n = (t / tiles_m) * FN + d;
            const bool live = n < N;
            const float dn = live ? down[n] : 0.f;
            // scales: one 16-byte load covers this row's 8 groups = 4 stages; the next one is in flight meanwhile
            const uint4* srow = reinterpret_cast<const uint4*>(ws + (size_t)(live ? n : 0) * G);
            const uint4 zero4 = make_uint4(0, 0, 0, 0);
            uint4 s_cur = zero4, s_nxt = live ? __ldg(srow + (ks0 >> 2)) : zero4;
            for (int ks = ks0; ks < ks1; ++ks) {
                if ((ks & 3) == 0) {
                    s_cur = s_nxt;
                    if (live && ks + 4 < ks1) s_nxt = __ldg(srow + (ks >> 2) + 1);
                }
                const uint32_t pair = (ks & 2) ? ((ks & 1) ? s_cur.w : s_cur.z) : ((ks & 1) ? s_cur.y : s_cur.x);   // groups 2ks, 2ks+1
                const float s_f = g ? bf16_hi(pair) : bf16_lo(pair);
                if (!tc::mbar_wait(&full[slot], phase)) { ok = false; break; }
                const uint4 w = *reinterpret_cast<const uint4*>(smem + slot * R_STAGE + RA_BYTES + d * 32 + g * 16);
                const __half2 s2 = __float2half2_rn(__fmul_rn(s_f, dn));                           // exact shift
                const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
                uint4 o[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) o[c] = widen_word_f16(ww[c], s2);
                __syncwarp();                                      // the packed words of this warp are in registers
                if (lane == 0) tc::mbar_arrive(&empty[slot]);
                if (!tc::mbar_wait(&bfree[buf], bphase ^ 1)) { ok = false; break; }
                uint8_t* brow = smem + R_BOFF + buf * QB_BYTES + d * 128;
#pragma unroll
                for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(brow + (((g * 4 + c) ^ (d & 7)) << 4)) = o[c];
                tc::fence_proxy_async();                           // generic-proxy writes -> visible to tcgen05.mma
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&widened[buf]);
                if (++slot == R_STAGES) { slot = 0; phase ^= 1; }
                if (++buf == R_BUFS) { buf = 0; bphase ^= 1; }
            }
        }
        if (!ok && lane == 0) atomicExch(err, 8);
    } else if (warp >= 4) {
        const int quarter = warp & 3, upper = warp >= 24 ? 1 : 0;      // warps 4-7: rows 0-127, warps 24-27: rows 128-255
        const int row = upper * FM + quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t ab = (uint32_t)upper;                            // column block of this half's accumulator
        uint32_t aphase = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
            const Unit un = decode_unit(plan, u);
            if (un.len == 0) continue;
            const int t = un.tile;
            const int m0 = (t % tiles_m) * 2 * FM, n0 = (t / tiles_m) * FN;
            float* prow = un.slot < 0 ? nullptr : part + ((size_t)un.slot * (2 * FM) + row) * FN;
            if (!tc::mbar_wait(&acc_full[0], aphase)) { ok = false; break; }
            tc::tc_fence_after();
            const int m = m0 + row;
            const float fm = (m < M) ? sc.fa[m] : 0.f;
#pragma unroll 1
            for (int c = 0; c < FN / 32; ++c) {
                uint32_t v[32];
                tc::tmem_ld32(tmem + lane_base + ab * FN + c * 32, v);
                tc::tmem_ld_wait();
                if (c == FN / 32 - 1) {
                    tc::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(&acc_empty[0]);
                }
                const int n = n0 + c * 32;
                if (prow) {                                     // 128 bytes per lane: four 32-byte stores
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        st_global_v8(prow + c * 32 + q * 8, make_uint4(v[q * 8], v[q * 8 + 1], v[q * 8 + 2], v[q * 8 + 3]),
                                     make_uint4(v[q * 8 + 4], v[q * 8 + 5], v[q * 8 + 6], v[q * 8 + 7]));
                } else if (m < M && n < N) {
                    __half* yr = y + (size_t)m * N + n;
                    const bool wide = ((reinterpret_cast<uintptr_t>(y) & 31) == 0) && (N & 15) == 0;   // 32-byte stores possible
                    uint4 prev = make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int v8 = 0; v8 < 4; ++v8) {
                        if (n + v8 * 8 + 8 <= N) {
                            const float4 f0 = *reinterpret_cast<const float4*>(sc.fb + n + v8 * 8);
                            const float4 f1 = *reinterpret_cast<const float4*>(sc.fb + n + v8 * 8 + 4);
                            const float fs[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
                            uint32_t o[4];
#pragma unroll
                            for (int p = 0; p < 4; ++p) {
                                __half2 h = __floats2half2_rn(__uint_as_float(v[v8 * 8 + 2 * p]) * (fm * fs[2 * p]),
                                                              __uint_as_float(v[v8 * 8 + 2 * p + 1]) * (fm * fs[2 * p + 1]));
                                o[p] = *reinterpret_cast<uint32_t*>(&h);
                            }
                            const uint4 cur = make_uint4(o[0], o[1], o[2], o[3]);
                            if (!wide) *reinterpret_cast<uint4*>(yr + v8 * 8) = cur;
                            else if (v8 & 1) st_global_v8(yr + (v8 - 1) * 8, prev, cur);
                            else prev = cur;
                        }
                    }
                }
            }
            aphase ^= 1;
        }
        if (!ok && lane == 0) atomicExch(err, 4);
    }

    tc::tc_fence_before();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------------------
// Pre-widened operands on 256 x 256 tiles (M > 2048)
// ------------------------------------------------------------------------------------------------
// TMA (128-byte swizzle) -> ring of stages -> tcgen05.mma -> TMEM -> epilogue warps; one weight tile per
// stage feeds two MMA groups
// (activation rows 0-127 -> TMEM columns 0-255, rows 128-255 -> columns 256-511): 64 KB of TMA writes
// and 96 KB of operand reads per 1240 MMA cycles instead of 48 + 48 KB per 620, which is what the
// shared memory of a multiprocessor can sustain.  The accumulator pair fills the TMEM, so the epilogue
// of a tile (eight warps) does not overlap the next tile's MMAs.
constexpr int T_STAGES = 3;
constexpr int T_THREADS = 384;                                    // warp 0 TMA, warp 1 MMA, warps 4-7 / 8-11 epilogue halves
constexpr int TA_BYTES = 2 * FM * 128, TB_BYTES = FN * 128;
constexpr int T_STAGE = TA_BYTES + TB_BYTES;                     // 64 KB
constexpr int T_BARS = T_STAGES * T_STAGE;
constexpr int T_TOTAL = T_BARS + (2 * T_STAGES + 2 + 1) * 8 + 16 + 1024;

template <bool I8>
__global__ void __launch_bounds__(T_THREADS, 1)
gemm_tile2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TileScale sc,
                      __half* __restrict__ y, int M, int N, int K, int* __restrict__ err,
                      int tile_n_first, int tile_n_count,                     // the column tiles this launch covers
                      const UnitPlan plan, float* __restrict__ part)          // tiles taken whole; K ranges of the others
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + T_BARS);
    uint64_t* empty = full + T_STAGES;
    uint64_t* acc_full = empty + T_STAGES;
    uint64_t* acc_empty = acc_full + 1;
    uint64_t* done_bar = acc_empty + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles_m = (M + 2 * FM - 1) / (2 * FM), n_tiles = tiles_m * tile_n_count;
    const int k_steps = K / (I8 ? 128 : 64);                 // a stage row is 128 bytes either way
    const int n_units = unit_count(plan);                    // whole tiles, then K ranges of the last wave's tiles

    // A dependent launched behind this grid (the widening of the next column tiles) may start as soon as
    // every CTA is resident: it runs in the threads and registers this kernel leaves free.
    pdl_launch_dependents();
    if (tid == 0) {
        for (int i = 0; i < T_STAGES; ++i) { tc::mbar_init(&full[i], 1); tc::mbar_init(&empty[i], 1); }
        tc::mbar_init(acc_full, 1);
        tc::mbar_init(acc_empty, 8);
        tc::mbar_init(done_bar, 1);
        tc::mbar_fence_init();
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, 512);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            tc::prefetch_tensormap(&map_a); tc::prefetch_tensormap(&map_b);
            uint32_t slot = 0, phase = 0;
            int issued = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
                const Unit un = decode_unit(plan, u);
                const int t = un.tile, ks_first = un.ks0, ks_end = un.ks0 + un.len;
                const int m0 = (t % tiles_m) * 2 * FM, n0 = (tile_n_first + t / tiles_m) * FN;
                for (int ks = ks_first; ks < ks_end; ++ks) {
                    if (!tc::mbar_wait(&empty[slot], phase ^ 1)) { ok = false; break; }
                    uint8_t* st = smem + slot * T_STAGE;
                    tc::mbar_expect_tx(&full[slot], T_STAGE);
                    tc::tma_load_2d(st, &map_a, &full[slot], ks * (I8 ? 128 : 64), m0);
                    tc::tma_load_2d(st + TA_BYTES, &map_b, &full[slot], ks * (I8 ? 128 : 64), n0);
                    ++issued;
                    if (++slot == T_STAGES) { slot = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                atomicExch(err, 1);
                for (int i = 0; i < (issued < T_STAGES ? issued : T_STAGES); ++i)
                    for (uint32_t spin = 0; spin < (1u << 16); ++spin)
                        if (tc::mbar_try_wait(&full[i], 0) || tc::mbar_try_wait(&full[i], 1)) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t slot = 0, phase = 0, aphase = 0;
            const uint32_t idesc = I8 ? tc::idesc_i8(FN) : tc::idesc_f16(FN);
            bool ok = true;
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
                const int unit_steps = decode_unit(plan, u).len;
                if (unit_steps == 0) continue;                                 // an empty piece of a run
                if (!tc::mbar_wait(acc_empty, aphase ^ 1)) { ok = false; break; }
                tc::tc_fence_after();
                for (int ks = 0; ks < unit_steps; ++ks) {
                    if (!tc::mbar_wait(&full[slot], phase)) { ok = false; break; }
                    tc::tc_fence_after();
                    const uint32_t sa = tc::smem_u32(smem + slot * T_STAGE), sb = sa + TA_BYTES;
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint64_t bdesc = smem_desc_sw128(sb + kk * 32);
                        if constexpr (I8) {
                            tc::mma_i8(tmem, smem_desc_sw128(sa + kk * 32), bdesc, idesc, (ks | kk) ? 1u : 0u);
                            tc::mma_i8(tmem + FN, smem_desc_sw128(sa + FM * 128 + kk * 32), bdesc, idesc, (ks | kk) ? 1u : 0u);
                        } else {
                            mma_f16(tmem, smem_desc_sw128(sa + kk * 32), bdesc, idesc, (ks | kk) ? 1u : 0u);
                            mma_f16(tmem + FN, smem_desc_sw128(sa + FM * 128 + kk * 32), bdesc, idesc, (ks | kk) ? 1u : 0u);
                        }
                    }
                    tc::mma_commit(&empty[slot]);
                    if (++slot == T_STAGES) { slot = 0; phase ^= 1; }
                }
                if (!ok) break;
                tc::mma_commit(acc_full);
                aphase ^= 1;
            }
            if (!ok) atomicExch(err, 2);
            tc::mma_commit(done_bar);
            for (uint32_t spin = 0; spin < WUSH_SPIN_LIMIT; ++spin)
                if (tc::mbar_try_wait(done_bar, 0)) break;
        }
    } else if (warp >= 4) {
        const int quarter = warp & 3, upper = warp >= 8 ? 1 : 0;        // warps 4-7: rows 0-127, warps 8-11: rows 128-255
        const int row = upper * FM + quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        uint32_t aphase = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
            const Unit un = decode_unit(plan, u);
            if (un.len == 0) continue;
            const int t = un.tile;
            const int m0 = (t % tiles_m) * 2 * FM, n0 = (tile_n_first + t / tiles_m) * FN;
            // a K range of a cut tile: raw fp32 (int32) accumulators, 256 x 256 per slot, row-major
            float* prow = un.slot < 0 ? nullptr : part + ((size_t)un.slot * (2 * FM) + row) * FN;
            if (!tc::mbar_wait(acc_full, aphase)) { ok = false; break; }
            tc::tc_fence_after();
            const int m = m0 + row;
            float fm;
            if constexpr (I8) fm = sc.alpha_dev ? __ldg(sc.alpha_dev) : sc.alpha;
            else fm = (m < M) ? sc.fa[m] : 0.f;
#pragma unroll 1
            for (int c = 0; c < FN / 32; ++c) {
                uint32_t v[32];
                tc::tmem_ld32(tmem + lane_base + upper * FN + c * 32, v);
                tc::tmem_ld_wait();
                if (c == FN / 32 - 1) {
                    tc::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(acc_empty);
                }
                const int n = n0 + c * 32;
                if (prow) {                                     // 128 bytes per lane: four 32-byte stores
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        st_global_v8(prow + c * 32 + q * 8, make_uint4(v[q * 8], v[q * 8 + 1], v[q * 8 + 2], v[q * 8 + 3]),
                                     make_uint4(v[q * 8 + 4], v[q * 8 + 5], v[q * 8 + 6], v[q * 8 + 7]));
                } else if (m < M && n < N) {
                    __half* yr = y + (size_t)m * N + n;
                    const bool wide = ((reinterpret_cast<uintptr_t>(y) & 31) == 0) && (N & 15) == 0;   // 32-byte stores possible
                    uint4 prev = make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int v8 = 0; v8 < 4; ++v8) {
                        if (n + v8 * 8 + 8 <= N) {
                            uint32_t o[4];
                            if constexpr (I8) {
#pragma unroll
                                for (int p = 0; p < 4; ++p) {                  // |acc| < 2^24: the conversion is exact
                                    __half2 h = __floats2half2_rn(__fmul_rn(fm, (float)(int)v[v8 * 8 + 2 * p]),
                                                                  __fmul_rn(fm, (float)(int)v[v8 * 8 + 2 * p + 1]));
                                    o[p] = *reinterpret_cast<uint32_t*>(&h);
                                }
                            } else {
                                const float4 f0 = *reinterpret_cast<const float4*>(sc.fb + n + v8 * 8);
                                const float4 f1 = *reinterpret_cast<const float4*>(sc.fb + n + v8 * 8 + 4);
                                const float fs[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
#pragma unroll
                                for (int p = 0; p < 4; ++p) {
                                    __half2 h = __floats2half2_rn(__uint_as_float(v[v8 * 8 + 2 * p]) * (fm * fs[2 * p]),
                                                                  __uint_as_float(v[v8 * 8 + 2 * p + 1]) * (fm * fs[2 * p + 1]));
                                    o[p] = *reinterpret_cast<uint32_t*>(&h);
                                }
                            }
                            const uint4 cur = make_uint4(o[0], o[1], o[2], o[3]);
                            if (!wide) *reinterpret_cast<uint4*>(yr + v8 * 8) = cur;
                            else if (v8 & 1) st_global_v8(yr + (v8 - 1) * 8, prev, cur);
                            else prev = cur;
                        }
                    }
                }
            }
            aphase ^= 1;
        }
        if (!ok && lane == 0) atomicExch(err, 4);
    }

    tc::tc_fence_before();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem, 512);
}

// Sum of the K ranges of the cut tiles (in a fixed order: deterministic), scaled and rounded to fp16 once.  One
// thread per 8 consecutive outputs of a row of a 256 x 256 tile; slots as written by the tile kernels.
template <bool I8, int ROWS>
__global__ void __launch_bounds__(256)
tail_sum_kernel(const float* __restrict__ part, const TileScale sc, __half* __restrict__ y, int M, int N, int tiles_m,
                int tile_n_first, const UnitPlan plan)
{
    const int tt = blockIdx.y;                                          // cut tile
    const int e = blockIdx.x * 256 + threadIdx.x;                       // 8-output vector inside the tile
    const int row = e >> 5, col = (e & 31) * 8;
    const int t = plan.full_tiles + tt;
    const int m = (t % tiles_m) * ROWS + row, n = (tile_n_first + t / tiles_m) * FN + col;
    if (m >= M || n + 8 > N) return;
    const float* p = part + (size_t)row * FN + col;                     // + slot * ROWS * 256
    constexpr size_t SLOT = (size_t)ROWS * FN;
    float acc[8];
    int iacc[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) { acc[q] = 0.f; iacc[q] = 0; }
    auto add = [&](int slot) {
        const float4 a = *reinterpret_cast<const float4*>(p + slot * SLOT);
        const float4 b = *reinterpret_cast<const float4*>(p + slot * SLOT + 4);
        const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            if constexpr (I8) iacc[q] += __float_as_int(f[q]);
            else acc[q] += f[q];
        }
    };
    pieces_of_tile(plan, tt, add);
    float fs[8];
    float fm;
    if constexpr (I8) {
        fm = sc.alpha_dev ? __ldg(sc.alpha_dev) : sc.alpha;
#pragma unroll
        for (int q = 0; q < 8; ++q) { acc[q] = (float)iacc[q]; fs[q] = 1.f; }
    } else {
        fm = sc.fa[m];
        const float4 f0 = *reinterpret_cast<const float4*>(sc.fb + n), f1 = *reinterpret_cast<const float4*>(sc.fb + n + 4);
        fs[0] = f0.x; fs[1] = f0.y; fs[2] = f0.z; fs[3] = f0.w; fs[4] = f1.x; fs[5] = f1.y; fs[6] = f1.z; fs[7] = f1.w;
    }
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        __half2 h;
        if constexpr (I8) h = __floats2half2_rn(__fmul_rn(fm, acc[2 * q]), __fmul_rn(fm, acc[2 * q + 1]));
        else h = __floats2half2_rn(acc[2 * q] * (fm * fs[2 * q]), acc[2 * q + 1] * (fm * fs[2 * q + 1]));
        o[q] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(y + (size_t)m * N + n) = make_uint4(o[0], o[1], o[2], o[3]);
}

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace

int pair_set_attributes();
int pair_launch(bool i8, const void* a, const void* b, const float* fa, const float* fb, float alpha, const float* alpha_dev,
                void* y, int64_t M, int64_t N, int64_t K, int* err, cudaStream_t st, int tile_n_first = 0, int tile_n_count = -1);
int pairs_resident();

// Which tile kernel the pre-widened routes run on.  Measured A/B on one B200, M = 4096, N = 57344, K = 8192, whole op
// (us, burst of 3 calls / mean of 100 back-to-back calls under the 1 kW power cap):
//   fp16-folded (kind::f16):  single-CTA 256 x 256 tiles 2939 / 3220     CTA pairs 3035 / 3459     (cuBLAS fp16 GEMM alone 2480 / 2730)
//   per-tensor  (kind::i8):   single-CTA 1375 / 1464                      CTA pairs 1316 / 1403
// The pair kernel keeps the tensor pipe busier (87 % of elapsed cycles against 71 % in ncu) but the f16 product is
// limited by the power cap, not by shared-memory traffic, so pairs only pay where the operand bytes per MMA cycle
// are twice as many: kind::i8.  WUSH_TILE_KERNEL=pair|single overrides the choice (read per call) for measurements.
static bool use_pair_tiles(bool i8)
{
    if (const char* v = std::getenv("WUSH_TILE_KERNEL")) {
        if (v[0] == 'p') return true;
        if (v[0] == 's') return false;
    }
    return i8;
}

int f16_set_attributes()
{
    if (int s = resolve_tensor_map_encoder()) return s;
    if (int s = pair_set_attributes()) return s;
    cudaError_t e = cudaFuncSetAttribute(gemm_f16_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Q_TOTAL);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_f16_fused2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, R_TOTAL);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tile2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, T_TOTAL);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tile2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, T_TOTAL);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "tile GEMM: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    return WUSH_OK;
}

// K in whole 64-element stages, 16-byte output vectors and factor vectors.
bool f16_supported(int64_t M, int64_t N, int64_t K) { return M >= 1 && K % 64 == 0 && N % 8 == 0; }

// Rows up to which the weights are widened inside the GEMM (no fp16 copy of W in the scratch).  Measured at
// K = 8192, N = 57344 (us, in-kernel widening vs weight pre-pass): M = 128: 209 vs 464, 256: 277 vs 529,
// 512: 517 vs 664, 1024: 872 vs 983, 2048: 1714 vs 1789, 4096: 3516 vs 3267; with the weight pre-pass overlapped
// with the GEMM (f16_dispatch): 512: 523 vs 766, 1024: 888 vs 1065, 1536: 1259 vs 1297, 2048: 1636 vs 1632.
constexpr int64_t FUSED_MAX_ROWS = 2048;
static bool use_fused(int64_t M, int64_t N, int64_t K) { return M <= FUSED_MAX_ROWS && K % 256 == 0; }   // whole 16-byte scale vectors

// K ranges of the 256-row in-kernel-widening kernel: as many as keep every multiprocessor busy when the
// tiles alone would not (N = 8192, M = 256: 32 tiles), each a whole number of scale vectors and at least
// 16 stages long.  More than one range also sends M <= 128 to the 256-row kernel (half-empty tiles, but
// all multiprocessors at work).
int f16_fused_split(int64_t M, int64_t N, int64_t K)
{
    if (!use_fused(M, N, K)) return 1;
    const int64_t tiles = ((M + 2 * FM - 1) / (2 * FM)) * ((N + FN - 1) / FN), stages = K / 64;
    int s = 1;
    while (s < 8 && tiles * s * 2 <= sm_count()) s *= 2;
    while (s > 1 && (stages % (4 * s) != 0 || stages / s < 16)) s >>= 1;
    return s;
}

// scratch: error word | fp16 activations (M x K) | [fp16 weights (N x K), unless widened in-kernel] |
// 2^e per row of each | 2^-e per weight row | [fp32 partial results of the K ranges]
// `fused` = the weights are widened inside the GEMM (no fp16 copy of W).  The route is decided ONCE per
// call (f16_takes_fused) and the scratch is checked against the layout of that route.
static size_t f16_layout_bytes(int64_t M, int64_t N, int64_t K, bool fused)
{
    const size_t w16 = fused ? 0 : align256((size_t)N * K * 2);
    return 256 + align256((size_t)M * K * 2) + w16 + align256((size_t)M * 4) + 2 * align256((size_t)N * 4);
}

// The in-kernel widening reads the weight scales as 16-byte vectors: besides the shape it needs `ws` on a
// 16-byte boundary.  A caller whose scale pointer is only 2-byte aligned gets the pre-widened route and
// must bring the scratch for it.
static bool f16_takes_fused(int64_t M, int64_t N, int64_t K, const void* ws) { return use_fused(M, N, K) && aligned16(ws); }

// The _min form leaves the partial results out: with that much the product runs without the K split
// (for a 16-byte-aligned `ws`, which is what wush_w4a4_gemm_workspace_bytes assumes).
size_t f16_workspace_bytes_min(int64_t M, int64_t N, int64_t K) { return f16_layout_bytes(M, N, K, use_fused(M, N, K)); }

// Room for the fp32 accumulators of the K ranges into which the tile kernels cut the tiles of their last, partly
// filled wave: at most one 256 x 256 piece per multiprocessor plus one per cut tile.
static size_t tail_part_bytes() { return (size_t)2 * sm_count() * (2 * FM) * FN * 4; }

size_t f16_workspace_bytes(int64_t M, int64_t N, int64_t K)
{
    // K ranges exist on the pre-widened route, on the 256-row kernel with in-kernel widening (M > 128) and where few
    // tiles are cut into ranges as a whole; their accumulators live behind the layout, on a 256-byte boundary
    return f16_workspace_bytes_min(M, N, K) + tail_part_bytes() + 256;
}

// The last wave of a persistent tile grid is rarely full (M = 4096, K = 8192: 3584 tiles are 24.2 waves of 148; a
// shard of 7168 columns 3.03; M = 256 at N = 57344 1.51).  The tiles beyond the whole waves are cut along K, either
// into a power-of-two number of equal ranges that all fit one round (mode 1), or -- when they are too many for
// that -- by dealing their stages to all CTAs as contiguous runs (mode 2); tail_sum_kernel adds the pieces.
// The choice is by estimate: rounds of stages at `step_us` each, plus what the fp32 pieces cost (measured:
// about 0.13 us per 256 x 256 piece written and read back, 5 us for the summing kernel), against one whole round.
// `workers` = CTAs of the grid; 0 = one per SM of the current device.
static UnitPlan plan_units(int64_t tiles, int k_steps, bool room, int gran, double step_us, double piece_us = 0.13,
                           int workers = 0)
{
    const int sms = workers > 0 ? workers : sm_count();
    UnitPlan p = {(int)tiles, k_steps, (int)tiles, 0, 1, sms, gran};
    const char* v = std::getenv("WUSH_TAIL_SPLIT");                    // 0: never cut; 1 / 2: only that mode (measurements, tests)
    if (!room || (v && v[0] == '0')) return p;
    const int full = (int)(tiles / sms) * sms, tail = (int)tiles - full;
    if (tail == 0) return p;
    double best = k_steps * step_us;                                   // the last wave as it is
    int r = 1;
    while (tail * r * 2 <= sms && k_steps % (r * 2) == 0 && k_steps / (r * 2) >= 4 && (k_steps / (r * 2)) % gran == 0) r *= 2;
    if (r > 1 && !(v && v[0] == '2')) {
        const double est = (k_steps / r) * step_us + tail * r * piece_us + 5.0;
        if (est < best || (v && v[0] == '1')) { best = est; p.full_tiles = full; p.mode = 1; p.split = r; }
    }
    if (k_steps % gran == 0 && !(v && v[0] == '1')) {
        const long long wg = (long long)tail * k_steps / gran;
        const double est = (double)((wg + sms - 1) / sms) * gran * step_us + (sms + tail) * piece_us + 5.0;
        if (wg >= sms && (est < best || (v && v[0] == '2'))) { best = est; p.full_tiles = full; p.mode = 2; p.split = 1; }
    }
    return p;
}

static int f16_fused_dispatch(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N,
                              int64_t K, void* y, void* workspace, size_t workspace_bytes, cudaStream_t st, int* sticky_err)
{
    uint8_t* base = reinterpret_cast<uint8_t*>(workspace);
    int* err = sticky_err ? sticky_err : reinterpret_cast<int*>(base);
    __half* a16 = reinterpret_cast<__half*>(base + 256);
    float* fa = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(a16) + align256((size_t)M * K * 2));
    float* fb = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(fa) + align256((size_t)M * 4));
    float* dn = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(fb) + align256((size_t)N * 4));
    // accumulators of K ranges: behind the layout, on the next 256-byte boundary of the address (32-byte stores)
    const uintptr_t part_addr = (reinterpret_cast<uintptr_t>(dn) + align256((size_t)N * 4) + 255) & ~uintptr_t(255);
    const bool part_room = part_addr + tail_part_bytes() <= reinterpret_cast<uintptr_t>(base) + workspace_bytes;
    float* part = part_room ? reinterpret_cast<float*>(part_addr) : nullptr;
    int split = f16_fused_split(M, N, K);
    if (!part_room || !aligned16(y)) split = 1;                          // scratch without room for the partial results
    if (!sticky_err) {
        cudaError_t e = cudaMemsetAsync(err, 0, sizeof(int), st);
        if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    }
    dequant_f16_kernel<true><<<(unsigned)((M + 7) / 8), 256, 0, st>>>(xq, (const __nv_bfloat16*)xs, a16, fa, (long long)M, (int)K);
    row_shift_kernel<<<(unsigned)((N + 7) / 8), 256, 0, st>>>((const __nv_bfloat16*)ws, fb, dn, (long long)N, (int)(K / 32));
    if (int s = check_launch("f16 pre-pass")) return s;
    CUtensorMap ma, mp;
    int s;
    const bool wide = M > FM || split > 1;                             // 256-row tiles: more than one 128-row tile, or K ranges
    if ((s = make_map_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a16, K, M, 64, wide ? 2 * FM : FM, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
    if ((s = make_map_2d(&mp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, K / 2, N, 32, FN, CU_TENSOR_MAP_SWIZZLE_NONE))) return s;
    const int tile_rows = wide ? 2 * FM : FM;
    const int64_t tiles = ((M + tile_rows - 1) / tile_rows) * ((N + FN - 1) / FN);
    const TileScale sc = {fa, fb, 0.f, nullptr};
    if (wide) {
        // few tiles: every tile in `split` K ranges; many tiles: only those of the last, partly filled wave
        UnitPlan up = {(int)tiles, (int)(K / 64), 0, 1, split, sm_count(), 4};
        if (split == 1) up = plan_units(tiles, (int)(K / 64), part_room && aligned16(y), 4, 1.07);
        const int64_t units = up.mode == 2 ? sm_count()
                                           : up.full_tiles + (up.mode == 1 ? (tiles - up.full_tiles) * up.split : 0);
        gemm_f16_fused2_kernel<<<(int)std::min<int64_t>(units, sm_count()), R_THREADS, R_TOTAL, st>>>(
            ma, mp, (const unsigned short*)ws, dn, sc, (__half*)y, (int)M, (int)N, (int)K, err, up, part);
        if (int s2 = check_launch("gemm_f16_fused")) return s2;
        if (up.mode != 0) {
            const dim3 grid((2 * FM) * FN / 8 / 256, (unsigned)(tiles - up.full_tiles));
            tail_sum_kernel<false, 2 * FM><<<grid, 256, 0, st>>>(part, sc, (__half*)y, (int)M, (int)N, (int)((M + 2 * FM - 1) / (2 * FM)), 0, up);
            return check_launch("tail_sum");
        }
        return WUSH_OK;
    }
    const UnitPlan up = plan_units(tiles, (int)(K / 64), part_room && aligned16(y), 4, 0.81, 0.07);
    const int64_t units = up.mode == 2 ? sm_count() : up.full_tiles + (up.mode == 1 ? (tiles - up.full_tiles) * up.split : 0);
    gemm_f16_fused_kernel<<<(int)std::min<int64_t>(units, sm_count()), Q_THREADS, Q_TOTAL, st>>>(
        ma, mp, (const unsigned short*)ws, dn, sc, (__half*)y, (int)M, (int)N, (int)K, err, up, part);
    if (int s2 = check_launch("gemm_f16_fused")) return s2;
    if (up.mode != 0) {
        const dim3 grid(FM * FN / 8 / 256, (unsigned)(tiles - up.full_tiles));
        tail_sum_kernel<false, FM><<<grid, 256, 0, st>>>(part, sc, (__half*)y, (int)M, (int)N, (int)((M + FM - 1) / FM), 0, up);
        return check_launch("tail_sum");
    }
    return WUSH_OK;
}

template <bool I8>
static int launch_tile2(const CUtensorMap& ma, const CUtensorMap& mb, const TileScale& sc, void* y, int64_t M, int64_t N, int64_t K,
                        int* err, int tile_n_first, int tile_n_count, float* part, cudaStream_t st)
{
    const int tiles_m = (int)((M + 2 * FM - 1) / (2 * FM));
    const int64_t tiles = (int64_t)tiles_m * tile_n_count;
    const UnitPlan up = plan_units(tiles, (int)(K / (I8 ? 128 : 64)), part != nullptr, 1, I8 ? 0.4 : 0.8);
    const int64_t units = up.mode == 2 ? sm_count() : up.full_tiles + (up.mode == 1 ? (tiles - up.full_tiles) * up.split : 0);
    gemm_tile2_kernel<I8><<<(int)std::min<int64_t>(units, sm_count()), T_THREADS, T_TOTAL, st>>>(
        ma, mb, sc, (__half*)y, (int)M, (int)N, (int)K, err, tile_n_first, tile_n_count, up, part);
    if (int s = check_launch("gemm_tile2")) return s;
    if (up.mode != 0) {
        const dim3 grid((2 * FM) * FN / 8 / 256, (unsigned)(tiles - up.full_tiles));
        tail_sum_kernel<I8, 2 * FM><<<grid, 256, 0, st>>>(part, sc, (__half*)y, (int)M, (int)N, tiles_m, tile_n_first, up);
        return check_launch("tail_sum");
    }
    return WUSH_OK;
}

// `sticky_err`: where the kernels record a bounded wait that gave up.  Null = word 0 of the scratch, cleared
// at the start of every call; otherwise a word the caller owns, which is only ever set (never cleared here).
int f16_dispatch(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N, int64_t K,
                 void* y, void* workspace, size_t workspace_bytes, cudaStream_t st, int* sticky_err)
{
    if (!aligned16(y) || !aligned16(workspace))
        return fail(WUSH_ERR_INVALID_ARGUMENT, "w4a4_gemm(f16): output and workspace must be 16-byte aligned");
    if ((reinterpret_cast<uintptr_t>(xs) | reinterpret_cast<uintptr_t>(ws)) & 1u)
        return fail(WUSH_ERR_INVALID_ARGUMENT, "w4a4_gemm(f16): the bf16 scales must be 2-byte aligned");
    const bool fused = f16_takes_fused(M, N, K, ws);                  // decided once; sizes the scratch below
    const size_t need = f16_layout_bytes(M, N, K, fused);
    if (workspace_bytes < need)
        return fail(WUSH_ERR_WORKSPACE,
                    "w4a4_gemm(f16): workspace of %zu bytes needed, %zu given%s", need, workspace_bytes,
                    (!fused && use_fused(M, N, K))
                        ? " (the weight scales are not 16-byte aligned, so the route with an fp16 copy of the weights is taken)"
                        : "");
    if (fused) return f16_fused_dispatch(xq, xs, wq, ws, M, N, K, y, workspace, workspace_bytes, st, sticky_err);
    uint8_t* base = reinterpret_cast<uint8_t*>(workspace);
    int* err = sticky_err ? sticky_err : reinterpret_cast<int*>(base);
    __half* a16 = reinterpret_cast<__half*>(base + 256);
    __half* b16 = reinterpret_cast<__half*>(base + 256 + align256((size_t)M * K * 2));
    float* fa = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(b16) + align256((size_t)N * K * 2));
    float* fb = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(fa) + align256((size_t)M * 4));
    if (!sticky_err) {
        cudaError_t e = cudaMemsetAsync(err, 0, sizeof(int), st);
        if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    }
    const __nv_bfloat16* ws16 = (const __nv_bfloat16*)ws;
    dequant_f16_kernel<false><<<(unsigned)((M + 7) / 8), 256, 0, st>>>(xq, (const __nv_bfloat16*)xs, a16, fa, (long long)M, (int)K);
    if (use_pair_tiles(false)) {
        dequant_f16_kernel<false><<<(unsigned)((N + 7) / 8), 256, 0, st>>>(wq, ws16, b16, fb, (long long)N, (int)K);
        if (int s = check_launch("dequant_f16")) return s;
        return pair_launch(false, a16, b16, fa, fb, 0.f, nullptr, y, M, N, K, err, st);
    }
    // The weight pre-pass is a tenth of the whole product at prefill sizes (N = 57344, K = 8192: 268 us of 2.87 ms,
    // 1.2 GB moved) and bound by HBM, while the GEMM is bound by the tensor pipe and the power cap.  So only the
    // first `head` column tiles are widened up front -- as many as make whole waves of tiles --; the rest is
    // widened by a programmatic dependent of the GEMM over those tiles, in the threads and registers the
    // persistent GEMM CTAs leave free, and a second GEMM launch takes the remaining column tiles.
    const int tiles_m = (int)((M + 2 * FM - 1) / (2 * FM)), tiles_n = (int)((N + FN - 1) / FN);
    int head = tiles_n;
    {
        int a = tiles_m, b = sm_count();
        while (b) { const int t = a % b; a = b; b = t; }                 // a = gcd(tiles_m, multiprocessors)
        const int wave_cols = sm_count() / a;                             // column tiles that make whole waves
        const char* v = std::getenv("WUSH_PREPASS_OVERLAP");              // 0 switches the overlap off (measurements)
        if (!(v && v[0] == '0') && tiles_n >= 3 * wave_cols) head = wave_cols;
    }
    const long long head_rows = std::min<long long>((long long)head * FN, N);
    dequant_f16_kernel<false><<<(unsigned)((head_rows + 7) / 8), 256, 0, st>>>(wq, ws16, b16, fb, head_rows, (int)K);
    if (int s = check_launch("dequant_f16")) return s;
    CUtensorMap ma, mb;
    int s;
    if ((s = make_map_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a16, K, M, 64, 2 * FM, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
    if ((s = make_map_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, b16, K, N, 64, FN, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
    const TileScale sc = {fa, fb, 0.f, nullptr};
    // the K ranges of the last wave's tiles need room behind the layout of this route
    // (the tile kernel writes them with 32-byte stores: the area starts on the next 256-byte boundary of the ADDRESS,
    // whatever the alignment of the scratch itself)
    const uintptr_t part_addr = (reinterpret_cast<uintptr_t>(base) + f16_layout_bytes(M, N, K, false) + 255) & ~uintptr_t(255);
    float* part = part_addr + tail_part_bytes() <= reinterpret_cast<uintptr_t>(base) + workspace_bytes
                      ? reinterpret_cast<float*>(part_addr) : nullptr;
    if ((s = launch_tile2<false>(ma, mb, sc, y, M, N, K, err, 0, head, head < tiles_n ? nullptr : part, st))) return s;
    if (head < tiles_n) {
        const long long rest = N - head_rows;
        // One CTA of 8 warps per multiprocessor, all resident beside the GEMM (measured, whole product in us at
        // M = 4096, N = 57344, K = 8192, no overlap 2854-2979: 8 warps 2763-2873, 16 warps 2798, 4 warps 2924,
        // 2 warps 3390 -- too slow, the second GEMM waits --, two CTAs of 8 warps 3270: the GEMM's single
        // issuing threads and its TMA loads suffer; streaming-store hints changed nothing).
        const long long ctas = std::min<long long>((rest + 7) / 8, (long long)sm_count());
        cudaError_t e = launch_dependent(dequant_f16_resident_kernel, dim3((unsigned)ctas), dim3(256), (size_t)0, st,
                                         wq + (size_t)head_rows * (K / 2), ws16 + (size_t)head_rows * (K / 32),
                                         b16 + (size_t)head_rows * K, fb + head_rows, rest, (int)K);
        if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "dequant_f16 (overlapped) launch: %s", cudaGetErrorString(e));
        if ((s = launch_tile2<false>(ma, mb, sc, y, M, N, K, err, head, tiles_n - head, part, st))) return s;
    }
    return WUSH_OK;
}

// ------------------------------------------------------------------------------------------------
// Per-tensor-scale product on the same tile kernel (kind::i8): y = alpha * (qa . qw)
// ------------------------------------------------------------------------------------------------
// A pre-pass widens the packed nibbles of both operands to int8 rows in the scratch; the tile
// kernel then runs tcgen05.mma kind::i8 with N = 256 over the whole K into int32 accumulators and
// scales once in the epilogue -- the shape in which the int8 tensor path runs near its peak.
namespace {
__global__ void __launch_bounds__(256)
widen_s8_kernel(const uint4* __restrict__ q, uint4* __restrict__ out, long long n_vec,     // 32 codes per step
                int wait_for_primary)       // launched beside a GEMM it does not depend on: do not complete before it has
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
        const uint4 w = ldg_nc_v4(q + i);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // byte b of the word holds codes 2b (low nibble) and 2b + 1 (high nibble)
            const uint32_t lo = ww[j] & 0x0F0F0F0Fu, hi = (ww[j] >> 4) & 0x0F0F0F0Fu;
            const uint32_t slo = lo | ((lo & 0x08080808u) * 0x1Eu);                // sign bit of each nibble copied into bits 4..7
            const uint32_t shi = hi | ((hi & 0x08080808u) * 0x1Eu);
            o[2 * j] = __byte_perm(slo, shi, 0x5140);                              // codes 0..3: lo0 hi0 lo1 hi1
            o[2 * j + 1] = __byte_perm(slo, shi, 0x7362);                          // codes 4..7: lo2 hi2 lo3 hi3
        }
        if ((reinterpret_cast<uintptr_t>(out) & 31) == 0) {
            st_global_v8(out + 2 * i, make_uint4(o[0], o[1], o[2], o[3]), make_uint4(o[4], o[5], o[6], o[7]));
        } else {
            out[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
            out[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
        }
    }
    if (wait_for_primary) pdl_wait();
}
}  // namespace

bool i8_tile_supported(int64_t M, int64_t N, int64_t K) { return M >= 1 && K % 128 == 0 && N % 8 == 0; }

// scratch: error word | int8 activations (M x K) | int8 weights (N x K)
size_t i8_tile_workspace_bytes(int64_t M, int64_t N, int64_t K)
{
    return 256 + align256((size_t)M * K) + align256((size_t)N * K);
}

int i8_tile_dispatch(const uint8_t* xq, const uint8_t* wq, int64_t M, int64_t N, int64_t K, float alpha, const float* alpha_dev,
                     void* y, void* workspace, size_t workspace_bytes, cudaStream_t st)
{
    if (!aligned16(y) || !aligned16(workspace))
        return fail(WUSH_ERR_INVALID_ARGUMENT, "gemm_tensor_scale: output and workspace must be 16-byte aligned");
    if (workspace_bytes < i8_tile_workspace_bytes(M, N, K))
        return fail(WUSH_ERR_WORKSPACE, "gemm_tensor_scale: workspace of %zu bytes needed, %zu given",
                    i8_tile_workspace_bytes(M, N, K), workspace_bytes);
    uint8_t* base = reinterpret_cast<uint8_t*>(workspace);
    int* err = reinterpret_cast<int*>(base);
    uint8_t* a8 = base + 256;
    uint8_t* b8 = a8 + align256((size_t)M * K);
    cudaError_t e = cudaMemsetAsync(err, 0, sizeof(int), st);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    const long long cap = (long long)sm_count() * 16;
    const long long va = M * K / 32, vb = N * K / 32;
    widen_s8_kernel<<<(unsigned)std::min<long long>((va + 255) / 256, cap), 256, 0, st>>>((const uint4*)xq, (uint4*)a8, va, 0);
    if (use_pair_tiles(true)) {
        // As in the fp16-folded product: widen the weights of the first whole waves of column tiles, multiply
        // them, and widen the rest beside that GEMM (a programmatic dependent with one CTA per multiprocessor).
        const int tiles_m = (int)((M + 2 * FM - 1) / (2 * FM)), tiles_n = (int)((N + FN - 1) / FN);
        int head = tiles_n;
        {
            const int wave = std::max(1, pairs_resident());
            int a = tiles_m, b = wave;
            while (b) { const int t = a % b; a = b; b = t; }
            const int wave_cols = wave / a;                                  // column tiles that make whole waves
            const char* v = std::getenv("WUSH_PREPASS_OVERLAP");
            if (!(v && v[0] == '0') && tiles_n >= 3 * wave_cols) head = wave_cols;
        }
        const long long head_rows = std::min<long long>((long long)head * FN, N), vh = head_rows * K / 32;
        widen_s8_kernel<<<(unsigned)std::min<long long>((vh + 255) / 256, cap), 256, 0, st>>>((const uint4*)wq, (uint4*)b8, vh, 0);
        if (int s = check_launch("widen_s8")) return s;
        if (int s = pair_launch(true, a8, b8, nullptr, nullptr, alpha, alpha_dev, y, M, N, K, err, st, 0, head)) return s;
        if (head < tiles_n) {
            const long long vr = vb - vh;
            // (whole product at M = 4096, N = 57344, K = 8192: 1243 us without the overlap, 1222 with one CTA per
            // multiprocessor, 1354 with two)
            e = launch_dependent(widen_s8_kernel, dim3((unsigned)std::min<long long>((vr + 255) / 256, (long long)sm_count())), dim3(256),
                                 (size_t)0, st, (const uint4*)wq + vh, (uint4*)b8 + 2 * vh, vr, 1);
            if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "widen_s8 (overlapped) launch: %s", cudaGetErrorString(e));
            if (int s = pair_launch(true, a8, b8, nullptr, nullptr, alpha, alpha_dev, y, M, N, K, err, st, head, tiles_n - head)) return s;
        }
        return WUSH_OK;
    }
    widen_s8_kernel<<<(unsigned)std::min<long long>((vb + 255) / 256, cap), 256, 0, st>>>((const uint4*)wq, (uint4*)b8, vb, 0);
    if (int s = check_launch("widen_s8")) return s;
    CUtensorMap ma, mb;
    int s;
    if ((s = make_map_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a8, K, M, 128, 2 * FM, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
    if ((s = make_map_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b8, K, N, 128, FN, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
    const TileScale sc = {nullptr, nullptr, alpha, alpha_dev};
    return launch_tile2<true>(ma, mb, sc, y, M, N, K, err, 0, (int)((N + FN - 1) / FN), nullptr, st);
}

}  // namespace wush

// ------------------------------------------------------------------------------------------------
// Variant for callers that may not allocate device memory
// ------------------------------------------------------------------------------------------------
// Some hosts give a plugin no way to obtain scratch: an inference server that sizes one arena at
// start-up and forbids cudaMalloc afterwards, a process confined to a fixed memory budget, or a
// latency-critical loop that cannot afford cudaMalloc's implicit device synchronisation.  For
// them the scratch of the fp16-folded product lives in this translation unit as a fixed array in
// device memory.  Every GPU that loads the library holds these WUSH_STATIC_SCRATCH_BYTES until the
// process exits, which is why the limit is modest.
//
// `g_static_scratch` names the array for DEVICE code; on the host the same identifier is only a
// handle, not an address.  The address a kernel can use is obtained once per device with
// cudaGetSymbolAddress (that device being current) and cached.
namespace wush {
namespace {

__device__ __align__(256) uint8_t g_static_scratch[WUSH_STATIC_SCRATCH_BYTES];
// Where this entry point's kernels record a bounded wait that gave up.  It is only ever set by them and
// cleared by wush_device_flag(), so a give-up is not lost when the next call starts.
__device__ int g_static_error;

constexpr int STATIC_MAX_DEVICES = 64;
void* g_static_ptr[STATIC_MAX_DEVICES];          // device address of the array, per device (null = not resolved yet)
int* g_static_err_ptr[STATIC_MAX_DEVICES];       // device address of g_static_error, per device
std::mutex g_static_mutex;

int static_scratch_pointer(void** out, int** err_out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= STATIC_MAX_DEVICES) return fail(WUSH_ERR_UNSUPPORTED, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[dev]) {
        void *p = nullptr, *pe = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);          // resolves the array on the CURRENT device
        if (e == cudaSuccess) e = cudaGetSymbolAddress(&pe, g_static_error);
        if (e != cudaSuccess || !p || !pe)
            return fail(WUSH_ERR_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
        g_static_err_ptr[dev] = static_cast<int*>(pe);
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    *err_out = g_static_err_ptr[dev];
    return WUSH_OK;
}

}  // namespace

// Used by wush_device_flag(): the role code a kernel of the static-scratch entry point left on the current
// device (0 = none, also when the entry point was never used there); clears it.  Synchronous.
int static_scratch_take_error(int* word)
{
    *word = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= STATIC_MAX_DEVICES) return WUSH_OK;
    int* p;
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        p = g_static_err_ptr[dev];
    }
    if (!p) return WUSH_OK;
    const int zero = 0;
    cudaError_t e = cudaMemcpy(word, p, sizeof(int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && *word) e = cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "device_flag(static scratch): %s", cudaGetErrorString(e));
    return WUSH_OK;
}

}  // namespace wush

WUSH_API size_t wush_w4a4_gemm_static_scratch_limit(void) { return WUSH_STATIC_SCRATCH_BYTES; }

WUSH_API int wush_w4a4_gemm_static_scratch(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M,
                                           int64_t N, int64_t K, void* y, void* stream)
{
    using namespace wush;
    if (int e = ensure_init()) return e;
    WUSH_REQUIRE(M >= 0 && N >= 0 && K > 0, "w4a4_gemm_static_scratch: bad shape");
    if (M == 0 || N == 0) return WUSH_OK;
    WUSH_REQUIRE(xq && xs && wq && ws && y, "w4a4_gemm_static_scratch: null pointer");
    WUSH_REQUIRE(aligned16(xq) && aligned16(wq), "w4a4_gemm_static_scratch: packed codes must be 16-byte aligned");
    if (!f16_supported(M, N, K))
        return fail(WUSH_ERR_UNSUPPORTED, "w4a4_gemm_static_scratch: needs K %% 64 == 0 and N %% 8 == 0 (got K=%lld, N=%lld)",
                    (long long)K, (long long)N);
    const size_t need = f16_layout_bytes(M, N, K, f16_takes_fused(M, N, K, ws));
    if (need > (size_t)WUSH_STATIC_SCRATCH_BYTES)
        return fail(WUSH_ERR_WORKSPACE,
                    "w4a4_gemm_static_scratch: M=%lld N=%lld K=%lld needs %zu bytes of scratch, the built-in array holds %zu; "
                    "use wush_w4a4_gemm with caller-provided scratch",
                    (long long)M, (long long)N, (long long)K, need, (size_t)WUSH_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    int* err = nullptr;
    if (int e = static_scratch_pointer(&scratch, &err)) return e;
    // Every byte of the array the kernels read is written first by this call's own pre-pass, so stale
    // contents of an earlier call are never consumed.  A bounded wait that gives up is recorded in a
    // library-owned word that wush_device_flag() returns (and clears).  f16_dispatch checks the array's
    // size against the route it really takes (a scale pointer that is not 16-byte aligned needs room for
    // an fp16 copy of the weights) before anything is launched.
    return f16_dispatch(xq, xs, wq, ws, M, N, K, y, scratch, (size_t)WUSH_STATIC_SCRATCH_BYTES, (cudaStream_t)stream, err);
}

// ------------------------------------------------------------------------------------------------
// Host-side check of the unit plans (no counterpart in the reference; used by the CPU test suite)
// ------------------------------------------------------------------------------------------------
// Walks the units exactly as the tile kernels do (CTA b takes units b, b + workers, ...) and the pieces exactly as
// tail_sum_kernel does.  cover[tile * k_steps + k] receives how many units cover stage k of the tile;
// returns 0 (else 101..107, one per property) if, besides, every piece a kernel writes for a cut tile is added exactly once by the summing kernel,
// every slot is below `slots` and written once, and (mode 2) unit u is met by CTA u mod workers = its run.
// `tiles` / `k_steps` / `gran` / `workers` as for plan_units; force_mode: -1 = take plan_units' choice for the given
// cost figures, else 1 or 2 with the plan built the same way.  plan_out (7 ints) receives the plan.
WUSH_API int wush_debug_unit_cover(int64_t tiles, int k_steps, int gran, int workers, int force_mode, double step_us,
                                   double piece_us, int* cover, int slots, int* plan_out)
{
    using namespace wush;
    if (tiles <= 0 || k_steps <= 0 || gran <= 0 || workers <= 0 || !cover || !plan_out)
        return fail(WUSH_ERR_INVALID_ARGUMENT, "debug_unit_cover: bad argument");
    UnitPlan p = {(int)tiles, k_steps, (int)tiles, 0, 1, workers, gran};
    {
        const int full = (int)(tiles / workers) * workers, tail = (int)tiles - full;
        if (force_mode < 0) {
            p = plan_units(tiles, k_steps, true, gran, step_us, piece_us, workers);
        } else if (tail > 0 && force_mode == 1) {
            int r = 1;
            while (tail * r * 2 <= workers && k_steps % (r * 2) == 0 && k_steps / (r * 2) >= 4 && (k_steps / (r * 2)) % gran == 0) r *= 2;
            if (r > 1) { p.full_tiles = full; p.mode = 1; p.split = r; }
        } else if (tail > 0 && force_mode == 2 && k_steps % gran == 0 && (long long)tail * k_steps / gran >= workers) {
            p.full_tiles = full; p.mode = 2;
        }
    }
    const int fields[7] = {p.n_tiles, p.k_steps, p.full_tiles, p.mode, p.split, p.ctas, p.gran};
    for (int i = 0; i < 7; ++i) plan_out[i] = fields[i];
    for (int64_t i = 0; i < tiles * k_steps; ++i) cover[i] = 0;
    std::vector<int> slot_tile((size_t)slots, -1);
    const int n_units = unit_count(p);
    const int grid = p.mode == 2 ? workers : std::min(n_units, workers);
    for (int b = 0; b < grid; ++b) {
        for (int u = b; u < n_units; u += grid) {
            const Unit un = decode_unit(p, u);
            if (un.len == 0) continue;
            if (un.tile < 0 || un.tile >= p.n_tiles || un.ks0 < 0 || un.ks0 + un.len > p.k_steps) return 101;
            if (un.ks0 % gran != 0) return 102;
            for (int k = un.ks0; k < un.ks0 + un.len; ++k) ++cover[(int64_t)un.tile * k_steps + k];
            if (un.slot < 0) { if (un.tile >= p.full_tiles) return 103; continue; }
            if (un.tile < p.full_tiles || un.slot >= slots || slot_tile[un.slot] != -1) return 104;
            slot_tile[un.slot] = un.tile;
            if (p.mode == 2 && (u - p.full_tiles) % p.ctas != b) return 105;
        }
    }
    if (p.mode != 0) {
        std::vector<int> added((size_t)slots, 0);
        for (int tt = 0; tt < p.n_tiles - p.full_tiles; ++tt) {
            int bad = 0;
            pieces_of_tile(p, tt, [&](int slot) {
                if (slot < 0 || slot >= slots || slot_tile[slot] != p.full_tiles + tt || added[slot]++) bad = 1;
            });
            if (bad) return 106;
        }
        for (int sl = 0; sl < slots; ++sl)
            if ((slot_tile[sl] != -1) != (added[sl] == 1)) return 107;
    }
    return 0;
}
