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
//   * The WEIGHTS are the wide MMA operand: each compute warp owns 16 weight rows (the M=16
//     side of mma.m16n8k32.s8) against 1, 2, 3 or 4 tiles of 8 activation rows.  The number of
//     compute warps per CTA (1..13) is chosen per call so that the whole grid is resident at
//     once, two CTAs per SM, all with the same number of rows: one balanced wave.
//   * One more warp is the producer: per stage of 4 groups it issues TMA tile loads of the
//     packed weight and activation codes (64-byte swizzle) into a ring of up to 8 stages
//     (~100 KB per CTA) and, with every even stage, the two bf16 scale tiles of 8 groups;
//     full/empty mbarriers, bounded waits.
//   * A further warp prepares the activations once per stage for everybody: nibbles widened
//     into MMA-fragment order, bf16 scales converted to fp32 pairs (otherwise every compute
//     warp would repeat that integer work, and the integer pipe is what limits this kernel).
//   * ldmatrix on the swizzled tile hands every lane the one 4-byte word of 8 nibbles it
//     needs per row (conflict free); one shift and two ANDs make two MMA registers of
//     signed bytes (16 * code).  The k order inside a group is permuted identically for both
//     operands.
//   * No integer->float conversion is executed: the MMA accumulates onto the bit pattern of
//     1.5 * 2^23, so its int32 result read as fp32 is 12582912 + 256 * P_g, and
//         t = fma(f, sw, -12582912 * sw)   (exact, = 256 * P_g * sw)
//         acc = fma(t, sx, acc)
//     applies both scales with two FMAs per output and group (issued as packed fp32x2
//     instructions on column pairs); 1/256 is applied once at the end.
//   * Narrow layers (fewer 16-row blocks than warp schedulers) are launched as clusters of
//     2, 4 or 8 CTAs that share their rows and split K; the partial sums reach the cluster's
//     first CTA through distributed shared memory (pick_split, KSPLIT below).
//   * PUSH variants write the result into the exchange buffers of all tensor-parallel ranks
//     instead of y (peer_common.cuh).
//
// Algorithmic HBM bytes: 9*N*K/16 (weights) + 9*M*K/16 (activations, L2 resident) + 2*M*N.
#include <cooperative_groups.h>

#include "common.cuh"
#include "peer_common.cuh"
#include "tc_common.cuh"
#include "tc_host.cuh"

namespace wush {

__device__ int g_device_flag;                       // library-owned error word of the streaming kernels

namespace {

namespace cg = cooperative_groups;

constexpr int ST_KS = 4;                            // groups per code stage (64 B of codes per row, 64-byte swizzle)
constexpr int ST_SG = 8;                            // groups per scale tile (16 B per row): one per two code stages
// compute warps per CTA (16 weight rows each): 13 + 2 warps, two CTAs per SM, 64 registers per thread
constexpr int max_warps(int) { return 13; }
constexpr int ST_EXTRA_WARPS = 2;                   // TMA producer + activation prep
constexpr int ST_MAX_STAGES = 8;
constexpr uint32_t MAGIC_BITS = 0x4B400000u;
constexpr float MAGIC = 12582912.0f;

// Shared-memory plan of one CTA with `warps` compute warps (host and device agree on it):
// a ring of code stages (weights + activations, 4 groups each) and a ring of scale slots
// (8 groups each, filled together with every even code stage).  A scale slot is reused
// `sslots` pairs later; sslots >= (stages + 1) / 2 makes the code ring's empty barriers
// sufficient to protect it.
struct StreamPlan {
    int rows, xc, stage, stages, scales, sx, sslot, sslots, prep, pslot, pscale, bars, red, total, tx_codes, tx_scales;
    // ksplit: the CTA is one of a cluster that shares its rows and splits K; a smaller ring so that
    // four CTAs fit a multiprocessor, and room for the fp32 partial results handed to the leader
    __host__ __device__ StreamPlan(int warps, int xrows, bool ksplit = false) {
        rows = warps * 16;
        xc = ((rows * 64 + 1023) / 1024) * 1024;             // activation codes after the weight codes
        stage = xc + ((xrows * 64 + 1023) / 1024) * 1024;
        sx = rows * 16;                                       // activation scales after the weight scales
        sslot = ((sx + xrows * 16 + 127) / 128) * 128;
        // per code stage, the activation tile once more in MMA-fragment order: [group][m-tile][lane]
        // (b0, b1) words, then [group][m-tile][tig] fp32 scale pairs
        pscale = ST_KS * (xrows / 8) * 32 * 8;
        pslot = pscale + ST_KS * (xrows / 8) * 4 * 8;
        stages = ST_MAX_STAGES;
        const int budget = ksplit ? 44 * 1024 : 100 * 1024;   // two CTAs per SM, four of a split cluster
        while (stages > 2 && stages * (stage + pslot) + ((stages + 2) / 2) * sslot > budget) --stages;
        sslots = (stages + 2) / 2;
        scales = stages * stage;
        prep = scales + sslots * sslot;
        bars = prep + stages * pslot;
        red = bars + 3 * ST_MAX_STAGES * 8 + 64;              // 16-byte aligned: bars is a multiple of 128
        total = red + (ksplit ? warps * (xrows / 8) * 32 * 16 : 0) + 1024;   // + slack for the 1 KB alignment
        tx_codes = rows * 64 + xrows * 64;
        tx_scales = rows * 16 + xrows * 16;
    }
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

// bf16 element e (0..3) of an 8-byte vector of scales, as fp32
__device__ __forceinline__ float scale_of(const uint2& v, int e) {
    const uint32_t w = (e < 2) ? v.x : v.y;
    return (e & 1) ? bf16_hi(w) : bf16_lo(w);
}

// `warps` compute warps own 16 weight rows each; warp index `warps` is the TMA producer.
// PUSH (one block of rows, gridDim.y == 1): instead of y the result goes into slot (step & 1, rank)
// of EVERY rank's exchange buffer, stored over NVLink from the epilogue; the CTA's last compute warp
// counts the CTA and the grid's last CTA publishes the step (peer_common.cuh).
// KSPLIT: launched as clusters of S CTAs along z that own the same rows and 1/S of K each; the
// partial sums of ranks 1..S-1 travel through distributed shared memory to rank 0, which adds them
// in rank order and writes the result.  Every thread of every CTA reaches both cluster barriers,
// whatever its role and whether or not one of its bounded waits gave up.
template <int MT, bool PARTIALS, bool PUSH = false, bool KSPLIT = false>
__global__ void __launch_bounds__(KSPLIT ? (4 + ST_EXTRA_WARPS) * 32 : (max_warps(MT) + ST_EXTRA_WARPS) * 32, KSPLIT ? 4 : 2)
w4a4_stream_kernel(const __grid_constant__ CUtensorMap map_wq, const __grid_constant__ CUtensorMap map_xq,
                   const __grid_constant__ CUtensorMap map_ws, const __grid_constant__ CUtensorMap map_xs,
                   __half* __restrict__ y, int32_t* __restrict__ part, int M, int N, int K, int warps,
                   const PeerTable peers)
{
    __shared__ unsigned int s_warps_done;
    constexpr int XROWS = MT * 8;
    const StreamPlan L(warps, XROWS, KSPLIT);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars);
    uint64_t* empty = full + ST_MAX_STAGES;
    uint64_t* xready = empty + ST_MAX_STAGES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = K >> 5;
    int n_chunks = G / ST_KS, kc0 = 0, crank = 0, csize = 1;
    if constexpr (KSPLIT) {
        cg::cluster_group cluster = cg::this_cluster();
        crank = (int)cluster.block_rank();
        csize = (int)cluster.num_blocks();
        n_chunks /= csize;                                   // the host made this an even number of whole chunks
        kc0 = crank * n_chunks;
    }
    const int n_base = blockIdx.x * L.rows, m_base = blockIdx.y * XROWS;
    float2 acc[MT][2];                                   // [m-tile][row gid | row gid+8] x (col 2tig, 2tig+1)
    bool ok = true;

    if (tid == 0) {
        for (int i = 0; i < L.stages; ++i) { tc::mbar_init(&full[i], 1); tc::mbar_init(&empty[i], warps); tc::mbar_init(&xready[i], 1); }
        tc::mbar_fence_init();
        s_warps_done = 0;
    }
    __syncthreads();

    if (warp == warps) {
        // ------------------------------ producer ----------------------------------------------
        if (lane == 0) {
            tc::prefetch_tensormap(&map_wq); tc::prefetch_tensormap(&map_xq);
            tc::prefetch_tensormap(&map_ws); tc::prefetch_tensormap(&map_xs);
            int slot = 0, issued = 0;
            uint32_t phase = 0;
            bool ok = true;
            int sslot = 0;
            for (int kc = 0; kc < n_chunks; ++kc) {
                if (!tc::mbar_wait(&empty[slot], phase ^ 1)) { ok = false; break; }
                uint8_t* st = smem + slot * L.stage;
                const bool with_scales = (kc & 1) == 0;
                tc::mbar_expect_tx(&full[slot], L.tx_codes + (with_scales ? L.tx_scales : 0));
                tc::tma_load_2d(st, &map_wq, &full[slot], (kc0 + kc) * 64, n_base);
                tc::tma_load_2d(st + L.xc, &map_xq, &full[slot], (kc0 + kc) * 64, m_base);
                if (with_scales) {
                    uint8_t* sc = smem + L.scales + sslot * L.sslot;
                    tc::tma_load_2d(sc, &map_ws, &full[slot], ((kc0 + kc) >> 1) * ST_SG, n_base);
                    tc::tma_load_2d(sc + L.sx, &map_xs, &full[slot], ((kc0 + kc) >> 1) * ST_SG, m_base);
                    if (++sslot == L.sslots) sslot = 0;
                }
                ++issued;
                if (++slot == L.stages) { slot = 0; phase ^= 1; }
            }
            if (!ok) {
                atomicExch(&g_device_flag, 1);
                // copies already issued must land before the CTA's memory is given back
                for (int i = 0; i < (issued < L.stages ? issued : L.stages); ++i)
                    for (uint32_t spin = 0; spin < (1u << 16); ++spin)
                        if (tc::mbar_try_wait(&full[i], 0) || tc::mbar_try_wait(&full[i], 1)) break;
            }
        }
    } else if (warp == warps + 1) {
        // ------------------------------ activation prep ------------------------------------------
        // Every compute warp needs the same activation fragments and scales; this warp widens the
        // nibbles and converts the bf16 scales ONCE per stage into MMA-fragment order so that the
        // compute warps get them with two 8-byte shared loads per group and m-tile.
        if constexpr (!PARTIALS) {
            int slot = 0, sslot = 0;
            uint32_t phase = 0;
            for (int kc = 0; kc < n_chunks; ++kc) {
                if (!tc::mbar_wait(&full[slot], phase)) { if (lane == 0) atomicExch(&g_device_flag, 3); break; }
                const uint8_t* xc = smem + slot * L.stage + L.xc;
                const uint8_t* sc = smem + L.scales + sslot * L.sslot + L.sx + (kc & 1) * 8;
                uint2* frag = reinterpret_cast<uint2*>(smem + L.prep + slot * L.pslot);
                float2* fsc = reinterpret_cast<float2*>(smem + L.prep + slot * L.pslot + L.pscale);
#pragma unroll
                for (int i = 0; i < ST_KS * MT; ++i) {                  // i = g * MT + mt
                    const int g = i / MT, mt = i % MT;
                    const int row = mt * 8 + (lane >> 2);
                    const uint32_t w = *reinterpret_cast<const uint32_t*>(xc + row * 64 + ((g ^ ((row >> 1) & 3)) << 4) + (lane & 3) * 4);
                    uint2 b;
                    unpack_x16(w, b.x, b.y);
                    frag[i * 32 + lane] = b;
                }
                for (int i = lane; i < ST_KS * MT * 4; i += 32) {        // i = (g * MT + mt) * 4 + tig
                    const int t = i & 3, gm = i >> 2, g = gm / MT, mt = gm % MT;
                    const unsigned short* r0 = reinterpret_cast<const unsigned short*>(sc + (mt * 8 + t * 2) * 16) + g;
                    fsc[i] = make_float2(bf16_bits_to_f32(r0[0]), bf16_bits_to_f32(r0[8]));   // rows 2t and 2t+1 (16 B apart)
                }
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&xready[slot]);
                if (++slot == L.stages) { slot = 0; phase ^= 1; }
                if ((kc & 1) && ++sslot == L.sslots) sslot = 0;
            }
        }
    }
    if constexpr (!KSPLIT) {
        if (warp >= warps) return;
    }
    const int gid = lane >> 2, tig = lane & 3;
    if (!KSPLIT || warp < warps) {
    // ---------------------------------- compute warps -------------------------------------------
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = make_float2(0.f, 0.f);
    // ldmatrix row addresses (the 128-byte swizzle XORs the 16-byte piece index with row & 7)
    const int w_row = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);        // matrices 0/2: rows 0-7, 1/3: rows 8-15
    const int w_gsel = lane >> 4;                                             // matrices 2,3 take the next group
    const int swz = ((lane >> 1) & 3) << 4;             // 64-byte swizzle: piece index ^= (row >> 1) & 3
    int slot = 0, sslot = 0;
    uint32_t phase = 0;
    for (int kc = 0; kc < n_chunks; ++kc) {
        if (!tc::mbar_wait(&full[slot], phase)) { ok = false; break; }
        if constexpr (!PARTIALS) {
            if (!tc::mbar_wait(&xready[slot], phase)) { ok = false; break; }
        }
        const uint8_t* st = smem + slot * L.stage;
        const uint8_t* wc = st + w_row * 64;
        const uint8_t* xc = st + L.xc;
        const uint2* frag = reinterpret_cast<const uint2*>(smem + L.prep + slot * L.pslot) + lane;
        const float2* fsc = reinterpret_cast<const float2*>(smem + L.prep + slot * L.pslot + L.pscale) + tig;
        const uint8_t* sc = smem + L.scales + sslot * L.sslot + (kc & 1) * 8;   // second half of the 16-byte rows on odd stages
        {
            constexpr int gq = 0;
            // scales of these four groups: one 8-byte vector per row
            uint2 swa, swb;
            if constexpr (!PARTIALS) {
                swa = *reinterpret_cast<const uint2*>(sc + (warp * 16 + gid) * 16);
                swb = *reinterpret_cast<const uint2*>(sc + (warp * 16 + gid + 8) * 16);
            }
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                const int g0 = gq + 2 * p;                    // first group of the pair (compile-time)
                uint32_t wa[4];
                ldsm_x4(wa, wc + (((g0 + w_gsel) << 4) ^ swz));
                uint32_t xb[2][MT];                           // PARTIALS only: activation words straight from the tile
                if constexpr (PARTIALS) {
#pragma unroll
                    for (int gg = 0; gg < 2; ++gg) {
                        uint32_t r[4];
                        ldsm_x4(r, xc + lane * 64 + (((g0 + gg) << 4) ^ swz));
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) xb[gg][mt] = r[mt];
                    }
                }
#pragma unroll
                for (int gg = 0; gg < 2; ++gg) {
                    const int e = 2 * p + gg;                 // group inside the quad (compile-time)
                    uint32_t a0, a1, a2, a3;
                    unpack_x16(wa[gg * 2 + 0], a0, a2);       // row gid:     even codes, odd codes
                    unpack_x16(wa[gg * 2 + 1], a1, a3);       // row gid + 8
                    float2 s_a, s_b, c_a, c_b;
                    if constexpr (!PARTIALS) {
                        const float fa = scale_of(swa, e), fb = scale_of(swb, e);
                        s_a = make_float2(fa, fa); s_b = make_float2(fb, fb);
                        c_a = make_float2(-MAGIC * fa, -MAGIC * fa);     // exact: 2 x 8 significant bits
                        c_b = make_float2(-MAGIC * fb, -MAGIC * fb);
                    }
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        uint32_t b0, b1, d[4];
                        if constexpr (PARTIALS) {
                            unpack_x16(xb[gg][mt], b0, b1);
                        } else {
                            const uint2 b = frag[((gq + e) * MT + mt) * 32];
                            b0 = b.x; b1 = b.y;
                        }
                        mma_s8_biased(d, a0, a1, a2, a3, b0, b1);
                        if constexpr (PARTIALS) {
                            const int g = (kc0 + kc) * ST_KS + gq + e;
                            const int na = n_base + warp * 16 + gid, nb = na + 8;
                            const int m0 = m_base + mt * 8 + tig * 2, m1 = m0 + 1;
                            if (m0 < M && na < N) part[((size_t)m0 * N + na) * G + g] = (int32_t)(d[0] - MAGIC_BITS) >> 8;
                            if (m1 < M && na < N) part[((size_t)m1 * N + na) * G + g] = (int32_t)(d[1] - MAGIC_BITS) >> 8;
                            if (m0 < M && nb < N) part[((size_t)m0 * N + nb) * G + g] = (int32_t)(d[2] - MAGIC_BITS) >> 8;
                            if (m1 < M && nb < N) part[((size_t)m1 * N + nb) * G + g] = (int32_t)(d[3] - MAGIC_BITS) >> 8;
                        } else {
                            const float2 x01 = fsc[((gq + e) * MT + mt) * 4];
                            const float2 fa2 = make_float2(__uint_as_float(d[0]), __uint_as_float(d[1]));
                            const float2 fb2 = make_float2(__uint_as_float(d[2]), __uint_as_float(d[3]));
                            acc[mt][0] = __ffma2_rn(__ffma2_rn(fa2, s_a, c_a), x01, acc[mt][0]);
                            acc[mt][1] = __ffma2_rn(__ffma2_rn(fb2, s_b, c_b), x01, acc[mt][1]);
                        }
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&empty[slot]);
        if (++slot == L.stages) { slot = 0; phase ^= 1; }
        if ((kc & 1) && ++sslot == L.sslots) sslot = 0;
    }
    if (!ok && lane == 0) atomicExch(&g_device_flag, 2);
    }   // roles

    if constexpr (KSPLIT) {
        cg::cluster_group cluster = cg::this_cluster();
        float4* red = reinterpret_cast<float4*>(smem + L.red);
        if (warp < warps && crank != 0) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
                red[(warp * MT + mt) * 32 + lane] = make_float4(acc[mt][0].x, acc[mt][0].y, acc[mt][1].x, acc[mt][1].y);
        }
        __syncwarp();                                         // the producer's lane 0 left its loop later than lanes 1-31
        cluster.sync();
        if (warp < warps && crank == 0) {
            for (int r = 1; r < csize; ++r) {
                const float4* other = cluster.map_shared_rank(red, r);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const float4 v = other[(warp * MT + mt) * 32 + lane];
                    acc[mt][0].x += v.x; acc[mt][0].y += v.y; acc[mt][1].x += v.z; acc[mt][1].y += v.w;
                }
            }
        }
        __syncwarp();
        cluster.sync();                                       // the partials are read: the other CTAs may leave
        if (crank != 0) return;
    }
    if (warp >= warps) return;
    if constexpr (!PUSH) {
        if (!ok) return;                                      // PUSH: still count the CTA, the peers wait for the flag
    }
    if constexpr (PUSH) {
        const int na = n_base + warp * 16 + gid, nb = na + 8;
        const float k = 1.0f / 256.0f;
        // the step counter is stable: the reduction of the previous step has completed on this stream
        const unsigned int step = *reinterpret_cast<volatile unsigned int*>(&peers.state->step);
        const size_t off = slot_offset(peers, step, peers.rank);
        if (ok) {
            for (int p = 0; p < peers.world; ++p) {
                __half* dst = reinterpret_cast<__half*>(peers.base[p] + off);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int m0 = m_base + mt * 8 + tig * 2, m1 = m0 + 1;
                    if (m0 < M && na < N) dst[(size_t)m0 * N + na] = __float2half_rn(acc[mt][0].x * k);
                    if (m1 < M && na < N) dst[(size_t)m1 * N + na] = __float2half_rn(acc[mt][0].y * k);
                    if (m0 < M && nb < N) dst[(size_t)m0 * N + nb] = __float2half_rn(acc[mt][1].x * k);
                    if (m1 < M && nb < N) dst[(size_t)m1 * N + nb] = __float2half_rn(acc[mt][1].y * k);
                }
            }
        }
        __threadfence_system();
        __syncwarp();
        unsigned int finished = 0;
        if (lane == 0) finished = atomicAdd(&s_warps_done, 1u);
        finished = __shfl_sync(0xffffffffu, finished, 0);
        if (finished == (unsigned int)warps - 1) comm_count_and_publish(peers, step, lane);
    } else if constexpr (!PARTIALS) {
        const int na = n_base + warp * 16 + gid, nb = na + 8;
        const float k = 1.0f / 256.0f;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int m0 = m_base + mt * 8 + tig * 2, m1 = m0 + 1;
            if (m0 < M && na < N) y[(size_t)m0 * N + na] = __float2half_rn(acc[mt][0].x * k);
            if (m1 < M && na < N) y[(size_t)m1 * N + na] = __float2half_rn(acc[mt][0].y * k);
            if (m0 < M && nb < N) y[(size_t)m0 * N + nb] = __float2half_rn(acc[mt][1].x * k);
            if (m1 < M && nb < N) y[(size_t)m1 * N + nb] = __float2half_rn(acc[mt][1].y * k);
        }
    }
}

// Compute warps per CTA: the rows are dealt so that ALL CTAs are resident at once (two per SM)
// and carry the same number of 16-row blocks -- a second, partly filled wave would cost as much
// as a full one because a CTA alone cannot pull more bandwidth than its pipeline depth allows.
int pick_warps(int64_t N, int64_t m_blocks, int limit)
{
    const int64_t blocks = (N + 15) / 16;
    int64_t slots = 2LL * sm_count() / (m_blocks > 0 ? m_blocks : 1);
    if (slots < 1) slots = 1;
    int64_t w = (blocks + slots - 1) / slots;
    if (w > limit) w = limit;
    if (w < 1) w = 1;
    return (int)w;
}

// K split over a cluster of CTAs.  A narrow layer has fewer 16-row blocks than the machine has warp
// schedulers (4 per multiprocessor), and every CTA walks the whole K alone -- its compute warps and
// its activation-prep warp alike -- so the time is that serial walk, not the weight stream.  Splitting
// K over 2, 4 or 8 CTAs shortens the walk and fills the schedulers.  Whole scale tiles (two chunks)
// per rank, and at least 8 chunks each.
int pick_split(int64_t N, int64_t m_blocks, int64_t K)
{
    // measured (us, no split / 2 / 4 / 8): N=8192 K=8192 M=32: 47 / 35 / 29 / 36, M=64: 54 / 48 / 52 / 62,
    // M=128: 74 / 84 / 91 / 109; N=4096 K=12288 M=32: 60 / 39 / 29 / 26; N=24576 K=4096 M=32: 37 / 42 / 46 / 61
    const int64_t compute_warps = ((N + 15) / 16) * m_blocks, chunks = K / 128, sms = sm_count();
    int s = compute_warps <= 2 * sms ? 8 : compute_warps <= 4 * sms ? 4 : compute_warps < 8 * sms ? 2 : 1;
    while (s > 1 && (chunks % (2 * s) != 0 || chunks < 8 * s)) s >>= 1;
    return s;
}

template <int MT, bool PARTIALS, bool PUSH = false>
int launch_stream(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N, int64_t K,
                  void* y, int32_t* part, cudaStream_t st, const PeerTable& peers = PeerTable{})
{
    constexpr int XROWS = MT * 8;
    const int64_t m_blocks = (M + XROWS - 1) / XROWS;
    if (m_blocks > 65535) return fail(WUSH_ERR_UNSUPPORTED, "w4a4_gemm(decode): M too large");
    const int split = PARTIALS ? 1 : pick_split(N, m_blocks, K);
    // split clusters: four CTAs of at most four compute warps per multiprocessor
    const int warps = split > 1 ? pick_warps(N, m_blocks * split / 2, 4) : pick_warps(N, m_blocks, max_warps(MT));
    const StreamPlan L(warps, XROWS, split > 1);
    CUtensorMap mwq, mxq, mws, mxs;
    int s;
    if ((s = make_map_2d(&mwq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, K / 2, N, 64, L.rows, CU_TENSOR_MAP_SWIZZLE_64B))) return s;
    if ((s = make_map_2d(&mxq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, K / 2, M, 64, XROWS, CU_TENSOR_MAP_SWIZZLE_64B))) return s;
    if ((s = make_map_2d(&mws, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ws, K / 32, N, ST_SG, L.rows, CU_TENSOR_MAP_SWIZZLE_NONE))) return s;
    if ((s = make_map_2d(&mxs, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, xs, K / 32, M, ST_SG, XROWS, CU_TENSOR_MAP_SWIZZLE_NONE))) return s;
    dim3 grid((unsigned)((N + L.rows - 1) / L.rows), (unsigned)m_blocks);
    if (PUSH && grid.y != 1) return fail(WUSH_ERR_UNSUPPORTED, "w4a4_gemm(decode, pushed): one block of rows only");
    if constexpr (!PARTIALS) {
        if (split > 1) {
            grid.z = (unsigned)split;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = grid;
            cfg.blockDim = dim3((warps + ST_EXTRA_WARPS) * 32);
            cfg.dynamicSmemBytes = L.total;
            cfg.stream = st;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 1;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = (unsigned)split;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            cudaError_t e = cudaLaunchKernelEx(&cfg, w4a4_stream_kernel<MT, false, PUSH, true>, mwq, mxq, mws, mxs, (__half*)y, part,
                                               (int)M, (int)N, (int)K, warps, peers);
            if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "w4a4_stream (split): %s", cudaGetErrorString(e));
            return check_launch("w4a4_stream");
        }
    }
    w4a4_stream_kernel<MT, PARTIALS, PUSH><<<grid, (warps + ST_EXTRA_WARPS) * 32, L.total, st>>>(
        mwq, mxq, mws, mxs, (__half*)y, part, (int)M, (int)N, (int)K, warps, peers);
    return check_launch("w4a4_stream");
}

template <int MT, bool P, bool PUSH = false>
cudaError_t set_attr() {
    if constexpr (!P) {
        cudaError_t e = cudaFuncSetAttribute(w4a4_stream_kernel<MT, P, PUSH, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
        if (e != cudaSuccess) return e;
    }
    return cudaFuncSetAttribute(w4a4_stream_kernel<MT, P, PUSH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
}

}  // namespace

int stream_set_attributes()
{
    if (int s = resolve_tensor_map_encoder()) return s;
    cudaError_t e;
    if ((e = set_attr<1, false>()) != cudaSuccess || (e = set_attr<2, false>()) != cudaSuccess ||
        (e = set_attr<3, false>()) != cudaSuccess ||
        (e = set_attr<4, false>()) != cudaSuccess || (e = set_attr<4, true>()) != cudaSuccess ||
        (e = set_attr<1, false, true>()) != cudaSuccess || (e = set_attr<2, false, true>()) != cudaSuccess ||
        (e = set_attr<3, false, true>()) != cudaSuccess || (e = set_attr<4, false, true>()) != cudaSuccess)
        return fail(WUSH_ERR_CUDA, "decode kernel: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    return WUSH_OK;
}

// Whole TMA stages only (K % 256 == 0) and 16-byte aligned scale rows/pointers.
bool stream_supported(int64_t K, const void* xs, const void* ws)
{
    return K % 256 == 0 && aligned16(xs) && aligned16(ws);
}

// Rows of activations per CTA (8 * tiles) for M rows.  Up to 32 rows: the smallest tile count that holds them.
// Beyond: every block of rows streams the weights again, so the count of blocks times the measured time of one
// block (70B layer: 55 / 76 / 105 / 117 us for 1..4 tiles) is what to minimise -- 40 rows are two blocks of 24,
// not two of 32.  `relative_cost`, if given, receives that product in units of the 4-tile block.
int stream_tiles_for(int64_t M, double* relative_cost)
{
    static const double block_us[5] = {0.0, 55.0, 76.0, 105.0, 117.0};
    int best = 4;
    double best_cost = 0.0;
    for (int mt = 1; mt <= 4; ++mt) {
        const double cost = (double)((M + 8 * mt - 1) / (8 * mt)) * block_us[mt];
        if (mt == 1 || cost < best_cost) { best = mt; best_cost = cost; }
    }
    if (relative_cost) *relative_cost = best_cost / block_us[4];
    return best;
}

int stream_dispatch(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N, int64_t K,
                    void* y, cudaStream_t st)
{
    switch (stream_tiles_for(M, nullptr)) {
        case 1: return launch_stream<1, false>(xq, xs, wq, ws, M, N, K, y, nullptr, st);
        case 2: return launch_stream<2, false>(xq, xs, wq, ws, M, N, K, y, nullptr, st);
        case 3: return launch_stream<3, false>(xq, xs, wq, ws, M, N, K, y, nullptr, st);
    }
    return launch_stream<4, false>(xq, xs, wq, ws, M, N, K, y, nullptr, st);
}

// M <= 32: the result goes into every rank's exchange slot instead of y (see the kernel).
int stream_dispatch_push(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N, int64_t K,
                         const PeerTable& peers, cudaStream_t st)
{
    if (M <= 8) return launch_stream<1, false, true>(xq, xs, wq, ws, M, N, K, nullptr, nullptr, st, peers);
    if (M <= 16) return launch_stream<2, false, true>(xq, xs, wq, ws, M, N, K, nullptr, nullptr, st, peers);
    if (M <= 24) return launch_stream<3, false, true>(xq, xs, wq, ws, M, N, K, nullptr, nullptr, st, peers);
    if (M <= 32) return launch_stream<4, false, true>(xq, xs, wq, ws, M, N, K, nullptr, nullptr, st, peers);
    return fail(WUSH_ERR_UNSUPPORTED, "w4a4_gemm(decode, pushed): at most 32 rows");
}

int stream_partials(const uint8_t* xq, const uint8_t* wq, int64_t M, int64_t N, int64_t K, int32_t* P, cudaStream_t st)
{
    // the scale tiles are still fetched; the codes are readable, aligned and large enough
    return launch_stream<4, true>(xq, xq, wq, wq, M, N, K, nullptr, P, st);
}

}  // namespace wush

namespace wush { int static_scratch_take_error(int* word); }

// Bits 0-7: role code of a streaming (decode) kernel whose wait ran out; bits 8-15: role code left by a
// kernel of wush_w4a4_gemm_static_scratch (whose scratch, unlike a caller's, cannot be inspected from outside).
WUSH_API int wush_device_flag(int* flag)
{
    using namespace wush;
    if (int e = ensure_init()) return e;
    WUSH_REQUIRE(flag, "device_flag: null pointer");
    int zero = 0, stream_word = 0, static_word = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&stream_word, g_device_flag, sizeof(int));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_device_flag, &zero, sizeof(int));
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "device_flag: %s", cudaGetErrorString(e));
    if (int s = static_scratch_take_error(&static_word)) return s;
    *flag = (stream_word & 0xff) | ((static_word & 0xff) << 8);
    return WUSH_OK;
}
