// Large-M product on CTA PAIRS: the tile kernel of the fp16-folded route (gemm_f16.cu) with one
// tcgen05.mma shared by the two multiprocessors of a TPC (cta_group::2).
//
// Same contract as the reference's w4a4_gemm_s4 (csrc/gemm_s4.cu:320-379); operands are the exactly
// representable fp16 values code * scale * 2^-e that the pre-pass of gemm_f16.cu writes, so the fp32
// accumulation over the whole K is exact to ~1e-6 and the epilogue only applies 2^(e_m + e_n).
//
// Why pairs.  A single-CTA 256 x 256 tile moves 64 KB of TMA writes and 96 KB of operand reads through
// one multiprocessor's shared memory per 64-wide K step and leaves no room in tensor memory for a second
// accumulator, so the epilogue of a tile never overlaps the next tile's MMAs.  In a pair, each CTA holds
// 128 rows of A and HALF of the 256 weight rows of the step (2 x 16 KB); the hardware feeds both halves
// of B to both tensor cores.  Per CTA and step: 32 KB written, 32 KB read, and only 256 of the 512
// tensor-memory columns per accumulator -- two accumulators rotate, the epilogue of tile i runs under the
// MMAs of tile i + 1.
//
// Roles per CTA (192 threads):
//   warp 0      TMA producer: its own A rows and its own half of B; completion bytes of BOTH CTAs are
//               counted on rank 0's `full` barrier (plain tile loads, each CTA fetches its own data)
//   warp 1      rank 0 only: issues the MMAs for the pair and commits to the barriers of both CTAs;
//               in both CTAs this warp allocates and frees the tensor memory
//   warps 2-5   epilogue: tcgen05.ld (lane quarter = warp index mod 4), scale, fp16 store; the last
//               read of an accumulator arrives on rank 0's `acc_empty`
// Every wait is bounded; a wait that gives up records a role code in the error word and the CTA falls
// through to the common exit (cluster barrier, then tensor memory is freed).
#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "tc_common.cuh"
#include "tc_host.cuh"

namespace wush {
namespace {

constexpr int PM = 128;                 // rows of A (and of the result) per CTA
constexpr int PN = 256;                 // columns of the pair's tile; each CTA loads PN / 2 weight rows
constexpr int P_STAGES = 6;
constexpr int P_ACC = 2;
constexpr int P_THREADS = 192;
constexpr int PA_BYTES = PM * 128, PB_BYTES = (PN / 2) * 128;
constexpr int P_STAGE = PA_BYTES + PB_BYTES;                       // 32 KB
constexpr int P_BARS = P_STAGES * P_STAGE;
constexpr int P_TOTAL = P_BARS + (2 * P_STAGES + 2 * P_ACC + 1) * 8 + 16 + 1024;

__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;                                     // leading byte offset: unused with swizzle
    d |= (uint64_t)(1024 >> 4) << 32;                           // stride between 8-row groups
    d |= 1ull << 46;                                            // descriptor version of sm_100
    d |= 2ull << 61;                                            // 128-byte swizzle
    return d;
}

struct PairScale {
    const float* fa;            // f16: 2^e per activation row
    const float* fb;            // f16: 2^e per weight row
    float alpha;                // i8: per-tensor factor (host value) ...
    const float* alpha_dev;     // ... or device scalar
};

// Order of the tiles.  The pairs that run at the same time should share operands (one HBM read, then L2
// hits), and what one wave of tiles read should still be in L2 for the next.  Tiles are therefore dealt in
// bands of `gm` row blocks: inside a band m runs fastest, so a wave covers gm row blocks x (pairs / gm)
// weight tiles, the band's activation rows (gm x 256 x K fp16) stay L2-resident while the band sweeps N,
// and the weights are streamed once per band.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int gm, int& tm, int& tn) {
    const int band = t / (gm * tiles_n), r = t - band * gm * tiles_n;
    const int rows = min(gm, tiles_m - band * gm);                  // the last band may be shorter
    tm = band * gm + r % rows;
    tn = r / rows;
}

template <bool I8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const PairScale sc,
                 __half* __restrict__ y, int M, int N, int K, int gm, int* __restrict__ err,
                 int tile_n_first, int tile_n_count)                 // the column tiles this launch covers
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + P_BARS);    // used in rank 0: both CTAs' stage data landed
    uint64_t* empty = full + P_STAGES;                               // per CTA: the MMAs reading this stage are done
    uint64_t* acc_full = empty + P_STAGES;                           // per CTA: a tile's accumulator is complete
    uint64_t* acc_empty = acc_full + P_ACC;                          // used in rank 0: both CTAs' epilogues have read it
    uint64_t* done_bar = acc_empty + P_ACC;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = tc::cluster_ctarank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int tiles_m = (M + 2 * PM - 1) / (2 * PM), tiles_n = tile_n_count, n_tiles = tiles_m * tiles_n;
    const int k_steps = K / (I8 ? 128 : 64);                         // a stage row is 128 bytes either way

    pdl_launch_dependents();            // a dependent (the widening of later column tiles) may run beside this grid

    if (tid == 0) {
        for (int i = 0; i < P_STAGES; ++i) { tc::mbar_init(&full[i], 1); tc::mbar_init(&empty[i], 1); }
        for (int i = 0; i < P_ACC; ++i) { tc::mbar_init(&acc_full[i], 1); tc::mbar_init(&acc_empty[i], 8); }
        tc::mbar_init(done_bar, 1);
        tc::mbar_fence_init();
    }
    if (warp == 1) {
        tc::tmem_alloc_pair(tmem_slot, 512);
        tc::tmem_relinquish_pair();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::cluster_sync_all();                                          // the other CTA's barriers exist before anything targets them
    tc::tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            tc::prefetch_tensormap(&map_a); tc::prefetch_tensormap(&map_b);
            uint32_t slot = 0, phase = 0;
            int issued = 0;
            bool ok = true;
            for (int t = pair; t < n_tiles && ok; t += n_pairs) {
                int tm, tn;
                tile_coords(t, tiles_m, tiles_n, gm, tm, tn);
                tn += tile_n_first;
                const int m0 = tm * 2 * PM + (int)rank * PM, n0 = tn * PN + (int)rank * (PN / 2);
                for (int ks = 0; ks < k_steps; ++ks) {
                    if (!tc::mbar_wait(&empty[slot], phase ^ 1)) { ok = false; break; }
                    uint8_t* st = smem + slot * P_STAGE;
                    const uint32_t bar = tc::map_to_rank(&full[slot], 0);
                    if (rank == 0) tc::mbar_expect_tx(&full[slot], 2 * P_STAGE);     // this CTA's bytes and the other's
                    tc::tma_load_2d_pair(st, &map_a, bar, ks * (I8 ? 128 : 64), m0);
                    tc::tma_load_2d_pair(st + PA_BYTES, &map_b, bar, ks * (I8 ? 128 : 64), n0);
                    ++issued;
                    if (++slot == P_STAGES) { slot = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                atomicExch(err, 1);
                // Copies already issued must land before this CTA's shared memory is given back.  On the normal
                // path the MMAs that read them have finished before anybody leaves; here give them a bounded
                // time: rank 0 can watch its `full` barriers, rank 1 (whose bytes are counted there) sleeps.
                if (rank == 0) {
                    for (int i = 0; i < (issued < P_STAGES ? issued : P_STAGES); ++i)
                        for (uint32_t spin = 0; spin < (1u << 16); ++spin)
                            if (tc::mbar_try_wait(&full[i], 0) || tc::mbar_try_wait(&full[i], 1)) break;
                } else {
                    for (int i = 0; i < 64; ++i) __nanosleep(20000);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            uint32_t slot = 0, phase = 0, ab = 0, aphase = 0;
            const uint32_t idesc = I8 ? tc::idesc_i8_pair(PN) : tc::idesc_f16_pair(PN);
            bool ok = true;
            for (int t = pair; t < n_tiles && ok; t += n_pairs) {
                if (!tc::mbar_wait(&acc_empty[ab], aphase ^ 1)) { ok = false; break; }
                tc::tc_fence_after();
                for (int ks = 0; ks < k_steps; ++ks) {
                    if (!tc::mbar_wait(&full[slot], phase)) { ok = false; break; }
                    tc::tc_fence_after();
                    const uint32_t sa = tc::smem_u32(smem + slot * P_STAGE), sb = sa + PA_BYTES;
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        if constexpr (I8)
                            tc::mma_i8_pair(tmem + ab * PN, desc_sw128(sa + kk * 32), desc_sw128(sb + kk * 32), idesc, (ks | kk) ? 1u : 0u);
                        else
                            tc::mma_f16_pair(tmem + ab * PN, desc_sw128(sa + kk * 32), desc_sw128(sb + kk * 32), idesc, (ks | kk) ? 1u : 0u);
                    }
                    tc::mma_commit_pair(&empty[slot]);                         // frees the stage in both CTAs
                    if (++slot == P_STAGES) { slot = 0; phase ^= 1; }
                }
                if (!ok) break;
                tc::mma_commit_pair(&acc_full[ab]);                            // both CTAs' epilogues may read
                if (++ab == P_ACC) { ab = 0; aphase ^= 1; }
            }
            if (!ok) atomicExch(err, 2);
            tc::mma_commit_pair(done_bar);
            for (uint32_t spin = 0; spin < WUSH_SPIN_LIMIT; ++spin)
                if (tc::mbar_try_wait(done_bar, 0)) break;
        }
    } else {
        const int quarter = warp & 3, row = quarter * 32 + lane;                // tcgen05.ld: a warp reads lanes 32 * (warp % 4) ...
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        uint32_t ab = 0, aphase = 0;
        bool ok = true;
        for (int t = pair; t < n_tiles && ok; t += n_pairs) {
            int tm, tn;
            tile_coords(t, tiles_m, tiles_n, gm, tm, tn);
            tn += tile_n_first;
            const int m0 = tm * 2 * PM + (int)rank * PM, n0 = tn * PN;
            if (!tc::mbar_wait(&acc_full[ab], aphase)) { ok = false; break; }
            tc::tc_fence_after();
            const int m = m0 + row;
            float fm;
            if constexpr (I8) fm = sc.alpha_dev ? __ldg(sc.alpha_dev) : sc.alpha;
            else fm = (m < M) ? sc.fa[m] : 0.f;
#pragma unroll 1
            for (int c = 0; c < PN / 32; ++c) {
                uint32_t v[32];
                tc::tmem_ld32(tmem + lane_base + ab * PN + c * 32, v);
                tc::tmem_ld_wait();
                if (c == PN / 32 - 1) {
                    tc::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive_cluster(tc::map_to_rank(&acc_empty[ab], 0));
                }
                const int n = n0 + c * 32;
                if (m < M && n < N) {
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
            if (++ab == P_ACC) { ab = 0; aphase ^= 1; }
        }
        if (!ok && lane == 0) atomicExch(err, 4);
    }

    // Common exit.  Neither CTA may leave while the other can still signal its barriers or while the
    // shared MMA reads its shared memory, and the tensor memory is freed by both together.
    tc::tc_fence_before();
    __syncthreads();
    tc::cluster_sync_all();
    if (warp == 1) tc::tmem_dealloc_pair(tmem, 512);
}

int g_pairs_resident[64];           // per device: pairs of this kernel that can be resident at once (0 = not asked yet)

}  // namespace

int pair_set_attributes()
{
    if (int s = resolve_tensor_map_encoder()) return s;
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_TOTAL);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_TOTAL);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "pair GEMM: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    // How many pairs fit the device at once (one CTA per multiprocessor, both CTAs of a pair in one TPC).
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * 74);
        cfg.blockDim = dim3(P_THREADS);
        cfg.dynamicSmemBytes = P_TOTAL;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        e = cudaOccupancyMaxActiveClusters(&clusters, gemm_pair_kernel<false>, &cfg);
        if (e != cudaSuccess || clusters <= 0) {
            cudaGetLastError();
            clusters = sm_count() / 2;
        }
        g_pairs_resident[dev] = clusters;
    }
    return WUSH_OK;
}

int pairs_resident()
{
    int dev = 0;
    cudaGetDevice(&dev);
    return (dev >= 0 && dev < 64 && g_pairs_resident[dev] > 0) ? g_pairs_resident[dev] : sm_count() / 2;
}

bool pair_supported(int64_t M, int64_t N, int64_t K, bool i8) { return M >= 1 && K % (i8 ? 128 : 64) == 0 && N % 8 == 0; }

// a (M x K) and b (N x K): fp16 rows for the folded route, int8 rows for the per-tensor route.
// The launch covers column tiles [tile_n_first, tile_n_first + tile_n_count) of 256 columns; a negative count means all.
int pair_launch(bool i8, const void* a, const void* b, const float* fa, const float* fb, float alpha, const float* alpha_dev,
                void* y, int64_t M, int64_t N, int64_t K, int* err, cudaStream_t st, int tile_n_first, int tile_n_count)
{
    if (tile_n_count < 0) { tile_n_first = 0; tile_n_count = (int)((N + PN - 1) / PN); }
    CUtensorMap ma, mb;
    int s;
    if (i8) {
        if ((s = make_map_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, K, M, 128, PM, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
        if ((s = make_map_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, K, N, 128, PN / 2, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
    } else {
        if ((s = make_map_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a, K, M, 64, PM, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
        if ((s = make_map_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, b, K, N, 64, PN / 2, CU_TENSOR_MAP_SWIZZLE_128B))) return s;
    }
    int dev = 0;
    cudaGetDevice(&dev);
    const int resident = (dev >= 0 && dev < 64 && g_pairs_resident[dev] > 0) ? g_pairs_resident[dev] : sm_count() / 2;
    const int64_t tiles = ((M + 2 * PM - 1) / (2 * PM)) * tile_n_count;
    const int pairs = (int)(tiles < resident ? tiles : resident);
    const PairScale sc = {fa, fb, alpha, alpha_dev};
    // Band height: as many row blocks as keep the band's activations within about a quarter of the L2
    // (32 MB), at least 2 (M = 4096, K = 8192: 16 for int8 operands, 8 for fp16 -- where 16 measured 3 % better
    // under sustained load and 8 read 14 % fewer DRAM bytes); WUSH_PAIR_BAND overrides it for measurements.
    const int64_t tiles_m = (M + 2 * PM - 1) / (2 * PM);
    const int64_t slab = 2 * PM * K * (i8 ? 1 : 2);
    int gm = (int)std::max<int64_t>(2, std::min<int64_t>(tiles_m, (32ll << 20) / slab));
    if (const char* v = std::getenv("WUSH_PAIR_BAND")) gm = std::max(1, atoi(v));
    if (gm > tiles_m) gm = (int)tiles_m;
    if (i8)
        gemm_pair_kernel<true><<<2 * pairs, P_THREADS, P_TOTAL, st>>>(ma, mb, sc, (__half*)y, (int)M, (int)N, (int)K, gm, err,
                                                                      tile_n_first, tile_n_count);
    else
        gemm_pair_kernel<false><<<2 * pairs, P_THREADS, P_TOTAL, st>>>(ma, mb, sc, (__half*)y, (int)M, (int)N, (int)K, gm, err,
                                                                       tile_n_first, tile_n_count);
    return check_launch("gemm_pair");
}

}  // namespace wush
