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
//   * ONE activation row (gemv_row_kernel): each warp owns one weight row per trip; lane l takes groups l,
//     l+32, ...: one 16-byte load of codes and one 2-byte load of the scale per group, eight groups (144 B per
//     lane) in flight before the first use; the next row's loads are issued before the reduction of the
//     current one, and the very first ones before the activation prologue.  Short rows (K <= 4096) are taken
//     two or four at a time so that a lane still has eight loads in flight.  A word of 8 nibbles becomes two
//     words of 4 signed bytes with one shift and two ANDs (byte = 16 * code, no sign extension needed), then
//     dp4a against the activation bytes: the exact group sum comes out multiplied by 256, which the
//     pre-scaled sx undoes;
//   * SEVERAL activation rows (gemv_dp4a_kernel, M = 2..4): with one weight row per warp every row would cost
//     a pass over M * K bytes of shared memory -- at M >= 2 more than the multiprocessor can deliver in the
//     time the weights take to arrive.  So a warp owns two weight rows per trip (four on short rows) and reads
//     the activation bytes once for all of them; because such a trip covers only half or a quarter of a row,
//     a slot is loaded again -- for the next trip of the unit, or the first trip of the warp's next unit -- as
//     soon as its words have been widened, which keeps eight loads per lane in flight at any time; and the
//     dot product accumulates onto the bit pattern of 1.5 * 2^23, so that read as fp32 it is
//     12582912 + 256 * P_g and fma(f, sw, -12582912 * sw) = 256 * P_g * sw exactly: no integer -> float
//     conversion per activation row;
//   * fp32 accumulation over groups per lane, xor-shuffle tree over lanes, fp16 store.
//
// The grid is persistent (every CTA resident) and the units are dealt round-robin to
// the warps; when the whole job is only a few rounds long, the number of warps per CTA and of
// CTAs per multiprocessor is chosen so that the rounds come out full.
// The kernel is launched as a programmatic dependent of the kernel before it (normally the
// fused transform+quantisation): it gets resident and prefetches while that kernel drains, and
// reads the activations only after griddepcontrol.wait.
// Algorithmic HBM bytes per call: 9*N*K/16 (codes + scales of W) + 9*M*K/16 + 2*M*N.
#include <cstdlib>

#include "common.cuh"
#include "peer_common.cuh"

namespace wush {

constexpr int GV_MAX_WARPS = 8;
constexpr uint32_t GV_MAGIC_BITS = 0x4B400000u;          // 1.5 * 2^23 as fp32
constexpr float GV_MAGIC = 12582912.0f;

// The loads of one trip of one warp: 8 slots of 16 bytes of codes + one scale per lane (144 B
// in flight per lane).  A trip covers R weight rows; row r of the unit owns slots
// r*U .. r*U+U-1 (U = 8/R), slot u holding group u*32 + lane of that row.
struct RowLoads {
    uint4 w[8];
    unsigned short s[8];
};

// Where the R rows of a trip start for this lane (group gb + lane of each row) and which of them exist.
template <int R>
struct TripBase {
    const uint8_t* wp[R];
    const unsigned short* sp[R];
    int g0;
    bool live[R];
};

template <int R>
__device__ __forceinline__ TripBase<R> trip_base(const uint8_t* __restrict__ wq, const unsigned short* __restrict__ ws16,
                                                 int unit, int gb, int lane, int G, int N, size_t K2, bool any)
{
    TripBase<R> t;
    t.g0 = gb + lane;
#pragma unroll
    for (int rr = 0; rr < R; ++rr) {
        const int row = unit * R + rr;
        t.live[rr] = any && row < N;
        t.wp[rr] = wq + (size_t)(t.live[rr] ? row : 0) * K2 + (size_t)t.g0 * 16;
        t.sp[rr] = ws16 + (size_t)(t.live[rr] ? row : 0) * G + t.g0;
    }
    return t;
}

// Slot u of every row of the trip: group g0 + 32 u.
template <int R>
__device__ __forceinline__ void issue_slot_loads(RowLoads& r, const TripBase<R>& t, int u, int G)
{
    constexpr int U = 8 / R;
#pragma unroll
    for (int rr = 0; rr < R; ++rr) {
        if (t.live[rr] && t.g0 + u * 32 < G) {
            r.w[rr * U + u] = ldg_nc_v4(t.wp[rr] + u * 512);
            r.s[rr * U + u] = __ldg(t.sp[rr] + u * 32);
        } else {
            r.w[rr * U + u] = make_uint4(0, 0, 0, 0);
            r.s[rr * U + u] = 0;
        }
    }
}

template <int R>
__device__ __forceinline__ void issue_unit_loads(RowLoads& r, const uint8_t* __restrict__ wq,
                                                 const unsigned short* __restrict__ ws16, int unit, int gb, int lane,
                                                 int G, int N, size_t K2)
{
    constexpr int U = 8 / R;
#pragma unroll
    for (int rr = 0; rr < R; ++rr) {
        const int row = unit * R + rr;
        const bool live = row < N;
        const int g0 = gb + lane;
        // one base address per row; the U slots sit at fixed offsets from it
        const uint8_t* wp = wq + (size_t)(live ? row : 0) * K2 + (size_t)g0 * 16;
        const unsigned short* sp = ws16 + (size_t)(live ? row : 0) * G + g0;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (live && g0 + u * 32 < G) {
                r.w[rr * U + u] = ldg_nc_v4(wp + u * 512);
                r.s[rr * U + u] = __ldg(sp + u * 32);
            } else {
                r.w[rr * U + u] = make_uint4(0, 0, 0, 0);
                r.s[rr * U + u] = 0;
            }
        }
    }
}

// ONE activation row.  R = weight rows per warp and trip; R > 1 is used when a row has at most 32 * (8/R) groups,
// so that short rows still put 8 loads per lane in flight; a trip is then a whole unit.  The loads of a trip go
// out together (the next unit's first trip before the reduction of the current one): with a single activation row
// there is so little arithmetic per byte that this simpler schedule streams at the HBM rate, in fewer registers
// (three CTAs per multiprocessor) than the slot-by-slot reloading of the kernel for several rows below.
// PUSH: instead of y the result goes into slot (step & 1, rank) of EVERY rank's exchange buffer
// (remote stores over NVLink from the epilogue); when the last CTA is done it publishes the step
// to all ranks.  The sum over ranks is then a purely local read (peer_reduce.cu).
template <int R, bool PUSH>
__global__ void __launch_bounds__(GV_MAX_WARPS * 32)
gemv_row_kernel(const uint32_t* __restrict__ xq,          // (MB, K/8) words
                 const __nv_bfloat16* __restrict__ xs,     // (MB, G)
                 const uint8_t* __restrict__ wq,           // (N, K/2)
                 const __nv_bfloat16* __restrict__ ws,     // (N, G)
                 __half* __restrict__ y,                   // (MB, N); unused with PUSH
                 int N, int K, const PeerTable peers)
{
    constexpr int U = 8 / R, MB = 1;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int G = K >> 5;
    uint4* xe = reinterpret_cast<uint4*>(smem_raw);                    // [MB][G] even codes * 16
    uint4* xo = xe + (size_t)MB * G;                                   // [MB][G] odd codes * 16
    float* sxf = reinterpret_cast<float*>(xo + (size_t)MB * G);        // [MB][G] sx / 256

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const size_t K2 = (size_t)K >> 1;
    const int units = (N + R - 1) / R;
    const int stride = gridDim.x * warps;
    int unit = blockIdx.x * warps + warp;
    const unsigned short* ws16 = reinterpret_cast<const unsigned short*>(ws);

    // While the producer of the activations may still be running, pull this warp's first unit
    // towards L2 (a prefetch cannot observe stale data), then wait for the producer.
    if (unit < units) {
        const int row0 = unit * R, nrows = min(R, N - row0);
        const uint8_t* cb = wq + (size_t)row0 * K2;
        for (size_t off = (size_t)lane * 128; off < (size_t)nrows * K2; off += 32 * 128) prefetch_l2(cb + off);
        const uint8_t* sb = reinterpret_cast<const uint8_t*>(ws16 + (size_t)row0 * G);
        for (size_t off = (size_t)lane * 128; off < (size_t)nrows * G * 2; off += 32 * 128) prefetch_l2(sb + off);
    }
    pdl_wait();

    // start the weight stream first: it does not depend on the shared-memory prologue
    RowLoads cur;
    if (unit < units) issue_unit_loads<R>(cur, wq, ws16, unit, 0, lane, G, N, K2);

    for (int idx = threadIdx.x; idx < MB * G; idx += blockDim.x) {
        uint4 w = *reinterpret_cast<const uint4*>(xq + (size_t)idx * 4);
        uint4 e, o;
        unpack_x16(w.x, e.x, o.x); unpack_x16(w.y, e.y, o.y);
        unpack_x16(w.z, e.z, o.z); unpack_x16(w.w, e.w, o.w);
        xe[idx] = e; xo[idx] = o;
        sxf[idx] = __bfloat162float(xs[idx]) * (1.0f / 256.0f);
    }
    __syncthreads();
    pdl_launch_dependents();            // a dependent may become resident as this grid drains; it waits before reading y
    unsigned int step = 0;
    size_t push_off = 0;
    if constexpr (PUSH) {               // the step counter is stable: the reduction of the previous step has completed
        step = *reinterpret_cast<volatile unsigned int*>(&peers.state->step);
        push_off = slot_offset(peers, step, peers.rank);
    }

    for (; unit < units; unit += stride) {
        float acc[R][MB];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MB; ++m) acc[r][m] = 0.f;
        for (int gb = 0; gb < G; gb += 32 * U) {
            if (gb) issue_unit_loads<R>(cur, wq, ws16, unit, gb, lane, G, N, K2);
#pragma unroll
            for (int slot = 0; slot < 8; ++slot) {
                const int g = min(gb + (slot % U) * 32 + lane, G - 1);  // lanes past the end carry zero weights
                uint4 ae, ao;
                unpack_x16(cur.w[slot].x, ae.x, ao.x); unpack_x16(cur.w[slot].y, ae.y, ao.y);
                unpack_x16(cur.w[slot].z, ae.z, ao.z); unpack_x16(cur.w[slot].w, ae.w, ao.w);
                const float sw = bf16_bits_to_f32(cur.s[slot]);
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    const uint4 ve = xe[m * G + g], vo = xo[m * G + g];
                    int d = dp4a_s8(ae.x, ve.x, 0); d = dp4a_s8(ao.x, vo.x, d);
                    d = dp4a_s8(ae.y, ve.y, d); d = dp4a_s8(ao.y, vo.y, d);
                    d = dp4a_s8(ae.z, ve.z, d); d = dp4a_s8(ao.z, vo.z, d);
                    d = dp4a_s8(ae.w, ve.w, d); d = dp4a_s8(ao.w, vo.w, d);
                    acc[slot / U][m] = fmaf((float)d, sxf[m * G + g] * sw, acc[slot / U][m]);
                }
            }
        }
        // next unit's first trip goes out before the reduction of this one
        const int next = unit + stride;
        if (next < units) issue_unit_loads<R>(cur, wq, ws16, next, 0, lane, G, N, K2);
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MB; ++m) {
#pragma unroll
                for (int off = 16; off; off >>= 1) acc[r][m] += __shfl_xor_sync(0xffffffffu, acc[r][m], off);
            }
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int n = unit * R + r;
                if (n < N) {
#pragma unroll
                    for (int m = 0; m < MB; ++m) {
                        const __half h = __float2half_rn(acc[r][m]);
                        if constexpr (PUSH) {
                            for (int p = 0; p < peers.world; ++p)
                                reinterpret_cast<__half*>(peers.base[p] + push_off)[(size_t)m * N + n] = h;
                        } else {
                            y[(size_t)m * N + n] = h;
                        }
                    }
                }
            }
        }
    }
    if constexpr (PUSH) {
        __threadfence_system();                            // this thread's remote stores are ordered before the flag
        __syncthreads();
        if (threadIdx.x < 32) comm_count_and_publish(peers, step, threadIdx.x);
    }
}

// SEVERAL activation rows (MB = 2..4).  R = weight rows per warp and trip (2 or 4): a trip is 32 * (8/R) groups of each.
// PUSH: instead of y the result goes into slot (step & 1, rank) of EVERY rank's exchange buffer
// (remote stores over NVLink from the epilogue); when the last CTA is done it publishes the step
// to all ranks.  The sum over ranks is then a purely local read (peer_reduce.cu).
template <int MB, int R, bool PUSH>
__global__ void __launch_bounds__(GV_MAX_WARPS * 32, 2)
gemv_dp4a_kernel(const uint32_t* __restrict__ xq,          // (MB, K/8) words
                 const __nv_bfloat16* __restrict__ xs,     // (MB, G)
                 const uint8_t* __restrict__ wq,           // (N, K/2)
                 const __nv_bfloat16* __restrict__ ws,     // (N, G)
                 __half* __restrict__ y,                   // (MB, N); unused with PUSH
                 int N, int K, const PeerTable peers)
{
    constexpr int U = 8 / R;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int G = K >> 5;
    uint4* xe = reinterpret_cast<uint4*>(smem_raw);                    // [MB][G] even codes * 16
    uint4* xo = xe + (size_t)MB * G;                                   // [MB][G] odd codes * 16
    float* sxf = reinterpret_cast<float*>(xo + (size_t)MB * G);        // [MB][G] sx / 256

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const size_t K2 = (size_t)K >> 1;
    const int units = (N + R - 1) / R;
    const int stride = gridDim.x * warps;
    int unit = blockIdx.x * warps + warp;
    const unsigned short* ws16 = reinterpret_cast<const unsigned short*>(ws);

    // While the producer of the activations may still be running, pull this warp's first unit
    // towards L2 (a prefetch cannot observe stale data), then wait for the producer.
    if (unit < units) {
        const int row0 = unit * R, nrows = min(R, N - row0);
        const uint8_t* cb = wq + (size_t)row0 * K2;
        for (size_t off = (size_t)lane * 128; off < (size_t)nrows * K2; off += 32 * 128) prefetch_l2(cb + off);
        const uint8_t* sb = reinterpret_cast<const uint8_t*>(ws16 + (size_t)row0 * G);
        for (size_t off = (size_t)lane * 128; off < (size_t)nrows * G * 2; off += 32 * 128) prefetch_l2(sb + off);
    }
    pdl_wait();

    // start the weight stream first: it does not depend on the shared-memory prologue
    RowLoads cur;
    {
        const TripBase<R> first = trip_base<R>(wq, ws16, unit, 0, lane, G, N, K2, unit < units);
#pragma unroll
        for (int u = 0; u < U; ++u) issue_slot_loads<R>(cur, first, u, G);
    }

    for (int idx = threadIdx.x; idx < MB * G; idx += blockDim.x) {
        uint4 w = *reinterpret_cast<const uint4*>(xq + (size_t)idx * 4);
        uint4 e, o;
        unpack_x16(w.x, e.x, o.x); unpack_x16(w.y, e.y, o.y);
        unpack_x16(w.z, e.z, o.z); unpack_x16(w.w, e.w, o.w);
        xe[idx] = e; xo[idx] = o;
        sxf[idx] = __bfloat162float(xs[idx]) * (1.0f / 256.0f);
    }
    __syncthreads();
    pdl_launch_dependents();            // a dependent may become resident as this grid drains; it waits before reading y
    unsigned int step = 0;
    size_t push_off = 0;
    if constexpr (PUSH) {               // the step counter is stable: the reduction of the previous step has completed
        step = *reinterpret_cast<volatile unsigned int*>(&peers.state->step);
        push_off = slot_offset(peers, step, peers.rank);
    }

    // The work of a warp is a sequence of trips: 32 * U groups of R rows each, unit after unit.  A slot is loaded
    // again, for the NEXT trip, as soon as its words have been widened, so the lane keeps 8 loads in flight all the
    // time -- across trips of a unit and across units alike.
    float acc[R][MB];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MB; ++m) acc[r][m] = 0.f;
    int gb = 0;
    while (unit < units) {
        int n_unit = unit, n_gb = gb + 32 * U;
        if (n_gb >= G) { n_gb = 0; n_unit = unit + stride; }
        const TripBase<R> nxt = trip_base<R>(wq, ws16, n_unit, n_gb, lane, G, N, K2, n_unit < units);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int g = min(gb + u * 32 + lane, G - 1);               // lanes past the end carry zero weights
            // the R rows' words of this group, widened once; then every activation row is read once for all of them
            uint4 ae[R], ao[R];
            float sw[R], csw[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint4 w = cur.w[r * U + u];
                unpack_x16(w.x, ae[r].x, ao[r].x); unpack_x16(w.y, ae[r].y, ao[r].y);
                unpack_x16(w.z, ae[r].z, ao[r].z); unpack_x16(w.w, ae[r].w, ao[r].w);
                sw[r] = bf16_bits_to_f32(cur.s[r * U + u]);
                csw[r] = -GV_MAGIC * sw[r];                              // exact: 2 x 8 significant bits
            }
            issue_slot_loads<R>(cur, nxt, u, G);
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                const uint4 ve = xe[m * G + g], vo = xo[m * G + g];
                const float sx = sxf[m * G + g];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    // the sum starts from the bits of 1.5 * 2^23: read as fp32 it is 12582912 + 256 * P_g, and
                    // fma(f, sw, -12582912 * sw) = 256 * P_g * sw exactly -- no integer -> float conversion
                    int d = dp4a_s8(ae[r].x, ve.x, (int)GV_MAGIC_BITS); d = dp4a_s8(ao[r].x, vo.x, d);
                    d = dp4a_s8(ae[r].y, ve.y, d); d = dp4a_s8(ao[r].y, vo.y, d);
                    d = dp4a_s8(ae[r].z, ve.z, d); d = dp4a_s8(ao[r].z, vo.z, d);
                    d = dp4a_s8(ae[r].w, ve.w, d); d = dp4a_s8(ao[r].w, vo.w, d);
                    acc[r][m] = fmaf(fmaf(__int_as_float(d), sw[r], csw[r]), sx, acc[r][m]);
                }
            }
        }
        if (n_gb == 0) {                                                 // the unit is complete
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MB; ++m) {
#pragma unroll
                    for (int off = 16; off; off >>= 1) acc[r][m] += __shfl_xor_sync(0xffffffffu, acc[r][m], off);
                }
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int n = unit * R + r;
                    if (n < N) {
#pragma unroll
                        for (int m = 0; m < MB; ++m) {
                            const __half h = __float2half_rn(acc[r][m]);
                            if constexpr (PUSH) {
                                for (int p = 0; p < peers.world; ++p)
                                    reinterpret_cast<__half*>(peers.base[p] + push_off)[(size_t)m * N + n] = h;
                            } else {
                                y[(size_t)m * N + n] = h;
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MB; ++m) acc[r][m] = 0.f;
        }
        unit = n_unit;
        gb = n_gb;
    }
    if constexpr (PUSH) {
        __threadfence_system();                            // this thread's remote stores are ordered before the flag
        __syncthreads();
        if (threadIdx.x < 32) comm_count_and_publish(peers, step, threadIdx.x);
    }
}

size_t gemv_smem_bytes(int M, int64_t K) { return (size_t)M * (K / 32) * (16 + 16 + 4); }

// The kernel of a template point: the single-row kernel for one activation row, the row-sharing one otherwise.
template <int MB, int R, bool PUSH>
constexpr auto kernel_of()
{
    if constexpr (MB == 1) return &gemv_row_kernel<R, PUSH>;
    else return &gemv_dp4a_kernel<MB, R, PUSH>;
}

// Shape of the persistent grid: `warps` per CTA and `ctas` per multiprocessor such that the
// units, dealt round-robin to all resident warps, fill whole rounds (a half-empty last round
// costs a full memory latency at a fraction of the bandwidth).
struct GemvShape { int warps, ctas_per_sm; };

template <int MB, int R, bool PUSH>
static GemvShape pick_shape(size_t smem, long long units)
{
    struct Cache { size_t smem; int per_sm[GV_MAX_WARPS + 1]; };
    static thread_local Cache cache = {~size_t(0), {}};
    if (cache.smem != smem) {
        for (int w = 4; w <= GV_MAX_WARPS; ++w) {
            int q = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&q, kernel_of<MB, R, PUSH>(), w * 32, smem) != cudaSuccess) q = 0;
            cache.per_sm[w] = q;
        }
        cache.smem = smem;
    }
    const int sms = sm_count();
    // Many rounds: warps drift apart and the last round costs little; take the most resident
    // warps in the fewest CTAs.  Few rounds: search for a shape that fills them.
    if (cache.per_sm[GV_MAX_WARPS] >= 1 &&
        (double)units / ((double)sms * GV_MAX_WARPS * cache.per_sm[GV_MAX_WARPS]) >= 8.0)
        return {GV_MAX_WARPS, cache.per_sm[GV_MAX_WARPS]};
    GemvShape best = {8, 1};
    double best_score = -1.0;
    for (int w = 4; w <= GV_MAX_WARPS; ++w) {
        for (int c = 1; c <= cache.per_sm[w]; ++c) {
            const int resident = w * c;
            if (resident < 16 && (w < GV_MAX_WARPS || c < cache.per_sm[w])) continue;      // too few loads in flight
            if (resident > 64) continue;
            const double rounds = (double)units / ((double)sms * resident);
            const double whole = rounds <= 1.0 ? 1.0 : (double)(long long)(rounds + 0.999999);
            // fullness of the rounds; a mild preference for more resident warps and for fewer,
            // larger CTAs (each CTA expands the activations for itself)
            const double score = rounds / whole + 0.002 * resident + 0.0002 * w;
            if (score > best_score) { best_score = score; best = {w, c}; }
        }
    }
    return best;
}

template <int MB, int R, bool PUSH>
static int launch_gemv(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t N,
                       int64_t K, void* y, const PeerTable& peers, cudaStream_t st)
{
    const size_t smem = gemv_smem_bytes(MB, K);
    const long long units = (N + R - 1) / R;
    // the choice depends on the shape only: remember the last one (decode calls repeat shapes)
    static thread_local long long last_units = -1;
    static thread_local size_t last_smem = 0;
    static thread_local GemvShape shape = {8, 1};
    if (last_units != units || last_smem != smem) {
        shape = pick_shape<MB, R, PUSH>(smem, units);
        last_units = units;
        last_smem = smem;
    }
    long long ctas = (long long)sm_count() * shape.ctas_per_sm;
    const long long needed = (units + shape.warps - 1) / shape.warps;
    if (ctas > needed) ctas = needed;
    cudaError_t e = launch_dependent(kernel_of<MB, R, PUSH>(), dim3((unsigned)ctas), dim3(shape.warps * 32), smem, st,
                                     (const uint32_t*)xq, (const __nv_bfloat16*)xs, wq, (const __nv_bfloat16*)ws, (__half*)y,
                                     (int)N, (int)K, peers);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "gemv launch: %s", cudaGetErrorString(e));
    return WUSH_OK;
}

template <int MB, int R>
static cudaError_t set_attr()
{
    cudaError_t e = cudaFuncSetAttribute(kernel_of<MB, R, false>(), cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e == cudaSuccess && MB <= 2)
        e = cudaFuncSetAttribute(kernel_of<MB, R, true>(), cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    return e;
}

int gemv_set_attributes()
{
    cudaError_t e;
    if ((e = set_attr<1, 1>()) != cudaSuccess || (e = set_attr<1, 2>()) != cudaSuccess || (e = set_attr<1, 4>()) != cudaSuccess ||
        (e = set_attr<2, 2>()) != cudaSuccess || (e = set_attr<2, 4>()) != cudaSuccess ||
        (e = set_attr<3, 2>()) != cudaSuccess || (e = set_attr<3, 4>()) != cudaSuccess ||
        (e = set_attr<4, 2>()) != cudaSuccess || (e = set_attr<4, 4>()) != cudaSuccess)
        return fail(WUSH_ERR_CUDA, "gemv: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    return WUSH_OK;
}

// Rows per warp and trip.  One activation row: as many rows as it takes for a lane's 8 loads to cover them (one row
// from K = 8192 on).  Several activation rows, from measurements at M = 2..4 on K x N = 1024 x 4096, 2048 x 8192,
// 4096 x 24576, 8192 x 7168, 8192 x 57344 and 28672 x 8192: two rows everywhere, except four on short rows;
// WUSH_GEMV_ROWS=2|4 overrides that choice (measurements).
template <int MB, bool PUSH>
static int launch_rows(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t N, int64_t K,
                       void* y, const PeerTable& peers, cudaStream_t st)
{
    const int64_t slots = (K / 32 + 31) / 32;              // 16-byte loads per lane and row
    if constexpr (MB == 1) {
        if (slots <= 2) return launch_gemv<1, 4, PUSH>(xq, xs, wq, ws, N, K, y, peers, st);
        if (slots <= 4) return launch_gemv<1, 2, PUSH>(xq, xs, wq, ws, N, K, y, peers, st);
        return launch_gemv<1, 1, PUSH>(xq, xs, wq, ws, N, K, y, peers, st);
    } else {
        int rows = slots <= 2 ? 4 : 2;
        if (const char* v = std::getenv("WUSH_GEMV_ROWS")) {
            if (v[0] == '2' || v[0] == '4') rows = v[0] - '0';
        }
        if (rows == 4) return launch_gemv<MB, 4, PUSH>(xq, xs, wq, ws, N, K, y, peers, st);
        return launch_gemv<MB, 2, PUSH>(xq, xs, wq, ws, N, K, y, peers, st);
    }
}

// M in 1..4, shared memory must fit (checked by the dispatcher).
int gemv_dispatch(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N,
                  int64_t K, void* y, cudaStream_t st)
{
    const PeerTable none = {};
    switch (M) {
        case 1: return launch_rows<1, false>(xq, xs, wq, ws, N, K, y, none, st);
        case 2: return launch_rows<2, false>(xq, xs, wq, ws, N, K, y, none, st);
        case 3: return launch_rows<3, false>(xq, xs, wq, ws, N, K, y, none, st);
        case 4: return launch_rows<4, false>(xq, xs, wq, ws, N, K, y, none, st);
    }
    return fail(WUSH_ERR_INVALID_ARGUMENT, "gemv: M=%lld outside 1..4", (long long)M);
}

// The same product with its result pushed into the exchange buffers of all ranks (M <= 2).
int gemv_dispatch_push(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M, int64_t N,
                       int64_t K, const PeerTable& peers, cudaStream_t st)
{
    switch (M) {
        case 1: return launch_rows<1, true>(xq, xs, wq, ws, N, K, nullptr, peers, st);
        case 2: return launch_rows<2, true>(xq, xs, wq, ws, N, K, nullptr, peers, st);
    }
    return fail(WUSH_ERR_UNSUPPORTED, "gemv(push): M=%lld outside 1..2", (long long)M);
}

}  // namespace wush
