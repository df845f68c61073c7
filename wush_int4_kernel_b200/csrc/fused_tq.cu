// Fused WUSH block transform + sigma-clip INT4 quantisation (C-ABI
// wush_fused_transform_quant_int4).
//
//   x'[r][g][j] = sum_i x[r][g][i] * T[g][j][i]      (fp32, NOT rounded to bf16)
//   (q, s)      = sigma-clip quantisation of each 32-wide group of x'
//
// Two variants behind one entry point:
//
// EXACT  (reference fused_transform_quant_int4, csrc/fused_tq_int4.cu:27-85): serial fp32
//   arithmetic in the reference's order -- i ascending, multiply and add rounded
//   separately, then the serial statistics -- so the bytes equal the fp32 mirror of the
//   reference's tests (tests/test_sw2.py:12-24).  One thread per (row, group); a CTA shares
//   one T block through shared memory (broadcast reads).
//
// FAST   (reference _wmma / _v3 / _smallm, csrc/fused_tq_wmma.cu:22-129,
//   csrc/fused_tq_v3.cu:26-107, csrc/fused_tq_smallm.cu:19-87): one warp owns one group g and
//   walks down the rows 16 at a time.  The 32x32 block of T lives in registers as the B
//   operand of bf16 tensor-core MMAs (bf16 products are exact in fp32, accumulation is
//   fp32), the 16x32 slab of x is the A operand, loaded with one 16-byte load per row per
//   lane.  The k index inside a group and the order of T's rows are permuted so that
//     - every operand register comes straight out of a 16-byte load (no shuffles), and
//     - each lane ends up with 8 CONSECUTIVE outputs of a row, i.e. one 4-byte word of
//       packed codes, and a quad holds the whole group.
//   Group statistics are an in-lane sum of 8 plus a two-step xor-shuffle across the quad.
//   Results differ from EXACT only through summation order (rare +-1 code flips).
//
// Algorithmic HBM bytes: 2*M*K (x) + 64*K (T, read once, L2 resident after) + M*K/2 (codes)
// + M*K/16 (scales).
#include <algorithm>

#include "common.cuh"

namespace wush {

// ----------------------------------------------------------------------------------------
// EXACT
// ----------------------------------------------------------------------------------------
constexpr int TQE_ROWS = 128;

__global__ void __launch_bounds__(TQE_ROWS)
fused_tq_exact_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ t,
                      uint4* __restrict__ q_out, __nv_bfloat16* __restrict__ s_out,
                      long long rows, int C)
{
    __shared__ float4 ts[32 * 8];                         // T[g] as fp32, [j][i]
    const int g = blockIdx.y;
    const __nv_bfloat16* tg = t + (size_t)g * 1024;
    for (int e = threadIdx.x; e < 256; e += TQE_ROWS) {   // 4 elements per step
        uint2 raw = *reinterpret_cast<const uint2*>(tg + e * 4);
        ts[e] = make_float4(bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y));
    }
    __syncthreads();
    const long long r = (long long)blockIdx.x * TQE_ROWS + threadIdx.x;
    if (r >= rows) return;

    float xv[32];
    const uint4* xg = reinterpret_cast<const uint4*>(x + ((size_t)r * C + g) * 32);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint4 v = xg[c];
        xv[c * 8 + 0] = bf16_lo(v.x); xv[c * 8 + 1] = bf16_hi(v.x);
        xv[c * 8 + 2] = bf16_lo(v.y); xv[c * 8 + 3] = bf16_hi(v.y);
        xv[c * 8 + 4] = bf16_lo(v.z); xv[c * 8 + 5] = bf16_hi(v.z);
        xv[c * 8 + 6] = bf16_lo(v.w); xv[c * 8 + 7] = bf16_hi(v.w);
    }
    float xj[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        float acc = 0.f;
#pragma unroll
        for (int i4 = 0; i4 < 8; ++i4) {
            float4 tv = ts[j * 8 + i4];
            acc = __fadd_rn(acc, __fmul_rn(xv[i4 * 4 + 0], tv.x));
            acc = __fadd_rn(acc, __fmul_rn(xv[i4 * 4 + 1], tv.y));
            acc = __fadd_rn(acc, __fmul_rn(xv[i4 * 4 + 2], tv.z));
            acc = __fadd_rn(acc, __fmul_rn(xv[i4 * 4 + 3], tv.w));
        }
        xj[j] = acc;
    }
    uint4 packed;
    uint32_t sbits;
    quant_group_exact(xj, &packed, &sbits);
    q_out[(size_t)r * C + g] = packed;
    s_out[(size_t)r * C + g] = __ushort_as_bfloat16((unsigned short)sbits);
}

// ----------------------------------------------------------------------------------------
// FAST
// ----------------------------------------------------------------------------------------
// D = A * B (no accumulator input: saves clearing the registers)
__device__ __forceinline__ void mma_bf16_16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                     uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Two rows' 8 outputs each (row a = gid, row b = gid + 8) held by one lane as four float2 per row ->
// statistics over the quad -> one word of codes per row.  Instruction count is what bounds this kernel
// at prefill sizes, hence:
//   * sums and sums of squares on packed fp32 pairs;
//   * the quad reduction is a transposing butterfly: after the first exchange even lanes carry row a's
//     (s1, s2) and odd lanes row b's, so the second exchange and the whole scale chain (square root,
//     bf16 rounding, reciprocal) run ONCE for both rows -- lanes of either parity work on their own row --
//     and one more exchange hands each lane the other row's reciprocal;
//   * clamping rides the FMA: u = sat(v / (14 scale) + 1/2) is clamp((q + 7) / 14, 0, 1), a second FMA
//     onto 1.5 * 2^23 rounds 14 u to the integer q + 7 in the low mantissa bits.  The intermediate
//     rounding of u moves a code only where v / scale is within ~1e-6 of a tie.
// `sbits` is row a's scale on even lanes and row b's on odd lanes.
__device__ __forceinline__ void quantise_two_row_octets(const float2 (&a)[4], const float2 (&b)[4], int lane, uint32_t* word_a,
                                                        uint32_t* word_b, uint32_t* sbits) {
    float2 sa = __fadd2_rn(__fadd2_rn(a[0], a[1]), __fadd2_rn(a[2], a[3]));
    float2 sb = __fadd2_rn(__fadd2_rn(b[0], b[1]), __fadd2_rn(b[2], b[3]));
    float2 qa = __ffma2_rn(a[3], a[3], __ffma2_rn(a[2], a[2], __ffma2_rn(a[1], a[1], __fmul2_rn(a[0], a[0]))));
    float2 qb = __ffma2_rn(b[3], b[3], __ffma2_rn(b[2], b[2], __ffma2_rn(b[1], b[1], __fmul2_rn(b[0], b[0]))));
    const float2 xa = make_float2(sa.x + sa.y, qa.x + qa.y), xb = make_float2(sb.x + sb.y, qb.x + qb.y);   // (s1, s2) per row
    const bool odd = lane & 1;
    float2 keep = odd ? xb : xa;
    const float2 send = odd ? xa : xb;
    keep.x += __shfl_xor_sync(0xffffffffu, send.x, 1);
    keep.y += __shfl_xor_sync(0xffffffffu, send.y, 1);
    keep.x += __shfl_xor_sync(0xffffffffu, keep.x, 2);
    keep.y += __shfl_xor_sync(0xffffffffu, keep.y, 2);
    float scale;
    *sbits = sigma_clip_scale(keep.x, keep.y, &scale);
    const float mine = __frcp_rn(scale) * (1.0f / 14.0f);
    const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
    const float inv_a = odd ? other : mine, inv_b = odd ? mine : other;
    const float2 fourteen = make_float2(14.f, 14.f), magic = make_float2(12582912.f, 12582912.f);   // 1.5 * 2^23
    uint32_t wa = 0, wb = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        float2 ua, ub;
        asm("fma.rn.sat.f32 %0, %1, %2, 0f3F000000;" : "=f"(ua.x) : "f"(a[e].x), "f"(inv_a));
        asm("fma.rn.sat.f32 %0, %1, %2, 0f3F000000;" : "=f"(ua.y) : "f"(a[e].y), "f"(inv_a));
        asm("fma.rn.sat.f32 %0, %1, %2, 0f3F000000;" : "=f"(ub.x) : "f"(b[e].x), "f"(inv_b));
        asm("fma.rn.sat.f32 %0, %1, %2, 0f3F000000;" : "=f"(ub.y) : "f"(b[e].y), "f"(inv_b));
        const float2 fa = __ffma2_rn(ua, fourteen, magic), fb = __ffma2_rn(ub, fourteen, magic);
        // bits(f) = bits(magic) + (q + 7): one multiply-add per element builds the word of nibbles q + 7 plus a constant
        wa = __float_as_uint(fa.x) * (1u << (8 * e)) + wa;
        wa = __float_as_uint(fa.y) * (1u << (8 * e + 4)) + wa;
        wb = __float_as_uint(fb.x) * (1u << (8 * e)) + wb;
        wb = __float_as_uint(fb.y) * (1u << (8 * e + 4)) + wb;
    }
    // constant off with q + 8 left in every nibble, then bit 3 flipped: two's complement nibbles
    *word_a = (wa - (0x4B400000u - 1u) * 0x11111111u) ^ 0x88888888u;
    *word_b = (wb - (0x4B400000u - 1u) * 0x11111111u) ^ 0x88888888u;
}

// SiLU(gate) * up of 8 fp16 pairs -> 8 bf16 in one 16-byte register set.  fp32 throughout:
// s = g / (1 + exp(-g)), h = bf16(s * u) -- what `(silu(gate.float()) * up.float()).bfloat16()`
// computes, the rounding of h to bf16 being forced by the transform op's input type.
__device__ __forceinline__ uint32_t silu_mul_pair(uint32_t g2, uint32_t u2) {
    const float2 g = __half22float2(*reinterpret_cast<const __half2*>(&g2));
    const float2 u = __half22float2(*reinterpret_cast<const __half2*>(&u2));
    const float a = __fmul_rn(__fdiv_rn(g.x, __fadd_rn(1.0f, expf(-g.x))), u.x);
    const float b = __fmul_rn(__fdiv_rn(g.y, __fadd_rn(1.0f, expf(-g.y))), u.y);
    return f32_to_bf16_bits(a) | (f32_to_bf16_bits(b) << 16);
}

// 8 consecutive inputs of row r for this lane.  SILU: `x` is the fp16 output of a fused gate+up
// projection, (rows, 2K) with the gate half first; the activation is computed on the fly.
// 8 consecutive inputs of one row for this lane, `p` pointing at them.  SILU: `p` points into the gate half of
// the fp16 output of a fused gate+up projection, (rows, 2K) with the gate half first and the up half K elements
// (C * 32) further; the activation is computed on the fly.
template <bool SILU>
__device__ __forceinline__ uint4 load_octet(const void* p, int C) {
    if constexpr (!SILU) {
        return ldg_nc_v4(p);
    } else {
        const __half* gate = reinterpret_cast<const __half*>(p);
        const uint4 gv = ldg_nc_v4(gate), uv = ldg_nc_v4(gate + (size_t)C * 32);
        return make_uint4(silu_mul_pair(gv.x, uv.x), silu_mul_pair(gv.y, uv.y), silu_mul_pair(gv.z, uv.z),
                          silu_mul_pair(gv.w, uv.w));
    }
}

template <bool SILU>
__global__ void __launch_bounds__(256)
fused_tq_fast_kernel(const void* __restrict__ x, const __nv_bfloat16* __restrict__ t,
                     uint32_t* __restrict__ q_out,        // rows * C * 4 words
                     __nv_bfloat16* __restrict__ s_out, long long rows, int C, int rows_per_cta)
{
    pdl_launch_dependents();                              // the consumer may get resident; it waits before reading q/s
    const int warps = blockDim.x >> 5;
    const int g = blockIdx.x * warps + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    // This kernel may itself have been launched early (programmatic dependent of the kernel that
    // produces x): pull the T block towards L2 meanwhile, read nothing before the wait.
    if (g < C) {
        const uint8_t* tb = reinterpret_cast<const uint8_t*>(t + (size_t)g * 1024);
        if (lane < 16) prefetch_l2(tb + lane * 128);
    }
    pdl_wait();
    if (g >= C) return;                                   // whole warp leaves together
    const long long r_begin = (long long)blockIdx.y * rows_per_cta;
    int left = (int)(min(rows, r_begin + rows_per_cta) - r_begin);      // rows of this CTA not yet done

    // B operand: T[g] rows in the permuted order j(nt, n) = 8*(n>>1) + 2*nt + (n&1), n = gid.
    uint4 bt[4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
        const int j = 8 * (gid >> 1) + 2 * nt + (gid & 1);
        bt[nt] = *reinterpret_cast<const uint4*>(t + (size_t)g * 1024 + j * 32 + tig * 8);
    }

    // Running pointers of this lane (row gid of the slab; row gid + 8 sits a fixed distance further): 64-bit index
    // arithmetic per access was a fifth of the loop's instructions.
    constexpr int XE = SILU ? 2 : 1;                      // input elements per output element and row (gate | up)
    const size_t x_row = (size_t)C * 32 * XE * 2;         // bytes per input row (2-byte elements)
    const uint8_t* xp = reinterpret_cast<const uint8_t*>(x) + (size_t)(r_begin + gid) * x_row + ((size_t)g * 32 + tig * 8) * 2;
    uint32_t* qp = q_out + ((size_t)(r_begin + gid) * C + g) * 4 + tig;
    // lane 0 of a quad stores row a's scale, lane 1 row b's
    __nv_bfloat16* sp = s_out + (size_t)(r_begin + gid + (tig == 1 ? 8 : 0)) * C + g;
    const size_t x_half = 8 * x_row, x_slab = 16 * x_row;
    const size_t q_half = (size_t)8 * C * 4, q_slab = (size_t)16 * C * 4, s_slab = (size_t)16 * C;
    const int s_row = gid + (tig == 1 ? 8 : 0);

    const uint4 zero4 = make_uint4(0, 0, 0, 0);
    uint4 xa = gid < left ? load_octet<SILU>(xp, C) : zero4;
    uint4 xb = gid + 8 < left ? load_octet<SILU>(xp + x_half, C) : zero4;
    for (; left > 0; left -= 16) {
        // prefetch the next slab while this one is in the tensor core
        xp += x_slab;
        // (pulling further slabs towards L2 with prefetch instructions changed nothing: 28.5 us at M = 4096, K = 8192
        // with or without; nor did cutting the instruction count from 19.4 M to 11.5 M, nor CTAs of 16 or 32 warps that read 1 or
        // 2 KB of a row at a time -- a warp needs about 1.7 us per slab whatever is done around it)
        uint4 nxa, nxb;
        if (left >= 32) {                                 // the common case: a whole next slab
            nxa = load_octet<SILU>(xp, C);
            nxb = load_octet<SILU>(xp + x_half, C);
        } else {
            nxa = gid + 16 < left ? load_octet<SILU>(xp, C) : zero4;
            nxb = gid + 24 < left ? load_octet<SILU>(xp + x_half, C) : zero4;
        }

        float acc[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            mma_bf16_16816_first(acc[nt], xa.x, xb.x, xa.y, xb.y, bt[nt].x, bt[nt].y);
            mma_bf16_16816(acc[nt], xa.z, xb.z, xa.w, xb.w, bt[nt].z, bt[nt].w);
        }
        float2 va[4], vb[4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            va[nt] = make_float2(acc[nt][0], acc[nt][1]);
            vb[nt] = make_float2(acc[nt][2], acc[nt][3]);
        }
        uint32_t wa, wb, sbits;
        quantise_two_row_octets(va, vb, lane, &wa, &wb, &sbits);   // all lanes take part in the shuffles
        if (left >= 16) {
            qp[0] = wa;
            qp[q_half] = wb;
            if (tig < 2) *sp = __ushort_as_bfloat16((unsigned short)sbits);
        } else {
            if (gid < left) qp[0] = wa;
            if (gid + 8 < left) qp[q_half] = wb;
            if (tig < 2 && s_row < left) *sp = __ushort_as_bfloat16((unsigned short)sbits);
        }
        qp += q_slab;
        sp += s_slab;
        xa = nxa; xb = nxb;
    }
}

// FAST launch: warps per CTA and rows per CTA chosen so that small M still spreads over the SMs.
template <bool SILU>
static int launch_fast(const void* x, const void* t, int64_t rows, int64_t C, uint8_t* q, void* s, cudaStream_t st)
{
    int warps, rows_per_cta;
    if (rows <= 32) { warps = 2; rows_per_cta = 32; }
    else if (rows <= 512) { warps = 4; rows_per_cta = 64; }
    else {
        // one balanced wave: four CTAs of 8 warps (64 registers per thread) are resident per multiprocessor; with
        // 128 rows per CTA, M = 4096 and K = 8192 made 1024 CTAs for 592 places (two rounds, the second 73 % full)
        warps = 8;
        const int64_t gx = (C + warps - 1) / warps, places = 4LL * sm_count();
        const int64_t gy_wave = std::max<int64_t>(1, places / gx);
        rows_per_cta = (int)std::max<int64_t>(128, ((rows + gy_wave - 1) / gy_wave + 15) / 16 * 16);
    }
    const int64_t gy = (rows + rows_per_cta - 1) / rows_per_cta;
    WUSH_REQUIRE(gy <= 65535, "fused_tq: too many rows");
    dim3 grid((unsigned)((C + warps - 1) / warps), (unsigned)gy);
    cudaError_t e = launch_dependent(fused_tq_fast_kernel<SILU>, grid, dim3(warps * 32), (size_t)0, st, x, (const __nv_bfloat16*)t,
                                     (uint32_t*)q, (__nv_bfloat16*)s, (long long)rows, (int)C, rows_per_cta);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "fused_tq_fast launch: %s", cudaGetErrorString(e));
    return WUSH_OK;
}

}  // namespace wush

WUSH_API int wush_fused_transform_quant_int4(const void* x, const void* t, int64_t rows, int64_t K,
                                             int variant, uint8_t* q, void* s, void* stream)
{
    using namespace wush;
    if (int e = ensure_init()) return e;
    WUSH_REQUIRE(rows >= 0 && K > 0 && K % 32 == 0, "fused_tq: K must be a positive multiple of 32");
    WUSH_REQUIRE(variant == WUSH_TQ_EXACT || variant == WUSH_TQ_FAST, "fused_tq: unknown variant %d", variant);
    if (rows == 0) return WUSH_OK;
    WUSH_REQUIRE(x && t && q && s, "fused_tq: null pointer");
    WUSH_REQUIRE(aligned16(x) && aligned16(t) && aligned16(q), "fused_tq: x, t and q must be 16-byte aligned");
    const int64_t C = K / 32;
    WUSH_REQUIRE(C <= 65535 * 8, "fused_tq: K too large");
    cudaStream_t st = (cudaStream_t)stream;
    if (variant == WUSH_TQ_EXACT) {
        WUSH_REQUIRE(C <= 65535, "fused_tq(exact): K too large");
        dim3 grid((unsigned)((rows + TQE_ROWS - 1) / TQE_ROWS), (unsigned)C);
        fused_tq_exact_kernel<<<grid, TQE_ROWS, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)t,
                                                         (uint4*)q, (__nv_bfloat16*)s, (long long)rows, (int)C);
        return check_launch("fused_tq_exact");
    }
    return launch_fast<false>(x, t, rows, C, q, s, st);
}

// No counterpart in the reference: its FFN callers run SiLU, the product with `up` and the cast
// to bf16 as separate torch kernels between the two projections (an HBM round trip of h).
WUSH_API int wush_fused_silu_mul_transform_quant_int4(const void* gate_up, const void* t, int64_t rows, int64_t K,
                                                      uint8_t* q, void* s, void* stream)
{
    using namespace wush;
    if (int e = ensure_init()) return e;
    WUSH_REQUIRE(rows >= 0 && K > 0 && K % 32 == 0, "fused_silu_mul_tq: K must be a positive multiple of 32");
    if (rows == 0) return WUSH_OK;
    WUSH_REQUIRE(gate_up && t && q && s, "fused_silu_mul_tq: null pointer");
    WUSH_REQUIRE(aligned16(gate_up) && aligned16(t) && aligned16(q), "fused_silu_mul_tq: gate_up, t and q must be 16-byte aligned");
    const int64_t C = K / 32;
    WUSH_REQUIRE(C <= 65535 * 8, "fused_silu_mul_tq: K too large");
    return launch_fast<true>(gate_up, t, rows, C, q, s, (cudaStream_t)stream);
}
