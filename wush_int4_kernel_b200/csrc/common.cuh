// Shared helpers for the sm_100a W4A4 kernels: error plumbing of the C ABI, bf16 bit
// helpers, the exact sigma-clip quantisation chain and nibble unpacking.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <string>

#include "../../include/wush_int4.h"

#define WUSH_API extern "C" __attribute__((visibility("default")))

namespace wush {

// ---- host side: error text of the calling thread ---------------------------------------
void set_error(const std::string& msg);
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);           // cudaGetLastError -> status
int ensure_init();                             // lazy wush_init()
int sm_count();                                // multiprocessors of the current device

#define WUSH_REQUIRE(cond, ...)                                         \
    do {                                                                \
        if (!(cond)) return ::wush::fail(WUSH_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- device side ------------------------------------------------------------------------
// 2.473650 / 7 in fp32: the Gaussian-MSE clip constant of the 15-level INT4 grid.
#define WUSH_C_CLIP 0.35337862372398376f

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b16) { return __uint_as_float(b16 << 16); }
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// fp32 -> bf16 bits, round to nearest even (finite inputs and inf; NaN never reaches here
// because the scale chain maps NaN variance to 1.0).
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}

// Scale of one group from its two sums, every operation rounded separately in fp32:
//   mean = s1/32; var = s2/32 - mean*mean; scale = var>=0 ? sqrt(var)*C + 1e-8 : 1.
// Returns the bf16 bit pattern; *scale_rt receives the bf16-rounded value as fp32.
__device__ __forceinline__ uint32_t sigma_clip_scale(float s1, float s2, float* scale_rt) {
    float mean = __fmul_rn(s1, 0.03125f);            // division by 32 is an exact exponent shift
    float var = __fsub_rn(__fmul_rn(s2, 0.03125f), __fmul_rn(mean, mean));
    float scale = 1.0f;
    if (var >= 0.f) scale = __fadd_rn(__fmul_rn(__fsqrt_rn(var), WUSH_C_CLIP), 1e-8f);
    uint32_t b = f32_to_bf16_bits(scale);
    *scale_rt = bf16_bits_to_f32(b);
    return b;
}

// Code of one value with IEEE division: clamp(rint(x / scale), -7, 7) as a 4-bit nibble.
__device__ __forceinline__ uint32_t code_exact(float x, float scale) {
    int q = __float2int_rn(__fdiv_rn(x, scale));     // saturating conversion, then clamp
    q = max(-7, min(7, q));
    return (uint32_t)q & 0xFu;
}

// The same code, bit for bit, without a division on the common path.  `r_lo` / `r_hi` bracket
// 1 / scale from below / above by a relative 2^-20 (the correctly rounded reciprocal times
// 1 -+ 2^-20), so for either sign of x the real quotient and fl(x / scale) lie strictly between
// x * r_lo and x * r_hi.  Adding 1.5 * 2^23 inside the FMA rounds each bound to the nearest-even
// integer; rounding is monotonic, so when both bounds round to the same integer, fl(x / scale)
// does too.  Otherwise (about 1.5e-5 of all elements, and every exact tie) the IEEE division
// decides.  Returns the bits of 1.5 * 2^23 + code.
__device__ __forceinline__ uint32_t code_bits_bracketed(float x, float scale, float r_lo, float r_hi) {
    const float magic = 12582912.f;
    float f = __fmaf_rn(x, r_lo, magic);
    const float g = __fmaf_rn(x, r_hi, magic);
    if (f != g) f = __fadd_rn(__fdiv_rn(x, scale), magic);
    f = fminf(fmaxf(f, magic - 7.f), magic + 7.f);
    return __float_as_uint(f);
}

// The whole bit-exact chain for one group held in registers.
__device__ __forceinline__ void quant_group_exact(const float (&v)[32], uint4* packed, uint32_t* scale_bits) {
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        s1 = __fadd_rn(s1, v[i]);
        s2 = __fadd_rn(s2, __fmul_rn(v[i], v[i]));
    }
    float scale;
    *scale_bits = sigma_clip_scale(s1, s2, &scale);
    const float r = __frcp_rn(scale);
    const float r_lo = __fmul_rn(r, 1.0f - 9.5367431640625e-7f), r_hi = __fmul_rn(r, 1.0f + 9.5367431640625e-7f);   // 2^-20
    uint32_t w[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        // bits = bits(magic) + code exactly, so sum_e bits_e * 16^e (mod 2^32) is the word of the offset
        // nibbles code + 8 plus a constant: one multiply-add per element, constant off, bit 3 flipped back
        uint32_t acc = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc = code_bits_bracketed(v[b * 8 + e], scale, r_lo, r_hi) * (1u << (4 * e)) + acc;
        w[b] = (acc - (0x4B400000u - 8u) * 0x11111111u) ^ 0x88888888u;
    }
    *packed = make_uint4(w[0], w[1], w[2], w[3]);
}

// Eight packed nibbles -> two words of four signed bytes, each byte = 16 * code:
//   even: codes 0,2,4,6   odd: codes 1,3,5,7.   The factor 16 is undone in the scale.
__device__ __forceinline__ void unpack_x16(uint32_t w, uint32_t& even, uint32_t& odd) {
    even = (w << 4) & 0xF0F0F0F0u;
    odd = w & 0xF0F0F0F0u;
}

__device__ __forceinline__ int dp4a_s8(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// 32 bytes per lane and store.  A lane that owns a run of 64 bytes and writes it as four 16-byte stores sends
// L2 half sectors (a warp's store instruction covers 16 of every 64 bytes); two 32-byte stores fill whole
// 32-byte sectors.  Measured on the fp16 widening pre-pass: 1.2 GB in 268 us with 16-byte stores, 189 us with these.
// `p` must be 32-byte aligned.
__device__ __forceinline__ void st_global_v8(void* p, const uint4& a, const uint4& b) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x),
                 "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}

__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// ---- programmatic dependent launch ------------------------------------------------------
// A producer calls pdl_launch_dependents() once its CTAs are resident; a consumer launched with
// launch_dependent() may then start, but sees the producer's writes only after pdl_wait(), which
// returns when the producer grid has finished and flushed.  Before the wait a consumer may only
// touch data in ways that cannot observe a stale value (here: L2 prefetches).  Both calls are
// no-ops when the neighbouring kernel does not take part.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Launch with the programmatic-stream-serialisation attribute (host side).
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                           cudaStream_t st, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace wush
