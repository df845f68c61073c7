// sigma-clip G=32 INT4 quantisation (C-ABI wush_quant_int4).
//
// Contract: bit-exact with the reference's rtn_int4.quant_int4 (my_int4/rtn_int4.py:33-55)
// and its CUDA twin (csrc/quant_int4.cu:51-101): the two sums run over i = 0..31 in order
// with separately rounded multiply and add, IEEE sqrt and division, bf16 scale, codes from
// the bf16-rounded scale.  That order forces one thread per group; what is free is how the
// bytes move.  A CTA of 256 threads owns 256 consecutive groups (16 KB of input):
//   1. the CTA reads its 16 KB with fully coalesced 16-byte loads into shared memory,
//      16-byte chunk c of group t stored at chunk slot 4t + (c ^ ((t>>1)&3)) so that the
//      later per-thread reads (stride 64 B) are bank-conflict free;
//   2. thread t reads its own 64 B, runs the serial chain in registers;
//   3. codes leave as one 16-byte store per thread (512 B contiguous per warp), scales as
//      2-byte stores (64 B contiguous per warp).
// HBM traffic = 2 B/element in, 9/16 B/element out: the kernel is bandwidth bound once the
// IEEE divisions are hidden, so the grid is sized to whole waves of the SM count by the host.
#include "common.cuh"

namespace wush {

constexpr int QTHREADS = 256;

__global__ void __launch_bounds__(QTHREADS)
quant_int4_kernel(const uint4* __restrict__ x,      // n_groups * 4 chunks of 8 bf16
                  uint4* __restrict__ q_out,        // n_groups chunks of 16 bytes
                  __nv_bfloat16* __restrict__ s_out,
                  long long n_groups)
{
    __shared__ uint4 stage[QTHREADS * 4];
    const int t = threadIdx.x;
    const long long g0 = (long long)blockIdx.x * QTHREADS;
    const long long chunks_left = (n_groups - g0) * 4;            // valid 16-B chunks of this CTA

    // 1. coalesced load: chunk index ci = k*256 + t belongs to group ci>>2, chunk ci&3
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        int ci = k * QTHREADS + t;
        if (ci < chunks_left) {
            int grp = ci >> 2, c = ci & 3;
            stage[grp * 4 + (c ^ ((grp >> 1) & 3))] = ldg_nc_v4(x + g0 * 4 + ci);
        }
    }
    __syncthreads();
    const long long g = g0 + t;
    if (g >= n_groups) return;

    // 2. own group -> registers (bf16 -> fp32 is exact)
    float v[32];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint4 r = stage[t * 4 + (c ^ ((t >> 1) & 3))];
        v[c * 8 + 0] = bf16_lo(r.x); v[c * 8 + 1] = bf16_hi(r.x);
        v[c * 8 + 2] = bf16_lo(r.y); v[c * 8 + 3] = bf16_hi(r.y);
        v[c * 8 + 4] = bf16_lo(r.z); v[c * 8 + 5] = bf16_hi(r.z);
        v[c * 8 + 6] = bf16_lo(r.w); v[c * 8 + 7] = bf16_hi(r.w);
    }
    uint4 packed;
    uint32_t sbits;
    quant_group_exact(v, &packed, &sbits);

    // 3. vector stores
    q_out[g] = packed;
    s_out[g] = __ushort_as_bfloat16((unsigned short)sbits);
}

}  // namespace wush

WUSH_API int wush_quant_int4(const void* x, int64_t n_groups, uint8_t* q, void* s, void* stream)
{
    using namespace wush;
    if (int e = ensure_init()) return e;
    WUSH_REQUIRE(n_groups >= 0, "quant_int4: negative group count");
    if (n_groups == 0) return WUSH_OK;
    WUSH_REQUIRE(x && q && s, "quant_int4: null pointer");
    WUSH_REQUIRE(aligned16(x) && aligned16(q), "quant_int4: x and q must be 16-byte aligned");
    const long long blocks = (n_groups + QTHREADS - 1) / QTHREADS;
    WUSH_REQUIRE(blocks <= 0x7fffffffLL, "quant_int4: too many groups");
    quant_int4_kernel<<<(unsigned)blocks, QTHREADS, 0, (cudaStream_t)stream>>>(
        (const uint4*)x, (uint4*)q, (__nv_bfloat16*)s, (long long)n_groups);
    return check_launch("quant_int4");
}
