/*
 * wush_int4.h -- C ABI of the B200 (sm_100a) INT4 W4A4 linear-layer kernels.
 *
 * Library: wush_int4_kernel_b200/libwush_int4_b200.so (nvcc, no torch dependency).
 *
 * Every entry point below is what the reference project's Python binding for the
 * same operator would call; the reference item each one replaces is cited as
 * file:line of rib12316/WUSH_int4_kernel.  The torch-facing module `my_int4._C`
 * of this repository is a thin C++ layer over exactly these functions.
 *
 * Conventions
 *   - All data pointers are DEVICE pointers on the current CUDA device, row-major,
 *     contiguous.  bf16 / fp16 are passed as `void*` (2-byte elements).
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 *   - Calls are asynchronous, never synchronise the host and never allocate
 *     device memory: scratch is passed in by the caller.  They are therefore
 *     safe to capture in a CUDA Graph.  One-time function-attribute set-up
 *     happens inside wush_init(), which must run once per device OUTSIDE capture
 *     (the other entry points call it lazily on first use).
 *   - Return value: WUSH_OK or an error code; wush_last_error() gives the text of
 *     the calling thread's most recent failure.
 *
 * Data formats (identical to the reference, my_int4/rtn_int4.py:53-55):
 *   packed codes : byte i of a row = (q[2i] & 0xF) | ((q[2i+1] & 0xF) << 4),
 *                  two's-complement nibbles, even element in the low nibble
 *   scales       : bf16, one per 32 consecutive K elements
 *   activations  : xq (M, K/2) u8, xs (M, K/32) bf16
 *   weights      : wq (N, K/2) u8, ws (N, K/32) bf16
 *   transform    : t (K/32, 32, 32) bf16, T[g][j][i] multiplies input i into output j
 *   output       : y (M, N) fp16
 */
#ifndef WUSH_INT4_H_
#define WUSH_INT4_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WUSH_ABI_VERSION 1

typedef enum {
    WUSH_OK = 0,
    WUSH_ERR_INVALID_ARGUMENT = 1, /* bad size / null pointer / misaligned pointer   */
    WUSH_ERR_CUDA = 2,             /* a CUDA runtime call or launch failed           */
    WUSH_ERR_UNSUPPORTED = 3,      /* device is not sm_100, or shape outside limits  */
    WUSH_ERR_WORKSPACE = 4,        /* scratch buffer missing or too small            */
    WUSH_ERR_DEVICE_FLAG = 5       /* a kernel reported a bounded-wait timeout       */
} wush_status;

int wush_abi_version(void);
const char* wush_last_error(void);

/* One-time per-device set-up (kernel attributes, driver entry points).  Call once
 * per device before any stream capture.  Fails with WUSH_ERR_UNSUPPORTED when the
 * current device is not compute capability 10.x. */
int wush_init(void);

/* Kernels that wait on barriers give up after a bounded number of polls and record that
 * instead of hanging.  Kernels that are handed scratch by the caller (wush_w4a4_gemm with the TILE
 * variants, wush_w4a4_gemm_tensor_scale_ws) use word 0 of that scratch.  The kernels without caller
 * scratch use library-owned device words, which this call (synchronous: it copies a few bytes from
 * the device) returns in *flag and clears: bits 0-7 the role code left by a streaming (DECODE)
 * kernel, bits 8-15 the role code left by a kernel of wush_w4a4_gemm_static_scratch.
 * 0 means no such kernel gave up since the last call. */
int wush_device_flag(int* flag);

/* --- a1: sigma-clip G=32 INT4 quantisation --------------------------------------
 * Replaces quant_int4 (csrc/quant_int4.cu:109-134); bit-exact with
 * rtn_int4.quant_int4 (my_int4/rtn_int4.py:33-55).
 * x: n_groups*32 bf16;  q: n_groups*16 bytes;  s: n_groups bf16. */
int wush_quant_int4(const void* x, int64_t n_groups, uint8_t* q, void* s, void* stream);

/* --- a4..a7: fused WUSH block transform + quantisation ----------------------------
 * x'_j = sum_i x_i * T[g][j][i] in fp32, then the a1 chain on the un-rounded x'.
 * Replaces fused_transform_quant_int4 (csrc/fused_tq_int4.cu:87-118, variant EXACT),
 * _wmma (csrc/fused_tq_wmma.cu:131-162), _v3 (csrc/fused_tq_v3.cu:109-140) and
 * _smallm (csrc/fused_tq_smallm.cu:89-121).
 *   WUSH_TQ_EXACT : serial fp32 arithmetic in the reference's order; bit-exact with
 *                   the fp32 mirror (tests/test_sw2.py:12-24 of the reference).
 *   WUSH_TQ_FAST  : tensor-core transform + warp-shuffle statistics; differs from
 *                   EXACT only by rare +-1 code flips (accumulation order).
 * x: rows*K bf16;  t: (K/32)*1024 bf16;  q: rows*K/2;  s: rows*K/32 bf16. */
typedef enum { WUSH_TQ_EXACT = 0, WUSH_TQ_FAST = 1 } wush_tq_variant;
int wush_fused_transform_quant_int4(const void* x, const void* t, int64_t rows, int64_t K,
                                    int variant, uint8_t* q, void* s, void* stream);

/* The same op (FAST arithmetic) fed by the fp16 output of a fused gate+up projection:
 *   h = bf16( SiLU(gate) * up ) in fp32, gate = gate_up[:, :K], up = gate_up[:, K:],
 * then the transform + quantisation of h.  No counterpart in the reference, whose FFN callers
 * compute h with separate torch kernels between the two projections.
 * gate_up: rows*2K fp16;  t: (K/32)*1024 bf16;  q: rows*K/2;  s: rows*K/32 bf16. */
int wush_fused_silu_mul_transform_quant_int4(const void* gate_up, const void* t, int64_t rows,
                                             int64_t K, uint8_t* q, void* s, void* stream);

/* --- a8..a10: group-scaled W4A4 product ---------------------------------------------
 * Y[m][n] = sum_g sx[m][g] * sw[n][g] * P_g,  P_g = sum_{k in g} qa*qw exact in int32,
 * fp32 accumulation over groups, fp16 output.
 * Replaces w4a4_gemm_s4 (csrc/gemm_s4.cu:320-379), w4a4_gemm / _v1 / _v2
 * (csrc/gemm_int4.cu:89-130, csrc/gemm_wmma.cu:128-172, csrc/gemm_wmma2.cu:141-181),
 * w4a4_gemv and w4a4_gemv_multi (csrc/gemv_int4.cu:145-223).
 *   WUSH_GEMM_AUTO     : pick by shape (GEMV for M <= 3, and for M = 4 unless N > 32768;
 *                        DECODE up to 32 rows; for 32 < M <= 512 the cheaper of DECODE in
 *                        32-row blocks and TILE_F16 by a measured cost estimate in N, K and
 *                        M; TILE_F16 beyond; the exact-sum TILE variant only on request)
 *   WUSH_GEMM_GEMV     : CUDA-core streaming kernel (M <= 4)
 *   WUSH_GEMM_DECODE   : tensor-core streaming kernel, weights as the wide operand (any M)
 *   WUSH_GEMM_DECODE_TC: tcgen05 kind::i8 with the WEIGHTS as the 128-row operand and up to 32
 *                        activation rows as N, exact int32 sum per group; the weight stream is dealt
 *                        to the multiprocessors in equal runs of 8-group stages, so tiles may be
 *                        split and their fp32 pieces pass through the scratch (about 5 MB);
 *                        K % 256 == 0, M <= 32, scales 16-byte aligned.  Same results as DECODE to
 *                        fp32 summation order; measured slower than DECODE on this part, so AUTO
 *                        never picks it (kept as the exact tcgen05 reference of the decode path)
 *   WUSH_GEMM_GEMV_MMA : the weights streamed from global memory straight into mma.sync
 *                        fragments, every lane its own ring of asynchronous copies, no
 *                        barriers (1 <= M <= 16, K % 128 == 0, the widened activations --
 *                        about 17/16 * K bytes per row, rows rounded up to even -- within
 *                        about 185 KB of shared memory, scales 4-byte aligned)
 *   WUSH_GEMM_TILE     : tcgen05 kind::i8 tile GEMM, exact int32 sum per group (any M)
 *   WUSH_GEMM_TILE_F16 : scales folded into exactly-representable fp16 operands, tcgen05
 *                        kind::f16 with fp32 accumulation over the whole K (any M; the fast
 *                        route for prefill; scratch = an fp16 copy of the activations,
 *                        beyond 2048 rows one of the weights, and room for the fp32 pieces
 *                        of output tiles that are cut along K -- all tiles of a layer with
 *                        few of them, else those of the last, partly filled wave of tiles:
 *                        256 KB per piece, at most two per multiprocessor.  A scratch
 *                        that holds the copies but not those pieces is accepted; the
 *                        product then runs without the cut)
 * K % 32 == 0.  Ask wush_w4a4_gemm_workspace_bytes() with the SAME variant for the scratch
 * size; `workspace` may be NULL when it returns 0.  Word 0 of the scratch is an error word:
 * non-zero after the call completes means a bounded wait inside the kernel gave up.
 * Alignment: xq, wq, y and the scratch on 16 bytes; the scales on 2 bytes, and `ws` should be on
 * 16 bytes too: up to 2048 rows TILE_F16 reads the weight scales as 16-byte vectors while it widens
 * the weights inside the GEMM.  With a `ws` that is not, it takes the route with an fp16 copy of
 * the weights instead, which needs 2*N*K more bytes of scratch (rounded up to 256) than
 * wush_w4a4_gemm_workspace_bytes() reports; a scratch without that room is refused with
 * WUSH_ERR_WORKSPACE before anything is launched. */
typedef enum {
    WUSH_GEMM_AUTO = 0,
    WUSH_GEMM_GEMV = 1,
    WUSH_GEMM_DECODE = 2,
    WUSH_GEMM_TILE = 3,
    WUSH_GEMM_TILE_F16 = 4,
    WUSH_GEMM_DECODE_TC = 5,
    WUSH_GEMM_GEMV_MMA = 6
} wush_gemm_variant;
size_t wush_w4a4_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int variant);
/* The variant WUSH_GEMM_AUTO stands for on the current device for this shape (one of the other
 * four values): what wush_w4a4_gemm and wush_w4a4_gemm_workspace_bytes resolve it to. */
int wush_w4a4_gemm_pick_variant(int64_t M, int64_t N, int64_t K);
int wush_w4a4_gemm(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws,
                   int64_t M, int64_t N, int64_t K, void* y, int variant, void* workspace,
                   size_t workspace_bytes, void* stream);

/* --- product without caller scratch (no counterpart in the reference) -----------------------
 * For hosts that cannot hand this library any scratch and may not allocate device memory
 * themselves once they are running: servers that size a single arena at start-up and forbid
 * cudaMalloc afterwards, processes held to a fixed device-memory budget, control loops that
 * cannot tolerate the implicit synchronisation of an allocation.  Same arithmetic as
 * wush_w4a4_gemm(..., WUSH_GEMM_TILE_F16, ...): that call, given the scratch its size query asks
 * for, cuts the tiles of a partly filled wave into K ranges and adds them afterwards, which this
 * entry point has no room for -- same products, another order of the fp32 additions; both are
 * within the same 1e-3 of the fp64 result, and bit-identical where no tile is cut.  The scratch is an array of WUSH_STATIC_SCRATCH_BYTES that is part
 * of the library image: every GPU that loads the library keeps it until the process exits, so
 * the limit is deliberately modest.
 *   - Scratch needed: about 2*M*K bytes when the weights are widened inside the GEMM (M <= 2048,
 *     K % 256 == 0 and `ws` 16-byte aligned), about 2*(M+N)*K otherwise.  Shapes beyond the limit
 *     are refused with WUSH_ERR_WORKSPACE and a message naming both sizes; nothing is launched.
 *   - A bounded wait that gives up inside one of its kernels shows in bits 8-15 of
 *     wush_device_flag().
 *   - Neither this call nor anything it uses calls cudaMalloc / cudaFree or an allocating
 *     library routine.
 *   - The first call on a device resolves the array's device address (cudaGetSymbolAddress
 *     with that device current); make that first call before any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents; the library
 *     re-initialises what it needs, but two calls that overlap on the GPU (different streams,
 *     no dependency between them) race on it.  Serialise them. */
#define WUSH_STATIC_SCRATCH_BYTES (32u << 20)
size_t wush_w4a4_gemm_static_scratch_limit(void);
int wush_w4a4_gemm_static_scratch(const uint8_t* xq, const void* xs, const uint8_t* wq,
                                  const void* ws, int64_t M, int64_t N, int64_t K, void* y,
                                  void* stream);

/* --- a11: tensor-core self-tests ------------------------------------------------------
 * wush_i8_atom_selftest replaces s4_atom_selftest (csrc/gemm_s4.cu:50-82):
 * a (8,32) int8 in [-8,7], b (32,8) int8 -> c (8,8) int32 through one int8 MMA atom.
 * wush_group_partials exposes the exact per-group partial sums P[m][n][g] (int32)
 * produced by the same tensor-core code path the GEMM uses (test-only; M*N*K/32 ints). */
int wush_i8_atom_selftest(const int8_t* a, const int8_t* b, int32_t* c, void* stream);
/* One tcgen05.mma kind::i8 instruction tile: a (128,32) int8, b (n,32) int8 ->
 * d (128,n) int32 = a . b^T, n a multiple of 16 up to 256.  layout_mode 0 is the layout the
 * GEMM uses; 1 (n <= 64 only) swaps the two descriptor strides and exists for diagnosis.
 * *status (device int, zeroed by the caller) becomes 1 if the bounded wait gave up. */
int wush_i8_tile_selftest(const int8_t* a, const int8_t* b, int32_t* d, int n, int layout_mode,
                          int* status, void* stream);
int wush_group_partials(const uint8_t* xq, const uint8_t* wq, int64_t M, int64_t N, int64_t K,
                        int32_t* P, void* stream);

/* --- per-tensor route ("next" row 1) ------------------------------------------------------
 * q = clamp(rint(x * inv_scale), -7, 7); inv_scale from the host value, or from device
 * memory when inv_scale_dev != NULL.  Replaces quant_int4_tensor_scale{,_dev}
 * (csrc/fast_path.cu:42-63, 92-109).  n % 32 == 0. */
int wush_quant_int4_tensor_scale(const void* x, int64_t n, float inv_scale,
                                 const float* inv_scale_dev, uint8_t* q, void* stream);
/* y = fp16(alpha * sum_k qa*qw) with full-K int32 accumulation; alpha from the host
 * value or from device memory when alpha_dev != NULL.  Replaces w4a4_gemm_cutlass{,_dev}
 * (csrc/gemm_cutlass_int4.cu:132-188). */
int wush_w4a4_gemm_tensor_scale(const uint8_t* xq, const uint8_t* wq, int64_t M, int64_t N,
                                int64_t K, float alpha, const float* alpha_dev, void* y,
                                void* stream);
/* The same product with caller-provided scratch: for M >= 128 (and K % 128 == 0, N % 8 == 0)
 * both operands are widened to int8 in the scratch and contracted by tcgen05.mma kind::i8
 * tiles of 256 x 256 over the whole K (int32 accumulators in TMEM, alpha applied once).
 * Results are bit-identical to wush_w4a4_gemm_tensor_scale.  _workspace_bytes returns 0 when
 * the shape takes the scratch-free kernel anyway; the first word of the scratch is an error
 * flag of the kernel's bounded waits (0 = fine), as for wush_w4a4_gemm. */
size_t wush_w4a4_gemm_tensor_scale_workspace_bytes(int64_t M, int64_t N, int64_t K);
int wush_w4a4_gemm_tensor_scale_ws(const uint8_t* xq, const uint8_t* wq, int64_t M, int64_t N,
                                   int64_t K, float alpha, const float* alpha_dev, void* y,
                                   void* workspace, size_t workspace_bytes, void* stream);

/* --- multi-GPU: one-shot all-reduce of small fp16 partial products over NVLink peer memory ------
 * No counterpart in the reference (single GPU).  The row-parallel down projection of a
 * tensor-parallel FFN block ends in a sum over ranks; at decode sizes a library all-reduce costs
 * several times the sharded product.  One process per GPU of one node:
 *   wush_comm_create   allocates this rank's exchange buffer (2 x world slots of slot_bytes, flags, state).
 *                      The ONLY call of this library that allocates device memory; set-up time.
 *   wush_comm_export   64-byte CUDA IPC handle of that buffer, to be sent to every other rank;
 *   wush_comm_connect  maps a peer's buffer from its handle (once per peer);
 *   wush_comm_allreduce_f16  out[i] = fp16( sum over ranks r = 0..world-1 of fp32(partial_r[i]) ), n % 8 == 0,
 *                      2n <= slot_bytes; every rank must call it the same number of times with the
 *                      same n.  One kernel launch, no host synchronisation, capturable; a rank waits for
 *                      its peers inside the kernel for about a second at most, then records an error;
 *   wush_comm_allreduce_two_phase_f16   the same sum, same result bit for bit, as a reduce-scatter and an
 *                      all-gather inside one kernel (it takes TWO steps of the communicator): rank r sums
 *                      its 1/world share of all ranks' partials and stores the result into every rank's
 *                      buffer.  (world-1)/world of the data crosses NVLink per direction instead of
 *                      (world-1) times the data being read: the form for results of a megabyte and more
 *                      (prefill), where the library all-reduce of an fp32 copy is the alternative;
 *   wush_comm_gemv_allreduce   decode product (the operands of wush_w4a4_gemm; M <= 2 by the CUDA-core
 *                      GEMV, M <= 32 with K % 256 == 0 by the streaming kernel) AND the sum over ranks: the product kernel's epilogue stores its fp16 result into every rank's
 *                      buffer over NVLink and its last CTA publishes the step; the reduction then reads
 *                      local memory only.  WUSH_ERR_UNSUPPORTED for other shapes (use wush_w4a4_gemm +
 *                      wush_comm_allreduce_f16).  Same calling discipline as wush_comm_allreduce_f16, and
 *                      the two may be mixed step by step;
 *   wush_comm_allgather_f16    all-gather of the column blocks of a column-parallel product: rank r gives a
 *                      (rows, widths[r]) fp16 block, every rank receives the (rows, sum of widths) matrix with
 *                      the blocks side by side in rank order.  widths: host array of `world` entries, each a
 *                      positive multiple of 8, rows * widths[r] * 2 <= slot_bytes.  Same kernel skeleton,
 *                      calling discipline and bounded wait as wush_comm_allreduce_f16;
 *   wush_comm_gemv_allgather   decode product of this rank's weight shard (N = widths[rank]; shapes as for
 *                      wush_comm_gemv_allreduce) AND the all-gather: the product's epilogue stores its block
 *                      into its slot of every rank's buffer, the gather then copies from local memory only.
 *                      Sums, gathers and their pushed forms may be mixed step by step;
 *   wush_comm_connect_pointer  the same for a peer buffer of THIS process (wush_comm_base of another
 *                      communicator on a device with peer access): emulation of several ranks in one
 *                      process, and tests;
 *   wush_comm_set_poll_limit   bound of the in-kernel wait, in polls of about half a microsecond
 *                      (default 2^21, about a second);
 *   wush_comm_error    (synchronous) 1 if a wait ever ran out on this rank;
 *   wush_comm_destroy  unmaps and frees. */
int wush_comm_create(int rank, int world, size_t slot_bytes, void** comm);
int wush_comm_export(void* comm, void* handle64);
int wush_comm_connect(void* comm, int peer_rank, const void* handle64);
int wush_comm_connect_pointer(void* comm, int peer_rank, void* peer_base);
int wush_comm_base(void* comm, void** base);
int wush_comm_set_poll_limit(void* comm, unsigned int polls);
int wush_comm_allreduce_f16(void* comm, const void* partial, void* out, int64_t n, void* stream);
int wush_comm_allreduce_two_phase_f16(void* comm, const void* partial, void* out, int64_t n, void* stream);
int wush_comm_gemv_allreduce(void* comm, const uint8_t* xq, const void* xs, const uint8_t* wq,
                             const void* ws, int64_t M, int64_t N, int64_t K, void* out, void* stream);
int wush_comm_allgather_f16(void* comm, const void* local, void* out, int64_t rows, const int64_t* widths,
                            void* stream);
int wush_comm_gemv_allgather(void* comm, const uint8_t* xq, const void* xs, const uint8_t* wq,
                             const void* ws, int64_t M, int64_t K, const int64_t* widths, void* out,
                             void* stream);
int wush_comm_error(void* comm, int* error);
int wush_comm_destroy(void* comm);

/* ---- Check of the work split of the persistent tile kernels (host only, no GPU) ----
 * No counterpart in the reference.  The tile kernels cut the tiles of their last, partly filled
 * wave along K (wush_w4a4_gemm above); this walks the resulting units exactly as the kernels' CTAs
 * and the summing kernel do, on the host, for a grid of `workers` CTAs.
 *   tiles, k_steps   output tiles of the launch and pipeline stages per tile;
 *   gran             bounds of K ranges are multiples of this many stages;
 *   force_mode       -1: the split the cost estimate picks for (step_us, piece_us);
 *                    1: equal K ranges; 2: contiguous runs of stages per CTA (either only if the
 *                    shape admits it, else no cut);
 *   cover            [tiles * k_steps] ints out: how many units cover each stage of each tile;
 *   slots            capacity of the scratch area in 256 x 256 fp32 pieces;
 *   plan_out         [7] ints out: n_tiles, k_steps, full_tiles, mode, split, ctas, gran.
 * Returns WUSH_OK if every unit is in range, every piece a CTA writes has its own slot below
 * `slots` and the summing kernel adds exactly the written pieces of each cut tile, once each;
 * 101..107, one per broken property, otherwise. */
/* Activation tiles of 8 rows per CTA that the streaming decode kernel (WUSH_GEMM_DECODE) takes for M rows:
 * the smallest count that holds them up to 32 rows; beyond, the count minimising (blocks of rows) x
 * (measured time of a block), since every block streams the weights again.  Host only, no GPU. */
int wush_debug_stream_tiles(int64_t M);
int wush_debug_unit_cover(int64_t tiles, int k_steps, int gran, int workers, int force_mode,
                          double step_us, double piece_us, int* cover, int slots, int* plan_out);

#ifdef __cplusplus
}
#endif
#endif /* WUSH_INT4_H_ */
