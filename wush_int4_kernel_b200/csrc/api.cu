// C-ABI glue: error text, one-time device set-up and the shape dispatcher of wush_w4a4_gemm.
#include <cstdarg>
#include <mutex>

#include "common.cuh"

namespace wush {

static thread_local std::string g_last_error;

void set_error(const std::string& msg) { g_last_error = msg; }

int fail(int code, const char* fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

int check_launch(const char* what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e));
    return WUSH_OK;
}

// per-device state, set up once (never during stream capture: call wush_init() first)
constexpr int MAX_DEVICES = 64;
static std::mutex g_mutex;
static int g_ready[MAX_DEVICES];        // 0 = not yet, 1 = ok, <0 = -(status)
static int g_sms[MAX_DEVICES];

int gemv_set_attributes();
int gemv_mma_set_attributes();
int mma_set_attributes();
int tc_set_attributes();
int stream_set_attributes();
int f16_set_attributes();
int decode_tc_set_attributes();

static int init_device(int dev)
{
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "wush_init: cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    if (prop.major != 10)
        return fail(WUSH_ERR_UNSUPPORTED, "wush_init: device %d is sm_%d%d; this library is built for sm_100a only",
                    dev, prop.major, prop.minor);
    g_sms[dev] = prop.multiProcessorCount;
    if (int s = gemv_set_attributes()) return s;
    if (int s = gemv_mma_set_attributes()) return s;
    if (int s = mma_set_attributes()) return s;
    if (int s = tc_set_attributes()) return s;
    if (int s = stream_set_attributes()) return s;
    if (int s = f16_set_attributes()) return s;
    if (int s = decode_tc_set_attributes()) return s;
    return WUSH_OK;
}

int ensure_init()
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(WUSH_ERR_CUDA, "cudaGetDevice: %s (is a CUDA device present?)", cudaGetErrorString(e));
    if (dev < 0 || dev >= MAX_DEVICES) return fail(WUSH_ERR_UNSUPPORTED, "device index %d out of range", dev);
    if (g_ready[dev] == 1) return WUSH_OK;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_ready[dev] == 0) {
        int s = init_device(dev);
        g_ready[dev] = (s == WUSH_OK) ? 1 : -s;
        return s;
    }
    if (g_ready[dev] == 1) return WUSH_OK;
    return fail(-g_ready[dev], "wush_init failed earlier on device %d", dev);
}

int sm_count()
{
    int dev = 0;
    cudaGetDevice(&dev);
    return (dev >= 0 && dev < MAX_DEVICES && g_sms[dev] > 0) ? g_sms[dev] : 148;
}

size_t gemv_smem_bytes(int M, int64_t K);
int gemv_dispatch(const uint8_t*, const void*, const uint8_t*, const void*, int64_t, int64_t, int64_t, void*, cudaStream_t);
int mma_dispatch(const uint8_t*, const void*, const uint8_t*, const void*, int64_t, int64_t, int64_t, void*, cudaStream_t);
int stream_tiles_for(int64_t M, double* relative_cost);
bool gemv_mma_supported(int64_t M, int64_t N, int64_t K, const void* xs, const void* ws);
int gemv_mma_dispatch(const uint8_t*, const void*, const uint8_t*, const void*, int64_t, int64_t, int64_t, void*, cudaStream_t);
bool tc_supported(int64_t M, int64_t N, int64_t K);
size_t tc_workspace_bytes(int64_t M, int64_t N, int64_t K);
int tc_dispatch(const uint8_t*, const void*, const uint8_t*, const void*, int64_t, int64_t, int64_t, void*, void*,
                size_t, cudaStream_t);
bool decode_tc_supported(int64_t M, int64_t N, int64_t K);
size_t decode_tc_workspace_bytes(int64_t M, int64_t N, int64_t K);
int decode_tc_dispatch(const uint8_t*, const void*, const uint8_t*, const void*, int64_t, int64_t, int64_t, void*, void*,
                       size_t, cudaStream_t);
bool f16_supported(int64_t M, int64_t N, int64_t K);
size_t f16_workspace_bytes(int64_t M, int64_t N, int64_t K);
int f16_fused_split(int64_t M, int64_t N, int64_t K);
int f16_dispatch(const uint8_t*, const void*, const uint8_t*, const void*, int64_t, int64_t, int64_t, void*, void*,
                 size_t, cudaStream_t, int* sticky_err);

// Which kernel a shape runs on.  GEMV: CUDA cores, M <= 4 (the exact per-group scaling costs
// three instructions per (m, n, group), so beyond a few rows the dot products must move to
// the tensor cores).  DECODE: weights-as-wide-operand tensor-core streaming, M <= 32.
// TILE: tcgen05 kind::i8 tile GEMM (exact integer group sums); chosen by AUTO only where the
// streaming kernel does not take K (K % 256 != 0) at 32 < M < 128.
// TILE_F16: scales folded into fp16 operands, tcgen05 kind::f16, for M >= 128 (several times
// faster: no per-group epilogue; needs scratch for the fp16 activations and, beyond 2048 rows,
// for an fp16 copy of the weights).
static int resolve_variant(int variant, int64_t M, int64_t N, int64_t K)
{
    if (variant != WUSH_GEMM_AUTO) return variant;
    const bool gemv_ok = gemv_smem_bytes((int)(M < 4 ? M : 4), K) <= 200 * 1024;
    // Up to three rows the CUDA-core GEMV is ahead everywhere (K = 8192, N = 57344: 38 / 39 / 48 us at M = 1 / 2 / 3
    // against 54 us of the streaming kernel); at four rows it is on all but the widest layers (that one: 56 against
    // 54 us; K = 4096, N = 24576: 16.7 against 19.5 us).
    if (M <= 4 && gemv_ok && (M <= 3 || K % 256 != 0 || N <= 32768)) return WUSH_GEMM_GEMV;
    // Up to 32 rows: the streaming kernel.  The tcgen05 kernel with swapped operands (DECODE_TC) computes the same
    // product but is slower on every shape measured so far (K = 8192, N = 57344: 93 / 96 / 139 us against 55 / 77 /
    // 119 us at M = 8 / 16 / 32), so AUTO never picks it.
    if (M <= 32) return WUSH_GEMM_DECODE;
    const bool f16_ok = f16_supported(M, N, K), stream_ok = K % 256 == 0;
    if (f16_ok && stream_ok && M <= 512) {
        // Both routes take the shape: the streaming kernel runs once per block of 32 rows and scales with
        // the layer, the fp16 route has a floor of one tile per multiprocessor over the whole K.  Times in
        // microseconds from measurements on the 70B gate+up layer (4.7e8 weights) and on narrow layers.
        const double elems = (double)N * (double)K, unit = elems / 4.7e8;
        const auto block_us = [&](double wide) { const double t = 1.2 * wide * unit; return t > 6.0 ? t : 6.0; };
        double blocks32 = 0.0;                                        // the streaming kernel's blocks of rows, in units of a 32-row block
        stream_tiles_for(M, &blocks32);
        const double t_stream = 10.0 + blocks32 * block_us(121.0);
        const int split = f16_fused_split(M, N, K);                   // K ranges: the 256-row kernel, also for M <= 128
        const bool wide = M > 128 || split > 1;
        const int64_t units = (wide ? (M + 255) / 256 : 1) * ((N + 255) / 256) * split;
        const double waves = (double)((units + sm_count() - 1) / sm_count());
        const double t_f16 = waves * (double)K / 64.0 / split * (wide ? 1.05 : 0.8) + 30.0 + (split > 1 ? 8.0 : 0.0);
        return t_stream <= t_f16 ? WUSH_GEMM_DECODE : WUSH_GEMM_TILE_F16;
    }
    if (M >= 128 && f16_ok) return WUSH_GEMM_TILE_F16;
    // 32 < M < 128 otherwise: the streaming kernel in blocks of 32 rows; the exact tile kernel where the
    // streaming kernel does not take K
    if (stream_ok) return WUSH_GEMM_DECODE;
    return tc_supported(M, N, K) ? WUSH_GEMM_TILE : WUSH_GEMM_DECODE;
}

}  // namespace wush

WUSH_API int wush_abi_version(void) { return WUSH_ABI_VERSION; }

WUSH_API const char* wush_last_error(void) { return wush::g_last_error.c_str(); }

WUSH_API int wush_init(void) { return wush::ensure_init(); }

WUSH_API size_t wush_w4a4_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int variant)
{
    using namespace wush;
    if (M <= 0 || N <= 0 || K <= 0 || K % 32) return 0;
    int v = resolve_variant(variant, M, N, K);
    if (v == WUSH_GEMM_DECODE_TC) return decode_tc_supported(M, N, K) ? decode_tc_workspace_bytes(M, N, K) : 0;
    if (v == WUSH_GEMM_TILE_F16 && f16_supported(M, N, K)) return f16_workspace_bytes(M, N, K);
    if ((v == WUSH_GEMM_TILE || v == WUSH_GEMM_TILE_F16) && tc_supported(M, N, K)) return tc_workspace_bytes(M, N, K);
    return 0;
}

WUSH_API int wush_w4a4_gemm_pick_variant(int64_t M, int64_t N, int64_t K)
{
    return wush::resolve_variant(WUSH_GEMM_AUTO, M, N, K);
}

WUSH_API int wush_w4a4_gemm(const uint8_t* xq, const void* xs, const uint8_t* wq, const void* ws, int64_t M,
                            int64_t N, int64_t K, void* y, int variant, void* workspace, size_t workspace_bytes,
                            void* stream)
{
    using namespace wush;
    if (int e = ensure_init()) return e;
    WUSH_REQUIRE(M >= 0 && N >= 0 && K > 0 && K % 32 == 0, "w4a4_gemm: K must be a positive multiple of 32");
    WUSH_REQUIRE(variant >= WUSH_GEMM_AUTO && variant <= WUSH_GEMM_GEMV_MMA, "w4a4_gemm: unknown variant %d", variant);
    if (M == 0 || N == 0) return WUSH_OK;
    WUSH_REQUIRE(xq && xs && wq && ws && y, "w4a4_gemm: null pointer");
    WUSH_REQUIRE(aligned16(xq) && aligned16(wq), "w4a4_gemm: packed codes must be 16-byte aligned");
    WUSH_REQUIRE(N < (1LL << 31) && M < (1LL << 31) && K < (1LL << 31), "w4a4_gemm: dimension too large");
    cudaStream_t st = (cudaStream_t)stream;
    const int v = resolve_variant(variant, M, N, K);
    switch (v) {
        case WUSH_GEMM_GEMV:
            WUSH_REQUIRE(M <= 4, "w4a4_gemm: the GEMV variant takes at most 4 rows (got %lld)", (long long)M);
            if (gemv_smem_bytes((int)M, K) > 200 * 1024)
                return fail(WUSH_ERR_UNSUPPORTED, "w4a4_gemm: K=%lld too large for the GEMV variant", (long long)K);
            return gemv_dispatch(xq, xs, wq, ws, M, N, K, y, st);
        case WUSH_GEMM_DECODE:
            return mma_dispatch(xq, xs, wq, ws, M, N, K, y, st);
        case WUSH_GEMM_GEMV_MMA:
            if (!gemv_mma_supported(M, N, K, xs, ws))
                return fail(WUSH_ERR_UNSUPPORTED, "w4a4_gemm: the GEMV_MMA variant takes 1..16 rows, K a multiple of 128 with the "
                                                  "activations in shared memory, 4-byte aligned scales (M=%lld K=%lld)",
                            (long long)M, (long long)K);
            return gemv_mma_dispatch(xq, xs, wq, ws, M, N, K, y, st);
        case WUSH_GEMM_DECODE_TC:
            return decode_tc_dispatch(xq, xs, wq, ws, M, N, K, y, workspace, workspace_bytes, st);
        case WUSH_GEMM_TILE_F16:
            if (f16_supported(M, N, K)) {
                if (!workspace) return fail(WUSH_ERR_WORKSPACE, "w4a4_gemm(f16): workspace of %zu bytes needed, none given",
                                            f16_workspace_bytes(M, N, K));
                return f16_dispatch(xq, xs, wq, ws, M, N, K, y, workspace, workspace_bytes, st, nullptr);
            }
            // fall through: shapes the fp16 route does not take run on the exact tile kernel
        case WUSH_GEMM_TILE:
            if (!tc_supported(M, N, K)) return mma_dispatch(xq, xs, wq, ws, M, N, K, y, st);
            if (workspace_bytes < tc_workspace_bytes(M, N, K) || (tc_workspace_bytes(M, N, K) && !workspace))
                return fail(WUSH_ERR_WORKSPACE, "w4a4_gemm: workspace of %zu bytes needed, %zu given",
                            tc_workspace_bytes(M, N, K), workspace_bytes);
            return tc_dispatch(xq, xs, wq, ws, M, N, K, y, workspace, workspace_bytes, st);
    }
    return fail(WUSH_ERR_INVALID_ARGUMENT, "w4a4_gemm: unknown variant %d", v);
}

// Host-side view of a dispatch rule, for the CPU test suite: activation tiles of 8 rows per CTA the streaming kernel
// takes for M rows.
WUSH_API int wush_debug_stream_tiles(int64_t M) { return M > 0 ? wush::stream_tiles_for(M, nullptr) : 0; }
