// tcgen05 tile GEMM (placeholder until the TMEM pipeline lands): reports "unsupported" so
// the dispatcher keeps every shape on the streaming tensor-core kernel.
#include "common.cuh"

namespace wush {
int tc_set_attributes() { return WUSH_OK; }
bool tc_supported(int64_t, int64_t, int64_t) { return false; }
size_t tc_workspace_bytes(int64_t, int64_t, int64_t) { return 0; }
int tc_dispatch(const uint8_t*, const void*, const uint8_t*, const void*, int64_t, int64_t, int64_t, void*, void*,
                size_t, cudaStream_t)
{
    return fail(WUSH_ERR_UNSUPPORTED, "tcgen05 tile GEMM not built");
}
}  // namespace wush
