// Library-level entry points and host-side error plumbing.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace locks {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail(LOCKS_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
    return LOCKS_OK;
}

// SM count of the current device, cached per device id (read-only after the
// first query; the only per-device state the library keeps).
int sm_count() {
    static int cache[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cache[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) !=
                cudaSuccess || n <= 0)
            n = 148;
        cache[dev] = n;
    }
    return cache[dev];
}

static int g_pdl = 1;
bool pdl_enabled() { return g_pdl != 0; }
static thread_local bool g_pdl_break = true;
void pdl_break() { g_pdl_break = true; }
bool pdl_take_break() { const bool b = g_pdl_break; g_pdl_break = false; return b; }

}  // namespace locks

extern "C" {

int locks_set_pdl(int enable) {
    const int old = locks::g_pdl;
    locks::g_pdl = enable ? 1 : 0;
    return old;
}

int locks_version(void) { return LOCKS_ABI_VERSION; }

const char* locks_last_error(void) { return locks::g_err; }

int locks_vtier_copy_run(void* dst, int64_t dst_pitch_bytes, const void* src,
                         int64_t src_pitch_bytes, int64_t block_bytes, int n_blocks,
                         locks_stream_t stream) {
    if (!dst || !src || block_bytes <= 0 || n_blocks < 0 ||
        dst_pitch_bytes < block_bytes || src_pitch_bytes < block_bytes)
        return locks::fail(LOCKS_ERR_ARG, "locks_vtier_copy_run: bad argument");
    if (n_blocks == 0) return LOCKS_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // one copy-engine transfer for the whole run: plain when both sides are
    // dense, a pitched 2-D copy (one row per block) otherwise
    const cudaError_t e =
        (dst_pitch_bytes == block_bytes && src_pitch_bytes == block_bytes)
            ? cudaMemcpyAsync(dst, src, (size_t)block_bytes * n_blocks,
                              cudaMemcpyHostToDevice, s)
            : cudaMemcpy2DAsync(dst, (size_t)dst_pitch_bytes, src,
                                (size_t)src_pitch_bytes, (size_t)block_bytes,
                                (size_t)n_blocks, cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess)
        return locks::fail(LOCKS_ERR_LAUNCH, "locks_vtier_copy_run: %s",
                           cudaGetErrorString(e));
    return LOCKS_OK;
}

int locks_record_bytes(int head_dim, int page) {
    if (head_dim != 128 || page != 16)
        return locks::fail(LOCKS_ERR_GEOMETRY,
                           "record layout is defined for head_dim 128 / page 16, "
                           "got %d / %d", head_dim, page);
    return LOCKS_REC_BYTES;
}

}  // extern "C"
