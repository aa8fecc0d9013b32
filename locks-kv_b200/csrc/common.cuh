// Shared device/host helpers for the sm_100a kernels of liblocks_b200.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/locks_b200.h"

namespace locks {

// ---- host-side error reporting (thread-local message, C return codes) ------
void set_error(const char* fmt, ...);
int  fail(int code, const char* fmt, ...);
int  check_launch(const char* what);
int  sm_count();
bool pdl_enabled();
// A launcher that writes what the scorer reads BEFORE its pdl_wait() (summary
// records, page parameters) calls pdl_break(); the next scorer launch then
// takes an ordinary full stream dependency instead of a programmatic one.
void pdl_break();
bool pdl_take_break();

#define LOCKS_REQUIRE(cond, code, ...)                                        \
    do {                                                                      \
        if (!(cond)) return ::locks::fail((code), __VA_ARGS__);               \
    } while (0)

// ---- summary record layout (bytes, one record per (block, kv-head)) --------
// d = 128, page = 16, rank 8, int4 basis.  832 B = 13 x 64 B.
constexpr int REC_BYTES = LOCKS_REC_BYTES;
constexpr int RO_V4  = 0;      // 8 columns x 64 B (128 nibbles, low = even d)
constexpr int RO_MU8 = 512;    // 128 x int8
constexpr int RO_C8  = 640;    // 16 tokens x 8 x int8
constexpr int RO_CS  = 768;    // 16 x bf16
constexpr int RO_VS  = 800;    // 8 x bf16
constexpr int RO_MUS = 816;    // 1 x bf16 (+14 B pad)

// ---- order-preserving float <-> uint key ----------------------------------
__host__ __device__ __forceinline__ uint32_t f2key(float f) {
#ifdef __CUDA_ARCH__
    uint32_t u = __float_as_uint(f);
#else
    uint32_t u; memcpy(&u, &f, 4);
#endif
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key2f(uint32_t k) {
    uint32_t u = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
    return __uint_as_float(u);
}

#ifdef __CUDACC__
// ---- shared-memory address, mbarrier, bulk async copy ----------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                 ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2^22 polls and reports through *status
// (LOCKS_ST_WAIT_TIMEOUT) instead of spinning forever.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity,
                                          int* status) {
    for (int it = 0; it < (1 << 22); ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it > 64) __nanosleep(32);
    }
    if (status) atomicExch(status, LOCKS_ST_WAIT_TIMEOUT);
    return false;
}
// Orders earlier generic-proxy accesses of shared memory before later
// async-proxy (bulk copy) writes to the same bytes.
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// 1-D bulk copy global -> shared (TMA engine), completion on an mbarrier.
// dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src,
                                         uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Programmatic dependent launch.  A kernel launched with the programmatic
// stream-serialization attribute may start while its predecessor is still
// running; pdl_wait() blocks until the predecessor grid has completed and its
// writes are visible (a no-op without the attribute).  pdl_trigger() lets the
// successor's CTAs be scheduled once every CTA of this grid has called it.
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_trigger() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// L2 eviction policies for data that is read once per step (evict_first) or
// that later kernels re-read (evict_last)
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
// bulk copy with an L2 cache-policy hint
__device__ __forceinline__ void bulk_g2s_hint(void* dst, const void* src,
                                              uint32_t bytes, uint64_t* bar,
                                              uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes"
        ".L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)),
          "l"(policy)
        : "memory");
}

// ---- warp-level tensor-core fragments (M = 16 rows: the GQA group) ---------
// D(16x8,s32) += A(16x32,s8,row) * B(32x8,s8,col)
__device__ __forceinline__ void mma_s8s8_k32(int (&d)[4], uint32_t a0,
                                             uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D(16x8,s32) = A(16x32,s8,row) * B(32x8,s8,col)   (zero accumulator)
__device__ __forceinline__ void mma_s8s8_k32_z(int (&d)[4], uint32_t a0,
                                               uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_k16(float (&d)[4], uint32_t a0,
                                             uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4],
                                                  uint32_t addr) {
    asm volatile(
        "ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b16) {
    return __uint_as_float(b16 << 16);
}
#endif  // __CUDACC__


// How many clusters of `cluster` CTAs of `kernel` (blocks of `threads`, `smem`
// bytes of dynamic shared memory) the device can hold at once; 0 if the query
// fails.  A 16-CTA cluster needs 16 free SMs inside one GPC, so fewer of them
// fit than SMs / 16 suggests -- a launch with more clusters than fit runs in
// two rounds.
template <class Kernel>
inline int max_active_clusters(Kernel kernel, int cluster, int threads, int smem) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cluster, 1, 1);
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

}  // namespace locks
