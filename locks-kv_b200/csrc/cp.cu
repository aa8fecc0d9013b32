// Context-parallel glue of the page selection: one long sequence whose pages are
// split over several GPUs.  Every rank runs the scorer and the selector on its
// own page range with the GLOBAL budget b, which leaves in its page table the
// sink / recent pages it holds plus its b best selectable pages.  The two
// kernels here sit on either side of the all-gather of those candidates:
//
//   cp_pack    page table + combined scores  ->  (score, global page) candidate
//              rows of this rank (forced pages and empty slots travel as -inf);
//   cp_select  the gathered candidates of all ranks  ->  the global exact-b cut
//              (score descending, page ascending: the single-GPU tie rule) and
//              this rank's final page table: its forced pages and those of its
//              candidates that made the cut, in ascending page order.
//
// A candidate's place in the global order is counted directly (how many
// candidates beat it): world * (b + forced) entries per kv-head are a few
// thousand at most, and the count needs no sort, no scratch and one launch.
#include <cstring>

#include "common.cuh"
#include "cp_link.cuh"

namespace locks {
namespace {

constexpr int CPT = 256;

__global__ void cp_pack_kernel(const int32_t* __restrict__ page_table,
                               const float* __restrict__ score,
                               float* __restrict__ cand_score,
                               float* __restrict__ cand_page, int max_pages,
                               int cap, int sink_loc, int nsh_loc, int p0) {
    const int kh = blockIdx.y;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= cap) return;
    const int e = page_table[(int64_t)kh * max_pages + j];
    const bool sel = e >= sink_loc && e < nsh_loc;       // e < 0: empty slot
    cand_score[(int64_t)kh * cap + j] =
        sel ? score[(int64_t)kh * max_pages + e] : -INFINITY;
    cand_page[(int64_t)kh * cap + j] = sel ? (float)(e + p0) : 16777216.f;
}

// cand: per rank (rows cand_stride floats apart) (2, n_kv, cap) floats --
// scores, then pages.  One CTA per kv-head; warp w decides entries w,
// w + nwarps, ... of this rank's table.
__global__ void __launch_bounds__(1024)
cp_select_kernel(const float* __restrict__ cand, int32_t* __restrict__ page_table,
                 int32_t* __restrict__ page_cnt, int64_t rank_stride, int world,
                 int rank, int n_kv, int cap, int max_pages, int b, int sink_loc,
                 int nsh_loc) {
    extern __shared__ int keep_sh[];       // cap flags | world * cap keys | pages
    __shared__ int wsum[32];
    const int kh = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nw = blockDim.x >> 5;
    int32_t* tab = page_table + (int64_t)kh * max_pages;
    uint32_t* ckey = reinterpret_cast<uint32_t*>(keep_sh + cap);
    float* cpage = reinterpret_cast<float*>(ckey + world * cap);
    // all candidates of this kv-head into shared memory (coalesced, all in
    // flight): the counting loop below would otherwise pay an L2 round trip per
    // candidate.  Key 0 = "no candidate" (a real score's key is never 0).
    for (int i = tid; i < world * cap; i += blockDim.x) {
        const int r = i / cap, c = i - r * cap;
        const float* s = cand + r * rank_stride + (int64_t)kh * cap;
        const float sc = s[c];
        ckey[i] = (sc > -INFINITY) ? max(f2key(sc), 1u) : 0u;
        cpage[i] = s[(int64_t)n_kv * cap + c];
    }
    __syncthreads();

    for (int j = warp; j < cap; j += nw) {
        const int e = tab[j];
        const bool live = e >= 0;
        const bool sel = live && e >= sink_loc && e < nsh_loc;
        int keep = live ? 1 : 0;
        if (sel) {                                        // warp-uniform
            const uint32_t key = ckey[rank * cap + j];
            const float pg = cpage[rank * cap + j];
            int beat = 0;
            for (int c = lane; c < world * cap; c += 32) {
                const uint32_t k2 = ckey[c];
                beat += (k2 > key || (k2 == key && k2 != 0u && cpage[c] < pg)) ? 1 : 0;
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1)
                beat += __shfl_xor_sync(0xffffffffu, beat, o);
            keep = (beat < b && key != 0u) ? 1 : 0;
        }
        if (lane == 0) keep_sh[j] = keep;
    }
    __syncthreads();
    // ordered compaction, 1024 entries per round
    int base = 0;
    for (int j0 = 0; j0 < cap; j0 += blockDim.x) {
        const int j = j0 + tid;
        const int k = (j < cap) ? keep_sh[j] : 0;
        const int e = (j < cap) ? tab[j] : -1;
        int inc = k;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) wsum[warp] = inc;
        __syncthreads();                                  // all reads of tab[j0..] done
        int wbase = 0, total = 0;
        for (int w = 0; w < nw; ++w) {
            const int v = wsum[w];
            if (w < warp) wbase += v;
            total += v;
        }
        if (k) tab[base + wbase + inc - 1] = e;           // slot <= j: never ahead of a reader
        base += total;
        __syncthreads();
    }
    for (int j = base + tid; j < cap; j += blockDim.x) tab[j] = -1;
    if (tid == 0) page_cnt[kh] = base;
}

}  // namespace
}  // namespace locks

using namespace locks;

extern "C" int locks_cp_pack(const int32_t* page_table, const float* score,
                             float* cand_rows, int n_kv, int max_pages, int cap,
                             int sink_loc, int nsh_loc, int p0,
                             locks_stream_t stream) {
    LOCKS_REQUIRE(page_table && score && cand_rows, LOCKS_ERR_ARG,
                  "locks_cp_pack: null pointer argument");
    LOCKS_REQUIRE(n_kv >= 1 && n_kv <= 65535 && cap >= 1 && cap <= max_pages,
                  LOCKS_ERR_ARG, "locks_cp_pack: bad size argument");
    cp_pack_kernel<<<dim3((cap + CPT - 1) / CPT, n_kv), CPT, 0,
                     static_cast<cudaStream_t>(stream)>>>(
        page_table, score, cand_rows, cand_rows + (int64_t)n_kv * cap, max_pages,
        cap, sink_loc, nsh_loc, p0);
    return check_launch("locks_cp_pack");
}

extern "C" int locks_cp_select(const float* cand, int64_t cand_stride,
                               int32_t* page_table, int32_t* page_cnt, int world,
                               int rank, int n_kv, int cap, int max_pages, int b,
                               int sink_loc, int nsh_loc, locks_stream_t stream) {
    LOCKS_REQUIRE(cand && page_table && page_cnt, LOCKS_ERR_ARG,
                  "locks_cp_select: null pointer argument");
    LOCKS_REQUIRE(world >= 1 && rank >= 0 && rank < world && n_kv >= 1 &&
                      n_kv <= 65535 && cap >= 1 && cap <= max_pages && b >= 0 &&
                      cand_stride >= (int64_t)2 * n_kv * cap,
                  LOCKS_ERR_ARG, "locks_cp_select: bad size argument");
    const size_t smem = ((size_t)cap + 2 * (size_t)world * cap) * sizeof(int);
    LOCKS_REQUIRE(smem <= 200 * 1024, LOCKS_ERR_SIZE,
                  "locks_cp_select: %d entries per rank x %d ranks beyond the "
                  "shared-memory staging area", cap, world);
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaFuncSetAttribute(cp_select_kernel,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr_done[dev] = true;
    }
    cp_select_kernel<<<n_kv, 1024, smem,
                       static_cast<cudaStream_t>(stream)>>>(
        cand, page_table, page_cnt, cand_stride, world, rank, n_kv, cap,
        max_pages, b, sink_loc, nsh_loc);
    return check_launch("locks_cp_select");
}

// ---------------------------------------------------------------------------
// Peer exchange: an all-gather (or all-reduce(max) of uint32 keys) of a small
// payload over NVLink peer memory, fused into ONE kernel per rank -- the three
// per-layer exchanges of the context-parallel path move 0.1 - 20 KB each, so a
// library collective's launch and protocol latency is the whole cost.
//
// Every rank owns an identical region (cudaMalloc, opened by the peers through
// CUDA IPC):   [0]   epoch counter of this rank (local use)
//              [64]  flags[2][8]: flags[e & 1][src] = e once src's payload of
//                    epoch e has landed here
//              [256] data[2][8][slot_bytes]
// The kernel bumps its epoch, stores its payload into slot [e & 1][rank] of
// every peer (plain peer stores), fences, raises the flags, then waits -- with a
// time limit -- until all ranks' flags of this epoch are set in its OWN region,
// and copies (or max-reduces) the gathered slots into a fixed local buffer that
// the next kernel reads.  Two data halves suffice: a rank can enter epoch e + 2
// only after every peer has pushed epoch e + 1, i.e. finished reading epoch e.
// Ranks run on different GPUs; a rank never waits for a kernel of its own GPU.
// ---------------------------------------------------------------------------
namespace locks {
namespace {

constexpr int XMAX = 8;                  // ranks
constexpr int X_FLAGS = 64, X_DATA = 256;
constexpr unsigned long long X_WAIT_NS = 2000000000ull;   // 2 s

struct XchgPeers { uint8_t* base[XMAX]; };

__device__ __forceinline__ unsigned long long gtime_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// mode 0: out = (world, nbytes) gathered payloads; mode 1: out = element-wise
// unsigned maximum of the ranks' uint32 payloads (nbytes / 4 words); modes 2, 3:
// the same two through 8-byte {word, epoch} packets (small payloads; a region
// is used with ONE of the two transports for its whole life)
__global__ void __launch_bounds__(1024)
cp_exchange_kernel(XchgPeers peers, int world, int rank, const uint4* payload,
                   int nbytes, int slot_bytes, uint8_t* out, int mode,
                   int* status) {
    __shared__ uint32_t s_epoch;
    __shared__ int s_timeout;
    const int tid = threadIdx.x;
    uint8_t* me = peers.base[rank];
    if (tid == 0) {
        uint32_t* ctr = reinterpret_cast<uint32_t*>(me);
        s_epoch = *ctr + 1u;
        *ctr = s_epoch;
        s_timeout = 0;
    }
    __syncthreads();
    const uint32_t e = s_epoch;
    const int par = (int)(e & 1u);
    const int n16 = nbytes >> 4;
    const int64_t slot_off = X_DATA + ((int64_t)par * XMAX + rank) * slot_bytes;
    if (mode & 2) {
        // ---- flag-in-packet transport for small payloads: every 32-bit word
        // travels as an 8-byte packet {word, epoch} (one store, atomic), the
        // receiver polls the packet itself: no fence, no separate flag ----------
        const int nwords = nbytes >> 2;
        const uint32_t* pw = reinterpret_cast<const uint32_t*>(payload);
        for (int r = 0; r < world; ++r) {
            uint2* dst = reinterpret_cast<uint2*>(peers.base[r] + slot_off);
            for (int i = tid; i < nwords; i += blockDim.x)
                asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};"
                             ::"l"(dst + i), "r"(pw[i]), "r"(e) : "memory");
        }
        const uint8_t* half = me + X_DATA + (int64_t)par * XMAX * slot_bytes;
        const unsigned long long t0 = gtime_ns();
        bool late = false;
        for (int i = tid; i < nwords; i += blockDim.x) {
            uint32_t m = 0u;
            for (int r = 0; r < world; ++r) {
                const uint2* src =
                    reinterpret_cast<const uint2*>(half + (int64_t)r * slot_bytes) + i;
                uint32_t x, y;
                for (;;) {
                    asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];"
                                 : "=r"(x), "=r"(y) : "l"(src) : "memory");
                    if (y == e) break;
                    if (gtime_ns() - t0 > X_WAIT_NS) { late = true; break; }
                }
                if (late) break;
                if (mode == 2)
                    reinterpret_cast<uint32_t*>(out)[(int64_t)r * nwords + i] = x;
                else
                    m = max(m, x);
            }
            if (late) break;
            if (mode == 3) reinterpret_cast<uint32_t*>(out)[i] = m;
        }
        if (late && status) atomicExch(status, LOCKS_ST_WAIT_TIMEOUT);
        return;
    }
    for (int r = 0; r < world; ++r) {
        uint4* dst = reinterpret_cast<uint4*>(peers.base[r] + slot_off);
        for (int i = tid; i < n16; i += blockDim.x) dst[i] = payload[i];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < world)
        st_release_sys(reinterpret_cast<uint32_t*>(peers.base[tid] + X_FLAGS) +
                           par * XMAX + rank, e);
    if (tid < world) {
        const uint32_t* f =
            reinterpret_cast<const uint32_t*>(me + X_FLAGS) + par * XMAX + tid;
        const unsigned long long t0 = gtime_ns();
        while (ld_acquire_sys(f) != e) {
            if (gtime_ns() - t0 > X_WAIT_NS) { s_timeout = 1; break; }
            __nanosleep(64);
        }
    }
    __syncthreads();
    if (s_timeout) {
        if (tid == 0 && status) atomicExch(status, LOCKS_ST_WAIT_TIMEOUT);
        return;                          // nothing of this context is left waiting
    }
    const uint8_t* slots = me + X_DATA + (int64_t)par * XMAX * slot_bytes;
    if (mode == 0) {
        for (int r = 0; r < world; ++r) {
            const uint4* src =
                reinterpret_cast<const uint4*>(slots + (int64_t)r * slot_bytes);
            uint4* dst = reinterpret_cast<uint4*>(out + (int64_t)r * nbytes);
            for (int i = tid; i < n16; i += blockDim.x) dst[i] = src[i];
        }
    } else {
        const int nw = nbytes >> 2;
        for (int i = tid; i < nw; i += blockDim.x) {
            uint32_t m = 0u;
            for (int r = 0; r < world; ++r)
                m = max(m, reinterpret_cast<const uint32_t*>(
                               slots + (int64_t)r * slot_bytes)[i]);
            reinterpret_cast<uint32_t*>(out)[i] = m;
        }
    }
}

}  // namespace
}  // namespace locks

extern "C" int locks_cp_region_bytes(int slot_bytes, int64_t* out) {
    LOCKS_REQUIRE(out && slot_bytes > 0 && (slot_bytes & 15) == 0, LOCKS_ERR_ARG,
                  "locks_cp_region_bytes: slot size must be a positive multiple "
                  "of 16");
    *out = X_DATA + (int64_t)2 * XMAX * slot_bytes;
    return LOCKS_OK;
}

extern "C" int locks_cp_alloc(int64_t bytes, void** out) {
    LOCKS_REQUIRE(out && bytes > 0, LOCKS_ERR_ARG, "locks_cp_alloc: bad argument");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, (size_t)bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, (size_t)bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess)
        return fail(LOCKS_ERR_LAUNCH, "locks_cp_alloc: %s", cudaGetErrorString(e));
    *out = p;
    return LOCKS_OK;
}

extern "C" int locks_cp_free(void* p) {
    if (p && cudaFree(p) != cudaSuccess)
        return fail(LOCKS_ERR_LAUNCH, "locks_cp_free: cudaFree failed");
    return LOCKS_OK;
}

extern "C" int locks_cp_ipc_export(void* p, unsigned char* handle64) {
    LOCKS_REQUIRE(p && handle64, LOCKS_ERR_ARG, "locks_cp_ipc_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess)
        return fail(LOCKS_ERR_LAUNCH, "locks_cp_ipc_export: %s",
                    cudaGetErrorString(e));
    memcpy(handle64, &h, 64);
    return LOCKS_OK;
}

extern "C" int locks_cp_ipc_open(const unsigned char* handle64, void** out) {
    LOCKS_REQUIRE(handle64 && out, LOCKS_ERR_ARG, "locks_cp_ipc_open: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess)
        return fail(LOCKS_ERR_LAUNCH, "locks_cp_ipc_open: %s", cudaGetErrorString(e));
    *out = p;
    return LOCKS_OK;
}

extern "C" int locks_cp_ipc_close(void* p) {
    if (p && cudaIpcCloseMemHandle(p) != cudaSuccess)
        return fail(LOCKS_ERR_LAUNCH, "locks_cp_ipc_close: failed");
    return LOCKS_OK;
}

extern "C" int locks_cp_exchange(void* const* peers, int world, int rank,
                                 const void* payload, int nbytes, int slot_bytes,
                                 void* out, int mode, int* status,
                                 locks_stream_t stream) {
    LOCKS_REQUIRE(peers && payload && out, LOCKS_ERR_ARG,
                  "locks_cp_exchange: null pointer argument");
    LOCKS_REQUIRE(world >= 1 && world <= XMAX && rank >= 0 && rank < world,
                  LOCKS_ERR_ARG, "locks_cp_exchange: supports 1..%d ranks", XMAX);
    LOCKS_REQUIRE(nbytes > 0 && (nbytes & 15) == 0 && nbytes <= slot_bytes &&
                      (slot_bytes & 15) == 0 && mode >= 0 && mode <= 3 &&
                      (!(mode & 2) || 2 * nbytes <= slot_bytes) &&
                      (reinterpret_cast<uintptr_t>(payload) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(out) & 15) == 0,
                  LOCKS_ERR_ARG,
                  "locks_cp_exchange: sizes must be multiples of 16 within the "
                  "slot, buffers 16-byte aligned");
    XchgPeers x;
    for (int r = 0; r < XMAX; ++r)
        x.base[r] = (r < world) ? static_cast<uint8_t*>(peers[r]) : nullptr;
    for (int r = 0; r < world; ++r)
        LOCKS_REQUIRE(x.base[r] != nullptr, LOCKS_ERR_ARG,
                      "locks_cp_exchange: peer %d has no region", r);
    cp_exchange_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
        x, world, rank, static_cast<const uint4*>(payload), nbytes, slot_bytes,
        static_cast<uint8_t*>(out), mode, status);
    return check_launch("locks_cp_exchange");
}

// ---------------------------------------------------------------------------
// Link regions of the in-kernel exchanges (cp_link.cuh)
// ---------------------------------------------------------------------------
namespace locks {
namespace {
__global__ void cp_begin_step_kernel(uint32_t* step) { *step += 1u; }
__global__ void cp_set_step_kernel(uint32_t* step, uint32_t v) { *step = v; }
}  // namespace
}  // namespace locks

extern "C" int locks_cp_link_bytes(int n_kv, int G, int cap, int64_t* out) {
    LOCKS_REQUIRE(out && n_kv >= 1 && G >= 1 && G <= 16 && cap >= 1, LOCKS_ERR_ARG,
                  "locks_cp_link_bytes: bad argument");
    *out = cp_region_bytes(n_kv, G, cap);
    return LOCKS_OK;
}

extern "C" int locks_cp_begin_step(void* region, locks_stream_t stream) {
    LOCKS_REQUIRE(region != nullptr, LOCKS_ERR_ARG,
                  "locks_cp_begin_step: null region");
    cp_begin_step_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint32_t*>(region));
    pdl_break();
    return check_launch("locks_cp_begin_step");
}

extern "C" int locks_cp_link_reset(void* region, int64_t bytes, uint32_t step,
                                   locks_stream_t stream) {
    LOCKS_REQUIRE(region != nullptr && bytes >= CP_HEADER_BYTES, LOCKS_ERR_ARG,
                  "locks_cp_link_reset: bad argument");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const cudaError_t e = cudaMemsetAsync(region, 0, (size_t)bytes, s);
    if (e != cudaSuccess)
        return fail(LOCKS_ERR_LAUNCH, "locks_cp_link_reset: %s", cudaGetErrorString(e));
    cp_set_step_kernel<<<1, 1, 0, s>>>(static_cast<uint32_t*>(region), step);
    pdl_break();
    return check_launch("locks_cp_link_reset");
}
