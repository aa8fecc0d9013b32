// KV-write neighbour of the decode hot path: rotate the new token's K, store K
// and V into the paged cache, and -- when the token completes a page -- build
// that page's rki4 summary in the same launch.
//
// One CTA (256 threads) per token row r.  slot = slot_mapping[r] (< 0: the row is
// skipped, the engine's "no write" mark); block = slot / page, t = slot % page.
//   phase 1  all threads: V is copied, K channels below rot_dim are rotated with
//            the (cos | sin) row of positions[r], the others copied.  Rotation
//            arithmetic: bf16 -> fp32, two separately rounded products and one
//            rounded sum / difference, round to bf16 (no fused multiply-add), in
//            half-split ("neox") or interleaved pairing.
//   phase 2  only when t == page - 1 and a summary slab was passed: after a CTA
//            barrier (the stores above are visible to the CTA) warps 0-3 run
//            rki4_build_one over the page's heads, reading the 15 older tokens
//            and the one just stored from the cache.
// The page summary is then valid in the same step its page is completed, inside
// whatever CUDA graph holds the KV write, with no host-side refresh decision.
// The build is a Jacobi eigen-solve of about 45 us per head, so a write that
// completes a page takes about 90 us (8 heads) instead of 4 us; where that
// latency matters, pass no summary slab here and launch locks_rki4_build_slots
// once per step on a forked graph branch instead (same slot_mapping, same
// result; the page is not scored before it leaves the recent window).
#include "rki4_build.cuh"

namespace locks {
namespace {

constexpr int KW_THREADS = 256;
constexpr int KW_BUILD_WARPS = 4;     // measured: 4 builders finish 8 heads sooner than 8

struct KvWriteParams {
    const __nv_bfloat16* key;
    const __nv_bfloat16* val;
    int64_t k_row, k_head, v_row, v_head;          // element strides of key / val
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    int64_t cb, ct, ch;                            // element strides of the cache planes
    const int64_t* slot;
    const int64_t* pos;
    const __nv_bfloat16* cos_sin;                  // (P, rot_dim): cos half | sin half
    int64_t cs_row;
    uint8_t* records;                              // this layer's (NB, n_kv, 832) or null
    __nv_bfloat16* tags;
    int rot_dim, neox, n_kv, page, num_blocks;
};

__device__ __forceinline__ float rope_elem(const __nv_bfloat16* x,
                                           const __nv_bfloat16* crow, int dd,
                                           int rot_dim, int neox) {
    const int half = rot_dim >> 1;
    if (neox) {
        const int lo = (dd < half) ? dd : dd - half;
        const float c = __bfloat162float(crow[lo]);
        const float s = __bfloat162float(crow[half + lo]);
        const float e = __bfloat162float(x[lo]);
        const float o = __bfloat162float(x[lo + half]);
        return (dd < half) ? __fsub_rn(__fmul_rn(e, c), __fmul_rn(o, s))
                           : __fadd_rn(__fmul_rn(o, c), __fmul_rn(e, s));
    }
    const int pr = dd >> 1;
    const float c = __bfloat162float(crow[pr]);
    const float s = __bfloat162float(crow[half + pr]);
    const float me = __bfloat162float(x[dd]);
    const float pa = __bfloat162float(x[dd ^ 1]);
    return (dd & 1) ? __fadd_rn(__fmul_rn(me, c), __fmul_rn(pa, s))
                    : __fsub_rn(__fmul_rn(me, c), __fmul_rn(pa, s));
}

__global__ void __launch_bounds__(KW_THREADS) kv_write_kernel(const KvWriteParams p) {
    __shared__ __align__(16) BuildWarpScratch scratch[KW_BUILD_WARPS];
    const int r = blockIdx.x;
    const int64_t s = p.slot[r];
    if (s < 0) return;
    const int64_t blk = s / p.page;
    const int t = (int)(s % p.page);
    if (blk >= p.num_blocks) return;
    const int tid = threadIdx.x;
    const int64_t base = blk * p.cb + (int64_t)t * p.ct;
    const __nv_bfloat16* crow =
        p.cos_sin ? p.cos_sin + p.pos[r] * p.cs_row : nullptr;
    for (int i = tid; i < p.n_kv * BUILD_HD; i += KW_THREADS) {
        const int kh = i / BUILD_HD, dd = i % BUILD_HD;
        const int64_t dst = base + (int64_t)kh * p.ch + dd;
        p.v_cache[dst] = p.val[(int64_t)r * p.v_row + (int64_t)kh * p.v_head + dd];
        const __nv_bfloat16* krow = p.key + (int64_t)r * p.k_row + (int64_t)kh * p.k_head;
        p.k_cache[dst] = (crow && dd < p.rot_dim)
            ? __float2bfloat16_rn(rope_elem(krow, crow, dd, p.rot_dim, p.neox))
            : krow[dd];
    }
    if (p.records == nullptr || t != p.page - 1) return;
    __syncthreads();                   // the page's last row is in the cache
    const int warp = tid >> 5, lane = tid & 31;
    if (warp >= KW_BUILD_WARPS) return;
    for (int kh = warp; kh < p.n_kv; kh += KW_BUILD_WARPS) {
        const int64_t cell = blk * p.n_kv + kh;
        rki4_build_one(scratch[warp], p.k_cache + blk * p.cb + (int64_t)kh * p.ch,
                       p.ct, p.records + cell * REC_BYTES,
                       p.tags + cell * LOCKS_TAG_WIDTH, lane);
        __syncwarp();
    }
}

}  // namespace
}  // namespace locks

using namespace locks;

extern "C" int locks_kv_write(
    const void* key, int64_t k_row_stride, int64_t k_head_stride, const void* val,
    int64_t v_row_stride, int64_t v_head_stride, void* k_cache, void* v_cache,
    int64_t kv_stride_block, int64_t kv_stride_tok, int64_t kv_stride_head,
    const int64_t* slot_mapping, const int64_t* positions, const void* cos_sin,
    int64_t cos_sin_row_stride, int rot_dim, int neox, void* records_layer,
    void* tags_layer, int n_tok, int n_kv, int head_dim, int page, int num_blocks,
    locks_stream_t stream) {
    LOCKS_REQUIRE(key && val && k_cache && v_cache && slot_mapping, LOCKS_ERR_ARG,
                  "locks_kv_write: null pointer argument");
    LOCKS_REQUIRE(head_dim == BUILD_HD && page == BUILD_PAGE_T, LOCKS_ERR_GEOMETRY,
                  "locks_kv_write: supports head_dim 128 / page 16, got %d / %d",
                  head_dim, page);
    LOCKS_REQUIRE(n_tok >= 0 && n_kv >= 1 && num_blocks >= 1, LOCKS_ERR_ARG,
                  "locks_kv_write: bad size argument");
    LOCKS_REQUIRE(cos_sin == nullptr ||
                      (positions && rot_dim >= 2 && rot_dim <= head_dim &&
                       (rot_dim & 1) == 0 && cos_sin_row_stride >= rot_dim),
                  LOCKS_ERR_ARG,
                  "locks_kv_write: rotation needs positions and an even rot_dim "
                  "<= head_dim");
    LOCKS_REQUIRE(records_layer == nullptr ||
                      (tags_layer != nullptr && (kv_stride_tok % 4) == 0 &&
                       (kv_stride_head % 4) == 0 && (kv_stride_block % 4) == 0 &&
                       (reinterpret_cast<uintptr_t>(k_cache) & 7) == 0),
                  LOCKS_ERR_ARG,
                  "locks_kv_write: the summary build needs tags and 8-byte "
                  "aligned K rows");
    if (n_tok == 0) return LOCKS_OK;
    KvWriteParams p;
    p.key = static_cast<const __nv_bfloat16*>(key);
    p.val = static_cast<const __nv_bfloat16*>(val);
    p.k_row = k_row_stride; p.k_head = k_head_stride;
    p.v_row = v_row_stride; p.v_head = v_head_stride;
    p.k_cache = static_cast<__nv_bfloat16*>(k_cache);
    p.v_cache = static_cast<__nv_bfloat16*>(v_cache);
    p.cb = kv_stride_block; p.ct = kv_stride_tok; p.ch = kv_stride_head;
    p.slot = slot_mapping; p.pos = positions;
    p.cos_sin = static_cast<const __nv_bfloat16*>(cos_sin);
    p.cs_row = cos_sin_row_stride;
    p.records = static_cast<uint8_t*>(records_layer);
    p.tags = static_cast<__nv_bfloat16*>(tags_layer);
    p.rot_dim = rot_dim; p.neox = neox; p.n_kv = n_kv; p.page = page;
    p.num_blocks = num_blocks;
    kv_write_kernel<<<n_tok, KW_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(p);
    if (records_layer) pdl_break();    // the scorer prefetches summaries before its wait
    return check_launch("locks_kv_write");
}
