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
// A launch that carries SEVERAL rows (a prefill chunk, speculative tokens) may
// hold rows 14 and 15 of one page in different CTAs, and CTAs are not ordered:
// such a launch runs phase 1 for all rows first and phase 2 as a second launch
// of the same kernel behind it, so the builder always reads a complete page.
// The page summary is then valid in the same step its page is completed, inside
// whatever CUDA graph holds the KV write, with no host-side refresh decision.
// The build is a Jacobi eigen-solve of about 45 us per head, so a write that
// completes a page takes about 90 us (8 heads) instead of 4 us; where that
// latency matters, pass no summary slab here and launch locks_rki4_build_slots
// once per step on a forked graph branch instead (same slot_mapping, same
// result; the page is not scored before it leaves the recent window).
#include "kv_append.cuh"
#include "rki4_build.cuh"

namespace locks {
namespace {

constexpr int KW_THREADS = 256;
constexpr int KW_BUILD_WARPS = 4;     // measured: 4 builders finish 8 heads sooner than 8

struct KvWriteParams {
    KvAppend a;
    uint8_t* records;                              // this layer's (NB, n_kv, 832) or null
    __nv_bfloat16* tags;
    int n_kv;
    int phases;                                    // bit 0: store the rows, bit 1: build
};

__global__ void __launch_bounds__(KW_THREADS) kv_write_kernel(const KvWriteParams p) {
    __shared__ __align__(16) BuildWarpScratch scratch[KW_BUILD_WARPS];
    const int r = blockIdx.x;
    const int64_t s = p.a.slot[r];
    if (s < 0) return;
    const int64_t blk = s / p.a.page;
    const int t = (int)(s % p.a.page);
    if (blk >= p.a.num_blocks) return;
    const int tid = threadIdx.x;
    if (p.phases & 1)
        for (int i = tid; i < p.n_kv * BUILD_HD; i += KW_THREADS)
            kv_append_elem(p.a, r, i / BUILD_HD, i % BUILD_HD);
    if (!(p.phases & 2) || p.records == nullptr || t != p.a.page - 1) return;
    __syncthreads();                   // the page's last row is in the cache
    const int warp = tid >> 5, lane = tid & 31;
    if (warp >= KW_BUILD_WARPS) return;
    for (int kh = warp; kh < p.n_kv; kh += KW_BUILD_WARPS) {
        const int64_t cell = blk * p.n_kv + kh;
        rki4_build_one(scratch[warp],
                       p.a.k_cache + blk * p.a.cb + (int64_t)kh * p.a.ch, p.a.ct,
                       p.records + cell * REC_BYTES,
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
    p.a.key = static_cast<const __nv_bfloat16*>(key);
    p.a.val = static_cast<const __nv_bfloat16*>(val);
    p.a.k_row = k_row_stride; p.a.k_head = k_head_stride;
    p.a.v_row = v_row_stride; p.a.v_head = v_head_stride;
    p.a.k_cache = static_cast<__nv_bfloat16*>(k_cache);
    p.a.v_cache = static_cast<__nv_bfloat16*>(v_cache);
    p.a.cb = kv_stride_block; p.a.ct = kv_stride_tok; p.a.ch = kv_stride_head;
    p.a.slot = slot_mapping; p.a.pos = positions;
    p.a.cos_sin = static_cast<const __nv_bfloat16*>(cos_sin);
    p.a.cs_row = cos_sin_row_stride;
    p.a.rot_dim = rot_dim; p.a.neox = neox; p.a.page = page;
    p.a.num_blocks = num_blocks; p.a.head_dim = head_dim;
    p.records = static_cast<uint8_t*>(records_layer);
    p.tags = static_cast<__nv_bfloat16*>(tags_layer);
    p.n_kv = n_kv;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (n_tok == 1 || records_layer == nullptr) {
        p.phases = 3;
        kv_write_kernel<<<n_tok, KW_THREADS, 0, s>>>(p);
    } else {
        // several rows: every row is in the cache before any page is summarised
        p.phases = 1;
        kv_write_kernel<<<n_tok, KW_THREADS, 0, s>>>(p);
        p.phases = 2;
        kv_write_kernel<<<n_tok, KW_THREADS, 0, s>>>(p);
    }
    if (records_layer) pdl_break();    // the scorer prefetches summaries before its wait
    return check_launch("locks_kv_write");
}
