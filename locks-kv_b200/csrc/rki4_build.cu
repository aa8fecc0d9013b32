// rki4 summary builder: one warp per (layer, physical block, kv-head) runs
// rki4_build_one (rki4_build.cuh); plus the content-tag scan that finds the
// blocks whose summaries are stale.
#include "rki4_build.cuh"

namespace locks {
namespace {

constexpr int BW = 4;                  // warps (jobs) per CTA

struct BuildParams {
    const void* const* k_layers;
    int64_t sb, st, sh;                // element strides of a K plane
    uint8_t* records;
    __nv_bfloat16* tags;
    const int32_t* blocks;
    const int64_t* slots;              // slot mode: job i looks at slots[i]
    int n_blocks, layer0, n_layers, nb_state, nb_cache, n_kv, page;
};


__global__ void __launch_bounds__(BW * 32) rki4_build_kernel(const BuildParams p) {
    __shared__ __align__(16) BuildWarpScratch scratch[BW];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t job = (int64_t)blockIdx.x * BW + warp;
    const int64_t n_jobs = (int64_t)p.n_layers * p.n_blocks * p.n_kv;
    if (job >= n_jobs) return;
    const int kh = (int)(job % p.n_kv);
    const int bi = (int)((job / p.n_kv) % p.n_blocks);
    const int layer = p.layer0 + (int)(job / ((int64_t)p.n_kv * p.n_blocks));
    int blk;
    if (p.slots) {
        // a cache slot that is the LAST token of its block names a page that
        // has just been completed; every other slot is nobody's job
        const int64_t s = p.slots[bi];
        if (s < 0 || (s % p.page) != p.page - 1) return;
        blk = (int)(s / p.page);
    } else {
        blk = p.blocks[bi];
    }
    if (blk < 0 || blk >= p.nb_state || blk >= p.nb_cache) return;
    const __nv_bfloat16* K =
        static_cast<const __nv_bfloat16*>(p.k_layers[layer]) +
        (int64_t)blk * p.sb + (int64_t)kh * p.sh;
    const int64_t cell = ((int64_t)layer * p.nb_state + blk) * p.n_kv + kh;
    rki4_build_one(scratch[warp], K, p.st, p.records + cell * REC_BYTES,
                   p.tags + cell * LOCKS_TAG_WIDTH, lane);
}

struct TagScanParams {
    const void* const* k_layers;
    int64_t sb, st, sh;
    const __nv_bfloat16* tags;
    const int32_t* blocks;
    const uint8_t* valid;
    uint8_t* stale;
    int n_blocks, n_layers, nb_state, n_kv, page;
};

// one warp per listed block; lanes stride over (layer, kv-head) pairs
__global__ void __launch_bounds__(128) tag_scan_kernel(const TagScanParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i = blockIdx.x * 4 + warp;
    if (i >= p.n_blocks) return;
    const int blk = p.blocks[i];
    bool bad = false;
    if (p.valid[i] && blk >= 0 && blk < p.nb_state) {
        const int n = p.n_layers * p.n_kv;
        for (int e = lane; e < n; e += 32) {
            const int l = e / p.n_kv, kh = e % p.n_kv;
            const __nv_bfloat16* cur =
                static_cast<const __nv_bfloat16*>(p.k_layers[l]) +
                (int64_t)blk * p.sb + (int64_t)(p.page - 1) * p.st +
                (int64_t)kh * p.sh;
            const __nv_bfloat16* old = p.tags +
                (((int64_t)l * p.nb_state + blk) * p.n_kv + kh) * LOCKS_TAG_WIDTH;
#pragma unroll
            for (int c = 0; c < LOCKS_TAG_WIDTH; ++c)
                bad |= !(__bfloat162float(cur[c]) == __bfloat162float(old[c]));
        }
    }
    bad = __any_sync(0xffffffffu, bad);
    if (lane == 0) p.stale[i] = (p.valid[i] && bad) ? 1 : 0;
}

}  // namespace
}  // namespace locks

using namespace locks;

extern "C" int locks_rki4_build(
    const void* const* k_layers, int64_t k_stride_block, int64_t k_stride_tok,
    int64_t k_stride_head, void* records, void* tags, const int32_t* blocks,
    int n_blocks, int layer0, int n_layers, int num_blocks_state,
    int num_blocks_cache, int n_kv, int head_dim, int page,
    locks_stream_t stream) {
    LOCKS_REQUIRE(k_layers && records && tags && (blocks || n_blocks == 0),
                  LOCKS_ERR_ARG, "locks_rki4_build: null pointer argument");
    LOCKS_REQUIRE(head_dim == BUILD_HD && page == BUILD_PAGE_T, LOCKS_ERR_GEOMETRY,
                  "locks_rki4_build: supports head_dim 128 / page 16, got %d / %d",
                  head_dim, page);
    LOCKS_REQUIRE(n_blocks >= 0 && layer0 >= 0 && n_layers >= 0 &&
                      num_blocks_state >= 1 && num_blocks_cache >= 1 && n_kv >= 1,
                  LOCKS_ERR_ARG, "locks_rki4_build: bad size argument");
    LOCKS_REQUIRE(k_stride_block % 4 == 0 && k_stride_tok % 4 == 0 &&
                      k_stride_head % 4 == 0,
                  LOCKS_ERR_ARG,
                  "locks_rki4_build: K strides must be multiples of 4 elements");
    const int64_t n_jobs = (int64_t)n_layers * n_blocks * n_kv;
    if (n_jobs == 0) return LOCKS_OK;
    LOCKS_REQUIRE((n_jobs + BW - 1) / BW <= 2147483647LL, LOCKS_ERR_SIZE,
                  "locks_rki4_build: too many (layer, block, head) jobs");
    BuildParams p;
    p.k_layers = k_layers; p.sb = k_stride_block; p.st = k_stride_tok;
    p.sh = k_stride_head;
    p.records = static_cast<uint8_t*>(records);
    p.tags = static_cast<__nv_bfloat16*>(tags);
    p.blocks = blocks; p.slots = nullptr; p.n_blocks = n_blocks; p.layer0 = layer0;
    p.n_layers = n_layers; p.nb_state = num_blocks_state;
    p.nb_cache = num_blocks_cache; p.n_kv = n_kv; p.page = page;
    rki4_build_kernel<<<(unsigned)((n_jobs + BW - 1) / BW), BW * 32, 0,
                        static_cast<cudaStream_t>(stream)>>>(p);
    pdl_break();
    return check_launch("locks_rki4_build");
}

extern "C" int locks_rki4_build_slots(
    const void* const* k_layers, int64_t k_stride_block, int64_t k_stride_tok,
    int64_t k_stride_head, void* records, void* tags, const int64_t* slot_mapping,
    int n_tok, int layer0, int n_layers, int num_blocks_state,
    int num_blocks_cache, int n_kv, int head_dim, int page,
    locks_stream_t stream) {
    LOCKS_REQUIRE(k_layers && records && tags && (slot_mapping || n_tok == 0),
                  LOCKS_ERR_ARG, "locks_rki4_build_slots: null pointer argument");
    LOCKS_REQUIRE(head_dim == BUILD_HD && page == BUILD_PAGE_T, LOCKS_ERR_GEOMETRY,
                  "locks_rki4_build_slots: supports head_dim 128 / page 16, got "
                  "%d / %d", head_dim, page);
    LOCKS_REQUIRE(n_tok >= 0 && layer0 >= 0 && n_layers >= 0 &&
                      num_blocks_state >= 1 && num_blocks_cache >= 1 && n_kv >= 1 &&
                      k_stride_block % 4 == 0 && k_stride_tok % 4 == 0 &&
                      k_stride_head % 4 == 0,
                  LOCKS_ERR_ARG, "locks_rki4_build_slots: bad size or stride");
    const int64_t n_jobs = (int64_t)n_layers * n_tok * n_kv;
    if (n_jobs == 0) return LOCKS_OK;
    LOCKS_REQUIRE((n_jobs + BW - 1) / BW <= 2147483647LL, LOCKS_ERR_SIZE,
                  "locks_rki4_build_slots: too many (layer, token, head) jobs");
    BuildParams p;
    p.k_layers = k_layers; p.sb = k_stride_block; p.st = k_stride_tok;
    p.sh = k_stride_head;
    p.records = static_cast<uint8_t*>(records);
    p.tags = static_cast<__nv_bfloat16*>(tags);
    p.blocks = nullptr; p.slots = slot_mapping; p.n_blocks = n_tok;
    p.layer0 = layer0; p.n_layers = n_layers; p.nb_state = num_blocks_state;
    p.nb_cache = num_blocks_cache; p.n_kv = n_kv; p.page = page;
    rki4_build_kernel<<<(unsigned)((n_jobs + BW - 1) / BW), BW * 32, 0,
                        static_cast<cudaStream_t>(stream)>>>(p);
    pdl_break();
    return check_launch("locks_rki4_build_slots");
}

extern "C" int locks_rki4_tag_scan(
    const void* const* k_layers, int64_t k_stride_block, int64_t k_stride_tok,
    int64_t k_stride_head, const void* tags, const int32_t* blocks,
    const uint8_t* valid, uint8_t* stale, int n_blocks, int n_layers,
    int num_blocks_state, int n_kv, int page, locks_stream_t stream) {
    LOCKS_REQUIRE(k_layers && tags && valid && stale && (blocks || n_blocks == 0),
                  LOCKS_ERR_ARG, "locks_rki4_tag_scan: null pointer argument");
    LOCKS_REQUIRE(n_blocks >= 0 && n_layers >= 1 && num_blocks_state >= 1 &&
                      n_kv >= 1 && page >= 1,
                  LOCKS_ERR_ARG, "locks_rki4_tag_scan: bad size argument");
    if (n_blocks == 0) return LOCKS_OK;
    TagScanParams p;
    p.k_layers = k_layers; p.sb = k_stride_block; p.st = k_stride_tok;
    p.sh = k_stride_head;
    p.tags = static_cast<const __nv_bfloat16*>(tags);
    p.blocks = blocks; p.valid = valid; p.stale = stale;
    p.n_blocks = n_blocks; p.n_layers = n_layers; p.nb_state = num_blocks_state;
    p.n_kv = n_kv; p.page = page;
    tag_scan_kernel<<<(n_blocks + 3) / 4, 128, 0,
                      static_cast<cudaStream_t>(stream)>>>(p);
    return check_launch("locks_rki4_tag_scan");
}
