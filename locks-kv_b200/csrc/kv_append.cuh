// The new token's K/V store, shared by the stand-alone KV-write kernel and by
// the selector (which can carry the store of its own (request, kv-head) row).
//
// One thread per channel dd of one (token row, kv-head): V is copied, K channels
// below rot_dim are rotated with the (cos | sin) row of the token's position,
// the others copied.  Rotation arithmetic: bf16 -> fp32, two separately rounded
// products and one rounded sum / difference, round to bf16 (no fused
// multiply-add), in half-split ("neox") or interleaved pairing.
#pragma once
#include "common.cuh"

namespace locks {

struct KvAppend {
    const __nv_bfloat16* key;                      // null: nothing to store
    const __nv_bfloat16* val;
    int64_t k_row, k_head, v_row, v_head;          // element strides of key / val
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    int64_t cb, ct, ch;                            // element strides of the cache planes
    const int64_t* slot;
    const int64_t* pos;
    const __nv_bfloat16* cos_sin;                  // (P, rot_dim): cos half | sin half
    int64_t cs_row;
    int rot_dim, neox, page, num_blocks, head_dim;
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

// Channel dd of head kh of token row r.  Returns without a store when the row's
// slot is negative (the engine's "no write" mark) or outside the cache.
__device__ __forceinline__ void kv_append_elem(const KvAppend& a, int r, int kh,
                                               int dd) {
    const int64_t s = a.slot[r];
    if (s < 0) return;
    const int64_t blk = s / a.page;
    if (blk >= a.num_blocks) return;
    const int t = (int)(s % a.page);
    const int64_t dst = blk * a.cb + (int64_t)t * a.ct + (int64_t)kh * a.ch + dd;
    a.v_cache[dst] = a.val[(int64_t)r * a.v_row + (int64_t)kh * a.v_head + dd];
    const __nv_bfloat16* krow = a.key + (int64_t)r * a.k_row + (int64_t)kh * a.k_head;
    a.k_cache[dst] = (a.cos_sin && dd < a.rot_dim)
        ? __float2bfloat16_rn(rope_elem(krow, a.cos_sin + a.pos[r] * a.cs_row, dd,
                                        a.rot_dim, a.neox))
        : krow[dd];
}

}  // namespace locks
