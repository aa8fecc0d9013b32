// Context-parallel exchanges done INSIDE the selector and the decode kernel.
//
// One long sequence is split over the GPUs of a node by contiguous page ranges.
// Per layer three small all-to-all exchanges make the result equal to the
// single-GPU path: the per-head score maxima (selector, before the combine), the
// best-b candidates (selector, after the local selection) and the attention
// partials (decode, before the normalisation).  Each is a few hundred bytes to
// 17 KB per rank, so what costs is the number of kernel hand-offs, not the
// bytes: the kernels therefore push their words straight into every peer's
// exchange region and poll their own region for the peers' words -- no exchange
// launch, no library collective.
//
// Transport: every 32-bit word travels as an 8-byte {word, epoch} packet written
// with one store (st.relaxed.sys.v2), so a packet is valid exactly when its
// epoch field equals the current epoch: no fence, no separate flag.  Every rank
// owns an identical region (cudaMalloc'ed, opened by the peers through CUDA
// IPC) with three areas (maxima, candidates, partials), each
//     [2 epoch parities][LOCKS_CP_MAX_RANKS source ranks][words] packets.
// The epoch of an exchange is  step * n_layers + layer + 1  where `step` is a
// device word every rank advances once per decode step (locks_cp_begin_step),
// so epochs agree across ranks without communication and never repeat.  Two
// parity halves suffice: a rank reaches the same exchange of layer e + 2 only
// after it has received every peer's words of layer e + 1, which a peer sends
// only after its kernel of layer e -- the last reader of the e-half -- has ended.
//
// A consumer reads LOCAL memory only; remote accesses are plain stores.  Every
// wait is bounded (LOCKS_ST_WAIT_TIMEOUT in the status word, then the kernel
// carries on with whatever it has and returns).
#pragma once

#include "common.cuh"

namespace locks {

constexpr int CP_MAX_RANKS = LOCKS_CP_MAX_RANKS;
constexpr unsigned long long CP_WAIT_NS = 2000000000ull;   // 2 s

struct CpLink {
    uint8_t* base[CP_MAX_RANKS];   // every rank's region (own one included)
    const uint32_t* step;          // decode-step counter (device word, per rank)
    int world, rank;               // world == 0: no context parallelism
    int layer, n_layers;
    int p0;                        // global number of this rank's local page 0
    int cap;                       // candidate slots per (rank, kv-head)
    int b_global;                  // the sequence's page budget
    int sink_loc, nsh_loc;         // selectable local pages: [sink_loc, nsh_loc)
    int64_t off_hmax, off_cand, off_part;   // byte offsets of the three areas
    int hmax_words, cand_words, part_words; // packets per source rank per parity
};

__device__ __forceinline__ unsigned long long cp_time_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t cp_epoch(const CpLink& c) {
    return __ldcg(c.step) * (uint32_t)c.n_layers + (uint32_t)c.layer + 1u;
}

// byte offset, inside a region, of packet `idx` of source rank `src`
__device__ __forceinline__ int64_t cp_slot(int64_t area, int words, uint32_t epoch,
                                           int src, int idx) {
    return area + ((((int64_t)(epoch & 1u) * CP_MAX_RANKS + src) * words + idx) << 3);
}

// this rank's word `idx` of an area -> every rank's region
__device__ __forceinline__ void cp_push(const CpLink& c, int64_t area, int words,
                                        uint32_t epoch, int idx, uint32_t value) {
    const int64_t off = cp_slot(area, words, epoch, c.rank, idx);
    for (int r = 0; r < c.world; ++r)
        asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};"
                     ::"l"(c.base[r] + off), "r"(value), "r"(epoch) : "memory");
}

__device__ __forceinline__ uint2 cp_load(const uint8_t* p) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];"
                 : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

// word `idx` of source rank `src`, polled in this rank's own region until its
// epoch field matches; false (and *late set) when the wait ran out
__device__ __forceinline__ bool cp_wait_word(const CpLink& c, int64_t area, int words,
                                             uint32_t epoch, int src, int idx,
                                             unsigned long long t0, uint32_t& value) {
    const uint8_t* p = c.base[c.rank] + cp_slot(area, words, epoch, src, idx);
    for (;;) {
        const uint2 v = cp_load(p);
        if (v.y == epoch) { value = v.x; return true; }
        if (cp_time_ns() - t0 > CP_WAIT_NS) { value = 0u; return false; }
    }
}

// Several words of this rank's own region at once: the loads are issued back to
// back (one L2 round trip for all of them) and re-issued until every epoch field
// matches.  addr[k] are byte addresses in the local region.
template <int K>
__device__ __forceinline__ bool cp_wait_words(const uint8_t* const (&addr)[K], int n,
                                              uint32_t epoch, uint32_t (&val)[K]) {
    const unsigned long long t0 = cp_time_ns();
    for (;;) {
        uint2 v[K];
#pragma unroll
        for (int k = 0; k < K; ++k)
            if (k < n) v[k] = cp_load(addr[k]);
        bool all = true;
#pragma unroll
        for (int k = 0; k < K; ++k)
            if (k < n) { val[k] = v[k].x; all = all && (v[k].y == epoch); }
        if (all) return true;
        if (cp_time_ns() - t0 > CP_WAIT_NS) return false;
    }
}

// ---- host side: region layout -------------------------------------------------
constexpr int64_t CP_HEADER_BYTES = 64;       // word 0: the decode-step counter
constexpr int CP_PART_WORDS_PER_HEAD = 128 + 2;   // m, l, O[128]

inline int64_t cp_area_bytes(int words) {
    return (int64_t)2 * CP_MAX_RANKS * words * 8;
}
inline int64_t cp_region_bytes(int n_kv, int G, int cap) {
    return CP_HEADER_BYTES + cp_area_bytes(n_kv * G) + cp_area_bytes(n_kv * cap * 2) +
           cp_area_bytes(n_kv * G * CP_PART_WORDS_PER_HEAD);
}
// 0 on success; the link of the public struct, checked and laid out
inline int cp_link_fill(CpLink& c, const locks_cp_link_t* l, int n_kv, int G,
                        const char* who) {
    LOCKS_REQUIRE(l != nullptr, LOCKS_ERR_ARG, "%s: null link description", who);
    LOCKS_REQUIRE(l->world >= 1 && l->world <= CP_MAX_RANKS && l->rank >= 0 &&
                      l->rank < l->world && l->n_layers >= 1 && l->layer >= 0 &&
                      l->layer < l->n_layers && l->cap >= 1 && l->b_global >= 0 &&
                      l->p0 >= 0,
                  LOCKS_ERR_ARG, "%s: bad link description (world %d, rank %d, "
                  "layer %d of %d, cap %d)", who, l->world, l->rank, l->layer,
                  l->n_layers, l->cap);
    for (int r = 0; r < CP_MAX_RANKS; ++r) {
        c.base[r] = (r < l->world) ? static_cast<uint8_t*>(l->regions[r]) : nullptr;
        LOCKS_REQUIRE(r >= l->world || c.base[r] != nullptr, LOCKS_ERR_ARG,
                      "%s: rank %d has no link region", who, r);
    }
    c.step = reinterpret_cast<const uint32_t*>(c.base[l->rank]);
    c.world = l->world; c.rank = l->rank; c.layer = l->layer;
    c.n_layers = l->n_layers; c.p0 = l->p0; c.cap = l->cap;
    c.b_global = l->b_global; c.sink_loc = l->sink_loc; c.nsh_loc = l->nsh_loc;
    c.hmax_words = n_kv * G;
    c.cand_words = n_kv * l->cap * 2;
    c.part_words = n_kv * G * CP_PART_WORDS_PER_HEAD;
    c.off_hmax = CP_HEADER_BYTES;
    c.off_cand = c.off_hmax + cp_area_bytes(c.hmax_words);
    c.off_part = c.off_cand + cp_area_bytes(c.cand_words);
    return LOCKS_OK;
}

}  // namespace locks
