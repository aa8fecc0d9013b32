// Sparse paged decode: split-K flash decode over the selected pages, the split
// merge, the one-launch fused variant and the dense full-KV baseline.
//
// One kernel serves all three.  A CTA (8 warps) owns one (request, kv-head) and
// a contiguous run of page-table entries; its warps take entries round-robin
// and each warp runs its own 2-stage shared-memory ring.  A page (16 key rows +
// 16 value rows of 256 B, found through the page table and the block table) is
// fetched with 16-byte cp.async copies, 16 per lane and one commit group per
// page: a warp walks only a few pages, so what counts is how fast the first
// copies are on their way, and 512 small bulk-copy requests per CTA queue up in
// the copy engine far longer than the same bytes as coalesced LSU copies.
// Rows past seq_len are zero-filled (source size 0), so stale cache bytes
// cannot leak.
//
// Math per page, on warp-level tensor-core fragments whose 16 rows are the
// query heads of the GQA group:  S = Q K^T (bf16, 16 m16n8k16 steps), online
// softmax in fp32, O += P V as an fp16 product with fp32 accumulation (P in fp16,
// V converted bf16 -> fp16 in registers: the reference decode's arithmetic).
// The warps' (m, l, O) are combined through shared memory; the CTA then stores one split partial (split mode), or, in
// fused mode, the CTAs of a thread-block cluster -- one cluster per (request,
// kv-head), each CTA walking its share of the page list -- exchange their
// (m, l, O) through distributed shared memory and write the normalised bf16
// output row directly: no partial buffers in HBM and no merge launch.
#include <cooperative_groups.h>
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "cp_link.cuh"
#include "tma.cuh"

namespace cg = cooperative_groups;

namespace locks {
namespace {


__device__ __forceinline__ uint32_t pack_f16x2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// two bf16 (packed) -> two fp16 (packed); exact for |x| < 65504 with <= 11
// significant bits, which bf16 values (8 bits) always have
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
    return pack_f16x2(__uint_as_float(v << 16), __uint_as_float(v & 0xFFFF0000u));
}
// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_f16_k16(float (&d)[4], uint32_t a0, uint32_t a1,
                                            uint32_t a2, uint32_t a3, uint32_t b0,
                                            uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int DW = 8;                 // warps per CTA
constexpr int DTHREADS = DW * 32;
constexpr int DSTAGES = 2;
constexpr int MAX_DCL = 16;             // largest cluster of the fused decode (non-portable size)
constexpr int PAGE_T = 16;
constexpr int HD = 128;
constexpr int ROWB = HD * 2 + 16;     // 272 B row pitch: conflict-free ldmatrix
constexpr int ACC_PITCH = HD + 4;     // floats

struct WarpBuf {
    uint8_t k[DSTAGES][PAGE_T][ROWB];
    uint8_t v[DSTAGES][PAGE_T][ROWB];
};
static_assert(sizeof(WarpBuf) >= 16 * ACC_PITCH * 4, "combine buffer must fit");

struct __align__(128) DecSmem {
    WarpBuf wb[DW];
    float cm[DW][16];
    float cl[DW][16];
    // cluster exchange (fused mode): CTA c pushes its (m, l) to every CTA and
    // the slice of its O that CTA d normalises into xacc[c] of CTA d
    float xm[MAX_DCL][16];
    float xl[MAX_DCL][16];
    float xacc[16 * HD + 16];
};

// TMA variant: a page of one kv-head arrives as two boxes of 16 rows x 64
// columns per plane, each a [16][128 B] tile with the 128-byte swizzle (no row
// padding needed: ldmatrix walks the swizzled pieces without bank conflicts).
constexpr int HALF_TILE = PAGE_T * 128;           // bytes of one box
constexpr int PAGE_TX = 4 * HALF_TILE;            // K + V bytes of one page
struct WarpBufT {
    uint8_t k[DSTAGES][2][PAGE_T][128];
    uint8_t v[DSTAGES][2][PAGE_T][128];
};
static_assert(sizeof(WarpBufT) >= 16 * ACC_PITCH * 4, "combine buffer must fit");
static_assert(sizeof(WarpBufT) % 1024 == 0, "swizzled tiles need 1 KiB alignment");

struct __align__(1024) DecSmemT {
    WarpBufT wb[DW];
    float cm[DW][16];
    float cl[DW][16];
    float xm[MAX_DCL][16];
    float xl[MAX_DCL][16];
    float xacc[16 * HD + 16];
    uint64_t full[DW][DSTAGES];    // one mbarrier per warp and ring stage
};

struct DecParams {
    const __nv_bfloat16* q;
    int64_t q_stride_req;
    const __nv_bfloat16* k_cache;
    const __nv_bfloat16* v_cache;
    int64_t stride_block, stride_tok, stride_head;
    const int32_t* block_table;
    int64_t bt_stride;
    const int32_t* page_table;     // nullptr: dense (entry j is page j)
    const int32_t* page_cnt;       // nullptr in dense mode
    const int32_t* seq_lens;
    float* m_part;
    float* l_part;
    float* acc_part;
    __nv_bfloat16* out;            // fused mode only
    int64_t out_stride_req;
    int n_kv, G, max_pages, split, pps_min, fused;
    int rows_per_block;            // tensor-map variant: token rows between blocks
    // V tier: v_cache is the pinned host pool (K's strides; read in place on a
    // miss), v_hot the staging buffer in device memory (slots hot_stride_block
    // apart, token and head strides as K's), v_map[block] the block's slot there
    // or -1.  Residency notes for the host: a hit marks vt_ref[slot]; a miss on a
    // complete page appends the block to vt_miss once per note round
    // (vt_pending[block] holds the round, *vt_epoch, in which it was last listed).
    const int32_t* v_map;
    const __nv_bfloat16* v_hot;
    int64_t hot_stride_block;
    uint8_t* vt_ref;
    int32_t* vt_pending;
    int32_t* vt_miss;
    int32_t* vt_miss_cnt;
    const int32_t* vt_epoch;
    int vt_miss_cap;
    float scale;
    int* status;
    const int32_t* row_order;      // grid row z handles request row_order[z] (or z)
    CpLink cp;          // context parallel: partials meet the peers' (world > 0)
};

// Context parallel: this rank's unnormalised partial of one output element --
// (m, l) of head g and O[g][dd], all relative to m -- meets the other ranks'.
// The words go to every rank's link region (the thread of channel 0 also sends
// the head's m and l), the peers' words are polled in the local region, and the
// merge of attention/merge.py:106-152 gives the sequence-wide (l, O).
__device__ __forceinline__ void cp_merge_element(const CpLink& cp, int kh, int G,
                                                 int g, int dd, float& M,
                                                 float& Lsum, float& o,
                                                 int* status) {
    const uint32_t epoch = cp_epoch(cp);
    const int idx = (kh * G + g) * CP_PART_WORDS_PER_HEAD;
    if (dd == 0) {
        cp_push(cp, cp.off_part, cp.part_words, epoch, idx, __float_as_uint(M));
        cp_push(cp, cp.off_part, cp.part_words, epoch, idx + 1, __float_as_uint(Lsum));
    }
    cp_push(cp, cp.off_part, cp.part_words, epoch, idx + 2 + dd, __float_as_uint(o));
    const uint8_t* mine = cp.base[cp.rank];
    uint2 vm[CP_MAX_RANKS], vl[CP_MAX_RANKS], vo[CP_MAX_RANKS];
    const unsigned long long t0 = cp_time_ns();
    bool late = false;
    for (;;) {
#pragma unroll
        for (int r = 0; r < CP_MAX_RANKS; ++r) {
            if (r < cp.world) {
                const uint8_t* a = mine + cp_slot(cp.off_part, cp.part_words, epoch, r, idx);
                vm[r] = cp_load(a);
                vl[r] = cp_load(a + 8);
                vo[r] = cp_load(a + 8 * (2 + dd));
            }
        }
        bool all = true;
#pragma unroll
        for (int r = 0; r < CP_MAX_RANKS; ++r)
            if (r < cp.world)
                all = all && vm[r].y == epoch && vl[r].y == epoch && vo[r].y == epoch;
        if (all) break;
        if (cp_time_ns() - t0 > CP_WAIT_NS) { late = true; break; }
    }
    if (late) {
        if (status) atomicExch(status, LOCKS_ST_WAIT_TIMEOUT);
        return;                                  // keep the local partial
    }
    float Mg = -INFINITY;
#pragma unroll
    for (int r = 0; r < CP_MAX_RANKS; ++r)
        if (r < cp.world && __uint_as_float(vl[r].x) > 0.f)
            Mg = fmaxf(Mg, __uint_as_float(vm[r].x));
    float Lg = 0.f, og = 0.f;
#pragma unroll
    for (int r = 0; r < CP_MAX_RANKS; ++r) {
        if (r < cp.world) {
            const float lr = __uint_as_float(vl[r].x);
            const float wt = (lr > 0.f) ? __expf(__uint_as_float(vm[r].x) - Mg) : 0.f;
            Lg += wt * lr;
            og += wt * __uint_as_float(vo[r].x);
        }
    }
    M = Mg; Lsum = Lg; o = og;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src,
                                           int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                 ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// One commit group per page: lane (h, c) = (lane >> 4, lane & 15) copies the
// 16-byte chunk c of rows h, h + 2, ..., h + 14 of K and of V.
// TIER: the V page comes from the staging buffer (slot >= 0) or, on a miss, in
// place from the pinned host pool -- the same bytes either way.
template <bool TIER>
__device__ __forceinline__ void issue_page(DecSmem& sm, const DecParams& p,
                                           int warp, int lane, int stage,
                                           int kh, int pt, int blk, int slot,
                                           int seq_len, int& n_valid_out) {
    const int n_valid = (pt >= 0) ? min(max(seq_len - pt * PAGE_T, 0), PAGE_T) : 0;
    blk = max(blk, 0);
    n_valid_out = n_valid;
    const int c = lane & 15, h = lane >> 4;
    const int64_t off = (int64_t)blk * p.stride_block + (int64_t)kh * p.stride_head +
                        8 * c;
    const __nv_bfloat16* ksrc = p.k_cache + off;
    const __nv_bfloat16* vsrc = p.v_cache + off;
    if constexpr (TIER) {
        if (slot >= 0)
            vsrc = p.v_hot + (int64_t)slot * p.hot_stride_block +
                   (int64_t)kh * p.stride_head + 8 * c;
    }
    const uint32_t kdst = smem_u32(&sm.wb[warp].k[stage][0][16 * c]);
    const uint32_t vdst = smem_u32(&sm.wb[warp].v[stage][0][16 * c]);
#pragma unroll
    for (int i = 0; i < PAGE_T / 2; ++i) {
        const int t = h + 2 * i;
        const int nb = (t < n_valid) ? 16 : 0;        // 0: zero-fill, nothing read
        const int64_t so = (int64_t)min(t, max(n_valid - 1, 0)) * p.stride_tok;
        cp_async16(kdst + t * ROWB, ksrc + so, nb);
        cp_async16(vdst + t * ROWB, vsrc + so, nb);
    }
    cp_async_commit();
}

// TMA variant of issue_page: lanes 0-3 each issue one box (K low / K high /
// V low / V high half of the head's 128 columns) of the page's 16 token rows.
// The whole block row range is copied; V rows past seq_len are cleared by the
// consumer and K rows past it only reach masked scores.
__device__ __forceinline__ void issue_page_tma(DecSmemT& sm, const DecParams& p,
                                               const CUtensorMap* tmk,
                                               const CUtensorMap* tmv, int warp,
                                               int lane, int stage, int kh, int pt,
                                               int blk, int seq_len,
                                               int& n_valid_out) {
    n_valid_out = (pt >= 0) ? min(max(seq_len - pt * PAGE_T, 0), PAGE_T) : 0;
    blk = max(blk, 0);
    uint64_t* bar = &sm.full[warp][stage];
    fence_proxy_async();
    if (lane == 0) mbar_expect_tx(bar, PAGE_TX);
    __syncwarp();
    if (lane < 4) {
        const int half = lane & 1;
        uint8_t* dst = (lane < 2) ? &sm.wb[warp].k[stage][half][0][0]
                                  : &sm.wb[warp].v[stage][half][0][0];
        tma_load_2d(dst, (lane < 2) ? tmk : tmv,
                    kh * (int)p.stride_head + 64 * half, blk * p.rows_per_block, bar);
    }
}

// CP: context parallel (cluster mode only): the partial exchange with the peer
// ranks is compiled in.
// TMA: K/V pages arrive by tiled tensor-map copies (cp.async.bulk.tensor.2d,
// completion on a per-warp mbarrier) instead of 16-byte cp.async.
template <bool G_HI, bool CLUSTER, bool CP, bool TMA, bool TIER = false>
__device__ __forceinline__ void decode_body(const DecParams& p, const CUtensorMap* tmk,
                                            const CUtensorMap* tmv) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    using Smem = typename std::conditional<TMA, DecSmemT, DecSmem>::type;
    // the swizzled tiles of the TMA variant sit on 1 KiB boundaries
    Smem& sm = *reinterpret_cast<Smem*>(
        TMA ? reinterpret_cast<uint8_t*>(
                  (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023))
            : smem_raw);

    const int sp = blockIdx.x, kh = blockIdx.y;
    const int r = p.row_order ? p.row_order[blockIdx.z] : (int)blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gid = lane >> 2, tig = lane & 3;
    const int G = p.G;
    const int64_t row = (int64_t)r * p.n_kv + kh;
    pdl_trigger();            // the next layer's scorer may start prefetching
    if constexpr (TMA) {
        if (lane == 0) {
            for (int s = 0; s < DSTAGES; ++s) mbar_init(&sm.full[warp][s], 1);
            mbar_fence_init();
        }
        __syncwarp();
    }
    // remote shared memory may be written once every CTA of the cluster runs;
    // this barrier costs nothing while the selector is still at work
    if (CLUSTER) cg::this_cluster().sync();
    const int seq_len = p.seq_lens[r];            // per-step constant
    pdl_wait();               // page tables / counts come from the selector

    // Cluster mode deals the list out round-robin over all warps of the cluster
    // (entry j -> CTA (j / DW) % CL, warp j % DW): which entries a warp reads
    // does not depend on the page count, so the count, the first window of
    // page-table entries and (one round trip later) their physical blocks are
    // fetched together.  Split mode gives a CTA a contiguous run of entries.
    int win_pt = -1, win_blk = 0, win_slot = -1;
    const int stride = CLUSTER ? DW * (int)gridDim.x : DW;
    if (CLUSTER) {
        const int j = sp * DW + warp + lane * stride;
        if (j < p.max_pages)
            win_pt = p.page_table ? __ldcg(&p.page_table[row * p.max_pages + j]) : j;
    }
    const int cnt = p.page_cnt ? __ldcg(&p.page_cnt[row])
                               : (max(seq_len, 0) + PAGE_T - 1) / PAGE_T;
    // V tier: what the host needs to keep the staging buffer useful
    auto tier_note = [&](int pt, int blk, int slot) {
        if (pt < 0) return;
        if (slot >= 0) {
            p.vt_ref[slot] = 1;
        } else if ((pt + 1) * PAGE_T <= seq_len) {      // complete pages only
            const int round = __ldcg(p.vt_epoch);
            if (atomicExch(&p.vt_pending[blk], round) != round) {
                const int idx = atomicAdd(p.vt_miss_cnt, 1);
                if (idx < p.vt_miss_cap) p.vt_miss[idx] = blk;
                else p.vt_pending[blk] = 0;  // not listed: may be noted again
            }
        }
    };
    if (CLUSTER) {
        win_blk = p.block_table[(int64_t)r * p.bt_stride + max(win_pt, 0)];
        if constexpr (TIER) {
            win_slot = p.v_map[max(win_blk, 0)];
            tier_note(win_pt, max(win_blk, 0), win_slot);
        }
    }
    int first, jend;
    if (CLUSTER) {
        // an empty share still takes part in the cluster barrier below
        first = sp * DW + warp;
        jend = cnt;
    } else {
        const int pps = max((cnt + p.split - 1) / p.split, p.pps_min);
        const int j0 = sp * pps;
        if (j0 >= cnt) return;                    // inactive split: no store
        first = j0 + warp;
        jend = min(j0 + pps, cnt);
    }
    const int n_mine = (first < jend) ? (jend - first + stride - 1) / stride : 0;
    int nv[DSTAGES] = {0, 0};
    // Page-table entry and physical block of the warp's pages, 32 at a time
    // (lane i holds entry i of the window), so that the two dependent index
    // loads are paid once per window instead of once per page.
    auto load_window = [&](int it0) {
        const int it = it0 + lane;
        win_pt = -1; win_blk = 0; win_slot = -1;
        if (it < n_mine) {
            const int j = first + it * stride;
            win_pt = p.page_table ? p.page_table[row * p.max_pages + j] : j;
            win_blk = p.block_table[(int64_t)r * p.bt_stride + max(win_pt, 0)];
            if constexpr (TIER) {
                win_slot = p.v_map[max(win_blk, 0)];
                tier_note(win_pt, max(win_blk, 0), win_slot);
            }
        }
    };
    auto issue_it = [&](int it) {
        const int pt = __shfl_sync(0xffffffffu, win_pt, it & 31);
        const int blk = __shfl_sync(0xffffffffu, win_blk, it & 31);
        if constexpr (TMA)
            issue_page_tma(sm, p, tmk, tmv, warp, lane, it % DSTAGES, kh, pt, blk,
                           seq_len, nv[it % DSTAGES]);
        else
            issue_page<TIER>(sm, p, warp, lane, it % DSTAGES, kh, pt, blk,
                             TIER ? __shfl_sync(0xffffffffu, win_slot, it & 31) : -1,
                             seq_len, nv[it % DSTAGES]);
    };
    if (!CLUSTER) load_window(0);
    for (int it = 0; it < DSTAGES && it < n_mine; ++it) issue_it(it);

    // ---- Q fragments (A operand), rows gid and gid+8 -------------------------
    uint32_t qa[8][4];
    {
        const __nv_bfloat16* q0 =
            p.q + (int64_t)r * p.q_stride_req + (int64_t)(kh * G) * HD;
        const bool live0 = gid < G, live1 = G_HI && (gid + 8 < G);
        const uint32_t* r0 = reinterpret_cast<const uint32_t*>(q0 + (int64_t)gid * HD);
        const uint32_t* r1 =
            reinterpret_cast<const uint32_t*>(q0 + (int64_t)(gid + 8) * HD);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            qa[ks][0] = live0 ? r0[8 * ks + tig] : 0u;
            qa[ks][1] = live1 ? r1[8 * ks + tig] : 0u;
            qa[ks][2] = live0 ? r0[8 * ks + 4 + tig] : 0u;
            qa[ks][3] = live1 ? r1[8 * ks + 4 + tig] : 0u;
        }
    }

    float acc[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    const float scale = p.scale;

    for (int it = 0; it < n_mine; ++it) {
        const int stage = it % DSTAGES;
        const int n_valid = nv[stage];
        if constexpr (TMA) {
            mbar_wait(&sm.full[warp][stage], (uint32_t)((it / DSTAGES) & 1), p.status);
            if (n_valid > 0 && n_valid < PAGE_T) {
                // rows past the sequence end hold whatever the block held before:
                // clear them in V (P is 0 there, but 0 x NaN is not)
                uint8_t* vt = reinterpret_cast<uint8_t*>(&sm.wb[warp].v[stage]);
                for (int i = lane; i < (PAGE_T - n_valid) * 16; i += 32) {
                    const int row = n_valid + (i >> 4), c = i & 15;
                    *reinterpret_cast<uint4*>(vt + (c >> 3) * HALF_TILE + row * 128 +
                                              (c & 7) * 16) = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }
        } else {
            // groups complete in order; at most the next page's is younger
            if (it + 1 < n_mine) cp_async_wait<1>(); else cp_async_wait<0>();
            __syncwarp();                           // every lane's copies landed
        }
        if (n_valid > 0) {
            const uint32_t kbase = smem_u32(&sm.wb[warp].k[stage]);
            const uint32_t vbase = smem_u32(&sm.wb[warp].v[stage]);
            // ---- S = Q K^T : two 16x8 token tiles ----------------------------
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
            {
                const int t = (lane & 7) + 8 * ((lane >> 4) & 1);
                const int pc = (lane >> 3) & 1;             // 16-byte piece parity
                const uint32_t a0 = TMA ? kbase + t * 128
                                        : kbase + t * ROWB + 16 * pc;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    uint32_t kb[4];
                    // swizzled tile: piece 2*(ks&3)+pc of half ks>>2, XOR row&7
                    ldmatrix_x4(kb, TMA ? a0 + (ks >> 2) * HALF_TILE +
                                              (((2 * (ks & 3) + pc) ^ (lane & 7)) << 4)
                                        : a0 + 32 * ks);
                    mma_bf16_k16(s0, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3],
                                 kb[0], kb[1]);
                    mma_bf16_k16(s1, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3],
                                 kb[2], kb[3]);
                }
            }
            // ---- scale, mask the tail of a partial page -----------------------
            const int ta = 2 * tig, tb = 2 * tig + 1;
            float x[8];        // [0..3] row gid: t = ta, tb, ta+8, tb+8; [4..7] row gid+8
            x[0] = (ta < n_valid) ? s0[0] * scale : -INFINITY;
            x[1] = (tb < n_valid) ? s0[1] * scale : -INFINITY;
            x[2] = (ta + 8 < n_valid) ? s1[0] * scale : -INFINITY;
            x[3] = (tb + 8 < n_valid) ? s1[1] * scale : -INFINITY;
            x[4] = (ta < n_valid) ? s0[2] * scale : -INFINITY;
            x[5] = (tb < n_valid) ? s0[3] * scale : -INFINITY;
            x[6] = (ta + 8 < n_valid) ? s1[2] * scale : -INFINITY;
            x[7] = (tb + 8 < n_valid) ? s1[3] * scale : -INFINITY;
            // ---- online softmax ----------------------------------------------
            float mx = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mn_lo = fmaxf(m_lo, mx);       // finite: token 0 is valid
            const float al_lo = __expf(m_lo - mn_lo);
            float pr[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) pr[i] = __expf(x[i] - mn_lo);
            l_lo = l_lo * al_lo + (pr[0] + pr[1] + pr[2] + pr[3]);
            m_lo = mn_lo;
            float al_hi = 1.f;
            if (G_HI) {
                float mh = fmaxf(fmaxf(x[4], x[5]), fmaxf(x[6], x[7]));
                mh = fmaxf(mh, __shfl_xor_sync(0xffffffffu, mh, 1));
                mh = fmaxf(mh, __shfl_xor_sync(0xffffffffu, mh, 2));
                const float mn_hi = fmaxf(m_hi, mh);
                al_hi = __expf(m_hi - mn_hi);
#pragma unroll
                for (int i = 4; i < 8; ++i) pr[i] = __expf(x[i] - mn_hi);
                l_hi = l_hi * al_hi + (pr[4] + pr[5] + pr[6] + pr[7]);
                m_hi = mn_hi;
            } else {
                pr[4] = pr[5] = pr[6] = pr[7] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                acc[i][0] *= al_lo; acc[i][1] *= al_lo;
                if (G_HI) { acc[i][2] *= al_hi; acc[i][3] *= al_hi; }
            }
            // ---- P in fp16 (A operand, k = 16 tokens); V bf16 -> fp16 on the fly.
            // Same arithmetic as the reference decode (fp16 P.V product with
            // fp32 accumulation, attention/decode.py:314) --------------------------
            uint32_t ph[4];
            ph[0] = pack_f16x2(pr[0], pr[1]);                // row gid,   t 0-7
            ph[1] = pack_f16x2(pr[4], pr[5]);                // row gid+8, t 0-7
            ph[2] = pack_f16x2(pr[2], pr[3]);                // row gid,   t 8-15
            ph[3] = pack_f16x2(pr[6], pr[7]);                // row gid+8, t 8-15
            // ---- O += P V ------------------------------------------------------
            {
                const int t = (lane & 7) + 8 * ((lane >> 3) & 1);
                const int pc = (lane >> 4) & 1;
                const uint32_t a0 = TMA ? vbase + t * 128
                                        : vbase + t * ROWB + 16 * pc;
#pragma unroll
                for (int dp = 0; dp < 8; ++dp) {
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, TMA ? a0 + (dp >> 2) * HALF_TILE +
                                                    (((2 * (dp & 3) + pc) ^ (lane & 7)) << 4)
                                              : a0 + 32 * dp);
#pragma unroll
                    for (int i = 0; i < 4; ++i) vb[i] = bf16x2_to_f16x2(vb[i]);
                    mma_f16_k16(acc[2 * dp], ph[0], ph[1], ph[2], ph[3], vb[0], vb[1]);
                    mma_f16_k16(acc[2 * dp + 1], ph[0], ph[1], ph[2], ph[3], vb[2], vb[3]);
                }
            }
        }
        __syncwarp();                               // stage fully consumed
        if (it + DSTAGES < n_mine) {
            if (((it + DSTAGES) & 31) == 0) load_window(it + DSTAGES);
            issue_it(it + DSTAGES);
        }
    }

    // ---- combine the warps of the CTA --------------------------------------------
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    if (G_HI) {
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    }
    __syncthreads();           // every warp's ring is idle: reuse it as fp32 scratch
    float* wacc = reinterpret_cast<float*>(&sm.wb[warp]);
    if (tig == 0) {
        sm.cm[warp][gid] = m_lo; sm.cl[warp][gid] = l_lo;
        sm.cm[warp][gid + 8] = G_HI ? m_hi : -INFINITY;
        sm.cl[warp][gid + 8] = G_HI ? l_hi : 0.f;
    }
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
        if (gid < G)
            *reinterpret_cast<float2*>(&wacc[gid * ACC_PITCH + 8 * nt + 2 * tig]) =
                make_float2(acc[nt][0], acc[nt][1]);
        if (G_HI)
            *reinterpret_cast<float2*>(
                &wacc[(gid + 8) * ACC_PITCH + 8 * nt + 2 * tig]) =
                make_float2(acc[nt][2], acc[nt][3]);
    }
    __syncthreads();

    if (!CLUSTER) {
        for (int e = tid; e < G * HD; e += DTHREADS) {
            const int g = e / HD, d = e % HD;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < DW; ++w) M = fmaxf(M, sm.cm[w][g]);
            float Lsum = 0.f, o = 0.f;
#pragma unroll
            for (int w = 0; w < DW; ++w) {
                const float lw = sm.cl[w][g];
                const float wt = (lw > 0.f) ? __expf(sm.cm[w][g] - M) : 0.f;
                Lsum += wt * lw;
                o += wt * reinterpret_cast<const float*>(&sm.wb[w])[g * ACC_PITCH + d];
            }
            const int64_t base = (row * p.split + sp) * G + g;
            p.acc_part[base * HD + d] = o;
            if (d == 0) { p.m_part[base] = M; p.l_part[base] = Lsum; }
        }
        return;
    }

    // ---- cluster mode: the CTA's (m, l, O) is pushed into the shared memory of
    // the CTAs that normalise it (CTA d owns output elements [d*per_e, (d+1)*per_e));
    // after one cluster barrier every CTA finishes its slice from local memory ----
    cg::cluster_group cluster = cg::this_cluster();
    const int CL = (int)gridDim.x;
    const int n_el = G * HD;
    const int per_e = (n_el + CL - 1) / CL;
    for (int e = tid; e < n_el; e += DTHREADS) {
        const int g = e / HD, d = e % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DW; ++w) M = fmaxf(M, sm.cm[w][g]);
        float Lsum = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < DW; ++w) {
            const float lw = sm.cl[w][g];
            const float wt = (lw > 0.f) ? __expf(sm.cm[w][g] - M) : 0.f;
            Lsum += wt * lw;
            o += wt * reinterpret_cast<const float*>(&sm.wb[w])[g * ACC_PITCH + d];
        }
        const int dst = e / per_e;
        cluster.map_shared_rank(sm.xacc, dst)[sp * per_e + (e - dst * per_e)] = o;
        if (d < CL) {                      // lane d tells CTA d this head's (m, l)
            cluster.map_shared_rank(&sm.xm[sp][g], d)[0] = M;
            cluster.map_shared_rank(&sm.xl[sp][g], d)[0] = Lsum;
        }
    }
    cluster.sync();                               // every CTA's pushes have landed
    for (int e = sp * per_e + tid; e < min((sp + 1) * per_e, n_el); e += DTHREADS) {
        const int g = e / HD, dd = e % HD;
        float mw[MAX_DCL], lw[MAX_DCL];
        float M = -INFINITY;
#pragma unroll
        for (int c = 0; c < MAX_DCL; ++c) {
            mw[c] = (c < CL) ? sm.xm[c][g] : -INFINITY;
            lw[c] = (c < CL) ? sm.xl[c][g] : 0.f;
            M = fmaxf(M, mw[c]);
        }
        float Lsum = 0.f, o = 0.f;
#pragma unroll
        for (int c = 0; c < MAX_DCL; ++c) {
            if (c < CL) {
                const float wt = (lw[c] > 0.f) ? __expf(mw[c] - M) : 0.f;
                Lsum += wt * lw[c];
                o += wt * sm.xacc[c * per_e + (e - sp * per_e)];
            }
        }
        if constexpr (CP) cp_merge_element(p.cp, kh, G, g, dd, M, Lsum, o, p.status);
        const float val = (Lsum > 0.f) ? o / Lsum : 0.f;
        p.out[(int64_t)r * p.out_stride_req + (int64_t)(kh * G + g) * HD + dd] =
            __float2bfloat16_rn(val);
    }
}

template <bool G_HI, bool CLUSTER, bool CP = false>
__global__ void __launch_bounds__(DTHREADS)
decode_kernel(const DecParams p) {
    decode_body<G_HI, CLUSTER, CP, false>(p, nullptr, nullptr);
}

// fused (cluster) decode whose V pages come from the tier (staging buffer in
// device memory, pinned host pool on a miss)
template <bool G_HI>
__global__ void __launch_bounds__(DTHREADS)
decode_vtier_kernel(const DecParams p) {
    decode_body<G_HI, true, false, false, true>(p, nullptr, nullptr);
}

// fused (cluster) decode with the pages staged by tensor-map copies
template <bool G_HI>
__global__ void __launch_bounds__(DTHREADS)
decode_tma_kernel(const __grid_constant__ CUtensorMap tmk,
                  const __grid_constant__ CUtensorMap tmv, const DecParams p) {
    decode_body<G_HI, true, false, true>(p, &tmk, &tmv);
}

struct MergeParams {
    const float* m_part;
    const float* l_part;
    const float* acc_part;
    const int32_t* page_cnt;       // or nullptr with seq_lens set (dense)
    const int32_t* seq_lens;
    __nv_bfloat16* out;
    int64_t out_stride_req;
    int n_kv, G, split, pps_min;
    int n_groups;                  // partial sets (one per rank when gathered)
    int64_t group_stride;          // floats between two sets (m, l and acc alike)
    int all_splits;                // read every split (empty ones carry l = 0)
};

// grid (n_kv*G, n_req), 128 threads.  Warp w merges splits w, w+4, ... online
// (lane l owns channels 4l..4l+3, float4 loads); the 4 warps meet in shared
// memory.  Only the ACTIVE splits are read.
__global__ void __launch_bounds__(HD) merge_kernel(const MergeParams p) {
    __shared__ float sM[4], sL[4];
    __shared__ __align__(16) float sO[4][HD];
    const int h = blockIdx.x, r = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kh = h / p.G, g = h % p.G;
    const int64_t row = (int64_t)r * p.n_kv + kh;
    int n_act = p.split;
    if (!p.all_splits) {
        const int cnt = p.page_cnt ? p.page_cnt[row]
                                   : (max(p.seq_lens[r], 0) + PAGE_T - 1) / PAGE_T;
        const int pps = max((cnt + p.split - 1) / p.split, p.pps_min);
        n_act = (cnt + pps - 1) / pps;
    }
    const int n_tot = n_act * max(p.n_groups, 1);
    const int64_t base = row * p.split * p.G + g;
    float M = -INFINITY, Ls = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int e = warp; e < n_tot; e += 4) {
        const int grp = e / n_act, s = e - grp * n_act;
        const int64_t i = base + (int64_t)s * p.G;
        const float* mp = p.m_part + grp * p.group_stride;
        const float* lp = p.l_part + grp * p.group_stride;
        const float* ap = p.acc_part + grp * p.group_stride;
        const float m = mp[i], l = lp[i];
        const float4 a = *reinterpret_cast<const float4*>(&ap[i * HD + 4 * lane]);
        if (l > 0.f) {
            const float Mn = fmaxf(M, m);
            const float ao = __expf(M - Mn), w = __expf(m - Mn);
            Ls = Ls * ao + w * l;
            o.x = o.x * ao + w * a.x; o.y = o.y * ao + w * a.y;
            o.z = o.z * ao + w * a.z; o.w = o.w * ao + w * a.w;
            M = Mn;
        }
    }
    if (lane == 0) { sM[warp] = M; sL[warp] = Ls; }
    *reinterpret_cast<float4*>(&sO[warp][4 * lane]) = o;
    __syncthreads();
    float Mt = fmaxf(fmaxf(sM[0], sM[1]), fmaxf(sM[2], sM[3]));
    float Lt = 0.f, ot = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const float wt = (sL[w] > 0.f) ? __expf(sM[w] - Mt) : 0.f;
        Lt += wt * sL[w];
        ot += wt * sO[w][tid];
    }
    const float val = (Lt > 0.f) ? ot / Lt : 0.f;
    p.out[(int64_t)r * p.out_stride_req + (int64_t)h * HD + tid] =
        __float2bfloat16_rn(val);
}

int check_geometry(const char* who, int G, int head_dim, int page) {
    LOCKS_REQUIRE(head_dim == HD && page == PAGE_T, LOCKS_ERR_GEOMETRY,
                  "%s: supports head_dim 128 / page 16, got %d / %d", who,
                  head_dim, page);
    LOCKS_REQUIRE(G >= 1 && G <= 16, LOCKS_ERR_GEOMETRY,
                  "%s: supports 1 <= G <= 16, got %d", who, G);
    return LOCKS_OK;
}

// cluster size of the fused decode: as many CTAs as fit in ONE wave (a CTA's
// rings take more than half an SM's shared memory, so one CTA per SM), a power
// of two, at most 8 (the portable cluster limit) -- or, where the caller's kernel
// allows it (`fit16` = how many 16-CTA clusters of it the device holds at once,
// 0 = not allowed), 16 when every row's cluster fits at once: the launch is a
// latency chain whose page loop shortens with every CTA added (config 1, 137
// pages per row: 15.9 / 10.7 / 8.2 us with 2 / 4 / 8 CTAs per row)
int fused_cluster_size(int n_req, int n_kv, int fit16 = 0) {
    const int want = sm_count() / max(1, n_req * n_kv);
    int cl = 1;
    while (cl * 2 <= want && cl < 8) cl *= 2;
    // (a few rows only: 16-CTA clusters each take 16 SMs of one GPC)
    if (cl == 8 && want >= 32 && n_req * n_kv <= fit16) cl = MAX_DCL;
    return cl;
}

int launch_decode(const char* who, const DecParams& p, int n_req, int grid_x,
                  cudaStream_t s) {
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    const int smem = (int)sizeof(DecSmem);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaFuncSetAttribute(decode_kernel<false, false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        cudaFuncSetAttribute(decode_kernel<true, false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        cudaFuncSetAttribute(decode_kernel<false, true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        cudaFuncSetAttribute(decode_kernel<true, true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        cudaFuncSetAttribute(decode_kernel<false, true, true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        cudaFuncSetAttribute(decode_kernel<true, true, true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        attr_done[dev] = true;
    }
    dim3 grid(grid_x, p.n_kv, n_req);
    if (!p.fused) {
        if (p.G > 8)
            decode_kernel<true, false><<<grid, DTHREADS, smem, s>>>(p);
        else
            decode_kernel<false, false><<<grid, DTHREADS, smem, s>>>(p);
        return check_launch(who);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(DTHREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = grid_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t e;
    if (p.cp.world > 0)
        e = (p.G > 8) ? cudaLaunchKernelEx(&cfg, decode_kernel<true, true, true>, p)
                      : cudaLaunchKernelEx(&cfg, decode_kernel<false, true, true>, p);
    else
        e = (p.G > 8) ? cudaLaunchKernelEx(&cfg, decode_kernel<true, true>, p)
                      : cudaLaunchKernelEx(&cfg, decode_kernel<false, true>, p);
    if (e != cudaSuccess)
        return fail(LOCKS_ERR_LAUNCH, "%s: %s", who, cudaGetErrorString(e));
    return check_launch(who);
}

int check_kv(const char* who, const void* q, const void* k, const void* v,
             int64_t q_stride_req, int64_t sb, int64_t st, int64_t sh) {
    LOCKS_REQUIRE((reinterpret_cast<uintptr_t>(k) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(v) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(q) & 3) == 0,
                  LOCKS_ERR_ARG, "%s: k/v caches must be 16-byte aligned", who);
    LOCKS_REQUIRE(sb % 8 == 0 && st % 8 == 0 && sh % 8 == 0 &&
                      q_stride_req % 2 == 0,
                  LOCKS_ERR_ARG,
                  "%s: cache strides must be multiples of 8 elements (16 bytes)",
                  who);
    return LOCKS_OK;
}

}  // namespace
}  // namespace locks

using namespace locks;


extern "C" int locks_decode_split(
    const void* q, int64_t q_stride_req, const void* k_cache,
    const void* v_cache, int64_t kv_stride_block, int64_t kv_stride_tok,
    int64_t kv_stride_head, const int32_t* block_table, int64_t bt_stride,
    const int32_t* page_table, const int32_t* page_cnt, const int32_t* seq_lens,
    float* m_part, float* l_part, float* acc_part, int n_req, int n_kv, int G,
    int head_dim, int page, int max_pages, int split, int pps_min, float scale,
    int* status, locks_stream_t stream) {
    LOCKS_REQUIRE(q && k_cache && v_cache && block_table && page_table &&
                      page_cnt && seq_lens && m_part && l_part && acc_part,
                  LOCKS_ERR_ARG, "locks_decode_split: null pointer argument");
    int rc = check_geometry("locks_decode_split", G, head_dim, page);
    if (rc) return rc;
    rc = check_kv("locks_decode_split", q, k_cache, v_cache, q_stride_req,
                  kv_stride_block, kv_stride_tok, kv_stride_head);
    if (rc) return rc;
    LOCKS_REQUIRE(n_req >= 0 && n_req <= 65535 && n_kv >= 1 && n_kv <= 65535 &&
                      split >= 1 && pps_min >= 1 && max_pages >= 1,
                  LOCKS_ERR_ARG, "locks_decode_split: bad size argument");
    if (n_req == 0) return LOCKS_OK;
    DecParams p{};
    p.q = static_cast<const __nv_bfloat16*>(q); p.q_stride_req = q_stride_req;
    p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
    p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
    p.stride_block = kv_stride_block; p.stride_tok = kv_stride_tok;
    p.stride_head = kv_stride_head;
    p.block_table = block_table; p.bt_stride = bt_stride;
    p.page_table = page_table; p.page_cnt = page_cnt; p.seq_lens = seq_lens;
    p.m_part = m_part; p.l_part = l_part; p.acc_part = acc_part;
    p.n_kv = n_kv; p.G = G; p.max_pages = max_pages; p.split = split;
    p.pps_min = pps_min; p.fused = 0; p.scale = scale; p.status = status;
    return launch_decode("locks_decode_split", p, n_req, split,
                         static_cast<cudaStream_t>(stream));
}

extern "C" int locks_merge_splits(
    const float* m_part, const float* l_part, const float* acc_part,
    const int32_t* page_cnt, void* out, int64_t out_stride_req, int n_req,
    int n_kv, int G, int head_dim, int split, int pps_min,
    locks_stream_t stream) {
    LOCKS_REQUIRE(m_part && l_part && acc_part && page_cnt && out, LOCKS_ERR_ARG,
                  "locks_merge_splits: null pointer argument");
    LOCKS_REQUIRE(head_dim == HD, LOCKS_ERR_GEOMETRY,
                  "locks_merge_splits: supports head_dim 128, got %d", head_dim);
    LOCKS_REQUIRE(n_req >= 0 && n_req <= 65535 && n_kv >= 1 && G >= 1 &&
                      split >= 1 && pps_min >= 1,
                  LOCKS_ERR_ARG, "locks_merge_splits: bad size argument");
    if (n_req == 0) return LOCKS_OK;
    MergeParams p{};
    p.m_part = m_part; p.l_part = l_part; p.acc_part = acc_part;
    p.page_cnt = page_cnt; p.seq_lens = nullptr;
    p.out = static_cast<__nv_bfloat16*>(out); p.out_stride_req = out_stride_req;
    p.n_kv = n_kv; p.G = G; p.split = split; p.pps_min = pps_min;
    p.n_groups = 1; p.group_stride = 0; p.all_splits = 0;
    merge_kernel<<<dim3(n_kv * G, n_req), HD, 0,
                   static_cast<cudaStream_t>(stream)>>>(p);
    return check_launch("locks_merge_splits");
}

extern "C" int locks_merge_gathered(
    const float* packs, int64_t pack_stride, int n_groups, void* out,
    int64_t out_stride_req, int n_req, int n_kv, int G, int head_dim, int split,
    locks_stream_t stream) {
    LOCKS_REQUIRE(packs && out, LOCKS_ERR_ARG,
                  "locks_merge_gathered: null pointer argument");
    LOCKS_REQUIRE(head_dim == HD, LOCKS_ERR_GEOMETRY,
                  "locks_merge_gathered: supports head_dim 128, got %d", head_dim);
    const int64_t n_ml = (int64_t)n_req * n_kv * split * G;
    LOCKS_REQUIRE(n_req >= 0 && n_req <= 65535 && n_kv >= 1 && G >= 1 &&
                      split >= 1 && n_groups >= 1 &&
                      pack_stride >= n_ml * (2 + HD) && (pack_stride % 4) == 0 &&
                      (n_ml % 2) == 0 &&
                      (reinterpret_cast<uintptr_t>(packs) & 15) == 0,
                  LOCKS_ERR_ARG,
                  "locks_merge_gathered: bad size, stride or alignment");
    if (n_req == 0) return LOCKS_OK;
    MergeParams p{};
    p.m_part = packs; p.l_part = packs + n_ml; p.acc_part = packs + 2 * n_ml;
    p.page_cnt = nullptr; p.seq_lens = nullptr;
    p.out = static_cast<__nv_bfloat16*>(out); p.out_stride_req = out_stride_req;
    p.n_kv = n_kv; p.G = G; p.split = split; p.pps_min = 1;
    p.n_groups = n_groups; p.group_stride = pack_stride; p.all_splits = 1;
    merge_kernel<<<dim3(n_kv * G, n_req), HD, 0,
                   static_cast<cudaStream_t>(stream)>>>(p);
    return check_launch("locks_merge_gathered");
}

static int decode_fused_impl(
    const int32_t* row_order,
    const void* q, int64_t q_stride_req, const void* k_cache,
    const void* v_cache, int64_t kv_stride_block, int64_t kv_stride_tok,
    int64_t kv_stride_head, const int32_t* block_table, int64_t bt_stride,
    const int32_t* page_table, const int32_t* page_cnt, const int32_t* seq_lens,
    void* out, int64_t out_stride_req, int n_req, int n_kv, int G, int head_dim,
    int page, int max_pages, float scale, int* status, locks_stream_t stream) {
    LOCKS_REQUIRE(q && k_cache && v_cache && block_table && page_table &&
                      page_cnt && seq_lens && out,
                  LOCKS_ERR_ARG, "locks_decode_fused: null pointer argument");
    int rc = check_geometry("locks_decode_fused", G, head_dim, page);
    if (rc) return rc;
    rc = check_kv("locks_decode_fused", q, k_cache, v_cache, q_stride_req,
                  kv_stride_block, kv_stride_tok, kv_stride_head);
    if (rc) return rc;
    LOCKS_REQUIRE(n_req >= 0 && n_req <= 65535 && n_kv >= 1 && n_kv <= 65535 &&
                      max_pages >= 1,
                  LOCKS_ERR_ARG, "locks_decode_fused: bad size argument");
    if (n_req == 0) return LOCKS_OK;
    DecParams p{};
    p.q = static_cast<const __nv_bfloat16*>(q); p.q_stride_req = q_stride_req;
    p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
    p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
    p.stride_block = kv_stride_block; p.stride_tok = kv_stride_tok;
    p.stride_head = kv_stride_head;
    p.block_table = block_table; p.bt_stride = bt_stride;
    p.page_table = page_table; p.page_cnt = page_cnt; p.seq_lens = seq_lens;
    p.out = static_cast<__nv_bfloat16*>(out); p.out_stride_req = out_stride_req;
    p.n_kv = n_kv; p.G = G; p.max_pages = max_pages; p.split = 1;
    p.pps_min = 1; p.fused = 1; p.scale = scale; p.status = status;
    p.row_order = row_order;
    // 16-CTA clusters (non-portable size) where all of them fit at once
    static int fit16[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    int fit = 0;
    if (dev >= 0 && dev < 64 && sm_count() / max(1, n_req * n_kv) >= 32) {
        if (fit16[dev] == 0) {
            cudaFuncSetAttribute(decode_kernel<false, true>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)sizeof(DecSmem));
            cudaFuncSetAttribute(decode_kernel<false, true>,
                                 cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            cudaFuncSetAttribute(decode_kernel<true, true>,
                                 cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            fit16[dev] = max(1, max_active_clusters(decode_kernel<false, true>, MAX_DCL,
                                                    DTHREADS, (int)sizeof(DecSmem)));
        }
        fit = fit16[dev];
    }
    return launch_decode("locks_decode_fused", p, n_req,
                         fused_cluster_size(n_req, n_kv, fit),
                         static_cast<cudaStream_t>(stream));
}

extern "C" int locks_decode_fused_tma(
    const void* q, int64_t q_stride_req, const void* k_cache,
    const void* v_cache, int64_t kv_stride_block, int64_t kv_stride_tok,
    int64_t kv_stride_head, const int32_t* block_table, int64_t bt_stride,
    const int32_t* page_table, const int32_t* page_cnt, const int32_t* seq_lens,
    void* out, int64_t out_stride_req, int n_req, int n_kv, int G, int head_dim,
    int page, int max_pages, int num_blocks, float scale, int* status,
    locks_stream_t stream) {
    LOCKS_REQUIRE(q && k_cache && v_cache && block_table && page_table &&
                      page_cnt && seq_lens && out,
                  LOCKS_ERR_ARG, "locks_decode_fused_tma: null pointer argument");
    int rc = check_geometry("locks_decode_fused_tma", G, head_dim, page);
    if (rc) return rc;
    rc = check_kv("locks_decode_fused_tma", q, k_cache, v_cache, q_stride_req,
                  kv_stride_block, kv_stride_tok, kv_stride_head);
    if (rc) return rc;
    LOCKS_REQUIRE(n_req >= 0 && n_req <= 65535 && n_kv >= 1 && n_kv <= 65535 &&
                      max_pages >= 1 && num_blocks >= 1,
                  LOCKS_ERR_ARG, "locks_decode_fused_tma: bad size argument");
    // the tensor maps see each plane as one matrix of token rows, kv_stride_tok
    // apart, whose boxes start at row blk * (block stride / token stride) and
    // column kh * head stride: a block's 16 rows evenly spaced, the block stride
    // a whole number of rows (16 for separate planes, 32 for K and V interleaved
    // per block), a head's 128 columns contiguous and inside the row
    LOCKS_REQUIRE(kv_stride_tok > 0 && kv_stride_block % kv_stride_tok == 0 &&
                      kv_stride_block / kv_stride_tok >= PAGE_T &&
                      kv_stride_head >= HD &&
                      (int64_t)(n_kv - 1) * kv_stride_head + HD <= kv_stride_tok &&
                      kv_stride_head % 64 == 0 &&
                      (int64_t)num_blocks * (kv_stride_block / kv_stride_tok) <
                          (int64_t)1 << 31,
                  LOCKS_ERR_GEOMETRY,
                  "locks_decode_fused_tma: the cache planes must be (num_blocks, 16, "
                  "n_kv, 128) with a block stride that is a multiple of the token "
                  "stride (got %lld, %lld, %lld); use locks_decode_fused for other "
                  "layouts",
                  (long long)kv_stride_block, (long long)kv_stride_tok,
                  (long long)kv_stride_head);
    const int64_t rpb = kv_stride_block / kv_stride_tok;
    const uint64_t rows = (uint64_t)(num_blocks - 1) * rpb + PAGE_T;
    if (n_req == 0) return LOCKS_OK;
    CUtensorMap tmk, tmv;
    CUresult cr = encode_bf16_rows_sw128(&tmk, k_cache, (uint64_t)kv_stride_tok, rows,
                                         (uint64_t)kv_stride_tok, PAGE_T);
    if (cr == CUDA_SUCCESS)
        cr = encode_bf16_rows_sw128(&tmv, v_cache, (uint64_t)kv_stride_tok, rows,
                                    (uint64_t)kv_stride_tok, PAGE_T);
    LOCKS_REQUIRE(cr == CUDA_SUCCESS, LOCKS_ERR_LAUNCH,
                  "locks_decode_fused_tma: cuTensorMapEncodeTiled failed (%d)", (int)cr);
    DecParams p{};
    p.q = static_cast<const __nv_bfloat16*>(q); p.q_stride_req = q_stride_req;
    p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
    p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
    p.stride_block = kv_stride_block; p.stride_tok = kv_stride_tok;
    p.stride_head = kv_stride_head;
    p.block_table = block_table; p.bt_stride = bt_stride;
    p.page_table = page_table; p.page_cnt = page_cnt; p.seq_lens = seq_lens;
    p.out = static_cast<__nv_bfloat16*>(out); p.out_stride_req = out_stride_req;
    p.n_kv = n_kv; p.G = G; p.max_pages = max_pages; p.split = 1;
    p.pps_min = 1; p.fused = 1; p.scale = scale; p.status = status;
    p.rows_per_block = (int)rpb;

    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    const int smem = (int)sizeof(DecSmemT) + 1024;     // room to align to 1 KiB
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaFuncSetAttribute(decode_tma_kernel<false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        cudaFuncSetAttribute(decode_tma_kernel<true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        attr_done[dev] = true;
    }
    const int cl = fused_cluster_size(n_req, n_kv);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cl, n_kv, n_req);
    cfg.blockDim = dim3(DTHREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cl;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    const cudaError_t e =
        (G > 8) ? cudaLaunchKernelEx(&cfg, decode_tma_kernel<true>, tmk, tmv, p)
                : cudaLaunchKernelEx(&cfg, decode_tma_kernel<false>, tmk, tmv, p);
    if (e != cudaSuccess)
        return fail(LOCKS_ERR_LAUNCH, "locks_decode_fused_tma: %s",
                    cudaGetErrorString(e));
    return check_launch("locks_decode_fused_tma");
}

extern "C" int locks_decode_fused(
    const void* q, int64_t q_stride_req, const void* k_cache,
    const void* v_cache, int64_t kv_stride_block, int64_t kv_stride_tok,
    int64_t kv_stride_head, const int32_t* block_table, int64_t bt_stride,
    const int32_t* page_table, const int32_t* page_cnt, const int32_t* seq_lens,
    void* out, int64_t out_stride_req, int n_req, int n_kv, int G, int head_dim,
    int page, int max_pages, float scale, int* status, locks_stream_t stream) {
    return decode_fused_impl(nullptr, q, q_stride_req, k_cache, v_cache,
                             kv_stride_block, kv_stride_tok, kv_stride_head,
                             block_table, bt_stride, page_table, page_cnt, seq_lens,
                             out, out_stride_req, n_req, n_kv, G, head_dim, page,
                             max_pages, scale, status, stream);
}

extern "C" int locks_decode_fused_rows(
    const void* q, int64_t q_stride_req, const void* k_cache,
    const void* v_cache, int64_t kv_stride_block, int64_t kv_stride_tok,
    int64_t kv_stride_head, const int32_t* block_table, int64_t bt_stride,
    const int32_t* page_table, const int32_t* page_cnt, const int32_t* seq_lens,
    void* out, int64_t out_stride_req, int n_req, int n_kv, int G, int head_dim,
    int page, int max_pages, const int32_t* row_order, float scale, int* status,
    locks_stream_t stream) {
    return decode_fused_impl(row_order, q, q_stride_req, k_cache, v_cache,
                             kv_stride_block, kv_stride_tok, kv_stride_head,
                             block_table, bt_stride, page_table, page_cnt, seq_lens,
                             out, out_stride_req, n_req, n_kv, G, head_dim, page,
                             max_pages, scale, status, stream);
}

extern "C" int locks_decode_fused_vtier(
    const void* q, int64_t q_stride_req, const void* k_cache, const void* v_host,
    int64_t kv_stride_block, int64_t kv_stride_tok, int64_t kv_stride_head,
    const void* v_hot, int64_t hot_stride_block, const int32_t* v_map,
    uint8_t* slot_ref, int32_t* pending, int32_t* miss_list, int32_t* miss_cnt,
    int miss_cap, const int32_t* note_round, const int32_t* block_table,
    int64_t bt_stride,
    const int32_t* page_table, const int32_t* page_cnt, const int32_t* seq_lens,
    void* out, int64_t out_stride_req, int n_req, int n_kv, int G, int head_dim,
    int page, int max_pages, float scale, int* status, locks_stream_t stream) {
    LOCKS_REQUIRE(q && k_cache && v_host && v_hot && v_map && slot_ref && pending &&
                      miss_list && miss_cnt && note_round && block_table &&
                      page_table && page_cnt && seq_lens && out,
                  LOCKS_ERR_ARG, "locks_decode_fused_vtier: null pointer argument");
    int rc = check_geometry("locks_decode_fused_vtier", G, head_dim, page);
    if (rc) return rc;
    rc = check_kv("locks_decode_fused_vtier", q, k_cache, v_host, q_stride_req,
                  kv_stride_block, kv_stride_tok, kv_stride_head);
    if (rc) return rc;
    LOCKS_REQUIRE((reinterpret_cast<uintptr_t>(v_hot) & 15) == 0 &&
                      hot_stride_block % 8 == 0 && miss_cap >= 0,
                  LOCKS_ERR_ARG,
                  "locks_decode_fused_vtier: the staging buffer must be 16-byte "
                  "aligned with a slot stride that is a multiple of 8 elements");
    LOCKS_REQUIRE(n_req >= 0 && n_req <= 65535 && n_kv >= 1 && n_kv <= 65535 &&
                      max_pages >= 1,
                  LOCKS_ERR_ARG, "locks_decode_fused_vtier: bad size argument");
    if (n_req == 0) return LOCKS_OK;
    DecParams p{};
    p.q = static_cast<const __nv_bfloat16*>(q); p.q_stride_req = q_stride_req;
    p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
    p.v_cache = static_cast<const __nv_bfloat16*>(v_host);
    p.v_hot = static_cast<const __nv_bfloat16*>(v_hot);
    p.v_map = v_map; p.hot_stride_block = hot_stride_block;
    p.vt_ref = slot_ref; p.vt_pending = pending; p.vt_miss = miss_list;
    p.vt_miss_cnt = miss_cnt; p.vt_miss_cap = miss_cap; p.vt_epoch = note_round;
    p.stride_block = kv_stride_block; p.stride_tok = kv_stride_tok;
    p.stride_head = kv_stride_head;
    p.block_table = block_table; p.bt_stride = bt_stride;
    p.page_table = page_table; p.page_cnt = page_cnt; p.seq_lens = seq_lens;
    p.out = static_cast<__nv_bfloat16*>(out); p.out_stride_req = out_stride_req;
    p.n_kv = n_kv; p.G = G; p.max_pages = max_pages; p.split = 1;
    p.pps_min = 1; p.fused = 1; p.scale = scale; p.status = status;

    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    const int smem = (int)sizeof(DecSmem);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaFuncSetAttribute(decode_vtier_kernel<false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        cudaFuncSetAttribute(decode_vtier_kernel<true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        attr_done[dev] = true;
    }
    const int cl = fused_cluster_size(n_req, n_kv);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cl, n_kv, n_req);
    cfg.blockDim = dim3(DTHREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cl;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    const cudaError_t e = (G > 8) ? cudaLaunchKernelEx(&cfg, decode_vtier_kernel<true>, p)
                                  : cudaLaunchKernelEx(&cfg, decode_vtier_kernel<false>, p);
    if (e != cudaSuccess)
        return fail(LOCKS_ERR_LAUNCH, "locks_decode_fused_vtier: %s",
                    cudaGetErrorString(e));
    return check_launch("locks_decode_fused_vtier");
}

extern "C" int locks_decode_fused_cp(
    const void* q, int64_t q_stride_req, const void* k_cache,
    const void* v_cache, int64_t kv_stride_block, int64_t kv_stride_tok,
    int64_t kv_stride_head, const int32_t* block_table, int64_t bt_stride,
    const int32_t* page_table, const int32_t* page_cnt, const int32_t* seq_lens,
    void* out, int64_t out_stride_req, int n_kv, int G, int head_dim, int page,
    int max_pages, float scale, const locks_cp_link_t* link, int* status,
    locks_stream_t stream) {
    LOCKS_REQUIRE(q && k_cache && v_cache && block_table && page_table &&
                      page_cnt && seq_lens && out && link,
                  LOCKS_ERR_ARG, "locks_decode_fused_cp: null pointer argument");
    int rc = check_geometry("locks_decode_fused_cp", G, head_dim, page);
    if (rc) return rc;
    rc = check_kv("locks_decode_fused_cp", q, k_cache, v_cache, q_stride_req,
                  kv_stride_block, kv_stride_tok, kv_stride_head);
    if (rc) return rc;
    LOCKS_REQUIRE(n_kv >= 1 && n_kv <= 65535 && max_pages >= 1, LOCKS_ERR_ARG,
                  "locks_decode_fused_cp: bad size argument");
    DecParams p{};
    rc = cp_link_fill(p.cp, link, n_kv, G, "locks_decode_fused_cp");
    if (rc) return rc;
    p.q = static_cast<const __nv_bfloat16*>(q); p.q_stride_req = q_stride_req;
    p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
    p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
    p.stride_block = kv_stride_block; p.stride_tok = kv_stride_tok;
    p.stride_head = kv_stride_head;
    p.block_table = block_table; p.bt_stride = bt_stride;
    p.page_table = page_table; p.page_cnt = page_cnt; p.seq_lens = seq_lens;
    p.out = static_cast<__nv_bfloat16*>(out); p.out_stride_req = out_stride_req;
    p.n_kv = n_kv; p.G = G; p.max_pages = max_pages; p.split = 1;
    p.pps_min = 1; p.fused = 1; p.scale = scale; p.status = status;
    return launch_decode("locks_decode_fused_cp", p, 1, fused_cluster_size(1, n_kv),
                         static_cast<cudaStream_t>(stream));
}

extern "C" int locks_dense_decode(
    const void* q, int64_t q_stride_req, const void* k_cache,
    const void* v_cache, int64_t kv_stride_block, int64_t kv_stride_tok,
    int64_t kv_stride_head, const int32_t* block_table, int64_t bt_stride,
    const int32_t* seq_lens, float* m_part, float* l_part, float* acc_part,
    void* out, int64_t out_stride_req, int n_req, int n_kv, int G, int head_dim,
    int page, int split, float scale, int* status, locks_stream_t stream) {
    LOCKS_REQUIRE(q && k_cache && v_cache && block_table && seq_lens && m_part &&
                      l_part && acc_part && out,
                  LOCKS_ERR_ARG, "locks_dense_decode: null pointer argument");
    int rc = check_geometry("locks_dense_decode", G, head_dim, page);
    if (rc) return rc;
    rc = check_kv("locks_dense_decode", q, k_cache, v_cache, q_stride_req,
                  kv_stride_block, kv_stride_tok, kv_stride_head);
    if (rc) return rc;
    LOCKS_REQUIRE(n_req >= 0 && n_req <= 65535 && n_kv >= 1 && n_kv <= 65535 &&
                      split >= 1 && split <= 65535,
                  LOCKS_ERR_ARG, "locks_dense_decode: bad size argument");
    if (n_req == 0) return LOCKS_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DecParams p{};
    p.q = static_cast<const __nv_bfloat16*>(q); p.q_stride_req = q_stride_req;
    p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
    p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
    p.stride_block = kv_stride_block; p.stride_tok = kv_stride_tok;
    p.stride_head = kv_stride_head;
    p.block_table = block_table; p.bt_stride = bt_stride;
    p.page_table = nullptr; p.page_cnt = nullptr; p.seq_lens = seq_lens;
    p.m_part = m_part; p.l_part = l_part; p.acc_part = acc_part;
    p.n_kv = n_kv; p.G = G; p.max_pages = 0; p.split = split; p.pps_min = 1;
    p.fused = 0; p.scale = scale; p.status = status;
    rc = launch_decode("locks_dense_decode", p, n_req, split, s);
    if (rc) return rc;
    MergeParams m{};
    m.m_part = m_part; m.l_part = l_part; m.acc_part = acc_part;
    m.page_cnt = nullptr; m.seq_lens = seq_lens;
    m.out = static_cast<__nv_bfloat16*>(out); m.out_stride_req = out_stride_req;
    m.n_kv = n_kv; m.G = G; m.split = split; m.pps_min = 1;
    merge_kernel<<<dim3(n_kv * G, n_req), HD, 0, s>>>(m);
    return check_launch("locks_dense_decode(merge)");
}

// --------------------------------------------------------------------------- //
// Split decode + merge for callers that must not allocate                      //
// --------------------------------------------------------------------------- //
// The split partials (m, l, acc) normally live in buffers the caller allocates
// once.  Some callers cannot do that: a plugin that is handed a stream inside a
// memory-pool-managed region where cudaMalloc would synchronise the device, or
// a host language binding that may only pass pointers it was given.  For them
// the partials live in the fixed array below.  It is part of the library image:
// every GPU that loads the library holds these bytes until the process exits.
namespace locks {
namespace {
constexpr int NOALLOC_MAX_ROWS = LOCKS_NOALLOC_MAX_ROWS;   // n_req*n_kv*split*G
constexpr size_t NOALLOC_FLOATS = (size_t)NOALLOC_MAX_ROWS * (HD + 2);
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_FLOATS];
// device address of the array, per device (the symbol itself is only a
// host-side handle and must never be passed to a kernel).  An address stays
// valid for the life of the device's primary context; the look-up is serialised
// so that first calls from several host threads do not race.
float* g_noalloc_ptr[64] = {nullptr};
std::mutex g_noalloc_mu;
}  // namespace
}  // namespace locks

extern "C" int locks_decode_split_noalloc(
    const void* q, int64_t q_stride_req, const void* k_cache,
    const void* v_cache, int64_t kv_stride_block, int64_t kv_stride_tok,
    int64_t kv_stride_head, const int32_t* block_table, int64_t bt_stride,
    const int32_t* page_table, const int32_t* page_cnt, const int32_t* seq_lens,
    void* out, int64_t out_stride_req, int n_req, int n_kv, int G, int head_dim,
    int page, int max_pages, int split, int pps_min, float scale, int* status,
    locks_stream_t stream) {
    LOCKS_REQUIRE(q && k_cache && v_cache && block_table && page_table &&
                      page_cnt && seq_lens && out,
                  LOCKS_ERR_ARG, "locks_decode_split_noalloc: null pointer argument");
    int rc = check_geometry("locks_decode_split_noalloc", G, head_dim, page);
    if (rc) return rc;
    rc = check_kv("locks_decode_split_noalloc", q, k_cache, v_cache, q_stride_req,
                  kv_stride_block, kv_stride_tok, kv_stride_head);
    if (rc) return rc;
    LOCKS_REQUIRE(n_req >= 0 && n_req <= 65535 && n_kv >= 1 && n_kv <= 65535 &&
                      split >= 1 && pps_min >= 1 && max_pages >= 1,
                  LOCKS_ERR_ARG, "locks_decode_split_noalloc: bad size argument");
    const int64_t rows = (int64_t)n_req * n_kv * split * G;
    LOCKS_REQUIRE(rows <= NOALLOC_MAX_ROWS, LOCKS_ERR_SIZE,
                  "locks_decode_split_noalloc: n_req*n_kv*split*G = %lld exceeds "
                  "the built-in scratch of %d partial rows; use locks_decode_split "
                  "with caller-owned buffers", (long long)rows, NOALLOC_MAX_ROWS);
    if (n_req == 0) return LOCKS_OK;

    // one-time set-up per device, with that device current: resolve the device
    // address of the scratch array
    int dev = -1;
    cudaError_t ce = cudaGetDevice(&dev);
    LOCKS_REQUIRE(ce == cudaSuccess && dev >= 0 && dev < 64, LOCKS_ERR_LAUNCH,
                  "locks_decode_split_noalloc: cudaGetDevice: %s",
                  cudaGetErrorString(ce));
    float* base = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mu);
        if (g_noalloc_ptr[dev] == nullptr) {
            float* ptr = nullptr;
            ce = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr),
                                      g_noalloc_scratch);
            LOCKS_REQUIRE(ce == cudaSuccess && ptr != nullptr, LOCKS_ERR_LAUNCH,
                          "locks_decode_split_noalloc: cudaGetSymbolAddress: %s",
                          cudaGetErrorString(ce));
            g_noalloc_ptr[dev] = ptr;
        }
        base = g_noalloc_ptr[dev];
    }
    float* m_part = base;
    float* l_part = base + NOALLOC_MAX_ROWS;
    float* acc_part = base + 2 * (size_t)NOALLOC_MAX_ROWS;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DecParams p{};
    p.q = static_cast<const __nv_bfloat16*>(q); p.q_stride_req = q_stride_req;
    p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
    p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
    p.stride_block = kv_stride_block; p.stride_tok = kv_stride_tok;
    p.stride_head = kv_stride_head;
    p.block_table = block_table; p.bt_stride = bt_stride;
    p.page_table = page_table; p.page_cnt = page_cnt; p.seq_lens = seq_lens;
    p.m_part = m_part; p.l_part = l_part; p.acc_part = acc_part;
    p.n_kv = n_kv; p.G = G; p.max_pages = max_pages; p.split = split;
    p.pps_min = pps_min; p.fused = 0; p.scale = scale; p.status = status;
    rc = launch_decode("locks_decode_split_noalloc", p, n_req, split, s);
    if (rc) return rc;
    MergeParams m{};
    m.m_part = m_part; m.l_part = l_part; m.acc_part = acc_part;
    m.page_cnt = page_cnt; m.seq_lens = nullptr;
    m.out = static_cast<__nv_bfloat16*>(out); m.out_stride_req = out_stride_req;
    m.n_kv = n_kv; m.G = G; m.split = split; m.pps_min = pps_min;
    merge_kernel<<<dim3(n_kv * G, n_req), HD, 0, s>>>(m);
    return check_launch("locks_decode_split_noalloc(merge)");
}
