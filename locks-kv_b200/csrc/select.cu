// Per-step page parameters, GQA score combine and exact top-b page selection.
//
// topb kernel, one launch for any page count, no global scratch.  Scores become
// 32-bit order-preserving keys that live in shared memory from the combine on.
//
// Rows of up to 16 384 pages -- OWNER mode (512 threads per CTA).  Up to four
// CTAs of a thread-block cluster share the GQA combine (nrm or max; the per-head
// maxima come from the keys the scorer published, or from a sweep) and push
// their keys into CTA 0 through distributed shared memory; CTA 0 selects alone.
// Longer rows -- SLICED mode: a cluster of 2, 4 or 8 CTAs, CTA c keeps and
// selects the keys of its page slice with the same code; per radix pass every CTA
// adds its non-empty bins to totals kept by CTA 0 (DSMEM atomics), CTA 0 finds
// the digit and stores it into every CTA; the per-CTA tie and kept totals are
// exchanged once more for the tie ranks and output slots.  Either way:
//   * the page classes are folded into the keys (0 = not a page of the row,
//     0xFFFFFFFF = sink / recent page, always kept), so the later passes test
//     nothing but the key;
//   * b-th largest key by an MSD radix select (11/11/10 bits) over four
//     interleaved histogram copies (fewer same-address atomics); the digit
//     search runs on 8 warps, each thread owning 8 consecutive bins; a pass whose
//     digit bin is taken whole ends the search (the usual case after 22 bits);
//   * keep flags and ascending compaction in one count loop, ONE barrier and one
//     write loop: every warp derives all warps' tie ranks and output slots from
//     the per-warp totals by itself; four consecutive keys per lane.
#include <cooperative_groups.h>

#include "common.cuh"
#include "cp_link.cuh"
#include "kv_append.cuh"

namespace cg = cooperative_groups;

namespace locks {
namespace {

constexpr int SEL_THREADS = 512;
constexpr int SEL_WARPS = 32;                // capacity of the per-warp arrays
constexpr int MAX_G = 16;

// static budget of one request: a page count (its own entry of budget_req when
// the caller passes per-request budgets, else the engine-wide budget_pages)
// clamped to [1, s], or the fraction `budget` of the s selectable pages rounded
// up in fp64 (reference selection/select.py:36-45)
__device__ __forceinline__ int budget_of(int s, int budget_pages, double budget) {
    if (budget_pages > 0) return max(min(budget_pages, max(s, 1)), 1);
    const double bf = ceil((double)s * budget);
    return min(max((int)bf, 1), max(s, 1));
}

__global__ void derive_kernel(const int32_t* __restrict__ seq_lens, int n_req,
                              int page, int window, int sink, int budget_pages,
                              const int32_t* __restrict__ budget_req,
                              double budget, int32_t* __restrict__ n_pages,
                              int32_t* __restrict__ n_sel_hi,
                              int32_t* __restrict__ b_fix) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_req) return;
    const int sl = seq_lens[i];
    const int npg = (sl + page - 1) / page;
    const int nsh = npg - window;
    const int s = nsh - sink;
    n_pages[i] = npg;
    n_sel_hi[i] = nsh;
    b_fix[i] = budget_of(s, budget_req ? budget_req[i] : budget_pages, budget);
}

// One decode step's bookkeeping for every request row, then its page parameters:
// the appended token's index is the current length, its slot comes from the block
// table, the length grows by one.  slot_prev keeps the slot of the step before
// (the summary build of pages that step completed reads it).
__global__ void advance_kernel(int32_t* __restrict__ seq_lens,
                               const int32_t* __restrict__ block_table,
                               int64_t bt_stride, int bt_width, int n_req, int page,
                               int window, int sink, int budget_pages,
                               const int32_t* __restrict__ budget_req, double budget,
                               int64_t* __restrict__ slot,
                               int64_t* __restrict__ slot_prev,
                               int64_t* __restrict__ pos,
                               int32_t* __restrict__ n_pages,
                               int32_t* __restrict__ n_sel_hi,
                               int32_t* __restrict__ b_fix) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_req) return;
    const int tok = seq_lens[i];
    const int pg = tok / page;
    slot_prev[i] = slot[i];
    if (tok < 0 || pg >= bt_width) {             // no block for the token: no write
        slot[i] = -1;
        pos[i] = max(tok, 0);
    } else {
        slot[i] = (int64_t)block_table[(int64_t)i * bt_stride + pg] * page + tok % page;
        pos[i] = tok;
    }
    const int sl = tok + 1;
    seq_lens[i] = sl;
    const int npg = (sl + page - 1) / page;
    const int nsh = npg - window;
    const int s = nsh - sink;
    n_pages[i] = npg;
    n_sel_hi[i] = nsh;
    b_fix[i] = budget_of(s, budget_req ? budget_req[i] : budget_pages, budget);
}

struct SelParams {
    int combine;
    const float* score_h;
    float* score;
    uint32_t* hmax;
    const int32_t* n_pages;
    const int32_t* n_sel_hi;
    const int32_t* b_fix;
    int32_t* page_table;
    int32_t* page_cnt;
    int n_kv, G, max_pages, sink;
    int owner_mode;     // keys of a whole row fit one CTA: helpers only combine
    int key_cap;        // key slots per CTA (the histogram copies follow them)
    KvAppend app;       // optional: the new token's K/V store of this layer (key != null)
    CpLink cp;          // context parallel: exchanges with the peer ranks (world > 0)
    int* status;        // bounded-wait status word (context parallel only)
    const int32_t* row_order;   // grid row z handles request row_order[z] (or z)
};

// Launch order of the rows of a large ragged batch: longest first, so that the
// last CTAs to start are the short ones (CTAs start roughly in grid order; with a
// few hundred rows of very different lengths over ~300 resident CTAs a long row
// that starts last is the whole tail).  One block; rank sort, ties by index.
// order_sel: by pages to select from; order_dec: by pages the decode will attend.
__global__ void row_order_kernel(const int32_t* __restrict__ n_pages,
                                 const int32_t* __restrict__ n_sel_hi,
                                 const int32_t* __restrict__ b_fix, int n_req,
                                 int sink, int32_t* __restrict__ order_sel,
                                 int32_t* __restrict__ order_dec) {
    for (int i = threadIdx.x; i < n_req; i += blockDim.x) {
        const int si = n_sel_hi[i];
        const int di = min(b_fix[i], max(n_sel_hi[i] - sink, 0)) +
                       (n_pages[i] - n_sel_hi[i]);
        int rs = 0, rd = 0;
        for (int j = 0; j < n_req; ++j) {
            const int sj = n_sel_hi[j];
            const int dj = min(b_fix[j], max(n_sel_hi[j] - sink, 0)) +
                           (n_pages[j] - n_sel_hi[j]);
            rs += (sj > si || (sj == si && j < i)) ? 1 : 0;
            rd += (dj > di || (dj == di && j < i)) ? 1 : 0;
        }
        order_sel[rs] = i;
        order_dec[rd] = i;
    }
}


constexpr int KEYS_PER_CTA = 16384;               // shared-memory key capacity
// single-CTA selection: the latency-bound radix / compaction steps run on a few
// warps with many keys per thread (barriers and scans cost per warp, not per key)
constexpr int AW = 8;                             // active warps
constexpr int ATH = AW * 32;
constexpr int HCOPIES = 4;                        // histogram copies, by lane & 3

constexpr int RBITS0 = 11, RBITS1 = 11, RBITS2 = 10;
constexpr int NBINS = 1 << RBITS0;                // 2048 (largest digit)
constexpr int MAX_CL = 16;            // > 8 needs the non-portable cluster attribute

struct SelSmem {
    int tot[NBINS];                // sliced mode: cluster totals of the digit (CTA 0)
    int wtot[SEL_WARPS];           // per-warp totals (scans)
    int wtot2[SEL_WARPS];
    float wmax[SEL_WARPS][MAX_G];
    float xmax[MAX_G];             // this CTA's per-head maxima (cluster sweep)
    float hm_sh[MAX_G];
    int sh_i0, sh_i1, sh_i2;
    int x_eq_all[MAX_CL];          // sliced mode: per-CTA tie / sure-kept totals
    int x_sure_all[MAX_CL];
};

__device__ __forceinline__ void bar_active() {
    asm volatile("bar.sync 1, %0;" ::"n"(ATH) : "memory");
}

// slot of a histogram bin: HCOPIES counters per bin, one spare slot after every
// 8 bins so that threads which each own 4 or 8 consecutive bins read them
// without shared-memory bank conflicts
__device__ __forceinline__ int hslot(int bin) { return bin + (bin >> 3); }
constexpr int HSLOTS = NBINS + NBINS / 8;

// find_digit run by the first AW warps (the others skip it) over a histogram
// kept as HCOPIES interleaved copies; nb is 1024 or 2048.  Thread t owns the
// nb / ATH bins just below nb - t * (nb / ATH) and clears them on the way, so
// the buffer is zero again afterwards.  The caller's next CTA-wide barrier
// publishes sm.sh_i0 = digit d, sm.sh_i1 = k - count(bins > d), sm.sh_i2 =
// count(d).
template <bool COPIES>
__device__ __forceinline__ void find_digit_active(SelSmem& sm, int* h4, int nb,
                                                  int k) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int bpl = nb / ATH;                              // 8 or 4
    const int hb = nb - 1 - (int)threadIdx.x * bpl;        // my highest bin
    int c[8];
    int mine = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        c[i] = 0;
        if (i < bpl) {
            if (COPIES) {
                int4* q = reinterpret_cast<int4*>(h4) + hslot(hb - i);
                const int4 v = *q;
                c[i] = v.x + v.y + v.z + v.w;
                *q = make_int4(0, 0, 0, 0);
            } else {                  // one plain counter per bin (cluster totals)
                c[i] = h4[hb - i];
                h4[hb - i] = 0;
            }
        }
        mine += c[i];
    }
    int inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) sm.wtot[warp] = inc;
    bar_active();
    const int wv = (lane < AW) ? sm.wtot[lane] : 0;
    int winc = wv;
#pragma unroll
    for (int o = 1; o < AW; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, winc, o);
        if (lane >= o) winc += t;
    }
    int above = __shfl_sync(0xffffffffu, winc - wv, warp) + inc - mine;
    if (above < k && k <= above + mine) {
        bool found = false;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (!found && i < bpl) {
                if (k <= above + c[i]) {
                    sm.sh_i0 = hb - i; sm.sh_i1 = k - above; sm.sh_i2 = c[i];
                    found = true;
                } else {
                    above += c[i];
                }
            }
        }
    }
}

// Sliced selection: the first AW warps add this CTA's bin counts (the copies
// summed) to the cluster totals kept by CTA 0 and clear the bins on the way.
__device__ __forceinline__ void push_bins(int* h4, int nb, int* tot0) {
    const int bpl = nb / ATH;
    const int hb = nb - 1 - (int)threadIdx.x * bpl;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (i < bpl) {
            int4* q = reinterpret_cast<int4*>(h4) + hslot(hb - i);
            const int4 v = *q;
            const int c = v.x + v.y + v.z + v.w;
            if (c) {
                *q = make_int4(0, 0, 0, 0);
                atomicAdd(&tot0[hb - i], c);
            }
        }
    }
}

// nrm combine of the groups [g_beg, g_end) of one warp: score = sum_g
// exp(S[g] - hm[g]).  GT = G rounded up to a power of two; rows beyond G are
// read from row G-1 and masked, so the loads are unconditional and all loads
// of a batch (CB groups, chosen to cover the warp's share in one batch when it
// can) are in flight together.  `sync_hm()` is called once by every thread,
// after the first batch of loads has been issued and before hm_sh is read: the
// barrier that publishes the per-head maxima overlaps the score loads.
template <int GT, int CBW, class SyncFn, class KeyFn>
__device__ __forceinline__ void combine_nrm_groups(
    const float* __restrict__ sh, float* __restrict__ score, uint32_t* keys,
    const float* hm_sh, int G, int MP, int s0, int n_loc, int n_comb,
    int g_beg, int g_end, int lane, SyncFn sync_hm, KeyFn fin_key) {
    constexpr int CB = (CBW * GT > 32) ? (GT >= 32 ? 1 : 32 / GT) : CBW;   // <= 32 loads in flight
    float hm[GT];
    bool first = true;
    int gb = g_beg;
    do {
        float v[CB][GT];
#pragma unroll
        for (int u = 0; u < CB; ++u) {
            const int j = (gb + u) * 32 + lane;
            const int i = max(min(s0 + j, n_comb - 1), 0);  // clamped: always valid
#pragma unroll
            for (int g = 0; g < GT; ++g)
                v[u][g] = __ldcg(&sh[(int64_t)min(g, G - 1) * MP + i]);
        }
        if (first) {
            sync_hm();
#pragma unroll
            for (int g = 0; g < GT; ++g) hm[g] = hm_sh[min(g, G - 1)];
            first = false;
        }
#pragma unroll
        for (int u = 0; u < CB; ++u) {
            const int j = (gb + u) * 32 + lane, i = s0 + j;
            if ((gb + u) < g_end && j < n_loc) {
                float acc = 0.f;
#pragma unroll
                for (int g = 0; g < GT; ++g) {
                    const float e = __expf(v[u][g] - hm[g]);
                    acc += (g < G) ? e : 0.f;
                }
                if (i < n_comb) score[i] = acc; else acc = 0.f;
                keys[j] = fin_key(f2key(acc), i);
            }
        }
        gb += CB;
    } while (gb < g_end);
}

// per-head maxima of the groups of one warp (clamped, unconditional loads)
template <int GT>
__device__ __forceinline__ void sweep_max_groups(
    const float* __restrict__ sh, float* wmax_row, int G, int MP, int s0,
    int n_loc, int n_comb, int g_beg, int g_end, int lane) {
    float lmax[GT];
#pragma unroll
    for (int g = 0; g < GT; ++g) lmax[g] = -INFINITY;
    for (int grp = g_beg; grp < g_end; ++grp) {
        const int j = grp * 32 + lane, i = s0 + j;
        const int ic = min(i, n_comb - 1);
        const bool ok = j < n_loc && i < n_comb;
#pragma unroll
        for (int g = 0; g < GT; ++g) {
            const float x = __ldcg(&sh[(int64_t)min(g, G - 1) * MP + ic]);
            lmax[g] = fmaxf(lmax[g], ok ? x : -INFINITY);
        }
    }
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        float m = lmax[g];
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1)
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0 && g < G) wmax_row[g] = m;
    }
}

#define LOCKS_DISPATCH_CB(N, CALL)                 \
    do {                                           \
        if ((N) <= 1) { constexpr int CBW = 1; CALL; }       \
        else if ((N) <= 2) { constexpr int CBW = 2; CALL; }  \
        else if ((N) <= 4) { constexpr int CBW = 4; CALL; }  \
        else { constexpr int CBW = 8; CALL; }                \
    } while (0)

#define LOCKS_DISPATCH_GT(G, CALL)                 \
    do {                                           \
        if ((G) <= 1) { constexpr int GT = 1; CALL; }        \
        else if ((G) <= 2) { constexpr int GT = 2; CALL; }   \
        else if ((G) <= 4) { constexpr int GT = 4; CALL; }   \
        else if ((G) <= 8) { constexpr int GT = 8; CALL; }   \
        else { constexpr int GT = 16; CALL; }                \
    } while (0)

// Context parallel, after the local selection with the sequence's budget: this
// rank's selected pages meet those of the other ranks.  One CTA per kv-head.  The
// local selection left its kept pages -- ascending, with their class-folded keys
// (0xFFFFFFFF = forced page) -- in CTA 0's shared memory instead of the table:
//   1. entry j becomes a candidate packet pair {score key, global page}; forced
//      pages and empty slots travel as key 0;
//   2. the candidates of all ranks are polled into shared memory;
//   3. a candidate stays when fewer than b candidates of ALL ranks beat it by
//      (key descending, page ascending) -- counted directly, world * cap entries
//      are a few thousand at most;
//   4. the table is written once: forced pages + surviving candidates,
//      ascending, -1 behind them up to the local count, and the final count.
// scratch (words): keep[cap] | ckey[world*cap] | cpage[world*cap] | lkey[cap] |
// lpage[cap]; the last two are the local list.
__device__ __forceinline__ uint32_t* cp_list_keys(uint32_t* scratch, int cap, int W) {
    return scratch + cap + 2 * W * cap;
}
template <int NT>
__device__ __forceinline__ void cp_global_cut(const CpLink& cp, int kh,
                                              int32_t* tab, int32_t* cnt_out,
                                              int cnt, uint32_t* scratch,
                                              int* wsum, int* status) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int NW = NT / 32;
    const int cap = cp.cap, W = cp.world;
    const uint32_t epoch = cp_epoch(cp);
    int* keep_sh = reinterpret_cast<int*>(scratch);
    uint32_t* ckey = scratch + cap;
    int32_t* cpage = reinterpret_cast<int32_t*>(ckey + W * cap);
    const uint32_t* lkey = cp_list_keys(scratch, cap, W);
    const int32_t* lpage = reinterpret_cast<const int32_t*>(lkey + cap);
    for (int j = tid; j < cap; j += NT) {
        const uint32_t k0 = (j < cnt) ? lkey[j] : 0u;
        const bool sel = k0 != 0u && k0 != 0xFFFFFFFFu;
        const int idx = (kh * cap + j) * 2;
        cp_push(cp, cp.off_cand, cp.cand_words, epoch, idx, sel ? k0 : 0u);
        cp_push(cp, cp.off_cand, cp.cand_words, epoch, idx + 1,
                (uint32_t)(sel ? lpage[j] + cp.p0 : 0x7FFFFFFF));
    }
    bool late = false;
    const uint8_t* mine = cp.base[cp.rank];
    for (int i0 = 0; i0 < W * cap; i0 += 2 * NT) {         // 2 candidates per thread
        const uint8_t* addr[4];
        uint32_t val[4];
        int n = 0, slot[2] = {-1, -1};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int i = i0 + u * NT + tid;
            if (i < W * cap) {
                const int r = i / cap, c = i - r * cap;
                const int idx = (kh * cap + c) * 2;
                addr[n] = mine + cp_slot(cp.off_cand, cp.cand_words, epoch, r, idx);
                addr[n + 1] = addr[n] + 8;
                slot[u] = i;
                n += 2;
            }
        }
        if (n > 0) {
            if (!cp_wait_words<4>(addr, n, epoch, val)) {
                late = true;
                val[0] = val[2] = 0u;                       // no candidate
            }
            int k = 0;
#pragma unroll
            for (int u = 0; u < 2; ++u)
                if (slot[u] >= 0) {
                    ckey[slot[u]] = val[k];
                    cpage[slot[u]] = (int32_t)val[k + 1];
                    k += 2;
                }
        }
    }
    if (late && status) atomicExch(status, LOCKS_ST_WAIT_TIMEOUT);
    __syncthreads();
    for (int j = warp; j < cap; j += NW) {
        const uint32_t k0 = (j < cnt) ? lkey[j] : 0u;
        const bool sel = k0 != 0u && k0 != 0xFFFFFFFFu;
        int keep = (k0 != 0u) ? 1 : 0;                      // forced pages stay
        if (sel) {                                          // warp-uniform
            const int pg = lpage[j] + cp.p0;
            int beat = 0;
            for (int c = lane; c < W * cap; c += 32) {
                const uint32_t k2 = ckey[c];
                beat += (k2 > k0 || (k2 == k0 && cpage[c] < pg)) ? 1 : 0;
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1)
                beat += __shfl_xor_sync(0xffffffffu, beat, o);
            keep = (beat < cp.b_global) ? 1 : 0;
        }
        if (lane == 0) keep_sh[j] = keep;
    }
    __syncthreads();
    int base = 0;
    for (int j0 = 0; j0 < cap; j0 += NT) {
        const int j = j0 + tid;
        const int k = (j < cap) ? keep_sh[j] : 0;
        int inc = k;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) wsum[warp] = inc;
        __syncthreads();
        int wbase = 0, total = 0;
        for (int w = 0; w < NW; ++w) {
            const int v = wsum[w];
            if (w < warp) wbase += v;
            total += v;
        }
        if (k) tab[base + wbase + inc - 1] = lpage[j];
        base += total;
        __syncthreads();
    }
    for (int j = base + tid; j < cnt; j += NT) tab[j] = -1;
    if (tid == 0) *cnt_out = base;
}

// NT threads per CTA.  OWNER: CTA 0 selects the whole row, the other CTAs of the
// cluster only combine (or there is no cluster); otherwise every CTA of the
// cluster keeps and selects the keys of its page slice.
// GT: the GQA group size rounded up to a power of two (a kernel per value keeps
// the once-through instruction stream short).
// APPEND: the launch also stores the new token's K/V of its rows (p.app).
// CP: context parallel (the exchanges with the peer ranks are compiled in).
template <int NT, bool OWNER, int GT, bool APPEND, bool CP>
__global__ void __launch_bounds__(NT)
topb_kernel(const SelParams p) {
    constexpr int NW = NT / 32;
    __shared__ SelSmem sm;
    extern __shared__ __align__(16) uint32_t keys[];   // keys of my page slice
    cg::cluster_group cluster = cg::this_cluster();

    pdl_trigger();               // the decode may be scheduled; it waits for us
    const int c_phys = blockIdx.x, CL_phys = gridDim.x;   // rank / size of cluster
    const int kh = blockIdx.y;
    const int r = p.row_order ? p.row_order[blockIdx.z] : (int)blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int MP = p.max_pages, G = p.G;
    const int npg = min(max(p.n_pages[r], 0), MP);
    const int nsh = p.n_sel_hi[r];
    int b = p.b_fix[r];
    const int lo = min(p.sink, npg);
    const int hi = max(min(nsh, npg), lo);
    const int L = hi - lo;
    const bool keep_all = (nsh - p.sink) <= 1 || L <= 1;

    const int64_t row = (int64_t)r * p.n_kv + kh;
    float* score = p.score + row * MP;
    const int n_comb = min(max(nsh, 0), MP);        // pages with a score
    const int span = max(npg, n_comb);

    // Owner mode (the keys of the whole row fit one CTA's shared memory): every
    // CTA of the cluster combines a slice of the scores and pushes the keys into
    // CTA 0 through distributed shared memory; CTA 0 alone selects, the helpers
    // write the -1 padding that no selection can reach and leave.
    // Sliced mode (long contexts): every CTA keeps and selects its slice; the
    // histograms meet in CTA 0, which finds each digit and tells the others.
    const bool owner = OWNER && CL_phys > 1;
    // slice whose scores this CTA combines
    const int cper = (((span + CL_phys - 1) / CL_phys) + 31) & ~31;
    const int cs0 = min(c_phys * cper, span), cs1 = min(cs0 + cper, span);
    const int cn_loc = cs1 - cs0;
    const int cn_grp = (cn_loc + 31) >> 5;
    const int cgpw = (cn_grp + NW - 1) / NW;
    const int cg_beg = min(warp * cgpw, cn_grp), cg_end = min(cg_beg + cgpw, cn_grp);
    uint32_t* kdst = owner ? cluster.map_shared_rank(keys, 0) + cs0 : keys;
    // slice this CTA selects from
    const int c = owner ? 0 : c_phys, CL = owner ? 1 : CL_phys;
    const int s0 = owner ? 0 : cs0, s1 = owner ? span : cs1;
    const int n_loc = s1 - s0;

    const bool selects = !owner || c_phys == 0;     // this CTA runs a selection
    int* h4 = reinterpret_cast<int*>(keys + p.key_cap);
    if (selects) {
        for (int i = tid; i < HSLOTS; i += NT)
            reinterpret_cast<int4*>(h4)[i] = make_int4(0, 0, 0, 0);
        for (int i = tid; i < NBINS; i += NT) sm.tot[i] = 0;
    }
    // remote shared memory may be touched once every CTA of the cluster runs;
    // this barrier costs nothing while the scorer is still at work
    if (CL_phys > 1) cluster.sync();
    pdl_wait();                  // score_h / hmax / score come from the scorer

    // The page classes are folded into the keys: 0 = not a page of the row,
    // 0xFFFFFFFF = always kept (sink / recent pages, short rows), anything
    // between = a selectable page's score key.
    auto fin_key = [&](uint32_t key, int i) -> uint32_t {
        if (i >= npg) return 0u;
        if (keep_all || i < lo || i >= hi) return 0xFFFFFFFFu;
        return min(max(key, 1u), 0xFFFFFFFEu);
    };
    if (selects)                     // key slots past the slice read as "no page"
        for (int i = n_loc + tid; i < p.key_cap; i += NT) keys[i] = 0u;

    // ---------------- 1. GQA combine -> score[slice], keys[slice] --------------
    // Context parallel: the per-head maxima are those of the WHOLE sequence.  CTA 0
    // of the row sends the keys the local scorer published (0 = nothing scored
    // here) to every rank; every CTA polls the local region for all ranks' keys.
    // A rank with nothing to combine still takes part.
    constexpr bool cp_on = CP;
    if (cp_on && tid < G) {
        const uint32_t epoch = cp_epoch(p.cp);
        const int idx = kh * G + tid;
        if (c_phys == 0)
            cp_push(p.cp, p.cp.off_hmax, p.cp.hmax_words, epoch, idx,
                    p.hmax[row * G + tid]);
        const uint8_t* addr[CP_MAX_RANKS];
        uint32_t val[CP_MAX_RANKS];
#pragma unroll
        for (int rr = 0; rr < CP_MAX_RANKS; ++rr)
            addr[rr] = p.cp.base[p.cp.rank] +
                       cp_slot(p.cp.off_hmax, p.cp.hmax_words, epoch, rr, idx);
        if (!cp_wait_words<CP_MAX_RANKS>(addr, p.cp.world, epoch, val) && p.status)
            atomicExch(p.status, LOCKS_ST_WAIT_TIMEOUT);
        uint32_t m = 0u;
#pragma unroll
        for (int rr = 0; rr < CP_MAX_RANKS; ++rr)
            if (rr < p.cp.world) m = max(m, val[rr]);
        sm.hm_sh[tid] = key2f(m);
    }
    if (p.combine == LOCKS_COMBINE_NRM && n_comb > 0) {
        const float* sh = p.score_h + row * (int64_t)G * MP;
        const bool published = p.hmax != nullptr;
        if (cp_on) {
            // hm_sh holds the sequence-wide maxima (published by sync_hm below)
        } else if (published) {
            if (tid < G) sm.hm_sh[tid] = key2f(p.hmax[row * G + tid]);
        } else {
            sweep_max_groups<GT>(sh, sm.wmax[warp], G, MP, cs0, cn_loc, n_comb, cg_beg,
                                 cg_end, lane);
            __syncthreads();
            if (tid < G) {
                float m = -INFINITY;
                for (int w = 0; w < NW; ++w) m = fmaxf(m, sm.wmax[w][tid]);
                sm.xmax[tid] = m;
            }
            if (CL_phys > 1) {
                cluster.sync();
                if (tid < G) {
                    float m = -INFINITY;
                    for (int cc = 0; cc < CL_phys; ++cc)
                        m = fmaxf(m, *cluster.map_shared_rank(&sm.xmax[tid], cc));
                    sm.hm_sh[tid] = m;
                }
            } else {
                __syncthreads();
                if (tid < G) sm.hm_sh[tid] = sm.xmax[tid];
            }
        }
        // the barrier below publishes hm_sh; the scorer's keys are re-armed
        // further down, behind a cluster barrier every CTA passes after this read
        auto sync_hm = [&]() { __syncthreads(); };
        LOCKS_DISPATCH_CB(cgpw, (combine_nrm_groups<GT, CBW>(
            sh, score, kdst, sm.hm_sh, G, MP, cs0, cn_loc, n_comb, cg_beg, cg_end,
            lane, sync_hm, fin_key)));
    } else if (p.combine == LOCKS_COMBINE_MAX && n_comb > 0) {
        const float* sh = p.score_h + row * (int64_t)G * MP;
        for (int grp = cg_beg; grp < cg_end; ++grp) {
            const int j = grp * 32 + lane, i = cs0 + j;
            if (j < cn_loc) {
                float m = 0.f;
                if (i < n_comb) {
                    m = -INFINITY;
                    for (int g = 0; g < G; ++g)
                        m = fmaxf(m, sh[(int64_t)g * MP + i]);
                    score[i] = m;
                }
                kdst[j] = fin_key(f2key(m), i);
            }
        }
    } else {
        for (int grp = cg_beg; grp < cg_end; ++grp) {
            const int j = grp * 32 + lane;
            if (j < cn_loc) kdst[j] = fin_key(f2key(score[cs0 + j]), cs0 + j);
        }
    }
    const bool rearm = p.combine == LOCKS_COMBINE_NRM && n_comb > 0 &&
                       p.hmax != nullptr;
    if (owner) {
        cluster.sync();                  // all keys have landed in CTA 0
        if (rearm && c_phys == 0 && tid < G) p.hmax[row * G + tid] = 0u;
        if (c_phys != 0) {
            // entries no selection can reach: beyond the forced pages + budget
            const int cnt_max = keep_all ? npg
                                         : min(npg, (npg - L) + min(max(b, 0), L));
            int32_t* tabp = p.page_table + row * MP;
            for (int i = cnt_max + (c_phys - 1) * NT + tid; i < MP;
                 i += (CL_phys - 1) * NT)
                tabp[i] = -1;
            // the last helper also stores the row's new token (K rotated) into
            // the cache: it is done here long before CTA 0 has selected, and the
            // decode that reads the cache starts only when this grid has ended
            if constexpr (APPEND) {
                if (c_phys == CL_phys - 1 && tid < p.app.head_dim)
                    kv_append_elem(p.app, r, kh, tid);
            }
            return;
        }
    } else {
        __syncthreads();
        // single CTA: every thread has read the keys; a cluster of slices re-arms
        // behind the exchange of the compaction totals below
        if (rearm && CL_phys == 1 && tid < G) p.hmax[row * G + tid] = 0u;
    }

    // ============ selection over keys[0, n_loc) (local index j = page - s0) ======
    // The per-key loops run on all warps, 4 consecutive keys per lane; the digit
    // search runs on the first AW warps (of CTA 0 in sliced mode).
    int32_t* tab = p.page_table + row * MP;
    // ---- 2. threshold: keys > tau_key are kept, `quota` of the keys equal to it
    // (in ascending page order) as well
    uint32_t tau_key = 0u;       // below every page's key: every page is kept
    int quota = 0;
    if (!keep_all && b <= 0) {
        tau_key = 0xFFFFFFFEu;   // only the always-kept pages lie above
    } else if (!keep_all && b < L) {
        uint32_t prefix = 0u, mask = 0u;
        int k = b, shift = 32;
        bool whole_bin = false;
        int* tot0 = (CL > 1) ? cluster.map_shared_rank(sm.tot, 0) : sm.tot;
#pragma unroll 1
        for (int pass = 0; pass < 3 && !whole_bin; ++pass) {
            const int bits = (pass == 0) ? RBITS0 : (pass == 1) ? RBITS1 : RBITS2;
            const int nb = 1 << bits;
            shift -= bits;
            const uint32_t dmask = (uint32_t)nb - 1u;
            for (int base = 4 * tid; base < n_loc; base += 4 * NT) {
                const uint4 kv = *reinterpret_cast<const uint4*>(&keys[base]);
                const uint32_t kk[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    const uint32_t key = kk[s];
                    if (key - 1u < 0xFFFFFFFEu && (key & mask) == prefix)
                        atomicAdd(&h4[(hslot((key >> shift) & dmask) << 2) |
                                      (lane & 3)], 1);
                }
            }
            __syncthreads();
            if (CL == 1) {
                if (warp < AW) find_digit_active<true>(sm, h4, nb, k);
                __syncthreads();
            } else {
                if (warp < AW) push_bins(h4, nb, tot0);
                cluster.sync();                       // the totals are complete
                if (c == 0) {
                    if (warp < AW) find_digit_active<false>(sm, sm.tot, nb, k);
                    __syncthreads();
                    if (tid > 0 && tid < CL) {        // tell the other CTAs
                        *cluster.map_shared_rank(&sm.sh_i0, tid) = sm.sh_i0;
                        *cluster.map_shared_rank(&sm.sh_i1, tid) = sm.sh_i1;
                        *cluster.map_shared_rank(&sm.sh_i2, tid) = sm.sh_i2;
                    }
                }
                cluster.sync();                       // the digit has arrived
            }
            prefix |= (uint32_t)sm.sh_i0 << shift;
            k = sm.sh_i1;
            mask |= dmask << shift;
            // the bin is taken whole: no finer digit and no tie rule needed
            whole_bin = (sm.sh_i2 == k);
        }
        if (whole_bin) { tau_key = prefix ? prefix - 1u : 0u; quota = 0; }
        else { tau_key = prefix; quota = k; }
    }

    // context parallel: where the kept (key, page) list lives (CTA 0 of the row)
    uint32_t* cpl_key = nullptr;
    if constexpr (CP) {
        uint32_t* l0 = cp_list_keys(reinterpret_cast<uint32_t*>(h4), p.cp.cap,
                                    p.cp.world);
        cpl_key = (CL > 1) ? cluster.map_shared_rank(l0, 0) : l0;
    }
    // ---- 3. keep flags + ascending compaction.  Warp w owns a contiguous run of
    // keys and walks it 128 keys at a time.
    const uint32_t lt_mask = (1u << lane) - 1u;
    const int WS = (((n_loc + NW - 1) / NW) + 127) & ~127;
    const int w0 = min(warp * WS, n_loc), w1 = min(w0 + WS, n_loc);
    const bool ties = quota > 0;
    int c_sure = 0, c_eq = 0;
    for (int it = w0; it < w1; it += 128) {
        const uint4 kv = *reinterpret_cast<const uint4*>(&keys[it + 4 * lane]);
        c_sure += (kv.x > tau_key) + (kv.y > tau_key) + (kv.z > tau_key) +
                  (kv.w > tau_key);
        c_eq += (kv.x == tau_key) + (kv.y == tau_key) + (kv.z == tau_key) +
                (kv.w == tau_key);
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        c_eq += __shfl_xor_sync(0xffffffffu, c_eq, o);
        c_sure += __shfl_xor_sync(0xffffffffu, c_sure, o);
    }
    if (lane == 0) { sm.wtot[warp] = c_eq; sm.wtot2[warp] = c_sure; }
    __syncthreads();
    // every warp derives all warps' tie ranks and output slots by itself
    const int e_w = (lane < NW) ? sm.wtot[lane] : 0;
    const int s_w = (lane < NW) ? sm.wtot2[lane] : 0;
    int einc = e_w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, einc, o);
        if (lane >= o) einc += t;
    }
    // sliced mode: ties and kept pages of the slices before mine
    int eq_before = 0, pos_before = 0, cnt_all = 0;
    if (CL > 1) {
        const int eq_mine = __shfl_sync(0xffffffffu, einc, 31);
        int sinc = s_w;
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1)
            sinc += __shfl_xor_sync(0xffffffffu, sinc, o);
        if (tid < CL) {
            *cluster.map_shared_rank(&sm.x_eq_all[c], tid) = eq_mine;
            *cluster.map_shared_rank(&sm.x_sure_all[c], tid) = sinc;
        }
        cluster.sync();
        if (rearm && c == 0 && tid < G) p.hmax[row * G + tid] = 0u;
        int eb = 0;
        for (int cc = 0; cc < CL; ++cc) {
            const int e = sm.x_eq_all[cc];
            const int kept = sm.x_sure_all[cc] + min(max(quota - eb, 0), e);
            if (cc < c) { eq_before += e; pos_before += kept; }
            cnt_all += kept;
            eb += e;
        }
    }
    const int k_w = s_w + min(max(quota - eq_before - (einc - e_w), 0), e_w);
    int kinc = k_w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, kinc, o);
        if (lane >= o) kinc += t;
    }
    int pos = pos_before + __shfl_sync(0xffffffffu, kinc - k_w, warp);
    int eqr = eq_before + __shfl_sync(0xffffffffu, einc - e_w, warp);
    const int cnt = (CL > 1) ? cnt_all : __shfl_sync(0xffffffffu, kinc, 31);
    for (int it = w0; it < w1; it += 128) {
        const int base = it + 4 * lane;
        const uint4 kv = *reinterpret_cast<const uint4*>(&keys[base]);
        const uint32_t kk[4] = {kv.x, kv.y, kv.z, kv.w};
        bool keep[4];
#pragma unroll
        for (int s = 0; s < 4; ++s) keep[s] = kk[s] > tau_key;
        if (ties) {
            uint32_t eb[4];
            int lower = 0, total = 0;
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                eb[s] = __ballot_sync(0xffffffffu, kk[s] == tau_key);
                lower += __popc(eb[s] & lt_mask);
                total += __popc(eb[s]);
            }
            int rank = eqr + lower;                  // ties before (lane, s = 0)
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                if (kk[s] == tau_key) { keep[s] = rank < quota; ++rank; }
            }
            eqr += total;
        }
        int slot = pos, total = 0;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const uint32_t kb = __ballot_sync(0xffffffffu, keep[s]);
            slot += __popc(kb & lt_mask);
            total += __popc(kb);
        }
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            if (keep[s]) {
                if constexpr (CP) {
                    // context parallel: the kept pages and their keys go to the
                    // list in CTA 0's shared memory; the table is written once,
                    // after the ranks' selections have met
                    if (slot < p.cp.cap) {
                        cpl_key[slot] = kk[s];
                        cpl_key[slot + p.cp.cap] = (uint32_t)(s0 + base + s);
                    }
                    ++slot;
                } else {
                    tab[slot++] = s0 + base + s;
                }
            }
        }
        pos += total;
    }
    // -1 padding of [cnt, MP): in owner mode the helper CTAs did the part no
    // selection can reach, in sliced mode the CTAs share it
    {
        const int cnt_max = keep_all ? npg
                                     : min(npg, (npg - L) + min(max(b, 0), L));
        const int pad_end = owner ? cnt_max : MP;
        for (int i = cnt + c * NT + tid; i < pad_end; i += CL * NT) tab[i] = -1;
    }
    if (c == 0 && tid == 0) p.page_cnt[row] = cnt;
    // without helper CTAs the last CTA of the row stores the new token
    if constexpr (APPEND) {
        if (!owner && c_phys == CL_phys - 1 && tid < p.app.head_dim)
            kv_append_elem(p.app, r, kh, tid);
    }
    // context parallel: the ranks' selections meet (CTA 0 of the row; the other
    // slices' table entries and scores are visible behind the cluster barrier)
    if constexpr (CP) {
        if (CL > 1) cluster.sync(); else __syncthreads();
        if (c == 0 && cnt > p.cp.cap && tid == 0 && p.status)
            atomicExch(p.status, LOCKS_ST_CP_OVERFLOW);     // caller sized cap too small
        if (c == 0)
            cp_global_cut<NT>(p.cp, kh, tab, &p.page_cnt[row], min(cnt, p.cp.cap),
                              reinterpret_cast<uint32_t*>(h4), sm.wtot, p.status);
    }
}

}  // namespace
}  // namespace locks


static int derive_impl(
    const int32_t* seq_lens, int n_req, int page, int window_pages,
    int sink_pages, int budget_pages, const int32_t* budget_req, double budget,
    int32_t* n_pages, int32_t* n_sel_hi, int32_t* b_fix, locks_stream_t stream) {
    using namespace locks;
    LOCKS_REQUIRE(seq_lens && n_pages && n_sel_hi && b_fix, LOCKS_ERR_ARG,
                  "locks_derive_page_params: null pointer argument");
    LOCKS_REQUIRE(n_req >= 0 && page > 0 && window_pages >= 0 && sink_pages >= 0,
                  LOCKS_ERR_ARG, "locks_derive_page_params: bad size argument");
    if (n_req == 0) return LOCKS_OK;
    derive_kernel<<<(n_req + 127) / 128, 128, 0,
                    static_cast<cudaStream_t>(stream)>>>(
        seq_lens, n_req, page, window_pages, sink_pages, budget_pages, budget_req,
        budget, n_pages, n_sel_hi, b_fix);
    pdl_break();
    return check_launch("locks_derive_page_params");
}

extern "C" int locks_derive_page_params(
    const int32_t* seq_lens, int n_req, int page, int window_pages,
    int sink_pages, int budget_pages, double budget, int32_t* n_pages,
    int32_t* n_sel_hi, int32_t* b_fix, locks_stream_t stream) {
    return derive_impl(seq_lens, n_req, page, window_pages, sink_pages,
                       budget_pages, nullptr, budget, n_pages, n_sel_hi, b_fix,
                       stream);
}

extern "C" int locks_derive_page_params_req(
    const int32_t* seq_lens, int n_req, int page, int window_pages,
    int sink_pages, const int32_t* budget_pages_req, double budget,
    int32_t* n_pages, int32_t* n_sel_hi, int32_t* b_fix, locks_stream_t stream) {
    LOCKS_REQUIRE(budget_pages_req != nullptr, LOCKS_ERR_ARG,
                  "locks_derive_page_params_req: null per-request budget array");
    return derive_impl(seq_lens, n_req, page, window_pages, sink_pages, 0,
                       budget_pages_req, budget, n_pages, n_sel_hi, b_fix, stream);
}

static int advance_impl(
    int32_t* seq_lens, const int32_t* block_table, int64_t bt_stride, int bt_width,
    int n_req, int page, int window_pages, int sink_pages, int budget_pages,
    const int32_t* budget_req, double budget, int64_t* slot_mapping,
    int64_t* slot_prev, int64_t* positions, int32_t* n_pages, int32_t* n_sel_hi,
    int32_t* b_fix, locks_stream_t stream) {
    using namespace locks;
    LOCKS_REQUIRE(seq_lens && block_table && slot_mapping && slot_prev && positions &&
                      n_pages && n_sel_hi && b_fix,
                  LOCKS_ERR_ARG, "locks_append_advance: null pointer argument");
    LOCKS_REQUIRE(n_req >= 0 && page > 0 && bt_width >= 1 && window_pages >= 0 &&
                      sink_pages >= 0,
                  LOCKS_ERR_ARG, "locks_append_advance: bad size argument");
    if (n_req == 0) return LOCKS_OK;
    advance_kernel<<<(n_req + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        seq_lens, block_table, bt_stride, bt_width, n_req, page, window_pages,
        sink_pages, budget_pages, budget_req, budget, slot_mapping, slot_prev,
        positions, n_pages, n_sel_hi, b_fix);
    pdl_break();
    return check_launch("locks_append_advance");
}

extern "C" int locks_append_advance(
    int32_t* seq_lens, const int32_t* block_table, int64_t bt_stride, int bt_width,
    int n_req, int page, int window_pages, int sink_pages, int budget_pages,
    double budget, int64_t* slot_mapping, int64_t* slot_prev, int64_t* positions,
    int32_t* n_pages, int32_t* n_sel_hi, int32_t* b_fix, locks_stream_t stream) {
    return advance_impl(seq_lens, block_table, bt_stride, bt_width, n_req, page,
                        window_pages, sink_pages, budget_pages, nullptr, budget,
                        slot_mapping, slot_prev, positions, n_pages, n_sel_hi, b_fix,
                        stream);
}

extern "C" int locks_append_advance_req(
    int32_t* seq_lens, const int32_t* block_table, int64_t bt_stride, int bt_width,
    int n_req, int page, int window_pages, int sink_pages,
    const int32_t* budget_pages_req, double budget, int64_t* slot_mapping,
    int64_t* slot_prev, int64_t* positions, int32_t* n_pages, int32_t* n_sel_hi,
    int32_t* b_fix, locks_stream_t stream) {
    LOCKS_REQUIRE(budget_pages_req != nullptr, LOCKS_ERR_ARG,
                  "locks_append_advance_req: null per-request budget array");
    return advance_impl(seq_lens, block_table, bt_stride, bt_width, n_req, page,
                        window_pages, sink_pages, 0, budget_pages_req, budget,
                        slot_mapping, slot_prev, positions, n_pages, n_sel_hi, b_fix,
                        stream);
}

static int topb_select_impl(
    int combine, const float* score_h, float* score, uint32_t* hmax,
    const int32_t* n_pages, const int32_t* n_sel_hi, const int32_t* b_fix,
    int32_t* page_table, int32_t* page_cnt, int n_req, int n_kv, int G,
    int max_pages, int sink_pages, const locks_kv_append_t* app,
    locks_stream_t stream, const locks_cp_link_t* link = nullptr,
    int* status = nullptr, const int32_t* row_order = nullptr) {
    using namespace locks;
    LOCKS_REQUIRE(combine >= 0 && combine <= 2, LOCKS_ERR_ARG,
                  "locks_topb_select: combine must be 0, 1 or 2, got %d", combine);
    LOCKS_REQUIRE(score && n_pages && n_sel_hi && b_fix && page_table && page_cnt,
                  LOCKS_ERR_ARG, "locks_topb_select: null pointer argument");
    LOCKS_REQUIRE(combine == LOCKS_COMBINE_NONE || score_h != nullptr,
                  LOCKS_ERR_ARG, "locks_topb_select: score_h required to combine");
    LOCKS_REQUIRE(G >= 1 && G <= MAX_G, LOCKS_ERR_GEOMETRY,
                  "locks_topb_select: supports 1 <= G <= 16, got %d", G);
    LOCKS_REQUIRE(n_req >= 0 && n_req <= 65535 && n_kv >= 1 && max_pages >= 1 &&
                      sink_pages >= 0,
                  LOCKS_ERR_ARG, "locks_topb_select: bad size argument");
    if (n_req == 0) return LOCKS_OK;
    SelParams p;
    p.combine = combine; p.score_h = score_h; p.score = score; p.hmax = hmax;
    p.n_pages = n_pages; p.n_sel_hi = n_sel_hi; p.b_fix = b_fix;
    p.page_table = page_table; p.page_cnt = page_cnt;
    p.n_kv = n_kv; p.G = G; p.max_pages = max_pages; p.sink = sink_pages;
    p.app = KvAppend{};
    p.cp = CpLink{};
    p.status = status;
    p.row_order = row_order;
    if (link != nullptr) {
        LOCKS_REQUIRE(n_req == 1 && combine == LOCKS_COMBINE_NRM && hmax != nullptr,
                      LOCKS_ERR_ARG,
                      "locks_topb_select_cp: one sequence, nrm combine and the "
                      "scorer's published maxima are required");
        const int rc = cp_link_fill(p.cp, link, n_kv, G, "locks_topb_select_cp");
        if (rc) return rc;
        LOCKS_REQUIRE(3 * p.cp.cap + 2 * p.cp.world * p.cp.cap <= HSLOTS * HCOPIES,
                      LOCKS_ERR_SIZE,
                      "locks_topb_select_cp: %d candidate slots x %d ranks beyond "
                      "the shared-memory staging area", p.cp.cap, p.cp.world);
    }
    if (app != nullptr) {
        LOCKS_REQUIRE(app->key && app->val && app->k_cache && app->v_cache &&
                          app->slot_mapping,
                      LOCKS_ERR_ARG, "locks_topb_select_append: null pointer in the "
                      "append description");
        LOCKS_REQUIRE(app->head_dim >= 1 && app->head_dim <= SEL_THREADS &&
                          app->page >= 1 && app->num_blocks >= 1,
                      LOCKS_ERR_GEOMETRY,
                      "locks_topb_select_append: head_dim %d / page %d unsupported",
                      app->head_dim, app->page);
        LOCKS_REQUIRE(app->cos_sin == nullptr ||
                          (app->positions && app->rot_dim >= 2 &&
                           app->rot_dim <= app->head_dim && (app->rot_dim & 1) == 0 &&
                           app->cos_sin_row_stride >= app->rot_dim),
                      LOCKS_ERR_ARG,
                      "locks_topb_select_append: rotation needs positions and an "
                      "even rot_dim <= head_dim");
        p.app.key = static_cast<const __nv_bfloat16*>(app->key);
        p.app.val = static_cast<const __nv_bfloat16*>(app->val);
        p.app.k_row = app->k_row_stride; p.app.k_head = app->k_head_stride;
        p.app.v_row = app->v_row_stride; p.app.v_head = app->v_head_stride;
        p.app.k_cache = static_cast<__nv_bfloat16*>(app->k_cache);
        p.app.v_cache = static_cast<__nv_bfloat16*>(app->v_cache);
        p.app.cb = app->kv_stride_block; p.app.ct = app->kv_stride_tok;
        p.app.ch = app->kv_stride_head;
        p.app.slot = app->slot_mapping; p.app.pos = app->positions;
        p.app.cos_sin = static_cast<const __nv_bfloat16*>(app->cos_sin);
        p.app.cs_row = app->cos_sin_row_stride;
        p.app.rot_dim = app->rot_dim; p.app.neox = app->neox;
        p.app.page = app->page; p.app.num_blocks = app->num_blocks;
        p.app.head_dim = app->head_dim;
    }
    // Short rows (keys fit one CTA): owner mode, up to 8 CTAs share the combine.
    // Long rows: the smallest power-of-two cluster whose CTAs hold the keys.
    int cl = 1;
    const bool owner_mode = max_pages <= KEYS_PER_CTA;
    if (owner_mode) {
        const int want = sm_count() / max(1, n_kv * n_req);
        // (rows of at least 1024 pages, at least 256 pages per CTA; measured with 8
        // rows: 8192 pages 15.7 / 12.9 / 10.9 / 9.9 us with 1 / 2 / 4 / 8 CTAs per
        // row, 2048 pages 8.2 / 7.0 us with 2 / 8, 512 pages 6.5 / 6.7 with 1 / 2)
        const int useful = (max_pages >= 1024) ? (max_pages + 255) / 256 : 1;
        while (cl * 2 <= want && cl * 2 <= useful && cl < 8) cl *= 2;
    } else {
        while (cl < MAX_CL && (max_pages + cl - 1) / cl > KEYS_PER_CTA) cl *= 2;
        // more CTAs share the combine when SMs are free
        const int want = sm_count() / max(1, n_kv * n_req);
        while (cl * 2 <= 8 && cl * 2 <= want && max_pages / (cl * 2) >= 4096)
            cl *= 2;
        // 16-CTA clusters each need a whole GPC: only for a few rows
        if (cl == 8 && 2 * 16 * n_kv * n_req <= sm_count() &&
            max_pages / 16 >= 4096)
            cl = 16;
    }
    LOCKS_REQUIRE(owner_mode || (max_pages + cl - 1) / cl <= KEYS_PER_CTA,
                  LOCKS_ERR_SIZE,
                  "locks_topb_select: max_pages %d beyond the supported %d",
                  max_pages, MAX_CL * KEYS_PER_CTA);
    p.owner_mode = owner_mode ? 1 : 0;
    // key slots per CTA (the compaction reads whole 128-key rows), followed by
    // the interleaved histogram copies
    const int slice = owner_mode ? max_pages
                                 : ((((max_pages + cl - 1) / cl) + 31) & ~31);
    const int per_cta = ((slice + 127) & ~127) + 128;
    p.key_cap = per_cta;
    const int dyn_smem = (per_cta + HSLOTS * HCOPIES) * 4;
    const int smem_max = (KEYS_PER_CTA + 512 + HSLOTS * HCOPIES) * 4;
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
#define LOCKS_SEL_ATTR_A(GTV, AP, CPV)                                             \
        cudaFuncSetAttribute(topb_kernel<SEL_THREADS, true, GTV, AP, CPV>,         \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max);\
        cudaFuncSetAttribute(topb_kernel<SEL_THREADS, false, GTV, AP, CPV>,        \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max);\
        cudaFuncSetAttribute(topb_kernel<SEL_THREADS, false, GTV, AP, CPV>,        \
                             cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
#define LOCKS_SEL_ATTR(GTV)                                                        \
    LOCKS_SEL_ATTR_A(GTV, false, false) LOCKS_SEL_ATTR_A(GTV, true, false)         \
    LOCKS_SEL_ATTR_A(GTV, false, true)
        LOCKS_SEL_ATTR(1) LOCKS_SEL_ATTR(2) LOCKS_SEL_ATTR(4) LOCKS_SEL_ATTR(8)
        LOCKS_SEL_ATTR(16)
#undef LOCKS_SEL_ATTR
#undef LOCKS_SEL_ATTR_A
        attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cl, n_kv, n_req);
    cfg.blockDim = dim3(SEL_THREADS, 1, 1);
    cfg.dynamicSmemBytes = dyn_smem;
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
    cudaError_t e = cudaSuccess;
    if (link != nullptr) {
        LOCKS_REQUIRE(app == nullptr, LOCKS_ERR_ARG,
                      "locks_topb_select_cp: the carried KV write is not available "
                      "with context parallelism");
        LOCKS_DISPATCH_GT(G, (e = owner_mode
            ? cudaLaunchKernelEx(&cfg, topb_kernel<SEL_THREADS, true, GT, false, true>, p)
            : cudaLaunchKernelEx(&cfg, topb_kernel<SEL_THREADS, false, GT, false, true>, p)));
    } else if (app == nullptr) {
        LOCKS_DISPATCH_GT(G, (e = owner_mode
            ? cudaLaunchKernelEx(&cfg, topb_kernel<SEL_THREADS, true, GT, false, false>, p)
            : cudaLaunchKernelEx(&cfg, topb_kernel<SEL_THREADS, false, GT, false, false>, p)));
    } else {
        LOCKS_DISPATCH_GT(G, (e = owner_mode
            ? cudaLaunchKernelEx(&cfg, topb_kernel<SEL_THREADS, true, GT, true, false>, p)
            : cudaLaunchKernelEx(&cfg, topb_kernel<SEL_THREADS, false, GT, true, false>, p)));
    }
    if (e != cudaSuccess)
        return fail(LOCKS_ERR_LAUNCH, "locks_topb_select: %s",
                    cudaGetErrorString(e));
    return check_launch("locks_topb_select");
}

extern "C" int locks_topb_select(
    int combine, const float* score_h, float* score, uint32_t* hmax,
    const int32_t* n_pages, const int32_t* n_sel_hi, const int32_t* b_fix,
    int32_t* page_table, int32_t* page_cnt, int n_req, int n_kv, int G,
    int max_pages, int sink_pages, locks_stream_t stream) {
    return topb_select_impl(combine, score_h, score, hmax, n_pages, n_sel_hi, b_fix,
                            page_table, page_cnt, n_req, n_kv, G, max_pages,
                            sink_pages, nullptr, stream);
}

extern "C" int locks_topb_select_rows(
    int combine, const float* score_h, float* score, uint32_t* hmax,
    const int32_t* n_pages, const int32_t* n_sel_hi, const int32_t* b_fix,
    int32_t* page_table, int32_t* page_cnt, int n_req, int n_kv, int G,
    int max_pages, int sink_pages, const int32_t* row_order,
    locks_stream_t stream) {
    return topb_select_impl(combine, score_h, score, hmax, n_pages, n_sel_hi, b_fix,
                            page_table, page_cnt, n_req, n_kv, G, max_pages,
                            sink_pages, nullptr, stream, nullptr, nullptr, row_order);
}

extern "C" int locks_row_order(const int32_t* n_pages, const int32_t* n_sel_hi,
                               const int32_t* b_fix, int n_req, int sink_pages,
                               int32_t* order_select, int32_t* order_decode,
                               locks_stream_t stream) {
    using namespace locks;
    LOCKS_REQUIRE(n_pages && n_sel_hi && b_fix && order_select && order_decode,
                  LOCKS_ERR_ARG, "locks_row_order: null pointer argument");
    LOCKS_REQUIRE(n_req >= 0 && n_req <= 4096 && sink_pages >= 0, LOCKS_ERR_ARG,
                  "locks_row_order: supports up to 4096 rows, got %d", n_req);
    if (n_req == 0) return LOCKS_OK;
    row_order_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        n_pages, n_sel_hi, b_fix, n_req, sink_pages, order_select, order_decode);
    pdl_break();
    return check_launch("locks_row_order");
}

extern "C" int locks_topb_select_cp(
    const float* score_h, float* score, uint32_t* hmax, const int32_t* n_pages,
    const int32_t* n_sel_hi, const int32_t* b_fix, int32_t* page_table,
    int32_t* page_cnt, int n_kv, int G, int max_pages, int sink_pages,
    const locks_cp_link_t* link, int* status, locks_stream_t stream) {
    using namespace locks;
    LOCKS_REQUIRE(link != nullptr, LOCKS_ERR_ARG,
                  "locks_topb_select_cp: null link description");
    return topb_select_impl(LOCKS_COMBINE_NRM, score_h, score, hmax, n_pages,
                            n_sel_hi, b_fix, page_table, page_cnt, 1, n_kv, G,
                            max_pages, sink_pages, nullptr, stream, link, status);
}

extern "C" int locks_topb_select_append(
    int combine, const float* score_h, float* score, uint32_t* hmax,
    const int32_t* n_pages, const int32_t* n_sel_hi, const int32_t* b_fix,
    int32_t* page_table, int32_t* page_cnt, int n_req, int n_kv, int G,
    int max_pages, int sink_pages, const locks_kv_append_t* append,
    locks_stream_t stream) {
    using namespace locks;
    LOCKS_REQUIRE(append != nullptr, LOCKS_ERR_ARG,
                  "locks_topb_select_append: null append description");
    return topb_select_impl(combine, score_h, score, hmax, n_pages, n_sel_hi, b_fix,
                            page_table, page_cnt, n_req, n_kv, G, max_pages,
                            sink_pages, append, stream);
}
