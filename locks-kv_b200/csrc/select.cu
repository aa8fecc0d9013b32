// Per-step page parameters, GQA score combine and exact top-b page selection.
//
// topb kernel: one thread-block CLUSTER (1..8 CTAs of 1024 threads) per
// (request, kv-head); CTA c owns a contiguous slice of the pages.
//   1. combine the per-head scores of the slice into one score per page (nrm
//      or max); the per-head maxima come from the scorer's published keys or
//      from a cluster-wide sweep,
//   2. find the b-th largest score of the selectable range with a 3-pass MSD
//      radix select (11/11/10 bits) on order-preserving 32-bit keys: every CTA
//      histograms its slice in shared memory, the cluster meets at a hardware
//      barrier, every CTA adds up all slices' histograms through distributed
//      shared memory and picks the digit with a block-wide suffix scan,
//   3. keep flags with the exact-b tie rule; tie ranks and output slots come
//      from block scans plus a cluster exchange of per-CTA totals; ascending
//      compaction, -1 padding.
// No global scratch and a single launch for any page count.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace locks {
namespace {

constexpr int SEL_THREADS = 1024;
constexpr int SEL_WARPS = SEL_THREADS / 32;
constexpr int MAX_G = 16;

__global__ void derive_kernel(const int32_t* __restrict__ seq_lens, int n_req,
                              int page, int window, int sink, int budget_pages,
                              double budget, int32_t* __restrict__ n_pages,
                              int32_t* __restrict__ n_sel_hi,
                              int32_t* __restrict__ b_fix) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_req) return;
    const int sl = seq_lens[i];
    const int npg = (sl + page - 1) / page;
    const int nsh = npg - window;
    const int s = nsh - sink;
    int b;
    if (budget_pages > 0) {
        b = max(min(budget_pages, max(s, 1)), 1);
    } else {
        const double bf = ceil((double)s * budget);
        b = min(max((int)bf, 1), max(s, 1));
    }
    n_pages[i] = npg;
    n_sel_hi[i] = nsh;
    b_fix[i] = b;
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
};

constexpr int RBITS0 = 11, RBITS1 = 11, RBITS2 = 10;
constexpr int NBINS = 1 << RBITS0;                // 2048 (largest digit)
constexpr int MAX_CL = 8;

struct SelSmem {
    int hist[2][NBINS];
    int warp_tot[32];
    float wmax[SEL_WARPS][MAX_G];
    float xmax[MAX_G];             // this CTA's per-head maxima (cluster sweep)
    float hm_sh[MAX_G];
    uint32_t sh_prefix;
    int sh_k;
    int x_eq;                      // this CTA's tie count / kept count
    int x_kept;
};

// exclusive prefix sum of one int per thread over the whole CTA;
// `total` receives the CTA-wide sum.  `warp_tot` is 32 ints of scratch.
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_tot,
                                                    int& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();                       // protect warp_tot reuse
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    int wv = (lane < SEL_WARPS) ? warp_tot[lane] : 0;
    int winc = wv;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, winc, o);
        if (lane >= o) winc += t;
    }
    total = __shfl_sync(0xffffffffu, winc, 31);
    const int wbase = __shfl_sync(0xffffffffu, winc - wv, warp);
    return wbase + inc - v;
}

__global__ void __launch_bounds__(SEL_THREADS)
topb_kernel(const SelParams p) {
    __shared__ SelSmem sm;
    cg::cluster_group cluster = cg::this_cluster();

    const int c = blockIdx.x, CL = gridDim.x;     // rank / size of the cluster
    const int kh = blockIdx.y, r = blockIdx.z;
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

    // contiguous page slice of this CTA (covers [0, max(npg, n_comb)))
    const int span = max(npg, n_comb);
    const int per_cta = (span + CL - 1) / CL;
    const int s0 = min(c * per_cta, span), s1 = min(s0 + per_cta, span);

    // ---------------- 1. GQA combine -> score[slice] --------------------------
    if (p.combine != LOCKS_COMBINE_NONE && n_comb > 0) {
        const float* sh = p.score_h + row * (int64_t)G * MP;
        const int e0 = s0, e1 = min(s1, n_comb);
        if (p.combine == LOCKS_COMBINE_NRM) {
            if (p.hmax != nullptr) {
                if (tid < G) sm.hm_sh[tid] = key2f(p.hmax[row * G + tid]);
                cluster.sync();                     // everyone has read the keys
                if (c == 0 && tid < G) p.hmax[row * G + tid] = 0u;
            } else {
                float lmax[MAX_G];
#pragma unroll
                for (int g = 0; g < MAX_G; ++g) lmax[g] = -INFINITY;
                for (int i = e0 + tid; i < e1; i += SEL_THREADS) {
#pragma unroll
                    for (int g = 0; g < MAX_G; ++g)
                        if (g < G)
                            lmax[g] = fmaxf(lmax[g], sh[(int64_t)g * MP + i]);
                }
#pragma unroll
                for (int g = 0; g < MAX_G; ++g) {
                    if (g < G) {
                        float m = lmax[g];
#pragma unroll
                        for (int o = 16; o >= 1; o >>= 1)
                            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                        if (lane == 0) sm.wmax[warp][g] = m;
                    }
                }
                __syncthreads();
                if (tid < G) {
                    float m = -INFINITY;
                    for (int w = 0; w < SEL_WARPS; ++w)
                        m = fmaxf(m, sm.wmax[w][tid]);
                    sm.xmax[tid] = m;
                }
                cluster.sync();
                if (tid < G) {
                    float m = -INFINITY;
                    for (int cc = 0; cc < CL; ++cc)
                        m = fmaxf(m, *cluster.map_shared_rank(&sm.xmax[tid], cc));
                    sm.hm_sh[tid] = m;
                }
            }
            __syncthreads();
            float hm[MAX_G];
#pragma unroll
            for (int g = 0; g < MAX_G; ++g) hm[g] = (g < G) ? sm.hm_sh[g] : 0.f;
            for (int i = e0 + tid; i < e1; i += SEL_THREADS) {
                float acc = 0.f;
#pragma unroll
                for (int g = 0; g < MAX_G; ++g)
                    if (g < G) acc += __expf(sh[(int64_t)g * MP + i] - hm[g]);
                score[i] = acc;
            }
        } else {                                    // LOCKS_COMBINE_MAX
            for (int i = e0 + tid; i < e1; i += SEL_THREADS) {
                float m = -INFINITY;
                for (int g = 0; g < G; ++g)
                    m = fmaxf(m, sh[(int64_t)g * MP + i]);
                score[i] = m;
            }
        }
        __syncthreads();        // this CTA re-reads only its own slice of score
    }

    // selectable part of the slice
    const int q0 = max(s0, lo), q1 = min(s1, hi);

    // ---------------- 2. threshold key (b-th largest of [lo, hi)) -------------
    uint32_t tau_key = 0u;       // below every real key: everything is "> tau"
    int quota = 0;
    if (!keep_all && b < L) {
        b = max(b, 1);
        uint32_t prefix = 0u, mask = 0u;
        int k = b;
        int shift = 32;
#pragma unroll 1
        for (int pass = 0; pass < 3; ++pass) {
            const int bits = (pass == 0) ? RBITS0 : (pass == 1) ? RBITS1 : RBITS2;
            shift -= bits;
            const uint32_t dmask = (1u << bits) - 1u;
            int* hist = sm.hist[pass & 1];
            for (int i = tid; i < NBINS; i += SEL_THREADS) hist[i] = 0;
            __syncthreads();
            for (int i = q0 + tid; i < q1; i += SEL_THREADS) {
                const uint32_t key = f2key(score[i]);
                if ((key & mask) == prefix)
                    atomicAdd(&hist[(key >> shift) & dmask], 1);
            }
            cluster.sync();                 // all slices' histograms are complete
            // thread t owns bins (NBINS-1-2t) and (NBINS-2-2t): descending order
            const int bin_a = NBINS - 1 - 2 * tid, bin_b = bin_a - 1;
            int ca = 0, cb = 0;
            for (int cc = 0; cc < CL; ++cc) {
                const int* rh = cluster.map_shared_rank(hist, cc);
                ca += rh[bin_a];
                cb += rh[bin_b];
            }
            int tot;
            const int above = block_exclusive_scan(ca + cb, sm.warp_tot, tot);
            if (above < k && k <= above + ca + cb) {
                if (k <= above + ca) {
                    sm.sh_prefix = prefix | ((uint32_t)bin_a << shift);
                    sm.sh_k = k - above;
                } else {
                    sm.sh_prefix = prefix | ((uint32_t)bin_b << shift);
                    sm.sh_k = k - above - ca;
                }
            }
            __syncthreads();
            prefix = sm.sh_prefix;
            k = sm.sh_k;
            mask |= dmask << shift;
        }
        tau_key = prefix;
        quota = k;
    }

    // ---------------- 3. keep flags + ascending compaction --------------------
    // thread-contiguous chunks inside the slice [s0, min(s1, npg))
    const int t1 = min(s1, npg), t0 = min(s0, t1);
    const int per = (t1 - t0 + SEL_THREADS - 1) / SEL_THREADS;
    const int c0 = min(t0 + tid * per, t1), c1 = min(c0 + per, t1);
    int n_eq = 0;
    if (!keep_all)
        for (int i = max(c0, lo); i < min(c1, hi); ++i)
            n_eq += (f2key(score[i]) == tau_key);
    int tot_eq;
    int eq_base = block_exclusive_scan(n_eq, sm.warp_tot, tot_eq);
    if (tid == 0) sm.x_eq = tot_eq;
    cluster.sync();
    for (int cc = 0; cc < c; ++cc)
        eq_base += *cluster.map_shared_rank(&sm.x_eq, cc);
    int kept = 0;
    {
        int eqr = eq_base;
        for (int i = c0; i < c1; ++i) {
            bool keep = true;
            if (!keep_all && i >= lo && i < hi) {
                const uint32_t key = f2key(score[i]);
                if (key == tau_key) keep = (++eqr <= quota);
                else keep = key > tau_key;
            }
            kept += keep;
        }
    }
    int tot_kept;
    int pos = block_exclusive_scan(kept, sm.warp_tot, tot_kept);
    if (tid == 0) sm.x_kept = tot_kept;
    cluster.sync();
    int cnt = 0;
    for (int cc = 0; cc < CL; ++cc) {
        const int v = *cluster.map_shared_rank(&sm.x_kept, cc);
        if (cc < c) pos += v;
        cnt += v;
    }
    int32_t* tab = p.page_table + row * MP;
    {
        int eqr = eq_base;
        for (int i = c0; i < c1; ++i) {
            bool keep = true;
            if (!keep_all && i >= lo && i < hi) {
                const uint32_t key = f2key(score[i]);
                if (key == tau_key) keep = (++eqr <= quota);
                else keep = key > tau_key;
            }
            if (keep) tab[pos++] = i;
        }
    }
    // -1 padding of [cnt, MP), shared by the cluster
    for (int i = cnt + c * SEL_THREADS + tid; i < MP; i += CL * SEL_THREADS)
        tab[i] = -1;
    if (c == 0 && tid == 0) p.page_cnt[row] = cnt;
    cluster.sync();              // keep shared memory alive for remote readers
}

}  // namespace
}  // namespace locks

extern "C" int locks_derive_page_params(
    const int32_t* seq_lens, int n_req, int page, int window_pages,
    int sink_pages, int budget_pages, double budget, int32_t* n_pages,
    int32_t* n_sel_hi, int32_t* b_fix, locks_stream_t stream) {
    using namespace locks;
    LOCKS_REQUIRE(seq_lens && n_pages && n_sel_hi && b_fix, LOCKS_ERR_ARG,
                  "locks_derive_page_params: null pointer argument");
    LOCKS_REQUIRE(n_req >= 0 && page > 0 && window_pages >= 0 && sink_pages >= 0,
                  LOCKS_ERR_ARG, "locks_derive_page_params: bad size argument");
    if (n_req == 0) return LOCKS_OK;
    derive_kernel<<<(n_req + 127) / 128, 128, 0,
                    static_cast<cudaStream_t>(stream)>>>(
        seq_lens, n_req, page, window_pages, sink_pages, budget_pages, budget,
        n_pages, n_sel_hi, b_fix);
    return check_launch("locks_derive_page_params");
}

extern "C" int locks_topb_select(
    int combine, const float* score_h, float* score, uint32_t* hmax,
    const int32_t* n_pages, const int32_t* n_sel_hi, const int32_t* b_fix,
    int32_t* page_table, int32_t* page_cnt, int n_req, int n_kv, int G,
    int max_pages, int sink_pages, locks_stream_t stream) {
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
    // cluster size: spread one (request, kv-head) over up to 8 SMs when the
    // grid is small; a power of two; never more CTAs than 1024-page slices
    int cl = 1;
    {
        const int want = sm_count() / max(1, n_kv * n_req);
        const int useful = (max_pages + SEL_THREADS - 1) / SEL_THREADS;
        while (cl * 2 <= want && cl * 2 <= useful && cl < MAX_CL) cl *= 2;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cl, n_kv, n_req);
    cfg.blockDim = dim3(SEL_THREADS, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cl;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, topb_kernel, p);
    if (e != cudaSuccess)
        return fail(LOCKS_ERR_LAUNCH, "locks_topb_select: %s",
                    cudaGetErrorString(e));
    return check_launch("locks_topb_select");
}
