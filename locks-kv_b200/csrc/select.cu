// Per-step page parameters, GQA score combine and exact top-b page selection.
//
// topb kernel: one CTA of 1024 threads per (request, kv-head).
//   1. combine the per-head scores into one score per page (nrm or max),
//   2. find the b-th largest score of the selectable range with a 4-pass MSD
//      radix select on order-preserving 32-bit keys (256-bin shared histogram,
//      the digit picked by one warp with a shuffle scan),
//   3. keep flags with the exact-b tie rule, block-wide exclusive scans for the
//      tie ranks and the output slots, ascending compaction, -1 padding.
#include "common.cuh"

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
    __shared__ int hist[256];
    __shared__ int warp_tot[32];
    __shared__ float wmax[SEL_WARPS][MAX_G];
    __shared__ float hm_sh[MAX_G];
    __shared__ uint32_t sh_prefix;
    __shared__ int sh_k;

    const int kh = blockIdx.x, r = blockIdx.y;
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

    // ---------------- 1. GQA combine -> score[0, n_comb) ----------------------
    if (p.combine != LOCKS_COMBINE_NONE && n_comb > 0) {
        const float* sh = p.score_h + row * (int64_t)G * MP;
        if (p.combine == LOCKS_COMBINE_NRM) {
            if (p.hmax != nullptr) {
                if (tid < G) {
                    uint32_t* hp = &p.hmax[row * G + tid];
                    hm_sh[tid] = key2f(*hp);
                    *hp = 0u;
                }
            } else {
                float lmax[MAX_G];
#pragma unroll
                for (int g = 0; g < MAX_G; ++g) lmax[g] = -INFINITY;
                for (int i = tid; i < n_comb; i += SEL_THREADS) {
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
                        if (lane == 0) wmax[warp][g] = m;
                    }
                }
                __syncthreads();
                if (tid < G) {
                    float m = -INFINITY;
                    for (int w = 0; w < SEL_WARPS; ++w) m = fmaxf(m, wmax[w][tid]);
                    hm_sh[tid] = m;
                }
            }
            __syncthreads();
            float hm[MAX_G];
#pragma unroll
            for (int g = 0; g < MAX_G; ++g) hm[g] = (g < G) ? hm_sh[g] : 0.f;
            for (int i = tid; i < n_comb; i += SEL_THREADS) {
                float acc = 0.f;
#pragma unroll
                for (int g = 0; g < MAX_G; ++g)
                    if (g < G) acc += __expf(sh[(int64_t)g * MP + i] - hm[g]);
                score[i] = acc;
            }
        } else {                                    // LOCKS_COMBINE_MAX
            for (int i = tid; i < n_comb; i += SEL_THREADS) {
                float m = -INFINITY;
                for (int g = 0; g < G; ++g)
                    m = fmaxf(m, sh[(int64_t)g * MP + i]);
                score[i] = m;
            }
        }
        __syncthreads();
    }

    // ---------------- 2. threshold key (b-th largest of [lo, hi)) -------------
    uint32_t tau_key = 0u;       // below every real key: everything is "> tau"
    int quota = 0;
    if (!keep_all && b < L) {
        b = max(b, 1);
        uint32_t prefix = 0u, mask = 0u;
        int k = b;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int i = tid; i < 256; i += SEL_THREADS) hist[i] = 0;
            __syncthreads();
            for (int i = lo + tid; i < hi; i += SEL_THREADS) {
                const uint32_t key = f2key(score[i]);
                if ((key & mask) == prefix)
                    atomicAdd(&hist[(key >> shift) & 255u], 1);
            }
            __syncthreads();
            if (warp == 0) {
                // lane l owns bins 255-8l .. 248-8l (descending)
                int cnt8[8], lsum = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    cnt8[j] = hist[255 - 8 * lane - j];
                    lsum += cnt8[j];
                }
                int inc = lsum;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int t = __shfl_up_sync(0xffffffffu, inc, o);
                    if (lane >= o) inc += t;
                }
                const int above = inc - lsum;       // count in higher bins
                if (above < k && k <= inc) {
                    int a = above;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (a < k && k <= a + cnt8[j]) {
                            sh_prefix = prefix |
                                ((uint32_t)(255 - 8 * lane - j) << shift);
                            sh_k = k - a;
                        }
                        a += cnt8[j];
                    }
                }
            }
            __syncthreads();
            prefix = sh_prefix;
            k = sh_k;
            mask |= 255u << shift;
        }
        tau_key = prefix;
        quota = k;
    }

    // ---------------- 3. keep flags + ascending compaction --------------------
    const int per = (npg + SEL_THREADS - 1) / SEL_THREADS;
    const int c0 = min(tid * per, npg), c1 = min(c0 + per, npg);
    int n_eq = 0;
    if (!keep_all)
        for (int i = max(c0, lo); i < min(c1, hi); ++i)
            n_eq += (f2key(score[i]) == tau_key);
    int tot_eq;
    const int eq_base = block_exclusive_scan(n_eq, warp_tot, tot_eq);
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
    int cnt;
    int pos = block_exclusive_scan(kept, warp_tot, cnt);
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
    for (int i = cnt + tid; i < MP; i += SEL_THREADS) tab[i] = -1;
    if (tid == 0) p.page_cnt[row] = cnt;
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
    topb_kernel<<<dim3(n_kv, n_req), SEL_THREADS, 0,
                  static_cast<cudaStream_t>(stream)>>>(p);
    return check_launch("locks_topb_select");
}
