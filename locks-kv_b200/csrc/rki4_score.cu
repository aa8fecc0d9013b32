// Page scorer: per-head page log-sum-exp from the packed rki4 summary records.
//
// Grid (zsplit, n_kv, n_req), 128 threads, 4 CTAs per SM.  The W = 4 * zsplit
// warps of a (request, kv-head) run INDEPENDENTLY and share its pages in chunks
// of 8, dealt round-robin (warp gw takes chunks gw, gw + W, ...: neighbouring
// warps read neighbouring block-table entries).  Each warp owns a 2-stage shared-
// memory ring: eight lanes turn block-table entries into record addresses and
// issue one 832-byte bulk async copy each (a record is one contiguous burst);
// completion is tracked by the warp's own mbarrier, so the main loop has no
// CTA-wide barrier.
//
// A chunk is scored with warp-level tensor-core fragments whose rows are the
// query heads of the GQA group:
//
//   mu.q     s8 x s8  m16n8k32, the 8 pages of the chunk as the 8 columns
//   V^T q    s8 x s8  m16n8k32, 4 k-steps per page; an int4 code is used in
//            the high half of a byte (code * 16, still a signed byte: one shift
//            and two masks per 8 codes), the factor 16 goes into the scale
//   C qt     f16      m16n8k16: qt = hi + lo in fp16 (22 significant bits);
//            C (int8) is exact in fp16
//   LSE      base-2, 4 tokens per lane, two shuffle steps for max and for sum
//
// With G <= 4 the 8 live fragment rows hold the group twice, and two pages are
// scored per pass: the k dimension of the C product is split between the two
// pages (block-diagonal A), so rows 0-3 come out as page A and rows 4-7 as page
// B, and the conversion / LSE / store work is done once per PAIR of pages.
//
// The integer dot products are exact, so score_h differs from an fp32
// evaluation only by summation order and the ex2/lg2 approximations.
#include "common.cuh"

namespace locks {
namespace {

constexpr int CHUNK = 8;                       // pages per ring stage (= mma n)
constexpr int STAGES = 2;
constexpr int NWARP = 4;
constexpr int NTHREADS = NWARP * 32;
constexpr int CTAS_PER_SM = 4;

struct __align__(128) ScoreSmem {
    uint8_t rec[NWARP][STAGES][CHUNK][REC_BYTES];
    int8_t q8[16][128];
    float qs[16];
    uint64_t full[NWARP][STAGES];
};

struct ScoreParams {
    const __nv_bfloat16* q;
    int64_t q_stride_req;
    const uint8_t* records;
    const int32_t* block_table;
    int64_t bt_stride;
    const int32_t* n_sel_hi;
    float* score_h;
    uint32_t* hmax;
    int n_kv, G, max_pages, bt_width, num_blocks;
    int n_req, ragged;
    const int32_t* row_order;  // ragged: the requests are dealt in this order (or 0, 1, ...)
    float scale;
    int* status;
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// D(16x8,f32) = A(16x16,f16,row) * B(16x8,f16,col) + C
__device__ __forceinline__ void mma_f16_k16(float (&d)[4], uint32_t a0,
                                            uint32_t a1, uint32_t a2,
                                            uint32_t a3, uint32_t b0,
                                            uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D = A * B   (zero accumulator)
__device__ __forceinline__ void mma_f16_k16_z(float (&d)[4], uint32_t a0,
                                              uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
// f0, f1 -> packed fp16 (hi parts) and packed fp16 (residuals)
__device__ __forceinline__ void split_f16x2(float f0, float f1, uint32_t& hi,
                                            uint32_t& lo) {
    const __half2 h = __floats2half2_rn(f0, f1);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(f0 - hf.x, f1 - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}
// two int8 (low 16 bits of cc) -> packed fp16, exactly
__device__ __forceinline__ uint32_t s8x2_to_f16x2(uint32_t cc) {
    const uint32_t biased = __byte_perm(cc ^ 0x8080u, 0x64646464u, 0x4140);
    const __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&biased),
                              __floats2half2_rn(1152.f, 1152.f));
    return *reinterpret_cast<const uint32_t*>(&h);
}

// c[row][r] = 16 * sum_d q8[row][d] * code[d][r] for one page
template <bool HI>
__device__ __forceinline__ void project_page(int (&c)[4], const uint8_t* rec,
                                             int gid, int tig,
                                             const uint32_t (&qe)[4],
                                             const uint32_t (&qo)[4],
                                             const uint32_t (&qe_hi)[4],
                                             const uint32_t (&qo_hi)[4]) {
    const uint4 vw =
        *reinterpret_cast<const uint4*>(rec + RO_V4 + gid * 64 + tig * 16);
    const uint32_t vword[4] = {vw.x, vw.y, vw.z, vw.w};
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const uint32_t even = (vword[s] << 4) & 0xF0F0F0F0u;   // low nibbles * 16
        const uint32_t odd = vword[s] & 0xF0F0F0F0u;           // high nibbles * 16
        if (s == 0)
            mma_s8s8_k32_z(c, qe[s], HI ? qe_hi[s] : 0u, qo[s], HI ? qo_hi[s] : 0u,
                           even, odd);
        else
            mma_s8s8_k32(c, qe[s], HI ? qe_hi[s] : 0u, qo[s], HI ? qo_hi[s] : 0u,
                         even, odd);
    }
}

// base-2 log-sum-exp of 4 values per lane over the 4 lanes of a quad
__device__ __forceinline__ float quad_lse2(float t0, float t1, float t2,
                                           float t3) {
    float mx = fmaxf(fmaxf(t0, t1), fmaxf(t2, t3));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    float sum = ex2_approx(t0 - mx) + ex2_approx(t1 - mx) +
                ex2_approx(t2 - mx) + ex2_approx(t3 - mx);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    return mx + lg2_approx(sum);
}


// GP = 4 : G <= 4, two pages per pass;  GP = 8 : G <= 8;  GP = 16 : G <= 16
template <int GP>
__global__ void __launch_bounds__(NTHREADS, CTAS_PER_SM)
rki4_score_kernel(const ScoreParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    ScoreSmem& sm = *reinterpret_cast<ScoreSmem*>(smem_raw);

    const int kh = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int z = blockIdx.x, Z = gridDim.x, r = blockIdx.z;
    if (p.ragged) {
        // Ragged batch: the gridDim.x CTAs of a kv-head are dealt to the requests
        // in proportion to their chunk counts (every request gets one, the other
        // `extra` go by share), so a 4K-token row and a 70K-token row finish
        // together.  Every lane walks requests lane, lane + 32, ...; the CTA's
        // request is the one whose run of CTAs contains blockIdx.x.
        const int R = p.n_req, cap0 = min(p.max_pages, p.bt_width);
        const int extra = (int)gridDim.x - R, b = (int)blockIdx.x;
        // (with a launch order the longest requests come first in the grid, so
        // the CTAs that start last are the light ones)
        auto req_at = [&](int i) -> int { return p.row_order ? p.row_order[i] : i; };
        int total = 0;
        for (int i = lane; i < R; i += 32)
            total += (min(max(p.n_sel_hi[req_at(i)], 0), cap0) + CHUNK - 1) / CHUNK;
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1)
            total += __shfl_xor_sync(0xffffffffu, total, o);
        // request i owns CTAs [i + floor(extra * c_before / total),
        //                      i + 1 + floor(extra * c_through / total)):
        // the runs tile the grid exactly, whatever the rounding
        int acc = 0;                                        // chunks of requests < i0
        r = -1;
        for (int i0 = 0; i0 < R && r < 0; i0 += 32) {
            const int i = i0 + lane;
            const int ri = (i < R) ? req_at(i) : 0;
            const int ci = (i < R)
                ? (min(max(p.n_sel_hi[ri], 0), cap0) + CHUNK - 1) / CHUNK : 0;
            int inc = ci;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += t;
            }
            const int64_t c_before = acc + inc - ci, c_through = acc + inc;
            const int beg = i + (int)((extra * c_before) / max(total, 1));
            const int end = i + 1 + (int)((extra * c_through) / max(total, 1));
            const bool hit = i < R && b >= beg && b < end;
            const uint32_t m = __ballot_sync(0xffffffffu, hit);
            if (m) {
                const int src = __ffs(m) - 1;
                r = __shfl_sync(0xffffffffu, ri, src);
                z = b - __shfl_sync(0xffffffffu, beg, src);
                Z = __shfl_sync(0xffffffffu, end - beg, src);
            }
            acc += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (r < 0) return;                       // (no request: an empty batch)
    }
    const int gid = lane >> 2, tig = lane & 3;
    const int G = p.G;

    // Warp gw takes chunks gw, gw + W, gw + 2W, ...  The first two chunks' place
    // does not depend on the page count, so their block-table entries are fetched
    // together with it and the copies start one round trip earlier.
    const int W = NWARP * Z;
    // warp-major numbering: when the chunks do not divide evenly, the warps that
    // take one chunk more are spread over all CTAs (and SMs) instead of filling
    // the first CTAs
    const int gw = warp * Z + z;
    const int cap = min(p.max_pages, p.bt_width);
    const int32_t* bt = p.block_table + (int64_t)r * p.bt_stride;
    auto bt_at = [&](int page0) -> int {
        const int pg = page0 + lane;
        return (lane < CHUNK && pg < cap) ? bt[pg] : 0;
    };
    const int blk0 = bt_at(gw * CHUNK), blk1 = bt_at((gw + W) * CHUNK);
    const int n_hi = min(p.n_sel_hi[r], cap);
    if (n_hi <= 0) return;
    const int NC = (n_hi + CHUNK - 1) / CHUNK;
    const int n_items = (gw < NC) ? (NC - gw + W - 1) / W : 0;
    auto item_page0 = [&](int k) -> int { return (gw + k * W) * CHUNK; };
    auto item_len = [&](int k) -> int { return min(CHUNK, n_hi - item_page0(k)); };

    if (tid == 0) {
        for (int w = 0; w < NWARP; ++w)
            for (int s = 0; s < STAGES; ++s) mbar_init(&sm.full[w][s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    const uint8_t* recs = p.records + (int64_t)kh * REC_BYTES;
    const int64_t blk_stride = (int64_t)p.n_kv * REC_BYTES;
    // summaries are streamed once per step: do not let them push the scores,
    // page tables and K/V pages of the following kernels out of L2
    const uint64_t stream_policy = l2_policy_evict_first();
    auto issue = [&](int stage, int n, int blk) {
        fence_proxy_async();
        if (lane == 0)
            mbar_expect_tx(&sm.full[warp][stage], (uint32_t)n * REC_BYTES);
        __syncwarp();
        if (lane < n) {
            blk = min(max(blk, 0), p.num_blocks - 1);
            bulk_g2s_hint(&sm.rec[warp][stage][lane][0], recs + blk * blk_stride,
                          REC_BYTES, &sm.full[warp][stage], stream_policy);
        }
    };
    if (n_items > 0) issue(0, item_len(0), blk0);
    if (n_items > 1) issue(1, item_len(1), blk1);

    // Everything above touches only per-step constants (block table, page
    // counts, summaries); q and the score buffers belong to the kernels before.
    // The selector may be scheduled as soon as CTAs of this grid retire: its
    // prologue then overlaps the scorer's tail (it waits for the whole grid).
    pdl_trigger();
    pdl_wait();

    // ---- per-head int8 round trip of q (overlaps the first copies) ----------
    for (int g = warp; g < G; g += NWARP) {
        const __nv_bfloat16* qp =
            p.q + (int64_t)r * p.q_stride_req + (int64_t)(kh * G + g) * 128;
        const uint2 raw = *reinterpret_cast<const uint2*>(qp + 4 * lane);
        float v[4] = {bf16_bits_to_f32(raw.x & 0xFFFFu),
                      bf16_bits_to_f32(raw.x >> 16),
                      bf16_bits_to_f32(raw.y & 0xFFFFu),
                      bf16_bits_to_f32(raw.y >> 16)};
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])),
                           fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1)
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float qs = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
        uint32_t packed = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = __float2int_rn(__fdiv_rn(v[i], qs));
            packed |= (uint32_t)(c & 0xFF) << (8 * i);
        }
        *reinterpret_cast<uint32_t*>(&sm.q8[g][4 * lane]) = packed;
        if (lane == 0) sm.qs[g] = qs;
    }
    __syncthreads();

    // ---- A fragments of q.  Row gid holds head gid % GP (the group is repeated
    // when it is shorter than 8 rows); rows 8..15 are used only for GP = 16. ----
    const float scale2 = p.scale * 1.4426950408889634f;     // base-2 logits
    constexpr int NR = (GP == 16) ? 2 : 1;
    constexpr bool HI = (GP == 16);
    constexpr int GROW = (GP < 8) ? GP : 8;
    uint32_t qn[NR][8], qe[NR][4], qo[NR][4];
    float qsc[NR];         // q scale * log2(e) * softmax scale (mu . q term)
    float qsv[NR];         // the same / 16 (the V codes enter as code * 16)
#pragma unroll
    for (int h = 0; h < NR; ++h) {
        const int g = (gid % GROW) + 8 * h;
        const bool live = g < G;
        const uint32_t* row =
            reinterpret_cast<const uint32_t*>(&sm.q8[live ? g : 0][0]);
#pragma unroll
        for (int i = 0; i < 8; ++i) qn[h][i] = live ? row[8 * tig + i] : 0u;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const int j = 4 * tig + s;               // packed V word index
            const uint32_t n0 = live ? row[2 * j] : 0u;
            const uint32_t n1 = live ? row[2 * j + 1] : 0u;
            qe[h][s] = __byte_perm(n0, n1, 0x6420);
            qo[h][s] = __byte_perm(n0, n1, 0x7531);
        }
        qsc[h] = live ? sm.qs[g] * scale2 : 0.f;
        qsv[h] = qsc[h] * 0.0625f;
    }

    float run_max[NR];
#pragma unroll
    for (int h = 0; h < NR; ++h) run_max[h] = -INFINITY;
    constexpr float LN2 = 0.6931471805599453f;
    float* out_base =
        p.score_h + ((int64_t)r * p.n_kv + kh) * (int64_t)G * p.max_pages;

    for (int k = 0; k < n_items; ++k) {
        const int stage = k & 1;
        const int p0 = item_page0(k);
        const int n = item_len(k);
        // block-table entries of the item that will reuse this stage
        const int next_blk = (k + 2 < n_items) ? bt_at(item_page0(k + 2)) : 0;
        mbar_wait(&sm.full[warp][stage], (uint32_t)((k >> 1) & 1), p.status);
        const uint8_t* crec = &sm.rec[warp][stage][0][0];

        // mu . q for the chunk's 8 pages: column (n) = page slot gid
        int muc[4];
        {
            const uint8_t* mrec = crec + gid * REC_BYTES + RO_MU8 + 32 * tig;
            const uint4 m0 = *reinterpret_cast<const uint4*>(mrec);
            const uint4 m1 = *reinterpret_cast<const uint4*>(mrec + 16);
            const uint32_t mw[8] = {m0.x, m0.y, m0.z, m0.w,
                                    m1.x, m1.y, m1.z, m1.w};
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                if (s == 0)
                    mma_s8s8_k32_z(muc, qn[0][0], HI ? qn[NR - 1][0] : 0u, qn[0][1],
                                   HI ? qn[NR - 1][1] : 0u, mw[0], mw[1]);
                else
                    mma_s8s8_k32(muc, qn[0][2 * s], HI ? qn[NR - 1][2 * s] : 0u,
                                 qn[0][2 * s + 1], HI ? qn[NR - 1][2 * s + 1] : 0u,
                                 mw[2 * s], mw[2 * s + 1]);
            }
        }

        if constexpr (GP == 4) {
            // ---- two pages per pass: rows 0-3 -> slot 2j, rows 4-7 -> 2j+1 ----
            const int sel = gid >> 2;
            // no per-pair exit test: slots past n hold stale bytes whose results
            // are dropped, and without the branch the pairs' dependency chains
            // interleave; a chunk of at most 4 pages runs the 2-pair variant
            auto do_pair = [&](int j) {
                const uint8_t* recA = crec + (2 * j) * REC_BYTES;
                const uint8_t* recB = recA + REC_BYTES;
                const uint8_t* own = sel ? recB : recA;
                int cA[4], cB[4];
                project_page<false>(cA, recA, gid, tig, qe[0], qo[0], qe[0], qo[0]);
                project_page<false>(cB, recB, gid, tig, qe[0], qo[0], qe[0], qo[0]);
                const int c0 = sel ? cB[0] : cA[0];
                const int c1 = sel ? cB[1] : cA[1];
                const uint32_t vs2 =
                    *reinterpret_cast<const uint32_t*>(own + RO_VS + 4 * tig);
                const float mus = bf16_bits_to_f32(
                    *reinterpret_cast<const uint16_t*>(own + RO_MUS));
                // mu.q of slot 2j+sel: lane (gid, j), register sel
                const int mq = __shfl_sync(0xffffffffu, sel ? muc[1] : muc[0],
                                           (lane & ~3) | j);
                uint32_t a_hi, a_lo;
                split_f16x2(
                    (float)c0 * (qsv[0] * bf16_bits_to_f32(vs2 & 0xFFFFu)),
                    (float)c1 * (qsv[0] * bf16_bits_to_f32(vs2 >> 16)),
                    a_hi, a_lo);
                const float mud = (float)mq * (qsc[0] * mus);
                // block-diagonal A: k 0-7 multiply page A's C, k 8-15 page B's
                const uint32_t a0h = sel ? 0u : a_hi, a2h = sel ? a_hi : 0u;
                const uint32_t a0l = sel ? 0u : a_lo, a2l = sel ? a_lo : 0u;
                float x[2][4];
#pragma unroll
                for (int th = 0; th < 2; ++th) {
                    const int off = RO_C8 + (8 * th + gid) * 8 + 2 * tig;
                    const uint32_t bA = s8x2_to_f16x2(
                        *reinterpret_cast<const uint16_t*>(recA + off));
                    const uint32_t bB = s8x2_to_f16x2(
                        *reinterpret_cast<const uint16_t*>(recB + off));
                    mma_f16_k16_z(x[th], a0h, 0u, a2h, 0u, bA, bB);
                    mma_f16_k16(x[th], a0l, 0u, a2l, 0u, bA, bB);
                }
                const uint32_t csa =
                    *reinterpret_cast<const uint32_t*>(own + RO_CS + 4 * tig);
                const uint32_t csb =
                    *reinterpret_cast<const uint32_t*>(own + RO_CS + 16 + 4 * tig);
                const float S = LN2 * quad_lse2(
                    fmaf(bf16_bits_to_f32(csa & 0xFFFFu), x[0][0], mud),
                    fmaf(bf16_bits_to_f32(csa >> 16), x[0][1], mud),
                    fmaf(bf16_bits_to_f32(csb & 0xFFFFu), x[1][0], mud),
                    fmaf(bf16_bits_to_f32(csb >> 16), x[1][1], mud));
                const int slot = 2 * j + sel;
                const int g = gid & 3;
                if (slot < n && g < G) {
                    if (tig == 0)
                        out_base[(int64_t)g * p.max_pages + p0 + slot] = S;
                    run_max[0] = fmaxf(run_max[0], S);
                }
            };
            if (n > CHUNK / 2) {
#pragma unroll
                for (int j = 0; j < CHUNK / 2; ++j) do_pair(j);
            } else {
#pragma unroll
                for (int j = 0; j < CHUNK / 4; ++j) do_pair(j);
            }
        } else {
            // ---- one page per pass, rows = heads (8, or 16 with the hi rows) --
            // as above: no exit test inside the unrolled group of pages
#pragma unroll 8
            for (int i = 0; i < CHUNK; ++i) {
                const uint8_t* rec = crec + i * REC_BYTES;
                int c1[4];
                project_page<HI>(c1, rec, gid, tig, qe[0], qo[0], qe[NR - 1],
                                 qo[NR - 1]);
                const uint32_t vs2 =
                    *reinterpret_cast<const uint32_t*>(rec + RO_VS + 4 * tig);
                const float vs0 = bf16_bits_to_f32(vs2 & 0xFFFFu);
                const float vs1 = bf16_bits_to_f32(vs2 >> 16);
                const float mus = bf16_bits_to_f32(
                    *reinterpret_cast<const uint16_t*>(rec + RO_MUS));
                const int src_lane = (lane & ~3) | (i >> 1);
                const int mlo = __shfl_sync(
                    0xffffffffu, (i & 1) ? muc[1] : muc[0], src_lane);
                int mhi = 0;
                if (HI)
                    mhi = __shfl_sync(0xffffffffu, (i & 1) ? muc[3] : muc[2],
                                      src_lane);
                uint32_t a_hi[NR], a_lo[NR];
                float mud[NR];
#pragma unroll
                for (int h = 0; h < NR; ++h) {
                    split_f16x2((float)c1[2 * h] * (qsv[h] * vs0),
                                (float)c1[2 * h + 1] * (qsv[h] * vs1),
                                a_hi[h], a_lo[h]);
                    mud[h] = (float)(h == 0 ? mlo : mhi) * (qsc[h] * mus);
                }
                float x[2][4];
#pragma unroll
                for (int th = 0; th < 2; ++th) {
                    const uint32_t bC =
                        s8x2_to_f16x2(*reinterpret_cast<const uint16_t*>(
                            rec + RO_C8 + (8 * th + gid) * 8 + 2 * tig));
                    mma_f16_k16_z(x[th], a_hi[0], HI ? a_hi[NR - 1] : 0u, a_lo[0],
                                  HI ? a_lo[NR - 1] : 0u, bC, bC);
                }
                const uint32_t csa =
                    *reinterpret_cast<const uint32_t*>(rec + RO_CS + 4 * tig);
                const uint32_t csb =
                    *reinterpret_cast<const uint32_t*>(rec + RO_CS + 16 + 4 * tig);
                const float cs0 = bf16_bits_to_f32(csa & 0xFFFFu);
                const float cs1 = bf16_bits_to_f32(csa >> 16);
                const float cs2 = bf16_bits_to_f32(csb & 0xFFFFu);
                const float cs3 = bf16_bits_to_f32(csb >> 16);
#pragma unroll
                for (int h = 0; h < NR; ++h) {
                    const float S = LN2 * quad_lse2(
                        fmaf(cs0, x[0][2 * h], mud[h]),
                        fmaf(cs1, x[0][2 * h + 1], mud[h]),
                        fmaf(cs2, x[1][2 * h], mud[h]),
                        fmaf(cs3, x[1][2 * h + 1], mud[h]));
                    const int g = gid + 8 * h;
                    if (g < G && i < n) {
                        if (tig == (i & 3))
                            out_base[(int64_t)g * p.max_pages + p0 + i] = S;
                        run_max[h] = fmaxf(run_max[h], S);
                    }
                }
            }
        }

        __syncwarp();                         // the warp is done with `stage`
        if (k + 2 < n_items) issue(stage, item_len(k + 2), next_blk);
    }

    if (p.hmax != nullptr && tig == 0) {
#pragma unroll
        for (int h = 0; h < NR; ++h) {
            const int g = (GP == 4 ? (gid & 3) : gid) + 8 * h;
            if (g < G && run_max[h] > -INFINITY)
                atomicMax(&p.hmax[((int64_t)r * p.n_kv + kh) * G + g],
                          f2key(run_max[h]));
        }
    }
}

}  // namespace
}  // namespace locks


static int score_impl(
    const void* q, int64_t q_stride_req, const void* records_layer,
    const int32_t* block_table, int64_t bt_stride, const int32_t* n_sel_hi,
    float* score_h, uint32_t* hmax, int n_req, int n_kv, int G, int head_dim,
    int page, int max_pages, int bt_width, int num_blocks, float scale,
    int zsplit, const int32_t* row_order, int* status, locks_stream_t stream) {
    using namespace locks;
    LOCKS_REQUIRE(q && records_layer && block_table && n_sel_hi && score_h,
                  LOCKS_ERR_ARG, "locks_rki4_score_bt: null pointer argument");
    LOCKS_REQUIRE(head_dim == 128 && page == 16, LOCKS_ERR_GEOMETRY,
                  "locks_rki4_score_bt: supports head_dim 128 / page 16, got "
                  "%d / %d", head_dim, page);
    LOCKS_REQUIRE(G >= 1 && G <= 16, LOCKS_ERR_GEOMETRY,
                  "locks_rki4_score_bt: supports 1 <= G <= 16, got %d", G);
    LOCKS_REQUIRE(n_req >= 0 && n_kv >= 1 && max_pages >= 1 && bt_width >= 1 &&
                      num_blocks >= 1 && n_kv <= 65535 && n_req <= 65535,
                  LOCKS_ERR_ARG, "locks_rki4_score_bt: bad size argument");
    LOCKS_REQUIRE((reinterpret_cast<uintptr_t>(records_layer) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(q) & 7) == 0 &&
                      (q_stride_req % 4) == 0,
                  LOCKS_ERR_ARG,
                  "locks_rki4_score_bt: records must be 16-byte aligned, q 8-byte");
    if (n_req == 0) return LOCKS_OK;

    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    const int smem = (int)sizeof(ScoreSmem);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaFuncSetAttribute(rki4_score_kernel<4>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        cudaFuncSetAttribute(rki4_score_kernel<8>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        cudaFuncSetAttribute(rki4_score_kernel<16>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        attr_done[dev] = true;
    }
    // a CTA should own at least one chunk per warp
    const int max_z = (max_pages + NWARP * CHUNK - 1) / (NWARP * CHUNK);
    int Z = zsplit;
    if (Z <= 0) {
        // fill every resident CTA slot, spread over the (request, kv-head) grid
        const int base = n_req * n_kv;
        Z = (CTAS_PER_SM * sm_count() + base - 1) / base;
    }
    Z = max(1, min(Z, min(max_z, 65535)));
    // several requests (of possibly very different lengths) and room for at least
    // two CTAs each: share the CTAs of a kv-head by length
    // (a few requests: one wave in all; many requests: one CTA each plus a whole
    // wave dealt by length -- the short rows' CTAs retire at once and the long
    // rows still get their share of the resident slots)
    const int slots = (CTAS_PER_SM * sm_count()) / max(1, n_kv);
    // Many requests: four whole waves of CTAs.  A request gets 1 + floor(extra *
    // its share) CTAs, so with few CTAs to deal a mid-size row loses up to half of
    // its share to the rounding (one wave: the slowest CTA carried 1.7x the mean
    // and the launch ran at 0.67 of the copy rate on 64 rows of 4K-250K tokens;
    // four waves: 0.76); whole waves, because a last wave that fills only part of
    // the GPU is pure tail.
    // (measured on shards of that batch: 16 rows gain from four waves, 0.73 ->
    // 0.76; 8 rows lose, 0.73 -> 0.60 -- too little work per CTA)
    const int Zt = (4 * n_req <= slots && n_req < 16)
        ? slots : ((n_req + 3 * slots + slots - 1) / slots) * slots;
    const bool ragged = zsplit <= 0 && n_req > 1 && n_req <= 1024;

    ScoreParams p;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.q_stride_req = q_stride_req;
    p.records = static_cast<const uint8_t*>(records_layer);
    p.block_table = block_table;
    p.bt_stride = bt_stride;
    p.n_sel_hi = n_sel_hi;
    p.score_h = score_h;
    p.hmax = hmax;
    p.n_kv = n_kv; p.G = G; p.max_pages = max_pages; p.bt_width = bt_width;
    p.num_blocks = num_blocks; p.scale = scale; p.status = status;
    p.n_req = n_req; p.ragged = ragged ? 1 : 0;
    p.row_order = ragged ? row_order : nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = ragged ? dim3(Zt, n_kv, 1) : dim3(Z, n_kv, n_req);
    cfg.blockDim = dim3(NTHREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (pdl_enabled() && !pdl_take_break()) ? 1 : 0;
    cudaError_t e = (G <= 4)   ? cudaLaunchKernelEx(&cfg, rki4_score_kernel<4>, p)
                    : (G <= 8) ? cudaLaunchKernelEx(&cfg, rki4_score_kernel<8>, p)
                               : cudaLaunchKernelEx(&cfg, rki4_score_kernel<16>, p);
    if (e != cudaSuccess)
        return fail(LOCKS_ERR_LAUNCH, "locks_rki4_score_bt: %s",
                    cudaGetErrorString(e));
    return check_launch("locks_rki4_score_bt");
}

extern "C" int locks_rki4_score_bt(
    const void* q, int64_t q_stride_req, const void* records_layer,
    const int32_t* block_table, int64_t bt_stride, const int32_t* n_sel_hi,
    float* score_h, uint32_t* hmax, int n_req, int n_kv, int G, int head_dim,
    int page, int max_pages, int bt_width, int num_blocks, float scale,
    int zsplit, int* status, locks_stream_t stream) {
    return score_impl(q, q_stride_req, records_layer, block_table, bt_stride,
                      n_sel_hi, score_h, hmax, n_req, n_kv, G, head_dim, page,
                      max_pages, bt_width, num_blocks, scale, zsplit, nullptr, status,
                      stream);
}

extern "C" int locks_rki4_score_bt_rows(
    const void* q, int64_t q_stride_req, const void* records_layer,
    const int32_t* block_table, int64_t bt_stride, const int32_t* n_sel_hi,
    float* score_h, uint32_t* hmax, int n_req, int n_kv, int G, int head_dim,
    int page, int max_pages, int bt_width, int num_blocks, float scale,
    int zsplit, const int32_t* row_order, int* status, locks_stream_t stream) {
    return score_impl(q, q_stride_req, records_layer, block_table, bt_stride,
                      n_sel_hi, score_h, hmax, n_req, n_kv, G, head_dim, page,
                      max_pages, bt_width, num_blocks, scale, zsplit, row_order,
                      status, stream);
}
