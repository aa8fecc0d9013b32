// Page scorer: per-head page log-sum-exp from the packed rki4 summary records.
//
// Grid (zsplit, n_kv, n_req), 128 threads.  A CTA owns one (request, kv-head)
// and every zsplit-th tile of 32 consecutive logical pages.  For each tile one
// warp turns the block table into 32 record addresses and issues 32 bulk async
// copies of 832 B (the whole record is one contiguous burst) into a 3-stage
// shared-memory ring, completion tracked by one mbarrier per stage.  Each of
// the 4 warps then scores 8 pages of the tile with warp-level tensor-core
// fragments whose 16 rows are the query heads of the GQA group:
//
//   mu.q     s8 x s8  m16n8k32, the 8 pages of the warp as the 8 columns
//   V^T q    s8 x u8  m16n8k32, 4 k-steps; the int4 codes are used biased by
//            +8 (one XOR per 8 nibbles) and 8*sum(q8) is subtracted afterwards
//   C qt     bf16     m16n8k16 with qt split into three bf16 terms (hi, mid in
//            one k=16 step, lo in a second), i.e. fp32-accurate products
//   LSE      4 tokens per lane, two shuffle steps for max and for the sum
//
// The integer dot products are exact, so score_h differs from an fp32
// evaluation only by summation order and the fast exp/log intrinsics.
#include "common.cuh"

namespace locks {
namespace {

constexpr int TILE = 32;
constexpr int STAGES = 3;
constexpr int NWARP = 4;
constexpr int NTHREADS = NWARP * 32;
constexpr int PAGES_PER_WARP = TILE / NWARP;   // 8 = n of the mu mma

struct __align__(128) ScoreSmem {
    uint8_t rec[STAGES][TILE][REC_BYTES];
    int8_t q8[16][128];
    float qs[16];
    int qsum[16];
    uint64_t full[STAGES];
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
    float scale;
    int* status;
};

__device__ __forceinline__ void issue_tile(ScoreSmem& sm, const ScoreParams& p,
                                           int r, int kh, int tile, int stage,
                                           int n_hi, int lane) {
    const int p0 = tile * TILE;
    const int n = min(TILE, n_hi - p0);
    fence_proxy_async();
    if (lane == 0) mbar_expect_tx(&sm.full[stage], (uint32_t)n * REC_BYTES);
    __syncwarp();
    if (lane < n) {
        int blk = p.block_table[(int64_t)r * p.bt_stride + p0 + lane];
        blk = min(max(blk, 0), p.num_blocks - 1);
        const uint8_t* src =
            p.records + ((int64_t)blk * p.n_kv + kh) * REC_BYTES;
        bulk_g2s(&sm.rec[stage][lane][0], src, REC_BYTES, &sm.full[stage]);
    }
}

template <bool G_HI>
__global__ void __launch_bounds__(NTHREADS)
rki4_score_kernel(const ScoreParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    ScoreSmem& sm = *reinterpret_cast<ScoreSmem*>(smem_raw);

    const int z = blockIdx.x, Z = gridDim.x;
    const int kh = blockIdx.y, r = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gid = lane >> 2, tig = lane & 3;
    const int G = p.G;

    int n_hi = p.n_sel_hi[r];
    n_hi = min(n_hi, min(p.max_pages, p.bt_width));
    if (n_hi <= 0) return;
    const int ntiles = (n_hi + TILE - 1) / TILE;
    if (z >= ntiles) return;
    const int nt = (ntiles - z + Z - 1) / Z;       // tiles of this CTA

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(&sm.full[s], 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == 0) {
        for (int k = 0; k < STAGES && k < nt; ++k)
            issue_tile(sm, p, r, kh, z + k * Z, k, n_hi, lane);
    }

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
        int sum = 0;
        uint32_t packed = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = __float2int_rn(__fdiv_rn(v[i], qs));
            sum += c;
            packed |= (uint32_t)(c & 0xFF) << (8 * i);
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1)
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        *reinterpret_cast<uint32_t*>(&sm.q8[g][4 * lane]) = packed;
        if (lane == 0) { sm.qs[g] = qs; sm.qsum[g] = sum; }
    }
    __syncthreads();

    // ---- A fragments of q: rows gid (and gid+8 when G > 8) ------------------
    constexpr int NR = G_HI ? 2 : 1;
    uint32_t qn[NR][8], qe[NR][4], qo[NR][4];
    float qsc[NR];
    int qsm8[NR];
#pragma unroll
    for (int h = 0; h < NR; ++h) {
        const int g = gid + 8 * h;
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
        qsc[h] = live ? sm.qs[g] : 0.f;
        qsm8[h] = live ? 8 * sm.qsum[g] : 0;
    }

    float run_max[NR];
#pragma unroll
    for (int h = 0; h < NR; ++h) run_max[h] = -INFINITY;
    const float scale = p.scale;
    float* out_base =
        p.score_h + ((int64_t)r * p.n_kv + kh) * (int64_t)G * p.max_pages;

    for (int k = 0; k < nt; ++k) {
        const int stage = k % STAGES;
        const int tile = z + k * Z;
        const int p0 = tile * TILE;
        const int n = min(TILE, n_hi - p0);
        mbar_wait(&sm.full[stage], (uint32_t)((k / STAGES) & 1), p.status);

        const uint8_t* wrec = &sm.rec[stage][warp * PAGES_PER_WARP][0];

        // mu . q for the warp's 8 pages: column (n) = page gid of the warp
        int muc[4] = {0, 0, 0, 0};
        {
            const uint8_t* mrec = wrec + gid * REC_BYTES + RO_MU8 + 32 * tig;
            const uint4 m0 = *reinterpret_cast<const uint4*>(mrec);
            const uint4 m1 = *reinterpret_cast<const uint4*>(mrec + 16);
            const uint32_t mw[8] = {m0.x, m0.y, m0.z, m0.w,
                                    m1.x, m1.y, m1.z, m1.w};
#pragma unroll
            for (int s = 0; s < 4; ++s)
                mma_s8s8_k32(muc, qn[0][2 * s], G_HI ? qn[NR - 1][2 * s] : 0u,
                             qn[0][2 * s + 1],
                             G_HI ? qn[NR - 1][2 * s + 1] : 0u, mw[2 * s],
                             mw[2 * s + 1]);
        }

#pragma unroll 2
        for (int i = 0; i < PAGES_PER_WARP; ++i) {
            const int li = warp * PAGES_PER_WARP + i;
            const uint8_t* rec = wrec + i * REC_BYTES;

            // ---- qt_int[g][r] = sum_d q8[g][d] * (code[d][r] + 8) -----------
            int c1[4] = {0, 0, 0, 0};
            const uint4 vw =
                *reinterpret_cast<const uint4*>(rec + RO_V4 + gid * 64 + tig * 16);
            const uint32_t vword[4] = {vw.x, vw.y, vw.z, vw.w};
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const uint32_t u = vword[s] ^ 0x88888888u;
                const uint32_t b0 = u & 0x0F0F0F0Fu;
                const uint32_t b1 = (u >> 4) & 0x0F0F0F0Fu;
                mma_s8u8_k32(c1, qe[0][s], G_HI ? qe[NR - 1][s] : 0u, qo[0][s],
                             G_HI ? qo[NR - 1][s] : 0u, b0, b1);
            }
            const uint32_t vs2 =
                *reinterpret_cast<const uint32_t*>(rec + RO_VS + 4 * tig);
            const float vs0 = bf16_bits_to_f32(vs2 & 0xFFFFu);
            const float vs1 = bf16_bits_to_f32(vs2 >> 16);
            const float mus = bf16_bits_to_f32(
                *reinterpret_cast<const uint16_t*>(rec + RO_MUS));

            // mu.q of page i sits in lane (gid, i/2), register i%2 (+2 for hi)
            const int src_lane = (lane & ~3) | (i >> 1);
            const int mlo = __shfl_sync(0xffffffffu, (i & 1) ? muc[1] : muc[0],
                                        src_lane);
            int mhi = 0;
            if (G_HI)
                mhi = __shfl_sync(0xffffffffu, (i & 1) ? muc[3] : muc[2],
                                  src_lane);

            // ---- A operand of the C product: qt as hi/mid/lo bf16 -----------
            uint32_t a_hi[NR], a_mid[NR], a_lo[NR];
            float mud[NR];
#pragma unroll
            for (int h = 0; h < NR; ++h) {
                const float f0 =
                    (float)(c1[2 * h] - qsm8[h]) * (qsc[h] * vs0);
                const float f1 =
                    (float)(c1[2 * h + 1] - qsm8[h]) * (qsc[h] * vs1);
                const float h0 = __bfloat162float(__float2bfloat16_rn(f0));
                const float h1 = __bfloat162float(__float2bfloat16_rn(f1));
                const float r0 = f0 - h0, r1 = f1 - h1;
                const float m0 = __bfloat162float(__float2bfloat16_rn(r0));
                const float m1 = __bfloat162float(__float2bfloat16_rn(r1));
                a_hi[h] = pack_bf16x2(h0, h1);
                a_mid[h] = pack_bf16x2(m0, m1);
                a_lo[h] = pack_bf16x2(r0 - m0, r1 - m1);
                mud[h] = (float)(h == 0 ? mlo : mhi) * (qsc[h] * mus);
            }

            // ---- X[g][t] = sum_r C8[t][r] * qt[g][r], two halves of 8 tokens
            float x[2][4];
#pragma unroll
            for (int th = 0; th < 2; ++th) {
                const uint16_t cc = *reinterpret_cast<const uint16_t*>(
                    rec + RO_C8 + (8 * th + gid) * 8 + 2 * tig);
                const uint32_t bC = pack_bf16x2(
                    (float)(int8_t)(cc & 0xFF), (float)(int8_t)(cc >> 8));
                x[th][0] = x[th][1] = x[th][2] = x[th][3] = 0.f;
                mma_bf16_k16(x[th], a_hi[0], G_HI ? a_hi[NR - 1] : 0u, a_mid[0],
                             G_HI ? a_mid[NR - 1] : 0u, bC, bC);
                mma_bf16_k16(x[th], a_lo[0], G_HI ? a_lo[NR - 1] : 0u, 0u, 0u,
                             bC, 0u);
            }

            // ---- tok = scale * (cs[t] * X + mu.q); LSE over the 16 tokens ---
            const uint32_t csa =
                *reinterpret_cast<const uint32_t*>(rec + RO_CS + 4 * tig);
            const uint32_t csb =
                *reinterpret_cast<const uint32_t*>(rec + RO_CS + 16 + 4 * tig);
            const float cs[4] = {bf16_bits_to_f32(csa & 0xFFFFu),
                                 bf16_bits_to_f32(csa >> 16),
                                 bf16_bits_to_f32(csb & 0xFFFFu),
                                 bf16_bits_to_f32(csb >> 16)};
#pragma unroll
            for (int h = 0; h < NR; ++h) {
                float t[4];
                t[0] = scale * fmaf(cs[0], x[0][2 * h], mud[h]);
                t[1] = scale * fmaf(cs[1], x[0][2 * h + 1], mud[h]);
                t[2] = scale * fmaf(cs[2], x[1][2 * h], mud[h]);
                t[3] = scale * fmaf(cs[3], x[1][2 * h + 1], mud[h]);
                float mx = fmaxf(fmaxf(t[0], t[1]), fmaxf(t[2], t[3]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                float sum = __expf(t[0] - mx) + __expf(t[1] - mx) +
                            __expf(t[2] - mx) + __expf(t[3] - mx);
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                const float S = mx + __logf(sum);
                const int g = gid + 8 * h;
                if (li < n && g < G) {
                    if (tig == (i & 3))
                        out_base[(int64_t)g * p.max_pages + p0 + li] = S;
                    run_max[h] = fmaxf(run_max[h], S);
                }
            }
        }

        __syncthreads();                      // every warp is done with `stage`
        if (warp == 0 && k + STAGES < nt)
            issue_tile(sm, p, r, kh, z + (k + STAGES) * Z, stage, n_hi, lane);
    }

    if (p.hmax != nullptr && tig == 0) {
#pragma unroll
        for (int h = 0; h < NR; ++h) {
            const int g = gid + 8 * h;
            if (g < G && run_max[h] > -INFINITY)
                atomicMax(&p.hmax[((int64_t)r * p.n_kv + kh) * G + g],
                          f2key(run_max[h]));
        }
    }
}

}  // namespace
}  // namespace locks

extern "C" int locks_rki4_score_bt(
    const void* q, int64_t q_stride_req, const void* records_layer,
    const int32_t* block_table, int64_t bt_stride, const int32_t* n_sel_hi,
    float* score_h, uint32_t* hmax, int n_req, int n_kv, int G, int head_dim,
    int page, int max_pages, int bt_width, int num_blocks, float scale,
    int zsplit, int* status, locks_stream_t stream) {
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
        cudaFuncSetAttribute(rki4_score_kernel<false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        cudaFuncSetAttribute(rki4_score_kernel<true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        attr_done[dev] = true;
    }
    const int max_tiles = (max_pages + TILE - 1) / TILE;
    int Z = zsplit;
    if (Z <= 0) {
        // two resident CTAs per SM, spread over the (request, kv-head) grid
        const int base = n_req * n_kv;
        Z = (2 * sm_count() + base - 1) / base;
    }
    Z = max(1, min(Z, min(max_tiles, 65535)));

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
    dim3 grid(Z, n_kv, n_req);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (G > 8)
        rki4_score_kernel<true><<<grid, NTHREADS, smem, s>>>(p);
    else
        rki4_score_kernel<false><<<grid, NTHREADS, smem, s>>>(p);
    return check_launch("locks_rki4_score_bt");
}
