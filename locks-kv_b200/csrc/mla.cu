// MLA (latent KV) path: page factor build, factored page scorer, keep-rule
// parameters and the decode over the kept pages of the latent cache.
//
// The 16 query heads share one latent head of width 512 (+64 rope channels), so
// every contraction has exactly 16 rows: the scorer and the decode run on
// warp-level tensor-core fragments (m16n8k16) with all 16 rows live.
#include <cooperative_groups.h>

#include "common.cuh"
#include "jacobi16.cuh"

namespace cg = cooperative_groups;

namespace locks {
namespace {

constexpr int LKV = LOCKS_MLA_LKV;        // 512
constexpr int ROPE = LOCKS_MLA_ROPE;      // 64
constexpr int WIDTH = LKV + ROPE;         // 576
constexpr int NH = LOCKS_MLA_HEADS;       // 16
constexpr int PG = 16;                    // tokens per page
constexpr int MREC = LOCKS_MLA_REC_BYTES; // 8448
constexpr int MRO_LF = 8192;              // Lf offset inside a record

__device__ __forceinline__ void mma_f16f16_k16(float (&d)[4], uint32_t a0,
                                               uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// =========================================================================== //
// Factor build: one warp per physical block                                    //
// =========================================================================== //
constexpr int FB_WARPS = 4;
constexpr int FB_PITCH = LKV + 8;         // bf16 elements per staged row

struct FbScratch {
    __nv_bfloat16 pg[PG][FB_PITCH];
    float A[PG][PG + 1];
    float U[PG][PG + 1];
    float rc[8], rs[8];
    float sig[8], inv[8];
    int idx[8];
};

struct FbParams {
    const __nv_bfloat16* cache;
    int64_t sb, st;
    uint8_t* records;
    const int32_t* blocks;         // block list, or null: jobs come from the rows
    int n_blocks, num_blocks;
    // row mode: job bi is page bi % max_pages of row bi / max_pages; it runs when
    // the row was flagged (need) and the page is one of its n_cache full pages
    const int32_t* need;
    const int32_t* n_cache;
    const int32_t* block_table;
    int64_t bt_stride;
    int max_pages;
};

__global__ void __launch_bounds__(FB_WARPS * 32) mla_factor_kernel(const FbParams p) {
    extern __shared__ __align__(16) uint8_t fb_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bi = blockIdx.x * FB_WARPS + warp;
    if (bi >= p.n_blocks) return;
    int blk;
    if (p.blocks != nullptr) {
        blk = p.blocks[bi];
    } else {
        const int row = bi / p.max_pages, page = bi - row * p.max_pages;
        if (!p.need[row] || page >= p.n_cache[row]) return;
        blk = p.block_table[(int64_t)row * p.bt_stride + page];
    }
    if (blk < 0 || blk >= p.num_blocks) return;
    FbScratch& ws = reinterpret_cast<FbScratch*>(fb_raw)[warp];
    const __nv_bfloat16* src = p.cache + (int64_t)blk * p.sb;

    // stage the 16 x 512 latent page (bf16) in shared memory
#pragma unroll 4
    for (int t = 0; t < PG; ++t) {
        const uint4* g = reinterpret_cast<const uint4*>(src + (int64_t)t * p.st);
        uint4* s = reinterpret_cast<uint4*>(&ws.pg[t][0]);
        s[lane] = g[lane];
        s[lane + 32] = g[lane + 32];
    }
    __syncwarp();

    // Gram (not centred): lane -> row i = lane/2, columns j0..j0+7
    {
        const int i = lane >> 1, j0 = (lane & 1) * 8;
        float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int d = 0; d < LKV; d += 2) {
            const float2 a = __bfloat1622float2(
                *reinterpret_cast<const __nv_bfloat162*>(&ws.pg[i][d]));
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float2 b = __bfloat1622float2(
                    *reinterpret_cast<const __nv_bfloat162*>(&ws.pg[j0 + j][d]));
                g[j] = fmaf(a.x, b.x, g[j]);
                g[j] = fmaf(a.y, b.y, g[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            ws.A[i][j0 + j] = g[j];
            ws.U[i][j0 + j] = (i == j0 + j) ? 1.f : 0.f;
        }
    }
    __syncwarp();
    jacobi16_warp(ws.A, ws.U, ws.rc, ws.rs, lane);

    // top-8 modes, DESCENDING; modes at or below sigma_1 * sqrt(eps) are dropped
    if (lane < PG) {
        const float lam = ws.A[lane][lane];
        int pos = 0;
        for (int j = 0; j < PG; ++j) {
            const float lj = ws.A[j][j];
            pos += (lj > lam) || (lj == lam && j < lane);
        }
        if (pos < 8) {
            ws.idx[pos] = lane;
            ws.sig[pos] = __fsqrt_rn(fmaxf(lam, 0.f));
        }
    }
    __syncwarp();
    if (lane < 8) {
        const float tol = ws.sig[0] * 3.4526698300124393e-4f;   // sqrt(fp32 eps)
        const float s = ws.sig[lane];
        const bool keep = s > tol;
        __syncwarp(0xffu);
        ws.sig[lane] = keep ? s : 0.f;
        ws.inv[lane] = keep ? __fdiv_rn(1.f, fmaxf(s, 1.1754944e-38f)) : 0.f;
    }
    __syncwarp();

    uint8_t* rec = p.records + (int64_t)blk * MREC;
    // Lf[t][r] = W[t][r] * sigma_r : lane -> token lane/2, modes r0..r0+3
    {
        const int t = lane >> 1, r0 = (lane & 1) * 4;
        __half2 h[2];
        h[0] = __floats2half2_rn(ws.U[t][ws.idx[r0]] * ws.sig[r0],
                                 ws.U[t][ws.idx[r0 + 1]] * ws.sig[r0 + 1]);
        h[1] = __floats2half2_rn(ws.U[t][ws.idx[r0 + 2]] * ws.sig[r0 + 2],
                                 ws.U[t][ws.idx[r0 + 3]] * ws.sig[r0 + 3]);
        *reinterpret_cast<uint2*>(rec + MRO_LF + (t * 8 + r0) * 2) =
            *reinterpret_cast<const uint2*>(h);
    }
    // Rf[r][D] = (sum_t W[t][r] * page[t][D]) / sigma_r : lane -> D = 16 lane ..
    for (int r = 0; r < 8; ++r) {
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.f;
        const int col = ws.idx[r];
        for (int t = 0; t < PG; ++t) {
            const float w = ws.U[t][col];
            const __nv_bfloat162* row =
                reinterpret_cast<const __nv_bfloat162*>(&ws.pg[t][16 * lane]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 x = __bfloat1622float2(row[i]);
                acc[2 * i] = fmaf(w, x.x, acc[2 * i]);
                acc[2 * i + 1] = fmaf(w, x.y, acc[2 * i + 1]);
            }
        }
        const float inv = ws.inv[r];
        __half2 o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            o[i] = __floats2half2_rn(acc[2 * i] * inv, acc[2 * i + 1] * inv);
        uint4* dst = reinterpret_cast<uint4*>(rec + (r * LKV + 16 * lane) * 2);
        dst[0] = reinterpret_cast<const uint4*>(o)[0];
        dst[1] = reinterpret_cast<const uint4*>(o)[1];
    }
}

// =========================================================================== //
// Which rows need (new) factors: decided on the device                           //
// =========================================================================== //
// One warp per row.  A row's factors are remembered under its FIRST block id:
// fp_tab[b0] is a content fingerprint, nc_tab[b0] the number of full pages the
// factors cover (-1: none).  The fingerprint is  f(block b0) + 1.0009 f(block of
// page nc - 1)  with f = the sum of the first 8 channels over the block's 16
// tokens: both blocks are full prompt pages, so the value does not change while
// the request decodes, and a request that reuses a finished one's block ids
// changes it.  A row is flagged when it has no entry, when it shrank below the
// stored page count (preemption), or when the fingerprint differs; a flagged
// row's entry is rewritten for its current length.  Generated pages are not
// added to an existing entry (they are attended while inside the recent window),
// as in the reference (backend/mla_attn.py:212-239), whose host-side
// bookkeeping and per-step .tolist() this kernel replaces.
struct GateParams {
    const __nv_bfloat16* cache;
    int64_t sb, st;
    const int32_t* block_table;
    int64_t bt_stride;
    const int32_t* seq_lens;
    float* fp_tab;
    int32_t* nc_tab;
    int32_t* need;
    int32_t* n_cache;
    int n_rows, num_blocks, max_pages;
};

__device__ __forceinline__ float block_fingerprint(const GateParams& p, int blk, int lane) {
    // 16 tokens x 8 channels = 128 values, 4 per lane, fixed summation order
    const int t = lane >> 1, c0 = (lane & 1) * 4;
    const __nv_bfloat16* src = p.cache + (int64_t)blk * p.sb + (int64_t)t * p.st + c0;
    float v = __bfloat162float(src[0]) + __bfloat162float(src[1]) +
              __bfloat162float(src[2]) + __bfloat162float(src[3]);
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__global__ void __launch_bounds__(128) mla_gate_kernel(const GateParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + warp;
    if (r >= p.n_rows) return;
    const int sl = p.seq_lens[r];
    if (sl <= 0) {
        if (lane == 0) { p.need[r] = 0; p.n_cache[r] = 0; }
        return;
    }
    const int32_t* bt = p.block_table + (int64_t)r * p.bt_stride;
    const int b0 = min(max(bt[0], 0), p.num_blocks - 1);
    const int nc_now = min(sl / PG, p.max_pages);
    const int nc_old = p.nc_tab[b0];
    const float f0 = block_fingerprint(p, b0, lane);
    bool need = nc_old < 0 || nc_now < nc_old;
    if (!need) {
        const int last = (nc_old > 0) ? min(max(bt[nc_old - 1], 0), p.num_blocks - 1) : b0;
        const float fp = f0 + 1.0009f * block_fingerprint(p, last, lane);
        need = !(fp == p.fp_tab[b0]);
    }
    if (need) {
        const int last = (nc_now > 0) ? min(max(bt[nc_now - 1], 0), p.num_blocks - 1) : b0;
        const float fp = f0 + 1.0009f * block_fingerprint(p, last, lane);
        if (lane == 0) { p.fp_tab[b0] = fp; p.nc_tab[b0] = nc_now; }
    }
    if (lane == 0) { p.need[r] = need ? 1 : 0; p.n_cache[r] = need ? nc_now : nc_old; }
}

// =========================================================================== //
// Keep-rule parameters                                                          //
// =========================================================================== //
__global__ void mla_derive_kernel(const int32_t* __restrict__ seq_lens, int n,
                                  int budget, int sink, int window,
                                  int32_t* __restrict__ n_pages,
                                  int32_t* __restrict__ n_sel_hi,
                                  int32_t* __restrict__ b_fix) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int L = max(seq_lens[i], 0);
    const int P = (L + PG - 1) / PG;
    int b;
    if (P <= budget) {
        b = P;                                   // keep every page
    } else {
        const int a = min(sink, P);
        const int s2 = max(0, P - window);
        const int forced = a + (P - max(s2, a));
        b = max(budget - forced, 0);
    }
    n_pages[i] = P;
    n_sel_hi[i] = P - window;
    b_fix[i] = b;
}

// =========================================================================== //
// Factored page scorer                                                          //
// =========================================================================== //
constexpr int SC_WARPS = 4;
constexpr int SC_STAGES = 2;
constexpr int RF_PITCH = LKV * 2 + 16;      // 1040 B per staged Rf row
constexpr int KR_PITCH = ROPE * 2 + 16;     // 144 B per staged rope row
constexpr int QC_PITCH = LKV * 2 + 16;      // 1040 B per q_c row (fp16)
constexpr int QR_PITCH = ROPE * 2 + 16;     // 144 B per q_rope row (bf16)

struct ScStage {
    uint8_t rf[8][RF_PITCH];
    uint8_t lf[256];
    uint8_t kr[PG][KR_PITCH];
};

struct __align__(128) ScSmem {
    ScStage st[SC_WARPS][SC_STAGES];
    uint8_t qc[NH][QC_PITCH];
    uint8_t qr[NH][QR_PITCH];
    uint64_t full[SC_WARPS][SC_STAGES];
};

struct MlaScoreParams {
    const __nv_bfloat16* q;
    int64_t q_stride_row;
    const uint8_t* records;
    const __nv_bfloat16* cache;
    int64_t sb, st;
    const int32_t* block_table;
    int64_t bt_stride;
    const int32_t* n_cache;
    const int32_t* n_pages;
    float* score;
    int max_pages, num_blocks;
    float scale;
    int* status;
};

__global__ void __launch_bounds__(SC_WARPS * 32, 2)
mla_score_kernel(const MlaScoreParams p) {
    extern __shared__ __align__(128) uint8_t sc_raw[];
    ScSmem& sm = *reinterpret_cast<ScSmem*>(sc_raw);
    const int z = blockIdx.x, Z = gridDim.x, row = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gid = lane >> 2, tig = lane & 3;

    const int n_pg = min(max(p.n_pages[row], 0), p.max_pages);
    const int n_c = min(max(p.n_cache[row], 0), n_pg);
    float* score = p.score + (int64_t)row * p.max_pages;
    pdl_trigger();                    // the selector may be scheduled; it waits for us
    if (n_c <= 0) {
        pdl_wait();                   // the score row belongs to the kernels before
        if (z == 0)                   // pages without factors score -inf
            for (int i = tid; i < n_pg; i += SC_WARPS * 32) score[i] = -INFINITY;
        return;
    }
    const int cg0 = (int)(((int64_t)n_c * z) / Z);
    const int cg1 = (int)(((int64_t)n_c * (z + 1)) / Z);
    if (cg1 <= cg0) return;
    const int pg0 = cg0 + (int)(((int64_t)(cg1 - cg0) * warp) / SC_WARPS);
    const int pg1 = cg0 + (int)(((int64_t)(cg1 - cg0) * (warp + 1)) / SC_WARPS);
    const int np = pg1 - pg0;

    if (tid == 0) {
        for (int w = 0; w < SC_WARPS; ++w)
            for (int s = 0; s < SC_STAGES; ++s) mbar_init(&sm.full[w][s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    const int32_t* bt = p.block_table + (int64_t)row * p.bt_stride;
    auto issue = [&](int k) {            // page pg0 + k -> stage k % SC_STAGES
        ScStage& S = sm.st[warp][k % SC_STAGES];
        uint64_t* bar = &sm.full[warp][k % SC_STAGES];
        int blk = bt[pg0 + k];
        blk = min(max(blk, 0), p.num_blocks - 1);
        fence_proxy_async();
        if (lane == 0) mbar_expect_tx(bar, 8192u + 256u + PG * ROPE * 2u);
        __syncwarp();
        const uint8_t* rec = p.records + (int64_t)blk * MREC;
        if (lane < 8) {
            bulk_g2s(&S.rf[lane][0], rec + lane * (LKV * 2), LKV * 2, bar);
        } else if (lane == 8) {
            bulk_g2s(&S.lf[0], rec + MRO_LF, 256, bar);
        } else if (lane >= 16) {
            const int t = lane - 16;
            bulk_g2s(&S.kr[t][0],
                     p.cache + (int64_t)blk * p.sb + (int64_t)t * p.st + LKV,
                     ROPE * 2, bar);
        }
    };
    for (int k = 0; k < SC_STAGES && k < np; ++k) issue(k);

    // Everything above reads per-step constants (page counts, block table, factor
    // records, rope keys); q and the score row belong to the kernels before.
    pdl_wait();
    if (z == 0)                       // pages without factors score -inf
        for (int i = n_c + tid; i < n_pg; i += SC_WARPS * 32) score[i] = -INFINITY;

    // ---- stage q: q_c as fp16, q_rope as bf16; 16-byte loads, all in flight ----
    {
        const uint4* q4 = reinterpret_cast<const uint4*>(p.q + (int64_t)row * p.q_stride_row);
        constexpr int C16 = WIDTH * 2 / 16;               // 72 chunks of 8 bf16 per head
        constexpr int NQ = (NH * C16 + SC_WARPS * 32 - 1) / (SC_WARPS * 32);
        uint4 v[NQ];
#pragma unroll
        for (int i = 0; i < NQ; ++i) {
            const int e = tid + i * SC_WARPS * 32;
            v[i] = (e < NH * C16) ? q4[e] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < NQ; ++i) {
            const int e = tid + i * SC_WARPS * 32;
            if (e >= NH * C16) continue;
            const int h = e / C16, c = e % C16;
            if (c < LKV * 2 / 16) {                        // latent part -> fp16
                const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __half2 hh = __floats2half2_rn(
                        __uint_as_float(w[j] << 16), __uint_as_float(w[j] & 0xFFFF0000u));
                    o[j] = *reinterpret_cast<const uint32_t*>(&hh);
                }
                *reinterpret_cast<uint4*>(&sm.qc[h][16 * c]) =
                    make_uint4(o[0], o[1], o[2], o[3]);
            } else {                                       // rope part stays bf16
                *reinterpret_cast<uint4*>(&sm.qr[h][16 * (c - LKV * 2 / 16)]) = v[i];
            }
        }
    }
    __syncthreads();

    // ldmatrix lane addresses of the A operands (16 rows x 16 columns per step)
    const int a_row = (lane & 7) + 8 * ((lane >> 3) & 1);
    const uint32_t qc_addr = smem_u32(&sm.qc[a_row][0]) + 16 * (lane >> 4);
    const uint32_t qr_addr = smem_u32(&sm.qr[a_row][0]) + 16 * (lane >> 4);

    for (int k = 0; k < np; ++k) {
        const int stage = k % SC_STAGES;
        mbar_wait(&sm.full[warp][stage], (uint32_t)((k / SC_STAGES) & 1), p.status);
        const ScStage& S = sm.st[warp][stage];

        // a[h][r] = sum_D q_c[h][D] * Rf[r][D]        (32 k-steps)
        float a[4] = {0.f, 0.f, 0.f, 0.f};
        const uint8_t* rfrow = &S.rf[gid][0] + 4 * tig;
#pragma unroll 8
        for (int s = 0; s < LKV / 16; ++s) {
            uint32_t qa[4];
            ldmatrix_x4(qa, qc_addr + 32 * s);
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(rfrow + 32 * s);
            const uint32_t b1 = *reinterpret_cast<const uint32_t*>(rfrow + 32 * s + 16);
            mma_f16f16_k16(a, qa[0], qa[1], qa[2], qa[3], b0, b1);
        }
        // hi / lo fp16 split of a -> A operand with k = [hi(8) | lo(8)]
        uint32_t ah0, al0, ah1, al1;
        {
            const __half2 h0 = __floats2half2_rn(a[0], a[1]);
            const __half2 h1 = __floats2half2_rn(a[2], a[3]);
            const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
            const __half2 l0 = __floats2half2_rn(a[0] - f0.x, a[1] - f0.y);
            const __half2 l1 = __floats2half2_rn(a[2] - f1.x, a[3] - f1.y);
            ah0 = *reinterpret_cast<const uint32_t*>(&h0);
            ah1 = *reinterpret_cast<const uint32_t*>(&h1);
            al0 = *reinterpret_cast<const uint32_t*>(&l0);
            al1 = *reinterpret_cast<const uint32_t*>(&l1);
        }
        float sc[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
            // nope part: sum_r a[h][r] * Lf[t][r]
            const uint32_t bl = *reinterpret_cast<const uint32_t*>(
                &S.lf[((8 * nt + gid) * 8 + 2 * tig) * 2]);
            mma_f16f16_k16(sc[nt], ah0, ah1, al0, al1, bl, bl);
        }
        // rope part: sum_d q_rope[h][d] * k_rope[t][d]     (4 k-steps)
#pragma unroll
        for (int s = 0; s < ROPE / 16; ++s) {
            uint32_t qa[4];
            ldmatrix_x4(qa, qr_addr + 32 * s);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const uint8_t* kr = &S.kr[8 * nt + gid][0] + 32 * s + 4 * tig;
                mma_bf16_k16(sc[nt], qa[0], qa[1], qa[2], qa[3],
                             *reinterpret_cast<const uint32_t*>(kr),
                             *reinterpret_cast<const uint32_t*>(kr + 16));
            }
        }
        float mx = fmaxf(fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[0][2], sc[0][3])),
                         fmaxf(fmaxf(sc[1][0], sc[1][1]), fmaxf(sc[1][2], sc[1][3])));
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1)
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) score[pg0 + k] = mx * p.scale;

        __syncwarp();
        if (k + SC_STAGES < np) issue(k + SC_STAGES);
    }
}

// =========================================================================== //
// Decode over the kept pages (one cluster per row)                              //
// =========================================================================== //
constexpr int MD_WARPS = 4;
constexpr int MD_THREADS = MD_WARPS * 32;
constexpr int MD_STAGES = 2;
constexpr int KV_PITCH = WIDTH * 2 + 16;      // 1168 B per staged row
constexpr int OUT_PITCH = LKV + 4;            // floats
constexpr int MD_MAX_CL = 16;                // > 8 needs the non-portable cluster attribute

struct __align__(128) MdSmem {
    uint8_t kv[MD_STAGES][PG][KV_PITCH];
    uint8_t q[NH][KV_PITCH];
    // cluster exchange: CTA c pushes its (m, l) to every CTA and the slice of
    // its O that CTA d normalises into xacc[c * per_e ...] of CTA d
    float xacc[NH * LKV + 64];
    float xm[MD_MAX_CL][NH], xl[MD_MAX_CL][NH];
    float sred[MD_WARPS][NH][PG + 1];   // per-warp partial logits of a page
    uint64_t full[MD_STAGES];
};

struct MlaDecParams {
    const __nv_bfloat16* q;
    int64_t q_stride_row;
    const __nv_bfloat16* cache;
    int64_t sb, st;
    const int32_t* block_table;
    int64_t bt_stride;
    const int32_t* page_table;
    const int32_t* page_cnt;
    const int32_t* seq_lens;
    __nv_bfloat16* out;
    float* lse;
    int max_pages;
    float scale;
    int* status;
};


__global__ void __launch_bounds__(MD_THREADS) mla_decode_kernel(const MlaDecParams p) {
    extern __shared__ __align__(128) uint8_t md_raw[];
    MdSmem& sm = *reinterpret_cast<MdSmem*>(md_raw);
    cg::cluster_group cluster = cg::this_cluster();
    const int c = blockIdx.x, CL = gridDim.x, row = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gid = lane >> 2, tig = lane & 3;

    if (tid == 0) {
        for (int s = 0; s < MD_STAGES; ++s) mbar_init(&sm.full[s], 1);
        mbar_fence_init();
    }
    pdl_trigger();                     // the next layer's scorer may start prefetching
    // remote shared memory may be written once every CTA of the cluster runs
    cluster.sync();
    pdl_wait();                        // the page table comes from the selector
    const int seq_len = p.seq_lens[row];
    const int cnt = min(max(p.page_cnt[row], 0), p.max_pages);
    const int per = (cnt + CL - 1) / CL;
    const int j0 = min(c * per, cnt), j1 = min(j0 + per, cnt);
    const int np = j1 - j0;

    const int32_t* tab = p.page_table + (int64_t)row * p.max_pages;
    const int32_t* bt = p.block_table + (int64_t)row * p.bt_stride;
    int nv[MD_STAGES] = {};
    // Page-table entry and physical block of this CTA's pages, 32 at a time (lane i
    // of every warp holds entry i of the window): the two dependent index loads
    // are paid once per window, not once per page.
    int win_pt = -1, win_blk = 0;
    auto load_window = [&](int k0) {
        const int k = k0 + lane;
        win_pt = -1; win_blk = 0;
        if (k < np) {
            win_pt = tab[j0 + k];
            win_blk = bt[max(win_pt, 0)];
        }
    };
    // every thread computes n_valid; the 16 row copies are issued by 4 lanes of
    // each warp (a bulk-copy request costs its issuer ~80 cycles)
    auto issue = [&](int k) {
        const int stage = k % MD_STAGES;
        const int pt = __shfl_sync(0xffffffffu, win_pt, k & 31);
        const int blk = max(__shfl_sync(0xffffffffu, win_blk, k & 31), 0);
        const int n_valid = (pt >= 0) ? min(max(seq_len - pt * PG, 0), PG) : 0;
        nv[stage] = n_valid;
        uint64_t* bar = &sm.full[stage];
        fence_proxy_async();
        if (tid == 0) mbar_expect_tx(bar, (uint32_t)n_valid * (WIDTH * 2));
        constexpr int RPW = PG / MD_WARPS;            // rows per warp
        if (lane < RPW) {
            const int t = warp * RPW + lane;
            uint8_t* dst = &sm.kv[stage][t][0];
            if (t < n_valid) {
                bulk_g2s(dst, p.cache + (int64_t)blk * p.sb + (int64_t)t * p.st,
                         WIDTH * 2, bar);
            } else {
                uint4* d4 = reinterpret_cast<uint4*>(dst);
                for (int i = 0; i < (WIDTH * 2) / 16; ++i) d4[i] = make_uint4(0, 0, 0, 0);
            }
        }
    };
    load_window(0);
    for (int k = 0; k < MD_STAGES && k < np; ++k) issue(k);

    // stage q (bf16, padded rows): 16-byte loads, all in flight before the stores
    {
        const uint4* q4 = reinterpret_cast<const uint4*>(p.q + (int64_t)row * p.q_stride_row);
        constexpr int C16 = WIDTH * 2 / 16;           // 72 chunks per head
        constexpr int NQ = (NH * C16 + MD_THREADS - 1) / MD_THREADS;
        uint4 v[NQ];
#pragma unroll
        for (int i = 0; i < NQ; ++i) {
            const int e = tid + i * MD_THREADS;
            v[i] = (e < NH * C16) ? q4[e] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < NQ; ++i) {
            const int e = tid + i * MD_THREADS;
            if (e < NH * C16)
                *reinterpret_cast<uint4*>(&sm.q[e / C16][16 * (e % C16)]) = v[i];
        }
    }
    __syncthreads();

    const int a_row = (lane & 7) + 8 * ((lane >> 3) & 1);
    const uint32_t q_addr = smem_u32(&sm.q[a_row][0]) + 16 * (lane >> 4);
    // K operand (non-transposed): token = (lane&7) + 8*((lane>>4)&1), col half (lane>>3)&1
    const int kt = (lane & 7) + 8 * ((lane >> 4) & 1);
    const int kcol = 16 * ((lane >> 3) & 1);
    // V operand (transposed): token = (lane&7) + 8*((lane>>3)&1), col half (lane>>4)&1
    const int vt = (lane & 7) + 8 * ((lane >> 3) & 1);
    const int vcol = 16 * ((lane >> 4) & 1) + warp * (128 * 2);

    float acc[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

    for (int k = 0; k < np; ++k) {
        const int stage = k % MD_STAGES;
        mbar_wait(&sm.full[stage], (uint32_t)((k / MD_STAGES) & 1), p.status);
        __syncthreads();                       // zero-filled rows are visible too
        const int n_valid = nv[stage];
        if (n_valid > 0) {
            const uint32_t kbase = smem_u32(&sm.kv[stage][0][0]);
            // Q K^T: the 36 k-steps are split over the 4 warps (9 each); the
            // partial 16 x 16 logit tiles meet in shared memory
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t ka = kbase + kt * KV_PITCH + kcol;
            constexpr int KS = (WIDTH / 16) / MD_WARPS;
#pragma unroll
            for (int si = 0; si < KS; ++si) {
                const int s = warp * KS + si;
                uint32_t qa[4], kb[4];
                ldmatrix_x4(qa, q_addr + 32 * s);
                ldmatrix_x4(kb, ka + 32 * s);
                mma_bf16_k16(s0, qa[0], qa[1], qa[2], qa[3], kb[0], kb[1]);
                mma_bf16_k16(s1, qa[0], qa[1], qa[2], qa[3], kb[2], kb[3]);
            }
            {
                float (*sr)[PG + 1] = sm.sred[warp];
                sr[gid][2 * tig] = s0[0];         sr[gid][2 * tig + 1] = s0[1];
                sr[gid + 8][2 * tig] = s0[2];     sr[gid + 8][2 * tig + 1] = s0[3];
                sr[gid][2 * tig + 8] = s1[0];     sr[gid][2 * tig + 9] = s1[1];
                sr[gid + 8][2 * tig + 8] = s1[2]; sr[gid + 8][2 * tig + 9] = s1[3];
            }
            __syncthreads();
#pragma unroll
            for (int i = 0; i < 4; ++i) s0[i] = s1[i] = 0.f;
#pragma unroll
            for (int w = 0; w < MD_WARPS; ++w) {
                const float (*sr)[PG + 1] = sm.sred[w];
                s0[0] += sr[gid][2 * tig];         s0[1] += sr[gid][2 * tig + 1];
                s0[2] += sr[gid + 8][2 * tig];     s0[3] += sr[gid + 8][2 * tig + 1];
                s1[0] += sr[gid][2 * tig + 8];     s1[1] += sr[gid][2 * tig + 9];
                s1[2] += sr[gid + 8][2 * tig + 8]; s1[3] += sr[gid + 8][2 * tig + 9];
            }
            const int ta = 2 * tig, tb = 2 * tig + 1;
            const float scale = p.scale;
            float x[8];
            x[0] = (ta < n_valid) ? s0[0] * scale : -INFINITY;
            x[1] = (tb < n_valid) ? s0[1] * scale : -INFINITY;
            x[2] = (ta + 8 < n_valid) ? s1[0] * scale : -INFINITY;
            x[3] = (tb + 8 < n_valid) ? s1[1] * scale : -INFINITY;
            x[4] = (ta < n_valid) ? s0[2] * scale : -INFINITY;
            x[5] = (tb < n_valid) ? s0[3] * scale : -INFINITY;
            x[6] = (ta + 8 < n_valid) ? s1[2] * scale : -INFINITY;
            x[7] = (tb + 8 < n_valid) ? s1[3] * scale : -INFINITY;
            float mx = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            float mh = fmaxf(fmaxf(x[4], x[5]), fmaxf(x[6], x[7]));
            mh = fmaxf(mh, __shfl_xor_sync(0xffffffffu, mh, 1));
            mh = fmaxf(mh, __shfl_xor_sync(0xffffffffu, mh, 2));
            const float mn_lo = fmaxf(m_lo, mx), mn_hi = fmaxf(m_hi, mh);
            const float al_lo = __expf(m_lo - mn_lo), al_hi = __expf(m_hi - mn_hi);
            float pr[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) pr[i] = __expf(x[i] - mn_lo);
#pragma unroll
            for (int i = 4; i < 8; ++i) pr[i] = __expf(x[i] - mn_hi);
            l_lo = l_lo * al_lo + (pr[0] + pr[1] + pr[2] + pr[3]);
            l_hi = l_hi * al_hi + (pr[4] + pr[5] + pr[6] + pr[7]);
            m_lo = mn_lo; m_hi = mn_hi;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                acc[i][0] *= al_lo; acc[i][1] *= al_lo;
                acc[i][2] *= al_hi; acc[i][3] *= al_hi;
            }
            uint32_t ph[4], pl[4];
            {
                float hi[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    hi[i] = __bfloat162float(__float2bfloat16_rn(pr[i]));
                ph[0] = pack_bf16x2(hi[0], hi[1]);
                ph[1] = pack_bf16x2(hi[4], hi[5]);
                ph[2] = pack_bf16x2(hi[2], hi[3]);
                ph[3] = pack_bf16x2(hi[6], hi[7]);
                pl[0] = pack_bf16x2(pr[0] - hi[0], pr[1] - hi[1]);
                pl[1] = pack_bf16x2(pr[4] - hi[4], pr[5] - hi[5]);
                pl[2] = pack_bf16x2(pr[2] - hi[2], pr[3] - hi[3]);
                pl[3] = pack_bf16x2(pr[6] - hi[6], pr[7] - hi[7]);
            }
            // O[:, 128 warp .. +128) += P V
            const uint32_t va = kbase + vt * KV_PITCH + vcol;
#pragma unroll
            for (int dp = 0; dp < 8; ++dp) {
                uint32_t vb[4];
                ldmatrix_x4_trans(vb, va + 32 * dp);
                mma_bf16_k16(acc[2 * dp], ph[0], ph[1], ph[2], ph[3], vb[0], vb[1]);
                mma_bf16_k16(acc[2 * dp], pl[0], pl[1], pl[2], pl[3], vb[0], vb[1]);
                mma_bf16_k16(acc[2 * dp + 1], ph[0], ph[1], ph[2], ph[3], vb[2], vb[3]);
                mma_bf16_k16(acc[2 * dp + 1], pl[0], pl[1], pl[2], pl[3], vb[2], vb[3]);
            }
        }
        __syncthreads();                       // the stage is free again
        if (k + MD_STAGES < np) {
            if (((k + MD_STAGES) & 31) == 0) load_window(k + MD_STAGES);
            issue(k + MD_STAGES);
        }
    }

    // ---- cluster merge, push style: every warp holds the same (m, l) and its own
    // 128 output channels in registers; each value goes straight into the shared
    // memory of the CTA that normalises it (CTA d owns output elements
    // [d * per_e, (d + 1) * per_e)); one cluster barrier, then a local finish ----
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const int n_el = NH * LKV;
    const int per_e = (((n_el + CL - 1) / CL) + 3) & ~3;      // multiple of 4: 16-byte pushes
    if (warp == 0 && tig == 0) {
        for (int d = 0; d < CL; ++d) {
            float* rm = cluster.map_shared_rank(&sm.xm[c][0], d);
            float* rl = cluster.map_shared_rank(&sm.xl[c][0], d);
            rm[gid] = m_lo; rm[gid + 8] = m_hi;
            rl[gid] = l_lo; rl[gid + 8] = l_hi;
        }
    }
    // O goes through local shared memory so that every push instruction sends 512
    // contiguous bytes of ONE head to ONE CTA (a fragment-shaped push would
    // scatter 32-byte pieces over 16 CTAs per instruction)
    // (the page ring is idle after the loop's last barrier: it is the staging area)
    static_assert(sizeof(sm.kv) >= NH * OUT_PITCH * sizeof(float), "staging fits the ring");
    float (*stage_o)[OUT_PITCH] = reinterpret_cast<float (*)[OUT_PITCH]>(&sm.kv[0][0][0]);
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
        const int col = warp * 128 + 8 * nt + 2 * tig;
        *reinterpret_cast<float2*>(&stage_o[gid][col]) = make_float2(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<float2*>(&stage_o[gid + 8][col]) = make_float2(acc[nt][2], acc[nt][3]);
    }
    __syncthreads();
    for (int i = tid; i < NH * (LKV / 4); i += MD_THREADS) {
        const int h = i / (LKV / 4), c4 = i % (LKV / 4);
        const float4 val = *reinterpret_cast<const float4*>(&stage_o[h][4 * c4]);
        const int e = h * LKV + 4 * c4;
        const int d = e / per_e;
        float* dst = cluster.map_shared_rank(&sm.xacc[0], d) + c * per_e +
                     (e - d * per_e);
        *reinterpret_cast<float4*>(dst) = val;
    }
    cluster.sync();                              // every CTA's pushes have landed
    // merge weights once per (CTA, head): w[cc][h] = exp(m - M) / sum, lse[h]
    for (int h = tid; h < NH; h += MD_THREADS) {
        float M = -INFINITY;
        for (int cc = 0; cc < CL; ++cc) M = fmaxf(M, sm.xm[cc][h]);
        float Ls = 0.f;
        for (int cc = 0; cc < CL; ++cc) {
            const float lw = sm.xl[cc][h];
            const float wt = (lw > 0.f) ? __expf(sm.xm[cc][h] - M) : 0.f;
            sm.xm[cc][h] = wt;                       // reuse: now the weight
            Ls += wt * lw;
        }
        const float inv = (Ls > 0.f) ? 1.f / Ls : 0.f;
        for (int cc = 0; cc < CL; ++cc) sm.xm[cc][h] *= inv;
        if (c == 0) p.lse[(int64_t)row * NH + h] = (Ls > 0.f) ? M + __logf(Ls) : 0.f;
    }
    __syncthreads();
    for (int el = tid; el < per_e; el += MD_THREADS) {
        const int e = c * per_e + el;
        if (e >= n_el) break;
        const int h = e / LKV, d = e % LKV;
        float o = 0.f;
        for (int cc = 0; cc < CL; ++cc) o += sm.xm[cc][h] * sm.xacc[cc * per_e + el];
        p.out[((int64_t)row * NH + h) * LKV + d] = __float2bfloat16_rn(o);
    }
}

}  // namespace
}  // namespace locks

using namespace locks;


extern "C" int locks_mla_build_factors(const void* cache, int64_t stride_block,
                                       int64_t stride_tok, void* records,
                                       const int32_t* blocks, int n_blocks,
                                       int num_blocks, locks_stream_t stream) {
    LOCKS_REQUIRE(cache && records && (blocks || n_blocks == 0), LOCKS_ERR_ARG,
                  "locks_mla_build_factors: null pointer argument");
    LOCKS_REQUIRE(n_blocks >= 0 && num_blocks >= 1, LOCKS_ERR_ARG,
                  "locks_mla_build_factors: bad size argument");
    LOCKS_REQUIRE(stride_block % 8 == 0 && stride_tok % 8 == 0 &&
                      (reinterpret_cast<uintptr_t>(cache) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(records) & 15) == 0,
                  LOCKS_ERR_ARG,
                  "locks_mla_build_factors: cache/records must be 16-byte aligned "
                  "with strides that are multiples of 8 elements");
    if (n_blocks == 0) return LOCKS_OK;
    const int smem = (int)sizeof(FbScratch) * FB_WARPS;
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaFuncSetAttribute(mla_factor_kernel,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        attr_done[dev] = true;
    }
    FbParams p;
    p.cache = static_cast<const __nv_bfloat16*>(cache);
    p.sb = stride_block; p.st = stride_tok;
    p.records = static_cast<uint8_t*>(records);
    p.blocks = blocks; p.n_blocks = n_blocks; p.num_blocks = num_blocks;
    p.need = nullptr; p.n_cache = nullptr; p.block_table = nullptr;
    p.bt_stride = 0; p.max_pages = 1;
    mla_factor_kernel<<<(n_blocks + FB_WARPS - 1) / FB_WARPS, FB_WARPS * 32, smem,
                        static_cast<cudaStream_t>(stream)>>>(p);
    pdl_break();                       // the scorer prefetches factor records before its wait
    return check_launch("locks_mla_build_factors");
}

extern "C" int locks_mla_refresh_rows(
    const void* cache, int64_t stride_block, int64_t stride_tok, void* records,
    const int32_t* block_table, int64_t bt_stride, const int32_t* seq_lens,
    float* fp_tab, int32_t* nc_tab, int32_t* need, int32_t* n_cache, int n_rows,
    int max_pages, int num_blocks, locks_stream_t stream) {
    LOCKS_REQUIRE(cache && records && block_table && seq_lens && fp_tab && nc_tab &&
                      need && n_cache,
                  LOCKS_ERR_ARG, "locks_mla_refresh_rows: null pointer argument");
    LOCKS_REQUIRE(n_rows >= 0 && max_pages >= 1 && num_blocks >= 1 &&
                      (int64_t)n_rows * max_pages < (int64_t)1 << 31,
                  LOCKS_ERR_ARG, "locks_mla_refresh_rows: bad size argument");
    LOCKS_REQUIRE(stride_block % 8 == 0 && stride_tok % 8 == 0 &&
                      (reinterpret_cast<uintptr_t>(cache) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(records) & 15) == 0,
                  LOCKS_ERR_ARG, "locks_mla_refresh_rows: misaligned argument");
    if (n_rows == 0) return LOCKS_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    GateParams g;
    g.cache = static_cast<const __nv_bfloat16*>(cache);
    g.sb = stride_block; g.st = stride_tok;
    g.block_table = block_table; g.bt_stride = bt_stride; g.seq_lens = seq_lens;
    g.fp_tab = fp_tab; g.nc_tab = nc_tab; g.need = need; g.n_cache = n_cache;
    g.n_rows = n_rows; g.num_blocks = num_blocks; g.max_pages = max_pages;
    mla_gate_kernel<<<(n_rows + 3) / 4, 128, 0, s>>>(g);
    const int smem = (int)sizeof(FbScratch) * FB_WARPS;
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaFuncSetAttribute(mla_factor_kernel,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        attr_done[dev] = true;
    }
    FbParams p;
    p.cache = g.cache; p.sb = stride_block; p.st = stride_tok;
    p.records = static_cast<uint8_t*>(records);
    p.blocks = nullptr; p.n_blocks = n_rows * max_pages; p.num_blocks = num_blocks;
    p.need = need; p.n_cache = n_cache; p.block_table = block_table;
    p.bt_stride = bt_stride; p.max_pages = max_pages;
    mla_factor_kernel<<<(p.n_blocks + FB_WARPS - 1) / FB_WARPS, FB_WARPS * 32, smem,
                        s>>>(p);
    pdl_break();
    return check_launch("locks_mla_refresh_rows");
}

extern "C" int locks_mla_derive(const int32_t* seq_lens, int n_rows,
                                int budget_pages, int sink_pages,
                                int window_pages, int32_t* n_pages,
                                int32_t* n_sel_hi, int32_t* b_fix,
                                locks_stream_t stream) {
    LOCKS_REQUIRE(seq_lens && n_pages && n_sel_hi && b_fix, LOCKS_ERR_ARG,
                  "locks_mla_derive: null pointer argument");
    LOCKS_REQUIRE(n_rows >= 0 && budget_pages >= 1 && sink_pages >= 0 &&
                      window_pages >= 0,
                  LOCKS_ERR_ARG, "locks_mla_derive: bad size argument");
    if (n_rows == 0) return LOCKS_OK;
    mla_derive_kernel<<<(n_rows + 127) / 128, 128, 0,
                        static_cast<cudaStream_t>(stream)>>>(
        seq_lens, n_rows, budget_pages, sink_pages, window_pages, n_pages,
        n_sel_hi, b_fix);
    pdl_break();                       // the scorer reads the page counts before its wait
    return check_launch("locks_mla_derive");
}

extern "C" int locks_mla_score(const void* q, int64_t q_stride_row,
                               const void* records, const void* cache,
                               int64_t stride_block, int64_t stride_tok,
                               const int32_t* block_table, int64_t bt_stride,
                               const int32_t* n_cache, const int32_t* n_pages,
                               float* score, int n_rows, int max_pages,
                               int num_blocks, float scale, int zsplit,
                               int* status, locks_stream_t stream) {
    LOCKS_REQUIRE(q && records && cache && block_table && n_cache && n_pages &&
                      score,
                  LOCKS_ERR_ARG, "locks_mla_score: null pointer argument");
    LOCKS_REQUIRE(n_rows >= 0 && n_rows <= 65535 && max_pages >= 1 &&
                      num_blocks >= 1 && scale > 0.f,
                  LOCKS_ERR_ARG, "locks_mla_score: bad size argument");
    LOCKS_REQUIRE(stride_block % 8 == 0 && stride_tok % 8 == 0 &&
                      q_stride_row % 8 == 0 &&
                      (reinterpret_cast<uintptr_t>(cache) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(records) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(q) & 15) == 0,
                  LOCKS_ERR_ARG, "locks_mla_score: misaligned argument");
    if (n_rows == 0) return LOCKS_OK;
    const int smem = (int)sizeof(ScSmem);
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaFuncSetAttribute(mla_score_kernel,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        attr_done[dev] = true;
    }
    int Z = zsplit;
    if (Z <= 0) Z = (2 * sm_count() + n_rows - 1) / n_rows;
    Z = max(1, min(Z, min((max_pages + 2 * SC_WARPS - 1) / (2 * SC_WARPS), 65535)));
    MlaScoreParams p;
    p.q = static_cast<const __nv_bfloat16*>(q); p.q_stride_row = q_stride_row;
    p.records = static_cast<const uint8_t*>(records);
    p.cache = static_cast<const __nv_bfloat16*>(cache);
    p.sb = stride_block; p.st = stride_tok;
    p.block_table = block_table; p.bt_stride = bt_stride;
    p.n_cache = n_cache; p.n_pages = n_pages; p.score = score;
    p.max_pages = max_pages; p.num_blocks = num_blocks; p.scale = scale;
    p.status = status;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(Z, n_rows, 1);
    cfg.blockDim = dim3(SC_WARPS * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (pdl_enabled() && !pdl_take_break()) ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, mla_score_kernel, p);
    if (e != cudaSuccess)
        return fail(LOCKS_ERR_LAUNCH, "locks_mla_score: %s", cudaGetErrorString(e));
    return check_launch("locks_mla_score");
}

extern "C" int locks_mla_decode(const void* q, int64_t q_stride_row,
                                const void* cache, int64_t stride_block,
                                int64_t stride_tok, const int32_t* block_table,
                                int64_t bt_stride, const int32_t* page_table,
                                const int32_t* page_cnt, const int32_t* seq_lens,
                                void* out, float* lse, int n_rows, int max_pages,
                                float scale, int* status, locks_stream_t stream) {
    LOCKS_REQUIRE(q && cache && block_table && page_table && page_cnt &&
                      seq_lens && out && lse,
                  LOCKS_ERR_ARG, "locks_mla_decode: null pointer argument");
    LOCKS_REQUIRE(n_rows >= 0 && n_rows <= 65535 && max_pages >= 1, LOCKS_ERR_ARG,
                  "locks_mla_decode: bad size argument");
    LOCKS_REQUIRE(stride_block % 8 == 0 && stride_tok % 8 == 0 &&
                      q_stride_row % 8 == 0 &&
                      (reinterpret_cast<uintptr_t>(cache) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(q) & 15) == 0,
                  LOCKS_ERR_ARG, "locks_mla_decode: misaligned argument");
    if (n_rows == 0) return LOCKS_OK;
    const int smem = (int)sizeof(MdSmem);
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaFuncSetAttribute(mla_decode_kernel,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        cudaFuncSetAttribute(mla_decode_kernel,
                             cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        attr_done[dev] = true;
    }
    int cl = 1;
    {
        const int want = sm_count() / max(1, n_rows);
        while (cl * 2 <= want && cl < 8) cl *= 2;
        // 16-CTA clusters each need 16 free SMs of one GPC: only when all rows'
        // clusters fit at once (otherwise the launch runs in two rounds)
        static int fit16[64] = {0};
        if (cl == 8 && 16 * n_rows <= sm_count() && dev >= 0 && dev < 64) {
            if (fit16[dev] == 0)
                fit16[dev] = max(1, max_active_clusters(mla_decode_kernel, MD_MAX_CL, MD_THREADS, smem));
            if (n_rows <= fit16[dev]) cl = MD_MAX_CL;
        }
    }
    MlaDecParams p;
    p.q = static_cast<const __nv_bfloat16*>(q); p.q_stride_row = q_stride_row;
    p.cache = static_cast<const __nv_bfloat16*>(cache);
    p.sb = stride_block; p.st = stride_tok;
    p.block_table = block_table; p.bt_stride = bt_stride;
    p.page_table = page_table; p.page_cnt = page_cnt; p.seq_lens = seq_lens;
    p.out = static_cast<__nv_bfloat16*>(out); p.lse = lse;
    p.max_pages = max_pages; p.scale = scale; p.status = status;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cl, n_rows, 1);
    cfg.blockDim = dim3(MD_THREADS, 1, 1);
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
    cudaError_t e = cudaLaunchKernelEx(&cfg, mla_decode_kernel, p);
    if (e != cudaSuccess)
        return fail(LOCKS_ERR_LAUNCH, "locks_mla_decode: %s", cudaGetErrorString(e));
    return check_launch("locks_mla_decode");
}
