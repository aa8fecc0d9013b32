// MLA decode on the 5th-generation tensor cores (tcgen05 + TMEM), TOKENS in the
// M dimension.
//
// The 16 query heads of an MLA layer share one latent head of 512 + 64 rope
// channels.  With the heads as matrix rows (the warp-level kernel of mla.cu) a
// tile has 16 rows; tcgen05.mma needs M = 128.  Transposed, the tiles are dense:
//
//   S^T [128 tokens x 16 heads]  = K   [128 tokens x 576] . Q^T [576 x 16]
//   O^T [512 ch     x 16 heads]  = V^T [512 ch x 128 tokens] . P^T [128 x 16]
//                                  (4 blocks of M = 128 channels)
//
// A CTA (4 warps) walks its share of a row's kept pages in tiles of 8 pages =
// 128 tokens:
//   * the 8 pages are gathered through the block table by TMA: a 2-D tensor map
//     over the latent cache viewed as (num_blocks * 16 tokens, 576) with a
//     (16 tokens, 64 channels) box and the 128-byte swizzle, 9 boxes per page,
//     all completing on one mbarrier.  The tile lands as 9 chunks of
//     [128 tokens][128 B]: read K-major (token rows) it is the A operand of
//     S^T, read MN-major (channel rows) chunks 0-7 are the A operand of O^T --
//     one copy of the page serves both products;
//   * one thread issues 36 tcgen05.mma (K = 16 each) for S^T into TMEM columns
//     0-15, commits to an mbarrier; the 128 threads read their token's 16
//     logits with tcgen05.ld (thread = TMEM lane = token), mask, and do the
//     per-head softmax statistics through shared memory (online over tiles);
//   * P (bf16) goes to shared memory in the K-major swizzled layout of a B
//     operand; one thread issues 4 x (pages of the tile) tcgen05.mma for O^T
//     into TMEM columns 16-79; every thread then owns one output channel of each
//     128-block (thread = TMEM lane = channel) and folds the tile into its
//     running 4 x 16 accumulators with the online-softmax rescale.
// The CTAs of a row's cluster meet exactly as in the warp-level kernel: each
// pushes its (m, l) and the output slice CTA d normalises into CTA d's shared
// memory, one cluster barrier, local finish.
//
// Every mbarrier wait is bounded (status word, then the kernel carries on and
// releases its TMEM).  All loads are of this GPU's own memory; no multicast.
#include <cooperative_groups.h>
#include <cuda.h>

#include "common.cuh"
#include "tma.cuh"

namespace cg = cooperative_groups;

namespace locks {
namespace {

constexpr int LKV = LOCKS_MLA_LKV;        // 512
constexpr int ROPE = LOCKS_MLA_ROPE;      // 64
constexpr int WIDTH = LKV + ROPE;         // 576
constexpr int NH = LOCKS_MLA_HEADS;       // 16
constexpr int PG = 16;
constexpr int TC_THREADS = 128;
constexpr int TILE_PAGES = 8;
constexpr int TILE_TOK = TILE_PAGES * PG;             // 128
constexpr int NCHUNK = WIDTH / 64;                    // 9 chunks of 64 channels
constexpr int CHUNK_BYTES = TILE_TOK * 128;           // 16 KiB: [token][128 B]
constexpr int PAGE_CHUNK_BYTES = PG * 128;            // one TMA box
constexpr int QP_CHUNK_BYTES = NH * 128;              // [head][128 B]
constexpr int TMEM_COLS = 128;                        // S: 0-15, O: 16-79
constexpr int TC_MAX_CL = 16;
constexpr int S_PITCH = TILE_TOK + 4;

struct __align__(1024) TcSmem {
    uint8_t kt[NCHUNK * CHUNK_BYTES];     // page tile (TMA, 128-byte swizzle)
    uint8_t q[NCHUNK * QP_CHUNK_BYTES];   // Q^T as a B operand (K-major, swizzled)
    uint8_t p[2 * QP_CHUNK_BYTES];        // P^T as a B operand: 2 chunks of 64 tokens
    float sS[NH][S_PITCH];                // logits / probabilities, head-major
    float xacc[NH * LKV + 64];            // cluster merge: slices pushed to this CTA
    float xm[TC_MAX_CL][NH], xl[TC_MAX_CL][NH];
    float mrun[NH], lrun[NH], mnew[NH], alpha[NH];
    int tile_pt[TILE_PAGES];
    uint64_t bar_full, bar_s, bar_o;
    uint32_t tmem_base;
};

struct TcParams {
    const __nv_bfloat16* q;
    int64_t q_stride_row;
    const int32_t* block_table;
    int64_t bt_stride;
    const int32_t* page_table;
    const int32_t* page_cnt;
    const int32_t* seq_lens;
    __nv_bfloat16* out;
    float* lse;
    int max_pages, num_blocks;
    int cnt_hint;                  // pages a long row keeps (the budget): a guess
    float scale;
    int* status;
};

// shared-memory matrix descriptor, 128-byte swizzle (layout type 2), version 1
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes,
                                              uint32_t sbo_bytes) {
    uint64_t d = (uint64_t)((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// instruction descriptor, kind::f16: bf16 x bf16 -> f32, M = 128, N = 16
constexpr uint32_t IDESC_BASE = (1u << 4) | (1u << 7) | (1u << 10) |
                                ((uint32_t)(NH >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t IDESC_S = IDESC_BASE;                 // A K-major, B K-major
constexpr uint32_t IDESC_O = IDESC_BASE | (1u << 15);    // A MN-major (V^T)

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a, uint64_t b,
                                         uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile(
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
        ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
          "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
          "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// byte offset of (row, byte-in-row) inside a [rows][128 B] tile with the 128-byte
// swizzle (16-byte pieces of a row XORed with the row number mod 8)
__device__ __forceinline__ int swz128(int row, int byte) {
    return row * 128 + ((((byte >> 4) ^ (row & 7)) << 4) | (byte & 15));
}

__global__ void __launch_bounds__(TC_THREADS)
mla_tc_decode_kernel(const __grid_constant__ CUtensorMap tmap, const TcParams p) {
    extern __shared__ __align__(16) uint8_t tc_raw[];
    // the swizzled tiles need a 1 KiB-aligned base (the launch reserves the slack;
    // the offset is the same in every CTA, so cluster-mapped addresses agree)
    TcSmem& sm = *reinterpret_cast<TcSmem*>(
        tc_raw + ((1024u - (smem_u32(tc_raw) & 1023u)) & 1023u));
    cg::cluster_group cluster = cg::this_cluster();
    const int c = blockIdx.x, CL = gridDim.x, row = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    if (tid == 0) {
        mbar_init(&sm.bar_full, 1);
        mbar_init(&sm.bar_s, 1);
        mbar_init(&sm.bar_o, 1);
        mbar_fence_init();
    }
    if (tid < NH) { sm.mrun[tid] = -INFINITY; sm.lrun[tid] = 0.f; }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;"
                     ::: "memory");
        tc_fence_before();
    }
    pdl_trigger();
    cluster.sync();                  // barriers, TMEM base and peers' CTAs are up
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    // ---- Q^T into the swizzled K-major B layout: [chunk][head][128 B].  q is an
    // input of the whole layer (the scorer of this layer has read it already), not
    // a product of the selector, so it is staged ahead of the dependency wait;
    // all loads are in flight before the first store --------------------------------
    {
        const uint4* q4 = reinterpret_cast<const uint4*>(p.q + (int64_t)row * p.q_stride_row);
        constexpr int C16 = WIDTH * 2 / 16;            // 72 pieces per head
        constexpr int NQ = NH * C16 / TC_THREADS;      // 9 per thread
        static_assert(NH * C16 % TC_THREADS == 0, "q pieces divide over the threads");
        uint4 v[NQ];
#pragma unroll
        for (int i = 0; i < NQ; ++i) v[i] = q4[tid + i * TC_THREADS];
#pragma unroll
        for (int i = 0; i < NQ; ++i) {
            const int e = tid + i * TC_THREADS;
            const int h = e / C16, pc = e % C16;       // piece pc = channels 8pc..8pc+7
            const int chunk = pc >> 3, byte = (pc & 7) << 4;
            *reinterpret_cast<uint4*>(&sm.q[chunk * QP_CHUNK_BYTES + swz128(h, byte)]) = v[i];
        }
        fence_proxy_async();
    }
    pdl_wait();                      // the page table comes from the selector

    const int32_t* tab = p.page_table + (int64_t)row * p.max_pages;
    const int32_t* bt = p.block_table + (int64_t)row * p.bt_stride;
    // The first tile's page-table entries are fetched TOGETHER with the page count,
    // at the place the count is expected to put them (a long row keeps exactly its
    // budget): one dependent round trip less when the guess holds.
    const int per_g = (p.cnt_hint + CL - 1) / CL;
    const int jg = c * per_g + lane;
    int spec_pt = -1;
    if (warp == 0 && lane < TILE_PAGES && jg < p.max_pages) spec_pt = __ldcg(&tab[jg]);
    const int seq_len = p.seq_lens[row];
    const int cnt = min(max(__ldcg(&p.page_cnt[row]), 0), p.max_pages);
    const int per = (cnt + CL - 1) / CL;
    const int j0 = min(c * per, cnt), j1 = min(j0 + per, cnt);
    const int np = j1 - j0;
    const bool spec_ok = per == per_g && j0 == c * per_g;

    float acc[4][NH];
#pragma unroll
    for (int mb = 0; mb < 4; ++mb)
#pragma unroll
        for (int h = 0; h < NH; ++h) acc[mb][h] = 0.f;

    const uint32_t kt_addr = smem_u32(sm.kt), q_addr = smem_u32(sm.q),
                   p_addr = smem_u32(sm.p);
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;

    int tile = 0;
    for (int t0 = 0; t0 < np; t0 += TILE_PAGES, ++tile) {
        const int nt = min(TILE_PAGES, np - t0);
        const uint32_t parity = (uint32_t)(tile & 1);
        // ---- gather the tile's pages: 9 boxes per page, one mbarrier -----------
        if (warp == 0) {
            int pt = -1, blk = 0;
            if (lane < nt) {
                pt = (t0 == 0 && spec_ok) ? spec_pt : tab[j0 + t0 + lane];
                blk = min(max(bt[max(pt, 0)], 0), p.num_blocks - 1);
                sm.tile_pt[lane] = pt;
            }
            if (lane == 0)
                mbar_expect_tx(&sm.bar_full, (uint32_t)nt * NCHUNK * PAGE_CHUNK_BYTES);
            __syncwarp();
            // the 9 x nt boxes are issued by all 32 lanes (a request costs its
            // issuer tens of cycles)
            // (every lane runs every round: the shuffle needs the whole warp)
            for (int i0 = 0; i0 < nt * NCHUNK; i0 += 32) {
                const int i = i0 + lane;
                const bool on = i < nt * NCHUNK;
                const int slot = on ? i / NCHUNK : 0, ch = i - slot * NCHUNK;
                const int b = __shfl_sync(0xffffffffu, blk, slot);
                if (on)
                    tma_load_2d(&sm.kt[ch * CHUNK_BYTES + slot * PAGE_CHUNK_BYTES],
                                &tmap, ch * 64, b * PG, &sm.bar_full);
            }
        }
        __syncthreads();                               // tile_pt is visible
        mbar_wait(&sm.bar_full, parity, p.status);
        // rows of a partial page at or beyond seq_len may hold anything: zero them
        // (their logits are masked, but 0 x NaN would poison P V)
        {
            const int last = nt - 1;
            const int nv = min(max(seq_len - sm.tile_pt[last] * PG, 0), PG);
            if (nv < PG) {
                const int nrow = PG - nv;
                for (int e = tid; e < NCHUNK * nrow * 8; e += TC_THREADS) {
                    const int ch = e / (nrow * 8), r = nv + (e / 8) % nrow, pc = e & 7;
                    *reinterpret_cast<uint4*>(&sm.kt[ch * CHUNK_BYTES +
                                                     (last * PG + r) * 128 + pc * 16]) =
                        make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();
            }
        }
        __syncthreads();
        // ---- S^T = K . Q^T : 9 chunks x 4 k-steps of 16 channels -------------------
        if (tid == 0) {
            tc_fence_after();
            // descriptors differ only in their start-address field (16-byte units)
            const uint64_t a0 = umma_desc(kt_addr, 16, 1024);
            const uint64_t b0 = umma_desc(q_addr, 16, 1024);
#pragma unroll
            for (int ch = 0; ch < NCHUNK; ++ch) {
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    umma_f16(tmem, a0 + (uint64_t)((ch * CHUNK_BYTES + ks * 32) >> 4),
                             b0 + (uint64_t)((ch * QP_CHUNK_BYTES + ks * 32) >> 4),
                             IDESC_S, (ch | ks) ? 1u : 0u);
                }
            }
            umma_commit(&sm.bar_s);
        }
        mbar_wait(&sm.bar_s, parity, p.status);
        tc_fence_after();
        // ---- this thread's token: 16 logits, masked ---------------------------------
        float x[NH];
        tmem_ld16(tmem + lane_off, x);
        {
            const int slot = tid >> 4, tt = tid & 15;
            const bool valid = slot < nt && (sm.tile_pt[slot < nt ? slot : 0] * PG + tt) < seq_len;
#pragma unroll
            for (int h = 0; h < NH; ++h) {
                x[h] = valid ? x[h] * p.scale : -INFINITY;
                sm.sS[h][tid] = x[h];
            }
        }
        __syncthreads();
        // per-head maximum of the tile: thread (h, seg) takes 16 tokens
        {
            const int h = tid >> 3, seg = tid & 7;
            float m = -INFINITY;
#pragma unroll
            for (int i = 0; i < 16; ++i) m = fmaxf(m, sm.sS[h][seg * 16 + i]);
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
            if (seg == 0) {
                const float mo = sm.mrun[h], mn = fmaxf(mo, m);
                sm.mnew[h] = mn;
                sm.alpha[h] = __expf(mo - mn);           // 0 on the first tile
            }
        }
        __syncthreads();
        // probabilities: bf16 into the B operand of P V, fp32 into sS for the sums
        {
            const int chunk = tid >> 6, byte = (tid & 63) * 2;
#pragma unroll
            for (int h = 0; h < NH; ++h) {
                const float pv = __expf(x[h] - sm.mnew[h]);
                sm.sS[h][tid] = pv;
                *reinterpret_cast<__nv_bfloat16*>(
                    &sm.p[chunk * QP_CHUNK_BYTES + swz128(h, byte)]) = __float2bfloat16_rn(pv);
            }
            fence_proxy_async();
        }
        tc_fence_before();
        __syncthreads();
        // ---- O^T = V^T . P^T : 4 channel blocks x nt k-steps of one page ----------
        if (tid == 0) {
            tc_fence_after();
            const uint64_t a0 = umma_desc(kt_addr, CHUNK_BYTES, 1024);
            const uint64_t b0 = umma_desc(p_addr, 16, 1024);
#pragma unroll
            for (int mb = 0; mb < 4; ++mb) {
#pragma unroll
                for (int ks = 0; ks < TILE_PAGES; ++ks) {
                    if (ks < nt)
                        umma_f16(tmem + 16 + 16 * mb,
                                 a0 + (uint64_t)(((2 * mb) * CHUNK_BYTES + ks * 2048) >> 4),
                                 b0 + (uint64_t)(((ks >> 2) * QP_CHUNK_BYTES + (ks & 3) * 32) >> 4),
                                 IDESC_O, ks ? 1u : 0u);
                }
            }
            umma_commit(&sm.bar_o);
        }
        // the tile's row sums, while the tensor cores work
        {
            const int h = tid >> 3, seg = tid & 7;
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) s += sm.sS[h][seg * 16 + i];
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            if (seg == 0) {
                sm.lrun[h] = sm.lrun[h] * sm.alpha[h] + s;
                sm.mrun[h] = sm.mnew[h];
            }
        }
        mbar_wait(&sm.bar_o, parity, p.status);
        tc_fence_after();
#pragma unroll
        for (int mb = 0; mb < 4; ++mb) {
            float o[NH];
            tmem_ld16(tmem + lane_off + 16 + 16 * mb, o);
#pragma unroll
            for (int h = 0; h < NH; ++h) acc[mb][h] = acc[mb][h] * sm.alpha[h] + o[h];
        }
        tc_fence_before();
        __syncthreads();                 // TMEM, the tile and the statistics are free
    }

    // ---- cluster merge (push style, as the warp-level kernel) ---------------------
    const int n_el = NH * LKV;
    const int per_e = (((n_el + CL - 1) / CL) + 3) & ~3;
    if (tid < NH) {
        for (int d = 0; d < CL; ++d) {
            cluster.map_shared_rank(&sm.xm[c][0], d)[tid] = sm.mrun[tid];
            cluster.map_shared_rank(&sm.xl[c][0], d)[tid] = sm.lrun[tid];
        }
    }
    // this thread owns channel mb * 128 + tid of every head: each value goes
    // straight to the CTA that normalises it (a warp's store covers 128
    // contiguous bytes of one head in one CTA)
#pragma unroll
    for (int mb = 0; mb < 4; ++mb) {
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            const int e = h * LKV + mb * 128 + tid;
            const int d = e / per_e;
            cluster.map_shared_rank(&sm.xacc[0], d)[c * per_e + (e - d * per_e)] =
                acc[mb][h];
        }
    }
    cluster.sync();                              // every CTA's pushes have landed
    if (warp == 0) {                             // all tcgen05.ld of this CTA are done
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
    {   // merge weights: 8 threads per head, each takes CTAs sub, sub + 8
        const int h = tid >> 3, sub = tid & 7;
        float mv[2], lv[2];
        float M = -INFINITY;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int cc = sub + 8 * i;
            mv[i] = (cc < CL) ? sm.xm[cc][h] : -INFINITY;
            lv[i] = (cc < CL) ? sm.xl[cc][h] : 0.f;
            M = fmaxf(M, mv[i]);
        }
        M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, 1));
        M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, 2));
        M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, 4));
        float wt[2], Ls = 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            wt[i] = (lv[i] > 0.f) ? __expf(mv[i] - M) : 0.f;
            Ls += wt[i] * lv[i];
        }
        Ls += __shfl_xor_sync(0xffffffffu, Ls, 1);
        Ls += __shfl_xor_sync(0xffffffffu, Ls, 2);
        Ls += __shfl_xor_sync(0xffffffffu, Ls, 4);
        const float inv = (Ls > 0.f) ? 1.f / Ls : 0.f;
        __syncwarp();                            // every lane has read xm / xl
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int cc = sub + 8 * i;
            if (cc < CL) sm.xm[cc][h] = wt[i] * inv;     // reuse: now the weight
        }
        if (c == 0 && sub == 0)
            p.lse[(int64_t)row * NH + h] = (Ls > 0.f) ? M + __logf(Ls) : 0.f;
    }
    __syncthreads();
    for (int el = tid; el < per_e; el += TC_THREADS) {
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

// Cluster size of a launch: as many CTAs per row as fit in one wave, a power of
// two up to 8; 16 (non-portable) only when every row's cluster fits at once AND
// eight CTAs would each walk more than four tiles -- for a short list two tiles in
// an 8-CTA cluster cost less than one tile plus a 16-CTA exchange.
static int tc_cluster_size(int n_rows, int pages_hint, int dev, int smem) {
    using namespace locks;
    int cl = 1;
    const int want = sm_count() / max(1, n_rows);
    while (cl * 2 <= want && cl < 8) cl *= 2;
    static int fit16[64] = {0};
    const int tiles_at_8 = (pages_hint + 8 * TILE_PAGES - 1) / (8 * TILE_PAGES);
    if (cl == 8 && 16 * n_rows <= sm_count() && tiles_at_8 > 4 && dev >= 0 &&
        dev < 64) {
        if (fit16[dev] == 0)
            fit16[dev] = max(1, max_active_clusters(mla_tc_decode_kernel, TC_MAX_CL,
                                                    TC_THREADS, smem));
        if (n_rows <= fit16[dev]) cl = TC_MAX_CL;
    }
    return cl;
}

extern "C" int locks_mla_decode_tc_cluster_size(int n_rows, int pages_hint) {
    using namespace locks;
    int dev = 0;
    cudaGetDevice(&dev);
    return tc_cluster_size(max(n_rows, 1), max(pages_hint, 0), dev,
                           (int)sizeof(TcSmem) + 1024);
}

using namespace locks;

extern "C" int locks_mla_decode_tc(const void* q, int64_t q_stride_row,
                                   const void* cache, int64_t stride_block,
                                   int64_t stride_tok, const int32_t* block_table,
                                   int64_t bt_stride, const int32_t* page_table,
                                   const int32_t* page_cnt, const int32_t* seq_lens,
                                   void* out, float* lse, int n_rows, int max_pages,
                                   int num_blocks, int cnt_hint, float scale,
                                   int* status, locks_stream_t stream) {
    LOCKS_REQUIRE(q && cache && block_table && page_table && page_cnt &&
                      seq_lens && out && lse,
                  LOCKS_ERR_ARG, "locks_mla_decode_tc: null pointer argument");
    LOCKS_REQUIRE(n_rows >= 0 && n_rows <= 65535 && max_pages >= 1 && num_blocks >= 1,
                  LOCKS_ERR_ARG, "locks_mla_decode_tc: bad size argument");
    LOCKS_REQUIRE(q_stride_row % 8 == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(cache) & 15) == 0,
                  LOCKS_ERR_ARG, "locks_mla_decode_tc: misaligned argument");
    // the tensor map sees the cache as one (num_blocks * 16, 576) matrix: token
    // rows must be evenly spaced across block boundaries, 16-byte multiples apart
    LOCKS_REQUIRE(stride_block == (int64_t)PG * stride_tok && stride_tok >= WIDTH &&
                      (stride_tok * 2) % 16 == 0,
                  LOCKS_ERR_GEOMETRY,
                  "locks_mla_decode_tc: the latent cache must be (num_blocks, 16, "
                  ">=576) with block stride 16 x token stride (got %lld, %lld); use "
                  "locks_mla_decode for other layouts",
                  (long long)stride_block, (long long)stride_tok);
    if (n_rows == 0) return LOCKS_OK;
    CUtensorMap tmap;
    const CUresult cr = encode_bf16_rows_sw128(&tmap, cache, WIDTH,
                                               (uint64_t)num_blocks * PG,
                                               (uint64_t)stride_tok, PG);
    LOCKS_REQUIRE(cr == CUDA_SUCCESS, LOCKS_ERR_LAUNCH,
                  "locks_mla_decode_tc: cuTensorMapEncodeTiled failed (%d)", (int)cr);
    const int smem = (int)sizeof(TcSmem) + 1024;       // room to align to 1 KiB
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaFuncSetAttribute(mla_tc_decode_kernel,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        cudaFuncSetAttribute(mla_tc_decode_kernel,
                             cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        attr_done[dev] = true;
    }
    const int p_hint = min(max(cnt_hint, 0), max_pages);
    const int cl = tc_cluster_size(n_rows, p_hint, dev, smem);
    TcParams p;
    p.q = static_cast<const __nv_bfloat16*>(q); p.q_stride_row = q_stride_row;
    p.block_table = block_table; p.bt_stride = bt_stride;
    p.page_table = page_table; p.page_cnt = page_cnt; p.seq_lens = seq_lens;
    p.out = static_cast<__nv_bfloat16*>(out); p.lse = lse;
    p.max_pages = max_pages; p.num_blocks = num_blocks; p.scale = scale;
    p.cnt_hint = min(max(cnt_hint, 0), max_pages);
    p.status = status;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cl, n_rows, 1);
    cfg.blockDim = dim3(TC_THREADS, 1, 1);
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
    cudaError_t e = cudaLaunchKernelEx(&cfg, mla_tc_decode_kernel, tmap, p);
    if (e != cudaSuccess)
        return fail(LOCKS_ERR_LAUNCH, "locks_mla_decode_tc: %s", cudaGetErrorString(e));
    return check_launch("locks_mla_decode_tc");
}
