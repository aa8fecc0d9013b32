// rki4 summary builder: one warp per (layer, physical block, kv-head).
//
//   load   16 x 128 bf16 keys (lane l owns channels 4l..4l+3 of every token)
//   mu     channel mean over the 16 tokens; dc = K - mu  -> shared memory (fp32)
//   Gram   16 x 16 = dc dc^T, 8 entries per lane
//   eigh   two-sided parallel-order Jacobi in shared memory: 15 rounds of 8
//          disjoint rotations per sweep, rotation angles by 8 lanes, row /
//          column / eigenvector updates by all 32, until a sweep rotates nothing
//   top-8  eigenpairs in ascending order (column 7 = largest)
//   C = U8 S8 (16 x 8), V = dc^T U8 / S8 (128 x 8), quantise + pack + store
//
// Eigenvectors are unique only up to sign, so the int4/int8 codes agree with a
// LAPACK-based build only after the per-column sign is aligned; scales, the
// centroid and every score computed from the record are sign-free.
#include "common.cuh"
#include "jacobi16.cuh"

namespace locks {
namespace {

constexpr int BW = 4;                  // warps (jobs) per CTA
constexpr int PAGE_T = 16;
constexpr int HD = 128;
constexpr int DC_PITCH = HD + 4;       // floats, keeps float4 rows conflict-free

struct WarpScratch {
    float dc[PAGE_T][DC_PITCH];
    float A[PAGE_T][PAGE_T + 1];
    float U[PAGE_T][PAGE_T + 1];
    float rc[8], rs[8];
    float s8[8];
    int idx[8];
};

struct BuildParams {
    const void* const* k_layers;
    int64_t sb, st, sh;                // element strides of a K plane
    uint8_t* records;
    __nv_bfloat16* tags;
    const int32_t* blocks;
    int n_blocks, layer0, n_layers, nb_state, nb_cache, n_kv;
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__global__ void __launch_bounds__(BW * 32) rki4_build_kernel(const BuildParams p) {
    __shared__ __align__(16) WarpScratch scratch[BW];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t job = (int64_t)blockIdx.x * BW + warp;
    const int64_t n_jobs = (int64_t)p.n_layers * p.n_blocks * p.n_kv;
    if (job >= n_jobs) return;
    const int kh = (int)(job % p.n_kv);
    const int bi = (int)((job / p.n_kv) % p.n_blocks);
    const int layer = p.layer0 + (int)(job / ((int64_t)p.n_kv * p.n_blocks));
    const int blk = p.blocks[bi];
    if (blk < 0 || blk >= p.nb_state || blk >= p.nb_cache) return;
    WarpScratch& ws = scratch[warp];

    const __nv_bfloat16* K =
        static_cast<const __nv_bfloat16*>(p.k_layers[layer]) +
        (int64_t)blk * p.sb + (int64_t)kh * p.sh;

    // ---- load, centroid, centred keys ----------------------------------------
    float kv[PAGE_T][4];
    float mu[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int t = 0; t < PAGE_T; ++t) {
        const uint2 raw =
            *reinterpret_cast<const uint2*>(K + (int64_t)t * p.st + 4 * lane);
        kv[t][0] = bf16_bits_to_f32(raw.x & 0xFFFFu);
        kv[t][1] = bf16_bits_to_f32(raw.x >> 16);
        kv[t][2] = bf16_bits_to_f32(raw.y & 0xFFFFu);
        kv[t][3] = bf16_bits_to_f32(raw.y >> 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) mu[i] += kv[t][i];
        if (t == PAGE_T - 1 && lane < 2) {
            // content tag: first 8 channels of the page-final token, raw bf16
            __nv_bfloat16* tg = p.tags +
                (((int64_t)layer * p.nb_state + blk) * p.n_kv + kh) * LOCKS_TAG_WIDTH;
            *reinterpret_cast<uint2*>(tg + 4 * lane) = raw;
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) mu[i] = __fdiv_rn(mu[i], (float)PAGE_T);
#pragma unroll
    for (int t = 0; t < PAGE_T; ++t)
        *reinterpret_cast<float4*>(&ws.dc[t][4 * lane]) =
            make_float4(kv[t][0] - mu[0], kv[t][1] - mu[1], kv[t][2] - mu[2],
                        kv[t][3] - mu[3]);
    __syncwarp();

    // ---- Gram: lane -> row i = lane/2, columns j0..j0+7 ------------------------
    {
        const int i = lane >> 1, j0 = (lane & 1) * 8;
        float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int d = 0; d < HD; d += 4) {
            const float4 a = *reinterpret_cast<const float4*>(&ws.dc[i][d]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float4 b = *reinterpret_cast<const float4*>(&ws.dc[j0 + j][d]);
                g[j] = fmaf(a.x, b.x, g[j]);
                g[j] = fmaf(a.y, b.y, g[j]);
                g[j] = fmaf(a.z, b.z, g[j]);
                g[j] = fmaf(a.w, b.w, g[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ws.A[i][j0 + j] = g[j];
        // U = identity
#pragma unroll
        for (int j = 0; j < 8; ++j) ws.U[i][j0 + j] = (i == j0 + j) ? 1.f : 0.f;
    }
    __syncwarp();
    // symmetrise exactly (the two triangles come from different FMA orders)
    if (lane < PAGE_T)
        for (int j = lane + 1; j < PAGE_T; ++j) ws.A[j][lane] = ws.A[lane][j];
    __syncwarp();

    jacobi16_warp(ws.A, ws.U, ws.rc, ws.rs, lane);

    // ---- rank the eigenvalues, keep the top 8 in ascending order ----------------
    if (lane < PAGE_T) {
        const float lam = ws.A[lane][lane];
        int pos = 0;
        for (int j = 0; j < PAGE_T; ++j) {
            const float lj = ws.A[j][j];
            pos += (lj < lam) || (lj == lam && j < lane);
        }
        if (pos >= 8) {
            ws.idx[pos - 8] = lane;
            ws.s8[pos - 8] = __fsqrt_rn(fmaxf(lam, 1e-10f));
        }
    }
    __syncwarp();

    uint8_t* rec = p.records +
        (((int64_t)layer * p.nb_state + blk) * p.n_kv + kh) * REC_BYTES;

    // ---- C = U8 * S8 : lane -> token t = lane/2, columns r0..r0+3 ---------------
    {
        const int t = lane >> 1, r0 = (lane & 1) * 4;
        float c[4], amax = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            c[j] = ws.U[t][ws.idx[r0 + j]] * ws.s8[r0 + j];
            amax = fmaxf(amax, fabsf(c[j]));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        const float cs = fmaxf(__fdiv_rn(amax, 127.f), 1e-8f);
        uint32_t packed = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float qv = fminf(fmaxf(rintf(__fdiv_rn(c[j], cs)), -127.f), 127.f);
            packed |= (uint32_t)((int)qv & 0xFF) << (8 * j);
        }
        *reinterpret_cast<uint32_t*>(rec + RO_C8 + t * 8 + r0) = packed;
        if ((lane & 1) == 0)
            *reinterpret_cast<__nv_bfloat16*>(rec + RO_CS + 2 * t) =
                __float2bfloat16_rn(cs);
    }

    // ---- V = dc^T U8 / S8 : lane -> channels 4l..4l+3, all 8 columns -------------
    {
        float v[8][4];
#pragma unroll
        for (int r = 0; r < 8; ++r) v[r][0] = v[r][1] = v[r][2] = v[r][3] = 0.f;
        for (int t = 0; t < PAGE_T; ++t) {
            const float4 x = *reinterpret_cast<const float4*>(&ws.dc[t][4 * lane]);
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const float u = ws.U[t][ws.idx[r]];
                v[r][0] = fmaf(x.x, u, v[r][0]);
                v[r][1] = fmaf(x.y, u, v[r][1]);
                v[r][2] = fmaf(x.z, u, v[r][2]);
                v[r][3] = fmaf(x.w, u, v[r][3]);
            }
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const float s8 = ws.s8[r];
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[r][i] = __fdiv_rn(v[r][i], s8);
                amax = fmaxf(amax, fabsf(v[r][i]));
            }
            amax = warp_max(amax);
            const float vs = fmaxf(__fdiv_rn(amax, 7.f), 1e-8f);
            int q[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                q[i] = (int)fminf(fmaxf(rintf(__fdiv_rn(v[r][i], vs)), -8.f), 7.f);
            // channels 4l,4l+1 -> byte 2l ; 4l+2,4l+3 -> byte 2l+1 (low = even)
            const uint32_t b0 = (uint32_t)(q[0] & 15) | ((uint32_t)(q[1] & 15) << 4);
            const uint32_t b1 = (uint32_t)(q[2] & 15) | ((uint32_t)(q[3] & 15) << 4);
            *reinterpret_cast<uint16_t*>(rec + RO_V4 + r * 64 + 2 * lane) =
                (uint16_t)(b0 | (b1 << 8));
            if (lane == r)
                *reinterpret_cast<__nv_bfloat16*>(rec + RO_VS + 2 * r) =
                    __float2bfloat16_rn(vs);
        }
    }

    // ---- centroid ------------------------------------------------------------------
    {
        float amax = fmaxf(fmaxf(fabsf(mu[0]), fabsf(mu[1])),
                           fmaxf(fabsf(mu[2]), fabsf(mu[3])));
        amax = warp_max(amax);
        const float ms = fmaxf(__fdiv_rn(amax, 127.f), 1e-8f);
        uint32_t packed = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float qv = fminf(fmaxf(rintf(__fdiv_rn(mu[i], ms)), -127.f), 127.f);
            packed |= (uint32_t)((int)qv & 0xFF) << (8 * i);
        }
        *reinterpret_cast<uint32_t*>(rec + RO_MU8 + 4 * lane) = packed;
        if (lane == 0)
            *reinterpret_cast<__nv_bfloat16*>(rec + RO_MUS) = __float2bfloat16_rn(ms);
    }
}

struct TagScanParams {
    const void* const* k_layers;
    int64_t sb, st, sh;
    const __nv_bfloat16* tags;
    const int32_t* blocks;
    const uint8_t* valid;
    uint8_t* stale;
    int n_blocks, n_layers, nb_state, n_kv, page;
};

// one warp per listed block; lanes stride over (layer, kv-head) pairs
__global__ void __launch_bounds__(128) tag_scan_kernel(const TagScanParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i = blockIdx.x * 4 + warp;
    if (i >= p.n_blocks) return;
    const int blk = p.blocks[i];
    bool bad = false;
    if (p.valid[i] && blk >= 0 && blk < p.nb_state) {
        const int n = p.n_layers * p.n_kv;
        for (int e = lane; e < n; e += 32) {
            const int l = e / p.n_kv, kh = e % p.n_kv;
            const __nv_bfloat16* cur =
                static_cast<const __nv_bfloat16*>(p.k_layers[l]) +
                (int64_t)blk * p.sb + (int64_t)(p.page - 1) * p.st +
                (int64_t)kh * p.sh;
            const __nv_bfloat16* old = p.tags +
                (((int64_t)l * p.nb_state + blk) * p.n_kv + kh) * LOCKS_TAG_WIDTH;
#pragma unroll
            for (int c = 0; c < LOCKS_TAG_WIDTH; ++c)
                bad |= !(__bfloat162float(cur[c]) == __bfloat162float(old[c]));
        }
    }
    bad = __any_sync(0xffffffffu, bad);
    if (lane == 0) p.stale[i] = (p.valid[i] && bad) ? 1 : 0;
}

}  // namespace
}  // namespace locks

using namespace locks;

extern "C" int locks_rki4_build(
    const void* const* k_layers, int64_t k_stride_block, int64_t k_stride_tok,
    int64_t k_stride_head, void* records, void* tags, const int32_t* blocks,
    int n_blocks, int layer0, int n_layers, int num_blocks_state,
    int num_blocks_cache, int n_kv, int head_dim, int page,
    locks_stream_t stream) {
    LOCKS_REQUIRE(k_layers && records && tags && (blocks || n_blocks == 0),
                  LOCKS_ERR_ARG, "locks_rki4_build: null pointer argument");
    LOCKS_REQUIRE(head_dim == HD && page == PAGE_T, LOCKS_ERR_GEOMETRY,
                  "locks_rki4_build: supports head_dim 128 / page 16, got %d / %d",
                  head_dim, page);
    LOCKS_REQUIRE(n_blocks >= 0 && layer0 >= 0 && n_layers >= 0 &&
                      num_blocks_state >= 1 && num_blocks_cache >= 1 && n_kv >= 1,
                  LOCKS_ERR_ARG, "locks_rki4_build: bad size argument");
    LOCKS_REQUIRE(k_stride_block % 4 == 0 && k_stride_tok % 4 == 0 &&
                      k_stride_head % 4 == 0,
                  LOCKS_ERR_ARG,
                  "locks_rki4_build: K strides must be multiples of 4 elements");
    const int64_t n_jobs = (int64_t)n_layers * n_blocks * n_kv;
    if (n_jobs == 0) return LOCKS_OK;
    LOCKS_REQUIRE((n_jobs + BW - 1) / BW <= 2147483647LL, LOCKS_ERR_SIZE,
                  "locks_rki4_build: too many (layer, block, head) jobs");
    BuildParams p;
    p.k_layers = k_layers; p.sb = k_stride_block; p.st = k_stride_tok;
    p.sh = k_stride_head;
    p.records = static_cast<uint8_t*>(records);
    p.tags = static_cast<__nv_bfloat16*>(tags);
    p.blocks = blocks; p.n_blocks = n_blocks; p.layer0 = layer0;
    p.n_layers = n_layers; p.nb_state = num_blocks_state;
    p.nb_cache = num_blocks_cache; p.n_kv = n_kv;
    rki4_build_kernel<<<(unsigned)((n_jobs + BW - 1) / BW), BW * 32, 0,
                        static_cast<cudaStream_t>(stream)>>>(p);
    pdl_break();
    return check_launch("locks_rki4_build");
}

extern "C" int locks_rki4_tag_scan(
    const void* const* k_layers, int64_t k_stride_block, int64_t k_stride_tok,
    int64_t k_stride_head, const void* tags, const int32_t* blocks,
    const uint8_t* valid, uint8_t* stale, int n_blocks, int n_layers,
    int num_blocks_state, int n_kv, int page, locks_stream_t stream) {
    LOCKS_REQUIRE(k_layers && tags && valid && stale && (blocks || n_blocks == 0),
                  LOCKS_ERR_ARG, "locks_rki4_tag_scan: null pointer argument");
    LOCKS_REQUIRE(n_blocks >= 0 && n_layers >= 1 && num_blocks_state >= 1 &&
                      n_kv >= 1 && page >= 1,
                  LOCKS_ERR_ARG, "locks_rki4_tag_scan: bad size argument");
    if (n_blocks == 0) return LOCKS_OK;
    TagScanParams p;
    p.k_layers = k_layers; p.sb = k_stride_block; p.st = k_stride_tok;
    p.sh = k_stride_head;
    p.tags = static_cast<const __nv_bfloat16*>(tags);
    p.blocks = blocks; p.valid = valid; p.stale = stale;
    p.n_blocks = n_blocks; p.n_layers = n_layers; p.nb_state = num_blocks_state;
    p.n_kv = n_kv; p.page = page;
    tag_scan_kernel<<<(n_blocks + 3) / 4, 128, 0,
                      static_cast<cudaStream_t>(stream)>>>(p);
    return check_launch("locks_rki4_tag_scan");
}
