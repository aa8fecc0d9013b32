// rki4 summary of ONE (block, kv-head) page, computed by one warp.  Shared by the
// summary builder (a warp per job) and by the KV-write kernel (the warp that
// stored a page's last token builds the page's summary in the same launch).
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
#pragma once
#include "common.cuh"
#include "jacobi16.cuh"

namespace locks {

constexpr int BUILD_PAGE_T = 16;
constexpr int BUILD_HD = 128;
constexpr int BUILD_DC_PITCH = BUILD_HD + 4;   // floats, keeps float4 rows conflict-free

struct BuildWarpScratch {
    float dc[BUILD_PAGE_T][BUILD_DC_PITCH];
    float A[BUILD_PAGE_T][BUILD_PAGE_T + 1];
    float U[BUILD_PAGE_T][BUILD_PAGE_T + 1];
    float rc[8], rs[8];
    float s8[8];
    int idx[8];
};

__device__ __forceinline__ float build_warp_max(float v) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// K: first token of the page for this head, tok_stride elements between tokens;
// rec: the 832-byte record; tag: LOCKS_TAG_WIDTH bf16.
__device__ __forceinline__ void rki4_build_one(BuildWarpScratch& ws,
                                               const __nv_bfloat16* K,
                                               int64_t tok_stride, uint8_t* rec,
                                               __nv_bfloat16* tag, int lane) {
    constexpr int PAGE_T = BUILD_PAGE_T, HD = BUILD_HD;
    // ---- load, centroid, centred keys ----------------------------------------
    float kv[PAGE_T][4];
    float mu[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int t = 0; t < PAGE_T; ++t) {
        const uint2 raw =
            *reinterpret_cast<const uint2*>(K + (int64_t)t * tok_stride + 4 * lane);
        kv[t][0] = bf16_bits_to_f32(raw.x & 0xFFFFu);
        kv[t][1] = bf16_bits_to_f32(raw.x >> 16);
        kv[t][2] = bf16_bits_to_f32(raw.y & 0xFFFFu);
        kv[t][3] = bf16_bits_to_f32(raw.y >> 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) mu[i] += kv[t][i];
        if (t == PAGE_T - 1 && lane < 2) {
            // content tag: first 8 channels of the page-final token, raw bf16
            *reinterpret_cast<uint2*>(tag + 4 * lane) = raw;
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
            amax = build_warp_max(amax);
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
        amax = build_warp_max(amax);
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

}  // namespace locks
