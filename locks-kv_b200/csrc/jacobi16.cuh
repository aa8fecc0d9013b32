// Warp-cooperative eigen-decomposition of a symmetric 16 x 16 matrix held in
// shared memory: two-sided parallel-order Jacobi.  Each sweep is 15 rounds of 8
// disjoint rotations (round-robin pairing); the angles of a round are computed
// by 8 lanes, the row, column and eigenvector updates by all 32.  Sweeps stop
// when one rotates nothing (rotations below the fp32 noise of the matrix are
// skipped), or after MAX_SWEEPS.
//
// On return A holds the eigenvalues on its diagonal (unsorted) and U the
// eigenvectors in its columns (A_in = U diag U^T).  The caller must have U set
// to the identity and A symmetric, and must __syncwarp() before the call.
#pragma once

namespace locks {

constexpr int JACOBI_MAX_SWEEPS = 14;

__device__ __forceinline__ void jacobi16_warp(float (*A)[17], float (*U)[17],
                                              float* rc, float* rs, int lane) {
    float trace = (lane < 16) ? A[lane][lane] : 0.f;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1)
        trace += __shfl_xor_sync(0xffffffffu, trace, o);
    const float floor_abs = 1e-9f * fabsf(trace);   // below fp32 noise of A
    for (int sweep = 0; sweep < JACOBI_MAX_SWEEPS; ++sweep) {
        bool rotated = false;
        for (int rd = 0; rd < 15; ++rd) {
            // pair k of this round
            int pk, qk;
            {
                const int k = lane & 7;
                const int a = (rd + k) % 15;
                const int b = (k == 0) ? 15 : (rd + 15 - k) % 15;
                pk = min(a, b); qk = max(a, b);
            }
            if (lane < 8) {
                const float app = A[pk][pk], aqq = A[qk][qk], apq = A[pk][qk];
                float c = 1.f, s = 0.f;
                if (fabsf(apq) > floor_abs &&
                    fabsf(apq) > 1e-7f * sqrtf(fabsf(app * aqq))) {
                    const float theta = __fdiv_rn(aqq - app, 2.f * apq);
                    const float t = __fdiv_rn(
                        copysignf(1.f, theta),
                        fabsf(theta) + sqrtf(fmaf(theta, theta, 1.f)));
                    c = __fdiv_rn(1.f, sqrtf(fmaf(t, t, 1.f)));
                    s = t * c;
                    rotated = true;
                }
                rc[lane] = c; rs[lane] = s;
            }
            __syncwarp();
            // rows:  A <- J^T A   (pair k, columns 4*(lane/8) .. +3)
            {
                const int k = lane & 7, jb = (lane >> 3) * 4;
                const float c = rc[k], s = rs[k];
#pragma unroll
                for (int j = jb; j < jb + 4; ++j) {
                    const float x = A[pk][j], y = A[qk][j];
                    A[pk][j] = c * x - s * y;
                    A[qk][j] = s * x + c * y;
                }
            }
            __syncwarp();
            // columns:  A <- A J,  U <- U J   (pair k, rows 4*(lane/8) .. +3)
            {
                const int k = lane & 7, ib = (lane >> 3) * 4;
                const float c = rc[k], s = rs[k];
#pragma unroll
                for (int i = ib; i < ib + 4; ++i) {
                    const float x = A[i][pk], y = A[i][qk];
                    A[i][pk] = c * x - s * y;
                    A[i][qk] = s * x + c * y;
                    const float u = U[i][pk], v = U[i][qk];
                    U[i][pk] = c * u - s * v;
                    U[i][qk] = s * u + c * v;
                }
            }
            __syncwarp();
        }
        if (!__any_sync(0xffffffffu, rotated)) break;
    }
}

}  // namespace locks
