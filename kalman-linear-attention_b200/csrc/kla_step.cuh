// Single-token decode step: one filter update of every (b, m, s) lane plus the
// read-out, in the reference's information form and with its floors
// (src/kla/ops/kla_ops.py:293-331). State-bound: per lane it reads lam, eta,
// a, p and writes lam, eta (24 B) for ~15 flops.
//
// One thread per (b, m, group of 4 consecutive states); the LPC threads of a
// channel are adjacent lanes, so state rows are read as 16-byte vectors and the
// read-out sum over s is log2(LPC) shuffle rounds.
#pragma once

#include "kla_common.cuh"

namespace kla {

struct StepParams {
    int B, M, S;
    const void *v, *lv, *k, *q;
    long long v_sb, lv_sb, k_sb, q_sb;
    const float *a, *p, *lam, *eta;
    void *y, *yv;
    float *lam_out, *eta_out;
};

template <typename T, typename TO, int LPC, bool PRIOR>
__global__ void __launch_bounds__(128) kla_step_kernel(const StepParams prm) {
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long bm = gid / LPC;
    const int j = (int)(gid % LPC);
    const int M = prm.M, S = prm.S;
    const bool row_live = bm < (long long)prm.B * M;  // whole lane groups are live or not
    const int b = row_live ? (int)(bm / M) : 0, m = row_live ? (int)(bm % M) : 0;

    float ys = 0.0f, yvs = 0.0f;
    if (row_live) {
        const float lv = to_f32<T>(static_cast<const T *>(prm.lv)[(long long)b * prm.lv_sb + m]);
        const float vl = to_f32<T>(static_cast<const T *>(prm.v)[(long long)b * prm.v_sb + m]) * lv;
        const T *kb = static_cast<const T *>(prm.k) + (long long)b * prm.k_sb;
        const T *qb = static_cast<const T *>(prm.q) + (long long)b * prm.q_sb;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int s = j * 4 + i;
            if (s < S) {
                const long long ms = (long long)m * S + s, bms = ((long long)b * M + m) * S + s;
                const float kv = to_f32<T>(kb[s]), qv = to_f32<T>(qb[s]);
                const float a = prm.a[ms];
                const float p = fmaxf(prm.p[ms], kPMin);                 // kla_ops.py:316
                const float a2 = fmaxf(a * a, kEps);                     // :317
                const float phi = fmaxf(lv * kv * kv, kEps);             // :310-312
                const float lam_prev = prm.lam[bms], eta_prev = prm.eta[bms];
                const float inv = 1.0f / fmaxf(a2 + p * lam_prev, kEps); // :319
                const float lam = lam_prev * inv + phi;                  // :320
                const float eta = (a * inv) * eta_prev + vl * kv;        // :321
                float var = 1.0f / fmaxf(lam, kEps);                     // :323
                float mean = eta * var;                                  // :324
                if (PRIOR) {                                             // :325-327
                    mean = a * mean;
                    var = a2 * var + p;
                }
                ys = fmaf(mean, qv, ys);                                 // :329
                yvs = fmaf(var, qv * qv, yvs);                           // :330
                prm.lam_out[bms] = lam;
                prm.eta_out[bms] = eta;
            }
        }
    }
#pragma unroll
    for (int off = LPC / 2; off > 0; off >>= 1) {
        ys += __shfl_xor_sync(0xffffffffu, ys, off);
        yvs += __shfl_xor_sync(0xffffffffu, yvs, off);
    }
    if (row_live && j == 0) {
        static_cast<TO *>(prm.y)[(long long)b * M + m] = from_f32<TO>(ys);
        static_cast<TO *>(prm.yv)[(long long)b * M + m] = from_f32<TO>(yvs);
    }
}

}  // namespace kla
