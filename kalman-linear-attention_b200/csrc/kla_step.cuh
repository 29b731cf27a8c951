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
    int vec;  // S % 4 == 0 and lam, eta, a, p, lam_out, eta_out 16-byte aligned: a lane's four states move as one vector
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
        const long long ms0 = (long long)m * S + j * 4, bms0 = ((long long)b * M + m) * S + j * 4;
        // One lane's four states as 16-byte vectors when the row length and the pointers allow it.
        // LPC is a power of two, so for S = 12, 20, 24, ... some lanes of a channel lie wholly past
        // the row (j * 4 >= S): they hold padding chains and touch no memory.
        const bool vec = prm.vec != 0, lane_live = j * 4 < S;
        float lamv[4], etav[4], av[4], pv[4], lo[4], eo[4];
        if (!lane_live) {
#pragma unroll
            for (int i = 0; i < 4; ++i) { lamv[i] = 1.0f; etav[i] = 0.0f; av[i] = 0.0f; pv[i] = 1.0f; }
        } else if (vec) {
            const float4 l4 = *reinterpret_cast<const float4 *>(prm.lam + bms0);
            const float4 e4 = *reinterpret_cast<const float4 *>(prm.eta + bms0);
            const float4 a4 = *reinterpret_cast<const float4 *>(prm.a + ms0);
            const float4 p4 = *reinterpret_cast<const float4 *>(prm.p + ms0);
            lamv[0] = l4.x; lamv[1] = l4.y; lamv[2] = l4.z; lamv[3] = l4.w;
            etav[0] = e4.x; etav[1] = e4.y; etav[2] = e4.z; etav[3] = e4.w;
            av[0] = a4.x; av[1] = a4.y; av[2] = a4.z; av[3] = a4.w;
            pv[0] = p4.x; pv[1] = p4.y; pv[2] = p4.z; pv[3] = p4.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const bool in = j * 4 + i < S;
                lamv[i] = in ? prm.lam[bms0 + i] : 1.0f;
                etav[i] = in ? prm.eta[bms0 + i] : 0.0f;
                av[i] = in ? prm.a[ms0 + i] : 0.0f;
                pv[i] = in ? prm.p[ms0 + i] : 1.0f;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int s = j * 4 + i;
            const bool in = s < S;
            const float kv = in ? to_f32<T>(kb[s]) : 0.0f, qv = in ? to_f32<T>(qb[s]) : 0.0f;
            const float a = av[i];
            const float p = fmaxf(pv[i], kPMin);                     // kla_ops.py:316
            const float a2 = fmaxf(a * a, kEps);                     // :317
            const float phi = fmaxf(lv * kv * kv, kEps);             // :310-312
            const float inv = 1.0f / fmaxf(a2 + p * lamv[i], kEps);  // :319
            const float lam = lamv[i] * inv + phi;                   // :320
            const float eta = (a * inv) * etav[i] + vl * kv;         // :321
            float var = 1.0f / fmaxf(lam, kEps);                     // :323
            float mean = eta * var;                                  // :324
            if (PRIOR) {                                             // :325-327
                mean = a * mean;
                var = a2 * var + p;
            }
            if (in) {
                ys = fmaf(mean, qv, ys);                             // :329
                yvs = fmaf(var, qv * qv, yvs);                       // :330
            }
            lo[i] = lam;
            eo[i] = eta;
        }
        if (!lane_live) {
            // padding lane: nothing to store
        } else if (vec) {
            *reinterpret_cast<float4 *>(prm.lam_out + bms0) = make_float4(lo[0], lo[1], lo[2], lo[3]);
            *reinterpret_cast<float4 *>(prm.eta_out + bms0) = make_float4(eo[0], eo[1], eo[2], eo[3]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (j * 4 + i < S) {
                    prm.lam_out[bms0 + i] = lo[i];
                    prm.eta_out[bms0 + i] = eo[i];
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
