// Fused forward scan kernel: lambda_v, v, k, q -> y, y_var, final state, and
// (for training) a checkpoint of every chain's state once per tile.
//
// Nothing of shape [B, L, M, S] is ever written: phi, r, the gain, the
// posterior and the read-out all live in registers. Per token the kernel reads
// v, lambda_v (2M) and k, q (2S, once per CTA of MC channels) and writes y,
// y_var (2M).
#pragma once

#include "kla_common.cuh"

namespace kla {

struct FwdParams {
    int B, L, M, S, NT;
    Tensor3 v, lv, k, q, y, yv;
    const float *a, *p, *lam0, *eta0;
    float *lam_fin, *eta_fin;
    float2 *ckpt;  // [B, NT, M, S] (P, mean) at the start of each tile, or nullptr
    int vec_v, vec_lv;
};

template <int SPT, int LPC, int CH, int NW, int TT>
struct ScanShape {
    static constexpr int kSPad = SPT * LPC;
    static constexpr int kCPW = (32 / LPC) * CH;  // channels per warp
    static constexpr int kMC = NW * kCPW;         // channels per CTA
    static constexpr int kThreads = NW * 32;
    static constexpr int kKqPer = (TT * kSPad + kThreads - 1) / kThreads;
};

template <typename T, typename TO, int SPT, int LPC, int CH, int NW, int TT, bool PRIOR>
__global__ void __launch_bounds__(NW * 32) kla_fwd_kernel(const FwdParams prm) {
    using Sh = ScanShape<SPT, LPC, CH, NW, TT>;
    constexpr int SPAD = Sh::kSPad, MC = Sh::kMC, NTHR = Sh::kThreads, KQ = Sh::kKqPer;
    static_assert(TT == kCkptInterval, "one checkpoint per tile");

    extern __shared__ __align__(16) unsigned char smem_raw[];
    float4 *kq4 = reinterpret_cast<float4 *>(smem_raw);                 // [2][TT][SPAD]
    T *vbuf = reinterpret_cast<T *>(kq4 + 2 * TT * SPAD);               // [2][TT][MC]
    T *lbuf = vbuf + 2 * TT * MC;                                       // [2][TT][MC]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int j = lane % LPC, cl = lane / LPC;
    const int b = blockIdx.y;
    const int m_cta = blockIdx.x * MC;
    const int cw = warp * Sh::kCPW + cl * CH;  // first channel of this thread, CTA-relative
    const int L = prm.L, M = prm.M, S = prm.S;

    const T *vb = static_cast<const T *>(prm.v.ptr) + (long long)b * prm.v.sb;
    const T *lb = static_cast<const T *>(prm.lv.ptr) + (long long)b * prm.lv.sb;
    const T *kb = static_cast<const T *>(prm.k.ptr) + (long long)b * prm.k.sb;
    const T *qb = static_cast<const T *>(prm.q.ptr) + (long long)b * prm.q.sb;
    TO *yb = static_cast<TO *>(prm.y.ptr) + (long long)b * prm.y.sb;
    TO *yvb = static_cast<TO *>(prm.yv.ptr) + (long long)b * prm.yv.sb;

    // Per-chain constants and state. Padding chains (s >= S or m >= M) get
    // a = 0, p = 1, so their variance sits at 1 and their mean at 0.
    float ca[CH][SPT], ca2[CH][SPT], cp[CH][SPT], P[CH][SPT], mean[CH][SPT];
#pragma unroll
    for (int ci = 0; ci < CH; ++ci) {
        const int m = m_cta + cw + ci;
#pragma unroll
        for (int i = 0; i < SPT; ++i) {
            const int s = i * LPC + j;
            const bool live = (m < M) && (s < S);
            const float av = live ? prm.a[(long long)m * S + s] : 0.0f;
            const float pv = live ? prm.p[(long long)m * S + s] : 1.0f;
            ca[ci][i] = av;
            ca2[ci][i] = live ? fmaxf(av * av, kEps) : 0.0f;
            cp[ci][i] = fmaxf(pv, kPMin);
            float lam = 1.0f, eta = 0.0f;
            if (live && prm.lam0 != nullptr) {
                lam = prm.lam0[((long long)b * M + m) * S + s];
                eta = prm.eta0[((long long)b * M + m) * S + s];
            }
            const float P0 = 1.0f / fmaxf(lam, kLamMin);
            P[ci][i] = P0;
            mean[ci][i] = eta * P0;
        }
    }

    float kreg[KQ], qreg[KQ];
    auto load_kq = [&](int t0) {
#pragma unroll
        for (int e = 0; e < KQ; ++e) {
            const int idx = tid + e * NTHR;
            const int row = idx / SPAD, s = idx % SPAD;
            float kv = 0.0f, qv = 0.0f;
            if (idx < TT * SPAD && s < S && t0 + row < L) {
                kv = to_f32<T>(kb[(long long)(t0 + row) * prm.k.st + s]);
                qv = to_f32<T>(qb[(long long)(t0 + row) * prm.q.st + s]);
            }
            kreg[e] = kv;
            qreg[e] = qv;
        }
    };
    auto store_kq = [&](int buf) {
#pragma unroll
        for (int e = 0; e < KQ; ++e) {
            const int idx = tid + e * NTHR;
            if (idx < TT * SPAD)
                kq4[buf * TT * SPAD + idx] = make_float4(kreg[e] * kreg[e], kreg[e], qreg[e], qreg[e] * qreg[e]);
        }
    };

    // One time step for every chain of this thread, then the read-out.
    auto step = [&](int buf, int tt, int t) {
        float lv[CH], vl[CH], ys[CH], yvs[CH];
#pragma unroll
        for (int ci = 0; ci < CH; ++ci) {
            lv[ci] = to_f32<T>(lbuf[(buf * TT + tt) * MC + cw + ci]);
            vl[ci] = to_f32<T>(vbuf[(buf * TT + tt) * MC + cw + ci]) * lv[ci];
            ys[ci] = 0.0f;
            yvs[ci] = 0.0f;
        }
#pragma unroll
        for (int i = 0; i < SPT; ++i) {
            const float4 c = kq4[(buf * TT + tt) * SPAD + i * LPC + j];  // k^2, k, q, q^2
#pragma unroll
            for (int ci = 0; ci < CH; ++ci) {
                const float phi = __fmul_rn(lv[ci], c.x);
                const float r = __fmul_rn(vl[ci], c.y);
                chain_step(P[ci][i], mean[ci][i], phi, r, ca[ci][i], ca2[ci][i], cp[ci][i]);
                if (PRIOR) {  // read out the one-step-ahead prior, kla_ops.py:284-286
                    ys[ci] = fmaf(c.z, ca[ci][i] * mean[ci][i], ys[ci]);
                    yvs[ci] = fmaf(c.w, fmaf(ca2[ci][i], P[ci][i], cp[ci][i]), yvs[ci]);
                } else {
                    ys[ci] = fmaf(c.z, mean[ci][i], ys[ci]);
                    yvs[ci] = fmaf(c.w, P[ci][i], yvs[ci]);
                }
            }
        }
#pragma unroll
        for (int ci = 0; ci < CH; ++ci) {
#pragma unroll
            for (int off = LPC / 2; off > 0; off >>= 1) {
                ys[ci] += __shfl_xor_sync(0xffffffffu, ys[ci], off);
                yvs[ci] += __shfl_xor_sync(0xffffffffu, yvs[ci], off);
            }
            const int m = m_cta + cw + ci;
            if (j == 0 && m < M) {
                yb[(long long)t * prm.y.st + m] = from_f32<TO>(ys[ci]);
                yvb[(long long)t * prm.yv.st + m] = from_f32<TO>(yvs[ci]);
            }
        }
    };

    // prologue: tile 0
    stage_tile<T, TT, MC, NTHR>(vbuf, vb, prm.v.st, 0, L, m_cta, M, prm.vec_v, tid);
    stage_tile<T, TT, MC, NTHR>(lbuf, lb, prm.lv.st, 0, L, m_cta, M, prm.vec_lv, tid);
    load_kq(0);
    store_kq(0);
    cp_async_wait_all();
    __syncthreads();

    for (int tile = 0; tile < prm.NT; ++tile) {
        const int cur = tile & 1, nxt = cur ^ 1;
        const int t0 = tile * TT;
        const bool more = tile + 1 < prm.NT;
        if (more) {
            stage_tile<T, TT, MC, NTHR>(vbuf + nxt * TT * MC, vb, prm.v.st, t0 + TT, L, m_cta, M, prm.vec_v, tid);
            stage_tile<T, TT, MC, NTHR>(lbuf + nxt * TT * MC, lb, prm.lv.st, t0 + TT, L, m_cta, M, prm.vec_lv, tid);
            load_kq(t0 + TT);
        }
        if (prm.ckpt != nullptr) {
#pragma unroll
            for (int ci = 0; ci < CH; ++ci) {
                const int m = m_cta + cw + ci;
#pragma unroll
                for (int i = 0; i < SPT; ++i) {
                    const int s = i * LPC + j;
                    if (m < M && s < S)
                        prm.ckpt[(((long long)b * prm.NT + tile) * M + m) * S + s] = make_float2(P[ci][i], mean[ci][i]);
                }
            }
        }
        if (t0 + TT <= L) {
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) step(cur, tt, t0 + tt);
        } else {
            for (int tt = 0; t0 + tt < L; ++tt) step(cur, tt, t0 + tt);
        }
        if (more) store_kq(nxt);
        cp_async_wait_all();
        __syncthreads();
    }

    // final state back in information form: lambda = 1/P, eta = mean * lambda
#pragma unroll
    for (int ci = 0; ci < CH; ++ci) {
        const int m = m_cta + cw + ci;
#pragma unroll
        for (int i = 0; i < SPT; ++i) {
            const int s = i * LPC + j;
            if (m < M && s < S) {
                const float lam = 1.0f / P[ci][i];
                prm.lam_fin[((long long)b * M + m) * S + s] = lam;
                prm.eta_fin[((long long)b * M + m) * S + s] = mean[ci][i] * lam;
            }
        }
    }
}

}  // namespace kla
