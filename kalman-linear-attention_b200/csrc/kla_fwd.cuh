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
    int vec_v, vec_lv, vec_y, vec_yv;
};

template <int SPT, int LPC, int CH, int NW, int TT>
struct ScanShape {
    static constexpr int kSPad = SPT * LPC;
    static constexpr int kCLS = 32 / LPC;         // channel groups per warp
    static constexpr int kCPW = kCLS * CH;        // channels per warp
    static constexpr int kMC = NW * kCPW;         // channels per CTA
    static constexpr int kThreads = NW * 32;
    static constexpr int kKqPer = (TT * kSPad + kThreads - 1) / kThreads;
    // Row length of the [TT][LPC][MCP] float2 partial-sum buffers. 8-byte
    // shared-memory accesses are served half a warp at a time; a half-warp
    // writes LPC rows of kCPW/2 channels each, so rows are offset by kCPW/2
    // channels modulo the 16 channels (32 banks) a wavefront covers.
    static constexpr int kHalf = kCPW / 2 > 0 ? kCPW / 2 : 1;
    static constexpr int kPadRaw = ((kHalf - kMC) % 16 + 16) % 16;
    static constexpr int kMCP = kMC + kPadRaw + (kPadRaw & 1);
    static_assert(kMC % 2 == 0, "the output pass works on pairs of channels");
};

// Sum the per-lane-group partials of one tile over the LPC lane groups and
// write two [rows x MC] output tiles. part: [TT][LPC][MCP] float2 in shared
// memory. Each thread handles pairs of channels, so consecutive lanes read
// consecutive 16-byte words. FIN maps (sum.x, sum.y, tt, channel) to the two
// output values. vec0/vec1: 2-element vector stores are legal for that output.
template <typename TO, int LPC, int MC, int MCP, int TT, int NTHR, typename Fin>
__device__ __forceinline__ void output_pass(const float2 *part, TO *o0, long long st0, int vec0, TO *o1,
                                            long long st1, int vec1, int nrows, int m0, int M, int tid, Fin fin) {
#pragma unroll
    for (int u0 = 0; u0 < TT * (MC / 2); u0 += NTHR) {
        const int u = u0 + tid;
        const int tt = u / (MC / 2), c = (u % (MC / 2)) * 2;
        if (u >= TT * (MC / 2) || tt >= nrows || m0 + c >= M) continue;
        float ax = 0.0f, ay = 0.0f, bx = 0.0f, by = 0.0f;
#pragma unroll
        for (int jj = 0; jj < LPC; ++jj) {
            const float4 x = *reinterpret_cast<const float4 *>(part + (tt * LPC + jj) * MCP + c);
            ax += x.x; ay += x.y; bx += x.z; by += x.w;
        }
        float r0[2], r1[2];
        fin(make_float2(ax, ay), tt, c, r0[0], r1[0]);
        fin(make_float2(bx, by), tt, c + 1, r0[1], r1[1]);
        TO *p0 = o0 + (long long)tt * st0 + m0 + c;
        TO *p1 = o1 + (long long)tt * st1 + m0 + c;
        const bool full = m0 + c + 1 < M;
        if (full && vec0) {
            if constexpr (sizeof(TO) == 4) {
                *reinterpret_cast<float2 *>(p0) = make_float2(r0[0], r0[1]);
            } else {
                *reinterpret_cast<__nv_bfloat162 *>(p0) = __floats2bfloat162_rn(r0[0], r0[1]);
            }
        } else {
            p0[0] = from_f32<TO>(r0[0]);
            if (full) p0[1] = from_f32<TO>(r0[1]);
        }
        if (full && vec1) {
            if constexpr (sizeof(TO) == 4) {
                *reinterpret_cast<float2 *>(p1) = make_float2(r1[0], r1[1]);
            } else {
                *reinterpret_cast<__nv_bfloat162 *>(p1) = __floats2bfloat162_rn(r1[0], r1[1]);
            }
        } else {
            p1[0] = from_f32<TO>(r1[0]);
            if (full) p1[1] = from_f32<TO>(r1[1]);
        }
    }
}

template <typename T, typename TO, int SPT, int LPC, int CH, int NW, int TT, bool PRIOR>
__global__ void __launch_bounds__(NW * 32) kla_fwd_kernel(const FwdParams prm) {
    using Sh = ScanShape<SPT, LPC, CH, NW, TT>;
    constexpr int SPAD = Sh::kSPad, MC = Sh::kMC, MCP = Sh::kMCP, NTHR = Sh::kThreads, KQ = Sh::kKqPer;
    static_assert(TT == kCkptInterval, "one checkpoint per tile");

    extern __shared__ __align__(16) unsigned char smem_raw[];
    float4 *kq4 = reinterpret_cast<float4 *>(smem_raw);                 // [2][TT][SPAD]
    float2 *ypart = reinterpret_cast<float2 *>(kq4 + 2 * TT * SPAD);    // [2][TT][LPC][MCP]
    T *vbuf = reinterpret_cast<T *>(ypart + 2 * TT * LPC * MCP);        // [2][TT][MC]
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

    // One time step for every chain of this thread; the per-thread share of the
    // read-out goes to shared memory and is summed over lane groups per tile.
    auto step = [&](const T *lrow, const T *vrow, const float4 *kqrow, float2 *yrow, int tt) {
        float lv[CH], vl[CH], ys[CH], yvs[CH];
#pragma unroll
        for (int ci = 0; ci < CH; ++ci) {
            lv[ci] = to_f32<T>(lrow[tt * MC + ci]);
            vl[ci] = to_f32<T>(vrow[tt * MC + ci]) * lv[ci];
            ys[ci] = 0.0f;
            yvs[ci] = 0.0f;
        }
#pragma unroll
        for (int i = 0; i < SPT; ++i) {
            const float4 c = kqrow[tt * SPAD + i * LPC];  // k^2, k, q, q^2
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
        for (int ci = 0; ci < CH; ++ci) yrow[tt * LPC * MCP + ci] = make_float2(ys[ci], yvs[ci]);
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
        const T *lrow = lbuf + cur * TT * MC + cw;
        const T *vrow = vbuf + cur * TT * MC + cw;
        const float4 *kqrow = kq4 + cur * TT * SPAD + j;
        float2 *yrow = ypart + cur * TT * LPC * MCP + j * MCP + cw;
        if (t0 + TT <= L) {
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) step(lrow, vrow, kqrow, yrow, tt);
        } else {
            for (int tt = 0; t0 + tt < L; ++tt) step(lrow, vrow, kqrow, yrow, tt);
        }
        if (more) store_kq(nxt);
        cp_async_wait_all();
        __syncthreads();
        output_pass<TO, LPC, MC, MCP, TT, NTHR>(
            ypart + cur * TT * LPC * MCP, yb + (long long)t0 * prm.y.st, prm.y.st, prm.vec_y,
            yvb + (long long)t0 * prm.yv.st, prm.yv.st, prm.vec_yv, min(TT, L - t0), m_cta, M, tid,
            [](float2 acc, int, int, float &o0, float &o1) { o0 = acc.x; o1 = acc.y; });
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
