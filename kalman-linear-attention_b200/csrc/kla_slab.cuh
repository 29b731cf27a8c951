// Slab aggregates for the sequence-sharded scan.
//
// When the time axis is split into slabs held by different GPUs, each GPU
// first needs the state its slab starts from, and in the backward the adjoint
// carry its slab ends with. Both come from per-chain aggregates of whole slabs
// that compose associatively, so they can be all-gathered and folded:
//
// * forward (MODE 0). In homogeneous coordinates h = (x, w, z) with P = w/x and
//   mean = z/x one filter step is linear,
//       x' = (1 + p phi) x + a2 phi w,   w' = p x + a2 w,   z' = r w' + a z,
//   (the variance-form step of kla_common.cuh multiplied through by its
//   denominator), so a slab is the product of its step matrices:
//   7 numbers (m00 m01 / m10 m11 / m20 m21 m22), rescaled every other step --
//   a common factor does not change P or mean. This is the reference's
//   trace-normalised 2x2 Moebius product (src/kla/ops/kla_ops.py:76-116)
//   extended by the row that carries the mean, which lets one pass serve both
//   recurrences instead of two dependent ones.
//
// * adjoint (MODE 1). With the forward trajectory fixed, the backward carries
//   obey c_{t-1} = J_t (c_t + e_t), J_t = [[a2 g^2, a2 g (r - phi mean_t)],
//   [0, a g]], e_t = (dyvar q^2, dy q): affine, upper triangular. Walking the
//   slab FORWARD in time, K_t = J_1 ... J_t and b = sum_t K_t e_t give the carry
//   that leaves the slab as K c_in + b (5 numbers). It needs the slab's true
//   initial state, i.e. it runs after the forward fold.
//
// Plain kernel: one thread per (channel, SPT states), tiles of TT steps staged
// through shared memory by the whole CTA with a register prefetch of the next
// tile; no cross-thread sums, one 32-byte record per chain at the end.
#pragma once

#include "kla_common.cuh"

namespace kla {

struct SlabParams {
    int B, L, M, S;
    Tensor3 v, lv, k, q, dy, dyv;      // dy, dyv, q: adjoint mode only
    const float *a, *p, *lam0, *eta0;  // lam0/eta0: adjoint mode only (nullptr = unit prior)
    float *out;                        // [B, M, S, 8]
};

template <typename T, typename TO, int SPT, int LPC, bool ADJ, bool PRIOR>
__global__ void __launch_bounds__(128) kla_slab_aggregate_kernel(const SlabParams prm) {
    constexpr int NW = 4, TT = 16, CLS = 32 / LPC, MC = NW * CLS, SPAD = SPT * LPC, NTHR = 128;
    constexpr int NIN = ADJ ? 4 : 2;                        // staged [TT x MC] tiles
    constexpr int PER = (TT * MC + NTHR - 1) / NTHR;        // elements per thread per tile
    constexpr int KQP = (TT * SPAD + NTHR - 1) / NTHR;
    __shared__ float tile[NIN][TT * MC];
    __shared__ float2 kq[TT * SPAD];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int j = lane % LPC, cl = lane / LPC;
    const int b = blockIdx.y, m_cta = blockIdx.x * MC, cw = warp * CLS + cl;
    const int L = prm.L, M = prm.M, S = prm.S;
    const int m = m_cta + cw;

    const T *vb = static_cast<const T *>(prm.v.ptr) + (long long)b * prm.v.sb;
    const T *lb = static_cast<const T *>(prm.lv.ptr) + (long long)b * prm.lv.sb;
    const T *kb = static_cast<const T *>(prm.k.ptr) + (long long)b * prm.k.sb;
    const T *qb = ADJ ? static_cast<const T *>(prm.q.ptr) + (long long)b * prm.q.sb : nullptr;
    const TO *dyb = ADJ ? static_cast<const TO *>(prm.dy.ptr) + (long long)b * prm.dy.sb : nullptr;
    const TO *dyvb = (ADJ && prm.dyv.ptr) ? static_cast<const TO *>(prm.dyv.ptr) + (long long)b * prm.dyv.sb : nullptr;

    float ca[SPT], ca2[SPT], cp[SPT];
    float A[SPT][7];  // forward: m00 m01 m10 m11 m20 m21 m22; adjoint: K00 K01 K11 b0 b1 P mean
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
        const int s = i * LPC + j;
        const bool live = (m < M) && (s < S);
        const float av = live ? prm.a[(long long)m * S + s] : 0.0f;
        const float pv = live ? prm.p[(long long)m * S + s] : 1.0f;
        ca[i] = av;
        ca2[i] = live ? fmaxf(av * av, kEps) : 0.0f;
        cp[i] = fmaxf(pv, kPMin);
        if (ADJ) {
            float lam = 1.0f, eta = 0.0f;
            if (live && prm.lam0 != nullptr) {
                lam = prm.lam0[((long long)b * M + m) * S + s];
                eta = prm.eta0[((long long)b * M + m) * S + s];
            }
            const float P0 = 1.0f / fmaxf(lam, kLamMin);
            A[i][0] = 1.0f; A[i][1] = 0.0f; A[i][2] = 1.0f; A[i][3] = 0.0f; A[i][4] = 0.0f;
            A[i][5] = P0; A[i][6] = eta * P0;
        } else {
            A[i][0] = 1.0f; A[i][1] = 0.0f; A[i][2] = 0.0f; A[i][3] = 1.0f;
            A[i][4] = 0.0f; A[i][5] = 0.0f; A[i][6] = 1.0f;
        }
    }

    float pre[NIN][PER], prek[KQP], preq[KQP];
    auto prefetch = [&](int t0) {
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const int idx = tid + e * NTHR, row = idx / MC, c = idx % MC;
            const bool in = idx < TT * MC && t0 + row < L && m_cta + c < M;
            const long long t = t0 + row;
            pre[0][e] = in ? to_f32<T>(vb[t * prm.v.st + m_cta + c]) : 0.0f;
            pre[1][e] = in ? to_f32<T>(lb[t * prm.lv.st + m_cta + c]) : 0.0f;
            if (ADJ) {
                pre[2][e] = in ? to_f32<TO>(dyb[t * prm.dy.st + m_cta + c]) : 0.0f;
                pre[3][e] = (in && dyvb) ? to_f32<TO>(dyvb[t * prm.dyv.st + m_cta + c]) : 0.0f;
            }
        }
#pragma unroll
        for (int e = 0; e < KQP; ++e) {
            const int idx = tid + e * NTHR, row = idx / SPAD, s = idx % SPAD;
            const bool in = idx < TT * SPAD && s < S && t0 + row < L;
            prek[e] = in ? to_f32<T>(kb[(long long)(t0 + row) * prm.k.st + s]) : 0.0f;
            preq[e] = (ADJ && in) ? to_f32<T>(qb[(long long)(t0 + row) * prm.q.st + s]) : 0.0f;
        }
    };
    auto commit = [&]() {
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const int idx = tid + e * NTHR;
            if (idx < TT * MC) {
#pragma unroll
                for (int n = 0; n < NIN; ++n) tile[n][idx] = pre[n][e];
            }
        }
#pragma unroll
        for (int e = 0; e < KQP; ++e) {
            const int idx = tid + e * NTHR;
            if (idx < TT * SPAD) kq[idx] = make_float2(prek[e], preq[e]);
        }
    };

    const int NT = (L + TT - 1) / TT;
    prefetch(0);
    commit();
    __syncthreads();
    for (int tl = 0; tl < NT; ++tl) {
        const int t0 = tl * TT;
        if (tl + 1 < NT) prefetch(t0 + TT);
        const int n = min(TT, L - t0);
#pragma unroll 4
        for (int tt = 0; tt < n; ++tt) {
            const float vv = tile[0][tt * MC + cw], lv = tile[1][tt * MC + cw];
            const float dy = ADJ ? tile[2][tt * MC + cw] : 0.0f;
            const float dyv = ADJ ? tile[3][tt * MC + cw] : 0.0f;
#pragma unroll
            for (int i = 0; i < SPT; ++i) {
                const float2 c = kq[tt * SPAD + i * LPC + j];
                float phi, r;
                chain_inputs(lv, vv, c.x, phi, r);
                if (ADJ) {
                    float Pp;
                    const float g = rcp_approx(chain_denominator(A[i][5], phi, ca2[i], cp[i], Pp));
                    chain_update(A[i][5], A[i][6], Pp, g, r, ca[i]);  // P_t, mean_t
                    const float a2g = ca2[i] * g;
                    const float j00 = a2g * g, j01 = a2g * fmaf(-phi, A[i][6], r), j11 = ca[i] * g;
                    float e0 = dyv * c.y * c.y, e1 = dy * c.y;
                    if (PRIOR) { e0 *= ca2[i]; e1 *= ca[i]; }
                    const float K00 = A[i][0] * j00;
                    const float K01 = fmaf(A[i][0], j01, A[i][1] * j11);
                    const float K11 = A[i][2] * j11;
                    A[i][0] = K00; A[i][1] = K01; A[i][2] = K11;
                    A[i][3] = fmaf(K00, e0, fmaf(K01, e1, A[i][3]));
                    A[i][4] = fmaf(K11, e1, A[i][4]);
                } else {
                    const float c0 = fmaf(cp[i], phi, 1.0f), c1 = ca2[i] * phi;
                    const float n00 = fmaf(c1, A[i][2], c0 * A[i][0]), n01 = fmaf(c1, A[i][3], c0 * A[i][1]);
                    const float n10 = fmaf(ca2[i], A[i][2], cp[i] * A[i][0]), n11 = fmaf(ca2[i], A[i][3], cp[i] * A[i][1]);
                    A[i][4] = fmaf(r, n10, ca[i] * A[i][4]);
                    A[i][5] = fmaf(r, n11, ca[i] * A[i][5]);
                    A[i][6] = ca[i] * A[i][6];
                    A[i][0] = n00; A[i][1] = n01; A[i][2] = n10; A[i][3] = n11;
                    if (tt & 1) {  // rescale: a common factor leaves P = w/x and mean = z/x unchanged
                        const float sc = rcp_approx(n00 + n01);
#pragma unroll
                        for (int e = 0; e < 7; ++e) A[i][e] *= sc;
                    }
                }
            }
        }
        __syncthreads();
        if (tl + 1 < NT) commit();
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < SPT; ++i) {
        const int s = i * LPC + j;
        if (m < M && s < S) {
            float4 *o = reinterpret_cast<float4 *>(prm.out + (((long long)b * M + m) * S + s) * 8);
            o[0] = make_float4(A[i][0], A[i][1], A[i][2], A[i][3]);
            o[1] = make_float4(A[i][4], A[i][5], A[i][6], 0.0f);
        }
    }
}

// ---------------------------------------------------------------------------
// Folds over the chunks of one sequence held on ONE GPU (time-parallel scan).
//
// The time axis of a [B, L, ...] problem is cut into C chunks that are scanned
// as B*C independent batch entries (entry b*C + c = chunk c of batch element b),
// which fills the GPU when B*M alone does not. Each chunk needs the state it
// starts from (forward) and the carry it ends with (backward); both follow from
// the per-chunk aggregates above by a short serial fold over c, done here with
// one thread per (b, m, s) lane in float64.
//
//   forward  in:  agg [B*C, M, S, 8] (MODE 0 records), lam0/eta0 [B, M, S] or nullptr
//            out: lam_in, eta_in [B*C, M, S], the state before each chunk's first step
//   adjoint  in:  agg [B*C, M, S, 8] (MODE 1 records), dlam_fin/deta_fin [B, M, S] or nullptr
//            out: dlam_seed, deta_seed [B*C, M, S]: passed to the backward kernel as the gradient
//                 of each chunk's returned state, they make it start from the right carry
struct ChunkFoldParams {
    int B, C, M, S;
    const float *agg;
    const float *in_a, *in_b;
    float *out_a, *out_b;
};

template <bool ADJ>
__global__ void __launch_bounds__(128) kla_chunk_fold_kernel(const ChunkFoldParams prm) {
    const long long lanes = (long long)prm.M * prm.S;
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (long long)prm.B * lanes) return;
    const long long b = gid / lanes, ms = gid % lanes;
    const int C = prm.C;
    auto rec = [&](int c, double (&A)[7]) {
        const float4 *src = reinterpret_cast<const float4 *>(prm.agg + (((b * C + c) * lanes) + ms) * 8);
        const float4 lo = src[0], hi = src[1];
        A[0] = lo.x; A[1] = lo.y; A[2] = lo.z; A[3] = lo.w; A[4] = hi.x; A[5] = hi.y; A[6] = hi.z;
    };
    double A[7];
    if (!ADJ) {
        double P = 1.0, mean = 0.0;
        if (prm.in_a != nullptr) {
            P = 1.0 / fmax((double)prm.in_a[gid], (double)kLamMin);
            mean = (double)prm.in_b[gid] * P;
        }
        for (int c = 0; c < C; ++c) {
            const long long o = (b * C + c) * lanes + ms;
            const double lam = 1.0 / P;
            prm.out_a[o] = (float)lam;
            prm.out_b[o] = (float)(mean * lam);
            if (c + 1 < C) {
                rec(c, A);
                const double x = A[0] + A[1] * P, w = A[2] + A[3] * P, z = A[4] + A[5] * P + A[6] * mean;
                P = w / x;
                mean = z / x;
            }
        }
    } else {
        rec(C - 1, A);
        const double dl = prm.in_a ? (double)prm.in_a[gid] : 0.0, de = prm.in_b ? (double)prm.in_b[gid] : 0.0;
        // (dL/dP, dL/dmean) at the end of the sequence from the gradient of (lam, eta) = (1/P, mean/P)
        const double lam = 1.0 / A[5], eta = A[6] * lam;
        double cP = -lam * (lam * dl + eta * de), cm = de * lam;
        for (int c = C - 1; c >= 0; --c) {
            if (c != C - 1) rec(c, A);
            const long long o = (b * C + c) * lanes + ms;
            const double P_end = A[5], mean_end = A[6];
            const double deta = cm * P_end;
            prm.out_b[o] = (float)deta;
            prm.out_a[o] = (float)(-(cP * P_end * P_end + mean_end * deta));
            const double nP = A[0] * cP + A[1] * cm + A[3];
            cm = A[2] * cm + A[4];
            cP = nP;
        }
    }
}

}  // namespace kla
