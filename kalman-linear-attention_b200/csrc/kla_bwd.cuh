// Fused backward scan kernel: the exact adjoint of kla_fwd_kernel.
//
// Time is walked in tiles, last tile first. For each tile the kernel replays
// the forward recurrence from the tile's checkpoint, keeping every chain's
// pre-step state (P', mean') in shared memory, then walks the adjoint back down
// the tile with the two carries (dL/dP, dL/dmean) in registers. The same
// statements differentiated by hand (variance form, see kla_common.cuh):
//
//   mean = g u,  u = a mean' + Pp r,  P = Pp g,  g = 1/d,  d = 1 + phi Pp,
//   Pp = a2 P' + p
//
//   mbar = c_mean + dy q            Pbar = c_P + dyvar q^2
//   dbar = -g (mbar mean + Pbar P)  ubar = mbar g
//   Ppbar = ubar r + Pbar g + dbar phi
//   rbar = ubar Pp                  phibar = dbar Pp
//   c_mean <- ubar a                c_P <- Ppbar a2
//   da += ubar mean'   da2 += Ppbar P'   dp += Ppbar
//
// Sums over s (dv, dlambda_v) finish with shuffles inside a channel's lane
// group. Sums over m (dk, dq) are formed per thread, parked in the shared-
// memory slot the replay just vacated, reduced over the CTA's channels after
// the tile, and added to global memory with one atomic per (t, s) per CTA.
// Sums over b and t (da, dp) stay in registers until the end.
#pragma once

#include "kla_fwd.cuh"

namespace kla {

struct BwdParams {
    int B, L, M, S, NT;
    Tensor3 v, lv, k, q, dy, dyv, dv, dlv;
    const float *a, *p, *lam0, *eta0;
    const float2 *ckpt;
    const float *dlam_fin, *deta_fin;
    float *dk, *dq, *da, *dp, *dlam0, *deta0;
    int vec_v, vec_lv, vec_dy, vec_dyv, vec_dv, vec_dlv;
};

template <typename T, typename TO, int SPT, int LPC, int CH, int NW, int TT, bool PRIOR>
__global__ void __launch_bounds__(NW * 32) kla_bwd_kernel(const BwdParams prm) {
    using Sh = ScanShape<SPT, LPC, CH, NW, TT>;
    constexpr int SPAD = Sh::kSPad, MC = Sh::kMC, MCP = Sh::kMCP, NTHR = Sh::kThreads, KQ = Sh::kKqPer;
    constexpr int CLS = Sh::kCLS;  // channel groups per warp
    static_assert(TT == kCkptInterval, "one checkpoint per tile");

    extern __shared__ __align__(16) unsigned char smem_raw[];
    float4 *kq4 = reinterpret_cast<float4 *>(smem_raw);                        // [2][TT][SPAD]
    float2 *traj = reinterpret_cast<float2 *>(kq4 + 2 * TT * SPAD);            // [TT*CH*SPT][NTHR]
    float2 *dpart = traj + TT * CH * SPT * NTHR;                               // [TT][LPC][MCP]
    T *vbuf = reinterpret_cast<T *>(dpart + TT * LPC * MCP);                   // [2][TT][MC] each
    T *lbuf = vbuf + 2 * TT * MC;
    TO *dybuf = reinterpret_cast<TO *>(lbuf + 2 * TT * MC);
    TO *dyvbuf = dybuf + 2 * TT * MC;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int j = lane % LPC, cl = lane / LPC;
    const int b = blockIdx.y;
    const int m_cta = blockIdx.x * MC;
    const int cw = warp * Sh::kCPW + cl * CH;
    const int L = prm.L, M = prm.M, S = prm.S, NT = prm.NT;
    const bool has_dyv = prm.dyv.ptr != nullptr;

    const T *vb = static_cast<const T *>(prm.v.ptr) + (long long)b * prm.v.sb;
    const T *lb = static_cast<const T *>(prm.lv.ptr) + (long long)b * prm.lv.sb;
    const T *kb = static_cast<const T *>(prm.k.ptr) + (long long)b * prm.k.sb;
    const T *qb = static_cast<const T *>(prm.q.ptr) + (long long)b * prm.q.sb;
    const TO *dyb = static_cast<const TO *>(prm.dy.ptr) + (long long)b * prm.dy.sb;
    const TO *dyvb = has_dyv ? static_cast<const TO *>(prm.dyv.ptr) + (long long)b * prm.dyv.sb : nullptr;
    T *dvb = static_cast<T *>(prm.dv.ptr) + (long long)b * prm.dv.sb;
    T *dlvb = static_cast<T *>(prm.dlv.ptr) + (long long)b * prm.dlv.sb;

    // Slot of (step tt, channel ci, state i) for this thread inside traj. Rows
    // are rotated inside each warp's 32 slots so that the reduction over
    // channels below reads shared memory without bank conflicts.
    auto slot = [&](int tt, int ci, int i, int w, int ln) {
        const int rot = LPC * ((tt * SPT + i) % CLS);
        return ((tt * CH + ci) * SPT + i) * NTHR + w * 32 + ((ln + rot) & 31);
    };

    float ca[CH][SPT], ca2[CH][SPT], cp[CH][SPT];
    float cP[CH][SPT], cm[CH][SPT], accA[CH][SPT], accA2[CH][SPT], accP[CH][SPT];
    float Pn[CH][SPT], mn[CH][SPT];
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
            cP[ci][i] = cm[ci][i] = accA[ci][i] = accA2[ci][i] = accP[ci][i] = 0.0f;
            Pn[ci][i] = 1.0f;
            mn[ci][i] = 0.0f;
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
    auto stage_all = [&](int buf, int t0) {
        stage_tile<T, TT, MC, NTHR>(vbuf + buf * TT * MC, vb, prm.v.st, t0, L, m_cta, M, prm.vec_v, tid);
        stage_tile<T, TT, MC, NTHR>(lbuf + buf * TT * MC, lb, prm.lv.st, t0, L, m_cta, M, prm.vec_lv, tid);
        stage_tile<TO, TT, MC, NTHR>(dybuf + buf * TT * MC, dyb, prm.dy.st, t0, L, m_cta, M, prm.vec_dy, tid);
        if (has_dyv)
            stage_tile<TO, TT, MC, NTHR>(dyvbuf + buf * TT * MC, dyvb, prm.dyv.st, t0, L, m_cta, M, prm.vec_dyv, tid);
    };
    float2 ck[CH][SPT];
    auto load_ck = [&](int tile) {
#pragma unroll
        for (int ci = 0; ci < CH; ++ci) {
            const int m = m_cta + cw + ci;
#pragma unroll
            for (int i = 0; i < SPT; ++i) {
                const int s = i * LPC + j;
                ck[ci][i] = (m < M && s < S) ? prm.ckpt[(((long long)b * NT + tile) * M + m) * S + s]
                                             : make_float2(1.0f, 0.0f);
            }
        }
    };

    if (!has_dyv) {  // dyvar absent: the tile stays zero for the whole kernel
        for (int idx = tid; idx < 2 * TT * MC; idx += NTHR) dyvbuf[idx] = from_f32<TO>(0.0f);
    }
    stage_all(0, (NT - 1) * TT);
    load_kq((NT - 1) * TT);
    store_kq(0);
    load_ck(NT - 1);
    cp_async_wait_all();
    __syncthreads();

    for (int tile = NT - 1; tile >= 0; --tile) {
        const int cur = (NT - 1 - tile) & 1, nxt = cur ^ 1;
        const int t0 = tile * TT;
        const int n = min(TT, L - t0);
        const bool more = tile > 0;

        // ---- replay the tile forward from its checkpoint
        float P[CH][SPT], mean[CH][SPT];
#pragma unroll
        for (int ci = 0; ci < CH; ++ci)
#pragma unroll
            for (int i = 0; i < SPT; ++i) {
                P[ci][i] = ck[ci][i].x;
                mean[ci][i] = ck[ci][i].y;
            }
        if (more) {  // prefetch the previous tile while this one is processed
            stage_all(nxt, t0 - TT);
            load_kq(t0 - TT);
            load_ck(tile - 1);
        }
        const T *lrow = lbuf + cur * TT * MC + cw;
        const T *vrow = vbuf + cur * TT * MC + cw;
        const TO *dyrow = dybuf + cur * TT * MC + cw;
        const TO *dyvrow = dyvbuf + cur * TT * MC + cw;
        const float4 *kqrow = kq4 + cur * TT * SPAD + j;
        float2 *drow = dpart + j * MCP + cw;
        auto replay_step = [&](int tt) {
            float lv[CH], vl[CH];
#pragma unroll
            for (int ci = 0; ci < CH; ++ci) {
                lv[ci] = to_f32<T>(lrow[tt * MC + ci]);
                vl[ci] = to_f32<T>(vrow[tt * MC + ci]) * lv[ci];
            }
#pragma unroll
            for (int i = 0; i < SPT; ++i) {
                const float4 c = kqrow[tt * SPAD + i * LPC];
#pragma unroll
                for (int ci = 0; ci < CH; ++ci) {
                    traj[slot(tt, ci, i, warp, lane)] = make_float2(P[ci][i], mean[ci][i]);
                    chain_step(P[ci][i], mean[ci][i], __fmul_rn(lv[ci], c.x), __fmul_rn(vl[ci], c.y),
                               ca[ci][i], ca2[ci][i], cp[ci][i]);
                }
            }
        };
        if (n == TT) {
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) replay_step(tt);
        } else {
            for (int tt = 0; tt < n; ++tt) replay_step(tt);
        }

        if (tile == NT - 1) {
            // Seed the carries from the gradient of the returned state:
            // lam_fin = 1/P, eta_fin = mean/P.
#pragma unroll
            for (int ci = 0; ci < CH; ++ci) {
                const int m = m_cta + cw + ci;
#pragma unroll
                for (int i = 0; i < SPT; ++i) {
                    const int s = i * LPC + j;
                    Pn[ci][i] = P[ci][i];
                    mn[ci][i] = mean[ci][i];
                    if (prm.dlam_fin != nullptr && m < M && s < S) {
                        const float Lb = prm.dlam_fin[((long long)b * M + m) * S + s];
                        const float Eb = prm.deta_fin[((long long)b * M + m) * S + s];
                        const float lam = 1.0f / P[ci][i];
                        const float eta = mean[ci][i] * lam;
                        cm[ci][i] = Eb * lam;
                        cP[ci][i] = -lam * (lam * Lb + eta * Eb);
                    }
                }
            }
        }

        // ---- walk the adjoint back down the tile
        auto reverse_step = [&](int tt) {
            float lv[CH], lv2[CH], vv[CH], vl[CH], dy[CH], dyv[CH], dyv2[CH], dvl[CH], dlphi[CH];
#pragma unroll
            for (int ci = 0; ci < CH; ++ci) {
                lv[ci] = to_f32<T>(lrow[tt * MC + ci]);
                vv[ci] = to_f32<T>(vrow[tt * MC + ci]);
                dy[ci] = to_f32<TO>(dyrow[tt * MC + ci]);
                dyv[ci] = to_f32<TO>(dyvrow[tt * MC + ci]);
                vl[ci] = vv[ci] * lv[ci];
                lv2[ci] = lv[ci] + lv[ci];
                dyv2[ci] = dyv[ci] + dyv[ci];
                dvl[ci] = 0.0f;
                dlphi[ci] = 0.0f;
            }
#pragma unroll
            for (int i = 0; i < SPT; ++i) {
                const float4 c = kqrow[tt * SPAD + i * LPC];  // k^2, k, q, q^2
                float X2 = 0.0f, Y = 0.0f, A_ = 0.0f, B2 = 0.0f;
#pragma unroll
                for (int ci = 0; ci < CH; ++ci) {
                    const float2 prev = traj[slot(tt, ci, i, warp, lane)];  // P', mean'
                    const float a = ca[ci][i], a2 = ca2[ci][i], p = cp[ci][i];
                    const float Pp = __fmaf_rn(a2, prev.x, p);
                    const float phi = __fmul_rn(lv[ci], c.x);
                    const float g = rcp_approx(__fmaf_rn(phi, Pp, 1.0f));
                    const float r = __fmul_rn(vl[ci], c.y);
                    float mbar, Pbar;
                    if (PRIOR) {  // y reads a*mean and a2*P + p
                        const float mob = dy[ci] * c.z, vob = dyv[ci] * c.w;
                        mbar = fmaf(mob, a, cm[ci][i]);
                        Pbar = fmaf(vob, a2, cP[ci][i]);
                        accA[ci][i] = fmaf(mob, mn[ci][i], accA[ci][i]);
                        accA2[ci][i] = fmaf(vob, Pn[ci][i], accA2[ci][i]);
                        accP[ci][i] += vob;
                        A_ = fmaf(dy[ci], a * mn[ci][i], A_);
                        B2 = fmaf(dyv2[ci], fmaf(a2, Pn[ci][i], p), B2);
                    } else {
                        mbar = fmaf(dy[ci], c.z, cm[ci][i]);
                        Pbar = fmaf(dyv[ci], c.w, cP[ci][i]);
                        A_ = fmaf(dy[ci], mn[ci][i], A_);
                        B2 = fmaf(dyv2[ci], Pn[ci][i], B2);
                    }
                    const float t2 = fmaf(Pbar, Pn[ci][i], mbar * mn[ci][i]);
                    const float dbar = -(g * t2);
                    const float ubar = mbar * g;
                    const float Ppbar = fmaf(dbar, phi, fmaf(Pbar, g, ubar * r));
                    const float rbar = ubar * Pp;
                    const float phibar = dbar * Pp;
                    cm[ci][i] = ubar * a;
                    cP[ci][i] = Ppbar * a2;
                    accA[ci][i] = fmaf(ubar, prev.y, accA[ci][i]);
                    accA2[ci][i] = fmaf(Ppbar, prev.x, accA2[ci][i]);
                    accP[ci][i] += Ppbar;
                    dlphi[ci] = fmaf(phibar, c.x, dlphi[ci]);
                    dvl[ci] = fmaf(rbar, c.y, dvl[ci]);
                    X2 = fmaf(phibar, lv2[ci], X2);
                    Y = fmaf(rbar, vl[ci], Y);
                    Pn[ci][i] = prev.x;
                    mn[ci][i] = prev.y;
                }
                // this thread's share of dk, dq for (t, s): parked where (P', mean') was
                traj[slot(tt, 0, i, warp, lane)] = make_float2(fmaf(c.y, X2, Y), fmaf(c.z, B2, A_));
            }
            // this thread's share of the sums over s; summed over lane groups per tile
#pragma unroll
            for (int ci = 0; ci < CH; ++ci) drow[tt * LPC * MCP + ci] = make_float2(dvl[ci], dlphi[ci]);
        };
        if (n == TT) {
#pragma unroll
            for (int tt = TT - 1; tt >= 0; --tt) reverse_step(tt);
        } else {
            for (int tt = n - 1; tt >= 0; --tt) reverse_step(tt);
        }
        __syncthreads();

        // ---- sum the (dv, dlambda_v) partials over lane groups and store them.
        // v enters only through v*lambda_v (kla_ops.py:177): with D = sum_s rbar k,
        // dv = D lambda_v and dlambda_v = sum_s phibar k^2 + D v.
        {
            const T *lt = lbuf + cur * TT * MC, *vt = vbuf + cur * TT * MC;
            output_pass<T, LPC, MC, MCP, TT, NTHR>(
                dpart, dvb + (long long)t0 * prm.dv.st, prm.dv.st, prm.vec_dv,
                dlvb + (long long)t0 * prm.dlv.st, prm.dlv.st, prm.vec_dlv, n, m_cta, M, tid,
                [&](float2 acc, int tt, int c, float &o0, float &o1) {
                    o0 = acc.x * to_f32<T>(lt[tt * MC + c]);
                    o1 = fmaf(acc.x, to_f32<T>(vt[tt * MC + c]), acc.y);
                });
        }

        // ---- sum dk, dq over the CTA's channels and add to global memory
        for (int pidx = tid; pidx < n * SPAD; pidx += NTHR) {
            const int jj = pidx % LPC, row = pidx / LPC;
            const int tt = row / SPT, i = row % SPT;
            const int s = i * LPC + jj;
            float sk = 0.0f, sq = 0.0f;
#pragma unroll
            for (int w = 0; w < NW; ++w) {
#pragma unroll
                for (int c = 0; c < CLS; ++c) {
                    const float2 x = traj[slot(tt, 0, i, w, c * LPC + jj)];
                    sk += x.x;
                    sq += x.y;
                }
            }
            if (s < S) {
                atomicAdd(prm.dk + ((long long)b * L + t0 + tt) * S + s, sk);
                atomicAdd(prm.dq + ((long long)b * L + t0 + tt) * S + s, sq);
            }
        }
        if (more) store_kq(nxt);
        cp_async_wait_all();
        __syncthreads();
    }

    // ---- end of sequence: gradients of a, p and of the carried-in state
#pragma unroll
    for (int ci = 0; ci < CH; ++ci) {
        const int m = m_cta + cw + ci;
#pragma unroll
        for (int i = 0; i < SPT; ++i) {
            const int s = i * LPC + j;
            if (m < M && s < S) {
                const long long ms = (long long)m * S + s, bms = ((long long)b * M + m) * S + s;
                const float a = ca[ci][i];
                const float da2_da = (a * a >= kEps) ? 2.0f * a : 0.0f;  // clamp_min subgradient
                atomicAdd(prm.da + ms, fmaf(accA2[ci][i], da2_da, accA[ci][i]));
                if (prm.p[ms] >= kPMin) atomicAdd(prm.dp + ms, accP[ci][i]);
                float lam0 = 1.0f, eta0 = 0.0f;
                if (prm.lam0 != nullptr) {
                    lam0 = prm.lam0[bms];
                    eta0 = prm.eta0[bms];
                }
                // P0 = 1/max(lam0, floor), mean0 = eta0 * P0
                const float P0 = 1.0f / fmaxf(lam0, kLamMin);
                prm.deta0[bms] = cm[ci][i] * P0;
                prm.dlam0[bms] = (lam0 >= kLamMin) ? -(cP[ci][i] + cm[ci][i] * eta0) * P0 * P0 : 0.0f;
            }
        }
    }
}

}  // namespace kla
