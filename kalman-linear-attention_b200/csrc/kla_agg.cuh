// Slab / chunk aggregates: how a whole stretch of time steps acts on the filter
// state (forward) and on the backward carry (adjoint), one 32-byte record per
// chain. They are what lets the time axis be cut -- into chunks that run side by
// side on one GPU, or into slabs held by different GPUs -- because they compose
// associatively and can be folded in a few operations per cut.
//
// * forward. In homogeneous coordinates h = (x, w, z) with P = w/x and
//   mean = z/x one filter step is linear,
//       x' = (1 + p phi) x + a2 phi w,   w' = p x + a2 w,   z' = r w' + a z,
//   (the variance-form step of kla_common.cuh multiplied through by its
//   denominator), so a stretch of steps is the product of its step matrices:
//   7 numbers (m00 m01 / m10 m11 / m20 m21 m22), rescaled every other step --
//   a common factor does not change P or mean. This is the reference's
//   trace-normalised 2x2 Moebius product (src/kla/ops/kla_ops.py:76-116)
//   extended by the row that carries the mean, which lets one pass serve both
//   recurrences instead of two dependent ones (kla_ops.py:248, 274-280).
//
// * adjoint. With the forward trajectory fixed, the backward carries obey
//   c_{t-1} = J_t (c_t + e_t), J_t = [[a2 g^2, a2 g (r - phi mean_t)], [0, a g]],
//   e_t = (dyvar q^2, dy q): affine, upper triangular. Walking FORWARD in time,
//   K_t = J_1 ... J_t and b = sum_t K_t e_t give the carry that leaves the
//   stretch at its first step as K c_in + b (5 numbers). It needs the stretch's
//   true initial state, i.e. it runs after the forward fold.
//
// Kernel shape: as the scan kernels. NW compute warps, each thread owning SPT
// states of one channel as pairs (paired fp32 instructions), and one loader warp
// that brings tiles of TT steps in: v, lambda_v (and dy, dy_var) as TMA tiles
// signalled on mbarriers, k (and q) regrouped by owning lane. The forward
// aggregate has no reciprocal on its dependent path, so one warp per scheduler
// already runs at the arithmetic rate. Nothing is written but the final record.
#pragma once

#include "kla_common.cuh"

namespace kla {

constexpr int kAggStages = 3;
constexpr int kAggTT = 32;  // steps per tile

struct alignas(64) AggParams {
    CUtensorMap tm_v, tm_lv, tm_dy, tm_dyv;  // rank-3 (M, L, B) maps with box (MC, kAggTT, 1); valid when use_tma
    int B, L, M, S;
    int use_tma;
    Tensor3 v, lv, k, q, dy, dyv;      // dy, dyv, q: adjoint only
    const float *a, *p, *lam0, *eta0;  // lam0/eta0: adjoint only (nullptr = unit prior)
    float *out;                        // [B, M, S, 8]
    WaitCtl wait;
};

template <typename T, typename TO, int SPT, int LPC, int NW, bool ADJ>
struct AggSmem {
    static constexpr int kMC = NW * (32 / LPC);
    static constexpr int kSPad = SPT * LPC;
    static constexpr size_t kBars = 128;
    static constexpr size_t kTileI = ((sizeof(T) * kAggTT * kMC + 127) / 128) * 128;
    static constexpr size_t kTileO = ((sizeof(TO) * kAggTT * kMC + 127) / 128) * 128;
    static constexpr size_t kKq = ((sizeof(float) * (ADJ ? 2 : 1) * kAggTT * kSPad + 127) / 128) * 128;
    static constexpr size_t kIn = 2 * kTileI + (ADJ ? 2 * kTileO : 0) + kKq;
    static constexpr size_t kTotal = kBars + kAggStages * kIn;
};

template <typename T, typename TO, int SPT, int LPC, int NW, bool ADJ, bool PRIOR>
__global__ void __launch_bounds__((NW + 1) * 32) kla_agg_kernel(const __grid_constant__ AggParams prm) {
    using Sm = AggSmem<T, TO, SPT, LPC, NW, ADJ>;
    constexpr int TT = kAggTT, NS = kAggStages, MC = Sm::kMC, SPAD = Sm::kSPad, CLS = 32 / LPC;
    constexpr int HP = SPT / 2, NK = ADJ ? 2 : 1;
    static_assert(SPT % 2 == 0, "states are processed in pairs");
    constexpr int kCompute = NW * 32;

    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t *full_in = reinterpret_cast<uint64_t *>(smem);  // [NS] loader -> compute
    uint64_t *empty_in = full_in + NS;                       // [NS] compute -> loader
    unsigned char *in_base = smem + Sm::kBars;
    auto vstage = [&](int s) { return reinterpret_cast<T *>(in_base + s * Sm::kIn); };
    auto lstage = [&](int s) { return reinterpret_cast<T *>(in_base + s * Sm::kIn + Sm::kTileI); };
    auto dystage = [&](int s) { return reinterpret_cast<TO *>(in_base + s * Sm::kIn + 2 * Sm::kTileI); };
    auto dyvstage = [&](int s) { return reinterpret_cast<TO *>(in_base + s * Sm::kIn + 2 * Sm::kTileI + Sm::kTileO); };
    // k (and q) of a step, grouped by owning lane: [TT][LPC][NK][SPT] floats, state s = i * LPC + j at [j][.][i]
    auto kqstage = [&](int s) {
        return reinterpret_cast<float *>(in_base + s * Sm::kIn + 2 * Sm::kTileI + (ADJ ? 2 * Sm::kTileO : 0));
    };

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.y, m_cta = blockIdx.x * MC;
    const int L = prm.L, M = prm.M, S = prm.S;
    const int NT = (L + TT - 1) / TT;
    const bool has_dyv = ADJ && prm.dyv.ptr != nullptr;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&full_in[s], 32);
            mbar_init(&empty_in[s], NW);
        }
        mbar_fence_init();
    }
    __syncthreads();

    if (warp < NW) {
        // =============================================================== compute
        const int j = lane % LPC, cl = lane / LPC;
        const int cw = warp * CLS + cl;  // this thread's channel, CTA-relative
        const int m = m_cta + cw;
        float2 ca[HP], ca2[HP], cp[HP];
        // forward: m00 m01 m10 m11 m20 m21 m22; adjoint: K00 K01 K11 b0 b1 P mean
        float2 A[7][HP];
#pragma unroll
        for (int i = 0; i < SPT; ++i) {
            const int s = i * LPC + j;
            const bool live = (m < M) && (s < S);
            const float av = live ? prm.a[(long long)m * S + s] : 0.0f;
            const float pv = live ? prm.p[(long long)m * S + s] : 1.0f;
            pair_el(ca, i) = av;
            pair_el(ca2, i) = live ? fmaxf(av * av, kEps) : 0.0f;
            pair_el(cp, i) = fmaxf(pv, kPMin);
            if (ADJ) {
                float lam = 1.0f, eta = 0.0f;
                if (live && prm.lam0 != nullptr) {
                    lam = prm.lam0[((long long)b * M + m) * S + s];
                    eta = prm.eta0[((long long)b * M + m) * S + s];
                }
                const float P0 = 1.0f / fmaxf(lam, kLamMin);
                pair_el(A[0], i) = 1.0f; pair_el(A[1], i) = 0.0f; pair_el(A[2], i) = 1.0f;
                pair_el(A[3], i) = 0.0f; pair_el(A[4], i) = 0.0f;
                pair_el(A[5], i) = P0; pair_el(A[6], i) = eta * P0;
            } else {
                pair_el(A[0], i) = 1.0f; pair_el(A[1], i) = 0.0f; pair_el(A[2], i) = 0.0f; pair_el(A[3], i) = 1.0f;
                pair_el(A[4], i) = 0.0f; pair_el(A[5], i) = 0.0f; pair_el(A[6], i) = 1.0f;
            }
        }

        auto step = [&](const T *vrow, const T *lrow, const TO *dyrow, const TO *dyvrow, const float *kqrow, int tt,
                        bool rescale) {
            const float2 lv = dup2(to_f32<T>(lrow[tt * MC])), vv = dup2(to_f32<T>(vrow[tt * MC]));
            const float *row = kqrow + tt * NK * SPAD;
            float2 kk[HP], qq[HP];
            if constexpr (SPT == 4) {
                const float4 k4 = *reinterpret_cast<const float4 *>(row);
                kk[0] = make_float2(k4.x, k4.y);
                kk[1] = make_float2(k4.z, k4.w);
                if (ADJ) {
                    const float4 q4 = *reinterpret_cast<const float4 *>(row + SPT);
                    qq[0] = make_float2(q4.x, q4.y);
                    qq[1] = make_float2(q4.z, q4.w);
                }
            } else {
#pragma unroll
                for (int h = 0; h < HP; ++h) {
                    kk[h] = *reinterpret_cast<const float2 *>(row + 2 * h);
                    if (ADJ) qq[h] = *reinterpret_cast<const float2 *>(row + SPT + 2 * h);
                }
            }
            if constexpr (!ADJ) {
#pragma unroll
                for (int h = 0; h < HP; ++h) {
                    float2 phi, r;
                    chain_inputs2(lv, vv, kk[h], phi, r);
                    // the step as two shears: w' = p x + a2 w, then x' = x + phi w' (= (1 + p phi) x + a2 phi w)
                    const float2 n10 = fma2(ca2[h], A[2][h], mul2(cp[h], A[0][h]));
                    const float2 n11 = fma2(ca2[h], A[3][h], mul2(cp[h], A[1][h]));
                    const float2 n00 = fma2(phi, n10, A[0][h]), n01 = fma2(phi, n11, A[1][h]);
                    A[4][h] = fma2(r, n10, mul2(ca[h], A[4][h]));
                    A[5][h] = fma2(r, n11, mul2(ca[h], A[5][h]));
                    A[6][h] = mul2(ca[h], A[6][h]);
                    A[0][h] = n00; A[1][h] = n01; A[2][h] = n10; A[3][h] = n11;
                    if (rescale) {  // a common factor leaves P = w/x and mean = z/x unchanged
                        const float2 sc = rcp_approx2(add2(n00, n01));
#pragma unroll
                        for (int e = 0; e < 7; ++e) A[e][h] = mul2(A[e][h], sc);
                    }
                }
            } else {
                const float dyf = to_f32<TO>(dyrow[tt * MC]), dyvf = to_f32<TO>(dyvrow[tt * MC]);
                float2 Pp[HP], g[HP], r[HP], phi[HP];
#pragma unroll
                for (int h = 0; h < HP; ++h) {
                    chain_inputs2(lv, vv, kk[h], phi[h], r[h]);
                    g[h] = chain_denominator2(A[5][h], phi[h], ca2[h], cp[h], Pp[h]);
                }
#pragma unroll
                for (int h = 0; h < HP; ++h) g[h] = rcp_approx2(g[h]);
#pragma unroll
                for (int h = 0; h < HP; ++h) {
                    chain_update2(A[5][h], A[6][h], Pp[h], g[h], r[h], ca[h]);  // P_t, mean_t
                    const float2 a2g = mul2(ca2[h], g[h]);
                    const float2 j00 = mul2(a2g, g[h]);
                    const float2 j01 = mul2(a2g, fma2(neg2(phi[h]), A[6][h], r[h]));
                    const float2 j11 = mul2(ca[h], g[h]);
                    float2 e0 = mul2(dup2(dyvf), mul2(qq[h], qq[h])), e1 = mul2(dup2(dyf), qq[h]);
                    if (PRIOR) {
                        e0 = mul2(e0, ca2[h]);
                        e1 = mul2(e1, ca[h]);
                    }
                    const float2 K00 = mul2(A[0][h], j00);
                    const float2 K01 = fma2(A[0][h], j01, mul2(A[1][h], j11));
                    const float2 K11 = mul2(A[2][h], j11);
                    A[0][h] = K00; A[1][h] = K01; A[2][h] = K11;
                    A[3][h] = fma2(K00, e0, fma2(K01, e1, A[3][h]));
                    A[4][h] = fma2(K11, e1, A[4][h]);
                }
            }
        };

        for (int tile = 0; tile < NT; ++tile) {
            const int s = tile % NS, t0 = tile * TT;
            if (!mbar_wait(prm.wait, &full_in[s], (tile / NS) & 1, 31)) break;
            const T *vrow = vstage(s) + cw, *lrow = lstage(s) + cw;
            const TO *dyrow = dystage(s) + cw, *dyvrow = dyvstage(s) + cw;
            const float *kqrow = kqstage(s) + j * NK * SPT;
            if (t0 + TT <= L) {
#pragma unroll 1
                for (int t4 = 0; t4 < TT; t4 += 4) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) step(vrow, lrow, dyrow, dyvrow, kqrow, t4 + u, (u & 1) != 0);
                }
            } else {
                for (int tt = 0; t0 + tt < L; ++tt) step(vrow, lrow, dyrow, dyvrow, kqrow, tt, (tt & 1) != 0);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_in[s]);
        }

#pragma unroll
        for (int i = 0; i < SPT; ++i) {
            const int s = i * LPC + j;
            if (m < M && s < S) {
                float4 *o = reinterpret_cast<float4 *>(prm.out + (((long long)b * M + m) * S + s) * 8);
                o[0] = make_float4(pair_el(A[0], i), pair_el(A[1], i), pair_el(A[2], i), pair_el(A[3], i));
                o[1] = make_float4(pair_el(A[4], i), pair_el(A[5], i), pair_el(A[6], i), 0.0f);
            }
        }
    } else {
        // ================================================================ loader warp
        constexpr uint32_t kBytesI = sizeof(T) * TT * MC, kBytesO = sizeof(TO) * TT * MC;
        const T *vb = static_cast<const T *>(prm.v.ptr) + (long long)b * prm.v.sb;
        const T *lb = static_cast<const T *>(prm.lv.ptr) + (long long)b * prm.lv.sb;
        const T *kb = static_cast<const T *>(prm.k.ptr) + (long long)b * prm.k.sb;
        const T *qb = ADJ ? static_cast<const T *>(prm.q.ptr) + (long long)b * prm.q.sb : nullptr;
        const TO *dyb = ADJ ? static_cast<const TO *>(prm.dy.ptr) + (long long)b * prm.dy.sb : nullptr;
        const TO *dyvb = has_dyv ? static_cast<const TO *>(prm.dyv.ptr) + (long long)b * prm.dyv.sb : nullptr;
        if (ADJ && !has_dyv) {  // dyvar absent: its stage buffers stay zero for the whole kernel
            for (int s = 0; s < NS; ++s)
                for (int idx = lane; idx < TT * MC; idx += 32) dyvstage(s)[idx] = from_f32<TO>(0.0f);
            fence_proxy_async();
        }
        constexpr int KQP = (TT * SPAD + 31) / 32;
        float kr[KQP], qr[ADJ ? KQP : 1];
        auto load_kq = [&](int t0) {
#pragma unroll
            for (int e = 0; e < KQP; ++e) {
                const int idx = lane + e * 32, row = idx / SPAD, sidx = idx % SPAD;
                const bool in = idx < TT * SPAD && sidx < S && t0 + row < L;
                kr[e] = in ? to_f32<T>(kb[(long long)(t0 + row) * prm.k.st + sidx]) : 0.0f;
                if (ADJ) qr[e] = in ? to_f32<T>(qb[(long long)(t0 + row) * prm.q.st + sidx]) : 0.0f;
            }
        };
        int produced = 0;
        bool ok = true;
        if (NT > 0) load_kq(0);
        for (int it = 0; it < NT; ++it) {
            const int s = it % NS, t0 = it * TT;
            if (it >= NS && !mbar_wait(prm.wait, &empty_in[s], (it / NS - 1) & 1, 32, 100)) { ok = false; break; }
            if (prm.use_tma) {
                if (lane == 0) {
                    mbar_arrive_expect_tx(&full_in[s], 2 * kBytesI + (ADJ ? (has_dyv ? 2 : 1) * kBytesO : 0));
                    tma_load_3d(vstage(s), &prm.tm_v, m_cta, t0, b, &full_in[s]);
                    tma_load_3d(lstage(s), &prm.tm_lv, m_cta, t0, b, &full_in[s]);
                    if (ADJ) {
                        tma_load_3d(dystage(s), &prm.tm_dy, m_cta, t0, b, &full_in[s]);
                        if (has_dyv) tma_load_3d(dyvstage(s), &prm.tm_dyv, m_cta, t0, b, &full_in[s]);
                    }
                }
            } else {
                stage_tile_plain<T, TT, MC, 32>(vstage(s), vb, prm.v.st, t0, L, m_cta, M, lane);
                stage_tile_plain<T, TT, MC, 32>(lstage(s), lb, prm.lv.st, t0, L, m_cta, M, lane);
                if (ADJ) {
                    stage_tile_plain<TO, TT, MC, 32>(dystage(s), dyb, prm.dy.st, t0, L, m_cta, M, lane);
                    if (has_dyv) stage_tile_plain<TO, TT, MC, 32>(dyvstage(s), dyvb, prm.dyv.st, t0, L, m_cta, M, lane);
                }
            }
            float *kq = kqstage(s);
#pragma unroll
            for (int e = 0; e < KQP; ++e) {
                const int idx = lane + e * 32, row = idx / SPAD, sidx = idx % SPAD;
                if (idx < TT * SPAD) {
                    float *dst = kq + row * NK * SPAD + (sidx % LPC) * NK * SPT + sidx / LPC;
                    dst[0] = kr[e];
                    if (ADJ) dst[SPT] = qr[e];
                }
            }
            if (it + 1 < NT) load_kq(t0 + TT);
            if (!(prm.use_tma && lane == 0)) mbar_arrive(&full_in[s]);
            produced = it + 1;
        }
        // leaving early (a wait ran out): do not end the CTA with bulk copies still in flight into its shared memory
        if (!ok && prm.use_tma && lane == 0)
            for (int t = max(0, produced - NS); t < produced; ++t) mbar_wait(prm.wait, &full_in[t % NS], (t / NS) & 1, 33);
    }
}

}  // namespace kla
