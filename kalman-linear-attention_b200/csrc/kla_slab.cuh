// Folds of per-chunk aggregates (kla_agg.cuh) for the time-parallel scan on one GPU.
#pragma once

#include "kla_common.cuh"

namespace kla {

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
    // The fold itself is serial over c, but a chunk's record does not depend on the carry: the next record is
    // fetched while the current one is applied, so the loop pays one memory latency, not C of them.
    auto fetch = [&](int c, float4 &lo, float4 &hi) {
        const float4 *src = reinterpret_cast<const float4 *>(prm.agg + (((b * C + c) * lanes) + ms) * 8);
        lo = src[0];
        hi = src[1];
    };
    float4 lo, hi, nlo = make_float4(0, 0, 0, 0), nhi = nlo;
    if (!ADJ) {
        // the state in homogeneous coordinates (x, w, z), P = w/x, mean = z/x: applying a record is a 3x3
        // product, and lam = x/w, eta = z/w need one reciprocal per chunk. Records are normalised, so the
        // coordinates stay far inside the float64 range for any chunk count the launcher accepts.
        double x = 1.0, w = 1.0, z = 0.0;
        if (prm.in_a != nullptr) {
            w = 1.0 / fmax((double)prm.in_a[gid], (double)kLamMin);
            z = (double)prm.in_b[gid] * w;
        }
        if (C > 1) fetch(0, nlo, nhi);
        for (int c = 0; c < C; ++c) {
            const long long o = (b * C + c) * lanes + ms;
            const double rw = 1.0 / w;
            prm.out_a[o] = (float)(x * rw);
            prm.out_b[o] = (float)(z * rw);
            if (c + 1 < C) {
                lo = nlo; hi = nhi;
                if (c + 2 < C) fetch(c + 1, nlo, nhi);
                const double nx = (double)lo.x * x + (double)lo.y * w, nw = (double)lo.z * x + (double)lo.w * w;
                z = (double)hi.x * x + (double)hi.y * w + (double)hi.z * z;
                x = nx;
                w = nw;
            }
        }
    } else {
        fetch(C - 1, lo, hi);
        if (C > 1) fetch(C - 2, nlo, nhi);
        const double dl = prm.in_a ? (double)prm.in_a[gid] : 0.0, de = prm.in_b ? (double)prm.in_b[gid] : 0.0;
        // (dL/dP, dL/dmean) at the end of the sequence from the gradient of (lam, eta) = (1/P, mean/P)
        const double lam = 1.0 / (double)hi.y, eta = (double)hi.z * lam;
        double cP = -lam * (lam * dl + eta * de), cm = de * lam;
        for (int c = C - 1; c >= 0; --c) {
            if (c != C - 1) {
                lo = nlo; hi = nhi;
                if (c > 0) fetch(c - 1, nlo, nhi);
            }
            const long long o = (b * C + c) * lanes + ms;
            const double P_end = hi.y, mean_end = hi.z;  // record: K00 K01 K11 b0 | b1 P_end mean_end
            const double deta = cm * P_end;
            prm.out_b[o] = (float)deta;
            prm.out_a[o] = (float)(-(cP * P_end * P_end + mean_end * deta));
            const double nP = (double)lo.x * cP + (double)lo.y * cm + (double)lo.w;
            cm = (double)lo.z * cm + (double)hi.x;
            cP = nP;
        }
    }
}

}  // namespace kla
