// Raw scan pair over materialised coefficients: the Moebius (precision)
// recurrence lam_t = (A_t lam' + B_t) / (C_t lam' + D_t) and the affine
// (information-vector) recurrence eta_t = alpha_t eta' + r_t, each with its
// exact backward. All tensors are [B, L, N] float32 with N = M*S lanes per
// (b, t) row; lanes are independent and time is the serial axis.
//
// These kernels move 12 to 40 bytes per lane-step for a handful of
// flops, so they are bound by HBM bandwidth. A CTA owns LC consecutive lanes of
// one batch entry and streams the sequence in tiles of TT steps:
//   producer warp   one elected thread issues a TMA tile load per input tensor
//                   into a ring of shared-memory stages (mbarrier hand-over);
//   compute warps   one thread per lane carries the recurrence down (or, for
//                   the backward kernels, up) the tile and writes the results
//                   to a shared-memory output tile;
//   stores          one elected thread sends each finished output tile with a
//                   TMA store; a ring of three output tiles lets the store of
//                   tile i overlap the computation of tile i+1.
// Tensors that do not meet the TMA alignment rules (N not a multiple of 4,
// unaligned base) are staged with plain loads by the producer warp and stored
// directly by the compute threads.
#pragma once

#include "kla_common.cuh"

namespace kla {

constexpr int kRawLC = 128;   // lanes per CTA (= compute threads)
constexpr int kRawTT = 8;     // steps per tile
constexpr int kRawNSO = 3;    // output tiles in the store ring
constexpr int kRawMaxIn = 6, kRawMaxOut = 4;

struct alignas(64) RawParams {
    CUtensorMap tm_in[kRawMaxIn];
    CUtensorMap tm_out[kRawMaxOut];
    const float *in[kRawMaxIn];
    float *out[kRawMaxOut];
    const float *state0;  // [B, N] or nullptr
    float *dstate0;       // [B, N] or nullptr
    int B, L, N, NT;
    int use_tma;
    WaitCtl wait;
};

// TMA store of a shared-memory tile into a rank-3 tensor map, tracked by the bulk-group mechanism
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *tm, const void *src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(tm)), "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

constexpr float kRawDenMin = 1e-12f;  // floor on the Moebius denominator, tiled_mobius_scan.py:102 and :246

// The four recurrences. REV: walks time downwards. HALO: index of the input that
// is also needed one step earlier (the saved forward output), or -1.
// step(x, prev, y): x = this step's inputs, prev = the HALO input at t-1 (the
// initial state at t = 0).
struct MobiusFwd {  // in: A B C D   out: lam
    static constexpr int NIN = 4, NOUT = 1, HALO = -1, NSI = 2;
    static constexpr bool REV = false;
    static constexpr float kPrior = 1.0f;  // lam0 when none is given, tiled_mobius_scan.py:303-305
    float lam;
    __device__ void init(float s0) { lam = s0; }
    __device__ void step(const float (&x)[NIN], float, float (&y)[NOUT]) {
        const float den = fmaxf(fmaf(x[2], lam, x[3]), kRawDenMin);
        lam = fmaf(x[0], lam, x[1]) / den;
        y[0] = lam;
    }
    __device__ float finish() const { return 0.0f; }
};
struct AffineFwd {  // in: alpha r   out: eta
    static constexpr int NIN = 2, NOUT = 1, HALO = -1, NSI = 3;
    static constexpr bool REV = false;
    static constexpr float kPrior = 0.0f;  // eta_{-1} = 0
    float eta;
    __device__ void init(float s0) { eta = s0; }
    __device__ void step(const float (&x)[NIN], float, float (&y)[NOUT]) {
        eta = fmaf(x[0], eta, x[1]);
        y[0] = eta;
    }
    __device__ float finish() const { return 0.0f; }
};
// Adjoint of the Moebius scan (tiled_mobius_scan.py:266-279): with
// den = C lam' + D and gain = (AD - BC)/den^2, nu_t = dlam_t + gain_{t+1} nu_{t+1},
// dA = nu lam'/den, dB = nu/den, dC = -nu lam lam'/den, dD = -nu lam/den, dlam0 = gain_0 nu_0.
struct MobiusBwd {  // in: A B C D lam dlam   out: dA dB dC dD
    static constexpr int NIN = 6, NOUT = 4, HALO = 4, NSI = 2;
    static constexpr bool REV = true;
    static constexpr float kPrior = 1.0f;
    float c;
    __device__ void init(float) { c = 0.0f; }
    __device__ void step(const float (&x)[NIN], float prev, float (&y)[NOUT]) {
        const float den = fmaxf(fmaf(x[2], prev, x[3]), kRawDenMin);
        const float nu = x[5] + c;
        const float nod = nu / den;
        y[0] = nod * prev;
        y[1] = nod;
        y[2] = -(nod * x[4]) * prev;
        y[3] = -(nod * x[4]);
        c = (fmaf(x[0], x[3], -(x[1] * x[2])) / (den * den)) * nu;
    }
    __device__ float finish() const { return c; }
};
// Adjoint of the affine scan (tiled_mobius_scan.py:289-296): mu_t = deta_t + alpha_{t+1} mu_{t+1},
// dalpha = mu eta', dr = mu.
struct AffineBwd {  // in: alpha eta deta   out: dalpha dr
    static constexpr int NIN = 3, NOUT = 2, HALO = 1, NSI = 2;
    static constexpr bool REV = true;
    static constexpr float kPrior = 0.0f;
    float c;
    __device__ void init(float) { c = 0.0f; }
    __device__ void step(const float (&x)[NIN], float prev, float (&y)[NOUT]) {
        const float mu = x[2] + c;
        y[0] = mu * prev;
        y[1] = mu;
        c = x[0] * mu;
    }
    __device__ float finish() const { return c; }
};

template <class Op>
struct RawSmem {
    static constexpr size_t kBars = 128;
    static constexpr size_t kInTile = sizeof(float) * (kRawTT + 1) * kRawLC;  // one extra row for the halo
    static constexpr size_t kOutTile = sizeof(float) * kRawTT * kRawLC;
    static constexpr size_t kIn = Op::NIN * kInTile, kOut = Op::NOUT * kOutTile;
    static constexpr size_t kTotal = kBars + Op::NSI * kIn + kRawNSO * kOut;
};

template <class Op>
__global__ void __launch_bounds__(kRawLC + 32) kla_rawscan_kernel(const __grid_constant__ RawParams prm) {
    using Sm = RawSmem<Op>;
    constexpr int LC = kRawLC, TT = kRawTT, NSI = Op::NSI, NSO = kRawNSO, NIN = Op::NIN, NOUT = Op::NOUT;
    constexpr int NCW = LC / 32;  // compute warps
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t *full_in = reinterpret_cast<uint64_t *>(smem);  // [NSI]
    uint64_t *empty_in = full_in + NSI;                      // [NSI]
    unsigned char *in_base = smem + Sm::kBars, *out_base = in_base + NSI * Sm::kIn;
    auto in_tile = [&](int s, int i) { return reinterpret_cast<float *>(in_base + s * Sm::kIn + i * Sm::kInTile); };
    auto out_tile = [&](int o, int k) { return reinterpret_cast<float *>(out_base + o * Sm::kOut + k * Sm::kOutTile); };

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.y, lane0 = blockIdx.x * LC;
    const int L = prm.L, N = prm.N, NT = prm.NT;
    const bool tma = prm.use_tma != 0;

    if (tid == 0) {
        for (int s = 0; s < NSI; ++s) {
            mbar_init(&full_in[s], tma ? 1 : 32);
            mbar_init(&empty_in[s], NCW);
        }
        mbar_fence_init();
    }
    __syncthreads();

    if (warp < NCW) {
        // =============================================================== compute
        const int ln = lane0 + tid;
        const bool live = ln < N;
        Op op;
        // state before the first step: given, or the recurrence's prior
        const float prev0 = (prm.state0 != nullptr && live) ? prm.state0[(long long)b * N + ln] : Op::kPrior;
        op.init(prev0);

        for (int ti = 0; ti < NT; ++ti) {
            const int tile = Op::REV ? NT - 1 - ti : ti;
            const int t0 = tile * TT, n = min(TT, L - t0);
            const int s = ti % NSI, o = ti % NSO;
            if (!mbar_wait(prm.wait, &full_in[s], (ti / NSI) & 1, 21)) break;
            auto one_step = [&](int u) {
                float x[NIN], y[NOUT];
#pragma unroll
                for (int i = 0; i < NIN; ++i) x[i] = in_tile(s, i)[(u + (i == Op::HALO ? 1 : 0)) * LC + tid];
                float prev = 0.0f;
                if (Op::HALO >= 0) prev = (t0 + u == 0) ? prev0 : in_tile(s, Op::HALO >= 0 ? Op::HALO : 0)[u * LC + tid];
                op.step(x, prev, y);
                if (tma) {
#pragma unroll
                    for (int k = 0; k < NOUT; ++k) out_tile(o, k)[u * LC + tid] = y[k];
                } else if (live) {
#pragma unroll
                    for (int k = 0; k < NOUT; ++k) prm.out[k][((long long)b * L + t0 + u) * N + ln] = y[k];
                }
            };
            if (n == TT) {
#pragma unroll
                for (int uu = 0; uu < TT; ++uu) one_step(Op::REV ? TT - 1 - uu : uu);
            } else {
                for (int uu = 0; uu < n; ++uu) one_step(Op::REV ? n - 1 - uu : uu);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_in[s]);
            if (tma) {
                // Tile ti's stores may start once every compute thread has written it. Before
                // that barrier the issuing thread makes sure the store of tile ti-2 has
                // finished reading shared memory, which frees the tile the next iteration writes.
                if (tid == 0) bulk_wait_read<1>();
                fence_proxy_async();
                named_bar_sync(1, LC);
                if (tid == 0) {
#pragma unroll
                    for (int k = 0; k < NOUT; ++k) tma_store_3d(&prm.tm_out[k], out_tile(o, k), lane0, t0, b);
                    bulk_commit();
                }
            }
        }
        if (tma && tid == 0) bulk_wait_read<0>();  // shared memory must outlive the stores that read it
        if (prm.dstate0 != nullptr && live) prm.dstate0[(long long)b * N + ln] = op.finish();
    } else {
        // ============================================================== producer
        int produced = 0;
        bool ok = true;
        for (int ti = 0; ti < NT; ++ti) {
            const int tile = Op::REV ? NT - 1 - ti : ti;
            const int t0 = tile * TT, s = ti % NSI;
            if (ti >= NSI && !mbar_wait(prm.wait, &empty_in[s], (ti / NSI - 1) & 1, 22, 50)) { ok = false; break; }
            if (tma) {
                if (lane == 0) {
                    constexpr uint32_t kBytes = sizeof(float) * LC * (NIN * TT + (Op::HALO >= 0 ? 1 : 0));
                    mbar_arrive_expect_tx(&full_in[s], kBytes);
#pragma unroll
                    for (int i = 0; i < NIN; ++i)
                        tma_load_3d(in_tile(s, i), &prm.tm_in[i], lane0, i == Op::HALO ? t0 - 1 : t0, b, &full_in[s]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < NIN; ++i) {
                    const int rows = TT + (i == Op::HALO ? 1 : 0), tstart = i == Op::HALO ? t0 - 1 : t0;
                    const float *src = prm.in[i] + (long long)b * L * N;
                    float *dst = in_tile(s, i);
                    for (int idx = lane; idx < rows * LC; idx += 32) {
                        const int row = idx / LC, c = idx % LC, t = tstart + row;
                        dst[idx] = (t >= 0 && t < L && lane0 + c < N) ? src[(long long)t * N + lane0 + c] : 0.0f;
                    }
                }
                mbar_arrive(&full_in[s]);
            }
            produced = ti + 1;
        }
        // Leaving early (a wait ran out): do not end the CTA with bulk copies in flight into its shared memory.
        if (!ok && tma && lane == 0)
            for (int t = max(0, produced - NSI); t < produced; ++t) mbar_wait(prm.wait, &full_in[t % NSI], (t / NSI) & 1, 23);
    }
}

}  // namespace kla
