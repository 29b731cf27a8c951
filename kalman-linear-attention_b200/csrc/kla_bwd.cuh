// Fused backward scan kernel: the exact adjoint of kla_fwd_kernel.
//
// Time is walked in tiles of kCkptInterval steps, last tile first. For each tile
// the forward recurrence is replayed from the tile's checkpoint, every chain's
// pre-step state (P', mean') going to shared memory, and then the adjoint is
// walked back down the tile with the two carries (dL/dP, dL/dmean) in registers.
// The same statements differentiated by hand (variance form, see kla_common.cuh):
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
// The CTA is three groups of four warps, each with the registers its role needs
// (the register file is re-divided between the groups when the kernel starts):
//   replay warps   run the forward recurrence of tile n+1 into one of two
//                  trajectory buffers while
//   reverse warps  walk the adjoint down tile n from the other buffer, leaving
//                  what crosses threads in shared memory:
//                    sums over s (dv, dlambda_v): LPC partials per (t, channel);
//                    sums over m (dk, dq): one partial per thread per (t, state),
//                    parked in the slot its (P', mean') occupied;
//                  sums over b and t (da, dp) stay in registers until the end;
//   helper warps   one loads (TMA tiles of v, lambda_v, dy, dy_var issued by one
//                  elected thread, and the (k, q) values of a tile, those
//                  of the next tile already in registers); three finish the sums:
//                  the CTA's channels of dk, dq and one atomic per (t, s), the
//                  lane groups of dv, dlambda_v and their stores.
// Replay and reverse are different instruction streams with little in common but
// the trajectory, so running them side by side doubles the warps a scheduler can
// choose from without doubling the registers: the replay needs half of what
// the reverse walk needs. All hand-overs go through mbarriers.
//
// With SEG a sequence is walked by several CTAs, last stretch first (SegCtl, kla_common.cuh): a CTA takes the two
// carries and the running sums for da, dp from the CTA that walked the stretch after its own, and hands its own
// on; the state its walk starts from needs no hand-over, the replay group computes it from the checkpoints.
//
// Measured on B200 at B=8, T=4096, M=1024, S=16 (1.49 ms unsegmented, 1.42 ms in 16 segments): the reverse walk alone takes 1.15 ms, the replay alone
// 0.53 ms, the sums 0.12 ms; side by side they overlap only in part. Variants that were measured and are not kept:
// the trajectory through tensor memory (tcgen05.st / tcgen05.ld, a third less shared-memory traffic: 1.56 ms),
// the reverse walk on paired fp32 instructions (a third fewer instructions: 1.68 ms), other register splits between
// the groups and deeper unrolling (1.54-1.79 ms), the reverse walk's shared-memory reads fetched one step ahead by hand
// (1.62 ms). No single resource is the limit: issue slots, the FP32 pipe and
// the shared-memory pipe are each a half to three quarters busy on the SMs that hold two CTAs.
#pragma once

#include "kla_fwd.cuh"

namespace kla {

constexpr int kBwdStages = 3;  // input stages in flight
#ifndef KLA_REV_UNROLL
#define KLA_REV_UNROLL 2
#endif
constexpr int kRevUnroll = KLA_REV_UNROLL;  // steps of the reverse walk unrolled per loop trip
#ifndef KLA_REP_UNROLL
#define KLA_REP_UNROLL 4
#endif
constexpr int kRepUnroll = KLA_REP_UNROLL;  // steps of the replay unrolled per loop trip

// Registers per thread of the three warp groups after the kernel's start. The kernel is compiled for
// kBwdRegsLaunch registers (384 threads, two CTAs per SM); the groups then hand registers to one another:
// 128 * (reverse + replay + helpers) must not exceed 384 * the compiled count, which the launcher checks
// against the compiled kernel before it launches (a group that asked for more than is there would wait for ever).
constexpr int kBwdRegsLaunch = 80;
#ifndef KLA_BWD_REGS_REVERSE
#define KLA_BWD_REGS_REVERSE 128
#endif
#ifndef KLA_BWD_REGS_REPLAY
#define KLA_BWD_REGS_REPLAY 64
#endif
constexpr int kBwdRegsReverse = KLA_BWD_REGS_REVERSE, kBwdRegsReplay = KLA_BWD_REGS_REPLAY;
constexpr int kBwdRegsHelper = 3 * kBwdRegsLaunch - kBwdRegsReverse - kBwdRegsReplay;
static_assert(kBwdRegsHelper >= 24 && kBwdRegsHelper % 8 == 0 && kBwdRegsReverse % 8 == 0 && kBwdRegsReplay % 8 == 0,
              "register counts are multiples of 8, at least 24");
static_assert(kBwdRegsReplay <= kBwdRegsLaunch && kBwdRegsHelper <= kBwdRegsLaunch && kBwdRegsReverse >= kBwdRegsLaunch,
              "two groups give registers up, one takes them");

template <int R>
__device__ __forceinline__ void regs_grow() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(R));
}
template <int R>
__device__ __forceinline__ void regs_shrink() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(R));
}

struct alignas(64) BwdParams {
    CUtensorMap tm_v, tm_lv, tm_dy, tm_dyv;
    int B, L, M, S, NT;  // NT tiles of kCkptInterval steps = checkpoints per sequence
    int use_tma;
    Tensor3 v, lv, k, q, dy, dyv, dv, dlv;
    const float *a, *p, *lam0, *eta0;
    const float2 *ckpt;
    const float *dlam_fin, *deta_fin;
    float *dk, *dq, *da, *dp, *dlam0, *deta0;
    int vec_dv, vec_dlv;
    // lv holds log-variances (see FwdParams); dlv then receives the gradient with respect to them
    int lv_log_sigma;
    float obs_var_min, obs_var_max;
    WaitCtl wait;
    SegCtl seg;  // hand: five planes [B, M, S]: the two carries and the running sums for da, da2, dp
};

template <typename T, typename TO, int SPT, int LPC, int CH, int NW, int NH, int TT>
struct BwdSmem {
    using Sh = ScanShape<SPT, LPC, CH, NW, NH, TT>;
    static constexpr size_t kBars = 128;
    static constexpr size_t kTileI = ((sizeof(T) * TT * Sh::kMC + 127) / 128) * 128;   // v or lambda_v
    static constexpr size_t kTileO = ((sizeof(TO) * TT * Sh::kMC + 127) / 128) * 128;  // dy or dyvar
    static constexpr size_t kKq = ((sizeof(float2) * TT * Sh::kSPad + 127) / 128) * 128;
    static constexpr size_t kLamF = sizeof(T) == 4 ? 0 : ((sizeof(float) * TT * Sh::kMC + 127) / 128) * 128;  // as in FwdSmem
    static constexpr size_t kIn = 2 * kTileI + 2 * kTileO + kKq + kLamF;
    static constexpr int kRowPad = 4;  // slots; 8 words = the span of LPC lanes' float2 reads
    static constexpr int kRow = Sh::kCompute + kRowPad;
    static constexpr size_t kTraj = ((sizeof(float2) * TT * CH * SPT * kRow + 127) / 128) * 128;  // one of two
    static constexpr size_t kDpart = ((sizeof(float2) * TT * LPC * Sh::kMCP + 127) / 128) * 128;  // one of two
    static constexpr size_t kPost = ((sizeof(float2) * CH * SPT * kRow + 127) / 128) * 128;       // state after the last step
    static constexpr size_t kTotal = kBars + kBwdStages * kIn + 2 * kTraj + 2 * kDpart + kPost;
};

constexpr int kBwdThreads = 384;  // reverse, replay and helper groups of four warps each

// LOGV: lambda_v arrives as a log-variance (BwdParams::lv_log_sigma). A separate instantiation, so that the plain
// kernel does not carry that code.
// SEG: sequences cut into segments (BwdParams::seg, SegCtl), also a separate instantiation: with that code in it the
// unsegmented kernel ran 8 % slower at one CTA per SM.
template <typename T, typename TO, int SPT, int LPC, int CH, int NW, int NH, int TT, bool PRIOR, bool LOGV, bool SEG>
__global__ void __launch_bounds__(kBwdThreads, 2) kla_bwd_kernel(const __grid_constant__ BwdParams prm) {
    using Sh = ScanShape<SPT, LPC, CH, NW, NH, TT>;
    using Sm = BwdSmem<T, TO, SPT, LPC, CH, NW, NH, TT>;
    constexpr int SPAD = Sh::kSPad, MC = Sh::kMC, MCP = Sh::kMCP, NTC = Sh::kCompute;
    constexpr int NS = kBwdStages;
    static_assert(NW == 4 && NH == 4, "three groups of four warps");
    static_assert(TT == kCkptInterval, "one checkpoint per tile");
    constexpr int kProducers = 32, kSummers = (NH - 1) * 32;
    constexpr int kStageUsers = 2 * NW + (NH - 1);  // warps that read an input stage: reverse, replay, summing helpers

    // Declared with its alignment (no run-time rounding of the pointer) so that
    // the compiler keeps every access below in the shared address space.
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t *full_in = reinterpret_cast<uint64_t *>(smem);  // [NS]  loader -> everyone: stage loaded
    uint64_t *empty_in = full_in + NS;                       // [NS]  its readers -> loader: stage no longer read
    uint64_t *traj_full = empty_in + NS;                     // [2]   replay -> reverse: trajectory of a tile written
    uint64_t *part_full = traj_full + 2;                     // [2]   reverse -> summing helpers: partial sums written
    uint64_t *buf_empty = part_full + 2;                     // [2]   summing helpers -> replay: buffer reusable
    static_assert((2 * NS + 6) * sizeof(uint64_t) <= Sm::kBars, "barriers fit their slot");
    unsigned char *in_base = smem + Sm::kBars;
    unsigned char *traj_base = in_base + NS * Sm::kIn;
    unsigned char *dpart_base = traj_base + 2 * Sm::kTraj;
    float2 *post = reinterpret_cast<float2 *>(dpart_base + 2 * Sm::kDpart);                       // [CH*SPT][ROW]
    auto trajbuf = [&](int bf) { return reinterpret_cast<float2 *>(traj_base + bf * Sm::kTraj); };      // [TT*CH*SPT][ROW]
    auto dpartbuf = [&](int bf) { return reinterpret_cast<float2 *>(dpart_base + bf * Sm::kDpart); };   // [TT][LPC][MCP]
    auto vstage = [&](int s) { return reinterpret_cast<T *>(in_base + s * Sm::kIn); };
    auto lstage = [&](int s) { return reinterpret_cast<T *>(in_base + s * Sm::kIn + Sm::kTileI); };
    auto dystage = [&](int s) { return reinterpret_cast<TO *>(in_base + s * Sm::kIn + 2 * Sm::kTileI); };
    auto dyvstage = [&](int s) { return reinterpret_cast<TO *>(in_base + s * Sm::kIn + 2 * Sm::kTileI + Sm::kTileO); };
    auto kqstage = [&](int s) { return reinterpret_cast<float2 *>(in_base + s * Sm::kIn + 2 * Sm::kTileI + 2 * Sm::kTileO); };
    auto lfstage = [&](int s) {
        return reinterpret_cast<float *>(in_base + s * Sm::kIn +
                                         (sizeof(T) == 4 ? Sm::kTileI : 2 * Sm::kTileI + 2 * Sm::kTileO + Sm::kKq));
    };
    constexpr bool pro = LOGV;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // This CTA's sequence and, when sequences are cut into segments, its stretch of it: t_off steps in, L steps long
    // (tiles and steps below count from the start of the stretch; segments are processed last-first).
    SegUnit unit{(int)blockIdx.x, (int)blockIdx.y, 0, 0};
    if constexpr (SEG) {
        unit = seg_assign(prm.seg, true);
        if (unit.seg < 0) return;
    }
    const int b = unit.b;
    const int m_cta = unit.bx * MC;
    const int M = prm.M, S = prm.S;
    const int t_off = SEG ? unit.seg * prm.seg.seg_len : 0, tile_off = t_off / TT;
    const int L = SEG ? min(prm.seg.seg_len, prm.L - t_off) : prm.L;
    const int NT = SEG ? (L + TT - 1) / TT : prm.NT;
    const bool first_seg = !SEG || unit.seg == 0, last_seg = !SEG || unit.seg == prm.seg.nseg - 1;
    const bool has_dyv = prm.dyv.ptr != nullptr;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&full_in[s], kProducers);
            mbar_init(&empty_in[s], kStageUsers);
        }
        for (int bf = 0; bf < 2; ++bf) {
            mbar_init(&traj_full[bf], NW);
            mbar_init(&part_full[bf], NW);
            mbar_init(&buf_empty[bf], NH - 1);
        }
        mbar_fence_init();
    }
    __syncthreads();

    // A trajectory buffer holds one float2 per compute thread for every (step u, channel ci, state i) of a tile:
    // row = (u*CH + ci)*SPT + i, rows of NTC slots padded by kRowPad so that the helpers, whose lanes read
    // different rows at the same column, do not collide on shared-memory banks. The replay thread and the
    // reverse thread with the same index within their groups own the same chains and the same column.
    constexpr int ROW = Sm::kRow;
    auto trow = [&](int u, int ci, int i) { return ((u * CH + ci) * SPT + i) * ROW; };

    if (warp < 2 * NW) {
        // ======================================================= the two compute groups
        const bool is_reverse = warp < NW;
        const int ctid = tid & (NTC - 1);  // index within the group
        const int cwarp = ctid >> 5;
        const int j = lane % LPC, cl = lane / LPC;
        const int cw = cwarp * Sh::kCPW + cl * CH;

        if (!is_reverse) {
            // ----------------------------------------------------------- replay
            regs_shrink<kBwdRegsReplay>();
            float ca[CH][SPT], ca2[CH][SPT], cp[CH][SPT];
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
                }
            }
            // checkpoint of the tile about to be replayed, fetched one tile ahead
            float2 ck[CH][SPT];
            auto load_ck = [&](int tile) {
                const float2 *src = prm.ckpt + (((long long)b * prm.NT + tile_off + tile) * M + (m_cta + cw)) * S + j;
#pragma unroll
                for (int ci = 0; ci < CH; ++ci)
#pragma unroll
                    for (int i = 0; i < SPT; ++i)
                        ck[ci][i] = (m_cta + cw + ci < M && i * LPC + j < S) ? src[ci * S + i * LPC] : make_float2(1.0f, 0.0f);
            };
            if (NT > 0) load_ck(NT - 1);

            for (int ti = 0; ti < NT; ++ti) {
                const int tile = NT - 1 - ti, s = ti % NS, bf = ti & 1;
                const int n = min(TT, L - tile * TT);
                if (!mbar_wait(prm.wait, &full_in[s], (ti / NS) & 1, 11)) break;
                if (pro) {  // this warp's channels of the tile: log-variance -> precision, float32
                    const T *raw = lstage(s) + cwarp * Sh::kCPW;
                    float *lf = lfstage(s) + cwarp * Sh::kCPW;
                    for (int e = lane; e < TT * Sh::kCPW; e += 32) {
                        const int at = (e / Sh::kCPW) * MC + e % Sh::kCPW;
                        lf[at] = precision_from_log_variance_fast(to_f32<T>(raw[at]), prm.obs_var_min, prm.obs_var_max);
                    }
                    fence_proxy_async();  // these plain stores are ordered before the bulk copy that refills the stage
                    __syncwarp();
                }
                const T *lrow = lstage(s) + cw;
                const float *lfrow = lfstage(s) + cw;
                const T *vrow = vstage(s) + cw;
                const float2 *kqrow = kqstage(s) + j;
                float2 *traj = trajbuf(bf);
                float P[CH][SPT], mean[CH][SPT];
#pragma unroll
                for (int ci = 0; ci < CH; ++ci)
#pragma unroll
                    for (int i = 0; i < SPT; ++i) {
                        P[ci][i] = ck[ci][i].x;
                        mean[ci][i] = ck[ci][i].y;
                    }
                if (tile > 0) load_ck(tile - 1);
                // the buffer still holds the partial sums of the tile before last until the helpers have consumed them
                if (ti >= 2 && !mbar_wait(prm.wait, &buf_empty[bf], (ti / 2 - 1) & 1, 12)) break;

                auto replay_step = [&](int u) {
                    float lv[CH], vv[CH], Pp[CH][SPT], g[CH][SPT], r[CH][SPT];
#pragma unroll
                    for (int ci = 0; ci < CH; ++ci) {
                        if constexpr (sizeof(T) == 4) lv[ci] = lfrow[u * MC + ci];  // the same tile as lrow
                        else lv[ci] = pro ? lfrow[u * MC + ci] : to_f32<T>(lrow[u * MC + ci]);
                        vv[ci] = to_f32<T>(vrow[u * MC + ci]);
                    }
#pragma unroll
                    for (int i = 0; i < SPT; ++i) {
                        const float kk = kqrow[u * SPAD + i * LPC].x;
#pragma unroll
                        for (int ci = 0; ci < CH; ++ci) {
                            traj[trow(u, ci, i) + ctid] = make_float2(P[ci][i], mean[ci][i]);
                            float phi;
                            chain_inputs(lv[ci], vv[ci], kk, phi, r[ci][i]);
                            g[ci][i] = chain_denominator(P[ci][i], phi, ca2[ci][i], cp[ci][i], Pp[ci][i]);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < SPT; ++i)
#pragma unroll
                        for (int ci = 0; ci < CH; ++ci) g[ci][i] = rcp_approx(g[ci][i]);
#pragma unroll
                    for (int i = 0; i < SPT; ++i)
#pragma unroll
                        for (int ci = 0; ci < CH; ++ci)
                            chain_update(P[ci][i], mean[ci][i], Pp[ci][i], g[ci][i], r[ci][i], ca[ci][i]);
                };
                if (n == TT) {
#pragma unroll 1
                    for (int h = 0; h < TT; h += kRepUnroll) {
#pragma unroll
                        for (int u = 0; u < kRepUnroll; ++u) replay_step(h + u);
                    }
                } else {
#pragma unroll 1
                    for (int u = 0; u < n; ++u) replay_step(u);
                }
                if (ti == 0) {  // the state after the sequence's last step: where the reverse walk starts
#pragma unroll
                    for (int ci = 0; ci < CH; ++ci)
#pragma unroll
                        for (int i = 0; i < SPT; ++i) post[(ci * SPT + i) * ROW + ctid] = make_float2(P[ci][i], mean[ci][i]);
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&traj_full[bf]);
                    mbar_arrive(&empty_in[s]);
                }
            }
        } else {
            // ---------------------------------------------------------- reverse
            regs_grow<kBwdRegsReverse>();
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

            for (int ti = 0; ti < NT; ++ti) {
                const int tile = NT - 1 - ti, s = ti % NS, bf = ti & 1;
                const int n = min(TT, L - tile * TT);
                if (!mbar_wait(prm.wait, &traj_full[bf], (ti / 2) & 1, 17)) break;
                if (!mbar_wait(prm.wait, &full_in[s], (ti / NS) & 1, 18)) break;
                const T *lrow = lstage(s) + cw;
                const float *lfrow = lfstage(s) + cw;
                const T *vrow = vstage(s) + cw;
                const TO *dyrow = dystage(s) + cw;
                const TO *dyvrow = dyvstage(s) + cw;
                const float2 *kqrow = kqstage(s) + j;
                float2 *traj = trajbuf(bf);
                float2 *dpart = dpartbuf(bf);

                if (ti == 0) {
                    // The walk starts from the state after the stretch's last step; at the end of the sequence the
                    // carries are seeded from the gradient of the returned state: lam_fin = 1/P, eta_fin = mean/P,
                    // at the end of an inner segment they and the running sums come from the segment after it.
                    bool carried = true;
                    if (!last_seg) carried = seg_wait(prm.wait, prm.seg.done + unit.seq, prm.seg.nseg - 1 - unit.seg, 19);
                    if (!carried) break;
                    const long long plane = (long long)prm.B * M * S;
#pragma unroll
                    for (int ci = 0; ci < CH; ++ci) {
                        const int m = m_cta + cw + ci;
#pragma unroll
                        for (int i = 0; i < SPT; ++i) {
                            const int st = i * LPC + j;
                            const float2 fin = post[(ci * SPT + i) * ROW + ctid];
                            Pn[ci][i] = fin.x;
                            mn[ci][i] = fin.y;
                            if (!last_seg) {
                                if (m < M && st < S) {
                                    const float *h = prm.seg.hand + ((long long)b * M + m) * S + st;
                                    cP[ci][i] = __ldcg(h);
                                    cm[ci][i] = __ldcg(h + plane);
                                    accA[ci][i] = __ldcg(h + 2 * plane);
                                    accA2[ci][i] = __ldcg(h + 3 * plane);
                                    accP[ci][i] = __ldcg(h + 4 * plane);
                                }
                            } else if (prm.dlam_fin != nullptr && m < M && st < S) {
                                const float Lb = prm.dlam_fin[((long long)b * M + m) * S + st];
                                const float Eb = prm.deta_fin[((long long)b * M + m) * S + st];
                                const float lam = 1.0f / fin.x;
                                const float eta = fin.y * lam;
                                cm[ci][i] = Eb * lam;
                                cP[ci][i] = -lam * (lam * Lb + eta * Eb);
                            }
                        }
                    }
                }

                auto reverse_step = [&](int u) {
                    float lv[CH], lv2[CH], vv[CH], vl[CH], dy[CH], dyv[CH], dyv2[CH], dvl[CH], dlphi[CH];
#pragma unroll
                    for (int ci = 0; ci < CH; ++ci) {
                        if constexpr (sizeof(T) == 4) lv[ci] = lfrow[u * MC + ci];
                        else lv[ci] = pro ? lfrow[u * MC + ci] : to_f32<T>(lrow[u * MC + ci]);
                        vv[ci] = to_f32<T>(vrow[u * MC + ci]);
                        dy[ci] = to_f32<TO>(dyrow[u * MC + ci]);
                        dyv[ci] = to_f32<TO>(dyvrow[u * MC + ci]);
                        vl[ci] = vv[ci] * lv[ci];
                        lv2[ci] = lv[ci] + lv[ci];
                        dyv2[ci] = dyv[ci] + dyv[ci];
                        dvl[ci] = 0.0f;
                        dlphi[ci] = 0.0f;
                    }
                    float2 prev[CH][SPT];
                    float4 c[SPT];  // k^2, k, q, q^2
                    float g[CH][SPT], Pp[CH][SPT], phi[CH][SPT], r[CH][SPT];
#pragma unroll
                    for (int i = 0; i < SPT; ++i) {
                        // (k, q) from shared memory, the squares formed here: shared-memory bandwidth, not arithmetic,
                        // is what this kernel runs out of
                        const float2 kq2 = kqrow[u * SPAD + i * LPC];
                        c[i] = make_float4(kq2.x * kq2.x, kq2.x, kq2.y, kq2.y * kq2.y);
#pragma unroll
                        for (int ci = 0; ci < CH; ++ci) {
                            prev[ci][i] = traj[trow(u, ci, i) + ctid];  // P', mean'
                            chain_inputs(lv[ci], vv[ci], c[i].y, phi[ci][i], r[ci][i]);
                            g[ci][i] = chain_denominator(prev[ci][i].x, phi[ci][i], ca2[ci][i], cp[ci][i], Pp[ci][i]);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < SPT; ++i)
#pragma unroll
                        for (int ci = 0; ci < CH; ++ci) g[ci][i] = rcp_approx(g[ci][i]);
#pragma unroll
                    for (int i = 0; i < SPT; ++i) {
                        float X2 = 0.0f, Y = 0.0f, A_ = 0.0f, B2 = 0.0f;
#pragma unroll
                        for (int ci = 0; ci < CH; ++ci) {
                            const float a = ca[ci][i], a2 = ca2[ci][i], p = cp[ci][i];
                            const float gg = g[ci][i];
                            float mbar, Pbar;
                            if (PRIOR) {  // y reads a*mean and a2*P + p
                                const float mob = dy[ci] * c[i].z, vob = dyv[ci] * c[i].w;
                                mbar = fmaf(mob, a, cm[ci][i]);
                                Pbar = fmaf(vob, a2, cP[ci][i]);
                                accA[ci][i] = fmaf(mob, mn[ci][i], accA[ci][i]);
                                accA2[ci][i] = fmaf(vob, Pn[ci][i], accA2[ci][i]);
                                accP[ci][i] += vob;
                                A_ = fmaf(dy[ci], a * mn[ci][i], A_);
                                B2 = fmaf(dyv2[ci], fmaf(a2, Pn[ci][i], p), B2);
                            } else {
                                mbar = fmaf(dy[ci], c[i].z, cm[ci][i]);
                                Pbar = fmaf(dyv[ci], c[i].w, cP[ci][i]);
                                A_ = fmaf(dy[ci], mn[ci][i], A_);
                                B2 = fmaf(dyv2[ci], Pn[ci][i], B2);
                            }
                            const float t2 = fmaf(Pbar, Pn[ci][i], mbar * mn[ci][i]);
                            const float dbar = -(gg * t2);
                            const float ubar = mbar * gg;
                            const float Ppbar = fmaf(dbar, phi[ci][i], fmaf(Pbar, gg, ubar * r[ci][i]));
                            const float rbar = ubar * Pp[ci][i];
                            const float phibar = dbar * Pp[ci][i];
                            cm[ci][i] = ubar * a;
                            cP[ci][i] = Ppbar * a2;
                            accA[ci][i] = fmaf(ubar, prev[ci][i].y, accA[ci][i]);
                            accA2[ci][i] = fmaf(Ppbar, prev[ci][i].x, accA2[ci][i]);
                            accP[ci][i] += Ppbar;
                            dlphi[ci] = fmaf(phibar, c[i].x, dlphi[ci]);
                            dvl[ci] = fmaf(rbar, c[i].y, dvl[ci]);
                            X2 = fmaf(phibar, lv2[ci], X2);
                            Y = fmaf(rbar, vl[ci], Y);
                            Pn[ci][i] = prev[ci][i].x;
                            mn[ci][i] = prev[ci][i].y;
                        }
                        // this thread's share of dk, dq for (t, s): parked where (P', mean') was
                        traj[trow(u, 0, i) + ctid] = make_float2(fmaf(c[i].y, X2, Y), fmaf(c[i].z, B2, A_));
                    }
                    // this thread's share of the sums over s
#pragma unroll
                    for (int ci = 0; ci < CH; ++ci) dpart[(u * LPC + j) * MCP + cw + ci] = make_float2(dvl[ci], dlphi[ci]);
                };
                if (n == TT) {
                    // unrolled by kRevUnroll steps, not the whole tile: the walk's code then stays within the instruction cache
#pragma unroll 1
                    for (int h = TT - kRevUnroll; h >= 0; h -= kRevUnroll) {
#pragma unroll
                        for (int u = kRevUnroll - 1; u >= 0; --u) reverse_step(h + u);
                    }
                } else {
#pragma unroll 1
                    for (int u = n - 1; u >= 0; --u) reverse_step(u);
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&part_full[bf]);
                    mbar_arrive(&empty_in[s]);
                }
            }

            if (!first_seg) {
                // ---- start of an inner segment: hand the carries and the running sums to the segment before it
                const long long plane = (long long)prm.B * M * S;
#pragma unroll
                for (int ci = 0; ci < CH; ++ci) {
                    const int m = m_cta + cw + ci;
#pragma unroll
                    for (int i = 0; i < SPT; ++i) {
                        const int st = i * LPC + j;
                        if (m < M && st < S) {
                            float *h = prm.seg.hand + ((long long)b * M + m) * S + st;
                            __stcg(h, cP[ci][i]);
                            __stcg(h + plane, cm[ci][i]);
                            __stcg(h + 2 * plane, accA[ci][i]);
                            __stcg(h + 3 * plane, accA2[ci][i]);
                            __stcg(h + 4 * plane, accP[ci][i]);
                        }
                    }
                }
                __threadfence();
                group_barrier_128();
                if (tid == 0) st_release_gpu(prm.seg.done + unit.seq, prm.seg.nseg - unit.seg);
            }
            // ---- start of the sequence: gradients of a, p and of the carried-in state
#pragma unroll
            for (int ci = 0; ci < CH; ++ci) {
                const int m = m_cta + cw + ci;
#pragma unroll
                for (int i = 0; i < SPT; ++i) {
                    const int st = i * LPC + j;
                    if (first_seg && m < M && st < S) {
                        const long long ms = (long long)m * S + st, bms = ((long long)b * M + m) * S + st;
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
    } else {
        // ================================================================ helpers
        regs_shrink<kBwdRegsHelper>();
        const int htid = tid - 2 * NTC;
        const int hlane = htid & 31;
        constexpr uint32_t kBytesI = sizeof(T) * TT * MC, kBytesO = sizeof(TO) * TT * MC;
        int produced = 0;
        bool ok = true;

        if (htid < kProducers) {
            // ---- loader: TMA tiles of v, lambda_v, dy, dy_var and (k, q), NS tiles ahead
            const T *vb = static_cast<const T *>(prm.v.ptr) + (long long)b * prm.v.sb + (long long)t_off * prm.v.st;
            const T *lb = static_cast<const T *>(prm.lv.ptr) + (long long)b * prm.lv.sb + (long long)t_off * prm.lv.st;
            const T *kb = static_cast<const T *>(prm.k.ptr) + (long long)b * prm.k.sb + (long long)t_off * prm.k.st;
            const T *qb = static_cast<const T *>(prm.q.ptr) + (long long)b * prm.q.sb + (long long)t_off * prm.q.st;
            const TO *dyb = static_cast<const TO *>(prm.dy.ptr) + (long long)b * prm.dy.sb + (long long)t_off * prm.dy.st;
            const TO *dyvb = has_dyv ? static_cast<const TO *>(prm.dyv.ptr) + (long long)b * prm.dyv.sb + (long long)t_off * prm.dyv.st : nullptr;
            if (!has_dyv) {  // dyvar absent: its stage buffers stay zero for the whole kernel
                for (int s = 0; s < NS; ++s)
                    for (int idx = htid; idx < TT * MC; idx += kProducers) dyvstage(s)[idx] = from_f32<TO>(0.0f);
            }
            // (k, q) of the next tile are fetched into registers while the current one
            // is handed over, so the loader never sits on a global-memory latency
            constexpr int KQP = (TT * SPAD + kProducers - 1) / kProducers;
            float kr[KQP], qr[KQP];
            auto load_kq = [&](int t0) {
#pragma unroll
                for (int e = 0; e < KQP; ++e) {
                    const int idx = htid + e * kProducers, row = idx / SPAD, sidx = idx % SPAD;
                    const bool in = idx < TT * SPAD && sidx < S && t0 + row < L;
                    kr[e] = in ? to_f32<T>(kb[(long long)(t0 + row) * prm.k.st + sidx]) : 0.0f;
                    qr[e] = in ? to_f32<T>(qb[(long long)(t0 + row) * prm.q.st + sidx]) : 0.0f;
                }
            };
            if (NT > 0) load_kq((NT - 1) * TT);
            for (int it = 0; it < NT; ++it) {
                const int tile = NT - 1 - it, s = it % NS, t0 = tile * TT;
                // the stage is free once the compute groups and the summing helpers are done with it
                if (it >= NS && !mbar_wait(prm.wait, &empty_in[s], (it / NS - 1) & 1, 13, 100)) { ok = false; break; }
                if (prm.use_tma) {
                    if (htid == 0) {
                        mbar_arrive_expect_tx(&full_in[s], 2 * kBytesI + (has_dyv ? 2 : 1) * kBytesO);
                        tma_load_3d(vstage(s), &prm.tm_v, m_cta, t_off + t0, b, &full_in[s]);
                        tma_load_3d(lstage(s), &prm.tm_lv, m_cta, t_off + t0, b, &full_in[s]);
                        tma_load_3d(dystage(s), &prm.tm_dy, m_cta, t_off + t0, b, &full_in[s]);
                        if (has_dyv) tma_load_3d(dyvstage(s), &prm.tm_dyv, m_cta, t_off + t0, b, &full_in[s]);
                    }
                } else {
                    stage_tile_plain<T, TT, MC, kProducers>(vstage(s), vb, prm.v.st, t0, L, m_cta, M, htid);
                    stage_tile_plain<T, TT, MC, kProducers>(lstage(s), lb, prm.lv.st, t0, L, m_cta, M, htid);
                    stage_tile_plain<TO, TT, MC, kProducers>(dystage(s), dyb, prm.dy.st, t0, L, m_cta, M, htid);
                    if (has_dyv)
                        stage_tile_plain<TO, TT, MC, kProducers>(dyvstage(s), dyvb, prm.dyv.st, t0, L, m_cta, M, htid);
                }
                float2 *kq = kqstage(s);
#pragma unroll
                for (int e = 0; e < KQP; ++e) {
                    const int idx = htid + e * kProducers;
                    if (idx < TT * SPAD) kq[idx] = make_float2(kr[e], qr[e]);
                }
                if (tile > 0) load_kq(t0 - TT);
                // (test hook, as in the forward: the wait for tile skip_tile runs out)
                if (!(prm.use_tma && htid == 0) && !(it == prm.wait.skip_tile && htid == 1)) mbar_arrive(&full_in[s]);
                produced = it + 1;
            }
        } else {
            // ---- summing helpers: finish the sums of each processed tile
            const int ctid = htid - kProducers;
            T *dvb = static_cast<T *>(prm.dv.ptr) + (long long)b * prm.dv.sb + (long long)t_off * prm.dv.st;
            T *dlvb = static_cast<T *>(prm.dlv.ptr) + (long long)b * prm.dlv.sb + (long long)t_off * prm.dlv.st;
            for (int jt = 0; jt < NT; ++jt) {
                const int tile = NT - 1 - jt, s = jt % NS, t0 = tile * TT, bf = jt & 1;
                const int n = min(TT, L - t0);
                const T *lt = lstage(s), *vt = vstage(s);
                const float *lft = lfstage(s);
                const float2 *traj = trajbuf(bf);
                const float2 *dpart = dpartbuf(bf);
                if (!mbar_wait(prm.wait, &part_full[bf], (jt / 2) & 1, 14, 100)) break;
                // dk, dq: add the CTA's channels. Compute thread t holds lane group j = t % LPC, so the partials
                // of state s = i*LPC + jj sit at columns jj, jj + LPC, ... of row (u, i).
                for (int pidx = ctid; pidx < TT * SPAD; pidx += kSummers) {
                    const int jj = pidx % LPC, row = pidx / LPC;  // row = (step, i)
                    const int u = row / SPT, i = row % SPT;
                    const int st = i * LPC + jj;
                    const float2 *src = traj + trow(u, 0, i) + jj;
                    float sk0 = 0.0f, sq0 = 0.0f, sk1 = 0.0f, sq1 = 0.0f;
#pragma unroll
                    for (int c = 0; c < NTC / LPC; c += 2) {
                        const float2 x0 = src[c * LPC], x1 = src[(c + 1) * LPC];
                        sk0 += x0.x; sq0 += x0.y;
                        sk1 += x1.x; sq1 += x1.y;
                    }
                    if (st < S && u < n) {
                        atomicAdd(prm.dk + ((long long)b * prm.L + t_off + t0 + u) * S + st, sk0 + sk1);
                        atomicAdd(prm.dq + ((long long)b * prm.L + t_off + t0 + u) * S + st, sq0 + sq1);
                    }
                }
                // dv, dlambda_v: add the lane groups. v enters only through v*lambda_v (kla_ops.py:177): with
                // D = sum_s rbar k, dv = D lambda_v and dlambda_v = sum_s phibar k^2 + D v.
                // (threads taken from the other end, so the two loops spread over the warps)
                for (int uidx = kSummers - 1 - ctid; uidx < TT * (MC / 2); uidx += kSummers) {
                    const int u = uidx / (MC / 2), c = (uidx % (MC / 2)) * 2;
                    if (u >= n || m_cta + c >= M) continue;
                    float ax = 0.0f, ay = 0.0f, bx = 0.0f, by = 0.0f;
#pragma unroll
                    for (int jj = 0; jj < LPC; ++jj) {
                        const float4 x = *reinterpret_cast<const float4 *>(dpart + (u * LPC + jj) * MCP + c);
                        ax += x.x; ay += x.y; bx += x.z; by += x.w;
                    }
                    float l0, l1;
                    if (pro || sizeof(T) == 4) {
                        l0 = lft[u * MC + c];
                        l1 = lft[u * MC + c + 1];
                    } else {
                        l0 = to_f32<T>(lt[u * MC + c]);
                        l1 = to_f32<T>(lt[u * MC + c + 1]);
                    }
                    const float v0 = to_f32<T>(vt[u * MC + c]), v1 = to_f32<T>(vt[u * MC + c + 1]);
                    const float dv0 = ax * l0, dv1 = bx * l1;
                    float dl0 = fmaf(ax, v0, ay), dl1 = fmaf(bx, v1, by);
                    if (pro) {  // chain through Lambda_v = 1 / min(softplus(x) + floor, ceiling)
                        dl0 *= precision_slope(l0, prm.obs_var_min, prm.obs_var_max);
                        dl1 *= precision_slope(l1, prm.obs_var_min, prm.obs_var_max);
                    }
                    T *p0 = dvb + (long long)(t0 + u) * prm.dv.st + m_cta + c;
                    T *p1 = dlvb + (long long)(t0 + u) * prm.dlv.st + m_cta + c;
                    const bool full = m_cta + c + 1 < M;
                    if (full && prm.vec_dv) {
                        if constexpr (sizeof(T) == 4) *reinterpret_cast<float2 *>(p0) = make_float2(dv0, dv1);
                        else *reinterpret_cast<__nv_bfloat162 *>(p0) = __floats2bfloat162_rn(dv0, dv1);
                    } else {
                        p0[0] = from_f32<T>(dv0);
                        if (full) p0[1] = from_f32<T>(dv1);
                    }
                    if (full && prm.vec_dlv) {
                        if constexpr (sizeof(T) == 4) *reinterpret_cast<float2 *>(p1) = make_float2(dl0, dl1);
                        else *reinterpret_cast<__nv_bfloat162 *>(p1) = __floats2bfloat162_rn(dl0, dl1);
                    } else {
                        p1[0] = from_f32<T>(dl0);
                        if (full) p1[1] = from_f32<T>(dl1);
                    }
                }
                __syncwarp();
                if (hlane == 0) {
                    mbar_arrive(&buf_empty[bf]);
                    mbar_arrive(&empty_in[s]);
                }
            }
        }
        if (!ok && prm.use_tma && htid == 0) {
            for (int t = max(0, produced - NS); t < produced; ++t) mbar_wait(prm.wait, &full_in[t % NS], (t / NS) & 1, 15);
        }
    }
}

}  // namespace kla
