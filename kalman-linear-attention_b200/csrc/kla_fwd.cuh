// Fused forward scan kernel: lambda_v, v, k, q -> y, y_var, final state, and
// (for training) a checkpoint of every chain's state once per checkpoint
// interval.
//
// Nothing of shape [B, L, M, S] is ever written: phi, r, the gain, the
// posterior and the read-out all live in registers. Per token the kernel reads
// v, lambda_v (2M) and k, q (2S, once per CTA of MC channels) and writes y,
// y_var (2M).
//
// The CTA is split into NW compute warps and NH helper warps.
//   compute warps  run the recurrence only. A thread owns SPT states of one
//                  channel and works on them two at a time with the paired
//                  fp32 instructions of sm_100 (kla_common.cuh). Per step it
//                  reads its inputs from a shared-memory stage and leaves its
//                  share of the read-out sums in shared memory. The time loop
//                  is software-pipelined by hand (see below).
//   loader warps   (the first NH/2 helpers) feed them: TMA tile loads of v and
//                  lambda_v issued by one elected thread, and the (k, q) values
//                  of a tile regrouped by owning lane; k, q of the next tile are
//                  already in registers when a stage becomes free.
//   drainer warps  (the other helpers) finish a tile: they add the LPC partial
//                  read-outs of every (step, channel) and store y, y_var.
// Stages are handed over with mbarriers, so the compute warps see neither
// global-memory latency nor a CTA-wide barrier inside the time loop.
// With SEG a sequence is walked by several CTAs one after the other (SegCtl,
// kla_common.cuh); the filter state travels between them as it is in registers,
// so the results are those of one CTA walking the whole sequence.
#pragma once

#include "kla_common.cuh"

namespace kla {

constexpr int kInStages = 3;   // input stages in flight
constexpr int kOutStages = 2;  // read-out partial buffers
constexpr int kEpiStages = 3;  // tiles of the epilogue operands (z, gate) in flight, as deep as the inputs
#ifndef KLA_FWD_UNROLL
#define KLA_FWD_UNROLL 16
#endif
constexpr int kFwdUnroll = KLA_FWD_UNROLL;  // steps unrolled per trip of the time loop

struct alignas(64) FwdParams {
    CUtensorMap tm_v, tm_lv;  // rank-3 (M, L, B) maps with box (MC, TT, 1); valid when use_tma
    int B, L, M, S, NT;  // NT tiles of TT steps
    int NC;              // checkpoints per sequence: one per kCkptInterval steps
    int use_tma;
    Tensor3 v, lv, k, q, y, yv;
    const float *a, *p, *lam0, *eta0;
    float *lam_fin, *eta_fin;
    float2 *ckpt;  // [B, NC, M, S] (P, mean) before every kCkptInterval-th step, or nullptr
    int vec_y, vec_yv;
    // lv holds the sensor projection's raw log-variance output instead of the precision:
    // Lambda_v = 1 / min(softplus(lv) + obs_var_min, obs_var_max) is formed in shared memory by the compute warps,
    // each for the channels it owns, when a tile arrives
    int lv_log_sigma;
    float obs_var_min, obs_var_max;
    // Forward-only epilogue of the layer (src/kla/layers/kla_layer.py:329-338), applied by the drainer warps at the
    // store: y += skip * z, then y *= g and y_var *= g^2 with g = act(gate). z / gate: [B, L, M] in the activation
    // type, ptr == nullptr when absent; skip: one value or one per channel.
    Tensor3 z, gate;
    const float *skip;
    // Training with the epilogue: the drainers also store the scan's own y, y_var (before skip and gate), which the
    // epilogue's adjoint needs; ptr == nullptr when no backward will follow.
    Tensor3 y_raw, yv_raw;
    int skip_len, gate_act, epilogue, epi_tma;
    WaitCtl wait;
    SegCtl seg;  // hand: one plane pair (P, mean) as float2 [B, M, S]
    alignas(64) CUtensorMap tm_z, tm_gate;  // maps of the epilogue operands, like tm_v; valid when epi_tma
};

// Shared-memory carve-up, shared by the kernel and the launcher.
template <typename T, int SPT, int LPC, int CH, int NW, int NH, int TT>
struct FwdSmem {
    using Sh = ScanShape<SPT, LPC, CH, NW, NH, TT>;
    static constexpr size_t kBars = 128;
    static constexpr size_t kTile = ((sizeof(T) * TT * Sh::kMC + 127) / 128) * 128;   // one of v / lambda_v
    static constexpr size_t kKq = ((sizeof(float2) * TT * Sh::kSPad + 127) / 128) * 128;
    // float32 precision tile written by the compute warps when lambda_v arrives as a log-variance;
    // for float32 activations it is the lambda_v tile itself (transformed in place)
    static constexpr size_t kLamF = sizeof(T) == 4 ? 0 : ((sizeof(float) * TT * Sh::kMC + 127) / 128) * 128;
    static constexpr size_t kIn = 2 * kTile + kKq + kLamF;
    static constexpr size_t kOut = ((sizeof(float2) * TT * LPC * Sh::kMCP + 127) / 128) * 128;
    static constexpr size_t kPlain = kBars + kInStages * kIn + kOutStages * kOut;  // without an epilogue
    static constexpr size_t kEpi = 2 * kTile;                                      // one z and one gate tile
    static constexpr size_t kTotal = kPlain + kEpiStages * kEpi;                   // epilogue stages sit at the end
};

// EPI: the forward-only layer epilogue (FwdParams::epilogue). A separate instantiation, so that the plain
// kernel does not carry that code: even untaken it costs the plain path a few per cent.
// SEG: sequences cut into segments (FwdParams::seg, SegCtl). Again a separate instantiation: the unsegmented kernel
// then carries none of that code (with it, one CTA per SM ran 3 % slower).
template <typename T, typename TO, int SPT, int LPC, int CH, int NW, int NH, int TT, bool PRIOR, bool EPI, bool SEG>
__global__ void __launch_bounds__((NW + NH) * 32) kla_fwd_kernel(const __grid_constant__ FwdParams prm) {
    using Sh = ScanShape<SPT, LPC, CH, NW, NH, TT>;
    using Sm = FwdSmem<T, SPT, LPC, CH, NW, NH, TT>;
    constexpr int SPAD = Sh::kSPad, MC = Sh::kMC, MCP = Sh::kMCP;
    constexpr int NS = kInStages, NO = kOutStages;
    constexpr int HP = SPT / 2;  // pairs of states per thread
    static_assert(SPT % 2 == 0, "states are processed in pairs");
    // helper warps split by task: the first NH/2 load and stage inputs, the others sum and store outputs
    // With the epilogue the drainers carry the heavier load (activation, skip, second store): three drainer warps
    // and one loader warp there, where that keeps a drainer thread on one channel pair from tile to tile.
    constexpr bool kWideDrain = EPI && NH == 4 && (3 * 32) % (MC / 2) == 0;
    constexpr int kProducers = kWideDrain ? 32 : (NH / 2) * 32, kDrainers = Sh::kHelpers - kProducers;
    static_assert(NH >= 2, "one loading and one storing helper warp at least");
    static_assert(TT % kCkptInterval == 0, "checkpoints fall on fixed steps of a tile");

    // Declared with its alignment (no run-time rounding of the pointer) so that
    // the compiler keeps every access below in the shared address space.
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t *full_in = reinterpret_cast<uint64_t *>(smem);  // [NS]
    uint64_t *empty_in = full_in + NS;                       // [NS]
    uint64_t *full_out = empty_in + NS;                      // [NO]
    uint64_t *empty_out = full_out + NO;                     // [NO]
    constexpr int NE = kEpiStages;
    uint64_t *epi_full = empty_out + NO;                     // [NE]  loaders -> drainers: z, gate tiles loaded
    uint64_t *epi_empty = epi_full + NE;                     // [NE]  drainers -> loaders: tiles consumed
    static_assert((2 * NS + 2 * NO + 2 * NE) * sizeof(uint64_t) <= Sm::kBars, "barriers fit their slot");
    unsigned char *in_base = smem + Sm::kBars;
    unsigned char *out_base = in_base + NS * Sm::kIn;
    unsigned char *epi_base = smem + Sm::kPlain;  // only there when the kernel was launched with an epilogue
    auto zstage = [&](int e) { return reinterpret_cast<T *>(epi_base + e * Sm::kEpi); };
    auto gstage = [&](int e) { return reinterpret_cast<T *>(epi_base + e * Sm::kEpi + Sm::kTile); };
    auto vstage = [&](int s) { return reinterpret_cast<T *>(in_base + s * Sm::kIn); };
    auto lstage = [&](int s) { return reinterpret_cast<T *>(in_base + s * Sm::kIn + Sm::kTile); };
    // (k, q) of a step, grouped by owning lane: [TT][LPC][2][SPT] floats, state s = i * LPC + j at [j][.][i]
    auto kqstage = [&](int s) { return reinterpret_cast<float *>(in_base + s * Sm::kIn + 2 * Sm::kTile); };
    auto lfstage = [&](int s) {
        return reinterpret_cast<float *>(in_base + s * Sm::kIn + (sizeof(T) == 4 ? Sm::kTile : 2 * Sm::kTile + Sm::kKq));
    };
    const bool pro = prm.lv_log_sigma != 0;
    auto ystage = [&](int o) { return reinterpret_cast<float2 *>(out_base + o * Sm::kOut); };

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // This CTA's sequence and, when sequences are cut into segments, its stretch of it: t_off steps in, L steps long
    // (everything below counts tiles and steps from the start of the stretch).
    SegUnit unit{(int)blockIdx.x, (int)blockIdx.y, 0, 0};
    if constexpr (SEG) {
        unit = seg_assign(prm.seg, false);
        if (unit.seg < 0) return;
    }
    const int b = unit.b;
    const int m_cta = unit.bx * MC;
    const int M = prm.M, S = prm.S;
    const int t_off = SEG ? unit.seg * prm.seg.seg_len : 0;
    const int L = SEG ? min(prm.seg.seg_len, prm.L - t_off) : prm.L;
    const int NT = SEG ? (L + TT - 1) / TT : prm.NT;
    const bool first_seg = !SEG || unit.seg == 0, last_seg = !SEG || unit.seg == prm.seg.nseg - 1;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&full_in[s], kProducers);
            mbar_init(&empty_in[s], NW);
        }
        for (int o = 0; o < NO; ++o) {
            mbar_init(&full_out[o], NW);
            mbar_init(&empty_out[o], kDrainers / 32);
        }
        if constexpr (EPI) {
            for (int e = 0; e < NE; ++e) {
                mbar_init(&epi_full[e], kProducers);
                mbar_init(&epi_empty[e], kDrainers / 32);
            }
        }
        mbar_fence_init();
    }
    __syncthreads();

    if (warp < NW) {
        // =============================================================== compute
        const int j = lane % LPC, cl = lane / LPC;
        const int cw = warp * Sh::kCPW + cl * CH;  // first channel of this thread, CTA-relative

        // Per-chain constants and state, held as pairs of chains (states i = 2h and
        // 2h + 1) so that the arithmetic below runs on the paired fp32
        // instructions. Padding chains (s >= S or m >= M) get a = 0, p = 1, so
        // their variance sits at 1 and their mean at 0.
        float2 ca[CH][HP], ca2[CH][HP], cp[CH][HP], P[CH][HP], mean[CH][HP];
#pragma unroll
        for (int ci = 0; ci < CH; ++ci) {
            const int m = m_cta + cw + ci;
#pragma unroll
            for (int i = 0; i < SPT; ++i) {
                const int s = i * LPC + j;
                const bool live = (m < M) && (s < S);
                const float av = live ? prm.a[(long long)m * S + s] : 0.0f;
                const float pv = live ? prm.p[(long long)m * S + s] : 1.0f;
                pair_el(ca[ci], i) = av;
                pair_el(ca2[ci], i) = live ? fmaxf(av * av, kEps) : 0.0f;
                pair_el(cp[ci], i) = fmaxf(pv, kPMin);
                float lam = 1.0f, eta = 0.0f;
                if (live && prm.lam0 != nullptr) {
                    lam = prm.lam0[((long long)b * M + m) * S + s];
                    eta = prm.eta0[((long long)b * M + m) * S + s];
                }
                const float P0 = 1.0f / fmaxf(lam, kLamMin);
                pair_el(P[ci], i) = P0;
                pair_el(mean[ci], i) = eta * P0;
            }
        }
        bool carried = true;
        if (!first_seg) {
            // the state the preceding segment ended in, as it left that CTA's registers
            carried = seg_wait(prm.wait, prm.seg.done + unit.seq, unit.seg, 9);
            const float2 *hand = reinterpret_cast<const float2 *>(prm.seg.hand);
#pragma unroll
            for (int ci = 0; ci < CH; ++ci) {
                const int m = m_cta + cw + ci;
#pragma unroll
                for (int i = 0; i < SPT; ++i) {
                    const int s = i * LPC + j;
                    if (carried && m < M && s < S) {
                        const float2 h = __ldcg(hand + ((long long)b * M + m) * S + s);
                        pair_el(P[ci], i) = h.x;
                        pair_el(mean[ci], i) = h.y;
                    }
                }
            }
        }
        // checkpoint pointer of chain (ci = 0, i = 0); advanced by one tile per tile
        float2 *ck = prm.ckpt;
        if (ck != nullptr) ck += (((long long)b * prm.NC + t_off / kCkptInterval) * M + (m_cta + cw)) * S + j;
        const long long ck_tile = (long long)M * S;
        auto store_ckpt = [&]() {  // the state before the step about to be taken; advances to the next checkpoint
#pragma unroll
            for (int ci = 0; ci < CH; ++ci)
#pragma unroll
                for (int i = 0; i < SPT; ++i)
                    if (m_cta + cw + ci < M && i * LPC + j < S)
                        ck[ci * S + i * LPC] = make_float2(pair_el(P[ci], i), pair_el(mean[ci], i));
            ck += ck_tile;
        };

        // The time loop is software-pipelined by hand, because a single warp is
        // bound by the latency of its dependent instructions, not by issue slots:
        //   fetch(t+1)   shared-memory loads of the next step's inputs
        //   update(t)    the serial part: P -> denominator -> reciprocal -> P, mean
        //   readout(t)   this thread's share of y, y_var to shared memory
        //   prep(t+1)    everything of the next step that does not depend on the
        //                state (phi, r)
        // so the loads and the state-independent arithmetic of step t+1 sit
        // between the dependent instructions of step t.
        struct StepIn {
            float lv[CH], vv[CH];
            float2 k[HP], q[HP];  // this thread's states, in pairs
        };
        struct StepPre {
            float2 r[CH][HP], phi[CH][HP], q[HP];
        };
        auto fetch = [&](StepIn &in, const T *lrow, const float *lfrow, const T *vrow, const float *kqrow, int tt) {
#pragma unroll
            for (int ci = 0; ci < CH; ++ci) {
                if constexpr (sizeof(T) == 4) in.lv[ci] = lfrow[tt * MC + ci];  // the same tile as lrow
                else in.lv[ci] = pro ? lfrow[tt * MC + ci] : to_f32<T>(lrow[tt * MC + ci]);
                in.vv[ci] = to_f32<T>(vrow[tt * MC + ci]);
            }
            const float *row = kqrow + tt * 2 * SPAD;
            if constexpr (SPT == 4) {
                const float4 kk = *reinterpret_cast<const float4 *>(row);
                const float4 qq = *reinterpret_cast<const float4 *>(row + SPT);
                in.k[0] = make_float2(kk.x, kk.y);
                in.k[1] = make_float2(kk.z, kk.w);
                in.q[0] = make_float2(qq.x, qq.y);
                in.q[1] = make_float2(qq.z, qq.w);
            } else {
#pragma unroll
                for (int h = 0; h < HP; ++h) {
                    in.k[h] = *reinterpret_cast<const float2 *>(row + 2 * h);
                    in.q[h] = *reinterpret_cast<const float2 *>(row + SPT + 2 * h);
                }
            }
        };
        auto prep = [&](StepPre &pr, const StepIn &in) {
#pragma unroll
            for (int h = 0; h < HP; ++h) {
                pr.q[h] = in.q[h];
#pragma unroll
                for (int ci = 0; ci < CH; ++ci) {
                    chain_inputs2(dup2(in.lv[ci]), dup2(in.vv[ci]), in.k[h], pr.phi[ci][h], pr.r[ci][h]);
                }
            }
        };
        auto update = [&](const StepPre &pr) {
            float2 Pp[CH][HP], g[CH][HP];
#pragma unroll
            for (int h = 0; h < HP; ++h)
#pragma unroll
                for (int ci = 0; ci < CH; ++ci) {
                    g[ci][h] = chain_denominator2(P[ci][h], pr.phi[ci][h], ca2[ci][h], cp[ci][h], Pp[ci][h]);
                }
#pragma unroll
            for (int h = 0; h < HP; ++h)
#pragma unroll
                for (int ci = 0; ci < CH; ++ci) g[ci][h] = rcp_approx2(g[ci][h]);
#pragma unroll
            for (int h = 0; h < HP; ++h)
#pragma unroll
                for (int ci = 0; ci < CH; ++ci)
                    chain_update2(P[ci][h], mean[ci][h], Pp[ci][h], g[ci][h], pr.r[ci][h], ca[ci][h]);
        };
        auto readout = [&](const StepPre &pr, float2 *yrow, int tt) {
#pragma unroll
            for (int ci = 0; ci < CH; ++ci) {
                float2 ys = make_float2(0.0f, 0.0f), yvs = ys;
#pragma unroll
                for (int h = 0; h < HP; ++h) {
                    const float2 q = pr.q[h];
                    float2 mo, Po;
                    if (PRIOR) {  // read out the one-step-ahead prior, kla_ops.py:284-286
                        mo = mul2(ca[ci][h], mean[ci][h]);
                        Po = fma2(ca2[ci][h], P[ci][h], cp[ci][h]);
                    } else {
                        mo = mean[ci][h];
                        Po = P[ci][h];
                    }
                    const float2 qP = mul2(q, Po);
                    if (h == 0) {
                        ys = mul2(q, mo);
                        yvs = mul2(q, qP);
                    } else {
                        ys = fma2(q, mo, ys);
                        yvs = fma2(q, qP, yvs);
                    }
                }
                yrow[tt * LPC * MCP + ci] = make_float2(ys.x + ys.y, yvs.x + yvs.y);
            }
        };

        for (int tile = 0; tile < (carried ? NT : 0); ++tile) {
            const int s = tile % NS, o = tile % NO;
            const int t0 = tile * TT;
            if (!mbar_wait(prm.wait, &full_in[s], (tile / NS) & 1, 1)) break;
            if (pro) {  // this warp's channels of the tile: log-variance -> precision, float32
                const T *raw = lstage(s) + warp * Sh::kCPW;
                float *lf = lfstage(s) + warp * Sh::kCPW;
                for (int e = lane; e < TT * Sh::kCPW; e += 32) {
                    const int at = (e / Sh::kCPW) * MC + e % Sh::kCPW;
                    lf[at] = precision_from_log_variance_fast(to_f32<T>(raw[at]), prm.obs_var_min, prm.obs_var_max);
                }
                fence_proxy_async();  // these plain stores are ordered before the bulk copy that refills the stage
                __syncwarp();
            }
            if (tile >= NO && !mbar_wait(prm.wait, &empty_out[o], (tile / NO - 1) & 1, 2)) break;
            if (ck != nullptr) store_ckpt();
            const T *lrow = lstage(s) + cw;
            const float *lfrow = lfstage(s) + cw;
            const T *vrow = vstage(s) + cw;
            const float *kqrow = kqstage(s) + j * 2 * SPT;
            float2 *yrow = ystage(o) + j * MCP + cw;
            StepIn in;
            StepPre pr, prn;
            fetch(in, lrow, lfrow, vrow, kqrow, 0);
            prep(pr, in);
            if (t0 + TT <= L) {
                // kFwdUnroll steps per trip: with the paired arithmetic a whole tile fits the instruction cache
#pragma unroll 1
                for (int t4 = 0; t4 < TT; t4 += kFwdUnroll) {
#pragma unroll
                    for (int u = 0; u < kFwdUnroll; ++u) {
                        const int tt = t4 + u;
                        if (tt > 0 && tt % kCkptInterval == 0 && ck != nullptr) store_ckpt();
                        fetch(in, lrow, lfrow, vrow, kqrow, (tt + 1) % TT);  // the wrap-around fetch is not used
                        update(pr);
                        readout(pr, yrow, tt);
                        prep(prn, in);
                        pr = prn;
                    }
                }
            } else {
                for (int tt = 0; t0 + tt < L; ++tt) {
                    if (tt > 0 && tt % kCkptInterval == 0 && ck != nullptr) store_ckpt();
                    fetch(in, lrow, lfrow, vrow, kqrow, (tt + 1) % TT);
                    update(pr);
                    readout(pr, yrow, tt);
                    prep(prn, in);
                    pr = prn;
                }
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&empty_in[s]);
                mbar_arrive(&full_out[o]);
            }
        }

        // final state back in information form: lambda = 1/P, eta = mean * lambda; between segments the state is
        // handed on as it is
        float2 *hand = reinterpret_cast<float2 *>(prm.seg.hand);
#pragma unroll
        for (int ci = 0; ci < CH; ++ci) {
            const int m = m_cta + cw + ci;
#pragma unroll
            for (int i = 0; i < SPT; ++i) {
                const int s = i * LPC + j;
                if (m < M && s < S) {
                    if (last_seg) {
                        const float lam = 1.0f / pair_el(P[ci], i);
                        prm.lam_fin[((long long)b * M + m) * S + s] = lam;
                        prm.eta_fin[((long long)b * M + m) * S + s] = pair_el(mean[ci], i) * lam;
                    } else {
                        __stcg(hand + ((long long)b * M + m) * S + s, make_float2(pair_el(P[ci], i), pair_el(mean[ci], i)));
                    }
                }
            }
        }
        if (!last_seg) {
            __threadfence();
            group_barrier_128();
            if (tid == 0) st_release_gpu(prm.seg.done + unit.seq, unit.seg + 1);
        }
    } else {
        // ================================================================ helpers
        const int htid = tid - Sh::kCompute;
        const int hlane = htid & 31;
        constexpr uint32_t kTileBytes = sizeof(T) * TT * MC;
        int produced = 0, epi_issued = 0;  // tiles whose input / epilogue copies have been issued
        bool ok = true;
        if (htid < kProducers) {
            // ---- loaders: TMA tiles of v, lambda_v and the (k, q) pairs, NS tiles ahead
            const T *vb = static_cast<const T *>(prm.v.ptr) + (long long)b * prm.v.sb + (long long)t_off * prm.v.st;
            const T *lb = static_cast<const T *>(prm.lv.ptr) + (long long)b * prm.lv.sb + (long long)t_off * prm.lv.st;
            const T *kb = static_cast<const T *>(prm.k.ptr) + (long long)b * prm.k.sb + (long long)t_off * prm.k.st;
            const T *qb = static_cast<const T *>(prm.q.ptr) + (long long)b * prm.q.sb + (long long)t_off * prm.q.st;
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
            load_kq(0);
            for (int it = 0; it < NT; ++it) {
                const int s = it % NS, t0 = it * TT;
                if (it >= NS && !mbar_wait(prm.wait, &empty_in[s], (it / NS - 1) & 1, 3, 100)) { ok = false; break; }
                if (prm.use_tma) {
                    if (htid == 0) {
                        mbar_arrive_expect_tx(&full_in[s], 2 * kTileBytes);
                        tma_load_3d(vstage(s), &prm.tm_v, m_cta, t_off + t0, b, &full_in[s]);
                        tma_load_3d(lstage(s), &prm.tm_lv, m_cta, t_off + t0, b, &full_in[s]);
                    }
                } else {
                    stage_tile_plain<T, TT, MC, kProducers>(vstage(s), vb, prm.v.st, t0, L, m_cta, M, htid);
                    stage_tile_plain<T, TT, MC, kProducers>(lstage(s), lb, prm.lv.st, t0, L, m_cta, M, htid);
                }
                float *kq = kqstage(s);
#pragma unroll
                for (int e = 0; e < KQP; ++e) {
                    const int idx = htid + e * kProducers, row = idx / SPAD, sidx = idx % SPAD;
                    if (idx < TT * SPAD) {
                        float *dst = kq + row * 2 * SPAD + (sidx % LPC) * 2 * SPT + sidx / LPC;
                        dst[0] = kr[e];
                        dst[SPT] = qr[e];
                    }
                }
                if (it + 1 < NT) load_kq(t0 + TT);
                // (test hook: one loader thread leaves out its arrive for tile skip_tile, so the wait for that tile runs out)
                if (!(prm.use_tma && htid == 0) && !(it == prm.wait.skip_tile && htid == 1)) mbar_arrive(&full_in[s]);
                produced = it + 1;
                if constexpr (EPI) {  // this tile's z and gate, for the drainers
                    const int e = it % NE;
                    if (it >= NE && !mbar_wait(prm.wait, &epi_empty[e], (it / NE - 1) & 1, 6, 100)) { ok = false; break; }
                    const bool has_z = prm.z.ptr != nullptr, has_g = prm.gate.ptr != nullptr;
                    if (prm.epi_tma) {
                        if (htid == 0) {
                            mbar_arrive_expect_tx(&epi_full[e], ((has_z ? 1 : 0) + (has_g ? 1 : 0)) * kTileBytes);
                            if (has_z) tma_load_3d(zstage(e), &prm.tm_z, m_cta, t_off + t0, b, &epi_full[e]);
                            if (has_g) tma_load_3d(gstage(e), &prm.tm_gate, m_cta, t_off + t0, b, &epi_full[e]);
                        }
                    } else {
                        if (has_z)
                            stage_tile_plain<T, TT, MC, kProducers>(
                                zstage(e), static_cast<const T *>(prm.z.ptr) + (long long)b * prm.z.sb + (long long)t_off * prm.z.st, prm.z.st, t0, L, m_cta, M, htid);
                        if (has_g)
                            stage_tile_plain<T, TT, MC, kProducers>(
                                gstage(e), static_cast<const T *>(prm.gate.ptr) + (long long)b * prm.gate.sb + (long long)t_off * prm.gate.st, prm.gate.st, t0, L, m_cta, M, htid);
                    }
                    if (!(prm.epi_tma && htid == 0)) mbar_arrive(&epi_full[e]);
                    epi_issued = it + 1;
                }
            }
        } else {
            // ---- drainers: per finished tile, sum the LPC partial read-outs and store y, y_var
            const int dtid = htid - kProducers;
            TO *yb = static_cast<TO *>(prm.y.ptr) + (long long)b * prm.y.sb + (long long)t_off * prm.y.st;
            TO *yvb = static_cast<TO *>(prm.yv.ptr) + (long long)b * prm.yv.sb + (long long)t_off * prm.yv.st;
            float skip0 = 0.0f, skip1 = 0.0f;
            if constexpr (EPI) {
                static_assert(kDrainers % (MC / 2) == 0, "a drainer thread keeps its channel pair from tile to tile");
                if (prm.skip != nullptr) {
                    const int c0 = (dtid % (MC / 2)) * 2;
                    skip0 = prm.skip[prm.skip_len > 1 ? min(m_cta + c0, M - 1) : 0];
                    skip1 = prm.skip[prm.skip_len > 1 ? min(m_cta + c0 + 1, M - 1) : 0];
                }
            }
            for (int jt = 0; jt < NT; ++jt) {
                const int o = jt % NO, t0 = jt * TT;
                if (!mbar_wait(prm.wait, &full_out[o], (jt / NO) & 1, 4, 100)) { ok = false; break; }
                if constexpr (EPI) {
                    const int e = jt % NE;
                    if (!mbar_wait(prm.wait, &epi_full[e], (jt / NE) & 1, 7, 100)) { ok = false; break; }
                    const T *zs = prm.z.ptr ? zstage(e) : nullptr, *gs = prm.gate.ptr ? gstage(e) : nullptr;
                    TO *yr = prm.y_raw.ptr ? static_cast<TO *>(prm.y_raw.ptr) + (long long)b * prm.y_raw.sb + (long long)(t_off + t0) * prm.y_raw.st : nullptr;
                    TO *yvr = prm.y_raw.ptr ? static_cast<TO *>(prm.yv_raw.ptr) + (long long)b * prm.yv_raw.sb + (long long)(t_off + t0) * prm.yv_raw.st : nullptr;
                    output_pass<TO, LPC, MC, MCP, TT, kDrainers>(
                        ystage(o), yb + (long long)t0 * prm.y.st, prm.y.st, prm.vec_y,
                        yvb + (long long)t0 * prm.yv.st, prm.yv.st, prm.vec_yv, min(TT, L - t0), m_cta, M, dtid,
                        [&](float2 acc, int tt, int c, float &o0, float &o1) {
                            const int m = m_cta + c;
                            if (m < M) {
                                if (yr != nullptr) {  // the scan's own outputs, for the epilogue's adjoint
                                    yr[(long long)tt * prm.y_raw.st + m] = from_f32<TO>(acc.x);
                                    yvr[(long long)tt * prm.yv_raw.st + m] = from_f32<TO>(acc.y);
                                }
                                // a drainer thread meets the same pair of channels in every tile: its skip values are in registers
                                if (zs != nullptr) acc.x = fmaf((c & 1) ? skip1 : skip0, to_f32<T>(zs[tt * MC + c]), acc.x);
                                if (gs != nullptr) {
                                    const float g = activate_fast(to_f32<T>(gs[tt * MC + c]), prm.gate_act);
                                    acc.x *= g;
                                    acc.y *= g * g;
                                }
                            }
                            o0 = acc.x;
                            o1 = acc.y;
                        });
                    __syncwarp();
                    if (hlane == 0) mbar_arrive(&epi_empty[e]);
                } else {
                    output_pass<TO, LPC, MC, MCP, TT, kDrainers>(
                        ystage(o), yb + (long long)t0 * prm.y.st, prm.y.st, prm.vec_y,
                        yvb + (long long)t0 * prm.yv.st, prm.yv.st, prm.vec_yv, min(TT, L - t0), m_cta, M, dtid,
                        [](float2 acc, int, int, float &o0, float &o1) { o0 = acc.x; o1 = acc.y; });
                }
                __syncwarp();
                if (hlane == 0) mbar_arrive(&empty_out[o]);
            }
        }
        // Leaving early (a wait ran out): do not end the CTA with bulk copies
        // still in flight into its shared memory.
        if (!ok && htid == 0) {
            if (prm.use_tma)
                for (int t = max(0, produced - NS); t < produced; ++t) mbar_wait(prm.wait, &full_in[t % NS], (t / NS) & 1, 5);
            if (EPI && prm.epi_tma)  // the epilogue tiles travel by TMA whether or not v and lambda_v do
                for (int t = max(0, epi_issued - NE); t < epi_issued; ++t) mbar_wait(prm.wait, &epi_full[t % NE], (t / NE) & 1, 8);
        }
    }
}

}  // namespace kla
