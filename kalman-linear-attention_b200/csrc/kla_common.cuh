// Shared device helpers for the KLA scan kernels (sm_100a).
//
// Thread mapping used by every scan kernel here. A "chain" is one (batch b,
// channel m, state s) lane of the filter; chains never interact except through
// the read-out sum over s and the gradient sums over m, b and t.
//
//   * a compute thread owns CH consecutive channels x SPT states: CH*SPT chains
//     whose state lives in registers for the whole sequence;
//   * LPC consecutive lanes of a warp share a channel group; lane j of such a
//     group owns states s = i*LPC + j, i = 0..SPT-1, so S is padded to
//     SPAD = SPT*LPC and sums over s are LPC partial sums per channel;
//   * a warp therefore covers (32/LPC)*CH channels and a CTA with NW compute
//     warps covers MC = NW*(32/LPC)*CH channels of one batch element; time is
//     the serial axis and is walked in tiles of TT steps staged through shared
//     memory by a second group of NH helper warps (loads, sums of partials,
//     stores), so the compute warps never wait on global memory.
//
// The recurrence is carried in variance form, which is the same filter as the
// reference's information form (src/kla/ops/kla_ops.py:9-14) with P = 1/lambda
// and mean = eta/lambda:
//
//   Pp   = a^2 P' + p                 predicted variance
//   d    = 1 + phi Pp,  g = 1/d       phi = lambda_v k^2
//   P    = Pp g                       posterior variance  (= 1/lambda_t)
//   mean = g (a mean' + Pp r)         r = (v lambda_v) k  (= eta_t / lambda_t)
//
// It needs one reciprocal per step where the information form needs two, and
// the read-out y = sum_s q mean, y_var = sum_s q^2 P uses the carried values
// directly.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kla {

constexpr float kEps = 1e-12f;      // EPS,   src/kla/ops/kla_ops.py:43
constexpr float kPMin = 1e-12f;     // P_MIN, src/kla/ops/kla_ops.py:44
constexpr float kLamMin = 1e-20f;   // floor on a carried-in precision before 1/lambda
constexpr int kCkptInterval = 8;    // steps between checkpoints of the filter state (= one tile of the backward)

// Device-side status word: 0 = ok, otherwise the code of the first bounded wait
// that ran out (kStatusWait | site). Read back by kla_b200_device_status().
constexpr int kStatusWait = 0x100;

// What a kernel needs for its bounded waits; part of every kernel's parameters.
struct WaitCtl {
    int *status;        // the device's status word (one per device, owned by the library)
    unsigned limit_ns;  // a wait gives up after about this long (1e9 in normal operation)
    int skip_tile;      // test hook: the loader leaves out one arrive for this tile, so that the wait
                        // for it runs out; -1 in normal operation
};

// Sequences cut into segments. A CTA of the scan kernels owns one (batch element, channel block) sequence
// for its whole length, and a grid rarely divides evenly over the SMs' CTA slots: at 256 sequences 40 of
// the 148 SMs hold one CTA instead of two and finish early; at 768 the last of three rounds is half empty. With
// nseg > 1 the grid has nseg CTAs per sequence. A CTA draws a ticket when it starts; tickets map to
// (segment, sequence) with the segment that must run first in the slowest position, so the CTA that owns the
// preceding segment of the same sequence always drew its ticket earlier, i.e. is running or done. The CTA
// brings its inputs in, waits (bounded) until `done[sequence]` says the preceding segment is finished, takes
// the carried state from `hand`, and leaves its own there. SMs that finish their CTAs early simply draw more
// tickets, which evens the load out. The arithmetic and its order are those of the unsegmented kernel.
struct SegCtl {
    int nseg;     // segments per sequence; 1 = off (nothing below is touched)
    int seg_len;  // steps per segment, a multiple of the kernels' tile lengths
    int *ticket;  // one counter, zero before the launch
    int *done;    // [sequences] segments finished so far, zero before the launch
    float *hand;  // carried state between segments, planes of [B, M, S] floats
};

// What a CTA works on: its channel block, batch element and segment.
struct SegUnit {
    int bx, b, seg, seq;
};

// Called by every thread of the CTA (contains a CTA-wide barrier). reverse: segments run last-first.
__device__ __forceinline__ SegUnit seg_assign(const SegCtl &sc, bool reverse) {
    SegUnit u{(int)blockIdx.x, (int)blockIdx.y, 0, (int)(blockIdx.y * gridDim.x + blockIdx.x)};
    if (sc.nseg > 1) {
        __shared__ int ticket;
        if (threadIdx.x == 0) ticket = atomicAdd(sc.ticket, 1);
        __syncthreads();
        const int nseq = gridDim.x * gridDim.y;
        const int order = ticket / nseq;
        if (ticket < 0 || order >= sc.nseg) {  // a counter that was not zero before the launch: touch nothing
            u.seg = -1;
            return u;
        }
        u.seq = ticket % nseq;
        u.bx = u.seq % gridDim.x;
        u.b = u.seq / gridDim.x;
        u.seg = reverse ? sc.nseg - 1 - order : order;
    }
    return u;
}

__device__ __forceinline__ int ld_acquire_gpu(const int *p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(int *p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Wait until `need` segments of the sequence are finished; every calling thread polls (and thereby acquires what
// the finishing CTA released). Gives up like mbar_wait: status word, false.
__device__ __forceinline__ bool seg_wait(const WaitCtl &w, const int *done, int need, int site) {
    const unsigned limit = w.limit_ns / 256u + 1u;
    for (unsigned it = 0;; ++it) {
        if (ld_acquire_gpu(done) >= need) return true;
        if (it >= limit) {
            atomicCAS(w.status, 0, kStatusWait | site);
            return false;
        }
        __nanosleep(200);
    }
}

// The 128 threads of a compute group meet here (hardware barrier 1; barrier 0 is __syncthreads).
__device__ __forceinline__ void group_barrier_128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

struct Tensor3 {
    void *ptr;
    long long sb, st;  // batch and time strides, in elements
};

template <int SPT, int LPC, int CH, int NW, int NH, int TT>
struct ScanShape {
    static constexpr int kSPad = SPT * LPC;
    static constexpr int kCLS = 32 / LPC;         // channel groups per warp
    static constexpr int kCPW = kCLS * CH;        // channels per warp
    static constexpr int kMC = NW * kCPW;         // channels per CTA
    static constexpr int kCompute = NW * 32;      // compute threads
    static constexpr int kHelpers = NH * 32;      // helper threads
    static constexpr int kThreads = kCompute + kHelpers;
    // Row length of the [TT][LPC][MCP] float2 partial-sum buffers. 8-byte
    // shared-memory accesses are served half a warp at a time; a half-warp
    // writes LPC rows of kCPW/2 channels each, so rows are offset by kCPW/2
    // channels modulo the 16 channels (32 banks) a wavefront covers.
    static constexpr int kHalf = kCPW / 2 > 0 ? kCPW / 2 : 1;
    static constexpr int kPadRaw = ((kHalf - kMC) % 16 + 16) % 16;
    static constexpr int kMCP = kMC + kPadRaw + (kPadRaw & 1);
    static_assert(kMC % 2 == 0, "the output pass works on pairs of channels");
};

__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// One predict+update step of one chain, in pieces so that callers can put the
// reciprocals of several independent chains in flight together. Explicit
// intrinsics pin the rounding so that the backward's replay reproduces the
// forward bit for bit.
//
// chain_inputs: phi = lambda_v k^2 and r = (v lambda_v) k from one product
// lambda_v k, so that only k itself has to come from shared memory.
__device__ __forceinline__ void chain_inputs(float lv, float v, float k, float &phi, float &r) {
    const float lk = __fmul_rn(lv, k);
    phi = __fmul_rn(lk, k);
    r = __fmul_rn(v, lk);
}
// chain_denominator: Pp = a2 P + p and d = 1 + phi Pp, two dependent FMAs. (Folding them into
// d = (a2 phi) P + (phi p + 1) puts only one FMA between the carried P and the reciprocal but costs
// two more operations per lane-step; the kernels are bound by the FP32 pipe, not by that chain:
// the two-FMA form is 10 % faster in the forward.)
__device__ __forceinline__ float chain_denominator(float P, float phi, float a2, float p, float &Pp) {
    Pp = __fmaf_rn(a2, P, p);
    return __fmaf_rn(phi, Pp, 1.0f);
}
// chain_update: P = Pp g, mean = g (a mean' + Pp r), with g = 1/d.
__device__ __forceinline__ void chain_update(float &P, float &mean, float Pp, float g, float r, float a) {
    P = __fmul_rn(Pp, g);
    mean = __fmul_rn(g, __fmaf_rn(Pp, r, __fmul_rn(a, mean)));
}

// The same pieces for two chains at a time. sm_100 issues an fp32 multiply, add
// or FMA on a pair of values held in an aligned register pair as one
// instruction; every lane of it rounds like the scalar instruction, so the pair
// forms give bit-identical results while taking half the issue slots.
__device__ __forceinline__ float2 mul2(float2 x, float2 y) { return __fmul2_rn(x, y); }
__device__ __forceinline__ float2 fma2(float2 x, float2 y, float2 z) { return __ffma2_rn(x, y, z); }
__device__ __forceinline__ float2 add2(float2 x, float2 y) { return __fadd2_rn(x, y); }
__device__ __forceinline__ float2 neg2(float2 x) { return make_float2(-x.x, -x.y); }
__device__ __forceinline__ float2 dup2(float x) { return make_float2(x, x); }
__device__ __forceinline__ float2 rcp_approx2(float2 x) { return make_float2(rcp_approx(x.x), rcp_approx(x.y)); }
// element i of an array of pairs (i is a compile-time constant after unrolling)
template <int N>
__device__ __forceinline__ float &pair_el(float2 (&arr)[N], int i) {
    return (i & 1) ? arr[i >> 1].y : arr[i >> 1].x;
}
__device__ __forceinline__ void chain_inputs2(float2 lv, float2 v, float2 k, float2 &phi, float2 &r) {
    const float2 lk = mul2(lv, k);
    phi = mul2(lk, k);
    r = mul2(v, lk);
}
__device__ __forceinline__ float2 chain_denominator2(float2 P, float2 phi, float2 a2, float2 p, float2 &Pp) {
    Pp = fma2(a2, P, p);
    return fma2(phi, Pp, make_float2(1.0f, 1.0f));
}
__device__ __forceinline__ void chain_update2(float2 &P, float2 &mean, float2 Pp, float2 g, float2 r, float2 a) {
    P = mul2(Pp, g);
    mean = mul2(g, fma2(Pp, r, mul2(a, mean)));
}

enum Activation { kActSilu = 0, kActGelu = 1, kActRelu = 2, kActNone = 3 };

__device__ __forceinline__ float activate(float x, int act) {
    switch (act) {
        case kActSilu: return x / (1.0f + expf(-x));
        case kActGelu: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
        case kActRelu: return fmaxf(x, 0.0f);
        default: return x;
    }
}

// The same for the scan's drainer warps, which have a tile time to finish a tile's outputs: hardware
// exp2 and reciprocal approximations (relative error ~1e-6) for the sigmoid of silu.
__device__ __forceinline__ float activate_fast(float x, int act) {
    if (act == kActSilu) return x * rcp_approx(1.0f + __expf(-x));
    return activate(x, act);
}

// torch.nn.functional.softplus with its default threshold of 20
__device__ __forceinline__ float softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
// Value precision from the sensor projection's raw output, as the reference layer forms it
// (src/kla/layers/kla_layer.py:224-231): 1 / min(softplus(x) + obs_var_min, obs_var_max); no ceiling when obs_var_max <= 0.
__device__ __forceinline__ float precision_from_log_variance(float x, float vmin, float vmax) {
    float sig = softplus(x) + vmin;
    if (vmax > 0.0f) sig = fminf(sig, vmax);
    return 1.0f / sig;
}
// The same two functions for the scan kernels, where they run in the helper warps beside the
// recurrence and every instruction counts: hardware exp2/log2/reciprocal approximations, with
// short series where those would lose relative accuracy (log1p(e) for small e, 1 - exp(-s) for
// small s). Relative error below 4e-6 over the whole range, against the 1e-5 parity bar.
__device__ __forceinline__ float softplus_fast(float x) {
    if (x > 20.0f) return x;
    const float e = __expf(x);
    if (e < 0.1f)  // log1p(e) = e - e^2/2 + e^3/3 - e^4/4 + e^5/5, next term below 2e-7 e
        return e * fmaf(e, fmaf(e, fmaf(e, fmaf(e, 0.2f, -0.25f), 0.33333333f), -0.5f), 1.0f);
    return __logf(1.0f + e);
}
__device__ __forceinline__ float precision_from_log_variance_fast(float x, float vmin, float vmax) {
    float sig = softplus_fast(x) + vmin;
    if (vmax > 0.0f) sig = fminf(sig, vmax);
    return rcp_approx(sig);
}
// d(precision)/dx expressed through the precision itself: -lam^2 sigmoid(x) with
// softplus(x) = 1/lam - vmin, sigmoid(x) = 1 - exp(-softplus(x)); zero where the ceiling binds.
__device__ __forceinline__ float precision_slope(float lam, float vmin, float vmax) {
    const float sig = rcp_approx(lam);
    if (vmax > 0.0f && sig >= vmax) return 0.0f;
    const float s = fmaxf(sig - vmin, 0.0f);
    // 1 - exp(-s): series below 0.1 (s - s^2/2 + s^3/6 - s^4/24), where the subtraction would cancel
    const float sgm = s < 0.1f ? s * fmaf(s, fmaf(s, fmaf(s, -0.041666667f, 0.16666667f), -0.5f), 1.0f) : 1.0f - __expf(-s);
    return -(lam * lam) * sgm;
}

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// ---------------------------------------------------------------- mbarrier + TMA
//
// Producer/consumer hand-off between helper and compute warps uses mbarrier
// objects in shared memory; tile loads use the tensor-map form of the bulk
// async copy (TMA), which signals the same mbarrier with its byte count.

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait. A waiting warp sleeps between polls (sleep_ns each) so that it
// does not take issue slots from the warps that are computing on the same
// scheduler. After about WaitCtl::limit_ns of polling (a second) it gives up,
// records where in the device's status word and returns false; the caller then
// leaves its loop so that the CTA ends instead of hanging the device.
__device__ __forceinline__ bool mbar_wait(const WaitCtl &w, uint64_t *bar, uint32_t parity, int site,
                                          unsigned sleep_ns = 100) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint32_t limit = w.limit_ns / (sleep_ns + 100);
    for (uint32_t i = 0; i < limit; ++i) {
        __nanosleep(sleep_ns);
        if (mbar_try_wait(bar, parity)) return true;
    }
    atomicCAS(w.status, 0, kStatusWait | site);
    return false;
}
// generic-proxy writes to shared memory -> visible to the async proxy (TMA)
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// TMA: tile (x: channel, y: time, z: batch) of a rank-3 tensor map -> shared memory
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *tm, int x, int y, int z, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}
// untiled bulk copy global -> shared (16-byte aligned, size a multiple of 16)
__device__ __forceinline__ void bulk_load_1d(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Named barrier over a subset of the CTA's warps (id 1..15).
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Cooperative fallback staging of a [TT x MC] tile (rows t0.., columns m0..) by
// NTHR threads with plain loads, zero-filling rows past L and columns past M;
// used when a tensor does not meet the tensor-map alignment rules.
template <typename T, int TT, int MC, int NTHR>
__device__ __forceinline__ void stage_tile_plain(T *smem, const T *base, long long st, int t0, int L, int m0, int M,
                                                 int tid) {
    for (int idx = tid; idx < TT * MC; idx += NTHR) {
        const int row = idx / MC, c = idx % MC;
        T v = from_f32<T>(0.0f);
        if (t0 + row < L && m0 + c < M) v = base[(long long)(t0 + row) * st + m0 + c];
        smem[row * MC + c] = v;
    }
}

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

}  // namespace kla
