// Single-token decode of one KLA layer around its three projections: the
// elementwise work between the GEMMs, fused into two kernels.
//
//   kla_conv_step_kernel   the causal depthwise convolution advanced by one token
//                          (reference: CausalConv1d.forward with L = 1,
//                          src/kla/layers/common.py:87-96): window update, dot
//                          product with the taps, bias, activation.
//   kla_step_layer_kernel  everything from the sensor projection's output to the
//                          input of the output projection
//                          (src/kla/layers/kla_layer.py:199-231, 277-293, 329-338):
//                          l2-normalised and clipped k, q; observation variance
//                          softplus(.) + floor -> precision; the filter step
//                          (kla_step, src/kla/ops/kla_ops.py:293-331); the skip
//                          path lambda_skip * z; the gate act(gate) on the mean and
//                          its square on the variance.
// Both are bound by the state they read and write; the fusion removes about 25
// elementwise launches and their round trips per layer and token.
#pragma once

#include "kla_common.cuh"

namespace kla {

struct ConvStepParams {
    int B, D, K;           // K taps, window of K-1 past inputs
    const void *x;         // [B, D] with batch stride
    long long x_sb;
    const float *w, *bias; // [D, K], [D] or nullptr
    void *state;           // [B, D, K-1], updated in place
    void *z;               // [B, D] out
    int act;
};

constexpr int kConvMaxTaps = 8;

template <typename T>
__global__ void __launch_bounds__(128) kla_conv_step_kernel(const ConvStepParams prm) {
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (long long)prm.B * prm.D) return;
    const int b = (int)(gid / prm.D), d = (int)(gid % prm.D), K = prm.K;
    T *st = static_cast<T *>(prm.state) + gid * (K - 1);
    const T xin = static_cast<const T *>(prm.x)[(long long)b * prm.x_sb + d];
    float win[kConvMaxTaps];
#pragma unroll
    for (int jj = 0; jj < kConvMaxTaps; ++jj)
        if (jj < K - 1) win[jj] = to_f32<T>(st[jj]);
    float acc = prm.bias != nullptr ? prm.bias[d] : 0.0f;
#pragma unroll
    for (int jj = 0; jj < kConvMaxTaps; ++jj)
        if (jj < K - 1) acc = fmaf(prm.w[(long long)d * K + jj], win[jj], acc);
    acc = fmaf(prm.w[(long long)d * K + K - 1], to_f32<T>(xin), acc);
#pragma unroll
    for (int jj = 0; jj < kConvMaxTaps; ++jj)
        if (jj + 1 < K - 1) st[jj] = from_f32<T>(win[jj + 1]);
    if (K > 1) st[K - 2] = xin;
    static_cast<T *>(prm.z)[gid] = from_f32<T>(activate(acc, prm.act));
}

// The same convolution over a whole prompt (CausalConv1d.forward for L > 1): one thread per channel
// and chunk of kConvChunk consecutive tokens keeps the K-1 previous inputs in registers, so every input
// is read once; lanes run over channels, so rows are read and written coalesced in the layer's own
// [B, L, D] layout (the reference transposes to [B, D, L] and back around its conv1d call). The block that
// owns the last chunk also writes the new window (the last K-1 inputs) to state_out.
struct ConvSeqParams {
    int B, L, D, K;
    Tensor3 x, z;          // [B, L, D]
    const float *w, *bias; // [D, K], [D] or nullptr
    const void *state;     // [B, D, K-1]: the window before the prompt
    void *state_out;       // [B, D, K-1]: the window after it (another buffer: blocks of other chunks still read state)
    int act;
};

constexpr int kConvChunk = 32;
constexpr int kConvBlock = 8;  // steps whose inputs are fetched before any of them is used

// VEC consecutive channels of one row, widened to float32 (VEC = 2: one 4- or 8-byte access)
template <typename T, int VEC>
__device__ __forceinline__ void conv_load(const T *p, float (&x)[VEC]) {
    if constexpr (VEC == 1) {
        x[0] = to_f32<T>(*p);
    } else if constexpr (sizeof(T) == 2) {
        const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162 *>(p);
        x[0] = __low2float(v);
        x[1] = __high2float(v);
    } else {
        const float2 v = *reinterpret_cast<const float2 *>(p);
        x[0] = v.x;
        x[1] = v.y;
    }
}
template <typename T, int VEC>
__device__ __forceinline__ void conv_store(T *p, const float (&x)[VEC]) {
    if constexpr (VEC == 1) {
        *p = from_f32<T>(x[0]);
    } else if constexpr (sizeof(T) == 2) {
        *reinterpret_cast<__nv_bfloat162 *>(p) = __floats2bfloat162_rn(x[0], x[1]);
    } else {
        *reinterpret_cast<float2 *>(p) = make_float2(x[0], x[1]);
    }
}

// A thread owns VEC adjacent channels (2 when the rows allow 4-/8-byte accesses) and fetches the inputs of
// kConvBlock steps before it uses any of them, so that a warp keeps kilobytes, not one 64-byte row, in flight.
// Window and taps sit right-aligned in arrays of kConvMaxTaps entries (zeros in front of the K live ones), which
// keeps every register index a compile-time constant for any K.
// KT: the length of those arrays, 4 for up to four taps (the layer's default), else kConvMaxTaps.
template <typename T, int VEC, int KT>
__global__ void __launch_bounds__(128) kla_conv_seq_kernel(const ConvSeqParams prm) {
    const int d = (blockIdx.x * blockDim.x + threadIdx.x) * VEC, b = blockIdx.z;
    const int t0 = blockIdx.y * kConvChunk;
    if (d >= prm.D) return;
    constexpr int MAXT = KT;
    const int K = prm.K, L = prm.L, lead = MAXT - K;
    const T *xb = static_cast<const T *>(prm.x.ptr) + (long long)b * prm.x.sb + d;
    T *zb = static_cast<T *>(prm.z.ptr) + (long long)b * prm.z.sb + d;
    const T *st = static_cast<const T *>(prm.state) + ((long long)b * prm.D + d) * (K - 1);
    T *sto = static_cast<T *>(prm.state_out) + ((long long)b * prm.D + d) * (K - 1);
    // xw[i]: input at time t - (MAXT-1) + i once step t has shifted its input in; before the first step the window
    // sits one place further back
    float wr[MAXT][VEC], xw[MAXT][VEC], bias[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
        bias[e] = prm.bias != nullptr ? prm.bias[d + e] : 0.0f;
#pragma unroll
        for (int i = 0; i < MAXT; ++i) {
            wr[i][e] = i >= lead ? prm.w[(long long)(d + e) * K + (i - lead)] : 0.0f;
            xw[i][e] = 0.0f;
            if (i > lead) {
                const int t = t0 - MAXT + i;  // before the prompt: the carried window
                xw[i][e] = t >= 0 ? to_f32<T>(xb[(long long)t * prm.x.st + e]) : to_f32<T>(st[(long long)e * (K - 1) + t + (K - 1)]);
            }
        }
    }
    const int t1 = min(L, t0 + kConvChunk);
    for (int tb = t0; tb < t1; tb += kConvBlock) {
        float xin[kConvBlock][VEC];
#pragma unroll
        for (int u = 0; u < kConvBlock; ++u)
            if (tb + u < t1) conv_load<T, VEC>(xb + (long long)(tb + u) * prm.x.st, xin[u]);
#pragma unroll
        for (int u = 0; u < kConvBlock; ++u) {
            if (tb + u < t1) {
                float out[VEC];
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
#pragma unroll
                    for (int i = 0; i < MAXT - 1; ++i) xw[i][e] = i >= lead ? xw[i + 1][e] : 0.0f;
                    xw[MAXT - 1][e] = xin[u][e];
                    float acc = bias[e];
#pragma unroll
                    for (int i = 0; i < MAXT; ++i) acc = fmaf(wr[i][e], xw[i][e], acc);
                    out[e] = activate_fast(acc, prm.act);
                }
                conv_store<T, VEC>(zb + (long long)(tb + u) * prm.z.st, out);
            }
        }
    }
    if (t1 == L) {
        // the window after the prompt is made of the last K-1 inputs; those older than the prompt come from the
        // carried window
#pragma unroll
        for (int e = 0; e < VEC; ++e)
            for (int jj = 0; jj < K - 1; ++jj) {
                const int t = L - (K - 1) + jj;
                sto[(long long)e * (K - 1) + jj] =
                    t >= 0 ? xb[(long long)t * prm.x.st + e] : st[(long long)e * (K - 1) + t + (K - 1)];
            }
    }
}

struct StepLayerParams {
    int B, M, S;
    const void *v, *ls, *k, *q, *z, *gate;  // z, gate may be nullptr
    long long v_sb, ls_sb, k_sb, q_sb, z_sb, gate_sb;
    const float *a, *p, *lam, *eta;
    float *lam_out, *eta_out;
    void *y, *yv;                  // [B, M] contiguous
    const float *skip;             // nullptr, one value, or [M]
    int skip_len;
    float obs_var_min, obs_var_max, clip;  // obs_var_max <= 0: none; clip <= 0: none
    int qk_norm, gate_act;
    int vec;  // as StepParams::vec
};

// One thread per (b, m, group of 4 consecutive states), LPC adjacent lanes per channel, as in kla_step_kernel.
template <typename T, typename TO, int LPC, bool PRIOR>
__global__ void __launch_bounds__(128) kla_step_layer_kernel(const StepLayerParams prm) {
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long bm = gid / LPC;
    const int j = (int)(gid % LPC);
    const int M = prm.M, S = prm.S;
    const bool row_live = bm < (long long)prm.B * M;
    const int b = row_live ? (int)(bm / M) : 0, m = row_live ? (int)(bm % M) : 0;

    // this lane's four k, q values and its share of their squared norms
    const T *kb = static_cast<const T *>(prm.k) + (long long)b * prm.k_sb;
    const T *qb = static_cast<const T *>(prm.q) + (long long)b * prm.q_sb;
    float kv[4], qv[4], k2 = 0.0f, q2 = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int s = j * 4 + i;
        const bool in = row_live && s < S;
        kv[i] = in ? to_f32<T>(kb[s]) : 0.0f;
        qv[i] = in ? to_f32<T>(qb[s]) : 0.0f;
        k2 = fmaf(kv[i], kv[i], k2);
        q2 = fmaf(qv[i], qv[i], q2);
    }
    if (prm.qk_norm) {  // x / max(||x||, 1e-12), src/kla/layers/common.py:25-27
#pragma unroll
        for (int off = LPC / 2; off > 0; off >>= 1) {
            k2 += __shfl_xor_sync(0xffffffffu, k2, off);
            q2 += __shfl_xor_sync(0xffffffffu, q2, off);
        }
        const float kn = fmaxf(sqrtf(k2), 1e-12f), qn = fmaxf(sqrtf(q2), 1e-12f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            kv[i] /= kn;
            qv[i] /= qn;
        }
    }
    if (prm.clip > 0.0f) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            kv[i] = fminf(fmaxf(kv[i], -prm.clip), prm.clip);
            qv[i] = fminf(fmaxf(qv[i], -prm.clip), prm.clip);
        }
    }

    float ys = 0.0f, yvs = 0.0f;
    if (row_live) {
        // observation-noise variance -> value precision, kla_layer.py:224-231
        const float lv = precision_from_log_variance(
            to_f32<T>(static_cast<const T *>(prm.ls)[(long long)b * prm.ls_sb + m]), prm.obs_var_min, prm.obs_var_max);
        const float vl = to_f32<T>(static_cast<const T *>(prm.v)[(long long)b * prm.v_sb + m]) * lv;
        const long long ms0 = (long long)m * S + j * 4, bms0 = ((long long)b * M + m) * S + j * 4;
        // lanes wholly past the row (j * 4 >= S, e.g. S = 12 with LPC = 4) hold padding chains and touch no memory
        const bool vec = prm.vec != 0, lane_live = j * 4 < S;
        float lamv[4], etav[4], av[4], pv[4], lo[4], eo[4];
        if (!lane_live) {
#pragma unroll
            for (int i = 0; i < 4; ++i) { lamv[i] = 1.0f; etav[i] = 0.0f; av[i] = 0.0f; pv[i] = 1.0f; }
        } else if (vec) {
            const float4 l4 = *reinterpret_cast<const float4 *>(prm.lam + bms0);
            const float4 e4 = *reinterpret_cast<const float4 *>(prm.eta + bms0);
            const float4 a4 = *reinterpret_cast<const float4 *>(prm.a + ms0);
            const float4 p4 = *reinterpret_cast<const float4 *>(prm.p + ms0);
            lamv[0] = l4.x; lamv[1] = l4.y; lamv[2] = l4.z; lamv[3] = l4.w;
            etav[0] = e4.x; etav[1] = e4.y; etav[2] = e4.z; etav[3] = e4.w;
            av[0] = a4.x; av[1] = a4.y; av[2] = a4.z; av[3] = a4.w;
            pv[0] = p4.x; pv[1] = p4.y; pv[2] = p4.z; pv[3] = p4.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const bool in = j * 4 + i < S;
                lamv[i] = in ? prm.lam[bms0 + i] : 1.0f;
                etav[i] = in ? prm.eta[bms0 + i] : 0.0f;
                av[i] = in ? prm.a[ms0 + i] : 0.0f;
                pv[i] = in ? prm.p[ms0 + i] : 1.0f;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const bool in = j * 4 + i < S;
            const float a = av[i];
            const float p = fmaxf(pv[i], kPMin);                     // kla_ops.py:316
            const float a2 = fmaxf(a * a, kEps);                     // :317
            const float phi = fmaxf(lv * kv[i] * kv[i], kEps);       // :310-312
            const float inv = 1.0f / fmaxf(a2 + p * lamv[i], kEps);  // :319
            const float lam = lamv[i] * inv + phi;                   // :320
            const float eta = (a * inv) * etav[i] + vl * kv[i];      // :321
            float var = 1.0f / fmaxf(lam, kEps);                     // :323
            float mean = eta * var;                                  // :324
            if (PRIOR) {                                             // :325-327
                mean = a * mean;
                var = a2 * var + p;
            }
            if (in) {
                ys = fmaf(mean, qv[i], ys);                          // :329
                yvs = fmaf(var, qv[i] * qv[i], yvs);                 // :330
            }
            lo[i] = lam;
            eo[i] = eta;
        }
        if (!lane_live) {
            // padding lane: nothing to store
        } else if (vec) {
            *reinterpret_cast<float4 *>(prm.lam_out + bms0) = make_float4(lo[0], lo[1], lo[2], lo[3]);
            *reinterpret_cast<float4 *>(prm.eta_out + bms0) = make_float4(eo[0], eo[1], eo[2], eo[3]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (j * 4 + i < S) {
                    prm.lam_out[bms0 + i] = lo[i];
                    prm.eta_out[bms0 + i] = eo[i];
                }
        }
    }
#pragma unroll
    for (int off = LPC / 2; off > 0; off >>= 1) {
        ys += __shfl_xor_sync(0xffffffffu, ys, off);
        yvs += __shfl_xor_sync(0xffffffffu, yvs, off);
    }
    if (row_live && j == 0) {
        // kla_layer.py:329-338: skip path, then the gate on the mean and its square on the variance
        if (prm.skip != nullptr && prm.z != nullptr) {
            const float sk = prm.skip[prm.skip_len > 1 ? m : 0];
            ys = fmaf(sk, to_f32<T>(static_cast<const T *>(prm.z)[(long long)b * prm.z_sb + m]), ys);
        }
        if (prm.gate != nullptr) {
            const float g = activate(to_f32<T>(static_cast<const T *>(prm.gate)[(long long)b * prm.gate_sb + m]), prm.gate_act);
            ys *= g;
            yvs *= g * g;
        }
        static_cast<TO *>(prm.y)[(long long)b * M + m] = from_f32<TO>(ys);
        static_cast<TO *>(prm.yv)[(long long)b * M + m] = from_f32<TO>(yvs);
    }
}

}  // namespace kla
