// Backward of the causal depthwise convolution over a sequence (kla_conv_seq_kernel,
// reference: CausalConv1d.forward, src/kla/layers/common.py:87-96, differentiated):
//
//   pre[t]  = bias + sum_j w[j] x[t - (K-1) + j]        z[t] = act(pre[t])
//   dpre[t] = dz[t] act'(pre[t])
//   dx[u]   = sum_j w[j] dpre[u + (K-1) - j]            (terms past the end dropped)
//   dw[j]   = sum_{b,t} dpre[t] x[t - (K-1) + j]        dbias = sum_{b,t} dpre[t]
//
// Same shape as the forward kernel: one thread per channel and chunk of
// consecutive steps, lanes over channels, everything in the layer's [B, L, D]
// layout. The thread recomputes pre from a register window of the last K inputs
// (nothing but x is kept from the forward), keeps the last K values of dpre in a
// second window and emits dx[u] once dpre[u + K-1] is known; for that it walks
// K-1 steps past its chunk. The weight and bias sums of a chunk stay in registers
// and leave with one atomic each per thread. Inputs before the sequence come from
// the carried window (`state`, or zeros).
#pragma once

#include <type_traits>

#include "kla_decode.cuh"
#include "kla_epilogue.cuh"

namespace kla {

constexpr int kConvBwdChunk = 64;

struct ConvSeqBwdParams {
    int B, L, D, K;
    Tensor3 x, dz, dx;     // [B, L, D]
    const float *w, *bias; // [D, K], [D] or nullptr
    const void *state;     // [B, D, K-1] (the window before the sequence) or nullptr = zeros
    float *dw, *dbias;     // [D, K], [D] (or nullptr): added to with atomics
    int act;
};

// derivative of the activation with the hardware's exp2 and reciprocal approximations for the sigmoid of silu
// (relative error ~1e-6), as activate_fast
__device__ __forceinline__ float activate_slope_fast(float x, int act) {
    if (act == kActSilu) {
        const float s = rcp_approx(1.0f + __expf(-x));
        return s * fmaf(x, 1.0f - s, 1.0f);
    }
    return activate_slope(x, act);
}

template <typename T, int VEC, int KT>
__global__ void __launch_bounds__(128) kla_conv_seq_bwd_kernel(const ConvSeqBwdParams prm) {
    const int d = (blockIdx.x * blockDim.x + threadIdx.x) * VEC, b = blockIdx.z;
    const int t0 = blockIdx.y * kConvBwdChunk;
    if (d >= prm.D) return;
    const int K = prm.K, L = prm.L;
    const T *xb = static_cast<const T *>(prm.x.ptr) + (long long)b * prm.x.sb + d;
    const T *gb = static_cast<const T *>(prm.dz.ptr) + (long long)b * prm.dz.sb + d;
    T *ob = static_cast<T *>(prm.dx.ptr) + (long long)b * prm.dx.sb + d;
    const T *st = prm.state != nullptr ? static_cast<const T *>(prm.state) + ((long long)b * prm.D + d) * (K - 1) : nullptr;
    // Windows and taps sit right-aligned in arrays of kConvMaxTaps entries, so that every index below is a
    // compile-time constant (the arrays stay in registers for any K): xw[i] is x at time t - (MAXT-1) + i with the
    // newest input last, wr the taps aligned the same way (zeros in front), dwin the last MAXT values of dpre,
    // wl the taps from the front (zeros behind). A thread owns VEC adjacent channels (see kla_conv_seq_kernel).
    constexpr int MAXT = KT;  // 4 for up to four taps, else kConvMaxTaps
    const int lead = MAXT - K;  // entries in front of the K live ones
    float wl[MAXT][VEC], wr[MAXT][VEC], xw[MAXT][VEC], dwin[MAXT][VEC], accw[MAXT][VEC], bias[VEC], accb[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
        bias[e] = prm.bias != nullptr ? prm.bias[d + e] : 0.0f;
        accb[e] = 0.0f;
#pragma unroll
        for (int i = 0; i < MAXT; ++i) {
            wl[i][e] = i < K ? prm.w[(long long)(d + e) * K + i] : 0.0f;
            wr[i][e] = i >= lead ? prm.w[(long long)(d + e) * K + (i - lead)] : 0.0f;
            dwin[i][e] = accw[i][e] = 0.0f;
            xw[i][e] = 0.0f;
            if (i > lead) {  // the K-1 inputs before t0, one place further back than in the loop, which shifts first
                const int t = t0 - MAXT + i;
                xw[i][e] = t >= 0 ? to_f32<T>(xb[(long long)t * prm.x.st + e])
                                  : (st != nullptr ? to_f32<T>(st[(long long)e * (K - 1) + t + (K - 1)]) : 0.0f);
            }
        }
    }
    const int t1 = min(L, t0 + kConvBwdChunk);
    const int tend = t1 + K - 1;  // dx[t1 - 1] needs dpre up to t1 + K - 2
    // One block of kConvBlock steps. FULL: every step lies inside the chunk and, from the second block on, every
    // dx it completes too, so none of the range checks is needed (all blocks but the first and the last ones).
    auto block = [&](int tb, auto full) {
        constexpr bool FULL = decltype(full)::value;
        float xin[kConvBlock][VEC], gin[kConvBlock][VEC];
#pragma unroll
        for (int u = 0; u < kConvBlock; ++u)
            if (FULL || (tb + u < tend && tb + u < L)) {
                conv_load<T, VEC>(xb + (long long)(tb + u) * prm.x.st, xin[u]);
                conv_load<T, VEC>(gb + (long long)(tb + u) * prm.dz.st, gin[u]);
            }
#pragma unroll
        for (int u = 0; u < kConvBlock; ++u) {
            const int t = tb + u;
            if (FULL || t < tend) {
                float out[VEC];
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    float dpre = 0.0f;
                    if (FULL || t < L) {
#pragma unroll
                        for (int i = 0; i < MAXT - 1; ++i) xw[i][e] = i >= lead ? xw[i + 1][e] : 0.0f;
                        xw[MAXT - 1][e] = xin[u][e];
                        float pre = bias[e];
#pragma unroll
                        for (int i = 0; i < MAXT; ++i) pre = fmaf(wr[i][e], xw[i][e], pre);
                        dpre = gin[u][e] * activate_slope_fast(pre, prm.act);
                        if (FULL || t < t1) {  // the sums over t belong to the chunk that owns t
                            accb[e] += dpre;
#pragma unroll
                            for (int i = 0; i < MAXT; ++i) accw[i][e] = fmaf(dpre, xw[i][e], accw[i][e]);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < MAXT - 1; ++i) dwin[i][e] = dwin[i + 1][e];
                    dwin[MAXT - 1][e] = dpre;
                    float acc = 0.0f;  // dx[u] = sum_j w[j] dpre[t - j], u = t - (K-1)
#pragma unroll
                    for (int jj = 0; jj < MAXT; ++jj) acc = fmaf(wl[jj][e], dwin[MAXT - 1 - jj][e], acc);
                    out[e] = acc;
                }
                if (FULL || t - (K - 1) >= t0) conv_store<T, VEC>(ob + (long long)(t - (K - 1)) * prm.dx.st, out);
            }
        }
    };
    for (int tb = t0; tb < tend; tb += kConvBlock) {
        if (tb >= t0 + kConvMaxTaps && tb + kConvBlock <= t1) block(tb, std::true_type{});
        else block(tb, std::false_type{});
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
#pragma unroll
        for (int i = 0; i < MAXT; ++i)
            if (i >= lead) atomicAdd(prm.dw + (long long)(d + e) * K + (i - lead), accw[i][e]);
        if (prm.dbias != nullptr) atomicAdd(prm.dbias + d + e, accb[e]);
    }
}

}  // namespace kla
