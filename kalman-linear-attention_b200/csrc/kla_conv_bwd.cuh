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

template <typename T>
__global__ void __launch_bounds__(128) kla_conv_seq_bwd_kernel(const ConvSeqBwdParams prm) {
    const int d = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.z;
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
    // wl the taps from the front (zeros behind).
    constexpr int MAXT = kConvMaxTaps;
    const int lead = MAXT - K;  // entries in front of the K live ones
    float wl[MAXT], wr[MAXT], xw[MAXT], dwin[MAXT], accw[MAXT];
#pragma unroll
    for (int i = 0; i < MAXT; ++i) {
        wl[i] = i < K ? prm.w[(long long)d * K + i] : 0.0f;
        wr[i] = i >= lead ? prm.w[(long long)d * K + (i - lead)] : 0.0f;
        dwin[i] = accw[i] = 0.0f;
        xw[i] = 0.0f;
        if (i > lead) {  // the K-1 inputs before t0, one place further back than in the loop, which shifts first
            const int t = t0 - MAXT + i;
            xw[i] = t >= 0 ? to_f32<T>(xb[(long long)t * prm.x.st]) : (st != nullptr ? to_f32<T>(st[t + (K - 1)]) : 0.0f);
        }
    }
    const float bias = prm.bias != nullptr ? prm.bias[d] : 0.0f;
    float accb = 0.0f;
    const int t1 = min(L, t0 + kConvBwdChunk);
    const int tend = t1 + K - 1;  // dx[t1 - 1] needs dpre up to t1 + K - 2
#pragma unroll 2
    for (int t = t0; t < tend; ++t) {
        float dpre = 0.0f;
        if (t < L) {
            const float xin = to_f32<T>(xb[(long long)t * prm.x.st]);
            const float g = to_f32<T>(gb[(long long)t * prm.dz.st]);
#pragma unroll
            for (int i = 0; i < MAXT - 1; ++i) xw[i] = i >= lead ? xw[i + 1] : 0.0f;
            xw[MAXT - 1] = xin;
            float pre = bias;
#pragma unroll
            for (int i = 0; i < MAXT; ++i) pre = fmaf(wr[i], xw[i], pre);
            dpre = g * activate_slope(pre, prm.act);
            if (t < t1) {  // the sums over t belong to the chunk that owns t
                accb += dpre;
#pragma unroll
                for (int i = 0; i < MAXT; ++i) accw[i] = fmaf(dpre, xw[i], accw[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < MAXT - 1; ++i) dwin[i] = dwin[i + 1];
        dwin[MAXT - 1] = dpre;
        const int u = t - (K - 1);
        if (u >= t0) {  // dx[u] = sum_j w[j] dpre[t - j]
            float acc = 0.0f;
#pragma unroll
            for (int jj = 0; jj < MAXT; ++jj) acc = fmaf(wl[jj], dwin[MAXT - 1 - jj], acc);
            ob[(long long)u * prm.dx.st] = from_f32<T>(acc);
        }
    }
#pragma unroll
    for (int i = 0; i < MAXT; ++i)
        if (i >= lead) atomicAdd(prm.dw + (long long)d * K + (i - lead), accw[i]);
    if (prm.dbias != nullptr) atomicAdd(prm.dbias + d, accb);
}

}  // namespace kla
