// Adjoint of the layer's output path (src/kla/layers/kla_layer.py:329-338) when the forward scan applied it
// inside the kernel:
//
//   u = y + skip z;   out = u g;   out_var = y_var g^2;   g = act(gate)
//
// Given the gradients of out and out_var, one pass over the [B, L, M] tensors produces the gradients the scan's
// own backward starts from and those of the path's other operands:
//
//   dy = dout g            dy_var = dout_var g^2
//   dz = dy skip           dskip += sum dy z   (per channel, or over everything for a scalar skip)
//   dgate = (dout u + 2 dout_var y_var g) act'(gate)
//
// y and y_var are the scan's outputs before the path was applied; the forward stores them for this purpose.
// Memory-bound: 6 tensors in, 4 out, one element of each per (b, t, m). A thread owns one channel and walks
// kEpiRows time steps, so consecutive lanes touch consecutive addresses and the skip gradient needs one atomic
// add per thread.
#pragma once

#include "kla_common.cuh"

namespace kla {

constexpr int kEpiRows = 32;

struct EpilogueBwdParams {
    int B, L, M;
    Tensor3 dout, dout_var;   // TO; dout_var.ptr may be nullptr (= zero)
    Tensor3 y_raw, yv_raw;    // TO
    Tensor3 z, gate;          // T; either may be nullptr (that half of the path is absent)
    const float *skip;
    int skip_len, gate_act;
    Tensor3 dy, dy_var;       // TO, out
    Tensor3 dz, dgate;        // T, out (nullptr when the operand is absent)
    float *dskip;             // [skip_len], accumulated
};

// derivative of the gate activation
__device__ __forceinline__ float activate_slope(float x, int act) {
    switch (act) {
        case kActSilu: {
            const float s = 1.0f / (1.0f + expf(-x));
            return s * (1.0f + x * (1.0f - s));
        }
        case kActGelu:
            return 0.5f * (1.0f + erff(x * 0.70710678118654752f)) + x * 0.3989422804014327f * expf(-0.5f * x * x);
        case kActRelu: return x > 0.0f ? 1.0f : 0.0f;
        default: return 1.0f;
    }
}

// VEC channels per thread (4 when every tensor allows 16-byte (float32) / 8-byte (bfloat16) accesses, else 1);
// HAS_Z / HAS_G: which halves of the path exist. All loads of a row are issued before its arithmetic, and two
// rows are in flight per thread, so that the memory system sees enough independent requests.
template <typename T, int VEC>
struct EpiVec {
    float x[VEC];
    __device__ __forceinline__ void load(const void *base, long long off) {
        const T *p = static_cast<const T *>(base) + off;
        if constexpr (VEC == 4 && sizeof(T) == 4) {
            const float4 v = *reinterpret_cast<const float4 *>(p);
            x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
        } else if constexpr (VEC == 4) {
            const uint2 raw = *reinterpret_cast<const uint2 *>(p);
            const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162 *>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162 *>(&raw.y);
            x[0] = __low2float(lo); x[1] = __high2float(lo); x[2] = __low2float(hi); x[3] = __high2float(hi);
        } else {
            x[0] = to_f32<T>(p[0]);
        }
    }
    __device__ __forceinline__ void store(void *base, long long off) const {
        T *p = static_cast<T *>(base) + off;
        if constexpr (VEC == 4 && sizeof(T) == 4) {
            *reinterpret_cast<float4 *>(p) = make_float4(x[0], x[1], x[2], x[3]);
        } else if constexpr (VEC == 4) {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]), hi = __floats2bfloat162_rn(x[2], x[3]);
            uint2 raw;
            raw.x = *reinterpret_cast<const unsigned *>(&lo);
            raw.y = *reinterpret_cast<const unsigned *>(&hi);
            *reinterpret_cast<uint2 *>(p) = raw;
        } else {
            p[0] = from_f32<T>(x[0]);
        }
    }
};

template <typename T, typename TO, int VEC, bool HAS_Z, bool HAS_G>
__global__ void __launch_bounds__(128) kla_epilogue_bwd_kernel(const EpilogueBwdParams prm) {
    const int m = (blockIdx.x * 128 + threadIdx.x) * VEC;
    const int b = blockIdx.z;
    const int t0 = blockIdx.y * kEpiRows;
    const bool live = m < prm.M;  // dead threads stay for the warp-wide sum at the end
    const int t1 = live ? min(prm.L, t0 + kEpiRows) : t0;
    auto at = [&](const Tensor3 &t, int tt) { return (long long)b * t.sb + (long long)tt * t.st + m; };
    const bool has_dv = prm.dout_var.ptr != nullptr;
    float skip[VEC], dskip[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
        skip[e] = (HAS_Z && live) ? prm.skip[prm.skip_len > 1 ? m + e : 0] : 0.0f;
        dskip[e] = 0.0f;
    }
    const int act = prm.gate_act;
#pragma unroll 2
    for (int tt = t0; tt < t1; ++tt) {
        EpiVec<TO, VEC> dout, dvar, y, yv, dy, dyv;
        EpiVec<T, VEC> z, gate, dz, dgate;
        dout.load(prm.dout.ptr, at(prm.dout, tt));
        if (has_dv) dvar.load(prm.dout_var.ptr, at(prm.dout_var, tt));
        if (HAS_G) {
            gate.load(prm.gate.ptr, at(prm.gate, tt));
            y.load(prm.y_raw.ptr, at(prm.y_raw, tt));
            yv.load(prm.yv_raw.ptr, at(prm.yv_raw, tt));
        }
        if (HAS_Z) z.load(prm.z.ptr, at(prm.z, tt));
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const float dv = has_dv ? dvar.x[e] : 0.0f;
            float g = 1.0f;
            if (HAS_G) {
                g = activate(gate.x[e], act);
                const float u = HAS_Z ? fmaf(skip[e], z.x[e], y.x[e]) : y.x[e];
                dgate.x[e] = fmaf(dout.x[e], u, 2.0f * dv * yv.x[e] * g) * activate_slope(gate.x[e], act);
            }
            dy.x[e] = dout.x[e] * g;
            dyv.x[e] = dv * g * g;
            if (HAS_Z) {
                dz.x[e] = dy.x[e] * skip[e];
                dskip[e] = fmaf(dy.x[e], z.x[e], dskip[e]);
            }
        }
        dy.store(prm.dy.ptr, at(prm.dy, tt));
        dyv.store(prm.dy_var.ptr, at(prm.dy_var, tt));
        if (HAS_G) dgate.store(prm.dgate.ptr, at(prm.dgate, tt));
        if (HAS_Z) dz.store(prm.dz.ptr, at(prm.dz, tt));
    }
    if (HAS_Z) {
        if (prm.skip_len > 1) {
            if (live) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) atomicAdd(prm.dskip + m + e, dskip[e]);
            }
        } else {  // scalar skip: one sum over everything; add the warp's share with one atomic
            float s = 0.0f;
#pragma unroll
            for (int e = 0; e < VEC; ++e) s += dskip[e];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
            if ((threadIdx.x & 31) == 0) atomicAdd(prm.dskip, s);
        }
    }
}

}  // namespace kla
