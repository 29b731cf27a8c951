// Shared device helpers for the KLA scan kernels (sm_100a).
//
// Thread mapping used by every scan kernel here. A "chain" is one (batch b,
// channel m, state s) lane of the filter; chains never interact except through
// the read-out sum over s and the gradient sums over m, b and t.
//
//   * a thread owns CH consecutive channels x SPT states: CH*SPT chains whose
//     state lives in registers for the whole sequence;
//   * LPC consecutive lanes of a warp share a channel group; lane j of such a
//     group owns states s = i*LPC + j, i = 0..SPT-1, so S is padded to
//     SPAD = SPT*LPC and sums over s finish with log2(LPC) shuffle rounds;
//   * a warp therefore covers (32/LPC)*CH channels and a CTA of NW warps covers
//     MC = NW*(32/LPC)*CH channels of one batch element; time is the serial axis
//     and is walked in tiles of TT steps staged through shared memory.
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

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kla {

constexpr float kEps = 1e-12f;      // EPS,   src/kla/ops/kla_ops.py:43
constexpr float kPMin = 1e-12f;     // P_MIN, src/kla/ops/kla_ops.py:44
constexpr float kLamMin = 1e-20f;   // floor on a carried-in precision before 1/lambda
constexpr int kCkptInterval = 16;   // steps between checkpoints of the filter state

struct Tensor3 {
    void *ptr;
    long long sb, st;  // batch and time strides, in elements
};

__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// One predict+update step of one chain. Explicit intrinsics pin the rounding so
// that the backward's replay reproduces the forward bit for bit.
struct StepOut {
    float Pp, g;
};
__device__ __forceinline__ StepOut chain_step(float &P, float &mean, float phi, float r,
                                              float a, float a2, float p) {
    StepOut o;
    o.Pp = __fmaf_rn(a2, P, p);
    const float d = __fmaf_rn(phi, o.Pp, 1.0f);
    o.g = rcp_approx(d);
    P = __fmul_rn(o.Pp, o.g);
    const float u = __fmaf_rn(o.Pp, r, __fmul_rn(a, mean));
    mean = __fmul_rn(o.g, u);
    return o;
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

__device__ __forceinline__ void cp_async_16(void *smem, const void *gmem) {
    const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_4(void *smem, const void *gmem) {
    const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// Stage a [TT x MC] tile of a [B, L, M] tensor (rows t0.., columns m0..) into
// shared memory as T, zero-filling rows past L and columns past M. `vec` says
// that 16-byte copies are legal for this tensor (base and strides aligned, M a
// multiple of the vector width).
template <typename T, int TT, int MC, int NTHR>
__device__ __forceinline__ void stage_tile(T *smem, const T *base, long long st, int t0, int L,
                                           int m0, int M, bool vec, int tid) {
    constexpr int VEC = 16 / sizeof(T);
    if (vec && (MC % VEC) == 0) {
        constexpr int CPR = (MC / VEC) > 0 ? (MC / VEC) : 1;  // chunks per row
        for (int idx = tid; idx < TT * CPR; idx += NTHR) {
            const int row = idx / CPR, c = (idx % CPR) * VEC;
            T *dst = smem + row * MC + c;
            if (t0 + row < L && m0 + c < M) {
                cp_async_16(dst, base + (long long)(t0 + row) * st + m0 + c);
            } else {
                *reinterpret_cast<uint4 *>(dst) = make_uint4(0, 0, 0, 0);
            }
        }
    } else {
        for (int idx = tid; idx < TT * MC; idx += NTHR) {
            const int row = idx / MC, c = idx % MC;
            T v = from_f32<T>(0.0f);
            if (t0 + row < L && m0 + c < M) v = base[(long long)(t0 + row) * st + m0 + c];
            smem[row * MC + c] = v;
        }
    }
}

}  // namespace kla
