// Definitions and explicit instantiations of the scan kernels' launchers
// (kla_launch.cuh). The build compiles this file once per slice:
//   KLA_INST_KIND   0 forward, 1 backward, 2 aggregates
//   KLA_INST_DT     0 (float, float), 1 (bfloat16, float), 2 (bfloat16, bfloat16)
//   KLA_INST_LPCS   0 lanes per channel 1, 2, 4;  1 lanes per channel 8, 16, 32
// Without those macros it holds every instantiation.
#include "kla_launch.cuh"

namespace kla {

template <typename T, typename TO, int LPC, bool PRIOR>
cudaError_t launch_fwd(const FwdParams &prm, cudaStream_t st) {
    using Sh = ScanShape<kSPT, LPC, kCH, kNW, kNH, kTT>;
    using Sm = FwdSmem<T, kSPT, LPC, kCH, kNW, kNH, kTT>;
    const bool seg = prm.seg.nseg > 1;
    auto kern = prm.epilogue ? (seg ? kla_fwd_kernel<T, TO, kSPT, LPC, kCH, kNW, kNH, kTT, PRIOR, true, true>
                                    : kla_fwd_kernel<T, TO, kSPT, LPC, kCH, kNW, kNH, kTT, PRIOR, true, false>)
                             : (seg ? kla_fwd_kernel<T, TO, kSPT, LPC, kCH, kNW, kNH, kTT, PRIOR, false, true>
                                    : kla_fwd_kernel<T, TO, kSPT, LPC, kCH, kNW, kNH, kTT, PRIOR, false, false>);
    const size_t smem = prm.epilogue ? Sm::kTotal : Sm::kPlain;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Sm::kTotal);
    if (e != cudaSuccess) return e;
    dim3 grid((unsigned)((prm.M + Sh::kMC - 1) / Sh::kMC), (unsigned)prm.B, (unsigned)prm.seg.nseg);
    kern<<<grid, Sh::kThreads, smem, st>>>(prm);
    return cudaGetLastError();
}

template <typename T, typename TO, int LPC, bool PRIOR>
cudaError_t launch_bwd(const BwdParams &prm, cudaStream_t st) {
    using Sh = ScanShape<kSPT, LPC, kCH, kNW, kNH, kBwdTT>;
    using Sm = BwdSmem<T, TO, kSPT, LPC, kCH, kNW, kNH, kBwdTT>;
    const bool seg = prm.seg.nseg > 1;
    auto kern = prm.lv_log_sigma ? (seg ? kla_bwd_kernel<T, TO, kSPT, LPC, kCH, kNW, kNH, kBwdTT, PRIOR, true, true>
                                        : kla_bwd_kernel<T, TO, kSPT, LPC, kCH, kNW, kNH, kBwdTT, PRIOR, true, false>)
                                 : (seg ? kla_bwd_kernel<T, TO, kSPT, LPC, kCH, kNW, kNH, kBwdTT, PRIOR, false, true>
                                        : kla_bwd_kernel<T, TO, kSPT, LPC, kCH, kNW, kNH, kBwdTT, PRIOR, false, false>);
    // The kernel's warp groups re-divide the registers the CTA was launched with; if the compiled kernel holds
    // fewer than the division assumes, the group that grows would wait for registers that never come. Checked
    // once per instantiation, before anything is launched.
    static int regs_ok[4] = {-1, -1, -1, -1};
    int &ok = regs_ok[(prm.lv_log_sigma ? 1 : 0) + (seg ? 2 : 0)];
    if (ok < 0) {
        cudaFuncAttributes attr;
        cudaError_t e = cudaFuncGetAttributes(&attr, kern);
        if (e != cudaSuccess) return e;
        ok = attr.numRegs * kBwdThreads >= 128 * (kBwdRegsReverse + kBwdRegsReplay + kBwdRegsHelper) ? 1 : 0;
    }
    if (!ok) return cudaErrorLaunchOutOfResources;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Sm::kTotal);
    if (e != cudaSuccess) return e;
    dim3 grid((unsigned)((prm.M + Sh::kMC - 1) / Sh::kMC), (unsigned)prm.B, (unsigned)prm.seg.nseg);
    kern<<<grid, kBwdThreads, Sm::kTotal, st>>>(prm);
    return cudaGetLastError();
}

template <typename T, typename TO, int LPC, bool PRIOR>
cudaError_t launch_agg(const AggParams &prm, bool adjoint, cudaStream_t st) {
    constexpr int MC = kNW * (32 / LPC);
    dim3 grid((unsigned)((prm.M + MC - 1) / MC), (unsigned)prm.B);
    cudaError_t e;
    if (adjoint) {
        auto kern = kla_agg_kernel<T, TO, kSPT, LPC, kNW, true, PRIOR>;
        constexpr size_t smem = AggSmem<T, TO, kSPT, LPC, kNW, true>::kTotal;
        if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
        kern<<<grid, (kNW + 1) * 32, smem, st>>>(prm);
    } else {
        auto kern = kla_agg_kernel<T, TO, kSPT, LPC, kNW, false, false>;
        constexpr size_t smem = AggSmem<T, TO, kSPT, LPC, kNW, false>::kTotal;
        if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
        kern<<<grid, (kNW + 1) * 32, smem, st>>>(prm);
    }
    return cudaGetLastError();
}

#define KLA_INST_AGG_ONE(T, TO, LPC)                                                       \
    template cudaError_t launch_agg<T, TO, LPC, false>(const AggParams &, bool, cudaStream_t); \
    template cudaError_t launch_agg<T, TO, LPC, true>(const AggParams &, bool, cudaStream_t);
#define KLA_INST_AGG(T, TO)                                                                      \
    KLA_INST_AGG_ONE(T, TO, 1) KLA_INST_AGG_ONE(T, TO, 2) KLA_INST_AGG_ONE(T, TO, 4) \
    KLA_INST_AGG_ONE(T, TO, 8) KLA_INST_AGG_ONE(T, TO, 16) KLA_INST_AGG_ONE(T, TO, 32)

#define KLA_INST_ONE(FN, PARAMS, T, TO, LPC)                                         \
    template cudaError_t FN<T, TO, LPC, false>(const PARAMS &, cudaStream_t);        \
    template cudaError_t FN<T, TO, LPC, true>(const PARAMS &, cudaStream_t);
#define KLA_INST_LOW(FN, PARAMS, T, TO) \
    KLA_INST_ONE(FN, PARAMS, T, TO, 1) KLA_INST_ONE(FN, PARAMS, T, TO, 2) KLA_INST_ONE(FN, PARAMS, T, TO, 4)
#define KLA_INST_HIGH(FN, PARAMS, T, TO) \
    KLA_INST_ONE(FN, PARAMS, T, TO, 8) KLA_INST_ONE(FN, PARAMS, T, TO, 16) KLA_INST_ONE(FN, PARAMS, T, TO, 32)

#if !defined(KLA_INST_LPCS) || KLA_INST_LPCS == 0
#define KLA_INST_L(FN, PARAMS, T, TO) KLA_INST_LOW(FN, PARAMS, T, TO)
#else
#define KLA_INST_L(FN, PARAMS, T, TO)
#endif
#if !defined(KLA_INST_LPCS) || KLA_INST_LPCS == 1
#define KLA_INST_H(FN, PARAMS, T, TO) KLA_INST_HIGH(FN, PARAMS, T, TO)
#else
#define KLA_INST_H(FN, PARAMS, T, TO)
#endif
#define KLA_INST_DTYPE(FN, PARAMS, T, TO) KLA_INST_L(FN, PARAMS, T, TO) KLA_INST_H(FN, PARAMS, T, TO)

#if !defined(KLA_INST_DT) || KLA_INST_DT == 0
#define KLA_INST_D0(FN, PARAMS) KLA_INST_DTYPE(FN, PARAMS, float, float)
#else
#define KLA_INST_D0(FN, PARAMS)
#endif
#if !defined(KLA_INST_DT) || KLA_INST_DT == 1
#define KLA_INST_D1(FN, PARAMS) KLA_INST_DTYPE(FN, PARAMS, __nv_bfloat16, float)
#else
#define KLA_INST_D1(FN, PARAMS)
#endif
#if !defined(KLA_INST_DT) || KLA_INST_DT == 2
#define KLA_INST_D2(FN, PARAMS) KLA_INST_DTYPE(FN, PARAMS, __nv_bfloat16, __nv_bfloat16)
#else
#define KLA_INST_D2(FN, PARAMS)
#endif
#define KLA_INST_ALL(FN, PARAMS) KLA_INST_D0(FN, PARAMS) KLA_INST_D1(FN, PARAMS) KLA_INST_D2(FN, PARAMS)

#if !defined(KLA_INST_KIND) || KLA_INST_KIND == 0
KLA_INST_ALL(launch_fwd, FwdParams)
#endif
#if !defined(KLA_INST_KIND) || KLA_INST_KIND == 1
KLA_INST_ALL(launch_bwd, BwdParams)
#endif
#if !defined(KLA_INST_KIND) || KLA_INST_KIND == 2
KLA_INST_AGG(float, float)
KLA_INST_AGG(__nv_bfloat16, float)
KLA_INST_AGG(__nv_bfloat16, __nv_bfloat16)
#endif

}  // namespace kla
