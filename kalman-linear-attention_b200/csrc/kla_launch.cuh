// Host-side launchers of the two scan kernels, one template instantiation per
// (activation types, lanes per channel, prior read-out). They are declared here
// and defined and instantiated in kla_scan_inst.cu, which the build compiles
// several times (one slice of the instantiations per object file) so that the
// slices compile in parallel; kla_capi.cu only calls them.
#pragma once

#include "kla_agg.cuh"
#include "kla_bwd.cuh"

namespace kla {

#ifndef KLA_NW
#define KLA_NW 4
#endif
constexpr int kNW = KLA_NW;            // compute warps per CTA
#ifndef KLA_NH
#define KLA_NH 4
#endif
constexpr int kNH = KLA_NH;            // helper warps per CTA
constexpr int kTT = 16;                // steps per tile of the forward (two checkpoints)
constexpr int kBwdTT = kCkptInterval;  // steps per tile of the backward
#ifndef KLA_SPT
#define KLA_SPT 4
#endif
constexpr int kSPT = KLA_SPT;          // states per thread
#ifndef KLA_CH
#define KLA_CH 1
#endif
constexpr int kCH = KLA_CH;            // channels per thread

// channels per CTA of the scan kernels for a given number of lanes per channel
inline int scan_channels_per_cta(int lpc) { return kNW * (32 / lpc) * kCH; }

// channels per CTA of the aggregate kernel
inline int agg_channels_per_cta(int lpc) { return kNW * (32 / lpc); }

// Launch on `st` with the grid and shared memory of the instantiation; prm must be complete
// (tensor maps included). Returns the launch's CUDA status.
template <typename T, typename TO, int LPC, bool PRIOR>
cudaError_t launch_fwd(const FwdParams &prm, cudaStream_t st);
template <typename T, typename TO, int LPC, bool PRIOR>
cudaError_t launch_bwd(const BwdParams &prm, cudaStream_t st);
// adjoint: prm.q, dy, dyv, lam0, eta0 are used and PRIOR matters; otherwise the forward aggregate
template <typename T, typename TO, int LPC, bool PRIOR>
cudaError_t launch_agg(const AggParams &prm, bool adjoint, cudaStream_t st);

}  // namespace kla
