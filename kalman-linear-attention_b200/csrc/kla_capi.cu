// extern "C" entry points of libkla_b200.so: argument checks, kernel-shape
// selection and launches. No torch types, no allocation, no exceptions.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/kla_b200.h"
#include "kla_conv_bwd.cuh"
#include "kla_decode.cuh"
#include "kla_epilogue.cuh"
#include "kla_launch.cuh"
#include "kla_rawscan.cuh"
#include "kla_slab.cuh"
#include "kla_step.cuh"

// The device's status word (kla_b200_device_status). Kernels get its device address in their
// parameters (WaitCtl::status): in host code the name below is only a handle.
static __device__ int g_kla_status = 0;

namespace {

using namespace kla;

std::atomic<long long> g_launches{0};
thread_local cudaError_t g_last_cuda = cudaSuccess;
thread_local char g_errbuf[256];
// KLA_B200_NO_TMA=1 forces the plain-load staging path (used by the tests to cover it)
const bool g_no_tma = [] { const char *e = getenv("KLA_B200_NO_TMA"); return e && e[0] == '1'; }();

int cuda_fail(cudaError_t e) {
    g_last_cuda = e;
    return KLA_B200_ECUDA;
}

Tensor3 t3(const kla_b200_tensor3 &t) { return Tensor3{t.ptr, t.stride_b, t.stride_t}; }

bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Vector stores of 2 output elements are legal when every row start is aligned to them.
template <typename T>
int vec2_ok(const kla_b200_tensor3 &t) {
    return t.ptr != nullptr && aligned(t.ptr, 2 * sizeof(T)) && (t.stride_b % 2) == 0 && (t.stride_t % 2) == 0;
}

// cuTensorMapEncodeTiled is fetched from the driver at run time, so the library
// links against the CUDA runtime only.
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Rank-3 tensor map over a [B, L, M] activation tensor, dims (M, L, B), box
// (box_m, box_t, 1). Returns false when the tensor does not meet the TMA rules
// (16-byte aligned base and strides); the kernels then stage with plain loads.
template <typename T>
bool make_tile_map(CUtensorMap *tm, const kla_b200_tensor3 &t, int64_t B, int64_t L, int64_t M, int box_m, int box_t) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr || t.ptr == nullptr || B <= 0 || L <= 0 || M <= 0) return false;
    // size-1 dimensions may carry arbitrary strides; give them the dense value
    const int64_t st = L > 1 ? t.stride_t : M;
    const int64_t sb = B > 1 ? t.stride_b : L * st;
    const uint64_t st_b = (uint64_t)st * sizeof(T), sb_b = (uint64_t)sb * sizeof(T);
    if (!aligned(t.ptr, 16) || st_b % 16 || sb_b % 16 || st < M || st_b >= (1ull << 40) || sb_b >= (1ull << 40))
        return false;
    if ((box_m * sizeof(T)) % 16 || box_m > 256 || box_t > 256) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)M, (cuuint64_t)L, (cuuint64_t)B};
    const cuuint64_t strides[2] = {st_b, sb_b};
    const cuuint32_t box[3] = {(cuuint32_t)box_m, (cuuint32_t)box_t, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapDataType dt = sizeof(T) == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    return enc(tm, dt, 3, t.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int lpc_for(int64_t S) {
    int lpc = 1;
    while ((int64_t)kSPT * lpc < S) lpc *= 2;
    return lpc;  // 1..32 for S <= 128
}

int check_common(int64_t B, int64_t L, int64_t M, int64_t S, int32_t in_dtype, int32_t out_dtype) {
    if (B < 0 || L < 0 || M < 0 || S < 0) return KLA_B200_EINVAL;
    if (S > KLA_B200_MAX_DSTATE) return KLA_B200_EUNSUPPORTED;
    if (in_dtype != KLA_B200_F32 && in_dtype != KLA_B200_BF16) return KLA_B200_EUNSUPPORTED;
    if (out_dtype != KLA_B200_F32 && out_dtype != KLA_B200_BF16) return KLA_B200_EUNSUPPORTED;
    if (in_dtype == KLA_B200_F32 && out_dtype == KLA_B200_BF16) return KLA_B200_EUNSUPPORTED;
    if (B > 65535 || L > (1 << 30) || M > (1 << 30)) return KLA_B200_EUNSUPPORTED;
    return KLA_B200_OK;
}

// rows of t can be read and written two elements at a time
bool pair_ok(const kla_b200_tensor3 &t, size_t esz) {
    return (reinterpret_cast<uintptr_t>(t.ptr) % (2 * esz)) == 0 && t.stride_b % 2 == 0 && t.stride_t % 2 == 0;
}

int check_t3(const kla_b200_tensor3 &t, size_t esz, bool required) {
    if (t.ptr == nullptr) return required ? KLA_B200_EINVAL : KLA_B200_OK;
    if (!aligned(t.ptr, esz)) return KLA_B200_EALIGN;
    if (t.stride_b < 0 || t.stride_t < 0) return KLA_B200_EINVAL;
    return KLA_B200_OK;
}

constexpr int kMaxDevices = 64;
std::mutex g_symbol_mu;
int *g_status_ptr[kMaxDevices] = {};
// test hooks (kla_b200_test_hooks): wait limit and the tile whose hand-over the loader leaves incomplete
std::atomic<unsigned> g_wait_limit_ns{1000000000u};
std::atomic<int> g_skip_tile{-1};

// Device address of the status word on the current device (looked up on first use), with the current
// wait settings. Returns a C-ABI status.
int wait_ctl(WaitCtl *w) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e);
    if (dev < 0 || dev >= kMaxDevices) return KLA_B200_EUNSUPPORTED;
    {
        std::lock_guard<std::mutex> lock(g_symbol_mu);
        if (g_status_ptr[dev] == nullptr) {
            void *ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_kla_status);
            if (e != cudaSuccess) return cuda_fail(e);
            g_status_ptr[dev] = static_cast<int *>(ptr);
        }
        w->status = g_status_ptr[dev];
    }
    w->limit_ns = g_wait_limit_ns.load();
    w->skip_tile = g_skip_tile.load();
    return KLA_B200_OK;
}

// ---- sequences cut into segments (SegCtl, kla_common.cuh): the scratch behind the checkpoints and the plan
//   [forward: ticket (256 B) | done, one int per (b, m)] [backward: the same] [forward hand-over: float2 per lane]
//   [backward hand-over: 5 floats per lane]
constexpr size_t kSegAlign = 256;
size_t seg_round(size_t n) { return (n + kSegAlign - 1) / kSegAlign * kSegAlign; }
struct SegScratch {
    size_t flags;   // bytes of one direction's ticket + done block
    size_t hand_f;  // offset of the forward's hand-over records
    size_t hand_b;  // offset of the backward's
    size_t total;
};
// false when the sizes do not fit size_t
bool seg_scratch(int64_t B, int64_t M, int64_t S, SegScratch *out) {
    if (B <= 0 || M <= 0 || S <= 0) { *out = SegScratch{0, 0, 0, 0}; return true; }
    const size_t bm = (size_t)B * (size_t)M;  // B <= 65535 and M <= 2^30 (check_common)
    if (bm > SIZE_MAX / ((size_t)S * 64)) return false;
    const size_t lanes = bm * (size_t)S;
    out->flags = kSegAlign + seg_round(bm * sizeof(int));
    out->hand_f = 2 * out->flags;
    out->hand_b = out->hand_f + seg_round(lanes * sizeof(float2));
    out->total = out->hand_b + seg_round(lanes * 5 * sizeof(float));
    return true;
}
size_t ckpt_part_bytes(int64_t B, int64_t L, int64_t M, int64_t S) {
    const int64_t nt = (L + kCkptInterval - 1) / kCkptInterval;
    // saturating product: a size that does not fit size_t reads as SIZE_MAX, never as a small number
    size_t n = sizeof(float2);
    for (const int64_t f : {B, nt, M, S}) {
        if (n > SIZE_MAX / (size_t)f) return SIZE_MAX;
        n *= (size_t)f;
    }
    return n > SIZE_MAX - kSegAlign ? SIZE_MAX : seg_round(n);
}

// How many segments for `ctas` sequences of L steps (and their length). Segments pay when the sequences do not
// fill the SMs' CTA slots evenly. Measured on B200 at T=4096, M=1024, S=16 (ms without -> with): backward, two
// CTAs per SM: B=8 1.50 -> 1.42, B=10 2.35 -> 1.68, B=12 2.35 -> 1.96, B=14 2.97 -> 2.32, B=16 2.96 -> 2.60;
// forward, four per SM: B=10 0.62 -> 0.59, B=14 0.81 -> 0.65, B=16 0.81 -> 0.71, but B=8 0.44 -> 0.55: with
// fewer sequences than half its slots the waiting CTAs spread the running ones unevenly over the SMs. So: the
// backward whenever there are more sequences than SMs (16 segments up to two per SM, else 8), the forward from
// two sequences per SM on. KLA_B200_SEGMENTS=0 switches segments off, =N asks for N in both kernels.
// forced: -1 = the policy above, 0 / 1 = off, N = N segments. sms: SMs of the device.
int plan_segments_for(int64_t ctas, int64_t L, bool backward, int sms, int forced, int *seg_len) {
    *seg_len = (int)L;
    if (forced == 0 || forced == 1 || L <= 0) return 1;
    int want = 8;
    int64_t min_len = 256;  // shorter segments cost more in hand-overs than they even out (chunks of 256 steps: no gain)
    if (forced > 1) {
        want = forced;
        min_len = kTT;
    } else {
        if (sms <= 0 || ctas <= (backward ? sms : 2 * sms)) return 1;
        if (backward && ctas <= 2 * sms) want = 16;
    }
    int64_t len = (L + want - 1) / want;
    len = (len + kTT - 1) / kTT * kTT;  // whole tiles of both kernels (and whole checkpoint intervals)
    if (len < min_len) len = min_len;
    const int64_t n = (L + len - 1) / len;
    if (n < 2 || n > 65535) return 1;
    *seg_len = (int)len;
    return (int)n;
}

int plan_segments(int64_t ctas, int64_t L, bool backward, int *seg_len) {
    const char *env = getenv("KLA_B200_SEGMENTS");  // read per launch: the tests switch it within one process
    const int forced = env != nullptr ? atoi(env) : -1;
    int dev = 0, sms = 0;
    if (forced < 0 && (cudaGetDevice(&dev) != cudaSuccess ||
                       cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess))
        sms = 0;
    return plan_segments_for(ctas, L, backward, sms, forced, seg_len);
}

// Fill prm.seg for one direction and clear its ticket and done words. The working memory is the bytes behind the
// checkpoints, or, for a forward without checkpoints, the caller's `work` buffer of the same layout.
template <typename Params>
int seg_setup(Params &prm, void *ckpt, void *work, int64_t B, int64_t L, int64_t M, int64_t S, int lpc, bool backward,
              cudaStream_t st) {
    prm.seg = SegCtl{1, (int)L, nullptr, nullptr, nullptr};
    if ((ckpt == nullptr && work == nullptr) || L <= 0) return KLA_B200_OK;
    const int mc = scan_channels_per_cta(lpc);
    const int64_t ctas = ((M + mc - 1) / mc) * B;
    int seg_len = (int)L;
    const int nseg = plan_segments(ctas, L, backward, &seg_len);
    if (nseg <= 1) return KLA_B200_OK;
    SegScratch sc;
    if (!seg_scratch(B, M, S, &sc)) return KLA_B200_OK;
    const size_t base = ckpt != nullptr ? ckpt_part_bytes(B, L, M, S) : 0;
    if (base == SIZE_MAX) return KLA_B200_OK;
    unsigned char *p = static_cast<unsigned char *>(ckpt != nullptr ? ckpt : work) + base;
    unsigned char *flags = p + (backward ? sc.flags : 0);
    const cudaError_t e = cudaMemsetAsync(flags, 0, sc.flags, st);
    if (e != cudaSuccess) return cuda_fail(e);
    prm.seg.nseg = nseg;
    prm.seg.seg_len = seg_len;
    prm.seg.ticket = reinterpret_cast<int *>(flags);
    prm.seg.done = reinterpret_cast<int *>(flags + kSegAlign);
    prm.seg.hand = reinterpret_cast<float *>(p + (backward ? sc.hand_b : sc.hand_f));
    return KLA_B200_OK;
}

// Tensor maps of the forward's tiles (box: the CTA's channels x one tile of steps), then the launch.
template <typename T, typename TO, int LPC, bool PRIOR>
int prep_fwd(FwdParams &prm, const kla_b200_fwd_args &a, cudaStream_t st) {
    const int mc = scan_channels_per_cta(LPC);
    if (int rc = seg_setup(prm, a.ckpt, a.work, a.B, a.L, a.M, a.S, LPC, false, st)) return rc;
    prm.use_tma = !g_no_tma && make_tile_map<T>(&prm.tm_v, a.v, a.B, a.L, a.M, mc, kTT) &&
                  make_tile_map<T>(&prm.tm_lv, a.lambda_v, a.B, a.L, a.M, mc, kTT);
    if (prm.epilogue)  // z and gate tiles travel like v and lambda_v when they meet the tensor-map rules
        prm.epi_tma = !g_no_tma && (a.z.ptr == nullptr || make_tile_map<T>(&prm.tm_z, a.z, a.B, a.L, a.M, mc, kTT)) &&
                      (a.gate.ptr == nullptr || make_tile_map<T>(&prm.tm_gate, a.gate, a.B, a.L, a.M, mc, kTT));
    const cudaError_t e = launch_fwd<T, TO, LPC, PRIOR>(prm, st);
    g_launches++;
    return e == cudaSuccess ? KLA_B200_OK : cuda_fail(e);
}

template <typename T, typename TO, int LPC, bool PRIOR>
int prep_bwd(BwdParams &prm, const kla_b200_bwd_args &a, cudaStream_t st) {
    const int mc = scan_channels_per_cta(LPC);
    if (int rc = seg_setup(prm, const_cast<void *>(a.ckpt), nullptr, a.B, a.L, a.M, a.S, LPC, true, st)) return rc;
    prm.use_tma = !g_no_tma && make_tile_map<T>(&prm.tm_v, a.v, a.B, a.L, a.M, mc, kBwdTT) &&
                  make_tile_map<T>(&prm.tm_lv, a.lambda_v, a.B, a.L, a.M, mc, kBwdTT) &&
                  make_tile_map<TO>(&prm.tm_dy, a.dy, a.B, a.L, a.M, mc, kBwdTT) &&
                  (a.dy_var.ptr == nullptr || make_tile_map<TO>(&prm.tm_dyv, a.dy_var, a.B, a.L, a.M, mc, kBwdTT));
    const cudaError_t e = launch_bwd<T, TO, LPC, PRIOR>(prm, st);
    g_launches++;
    return e == cudaSuccess ? KLA_B200_OK : cuda_fail(e);
}

template <typename T, typename TO, int LPC, bool PRIOR>
int launch_step(const StepParams &prm, cudaStream_t st) {
    const long long threads = (long long)prm.B * prm.M * LPC;
    if ((threads + 127) / 128 > 0x7fffffffll) return KLA_B200_EUNSUPPORTED;  // grid.x limit
    const unsigned blocks = (unsigned)((threads + 127) / 128);
    kla_step_kernel<T, TO, LPC, PRIOR><<<blocks, 128, 0, st>>>(prm);
    g_launches++;
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? KLA_B200_OK : cuda_fail(e);
}

// Expand (dtype pair, lanes per channel, prior flag) into a template instantiation.
#define KLA_DISPATCH_LPC(FN, T, TO, PRIOR, lpc, ...)          \
    switch (lpc) {                                            \
        case 1: return FN<T, TO, 1, PRIOR>(__VA_ARGS__);      \
        case 2: return FN<T, TO, 2, PRIOR>(__VA_ARGS__);      \
        case 4: return FN<T, TO, 4, PRIOR>(__VA_ARGS__);      \
        case 8: return FN<T, TO, 8, PRIOR>(__VA_ARGS__);      \
        case 16: return FN<T, TO, 16, PRIOR>(__VA_ARGS__);    \
        case 32: return FN<T, TO, 32, PRIOR>(__VA_ARGS__);    \
        default: return KLA_B200_EUNSUPPORTED;                \
    }
#define KLA_DISPATCH_PRIOR(FN, T, TO, prior, lpc, ...)                  \
    if (prior) { KLA_DISPATCH_LPC(FN, T, TO, true, lpc, __VA_ARGS__) }  \
    else { KLA_DISPATCH_LPC(FN, T, TO, false, lpc, __VA_ARGS__) }
#define KLA_DISPATCH(FN, din, dout, prior, lpc, ...)                                         \
    do {                                                                                     \
        if ((din) == KLA_B200_F32 && (dout) == KLA_B200_F32) {                               \
            KLA_DISPATCH_PRIOR(FN, float, float, prior, lpc, __VA_ARGS__)                    \
        } else if ((din) == KLA_B200_BF16 && (dout) == KLA_B200_F32) {                       \
            KLA_DISPATCH_PRIOR(FN, __nv_bfloat16, float, prior, lpc, __VA_ARGS__)            \
        } else if ((din) == KLA_B200_BF16 && (dout) == KLA_B200_BF16) {                      \
            KLA_DISPATCH_PRIOR(FN, __nv_bfloat16, __nv_bfloat16, prior, lpc, __VA_ARGS__)    \
        } else {                                                                             \
            return KLA_B200_EUNSUPPORTED;                                                    \
        }                                                                                    \
    } while (0)

int dispatch_fwd(int din, int dout, bool prior, int lpc, FwdParams &prm, const kla_b200_fwd_args &a, cudaStream_t st) {
    KLA_DISPATCH(prep_fwd, din, dout, prior, lpc, prm, a, st);
}
int dispatch_bwd(int din, int dout, bool prior, int lpc, BwdParams &prm, const kla_b200_bwd_args &a, cudaStream_t st) {
    KLA_DISPATCH(prep_bwd, din, dout, prior, lpc, prm, a, st);
}
// Tensor maps of the aggregate kernel's tiles, then the launch.
template <typename T, typename TO, int LPC, bool PRIOR>
int prep_agg(AggParams &prm, const kla_b200_slab_args &a, cudaStream_t st) {
    const int mc = agg_channels_per_cta(LPC);
    const bool adj = a.adjoint != 0;
    prm.use_tma = !g_no_tma && a.L > 0 && make_tile_map<T>(&prm.tm_v, a.v, a.B, a.L, a.M, mc, kAggTT) &&
                  make_tile_map<T>(&prm.tm_lv, a.lambda_v, a.B, a.L, a.M, mc, kAggTT) &&
                  (!adj || (make_tile_map<TO>(&prm.tm_dy, a.dy, a.B, a.L, a.M, mc, kAggTT) &&
                            (a.dy_var.ptr == nullptr || make_tile_map<TO>(&prm.tm_dyv, a.dy_var, a.B, a.L, a.M, mc, kAggTT))));
    const cudaError_t e = launch_agg<T, TO, LPC, PRIOR>(prm, adj, st);
    g_launches++;
    return e == cudaSuccess ? KLA_B200_OK : cuda_fail(e);
}
int dispatch_slab(int din, int dout, bool prior, int lpc, AggParams &prm, const kla_b200_slab_args &a, cudaStream_t st) {
    KLA_DISPATCH(prep_agg, din, dout, prior, lpc, prm, a, st);
}
int dispatch_step(int din, int dout, bool prior, int lpc, const StepParams &prm, cudaStream_t st) {
    KLA_DISPATCH(launch_step, din, dout, prior, lpc, prm, st);
}
template <typename T, typename TO, int LPC, bool PRIOR>
int launch_step_layer(const StepLayerParams &prm, cudaStream_t st) {
    const long long threads = (long long)prm.B * prm.M * LPC;
    if ((threads + 127) / 128 > 0x7fffffffll) return KLA_B200_EUNSUPPORTED;  // grid.x limit
    const unsigned blocks = (unsigned)((threads + 127) / 128);
    kla_step_layer_kernel<T, TO, LPC, PRIOR><<<blocks, 128, 0, st>>>(prm);
    g_launches++;
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? KLA_B200_OK : cuda_fail(e);
}
int dispatch_step_layer(int din, int dout, bool prior, int lpc, const StepLayerParams &prm, cudaStream_t st) {
    KLA_DISPATCH(launch_step_layer, din, dout, prior, lpc, prm, st);
}

}  // namespace

namespace {
template <class Op>
int launch_rawscan(const kla_b200_rawscan_args *a, void *stream, bool takes_state0, bool gives_dstate0) {
    if (a == nullptr || a->B < 0 || a->L < 0 || a->N < 0) return KLA_B200_EINVAL;
    if (a->B > 65535 || a->L > (1 << 30) || a->N > (1 << 30)) return KLA_B200_EUNSUPPORTED;
    if ((!takes_state0 && a->state0 != nullptr) || (!gives_dstate0 && a->dstate0 != nullptr)) return KLA_B200_EINVAL;
    for (int i = 0; i < Op::NIN; ++i) {
        if (a->in[i] == nullptr) return KLA_B200_EINVAL;
        if (!aligned(a->in[i], sizeof(float))) return KLA_B200_EALIGN;
    }
    for (int k = 0; k < Op::NOUT; ++k) {
        if (a->out[k] == nullptr) return KLA_B200_EINVAL;
        if (!aligned(a->out[k], sizeof(float))) return KLA_B200_EALIGN;
    }
    if (a->B == 0 || a->N == 0) return KLA_B200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RawParams prm{};
    prm.B = (int)a->B; prm.L = (int)a->L; prm.N = (int)a->N;
    prm.NT = (int)((a->L + kRawTT - 1) / kRawTT);
    prm.state0 = a->state0; prm.dstate0 = a->dstate0;
    bool tma = !g_no_tma && a->L > 0;
    for (int i = 0; i < Op::NIN; ++i) {
        prm.in[i] = a->in[i];
        const kla_b200_tensor3 t{const_cast<float *>(a->in[i]), a->L * a->N, a->N};
        tma = tma && make_tile_map<float>(&prm.tm_in[i], t, a->B, a->L, a->N, kRawLC, kRawTT + (i == Op::HALO ? 1 : 0));
    }
    for (int k = 0; k < Op::NOUT; ++k) {
        prm.out[k] = a->out[k];
        const kla_b200_tensor3 t{a->out[k], a->L * a->N, a->N};
        tma = tma && make_tile_map<float>(&prm.tm_out[k], t, a->B, a->L, a->N, kRawLC, kRawTT);
    }
    prm.use_tma = tma;
    if (int rc = wait_ctl(&prm.wait)) return rc;
    prm.wait.skip_tile = -1;  // the hook is for the fused scan kernels
    auto kern = kla_rawscan_kernel<Op>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RawSmem<Op>::kTotal);
    if (e != cudaSuccess) return cuda_fail(e);
    dim3 grid((unsigned)((a->N + kRawLC - 1) / kRawLC), (unsigned)a->B);
    kern<<<grid, kRawLC + 32, RawSmem<Op>::kTotal, st>>>(prm);
    g_launches++;
    e = cudaGetLastError();
    return e == cudaSuccess ? KLA_B200_OK : cuda_fail(e);
}
}  // namespace


extern "C" {

int64_t kla_b200_ckpt_interval(void) { return kCkptInterval; }

size_t kla_b200_ckpt_bytes(int64_t B, int64_t L, int64_t M, int64_t S) {
    if (B <= 0 || L <= 0 || M <= 0 || S <= 0) return 0;
    if (B > 65535 || M > (1 << 30)) return SIZE_MAX;
    const size_t ck = ckpt_part_bytes(B, L, M, S);
    SegScratch sc;
    if (ck == SIZE_MAX || !seg_scratch(B, M, S, &sc) || ck > SIZE_MAX - sc.total) return SIZE_MAX;
    return ck + sc.total;
}

int kla_b200_plan_segments(int64_t sequences, int64_t L, int backward, int sms, int forced, int *seg_len) {
    int len = 0;
    const int n = plan_segments_for(sequences, L, backward != 0, sms, forced, &len);
    if (seg_len != nullptr) *seg_len = len;
    return n;
}

size_t kla_b200_segment_scratch_bytes(int64_t B, int64_t M, int64_t S) {
    SegScratch sc;
    if (B > 65535 || M > (1 << 30) || !seg_scratch(B, M, S, &sc)) return SIZE_MAX;
    return sc.total;
}

int kla_b200_scan_fwd(const kla_b200_fwd_args *a, void *stream) {
    if (a == nullptr) return KLA_B200_EINVAL;
    int rc = check_common(a->B, a->L, a->M, a->S, a->in_dtype, a->out_dtype);
    if (rc) return rc;
    const size_t esz = a->in_dtype == KLA_B200_F32 ? 4 : 2, osz = a->out_dtype == KLA_B200_F32 ? 4 : 2;
    const bool empty = a->B == 0 || a->M == 0 || a->S == 0;
    if (empty) return KLA_B200_OK;
    if (!a->a || !a->p || !a->lam_fin || !a->eta_fin) return KLA_B200_EINVAL;
    if ((a->lam0 == nullptr) != (a->eta0 == nullptr)) return KLA_B200_EINVAL;
    if (a->L > 0) {
        const kla_b200_tensor3 *ts[] = {&a->v, &a->lambda_v, &a->k, &a->q};
        for (const kla_b200_tensor3 *t : ts)
            if ((rc = check_t3(*t, esz, true))) return rc;
        if ((rc = check_t3(a->y, osz, true))) return rc;
        if ((rc = check_t3(a->y_var, osz, true))) return rc;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    FwdParams prm{};
    prm.B = (int)a->B; prm.L = (int)a->L; prm.M = (int)a->M; prm.S = (int)a->S;
    prm.NT = (int)((a->L + kTT - 1) / kTT);
    prm.NC = (int)((a->L + kCkptInterval - 1) / kCkptInterval);
    prm.v = t3(a->v); prm.lv = t3(a->lambda_v); prm.k = t3(a->k); prm.q = t3(a->q);
    prm.y = t3(a->y); prm.yv = t3(a->y_var);
    prm.a = a->a; prm.p = a->p; prm.lam0 = a->lam0; prm.eta0 = a->eta0;
    prm.lam_fin = a->lam_fin; prm.eta_fin = a->eta_fin;
    prm.ckpt = static_cast<float2 *>(a->ckpt);
    prm.lv_log_sigma = a->lambda_v_is_log_variance != 0;
    prm.obs_var_min = a->obs_var_min; prm.obs_var_max = a->obs_var_max;
    {
        const bool has_skip = a->lambda_skip_len != 0, has_gate = a->gate.ptr != nullptr;
        if (has_skip || has_gate) {
            // with a backward to follow, the scan's own outputs must be kept for the epilogue's adjoint
            // (the gate's adjoint reads them; the skip path alone does not)
            if (a->ckpt != nullptr && has_gate && (a->y_raw.ptr == nullptr || a->y_var_raw.ptr == nullptr)) return KLA_B200_EUNSUPPORTED;
            if ((a->y_raw.ptr == nullptr) != (a->y_var_raw.ptr == nullptr)) return KLA_B200_EINVAL;
            if (a->y_raw.ptr != nullptr) {
                if ((rc = check_t3(a->y_raw, osz, true)) || (rc = check_t3(a->y_var_raw, osz, true))) return rc;
                prm.y_raw = t3(a->y_raw); prm.yv_raw = t3(a->y_var_raw);
            }
            if (has_skip && ((a->lambda_skip_len != 1 && a->lambda_skip_len != a->M) || !a->lambda_skip || !a->z.ptr))
                return KLA_B200_EINVAL;
            if (a->gate_activation < KLA_B200_ACT_SILU || a->gate_activation > KLA_B200_ACT_NONE) return KLA_B200_EINVAL;
            if (has_skip && (rc = check_t3(a->z, esz, true))) return rc;
            if (has_gate && (rc = check_t3(a->gate, esz, true))) return rc;
            prm.epilogue = 1;
            if (has_skip) { prm.z = t3(a->z); prm.skip = a->lambda_skip; prm.skip_len = a->lambda_skip_len; }
            if (has_gate) { prm.gate = t3(a->gate); prm.gate_act = a->gate_activation; }
        }
    }
    if ((rc = wait_ctl(&prm.wait))) return rc;
    prm.vec_y = a->out_dtype == KLA_B200_F32 ? vec2_ok<float>(a->y) : vec2_ok<__nv_bfloat16>(a->y);
    prm.vec_yv = a->out_dtype == KLA_B200_F32 ? vec2_ok<float>(a->y_var) : vec2_ok<__nv_bfloat16>(a->y_var);
    return dispatch_fwd(a->in_dtype, a->out_dtype, a->decode_from_prior != 0, lpc_for(a->S), prm, *a, st);
}

int kla_b200_scan_bwd(const kla_b200_bwd_args *a, void *stream) {
    if (a == nullptr) return KLA_B200_EINVAL;
    int rc = check_common(a->B, a->L, a->M, a->S, a->in_dtype, a->out_dtype);
    if (rc) return rc;
    const size_t esz = a->in_dtype == KLA_B200_F32 ? 4 : 2, osz = a->out_dtype == KLA_B200_F32 ? 4 : 2;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t n_bls = (size_t)a->B * a->L * a->S, n_ms = (size_t)a->M * a->S, n_bms = (size_t)a->B * a->M * a->S;
    if (n_bls && (!a->dk || !a->dq)) return KLA_B200_EINVAL;
    if (n_ms && (!a->da || !a->dp)) return KLA_B200_EINVAL;
    if (n_bms && (!a->dlam0 || !a->deta0)) return KLA_B200_EINVAL;
    if ((a->lam0 == nullptr) != (a->eta0 == nullptr)) return KLA_B200_EINVAL;
    if ((a->dlam_fin == nullptr) != (a->deta_fin == nullptr)) return KLA_B200_EINVAL;
    cudaError_t e;
    if (n_bls) {
        if ((e = cudaMemsetAsync(a->dk, 0, n_bls * 4, st)) != cudaSuccess) return cuda_fail(e);
        if ((e = cudaMemsetAsync(a->dq, 0, n_bls * 4, st)) != cudaSuccess) return cuda_fail(e);
    }
    if (n_ms) {
        if ((e = cudaMemsetAsync(a->da, 0, n_ms * 4, st)) != cudaSuccess) return cuda_fail(e);
        if ((e = cudaMemsetAsync(a->dp, 0, n_ms * 4, st)) != cudaSuccess) return cuda_fail(e);
    }
    if (n_bms == 0) return KLA_B200_OK;
    if (a->L == 0) {  // nothing to scan: the state gradient passes straight through
        if (a->dlam_fin) {
            if ((e = cudaMemcpyAsync(a->dlam0, a->dlam_fin, n_bms * 4, cudaMemcpyDeviceToDevice, st)) != cudaSuccess) return cuda_fail(e);
            if ((e = cudaMemcpyAsync(a->deta0, a->deta_fin, n_bms * 4, cudaMemcpyDeviceToDevice, st)) != cudaSuccess) return cuda_fail(e);
        } else {
            if ((e = cudaMemsetAsync(a->dlam0, 0, n_bms * 4, st)) != cudaSuccess) return cuda_fail(e);
            if ((e = cudaMemsetAsync(a->deta0, 0, n_bms * 4, st)) != cudaSuccess) return cuda_fail(e);
        }
        return KLA_B200_OK;
    }
    if (!a->a || !a->p || !a->ckpt) return KLA_B200_EINVAL;
    const kla_b200_tensor3 *ts[] = {&a->v, &a->lambda_v, &a->k, &a->q, &a->dv, &a->dlambda_v};
    for (const kla_b200_tensor3 *t : ts)
        if ((rc = check_t3(*t, esz, true))) return rc;
    if ((rc = check_t3(a->dy, osz, true))) return rc;
    if ((rc = check_t3(a->dy_var, osz, false))) return rc;

    BwdParams prm{};
    prm.B = (int)a->B; prm.L = (int)a->L; prm.M = (int)a->M; prm.S = (int)a->S;
    prm.NT = (int)((a->L + kBwdTT - 1) / kBwdTT);
    prm.v = t3(a->v); prm.lv = t3(a->lambda_v); prm.k = t3(a->k); prm.q = t3(a->q);
    prm.dy = t3(a->dy); prm.dyv = t3(a->dy_var); prm.dv = t3(a->dv); prm.dlv = t3(a->dlambda_v);
    prm.a = a->a; prm.p = a->p; prm.lam0 = a->lam0; prm.eta0 = a->eta0;
    prm.ckpt = static_cast<const float2 *>(a->ckpt);
    prm.lv_log_sigma = a->lambda_v_is_log_variance != 0;
    prm.obs_var_min = a->obs_var_min; prm.obs_var_max = a->obs_var_max;
    prm.dlam_fin = a->dlam_fin; prm.deta_fin = a->deta_fin;
    prm.dk = a->dk; prm.dq = a->dq; prm.da = a->da; prm.dp = a->dp;
    prm.dlam0 = a->dlam0; prm.deta0 = a->deta0;
    if ((rc = wait_ctl(&prm.wait))) return rc;
    prm.vec_dv = a->in_dtype == KLA_B200_F32 ? vec2_ok<float>(a->dv) : vec2_ok<__nv_bfloat16>(a->dv);
    prm.vec_dlv = a->in_dtype == KLA_B200_F32 ? vec2_ok<float>(a->dlambda_v) : vec2_ok<__nv_bfloat16>(a->dlambda_v);
    return dispatch_bwd(a->in_dtype, a->out_dtype, a->decode_from_prior != 0, lpc_for(a->S), prm, *a, st);
}

int kla_b200_slab_aggregate(const kla_b200_slab_args *a, void *stream) {
    if (a == nullptr) return KLA_B200_EINVAL;
    int rc = check_common(a->B, a->L, a->M, a->S, a->in_dtype, a->out_dtype);
    if (rc) return rc;
    if (a->B == 0 || a->M == 0 || a->S == 0) return KLA_B200_OK;
    if (!a->a || !a->p || !a->out) return KLA_B200_EINVAL;
    if ((a->lam0 == nullptr) != (a->eta0 == nullptr)) return KLA_B200_EINVAL;
    const size_t esz = a->in_dtype == KLA_B200_F32 ? 4 : 2, osz = a->out_dtype == KLA_B200_F32 ? 4 : 2;
    if (a->L > 0) {
        if ((rc = check_t3(a->v, esz, true)) || (rc = check_t3(a->lambda_v, esz, true)) || (rc = check_t3(a->k, esz, true)))
            return rc;
        if (a->adjoint && ((rc = check_t3(a->q, esz, true)) || (rc = check_t3(a->dy, osz, true)) ||
                           (rc = check_t3(a->dy_var, osz, false))))
            return rc;
    }
    AggParams prm{};
    prm.B = (int)a->B; prm.L = (int)a->L; prm.M = (int)a->M; prm.S = (int)a->S;
    prm.v = t3(a->v); prm.lv = t3(a->lambda_v); prm.k = t3(a->k); prm.q = t3(a->q);
    prm.dy = t3(a->dy); prm.dyv = t3(a->dy_var);
    prm.a = a->a; prm.p = a->p; prm.lam0 = a->lam0; prm.eta0 = a->eta0; prm.out = a->out;
    if ((rc = wait_ctl(&prm.wait))) return rc;
    prm.wait.skip_tile = -1;  // the hook is for the scan kernels
    return dispatch_slab(a->in_dtype, a->out_dtype, a->decode_from_prior != 0, lpc_for(a->S), prm, *a,
                         static_cast<cudaStream_t>(stream));
}

int kla_b200_epilogue_bwd(const kla_b200_epilogue_bwd_args *a, void *stream) {
    if (a == nullptr || a->B < 0 || a->L < 0 || a->M < 0) return KLA_B200_EINVAL;
    if (a->in_dtype != KLA_B200_F32 && a->in_dtype != KLA_B200_BF16) return KLA_B200_EUNSUPPORTED;
    if (a->out_dtype != KLA_B200_F32 && a->out_dtype != KLA_B200_BF16) return KLA_B200_EUNSUPPORTED;
    if (a->in_dtype == KLA_B200_F32 && a->out_dtype == KLA_B200_BF16) return KLA_B200_EUNSUPPORTED;
    if (a->B > 65535 || a->L > (1 << 30) || a->M > (1 << 30)) return KLA_B200_EUNSUPPORTED;
    if (a->gate_activation < KLA_B200_ACT_SILU || a->gate_activation > KLA_B200_ACT_NONE) return KLA_B200_EINVAL;
    const bool has_skip = a->lambda_skip_len != 0, has_gate = a->gate.ptr != nullptr;
    if (has_skip && ((a->lambda_skip_len != 1 && a->lambda_skip_len != a->M) || !a->lambda_skip || !a->dlambda_skip)) return KLA_B200_EINVAL;
    const size_t esz = a->in_dtype == KLA_B200_F32 ? 4 : 2, osz = a->out_dtype == KLA_B200_F32 ? 4 : 2;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (has_skip && (e = cudaMemsetAsync(a->dlambda_skip, 0, sizeof(float) * (size_t)a->lambda_skip_len, st)) != cudaSuccess)
        return cuda_fail(e);
    if (a->B == 0 || a->L == 0 || a->M == 0) return KLA_B200_OK;
    int rc;
    if ((rc = check_t3(a->dout, osz, true)) || (rc = check_t3(a->dout_var, osz, false)) || (rc = check_t3(a->dy, osz, true)) ||
        (rc = check_t3(a->dy_var, osz, true)))
        return rc;
    if (has_gate && ((rc = check_t3(a->gate, esz, true)) || (rc = check_t3(a->dgate, esz, true)) ||
                     (rc = check_t3(a->y_raw, osz, true)) || (rc = check_t3(a->y_var_raw, osz, true))))
        return rc;
    if (has_skip && ((rc = check_t3(a->z, esz, true)) || (rc = check_t3(a->dz, esz, true)))) return rc;
    const long long row_blocks = (a->L + kEpiRows - 1) / kEpiRows;
    if (row_blocks > 65535) return KLA_B200_EUNSUPPORTED;
    EpilogueBwdParams prm{};
    prm.B = (int)a->B; prm.L = (int)a->L; prm.M = (int)a->M;
    prm.dout = t3(a->dout); prm.dout_var = t3(a->dout_var); prm.y_raw = t3(a->y_raw); prm.yv_raw = t3(a->y_var_raw);
    if (has_skip) { prm.z = t3(a->z); prm.dz = t3(a->dz); prm.skip = a->lambda_skip; prm.skip_len = a->lambda_skip_len; prm.dskip = a->dlambda_skip; }
    if (has_gate) { prm.gate = t3(a->gate); prm.dgate = t3(a->dgate); prm.gate_act = a->gate_activation; }
    prm.dy = t3(a->dy); prm.dy_var = t3(a->dy_var);
    // four channels per thread when every tensor can be read and written as 4-element vectors
    auto vec_ok = [&](const kla_b200_tensor3 &t, size_t sz) {
        return t.ptr == nullptr || (aligned(t.ptr, 4 * sz) && t.stride_b % 4 == 0 && t.stride_t % 4 == 0);
    };
    const bool vec = a->M % 4 == 0 && vec_ok(a->dout, osz) && vec_ok(a->dout_var, osz) && vec_ok(a->dy, osz) &&
                     vec_ok(a->dy_var, osz) && (!has_gate || (vec_ok(a->gate, esz) && vec_ok(a->dgate, esz) &&
                     vec_ok(a->y_raw, osz) && vec_ok(a->y_var_raw, osz))) && (!has_skip || (vec_ok(a->z, esz) && vec_ok(a->dz, esz)));
    const int per = vec ? 4 : 1;
    dim3 grid((unsigned)((a->M + 128 * per - 1) / (128 * per)), (unsigned)row_blocks, (unsigned)a->B);
#define KLA_EPI_LAUNCH(T, TO)                                                                                   \
    do {                                                                                                        \
        if (vec) {                                                                                              \
            if (has_skip && has_gate) kla_epilogue_bwd_kernel<T, TO, 4, true, true><<<grid, 128, 0, st>>>(prm);  \
            else if (has_skip) kla_epilogue_bwd_kernel<T, TO, 4, true, false><<<grid, 128, 0, st>>>(prm);        \
            else kla_epilogue_bwd_kernel<T, TO, 4, false, true><<<grid, 128, 0, st>>>(prm);                      \
        } else {                                                                                                \
            if (has_skip && has_gate) kla_epilogue_bwd_kernel<T, TO, 1, true, true><<<grid, 128, 0, st>>>(prm);  \
            else if (has_skip) kla_epilogue_bwd_kernel<T, TO, 1, true, false><<<grid, 128, 0, st>>>(prm);        \
            else kla_epilogue_bwd_kernel<T, TO, 1, false, true><<<grid, 128, 0, st>>>(prm);                      \
        }                                                                                                       \
    } while (0)
    if (!has_skip && !has_gate) return KLA_B200_EINVAL;  // nothing to differentiate
    if (a->in_dtype == KLA_B200_F32) KLA_EPI_LAUNCH(float, float);
    else if (a->out_dtype == KLA_B200_F32) KLA_EPI_LAUNCH(__nv_bfloat16, float);
    else KLA_EPI_LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef KLA_EPI_LAUNCH
    g_launches++;
    e = cudaGetLastError();
    return e == cudaSuccess ? KLA_B200_OK : cuda_fail(e);
}

int kla_b200_chunk_fold(const kla_b200_chunk_fold_args *a, void *stream) {
    if (a == nullptr || a->B < 0 || a->C < 1 || a->M < 0 || a->S < 0) return KLA_B200_EINVAL;
    if (a->S > KLA_B200_MAX_DSTATE || a->B * a->C > 65535 || a->M > (1 << 30)) return KLA_B200_EUNSUPPORTED;
    if (a->B == 0 || a->M == 0 || a->S == 0) return KLA_B200_OK;
    if (!a->agg || !a->out_a || !a->out_b || (a->in_a == nullptr) != (a->in_b == nullptr)) return KLA_B200_EINVAL;
    if (!aligned(a->agg, 16)) return KLA_B200_EALIGN;
    ChunkFoldParams prm{};
    prm.B = (int)a->B; prm.C = (int)a->C; prm.M = (int)a->M; prm.S = (int)a->S;
    prm.agg = a->agg; prm.in_a = a->in_a; prm.in_b = a->in_b; prm.out_a = a->out_a; prm.out_b = a->out_b;
    const long long lanes = a->B * a->M * a->S;
    const unsigned blocks = (unsigned)((lanes + 127) / 128);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (a->adjoint) kla_chunk_fold_kernel<true><<<blocks, 128, 0, st>>>(prm);
    else kla_chunk_fold_kernel<false><<<blocks, 128, 0, st>>>(prm);
    g_launches++;
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? KLA_B200_OK : cuda_fail(e);
}

int kla_b200_step(const kla_b200_step_args *a, void *stream) {
    if (a == nullptr) return KLA_B200_EINVAL;
    int rc = check_common(a->B, 1, a->M, a->S, a->in_dtype, a->out_dtype);
    if (rc) return rc;
    if (a->B == 0 || a->M == 0) return KLA_B200_OK;
    if (!a->v || !a->lambda_v || !a->y || !a->y_var || !a->a || !a->p) return KLA_B200_EINVAL;
    if (a->S > 0 && (!a->k || !a->q || !a->lam || !a->eta || !a->lam_out || !a->eta_out)) return KLA_B200_EINVAL;
    const size_t esz = a->in_dtype == KLA_B200_F32 ? 4 : 2, osz = a->out_dtype == KLA_B200_F32 ? 4 : 2;
    const void *ps[] = {a->v, a->lambda_v, a->k, a->q};
    for (const void *p : ps)
        if (p && !aligned(p, esz)) return KLA_B200_EALIGN;
    if (!aligned(a->y, osz) || !aligned(a->y_var, osz)) return KLA_B200_EALIGN;
    StepParams prm{};
    prm.B = (int)a->B; prm.M = (int)a->M; prm.S = (int)a->S;
    prm.v = a->v; prm.lv = a->lambda_v; prm.k = a->k; prm.q = a->q;
    prm.v_sb = a->v_stride_b; prm.lv_sb = a->lambda_v_stride_b; prm.k_sb = a->k_stride_b; prm.q_sb = a->q_stride_b;
    prm.a = a->a; prm.p = a->p; prm.lam = a->lam; prm.eta = a->eta;
    prm.y = a->y; prm.yv = a->y_var; prm.lam_out = a->lam_out; prm.eta_out = a->eta_out;
    prm.vec = a->S % 4 == 0 && aligned(a->lam, 16) && aligned(a->eta, 16) && aligned(a->a, 16) && aligned(a->p, 16) &&
              aligned(a->lam_out, 16) && aligned(a->eta_out, 16);
    int lpc = 1;
    while (lpc * 4 < a->S) lpc *= 2;
    return dispatch_step(a->in_dtype, a->out_dtype, a->decode_from_prior != 0, lpc, prm, static_cast<cudaStream_t>(stream));
}

int kla_b200_conv_step(const kla_b200_conv_step_args *a, void *stream) {
    if (a == nullptr || a->B < 0 || a->D < 0) return KLA_B200_EINVAL;
    if (a->K < 1 || a->K > KLA_B200_MAX_CONV_TAPS) return KLA_B200_EUNSUPPORTED;
    if (a->dtype != KLA_B200_F32 && a->dtype != KLA_B200_BF16) return KLA_B200_EUNSUPPORTED;
    if (a->activation < KLA_B200_ACT_SILU || a->activation > KLA_B200_ACT_NONE) return KLA_B200_EINVAL;
    if (a->B == 0 || a->D == 0) return KLA_B200_OK;
    if (!a->x || !a->weight || !a->z || (a->K > 1 && !a->state) || a->x_stride_b < 0) return KLA_B200_EINVAL;
    if (a->B * a->D > (1ll << 40)) return KLA_B200_EUNSUPPORTED;
    const size_t esz = a->dtype == KLA_B200_F32 ? 4 : 2;
    if (!aligned(a->x, esz) || !aligned(a->z, esz) || (a->state && !aligned(a->state, esz))) return KLA_B200_EALIGN;
    ConvStepParams prm{};
    prm.B = (int)a->B; prm.D = (int)a->D; prm.K = (int)a->K;
    prm.x = a->x; prm.x_sb = a->x_stride_b; prm.w = a->weight; prm.bias = a->bias;
    prm.state = a->state; prm.z = a->z; prm.act = a->activation;
    const unsigned blocks = (unsigned)((a->B * a->D + 127) / 128);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (a->dtype == KLA_B200_F32) kla_conv_step_kernel<float><<<blocks, 128, 0, st>>>(prm);
    else kla_conv_step_kernel<__nv_bfloat16><<<blocks, 128, 0, st>>>(prm);
    g_launches++;
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? KLA_B200_OK : cuda_fail(e);
}

int kla_b200_conv_seq(const kla_b200_conv_seq_args *a, void *stream) {
    if (a == nullptr || a->B < 0 || a->L < 0 || a->D < 0) return KLA_B200_EINVAL;
    if (a->K < 1 || a->K > KLA_B200_MAX_CONV_TAPS) return KLA_B200_EUNSUPPORTED;
    if (a->dtype != KLA_B200_F32 && a->dtype != KLA_B200_BF16) return KLA_B200_EUNSUPPORTED;
    if (a->activation < KLA_B200_ACT_SILU || a->activation > KLA_B200_ACT_NONE) return KLA_B200_EINVAL;
    if (a->B > 65535 || a->L > (1 << 30) || a->D > (1 << 30)) return KLA_B200_EUNSUPPORTED;
    if (a->B == 0 || a->D == 0 || a->L == 0) return KLA_B200_OK;
    if (!a->weight || (a->K > 1 && (!a->state || !a->state_out || a->state == a->state_out))) return KLA_B200_EINVAL;
    const size_t esz = a->dtype == KLA_B200_F32 ? 4 : 2;
    int rc;
    if ((rc = check_t3(a->x, esz, true))) return rc;
    if ((rc = check_t3(a->z, esz, true))) return rc;
    if ((a->state && !aligned(a->state, esz)) || (a->state_out && !aligned(a->state_out, esz))) return KLA_B200_EALIGN;
    const int64_t chunks = (a->L + kConvChunk - 1) / kConvChunk;
    if (chunks > 65535) return KLA_B200_EUNSUPPORTED;
    ConvSeqParams prm{};
    prm.B = (int)a->B; prm.L = (int)a->L; prm.D = (int)a->D; prm.K = (int)a->K;
    prm.x = t3(a->x); prm.z = t3(a->z); prm.w = a->weight; prm.bias = a->bias; prm.state = a->state;
    prm.state_out = a->state_out; prm.act = a->activation;
    // two channels per thread when every row starts on a 2-element boundary
    const bool pair = a->D % 2 == 0 && pair_ok(a->x, esz) && pair_ok(a->z, esz);
    const int64_t lanes = pair ? a->D / 2 : a->D;
    dim3 grid((unsigned)((lanes + 127) / 128), (unsigned)chunks, (unsigned)a->B);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define KLA_CONV_LAUNCH(KERNEL, T)                                                    \
    do {                                                                              \
        if (a->K <= 4) {                                                              \
            if (pair) KERNEL<T, 2, 4><<<grid, 128, 0, st>>>(prm);                     \
            else KERNEL<T, 1, 4><<<grid, 128, 0, st>>>(prm);                          \
        } else {                                                                      \
            if (pair) KERNEL<T, 2, kConvMaxTaps><<<grid, 128, 0, st>>>(prm);          \
            else KERNEL<T, 1, kConvMaxTaps><<<grid, 128, 0, st>>>(prm);               \
        }                                                                             \
    } while (0)
    if (a->dtype == KLA_B200_F32) KLA_CONV_LAUNCH(kla_conv_seq_kernel, float);
    else KLA_CONV_LAUNCH(kla_conv_seq_kernel, __nv_bfloat16);
#undef KLA_CONV_LAUNCH
    g_launches++;
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? KLA_B200_OK : cuda_fail(e);
}

int kla_b200_conv_seq_bwd(const kla_b200_conv_seq_bwd_args *a, void *stream) {
    if (a == nullptr || a->B < 0 || a->L < 0 || a->D < 0) return KLA_B200_EINVAL;
    if (a->K < 1 || a->K > KLA_B200_MAX_CONV_TAPS) return KLA_B200_EUNSUPPORTED;
    if (a->dtype != KLA_B200_F32 && a->dtype != KLA_B200_BF16) return KLA_B200_EUNSUPPORTED;
    if (a->activation < KLA_B200_ACT_SILU || a->activation > KLA_B200_ACT_NONE) return KLA_B200_EINVAL;
    if (a->B > 65535 || a->L > (1 << 30) || a->D > (1 << 30)) return KLA_B200_EUNSUPPORTED;
    if (a->B == 0 || a->D == 0 || a->L == 0) return KLA_B200_OK;
    if (!a->weight || !a->dweight) return KLA_B200_EINVAL;
    const size_t esz = a->dtype == KLA_B200_F32 ? 4 : 2;
    int rc;
    if ((rc = check_t3(a->x, esz, true)) || (rc = check_t3(a->dz, esz, true)) || (rc = check_t3(a->dx, esz, true))) return rc;
    if (a->state && !aligned(a->state, esz)) return KLA_B200_EALIGN;
    const int64_t chunks = (a->L + kConvBwdChunk - 1) / kConvBwdChunk;
    if (chunks > 65535) return KLA_B200_EUNSUPPORTED;
    ConvSeqBwdParams prm{};
    prm.B = (int)a->B; prm.L = (int)a->L; prm.D = (int)a->D; prm.K = (int)a->K;
    prm.x = t3(a->x); prm.dz = t3(a->dz); prm.dx = t3(a->dx); prm.w = a->weight; prm.bias = a->bias;
    prm.state = a->state; prm.dw = a->dweight; prm.dbias = a->dbias; prm.act = a->activation;
    // one channel per thread: with two, the backward's five register windows cost more in occupancy than the wider
    // accesses give back (0.35 against 0.22 ms at B=16, L=2048, D=1536, bfloat16)
    dim3 grid((unsigned)((a->D + 127) / 128), (unsigned)chunks, (unsigned)a->B);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define KLA_CONV_BWD_LAUNCH(T)                                                                  \
    do {                                                                                        \
        if (a->K <= 4) kla_conv_seq_bwd_kernel<T, 1, 4><<<grid, 128, 0, st>>>(prm);             \
        else kla_conv_seq_bwd_kernel<T, 1, kConvMaxTaps><<<grid, 128, 0, st>>>(prm);            \
    } while (0)
    if (a->dtype == KLA_B200_F32) KLA_CONV_BWD_LAUNCH(float);
    else KLA_CONV_BWD_LAUNCH(__nv_bfloat16);
#undef KLA_CONV_BWD_LAUNCH
    g_launches++;
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? KLA_B200_OK : cuda_fail(e);
}

int kla_b200_step_layer(const kla_b200_step_layer_args *a, void *stream) {
    if (a == nullptr) return KLA_B200_EINVAL;
    int rc = check_common(a->B, 1, a->M, a->S, a->in_dtype, a->out_dtype);
    if (rc) return rc;
    if (a->gate_activation < KLA_B200_ACT_SILU || a->gate_activation > KLA_B200_ACT_NONE) return KLA_B200_EINVAL;
    if (a->lambda_skip_len != 0 && a->lambda_skip_len != 1 && a->lambda_skip_len != a->M) return KLA_B200_EINVAL;
    if (a->B == 0 || a->M == 0) return KLA_B200_OK;
    if (!a->v || !a->log_sigma_v || !a->y || !a->y_var || !a->a || !a->p) return KLA_B200_EINVAL;
    if (a->S > 0 && (!a->k || !a->q || !a->lam || !a->eta || !a->lam_out || !a->eta_out)) return KLA_B200_EINVAL;
    if (a->lambda_skip_len != 0 && (!a->lambda_skip || !a->z)) return KLA_B200_EINVAL;
    const size_t esz = a->in_dtype == KLA_B200_F32 ? 4 : 2, osz = a->out_dtype == KLA_B200_F32 ? 4 : 2;
    const void *ps[] = {a->v, a->log_sigma_v, a->k, a->q, a->z, a->gate};
    for (const void *p : ps)
        if (p && !aligned(p, esz)) return KLA_B200_EALIGN;
    if (!aligned(a->y, osz) || !aligned(a->y_var, osz)) return KLA_B200_EALIGN;
    StepLayerParams prm{};
    prm.B = (int)a->B; prm.M = (int)a->M; prm.S = (int)a->S;
    prm.v = a->v; prm.ls = a->log_sigma_v; prm.k = a->k; prm.q = a->q;
    prm.z = a->lambda_skip_len != 0 ? a->z : nullptr; prm.gate = a->gate;
    prm.v_sb = a->v_stride_b; prm.ls_sb = a->log_sigma_v_stride_b; prm.k_sb = a->k_stride_b; prm.q_sb = a->q_stride_b;
    prm.z_sb = a->z_stride_b; prm.gate_sb = a->gate_stride_b;
    prm.a = a->a; prm.p = a->p; prm.lam = a->lam; prm.eta = a->eta;
    prm.lam_out = a->lam_out; prm.eta_out = a->eta_out; prm.y = a->y; prm.yv = a->y_var;
    prm.skip = a->lambda_skip_len != 0 ? a->lambda_skip : nullptr; prm.skip_len = a->lambda_skip_len;
    prm.obs_var_min = a->obs_var_min; prm.obs_var_max = a->obs_var_max; prm.clip = a->clip_value;
    prm.qk_norm = a->qk_norm; prm.gate_act = a->gate_activation;
    prm.vec = a->S % 4 == 0 && aligned(a->lam, 16) && aligned(a->eta, 16) && aligned(a->a, 16) && aligned(a->p, 16) &&
              aligned(a->lam_out, 16) && aligned(a->eta_out, 16);
    int lpc = 1;
    while (lpc * 4 < a->S) lpc *= 2;
    return dispatch_step_layer(a->in_dtype, a->out_dtype, a->decode_from_prior != 0, lpc, prm, static_cast<cudaStream_t>(stream));
}

const char *kla_b200_strerror(int code) {
    switch (code) {
        case KLA_B200_OK: return "ok";
        case KLA_B200_EINVAL: return "invalid argument (NULL pointer, negative size or stride, or half of a pointer pair missing)";
        case KLA_B200_EUNSUPPORTED: return "unsupported configuration (d_state above 128, unsupported dtype pair, or a dimension too large)";
        case KLA_B200_EALIGN: return "pointer not aligned to its element size";
        case KLA_B200_ETOOBIG: return "problem too large for the library's built-in checkpoint scratch (KLA_B200_STATIC_CKPT_BYTES); use kla_b200_scan_fwd with caller-provided scratch";
        case KLA_B200_ECUDA:
            snprintf(g_errbuf, sizeof(g_errbuf), "CUDA error: %s", cudaGetErrorString(g_last_cuda));
            return g_errbuf;
        default: return "unknown error code";
    }
}

int kla_b200_version(void) { return 100; }

int64_t kla_b200_launch_count(void) { return g_launches.load(); }

// ---------------------------------------------------------------------------
// Forward scan with its checkpoint scratch inside the library.
//
// The scratch is a fixed array in device memory that every GPU loading this
// library carries until the process exits. In host code the name of a
// __device__ array is only a handle, not an address a kernel can use, so the
// device address is looked up once per device with cudaGetSymbolAddress and
// cached here.
static __device__ __align__(256) unsigned char g_static_ckpt[KLA_B200_STATIC_CKPT_BYTES];

namespace {
std::mutex g_static_mu;
void *g_static_ckpt_ptr[kMaxDevices] = {};

// Device address of g_static_ckpt on the current device (set up on first use).
int static_ckpt_address(void **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e);
    if (dev < 0 || dev >= kMaxDevices) return KLA_B200_EUNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (g_static_ckpt_ptr[dev] == nullptr) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_ckpt);
        if (e != cudaSuccess) return cuda_fail(e);
        g_static_ckpt_ptr[dev] = ptr;
    }
    *out = g_static_ckpt_ptr[dev];
    return KLA_B200_OK;
}
}  // namespace

int kla_b200_scan_fwd_static(const kla_b200_fwd_args *args, void *stream, const void **ckpt) {
    if (args == nullptr || ckpt == nullptr) return KLA_B200_EINVAL;
    *ckpt = nullptr;
    int rc = check_common(args->B, args->L, args->M, args->S, args->in_dtype, args->out_dtype);
    if (rc) return rc;
    if (kla_b200_ckpt_bytes(args->B, args->L, args->M, args->S) > (size_t)KLA_B200_STATIC_CKPT_BYTES)
        return KLA_B200_ETOOBIG;
    void *scratch = nullptr;
    if ((rc = static_ckpt_address(&scratch))) return rc;
    kla_b200_fwd_args a = *args;
    a.ckpt = scratch;  // whatever the caller put there is ignored
    rc = kla_b200_scan_fwd(&a, stream);
    if (rc == KLA_B200_OK) *ckpt = scratch;
    return rc;
}

int kla_b200_mobius_scan_fwd(const kla_b200_rawscan_args *a, void *stream) {
    return launch_rawscan<MobiusFwd>(a, stream, true, false);
}
int kla_b200_mobius_scan_bwd(const kla_b200_rawscan_args *a, void *stream) {
    return launch_rawscan<MobiusBwd>(a, stream, true, true);
}
int kla_b200_affine_scan_fwd(const kla_b200_rawscan_args *a, void *stream) {
    return launch_rawscan<AffineFwd>(a, stream, false, false);
}
int kla_b200_affine_scan_bwd(const kla_b200_rawscan_args *a, void *stream) {
    return launch_rawscan<AffineBwd>(a, stream, false, false);
}

int kla_b200_device_status(int *status) {
    if (status == nullptr) return KLA_B200_EINVAL;
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(status, g_kla_status, sizeof(int));
    if (e != cudaSuccess) return cuda_fail(e);
    if (*status != 0) {
        e = cudaMemcpyToSymbol(g_kla_status, &zero, sizeof(int));
        if (e != cudaSuccess) return cuda_fail(e);
    }
    return KLA_B200_OK;
}

int kla_b200_test_hooks(int64_t wait_limit_ns, int32_t skip_tile) {
    if (wait_limit_ns < 0 || wait_limit_ns > 4000000000ll) return KLA_B200_EINVAL;
    g_wait_limit_ns.store(wait_limit_ns == 0 ? 1000000000u : (unsigned)wait_limit_ns);
    g_skip_tile.store(skip_tile < 0 ? -1 : skip_tile);
    return KLA_B200_OK;
}

}  // extern "C"
