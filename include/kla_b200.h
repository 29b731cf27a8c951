/*
 * kla_b200.h -- C ABI of the B200 (sm_100a) backend for the Kalman Linear
 * Attention scan.
 *
 * The library replaces one path of the reference package `kla`: the fused scan
 * `kla.ops.kla_scan` (forward and backward) and the single-token decode step
 * `kla.ops.kla_step`. Every entry point takes plain device pointers, sizes and
 * element strides; none takes or returns a torch type; none allocates device
 * memory (the caller owns outputs and scratch); none throws. All work is
 * enqueued on the CUDA stream passed in (`stream` is a `cudaStream_t` cast to
 * `void*`; NULL is the default stream) on the current device. The first scan
 * call on a device looks up the address of the library's status word on that
 * device; make that first call outside any stream capture.
 *
 * Notation follows the reference (src/kla/ops/kla_ops.py:1-32):
 *   B batch, L sequence length, M channels, S states per channel
 *   v, lambda_v, y, y_var : [B, L, M]   k, q : [B, L, S]   a, p : [M, S]
 *   filter state (lam, eta): [B, M, S]
 * Strides are in ELEMENTS. The innermost dimension always has unit stride.
 *
 * Return value: 0 on success, a KLA_B200_E* code otherwise (see
 * kla_b200_strerror). Errors are detected before any kernel is launched.
 */
#ifndef KLA_B200_H
#define KLA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KLA_B200_OK 0
#define KLA_B200_EINVAL 1      /* NULL pointer, negative size, bad stride or flag */
#define KLA_B200_EUNSUPPORTED 2 /* S above KLA_B200_MAX_DSTATE, unknown dtype */
#define KLA_B200_ECUDA 3       /* a CUDA runtime call failed (cudaGetLastError text via strerror) */
#define KLA_B200_EALIGN 4      /* pointer not aligned to its element size */
#define KLA_B200_ETOOBIG 5     /* kla_b200_scan_fwd_static: checkpoints would not fit the built-in scratch */

/* Largest d_state the kernels are instantiated for. The reference's fused
 * kernels have the same kind of cap (src/kla/ops/cuda_backend.py:134,274-275). */
#define KLA_B200_MAX_DSTATE 128

/* Element types of the activation tensors. `in_dtype` is the type of v,
 * lambda_v, k, q (and of the gradients dv, dlambda_v); `out_dtype` is the type
 * of y, y_var (and of the incoming dy, dy_var). The recurrence itself always
 * runs in float32, as in the reference (src/kla/ops/kla_ops.py:126-137), which
 * also returns float32 for low-precision inputs -- the (BF16, F32) pair.
 * Supported pairs: (F32, F32), (BF16, F32), (BF16, BF16). */
#define KLA_B200_F32 0
#define KLA_B200_BF16 1

/* Activation functions of the layer's gate and of its causal convolution. */
#define KLA_B200_ACT_SILU 0
#define KLA_B200_ACT_GELU 1
#define KLA_B200_ACT_RELU 2
#define KLA_B200_ACT_NONE 3

/* A [B, L, X] activation tensor: base pointer plus batch and time strides. */
typedef struct kla_b200_tensor3 {
    void *ptr;
    int64_t stride_b;
    int64_t stride_t;
} kla_b200_tensor3;

/*
 * Forward scan. Replaces the backend callable the reference dispatches to from
 * kla_scan (src/kla/ops/kla_ops.py:486-541; contract of the callable:
 * kla_scan_torch, src/kla/ops/kla_ops.py:188-290), including the fold
 * v*lambda_v (kla_ops.py:177), the floor on p (kla_ops.py:181-185), the floor
 * on a*a (kla_ops.py:240) and the optional read-out from the one-step-ahead
 * prior (kla_ops.py:284-286).
 */
typedef struct kla_b200_fwd_args {
    int64_t B, L, M, S;
    int32_t in_dtype, out_dtype; /* KLA_B200_F32 or KLA_B200_BF16 */
    int32_t decode_from_prior;
    kla_b200_tensor3 v, lambda_v; /* in  [B, L, M] */
    kla_b200_tensor3 k, q;        /* in  [B, L, S] */
    const float *a, *p;           /* in  [M, S] contiguous float32 */
    const float *lam0, *eta0;     /* in  [B, M, S] contiguous float32, or both NULL = unit prior (kla_ops.py:54-61) */
    kla_b200_tensor3 y, y_var;    /* out [B, L, M] */
    float *lam_fin, *eta_fin;     /* out [B, M, S] contiguous float32 */
    void *ckpt;                   /* out scratch of kla_b200_ckpt_bytes(), or NULL when no backward will follow */
    /* Fused sensor prologue (src/kla/layers/kla_layer.py:224-231). When
     * lambda_v_is_log_variance != 0 the lambda_v tensor holds the sensor
     * projection's raw log-variance output x and the kernels form
     * Lambda_v = 1 / min(softplus(x) + obs_var_min, obs_var_max) themselves
     * (no ceiling when obs_var_max <= 0), in float32 whatever in_dtype is. */
    int32_t lambda_v_is_log_variance;
    float obs_var_min, obs_var_max;
    /* Fused layer epilogue (src/kla/layers/kla_layer.py:329-338):
     * y += lambda_skip * z (when lambda_skip_len is 1 or M; z: [B, L, M] in
     * in_dtype), then y *= g, y_var *= g^2 with g = act(gate) (when gate.ptr is
     * not NULL; KLA_B200_ACT_*). When a backward will follow (ckpt != NULL) the
     * scan's own outputs, before skip and gate, must also be kept for the
     * epilogue's adjoint (kla_b200_epilogue_bwd): y_raw, y_var_raw, [B, L, M] in
     * out_dtype; without them the combination is refused with
     * KLA_B200_EUNSUPPORTED. */
    kla_b200_tensor3 z, gate;
    const float *lambda_skip;
    int32_t lambda_skip_len;
    int32_t gate_activation;
    kla_b200_tensor3 y_raw, y_var_raw; /* out, or ptr NULL */
    /* Optional, for a forward without checkpoints (ckpt == NULL): kla_b200_segment_scratch_bytes(B, M, S) bytes of
     * working memory, with which this forward too can hand its sequences from CTA to CTA in segments; NULL: it runs
     * unsegmented. Ignored when ckpt is given (the working memory then sits behind the checkpoints). */
    void *work;
} kla_b200_fwd_args;

/* Bytes of the scratch the forward writes for the backward: the filter state
 * of every lane once per kla_b200_ckpt_interval() steps (rounded up to 256
 * bytes), followed by kla_b200_segment_scratch_bytes(B, M, S) of working memory
 * that both kernels use when they cut the sequences into segments to even out
 * the load of the SMs (tickets, completion counts and the state handed from a
 * segment to the next: 28 bytes per (b, m, s) plus 8 per (b, m)). */
size_t kla_b200_ckpt_bytes(int64_t B, int64_t L, int64_t M, int64_t S);
size_t kla_b200_segment_scratch_bytes(int64_t B, int64_t M, int64_t S);
/* The segment plan the scan kernels use for `sequences` = B * ceil(M / channels per CTA) sequences of L steps on a
 * device with `sms` SMs: returns the segments per sequence (1 = unsegmented) and their length in *seg_len.
 * forced: -1 = the library's policy, 0 = off, N > 1 = N segments (what KLA_B200_SEGMENTS sets). No device call. */
int kla_b200_plan_segments(int64_t sequences, int64_t L, int backward, int sms, int forced, int *seg_len);
int64_t kla_b200_ckpt_interval(void);

int kla_b200_scan_fwd(const kla_b200_fwd_args *args, void *stream);

/*
 * Forward scan for callers that cannot allocate device memory. It has no
 * counterpart in the reference; it exists for hosts that are handed their
 * tensors by someone else and have no allocator of their own to ask for the
 * checkpoint scratch: a plugin running inside another runtime's memory arena,
 * a step that must not touch the allocator because an allocation there would
 * synchronise or fail, a real-time loop with a fixed memory budget.
 *
 * Same computation as kla_b200_scan_fwd in training mode, but the checkpoints
 * go to a fixed buffer of KLA_B200_STATIC_CKPT_BYTES that lives inside the
 * library (every GPU that loads the library holds it until the process exits).
 * args->ckpt is ignored; on success *ckpt receives the device address of the
 * built-in buffer, to be passed as kla_b200_bwd_args.ckpt to the backward of
 * the same step. Problems whose checkpoints (kla_b200_ckpt_bytes) exceed the
 * buffer are refused with KLA_B200_ETOOBIG and nothing is launched. The call
 * itself allocates nothing, on the host or on the device.
 *
 * The first call on each device looks up the buffer's address (the device must
 * be current); make that first call outside any stream capture. All calls on a
 * device share the one buffer and it keeps what the last call wrote: a forward
 * overwrites exactly the part its own backward will read, so nothing has to be
 * cleared, but a second forward issued before the first step's backward has
 * finished (other stream, other thread) overwrites that step's checkpoints --
 * calls that can overlap on the GPU race, so keep one step in flight per device.
 */
#define KLA_B200_STATIC_CKPT_BYTES (32u << 20)
int kla_b200_scan_fwd_static(const kla_b200_fwd_args *args, void *stream, const void **ckpt);

/*
 * Backward scan: exact adjoint of kla_b200_scan_fwd. Replaces what torch
 * autograd does for the reference's CPU path and what the reference's
 * hand-written fused adjoint does on its GPU paths
 * (src/kla/ops/kernels/mps/fused_kla_scan.metal:135-324; autograd wrapper
 * src/kla/ops/cuda_backend.py:196-236). Gradients flow into the carried state
 * (dlam0, deta0) and out of the returned one (dlam_fin, deta_fin), as the
 * reference requires (tests/test_backends.py:802-839).
 *
 * dk, dq, da, dp are accumulated with atomic adds after the library zeroes
 * them; dv, dlambda_v, dlam0, deta0 are written outright.
 */
typedef struct kla_b200_bwd_args {
    int64_t B, L, M, S;
    int32_t in_dtype, out_dtype;
    int32_t decode_from_prior;
    kla_b200_tensor3 v, lambda_v, k, q; /* in, as in the forward */
    const float *a, *p;
    const float *lam0, *eta0;           /* or both NULL */
    const void *ckpt;                   /* in: what the forward wrote (the working memory behind the checkpoints is written) */
    kla_b200_tensor3 dy;                /* in  [B, L, M] */
    kla_b200_tensor3 dy_var;            /* in  [B, L, M], ptr may be NULL = zero */
    const float *dlam_fin, *deta_fin;   /* in  [B, M, S] contiguous, or both NULL = zero */
    kla_b200_tensor3 dv, dlambda_v;     /* out [B, L, M] */
    float *dk, *dq;                     /* out [B, L, S] contiguous float32 */
    float *da, *dp;                     /* out [M, S] contiguous float32 */
    float *dlam0, *deta0;               /* out [B, M, S] contiguous float32 */
    /* as in kla_b200_fwd_args; dlambda_v then receives the gradient with respect to the log-variances */
    int32_t lambda_v_is_log_variance;
    float obs_var_min, obs_var_max;
} kla_b200_bwd_args;

int kla_b200_scan_bwd(const kla_b200_bwd_args *args, void *stream);

/*
 * Slab aggregate for the sequence-sharded scan. The reference has no
 * multi-device path; what it does have is the algebra this rests on: Moebius
 * maps compose associatively under a common rescaling
 * (src/kla/ops/kla_ops.py:76-116) and a carried state folds onto a scanned
 * chunk (src/kla/ops/kernels/triton/tiled_mobius_scan.py:91-102, 194-196).
 *
 * One 32-byte record per lane, out[B, M, S, 8]:
 *  adjoint == 0: the slab's state map in homogeneous coordinates (x, w, z),
 *    P = w/x, mean = z/x: (m00 m01 m10 m11 m20 m21 m22 0) with
 *    x' = m00 x + m01 w, w' = m10 x + m11 w, z' = m20 x + m21 w + m22 z, up to a
 *    common factor. Needs v, lambda_v, k, a, p only.
 *  adjoint != 0: with the slab's true initial state (lam0, eta0; NULL = unit
 *    prior) and the upstream dy, dy_var: (K00 K01 K11 b0 b1 P_end mean_end 0),
 *    where the backward carry (dL/dP, dL/dmean) leaving the slab's first step
 *    is [[K00 K01][0 K11]] c_in + (b0 b1) for a carry c_in entering at its end.
 */
typedef struct kla_b200_slab_args {
    int64_t B, L, M, S;
    int32_t in_dtype, out_dtype;
    int32_t decode_from_prior;
    int32_t adjoint;
    kla_b200_tensor3 v, lambda_v, k, q; /* q: adjoint only */
    const float *a, *p;
    const float *lam0, *eta0;           /* adjoint only; both NULL = unit prior */
    kla_b200_tensor3 dy, dy_var;        /* adjoint only; dy_var.ptr may be NULL */
    float *out;                         /* [B, M, S, 8] float32 */
} kla_b200_slab_args;

int kla_b200_slab_aggregate(const kla_b200_slab_args *args, void *stream);

/*
 * Adjoint of the fused layer epilogue. Replaces what torch autograd does for
 * the reference layer's output path (src/kla/layers/kla_layer.py:329-338:
 * y + lambda_skip * z, then the gate on y and its square on y_var). One
 * memory-bound pass: from the gradients of the gated outputs it forms the
 * gradients kla_b200_scan_bwd takes as dy, dy_var, plus dz, dgate and
 * dlambda_skip (accumulated with atomic adds after the library zeroes it).
 * z/dz and lambda_skip, or gate/dgate, are NULL when that half of the path is
 * absent. Activation tensors (z, gate, dz, dgate) are in_dtype, the others
 * out_dtype, as in the forward.
 */
typedef struct kla_b200_epilogue_bwd_args {
    int64_t B, L, M;
    int32_t in_dtype, out_dtype;
    int32_t gate_activation;        /* KLA_B200_ACT_* */
    int32_t lambda_skip_len;        /* 0 (none), 1 or M */
    kla_b200_tensor3 dout, dout_var; /* in  [B, L, M]; dout_var.ptr may be NULL = zero */
    kla_b200_tensor3 y_raw, y_var_raw; /* in: what the forward stored */
    kla_b200_tensor3 z, gate;       /* in, as in the forward */
    const float *lambda_skip;       /* in  [lambda_skip_len] */
    kla_b200_tensor3 dy, dy_var;    /* out [B, L, M], out_dtype */
    kla_b200_tensor3 dz, dgate;     /* out [B, L, M], in_dtype */
    float *dlambda_skip;            /* out [lambda_skip_len] float32 */
} kla_b200_epilogue_bwd_args;

int kla_b200_epilogue_bwd(const kla_b200_epilogue_bwd_args *args, void *stream);

/*
 * Fold of per-chunk aggregates for the time-parallel scan on one GPU. The
 * reference parallelises its scan over time with associative scans of
 * trace-normalised Moebius matrices and affine pairs
 * (src/kla/ops/kla_ops.py:76-123, 248, 274-280) and folds a carried state onto a
 * scanned chunk (src/kla/ops/kernels/triton/tiled_mobius_scan.py:86-102); this
 * is the carry pass of the same idea at chunk granularity.
 *
 * A [B, L, ...] problem whose (b, m) grid is too small to fill the GPU is cut
 * into C chunks of L/C steps that are scanned as B*C batch entries (entry
 * b*C + c is chunk c of batch element b; for tensors whose batch stride is
 * L times their time stride this is the same memory with other strides):
 *   1. kla_b200_slab_aggregate (adjoint = 0) over the B*C entries;
 *   2. kla_b200_chunk_fold (adjoint = 0): the state before each chunk,
 *      lam_in / eta_in [B*C, M, S], from the aggregates and the initial state;
 *   3. kla_b200_scan_fwd over the B*C entries with lam0 = lam_in, eta0 = eta_in;
 *      the state after the sequence is entry b*C + C-1 of lam_fin / eta_fin.
 * Backward: kla_b200_slab_aggregate (adjoint = 1, lam0 = lam_in, eta0 = eta_in),
 * kla_b200_chunk_fold (adjoint = 1) from the gradient of the returned state
 * (in_a = dlam_fin, in_b = deta_fin, [B, M, S], or both NULL), then
 * kla_b200_scan_bwd over the B*C entries with dlam_fin / deta_fin = the seeds
 * out_a / out_b; the gradient of the initial state is entry b*C of dlam0 / deta0.
 * The folds run in float64, one thread per (b, m, s).
 */
typedef struct kla_b200_chunk_fold_args {
    int64_t B, C, M, S;
    int32_t adjoint;
    const float *agg;         /* [B*C, M, S, 8] from kla_b200_slab_aggregate */
    const float *in_a, *in_b; /* [B, M, S] or both NULL: (lam0, eta0) / (dlam_fin, deta_fin) */
    float *out_a, *out_b;     /* [B*C, M, S]: (lam_in, eta_in) / (dlam_seed, deta_seed) */
} kla_b200_chunk_fold_args;

int kla_b200_chunk_fold(const kla_b200_chunk_fold_args *args, void *stream);

/*
 * One decode step. Replaces kla_step (src/kla/ops/kla_ops.py:293-331), which
 * the reference layer calls directly for single-token decode
 * (src/kla/layers/kla_layer.py:277-293). phi is floored at 1e-12 as there
 * (kla_ops.py:310-312). lam_out/eta_out may alias lam/eta (in-place update).
 * v, lambda_v, y, y_var: [B, M] with a batch stride; k, q: [B, S].
 */
typedef struct kla_b200_step_args {
    int64_t B, M, S;
    int32_t in_dtype, out_dtype;
    int32_t decode_from_prior;
    const void *v, *lambda_v;     /* [B, M] */
    int64_t v_stride_b, lambda_v_stride_b;
    const void *k, *q;            /* [B, S] */
    int64_t k_stride_b, q_stride_b;
    const float *a, *p;           /* [M, S] */
    const float *lam, *eta;       /* [B, M, S] */
    void *y, *y_var;              /* [B, M] contiguous */
    float *lam_out, *eta_out;     /* [B, M, S] */
} kla_b200_step_args;

int kla_b200_step(const kla_b200_step_args *args, void *stream);

/*
 * Decode of one layer, token by token: the elementwise work around the layer's
 * three projections as two calls. The projections themselves (in_proj,
 * sensor_proj, out_proj: plain GEMMs) stay with the caller.
 *
 * kla_b200_conv_step advances the causal depthwise convolution by one token.
 * Replaces CausalConv1d.forward for L = 1 (src/kla/layers/common.py:87-96):
 * z = act(bias + sum_j w[d, j] window[j]), window = (state, x), then the state
 * keeps the last K-1 inputs. x, state and z share one element type (dtype).
 */
#define KLA_B200_MAX_CONV_TAPS 8

typedef struct kla_b200_conv_step_args {
    int64_t B, D, K;      /* K taps, 1 <= K <= KLA_B200_MAX_CONV_TAPS */
    int32_t dtype;        /* KLA_B200_F32 or KLA_B200_BF16 */
    int32_t activation;   /* KLA_B200_ACT_* */
    const void *x;        /* in  [B, D] */
    int64_t x_stride_b;
    const float *weight;  /* in  [D, K] contiguous float32 (the [D, 1, K] parameter) */
    const float *bias;    /* in  [D] float32 or NULL */
    void *state;          /* in/out [B, D, K-1] contiguous */
    void *z;              /* out [B, D] contiguous */
} kla_b200_conv_step_args;

int kla_b200_conv_step(const kla_b200_conv_step_args *args, void *stream);

/*
 * The same convolution over a whole prompt: CausalConv1d.forward for L > 1
 * (src/kla/layers/common.py:87-96), in the layer's [B, L, D] layout (the
 * reference transposes to [B, D, L] and back around conv1d). state holds the
 * K-1 inputs before the prompt; the last K-1 inputs are written to state_out,
 * which must be a different buffer (blocks working on other parts of the prompt
 * still read state).
 */
typedef struct kla_b200_conv_seq_args {
    int64_t B, L, D, K;
    int32_t dtype, activation;
    kla_b200_tensor3 x;   /* in  [B, L, D] */
    const float *weight;  /* in  [D, K] */
    const float *bias;    /* in  [D] or NULL */
    const void *state;    /* in  [B, D, K-1] contiguous */
    void *state_out;      /* out [B, D, K-1] contiguous, not aliasing state */
    kla_b200_tensor3 z;   /* out [B, L, D] */
} kla_b200_conv_seq_args;

int kla_b200_conv_seq(const kla_b200_conv_seq_args *args, void *stream);

/*
 * Backward of kla_b200_conv_seq, i.e. what torch autograd computes for
 * CausalConv1d.forward (src/kla/layers/common.py:87-96: cat, conv1d, activation,
 * transposes): given x and the gradient dz of the activated output, dx and the
 * sums dweight, dbias. The pre-activation is recomputed from x; nothing else of
 * the forward is kept. dweight and dbias are ADDED to (zero them, or pass an
 * accumulator); no gradient is formed for the carried window.
 */
typedef struct kla_b200_conv_seq_bwd_args {
    int64_t B, L, D, K;
    int32_t dtype, activation;
    kla_b200_tensor3 x;   /* in  [B, L, D] */
    kla_b200_tensor3 dz;  /* in  [B, L, D] */
    const float *weight;  /* in  [D, K] */
    const float *bias;    /* in  [D] or NULL */
    const void *state;    /* in  [B, D, K-1] contiguous: the window before the sequence; NULL = zeros */
    kla_b200_tensor3 dx;  /* out [B, L, D] */
    float *dweight;       /* in/out [D, K] float32 */
    float *dbias;         /* in/out [D] float32 or NULL */
} kla_b200_conv_seq_bwd_args;

int kla_b200_conv_seq_bwd(const kla_b200_conv_seq_bwd_args *args, void *stream);

/*
 * kla_b200_step_layer is kla_b200_step with the layer's prologue and epilogue
 * folded in (src/kla/layers/kla_layer.py:199-231, 277-293, 329-338): it takes
 * the sensor projection's raw outputs and produces the input of out_proj.
 *   k, q       l2-normalised over S when qk_norm (x / max(|x|, 1e-12)), then
 *              clamped to [-clip_value, clip_value] when clip_value > 0
 *   lambda_v   1 / min(softplus(log_sigma_v) + obs_var_min, obs_var_max)
 *              (no upper clamp when obs_var_max <= 0)
 *   y, y_var   of kla_step, then y += lambda_skip * z (lambda_skip: one value or
 *              one per channel; skipped when NULL), then y *= g, y_var *= g^2 with
 *              g = act(gate) (skipped when gate is NULL)
 * All arithmetic is float32; with bfloat16 tensors the result is rounded once,
 * at the store (the reference rounds after several of these steps).
 */
typedef struct kla_b200_step_layer_args {
    int64_t B, M, S;
    int32_t in_dtype, out_dtype;
    int32_t decode_from_prior;
    int32_t qk_norm;
    int32_t gate_activation;      /* KLA_B200_ACT_* */
    int32_t lambda_skip_len;      /* 0 (none), 1 or M */
    float obs_var_min, obs_var_max, clip_value;
    const void *v, *log_sigma_v;  /* [B, M] */
    int64_t v_stride_b, log_sigma_v_stride_b;
    const void *k, *q;            /* [B, S], raw */
    int64_t k_stride_b, q_stride_b;
    const void *z, *gate;         /* [B, M] or NULL */
    int64_t z_stride_b, gate_stride_b;
    const float *lambda_skip;     /* [lambda_skip_len] float32 or NULL */
    const float *a, *p;           /* [M, S] */
    const float *lam, *eta;       /* [B, M, S] */
    void *y, *y_var;              /* [B, M] contiguous */
    float *lam_out, *eta_out;     /* [B, M, S]; may alias lam, eta */
} kla_b200_step_layer_args;

int kla_b200_step_layer(const kla_b200_step_layer_args *args, void *stream);

/*
 * Raw scan pair over materialised coefficients. Replaces the reference's
 * tiled_mobius_scan(A, B, C, D, lam0) and tiled_affine_scan(alpha, r)
 * (src/kla/ops/kernels/triton/tiled_mobius_scan.py:301-311) and their exact
 * backwards (TiledMobiusScan.backward, :266-279; TiledAffineScan.backward,
 * :289-296), for callers that already hold the per-(b, t, m, s) coefficients:
 *
 *   Moebius  lam_t = (A_t lam' + B_t) / max(C_t lam' + D_t, 1e-12),  lam_{-1} = lam0 (default 1)
 *   affine   eta_t = alpha_t eta' + r_t,                             eta_{-1} = 0
 *
 * Every tensor is a contiguous float32 [B, L, N] with N = M*S lanes per row
 * (the reference's [B, L, M, S]); state0 / dstate0 are [B, N].
 *
 *   call             in[]                       out[]
 *   mobius_scan_fwd  A B C D                    lam
 *   mobius_scan_bwd  A B C D lam dlam           dA dB dC dD   (+ dstate0 = dlam0, may be NULL)
 *   affine_scan_fwd  alpha r                    eta
 *   affine_scan_bwd  alpha eta deta             dalpha dr
 */
typedef struct kla_b200_rawscan_args {
    int64_t B, L, N;
    const float *in[6];
    float *out[4];
    const float *state0; /* Moebius calls: lam0 [B, N] or NULL = 1; affine calls: must be NULL */
    float *dstate0;      /* mobius_scan_bwd: out [B, N] or NULL; other calls: must be NULL */
} kla_b200_rawscan_args;

int kla_b200_mobius_scan_fwd(const kla_b200_rawscan_args *args, void *stream);
int kla_b200_mobius_scan_bwd(const kla_b200_rawscan_args *args, void *stream);
int kla_b200_affine_scan_fwd(const kla_b200_rawscan_args *args, void *stream);
int kla_b200_affine_scan_bwd(const kla_b200_rawscan_args *args, void *stream);

/* Human-readable text for a return code; for KLA_B200_ECUDA it includes the
 * CUDA error string of the failing call on this thread. */
const char *kla_b200_strerror(int code);

/* Library version, major*100 + minor. */
int kla_b200_version(void);

/* Number of kernels the library has launched in this process so far
 * (memsets are not counted). Used by the benchmark to report its launch count. */
int64_t kla_b200_launch_count(void);

/*
 * Device-side status of the kernels launched so far on the current device.
 * Synchronises with the device. *status is 0 when every kernel ran to the end;
 * 0x100 | site when a bounded wait inside a kernel (producer/consumer hand-off
 * between its warps) ran out and the kernel gave up instead of hanging -- the
 * outputs of that launch are then invalid. Reading a non-zero status clears it.
 */
int kla_b200_device_status(int *status);

/*
 * Test hooks for the bounded waits; not for production use. The reference has
 * no counterpart (its kernels use block-wide barriers, which cannot run out).
 * wait_limit_ns: how long a warp polls a hand-over barrier before it gives up
 *   (0 restores the default of one second).
 * skip_tile: the scan kernels' loader leaves the hand-over of this tile
 *   incomplete, so that the wait for it runs out after wait_limit_ns, the kernel
 *   returns and kla_b200_device_status reports 0x100 | site; -1 switches it off.
 * The settings are process-wide and are read when a scan is launched. A tile that
 * is skipped is loaded all the same: nothing is left in flight and nothing faults.
 */
int kla_b200_test_hooks(int64_t wait_limit_ns, int32_t skip_tile);

#ifdef __cplusplus
}
#endif

#endif /* KLA_B200_H */
