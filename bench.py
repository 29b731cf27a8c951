#!/usr/bin/env python
"""Benchmark of the KLA scan hot path on B200: forward + backward of the fused
scan at the headline raw-op workload (B=8, T=4096, M=1024, S=16, float32).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one forward + one backward pass of the scan over one batch of
synthetic input. With N > 1 (launched under torch.distributed.run) every rank
scans its own batch shard of the same size -- lanes are independent over
(batch, channel), so there is no data-path collective -- and the value is the
total over ranks divided by the slowest rank's time (weak scaling). The same
line carries two more measured blocks: ``strong`` -- the ONE B=8 problem split
over the N ranks by batch x channel with the gradient all-reduces inside the
timed region, checked against rank 0's one-GPU result -- and, for N > 1,
``seqshard`` -- the long sequence split into time slabs over the ranks.

Prints ONE JSON line (rank 0). ``--impl reference`` times the reference's own
CPU path instead (``kla.ops.kla_scan(..., backend="torch")`` forward and
``torch.autograd.grad``, from the unmodified copy under ``baseline/_ref``) on
the host cores; without that copy it times the CPU oracle (a port of the
reference's sequential float32 scan and its adjoint) and says so.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The workload: the raw op, float32, batch 8 x 4096 steps x 1024 channels x 16 states per channel.
WORK = dict(B=8, L=4096, M=1024, S=16)
METRIC = "KLA scan fwd+bwd tokens/s"
UNIT = "tokens/s"


def algorithmic_bytes_per_token(M, S, esz=4):
    """Compulsory HBM bytes of the fused op per (b, t) token: forward reads v,
    lambda_v (2M) and k, q (2S) and writes y, y_var (2M); backward reads dy,
    dyvar, v, lambda_v (4M) and k, q (2S) and writes dv, dlambda_v (2M) and dk,
    dq (2S). Checkpoints, re-reads and anything [B,L,M,S]-shaped are overhead."""
    fwd = esz * (4 * M + 2 * S)
    bwd = esz * (6 * M + 4 * S)
    return fwd, bwd


def ncu_traffic():
    """DRAM traffic per launch (bytes, read + write) from the last ncu captures of the kernels, kept as data
    beside the capture summaries (profiles/ncu_traffic.json: kernel -> bytes at the stated shape). A kernel
    that is missing there reports ``traffic: null``."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
            return {k: float(v["bytes"]) for k, v in json.load(f)["kernels"].items()}
    except (OSError, ValueError, KeyError):
        return {}


NCU_TRAFFIC = ncu_traffic()


def make_inputs(seed=0, **w):
    """Seeded synthetic inputs with the coefficient distributions the workload
    names: a = sigmoid(N(0,1)), p = softplus(N(0,1)), lambda_v = 1/softplus(N(0,1)),
    v ~ N(0,1), l2-normalised k, q ~ N(0,1) (as the reference layer does with
    qk_norm); upstream gradients ~ N(0,1) from seed+1."""
    import torch
    import torch.nn.functional as F

    B, L, M, S = w["B"], w["L"], w["M"], w["S"]
    g = torch.Generator(device="cpu").manual_seed(seed)
    v = torch.randn(B, L, M, generator=g)
    lambda_v = 1.0 / F.softplus(torch.randn(B, L, M, generator=g))
    k = torch.randn(B, L, S, generator=g)
    q = torch.randn(B, L, S, generator=g)
    k = k / k.norm(dim=-1, keepdim=True)
    q = q / q.norm(dim=-1, keepdim=True)
    a = torch.sigmoid(torch.randn(M, S, generator=g))
    p = F.softplus(torch.randn(M, S, generator=g))
    g1 = torch.Generator(device="cpu").manual_seed(seed + 1)
    dy = torch.randn(B, L, M, generator=g1)
    dyvar = torch.randn(B, L, M, generator=g1)
    return dict(v=v, lambda_v=lambda_v, k=k, q=q, a=a, p=p, dy=dy, dyvar=dyvar)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.gpu)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for n, val in zip(names, f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            sm.sort()
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(mx), samples=len(sm))
        out["reasons"] = sorted(reasons)
        return out


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def cpu_oracle_run(sample, threads=None):
    """Time the CPU oracle (float32, forward + backward) on `sample`; returns
    (tokens_per_s_at_full_width, seconds, threads). The sample keeps B*L tokens
    but may hold fewer channels than the workload: lanes are independent over
    channels, so cost is linear in M and the rate is scaled by M_sample/M."""
    import numpy as np

    # launchers such as torchrun export OMP_NUM_THREADS=1; the CPU legs use every host core
    if "kla_oracle" not in "".join(sys.modules):
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    from oracle import kla_oracle as O

    ins = make_inputs(**sample)
    arr = {n: t.numpy() for n, t in ins.items()}
    t0 = time.perf_counter()
    O.scan_fwd(arr["v"], arr["lambda_v"], arr["k"], arr["q"], arr["a"], arr["p"], dtype=np.float32)
    O.scan_bwd(arr["v"], arr["lambda_v"], arr["k"], arr["q"], arr["a"], arr["p"], arr["dy"], arr["dyvar"],
               dtype=np.float32)
    dt = time.perf_counter() - t0
    tokens = sample["B"] * sample["L"] * (sample["M"] / WORK["M"])
    return tokens / dt, dt, int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))


def headline_config(B=None):
    """The `config` object of the headline line; the same for both arms (the CPU arm says what bounded sample
    of it a step was under cpu_baseline.sample)."""
    B = WORK["B"] if B is None else B
    return {"workload": f"raw KLA scan fwd+bwd, B={B} T=4096 M=1024 S=16 per GPU, fp32 I/O and state"
                        + ("" if B == 8 else " (batch sweep, not the headline workload)"),
            **WORK, "sharding": "batch shard per rank, no collective",
            "l2": "inputs+outputs per step (1.1 GB) exceed the 126 MB L2; no explicit flush"}


def reference_dir():
    """Where the unmodified reference package lives (baseline/install_reference.py puts it there), or None."""
    d = os.path.join(ROOT, "baseline", "_ref")
    return d if os.path.isfile(os.path.join(d, "kla", "__init__.py")) else None


def cpu_reference_run(sample, threads=None):
    """Time the reference's own CPU path on `sample`: ``kla.ops.kla_scan(..., backend="torch")`` forward plus
    ``torch.autograd.grad`` with the seeded upstream gradients, float32, all host threads. Returns
    (tokens_per_s_at_full_width, seconds, threads); the sample may hold fewer channels than the workload (the
    reference's path needs ~240 B per (b, t, m, s), 128 GB for the whole workload), lanes are independent over
    channels, so the rate is scaled by M_sample/M."""
    import torch

    d = reference_dir()
    if d not in sys.path:
        sys.path.insert(0, d)
    from kla.ops import kla_scan

    n = threads or os.cpu_count() or 1
    torch.set_num_threads(n)
    ins = make_inputs(**sample)
    t = [ins[k].clone().requires_grad_(True) for k in ("v", "lambda_v", "k", "q", "a", "p")]
    t0 = time.perf_counter()
    y, y_var, _ = kla_scan(*t, backend="torch")
    torch.autograd.grad([y, y_var], t, [ins["dy"], ins["dyvar"]])
    dt = time.perf_counter() - t0
    tokens = sample["B"] * sample["L"] * (sample["M"] / WORK["M"])
    return tokens / dt, dt, n


def run_reference_torch_cpu(args):
    """The reference arm proper: the reference's own code on the host cores. One step = one channel block of
    128 channels of `bs` batch elements at full length (the blocks of the workload are independent), sized so
    that a step takes a few seconds."""
    cores = os.cpu_count() or 1
    sample = dict(B=1, L=WORK["L"], M=128, S=WORK["S"])
    cpu_reference_run(sample)                      # absorbs the compilation of the reference's associative scan
    _, dt, _ = cpu_reference_run(sample)
    sample["B"] = int(min(4, WORK["B"], max(1, round(3.0 / max(dt, 1e-3)))))  # memory: ~3 GB per batch element
    for _ in range(args.warmup):
        cpu_reference_run(sample)
    times = []
    for _ in range(args.steps):
        _, dt, _ = cpu_reference_run(sample)
        times.append(dt)
    tokens = sample["B"] * sample["L"] * (sample["M"] / WORK["M"])
    value = tokens * args.steps / sum(times)
    best = tokens / min(times)
    desc = (f"kla.ops.kla_scan(backend='torch') fwd + autograd.grad, float32: one block of M={sample['M']} of {WORK['M']} "
            f"channels x B={sample['B']} of {WORK['B']} batch elements x T={sample['L']} per step; rate scaled by the "
            f"block's share of the workload (blocks are independent; the whole workload does not fit host memory)")
    port_rate, port_dt, _ = cpu_oracle_run(dict(B=1, L=WORK["L"], M=256, S=WORK["S"]))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(times) / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": headline_config(),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "reference", "sample": desc,
                         "best_step": best},
        "cpu_port": {"value": port_rate, "unit": UNIT, "cores": cores, "kind": "port",
                     "sample": f"the C/OpenMP restatement of the same algorithm, B=1 x T={WORK['L']} x M=256, {port_dt:.2f} s"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_reference(args):
    """The reference arm: the reference's own CPU path when its package is installed under baseline/_ref,
    otherwise the reference's CPU algorithm as restated by the oracle (float32, OpenMP over channels); on the
    host cores, same workload definition."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if reference_dir() is not None:
        return run_reference_torch_cpu(args)
    cores = os.cpu_count() or 1
    # bounded sample: one batch element, all T, a channel block; calibrate its width
    sample = dict(B=1, L=WORK["L"], M=64, S=WORK["S"])
    rate, dt, _ = cpu_oracle_run(sample)
    # aim at ~5 s of CPU work per step: widen the channel block, then the batch
    units = max(1.0, 5.0 / max(dt, 1e-3))  # in 64-channel blocks of one batch element
    sample["M"] = int(min(WORK["M"], 64 * round(units)))
    sample["B"] = int(min(WORK["B"], max(1, round(units * 64 / WORK["M"]))))
    for _ in range(max(args.warmup, 1) if args.warmup else 0):
        cpu_oracle_run(sample)
    times, rates = [], []
    for _ in range(args.steps):
        r, dt, _ = cpu_oracle_run(sample)
        rates.append(r)
        times.append(dt)
    tot_tokens = sample["B"] * sample["L"] * (sample["M"] / WORK["M"]) * args.steps
    value = tot_tokens / sum(times)
    desc = (f"B={sample['B']} x T={sample['L']} x M={sample['M']} of {WORK['M']} channels x S={sample['S']} per step, "
            f"rate scaled by M/{WORK['M']} (lanes independent over channels)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(times) / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": headline_config(),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_b200(args):
    import torch
    import torch.distributed as dist

    import kla_b200
    lib = __import__("importlib").import_module("kalman-linear-attention_b200._lib")
    L = lib.load()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU fallback)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    B, T, M, S = WORK["B"], WORK["L"], WORK["M"], WORK["S"]
    if args.profile_batch:
        B = args.profile_batch
    host = make_inputs(seed=rank, **{**WORK, "B": B})
    d = {n: t.to(dev) for n, t in host.items()}
    # preallocated outputs and scratch: the C-ABI allocates nothing
    f32 = dict(device=dev, dtype=torch.float32)
    y, y_var = torch.empty(B, T, M, **f32), torch.empty(B, T, M, **f32)
    lam_fin, eta_fin = torch.empty(B, M, S, **f32), torch.empty(B, M, S, **f32)
    ckpt = torch.empty(L.kla_b200_ckpt_bytes(B, T, M, S), device=dev, dtype=torch.uint8)
    dv, dlv = torch.empty(B, T, M, **f32), torch.empty(B, T, M, **f32)
    dk, dq = torch.empty(B, T, S, **f32), torch.empty(B, T, S, **f32)
    da, dp = torch.empty(M, S, **f32), torch.empty(M, S, **f32)
    dlam0, deta0 = torch.empty(B, M, S, **f32), torch.empty(B, M, S, **f32)

    def t3(t):
        return lib.Tensor3(t.data_ptr(), t.stride(0), t.stride(1))

    P = lambda t: ctypes.c_void_p(t.data_ptr())
    fa = lib.FwdArgs(B=B, L=T, M=M, S=S, in_dtype=0, out_dtype=0, decode_from_prior=0,
                     v=t3(d["v"]), lambda_v=t3(d["lambda_v"]), k=t3(d["k"]), q=t3(d["q"]),
                     a=P(d["a"]), p=P(d["p"]), lam0=None, eta0=None, y=t3(y), y_var=t3(y_var),
                     lam_fin=P(lam_fin), eta_fin=P(eta_fin), ckpt=P(ckpt))
    ba = lib.BwdArgs(B=B, L=T, M=M, S=S, in_dtype=0, out_dtype=0, decode_from_prior=0,
                     v=t3(d["v"]), lambda_v=t3(d["lambda_v"]), k=t3(d["k"]), q=t3(d["q"]),
                     a=P(d["a"]), p=P(d["p"]), lam0=None, eta0=None, ckpt=P(ckpt),
                     dy=t3(d["dy"]), dy_var=t3(d["dyvar"]), dlam_fin=None, deta_fin=None,
                     dv=t3(dv), dlambda_v=t3(dlv), dk=P(dk), dq=P(dq), da=P(da), dp=P(dp),
                     dlam0=P(dlam0), deta0=P(deta0))
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    def step():
        lib.check(L.kla_b200_scan_fwd(ctypes.byref(fa), stream))
        lib.check(L.kla_b200_scan_bwd(ctypes.byref(ba), stream))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.profile_batch:
        if args.profile_chunks > 1:
            # the time-parallel path through the public API: aggregate, fold, forward; aggregate, fold, backward
            req = {n: d[n].clone().requires_grad_(True) for n in ("v", "lambda_v", "k", "q", "a", "p")}
            yy, yyv, _ = kla_b200.kla_scan_b200(*(req[n] for n in ("v", "lambda_v", "k", "q", "a", "p")),
                                                time_chunks=args.profile_chunks)
            torch.autograd.backward((yy, yyv), (d["dy"], d["dyvar"]))
        else:
            step()
        barrier()
        print(json.dumps({"profile_only": True, "B": B, "L": T, "M": M, "S": S, "time_chunks": max(args.profile_chunks, 1)}))
        return
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to start: begin before the warm-up
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    # ---- device-resident timing: K steps, CUDA events on the launching stream.
    # Inputs and gradients (4 x 134 MB read per step, 4 x 134 MB written) exceed
    # the 126 MB L2, so no explicit flush is needed between iterations.
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * args.steps + 1)]
    launches0 = L.kla_b200_launch_count()
    barrier()
    ev[0].record()
    for i in range(args.steps):
        lib.check(L.kla_b200_scan_fwd(ctypes.byref(fa), stream))
        ev[2 * i + 1].record()
        lib.check(L.kla_b200_scan_bwd(ctypes.byref(ba), stream))
        ev[2 * i + 2].record()
    barrier()
    launches = L.kla_b200_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    total_ms = ev[0].elapsed_time(ev[-1])
    fwd_ms = sum(ev[2 * i].elapsed_time(ev[2 * i + 1]) for i in range(args.steps)) / args.steps
    bwd_ms = sum(ev[2 * i + 1].elapsed_time(ev[2 * i + 2]) for i in range(args.steps)) / args.steps

    # ---- two more measured blocks on the same ranks (see their docstrings); a failure there must not cost
    # the headline, so it is reported in place of the block
    extra = {}
    if not args.batch:
        for name, fn, n in (("strong", strong_block, min(args.steps, 30)), ("seqshard", seqshard_block, min(args.steps, 5))):
            if name == "seqshard" and world < 2:
                continue
            try:
                extra[name] = fn(dev, rank, world, max(n, 1))
            except Exception as exc:  # noqa: BLE001
                if world > 1:
                    raise  # a rank that skips a collective would leave the others waiting
                extra[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
            torch.cuda.empty_cache()

    # ---- end to end through the public API with HOST buffers: pinned inputs
    # copied in, kla_scan_b200 + autograd, every result copied back out.
    pin = {n: t.pin_memory() for n, t in host.items()}
    outs_host = None
    e2e_steps = max(1, min(args.steps, 5))

    def e2e_step():
        # the package's host-buffer entry point: batch chunks on several streams, so copy-in, kernels and
        # copy-out of different chunks overlap (kalman-linear-attention_b200/hostpipe.py)
        nonlocal outs_host
        outs_host = kla_b200.scan_fwd_bwd_host(pin, dev, out=outs_host)
        return outs_host

    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    h2d = sum(t.numel() * t.element_size() for t in pin.values())
    d2h = sum(t.numel() * t.element_size() for t in outs_host.values())

    # ---- max over ranks
    tm = torch.tensor([total_ms, fwd_ms, bwd_ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    total_ms, fwd_ms, bwd_ms, e2e_ms = tm.tolist()
    tokens_step = B * T * world
    value = tokens_step * args.steps / (total_ms * 1e-3)
    e2e_value = tokens_step / (e2e_ms * 1e-3)

    if rank == 0:
        peak, peak_src = peaks()
        fb, bb = algorithmic_bytes_per_token(M, S)
        bwd_bytes, fwd_bytes = bb * B * T, fb * B * T
        ach_bwd = bwd_bytes / (bwd_ms * 1e-3) / 1e9
        ach_fwd = fwd_bytes / (fwd_ms * 1e-3) / 1e9
        ach_step = (fwd_bytes + bwd_bytes) / ((fwd_ms + bwd_ms) * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": headline_config(B),
            "roofline": {"bound": "hbm", "kernel": "kla_bwd_kernel", "achieved": ach_bwd, "peak": peak,
                         "unit": "GB/s", "frac": ach_bwd / peak, "traffic": NCU_TRAFFIC["kla_bwd_kernel"] * B / 8 if "kla_bwd_kernel" in NCU_TRAFFIC else None,
                         "peak_source": peak_src, "algorithmic_bytes": bwd_bytes, "ms": bwd_ms,
                         "nominal_peak_gbs": 8000.0, "frac_of_nominal": ach_bwd / 8000.0,
                         "note": "not HBM-bound at d_state=16: 66 warp-instructions per 32 lane-steps against 24.8 KB per "
                                 "token; ncu shows issue slots 71 % busy on average over all SMs (75 % on the busiest scheduler; the "
                                 "256 sequences run as 16 segments each, handed from CTA to CTA), the FP32 pipe 49 %"},
            "roofline_fwd": {"bound": "hbm", "kernel": "kla_fwd_kernel", "achieved": ach_fwd, "peak": peak,
                             "unit": "GB/s", "frac": ach_fwd / peak, "traffic": NCU_TRAFFIC["kla_fwd_kernel"] * B / 8 if "kla_fwd_kernel" in NCU_TRAFFIC else None,
                             "algorithmic_bytes": fwd_bytes, "ms": fwd_ms},
            "roofline_step": {"achieved": ach_step, "peak": peak, "unit": "GB/s", "frac": ach_step / peak},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "steps": e2e_steps},
            "gpu_launches": int(launches),
            "clocks": clocks,
            **extra,
        }
        if world == 1 and not args.no_cpu and reference_dir() is not None:
            sample = dict(B=2, L=T, M=128, S=S)
            cpu_reference_run(dict(sample, B=1))  # warm-up: the reference's associative scan is compiled on first use
            runs = [cpu_reference_run(sample) for _ in range(3)]
            rate, dt, cores = max(runs)
            line["cpu_baseline"] = {
                "value": rate, "unit": UNIT, "cores": cores, "kind": "reference",
                "sample": f"kla.ops.kla_scan(backend='torch') fwd + autograd.grad, float32, one block of B={sample['B']} x T={T} x "
                          f"M={sample['M']} of {M} channels, best of 3 after a warm-up ({dt:.1f} s); rate scaled by the block's "
                          f"share of the workload (blocks are independent; the whole workload needs ~128 GB on this path)"}
            prate, pdt, pcores = cpu_oracle_run(dict(B=1, L=T, M=512, S=S))
            line["cpu_port"] = {"value": prate, "unit": UNIT, "cores": pcores, "kind": "port",
                                "sample": f"the C/OpenMP restatement of the same algorithm, B=1 x T={T} x M=512, {pdt:.1f} s"}
        elif world == 1 and not args.no_cpu:
            sample = dict(B=1, L=T, M=128, S=S)
            rate, dt, cores = cpu_oracle_run(sample)
            # grow the sample towards ~10 s of CPU work: channels first, then batch
            units = max(1.0, 10.0 / max(dt, 1e-3))
            sample["M"] = int(min(M, 128 * round(units)))
            sample["B"] = int(min(WORK["B"], max(1, round(units * 128 / M))))
            rate, dt, cores = cpu_oracle_run(sample)
            line["cpu_baseline"] = {
                "value": rate, "unit": UNIT, "cores": cores, "kind": "port",
                "sample": f"B={sample['B']} x T={T} x M={sample['M']} of {M} channels x S={S}, float32 oracle fwd+bwd, "
                          f"{dt:.1f} s; rate scaled by M/{M} (lanes independent over channels)"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _event_time(fn, steps, warm, barrier):
    """Average milliseconds of fn() over `steps` calls, CUDA events on the current stream, after `warm` calls."""
    import torch

    for _ in range(warm):
        fn()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    barrier()
    return e0.elapsed_time(e1) / steps


def _dev_ratio(got, ref, rtol=1e-5, atol=1e-6):
    """max |got - ref| / (atol + rtol |ref|), on the device."""
    got, ref = got.detach().double(), ref.detach().double()
    return float(((got - ref).abs() / (atol + rtol * ref.abs())).max()) if ref.numel() else 0.0


def _dev_rel(got, ref):
    got, ref = got.detach().double(), ref.detach().double()
    return float((got - ref).abs().max() / (ref.abs().max() + 1.0)) if ref.numel() else 0.0


def strong_block(dev, rank, world, steps):
    """ONE problem of the headline shape split over the ranks by batch x channel (shard.block_of), forward +
    backward through the public API with the gradient all-reduces (da, dp over the batch group; dk, dq over the
    channel group) INSIDE the timed region. Every rank also runs the whole problem alone on its GPU: that is the
    parity reference (max deviation over all outputs and ranks) and the one-GPU time the efficiency is taken
    against. A rank's block holds few (batch, channel) lanes, so the scan cuts its sequence into time chunks."""
    import importlib

    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    import kla_b200
    shard = kla_b200.shard
    ops = importlib.import_module("kalman-linear-attention_b200.ops")

    B, T, M, S = 8, WORK["L"], WORK["M"], WORK["S"]
    g = torch.Generator(device=dev).manual_seed(4321)  # the same problem on every rank
    r = lambda *sh: torch.randn(*sh, device=dev, generator=g)
    v, lv = r(B, T, M), 1.0 / F.softplus(r(B, T, M))
    k, q = F.normalize(r(B, T, S), dim=-1), F.normalize(r(B, T, S), dim=-1)
    a, p = torch.sigmoid(r(M, S)), F.softplus(r(M, S))
    dy, dyv = r(B, T, M), r(B, T, M)
    full = [v, lv, k, q, a, p]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def run(ins, groups, gy, gyv, chunks=None):
        leaves = [t.detach().requires_grad_(True) for t in ins]
        if groups is None:
            y, yv, _ = kla_b200.kla_scan_b200(*leaves, time_chunks=chunks)
        else:
            y, yv, _ = shard.scan_block(kla_b200.kla_scan_b200, groups, *leaves)
        return (y, yv) + torch.autograd.grad([y, yv], leaves, [gy, gyv])

    ref = run(full, None, dy, dyv, chunks=1)
    t1 = _event_time(lambda: run(full, None, dy, dyv, chunks=1), steps, 3, barrier)

    blk = shard.block_of(B, M, world, rank)
    groups = shard.make_groups(world, blk.batch_parts, blk.channel_parts) if world > 1 else shard.Groups(None, None)
    bs, ms = slice(blk.b0, blk.b1), slice(blk.m0, blk.m1)
    mine = [v[bs, :, ms].contiguous(), lv[bs, :, ms].contiguous(), k[bs].contiguous(), q[bs].contiguous(),
            a[ms].contiguous(), p[ms].contiguous()]
    dyb, dyvb = dy[bs, :, ms].contiguous(), dyv[bs, :, ms].contiguous()
    out = run(mine, groups, dyb, dyvb)
    tn = _event_time(lambda: run(mine, groups, dyb, dyvb), steps, 3, barrier)

    # The same step with the host taken out of the way: at 8 ranks a block's kernels take about half a millisecond,
    # less than Python needs to issue them. The block's forward + backward (same kernels, same autograd path) are
    # captured once in a CUDA graph and replayed; the all-reduces are issued after each replay, outside the graph,
    # as one NCCL call per group (da and dp, and dk and dq, share a buffer).
    graphed = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                run(mine, None, dyb, dyvb)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            g_out = run(mine, None, dyb, dyvb)
            ap_buf = torch.stack([g_out[6], g_out[7]])   # da, dp
            kq_buf = torch.stack([g_out[4], g_out[5]])   # dk, dq

        def replay():
            graph.replay()
            if groups.batch_group is not None:
                dist.all_reduce(ap_buf, group=groups.batch_group)
            if groups.channel_group is not None:
                dist.all_reduce(kq_buf, group=groups.channel_group)

        tg = _event_time(replay, steps, 3, barrier)
        replay()
        dev_g = max(_dev_rel(ap_buf[0], ref[6][ms]), _dev_rel(ap_buf[1], ref[7][ms]),
                    _dev_rel(kq_buf[0], ref[4][bs]), _dev_rel(kq_buf[1], ref[5][bs]),
                    _dev_rel(g_out[0], ref[0][bs, :, ms]), _dev_rel(g_out[2], ref[2][bs, :, ms]))
        graphed = [tg, dev_g]
    except Exception as exc:  # noqa: BLE001
        if world > 1:
            raise
        graphed = f"{type(exc).__name__}: {exc}"[:200]

    y, yv, dv, dlv, dk, dq, da, dp = out
    ry, ryv, rdv, rdlv, rdk, rdq, rda, rdp = ref
    elem = max(_dev_ratio(y, ry[bs, :, ms]), _dev_ratio(yv, ryv[bs, :, ms]), _dev_ratio(dv, rdv[bs, :, ms]),
               _dev_ratio(dlv, rdlv[bs, :, ms]))
    red = max(_dev_rel(dk, rdk[bs]), _dev_rel(dq, rdq[bs]), _dev_rel(da, rda[ms]), _dev_rel(dp, rdp[ms]))
    tm = torch.tensor([tn, t1, elem, red] + (graphed if isinstance(graphed, list) else [0.0, 0.0]), device=dev,
                      dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    tn, t1, elem, red, tg, dev_g = tm.tolist()
    Bb, Mb = blk.b1 - blk.b0, blk.m1 - blk.m0
    return {
        "workload": f"ONE problem B={B} T={T} M={M} S={S} fp32 split over {world} rank(s): {blk.batch_parts} batch x "
                    f"{blk.channel_parts} channel blocks of B={Bb}, M={Mb}; forward + backward + all-reduces of da, dp "
                    f"(batch group) and dk, dq (channel group) timed together",
        "scaling": "strong", "ms_per_step": tn, "tokens_per_s": B * T / (tn * 1e-3),
        "one_gpu_ms_per_step": t1, "efficiency": t1 / (world * tn),
        "time_chunks_per_rank": ops.pick_time_chunks(Bb, T, Mb, S),
        "parity": {"elementwise_max_ratio_of_rtol1e-5_atol1e-6": elem, "reduced_gradients_max_rel_err": red,
                   "against": "the same problem scanned whole on one GPU by the lane-serial kernels"},
        "graphed": ({"ms_per_step": tg, "tokens_per_s": B * T / (tg * 1e-3), "efficiency": t1 / (world * tg),
                     "max_rel_err": dev_g,
                     "what": "the block's forward + backward replayed from a CUDA graph, the all-reduces issued after each "
                             "replay (one NCCL call per group): the same kernels without the host's launch cost"}
                    if isinstance(graphed, list) else {"error": graphed}),
        "steps": steps,
    }


def seqshard_block(dev, rank, world, steps):
    """The long sequence (B=2, T=131072, M=4096, S=16, bfloat16 I/O, float32 state) split into `world` time slabs,
    forward + backward through kla_scan_seq_sharded, with its all-gathers and all-reduces inside the timed region.
    Parity: the same slabs scanned one after the other by the plain kernels, the state handed from rank to rank
    (and the state gradient back) with point-to-point copies -- what one GPU would compute sequentially."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    import kla_b200

    B, T, M, S = 2, 131072, 4096, 16
    Ls = T // world
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    bf = torch.bfloat16
    r = lambda *sh: torch.randn(*sh, device=dev, generator=g)
    v, lv = r(B, Ls, M).to(bf), (1.0 / F.softplus(r(B, Ls, M))).to(bf)
    k, q = F.normalize(r(B, Ls, S), dim=-1).to(bf), F.normalize(r(B, Ls, S), dim=-1).to(bf)
    g0 = torch.Generator(device=dev).manual_seed(1234)  # a, p are shared by all ranks
    a = torch.sigmoid(torch.randn(M, S, generator=g0, device=dev))
    p = F.softplus(torch.randn(M, S, generator=g0, device=dev))
    dy, dyv = r(B, Ls, M).to(bf), r(B, Ls, M).to(bf)
    ins = [t.requires_grad_(True) for t in (v, lv, k, q, a, p)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        y, yv, st = kla_b200.kla_scan_seq_sharded(*ins, out_dtype=bf)
        return (y, yv, st) + torch.autograd.grad([y, yv], ins, [dy, dyv])

    out = step()
    ms = _event_time(step, steps, 2, barrier)

    # the same slabs, scanned one after the other by the plain kernels
    f32 = dict(device=dev, dtype=torch.float32)
    init = None
    if rank > 0:
        lam_in, eta_in = torch.empty(B, M, S, **f32), torch.empty(B, M, S, **f32)
        dist.recv(lam_in, src=rank - 1)
        dist.recv(eta_in, src=rank - 1)
        init = (lam_in.requires_grad_(True), eta_in.requires_grad_(True))
    leaves = [t.detach().requires_grad_(True) for t in ins]
    y2, yv2, st2 = kla_b200.kla_scan_b200(*leaves, initial_state=init, out_dtype=bf, time_chunks=1)
    if rank < world - 1:
        dist.send(st2.lam.detach().contiguous(), dst=rank + 1)
        dist.send(st2.eta.detach().contiguous(), dst=rank + 1)
        dl, de = torch.empty(B, M, S, **f32), torch.empty(B, M, S, **f32)
        dist.recv(dl, src=rank + 1)
        dist.recv(de, src=rank + 1)
    else:
        dl, de = torch.zeros(B, M, S, **f32), torch.zeros(B, M, S, **f32)
    g2 = torch.autograd.grad([y2, yv2, st2.lam, st2.eta], leaves + (list(init) if init else []), [dy, dyv, dl, de])
    if rank > 0:
        dist.send(g2[6].contiguous(), dst=rank - 1)
        dist.send(g2[7].contiguous(), dst=rank - 1)
    da2, dp2 = g2[4].clone(), g2[5].clone()
    if world > 1:
        dist.all_reduce(da2)
        dist.all_reduce(dp2)
    y, yv, st, dv, dlv, dk, dq, da, dp = out
    dev_out = max(_dev_rel(y, y2), _dev_rel(yv, yv2))
    dev_grad = max(_dev_rel(dv, g2[0]), _dev_rel(dlv, g2[1]), _dev_rel(dk, g2[2]), _dev_rel(dq, g2[3]),
                   _dev_rel(da, da2), _dev_rel(dp, dp2))
    dev_state = max(_dev_rel(st.lam, st2.lam), _dev_rel(st.eta, st2.eta)) if rank == world - 1 else 0.0
    tm = torch.tensor([ms, dev_out, dev_grad, dev_state], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    ms, dev_out, dev_grad, dev_state = tm.tolist()
    fb, bb = algorithmic_bytes_per_token(M, S, esz=2)
    peak, _ = peaks()
    return {
        "workload": f"sequence-sharded KLA scan fwd+bwd, B={B} T={T} M={M} S={S}, bf16 I/O, float32 state, time split "
                    f"into {world} slabs of {Ls} steps; slab aggregates, NCCL all-gathers and the da, dp all-reduce inside "
                    f"the timed region",
        "scaling": "strong", "ms_per_step": ms, "tokens_per_s": B * T / (ms * 1e-3), "steps": steps,
        "roofline_frac_per_gpu": (fb + bb) * B * T / world / (ms * 1e-3) / 1e9 / peak,
        "parity": {"outputs_max_rel_err": dev_out, "gradients_max_rel_err": dev_grad, "final_state_max_rel_err": dev_state,
                   "against": "the slabs scanned one after the other by the plain kernels, state and state gradient "
                              "handed from rank to rank (bf16 outputs: one rounding step is 4e-3 relative)"},
    }


def run_seqshard(args):
    """Secondary workload (not the default line): the long
    sequence split into time slabs over the ranks -- B=2, T=131072, M=4096, S=16,
    bfloat16 I/O with float32 state, forward + backward through
    ``kla_scan_seq_sharded`` (slab aggregates, NCCL all-gathers, fused scans).
    Strong scaling: the sequence is fixed, each of N ranks holds T/N steps."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    import kla_b200

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    B, T, M, S = 2, 131072, 4096, 16
    Ls = T // world
    g = torch.Generator(device=dev).manual_seed(rank)
    bf = torch.bfloat16
    v = torch.randn(B, Ls, M, generator=g, device=dev).to(bf)
    lv = (1.0 / F.softplus(torch.randn(B, Ls, M, generator=g, device=dev))).to(bf)
    k = torch.randn(B, Ls, S, generator=g, device=dev)
    q = torch.randn(B, Ls, S, generator=g, device=dev)
    k, q = (k / k.norm(dim=-1, keepdim=True)).to(bf), (q / q.norm(dim=-1, keepdim=True)).to(bf)
    g0 = torch.Generator(device=dev).manual_seed(1234)  # a, p are shared by all ranks
    a = torch.sigmoid(torch.randn(M, S, generator=g0, device=dev))
    p = F.softplus(torch.randn(M, S, generator=g0, device=dev))
    dy = torch.randn(B, Ls, M, generator=g, device=dev).to(bf)
    dyv = torch.randn(B, Ls, M, generator=g, device=dev).to(bf)
    ins = [t.requires_grad_(True) for t in (v, lv, k, q, a, p)]

    def step():
        y, yv, st = kla_b200.kla_scan_seq_sharded(*ins, out_dtype=bf)
        return torch.autograd.grad([y, yv], ins, [dy, dyv])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = ms.item()
        fb, bb = algorithmic_bytes_per_token(M, S, esz=2)
        peak, src = peaks()
        ach = (fb + bb) * B * T / world / (ms * 1e-3) / 1e9  # per GPU
        print(json.dumps({
            "metric": METRIC, "value": B * T / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "sequence-sharded KLA scan fwd+bwd, B=2 T=131072 M=4096 S=16, bf16 I/O, "
                                   "float32 state, time split into N slabs", "B": B, "L": T, "M": M, "S": S,
                       "slab": Ls},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                         "traffic": None, "peak_source": src, "note": "per GPU, whole step, algorithmic bytes"},
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_decode(args):
    """Secondary workload: the single-token decode step of the prefill-then-decode configuration
    (B=32, M=2048, S=16, float32 state updated in place), 256 steps per timed
    pass through the C ABI. State-bound: per step every lane's (lam, eta) is read
    and written (16 B) and a, p are read (8 B per (m, s), shared over the batch)."""
    import torch

    lib = __import__("importlib").import_module("kalman-linear-attention_b200._lib")
    L = lib.load()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, M, S, NSTEP = 32, 2048, 16, 256
    g = torch.Generator(device=dev).manual_seed(0)
    f32 = dict(device=dev, dtype=torch.float32)
    v = torch.randn(NSTEP, B, M, generator=g, **f32)
    lv = 1.0 / torch.nn.functional.softplus(torch.randn(NSTEP, B, M, generator=g, **f32))
    k = torch.nn.functional.normalize(torch.randn(NSTEP, B, S, generator=g, **f32), dim=-1)
    q = torch.nn.functional.normalize(torch.randn(NSTEP, B, S, generator=g, **f32), dim=-1)
    a = torch.sigmoid(torch.randn(M, S, generator=g, **f32))
    p = torch.nn.functional.softplus(torch.randn(M, S, generator=g, **f32))
    lam, eta = torch.ones(B, M, S, **f32), torch.zeros(B, M, S, **f32)
    y, yv = torch.empty(NSTEP, B, M, **f32), torch.empty(NSTEP, B, M, **f32)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    sa = [lib.StepArgs(B=B, M=M, S=S, in_dtype=0, out_dtype=0, decode_from_prior=0, v=P(v[t]), lambda_v=P(lv[t]),
                       v_stride_b=M, lambda_v_stride_b=M, k=P(k[t]), q=P(q[t]), k_stride_b=S, q_stride_b=S,
                       a=P(a), p=P(p), lam=P(lam), eta=P(eta), y=P(y[t]), y_var=P(yv[t]),
                       lam_out=P(lam), eta_out=P(eta)) for t in range(NSTEP)]

    def one_pass(st):
        for t in range(NSTEP):
            lib.check(L.kla_b200_step(ctypes.byref(sa[t]), st))

    for _ in range(max(args.warmup, 3)):
        one_pass(stream)
    torch.cuda.synchronize()
    # The 256 launches of a pass are captured once into a CUDA graph and replayed:
    # a decode step is a few microseconds of GPU work, less than a host-side launch.
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        one_pass(ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (args.steps * NSTEP)
    bytes_step = B * M * S * 16 + M * S * 8 + B * (2 * M + 2 * S + 2 * M) * 4
    peak, src = peaks()
    ach = bytes_step / (us * 1e-6) / 1e9
    print(json.dumps({
        "metric": "KLA decode steps/s (tokens/s = steps/s x batch)", "value": B / (us * 1e-6), "unit": UNIT,
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": us * NSTEP * 1e-3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "single-token decode step, B=32 M=2048 S=16, 256 steps per pass (one CUDA graph), state in place",
                   "us_per_decode_step": us, "note": "the 16 MB state stays in the 126 MB L2 between steps"},
        "roofline": {"bound": "hbm", "kernel": "kla_step_kernel", "achieved": ach, "peak": peak, "unit": "GB/s",
                     "frac": ach / peak, "traffic": None, "peak_source": src, "algorithmic_bytes": bytes_step},
    }), flush=True)


def run_rawpair(args):
    """Secondary line: the raw scan pair over materialised [B, L, M, S] coefficients
    (Moebius scan + affine scan, forward and backward: four launches per step), at the
    headline shape. These kernels move 12-40 bytes per lane-step and are HBM-bound."""
    import torch

    lib = __import__("importlib").import_module("kalman-linear-attention_b200._lib")
    L_ = lib.load()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, T, M, S = (args.batch or 4), WORK["L"], WORK["M"], WORK["S"]
    N = M * S
    g = torch.Generator(device=dev).manual_seed(0)
    f32 = dict(device=dev, dtype=torch.float32)
    shape = (B, T, N)
    # leaves in the filter's operating range: a contracting Moebius map and gains below one
    A = 0.5 + 0.5 * torch.rand(shape, generator=g, **f32)
    Bc = 0.1 * torch.rand(shape, generator=g, **f32)
    C = 0.2 * torch.rand(shape, generator=g, **f32)
    D = torch.ones(shape, **f32)
    alpha = 0.5 + 0.5 * torch.rand(shape, generator=g, **f32)
    r = torch.randn(shape, generator=g, **f32)
    dout = torch.randn(shape, generator=g, **f32)
    lam, eta = torch.empty(shape, **f32), torch.empty(shape, **f32)
    d4 = [torch.empty(shape, **f32) for _ in range(4)]
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    def mk(ins, outs):
        a = lib.RawScanArgs(B=B, L=T, N=N)
        for i, t in enumerate(ins):
            a.inp[i] = t.data_ptr()
        for i, t in enumerate(outs):
            a.out[i] = t.data_ptr()
        return a

    calls = [
        ("mobius_scan_fwd", mk((A, Bc, C, D), (lam,)), 5),
        ("mobius_scan_bwd", mk((A, Bc, C, D, lam, dout), d4), 10),
        ("affine_scan_fwd", mk((alpha, r), (eta,)), 3),
        ("affine_scan_bwd", mk((alpha, eta, dout), d4[:2]), 5),
    ]
    fns = [(name, getattr(L_, "kla_b200_" + name), a, words) for name, a, words in calls]

    def one_step(ev=None):
        for i, (name, fn, a, _) in enumerate(fns):
            if ev is not None:
                ev[i][0].record()
            lib.check(fn(ctypes.byref(a), stream))
            if ev is not None:
                ev[i][1].record()

    for _ in range(max(args.warmup, 3)):
        one_step()
    torch.cuda.synchronize()
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    evs = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in fns]
           for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        one_step(evs[i])
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    total_ms = e0.elapsed_time(e1)
    peak, src = peaks()
    per = {}
    for i, (name, _, _, words) in enumerate(fns):
        ms = sum(e[i][0].elapsed_time(e[i][1]) for e in evs) / args.steps
        by = words * 4 * B * T * N
        per[name] = {"ms": ms, "algorithmic_bytes": by, "achieved": by / (ms * 1e-3) / 1e9,
                     "frac": by / (ms * 1e-3) / 1e9 / peak}
    top = "mobius_scan_bwd"
    all_bytes = sum(v["algorithmic_bytes"] for v in per.values())
    print(json.dumps({
        "metric": "raw scan pair (Moebius + affine, fwd+bwd) tokens/s", "value": B * T * args.steps / (total_ms * 1e-3),
        "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "gpu_launches": 4 * args.steps,
        "config": {"workload": f"raw scan pair over [B, L, M, S] coefficients, B={B} T={T} M={M} S={S}, fp32; "
                               "four launches per step (Moebius fwd, bwd, affine fwd, bwd)",
                   "l2": f"each launch streams {5 * 4 * B * T * N / 1e9:.1f}-{10 * 4 * B * T * N / 1e9:.1f} GB, far beyond the 126 MB L2"},
        "roofline": {"bound": "hbm", "kernel": "kla_rawscan_kernel<MobiusBwd>", "achieved": per[top]["achieved"],
                     "peak": peak, "unit": "GB/s", "frac": per[top]["frac"], "traffic": NCU_TRAFFIC["rawscan_mobius_bwd_per_batch"] * B if "rawscan_mobius_bwd_per_batch" in NCU_TRAFFIC else None,
                     "peak_source": src, "algorithmic_bytes": per[top]["algorithmic_bytes"], "ms": per[top]["ms"]},
        "roofline_all": per,
        "step_gbs": all_bytes / (total_ms / args.steps * 1e-3) / 1e9,
        "clocks": clocks,
    }), flush=True)


def run_decode_layer(args):
    """Secondary line: one layer decoding token by token at the decode configuration
    (d_model 1024 -> M = 2048 channels, S = 16, batch 32): in_proj, conv step, sensor_proj,
    fused filter step, out_proj per token; 64 tokens captured in one CUDA graph. Beside it,
    the same arithmetic as the eager elementwise torch ops the reference layer issues
    (src/kla/layers/kla_layer.py:199-231, 277-345; kla_ops.py:293-331), also graph-captured,
    so the difference is the fusion and not launch overhead."""
    import torch
    import torch.nn.functional as F

    dec_mod = __import__("importlib").import_module("kalman-linear-attention_b200.decode")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, DM, S, K, NTOK = 32, 1024, 16, 4, 64
    M = 2 * DM
    dt = torch.bfloat16
    g = torch.Generator(device="cpu").manual_seed(0)
    rn = lambda *sh, scale=1.0: (torch.randn(*sh, generator=g) * scale)
    weights = {
        "in_proj.weight": rn(2 * M, DM, scale=DM ** -0.5).to(dt), "sensor_proj.weight": rn(2 * M + 2 * S, M, scale=M ** -0.5).to(dt),
        "out_proj.weight": rn(DM, M, scale=M ** -0.5).to(dt), "conv.weight": rn(M, 1, K, scale=0.5), "conv.bias": torch.zeros(M),
        "delta": rn(M, S) - 4.0, "lambda_log": rn(M, S, scale=0.1), "process_noise": torch.full((M, S), 0.01),
        "lambda_skip": torch.tensor(-1.0),
    }
    config = dict(d_state=S, discretization="ou", zero_process_noise=False, clip_value=None, obs_var_min=1e-4,
                  obs_var_max=None, value_rank="full", qk_norm=True, use_conv=True, conv_kernel_size=K,
                  conv_activation="silu", use_gating=True, gating_activation="silu", use_lambda_skip=True,
                  return_variance=False, decode_from_prior=False)
    dec = dec_mod.LayerDecoder(weights, config).to(dev)
    xs = rn(NTOK, B, DM).to(dev, dt)

    def eager_step(x, st):  # the reference route, op for op
        conv, lam, eta = st
        projected = F.linear(x, dec.w["in_proj.weight"])
        z, gate = projected.chunk(2, dim=-1)
        x_pad = torch.cat((conv, z.unsqueeze(-1)), dim=-1)
        zc = F.silu(F.conv1d(x_pad, dec.w["conv.weight"].to(dt), dec.w["conv.bias"].to(dt), groups=M)).squeeze(-1)
        conv.copy_(x_pad[..., 1:])
        v, ls, k, q = torch.split(F.linear(zc, dec.w["sensor_proj.weight"]), [M, M, S, S], dim=-1)
        k = k / k.norm(dim=-1, keepdim=True).clamp_min(1e-12)
        q = q / q.norm(dim=-1, keepdim=True).clamp_min(1e-12)
        lam_v = 1.0 / (F.softplus(ls.float()) + 1e-4)
        v, k, q = v.float(), k.float(), q.float()
        a, p = dec.a_bar, dec.p_bar.clamp_min(1e-12)
        a2 = (a * a).clamp_min(1e-12)
        phi = (lam_v.unsqueeze(-1) * (k * k).unsqueeze(1)).clamp_min(1e-12)
        r = (v * lam_v).unsqueeze(-1) * k.unsqueeze(1)
        inv = 1.0 / (a2 + p * lam).clamp_min(1e-12)
        lam.copy_(lam * inv + phi)
        eta.copy_(a * inv * eta + r)
        var = 1.0 / lam.clamp_min(1e-12)
        mean = eta * var
        y = torch.einsum("bms,bs->bm", mean, q).to(dt)
        y = y + dec.w["lambda_skip"].to(dt) * zc
        y = y * F.silu(gate)
        return F.linear(y, dec.w["out_proj.weight"])

    def graph_of(step_fn):
        st = dec.init_state(B, dev, dt)
        step_fn(xs[0], st)
        torch.cuda.synchronize()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for t in range(NTOK):
                    out = step_fn(xs[t], st)
        torch.cuda.current_stream().wait_stream(s)
        return gr, out

    def time_graph(gr):
        for _ in range(max(args.warmup, 3)):
            gr.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            gr.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (args.steps * NTOK)

    lib = __import__("importlib").import_module("kalman-linear-attention_b200._lib")
    n0 = lib.load().kla_b200_launch_count()
    g_fused, out_f = graph_of(dec.step)
    launches_per_pass = lib.load().kla_b200_launch_count() - n0 - 2
    g_eager, out_e = graph_of(eager_step)
    us_f, us_e = time_graph(g_fused), time_graph(g_eager)
    # bytes a token must move besides the three GEMMs: state (lam, eta, conv window) read + write, a, p, activations
    esz = 2
    bytes_tok = B * M * S * 16 + M * S * 8 + 2 * B * M * (K - 1) * esz + B * (2 * M + 2 * M + 2 * S + 3 * M) * esz
    gemm_bytes = (2 * M * DM + (2 * M + 2 * S) * M + DM * M) * esz
    peak, src = peaks()
    print(json.dumps({
        "metric": "KLA layer decode tokens/s (one layer, batch 32)", "value": B / (us_f * 1e-6), "unit": UNIT,
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": us_f * NTOK * 1e-3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 activations and projections, f32 filter state",
        "data": "synthetic", "gpu_launches": int(launches_per_pass) * args.steps,
        "config": {"workload": f"one KLA layer, token-by-token decode, B={B} d_model={DM} M={M} S={S} conv K={K}; "
                               f"{NTOK} tokens per pass in one CUDA graph; 3 GEMMs + 2 fused kernels per token",
                   "us_per_token": us_f, "eager_torch_us_per_token": us_e, "speedup_vs_eager_ops": us_e / us_f,
                   "note": "the eager line issues the reference layer's elementwise ops one by one, also graph-captured"},
        "roofline": {"bound": "hbm", "kernel": "per token: conv step + fused step + 3 GEMMs (weights re-read each token)",
                     "achieved": (bytes_tok + gemm_bytes) / (us_f * 1e-6) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": (bytes_tok + gemm_bytes) / (us_f * 1e-6) / 1e9 / peak, "traffic": None, "peak_source": src,
                     "algorithmic_bytes": bytes_tok + gemm_bytes,
                     "note": "state (32 MB) and weights (25 MB) fit the 126 MB L2 between tokens, so DRAM sees less than this"},
        "max_abs_diff_vs_eager": float((out_f.float() - out_e.float()).abs().max()),
    }), flush=True)


def run_prologue(args):
    """Secondary line: the scan with the layer's sensor prologue fused in (log-variance in, its
    gradient out; kla_layer.py:224-231) beside the same step with the prologue as the eager torch
    ops the reference layer issues (softplus, add, reciprocal and their autograd backward), both
    through the public autograd API at the headline shape."""
    import torch
    import torch.nn.functional as F
    import kla_b200

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, T, M, S = (args.batch or WORK["B"]), WORK["L"], WORK["M"], WORK["S"]
    host = make_inputs(seed=0, **{**WORK, "B": B})
    g = torch.Generator().manual_seed(7)
    x = torch.randn(B, T, M, generator=g).to(dev)
    d = {n: t.to(dev) for n, t in host.items()}
    leaves = [d["v"], x, d["k"], d["q"], d["a"], d["p"]]

    def fused():
        ins = [t.detach().requires_grad_(True) for t in leaves]
        y, yv, _ = kla_b200.kla_scan_b200(*ins, log_variance=(1e-4, None))
        return torch.autograd.grad([y, yv], ins, [d["dy"], d["dyvar"]])

    def eager():
        ins = [t.detach().requires_grad_(True) for t in leaves]
        lam_v = 1.0 / (F.softplus(ins[1]) + 1e-4)
        y, yv, _ = kla_b200.kla_scan_b200(ins[0], lam_v, *ins[2:])
        return torch.autograd.grad([y, yv], ins, [d["dy"], d["dyvar"]])

    def timeit(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps

    gf, ge = fused(), eager()
    diff = float((gf[1] - ge[1]).abs().max() / (ge[1].abs().max() + 1e-12))
    ms_f, ms_e = timeit(fused), timeit(eager)
    print(json.dumps({
        "metric": "KLA scan fwd+bwd with fused sensor prologue, tokens/s", "value": B * T / (ms_f * 1e-3), "unit": UNIT,
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_f, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"raw KLA scan fwd+bwd through autograd, B={B} T={T} M={M} S={S}, log-variance input "
                               "(precision formed inside the kernels)",
                   "ms_fused": ms_f, "ms_eager_prologue": ms_e, "speedup_vs_eager_prologue": ms_e / ms_f,
                   "max_rel_diff_of_dx": diff},
    }), flush=True)


def run_epilogue(args):
    """Secondary line: the scan with the layer's output path fused in for TRAINING (skip + gate applied at the forward
    kernel's store, their adjoint as one memory-bound kernel before the scan's backward; kla_layer.py:329-338) beside
    the same step with that path as the eager torch operations the reference layer issues and torch autograd's
    backward of them; both through the public autograd API at the headline shape."""
    import torch
    import torch.nn.functional as F
    import kla_b200

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, T, M, S = (args.batch or WORK["B"]), WORK["L"], WORK["M"], WORK["S"]
    host = make_inputs(seed=0, **{**WORK, "B": B})
    g = torch.Generator().manual_seed(7)
    z, gate = torch.randn(B, T, M, generator=g).to(dev), torch.randn(B, T, M, generator=g).to(dev)
    skip = torch.tensor(-1.0, device=dev)
    d = {n: t.to(dev) for n, t in host.items()}
    leaves = [d["v"], d["lambda_v"], d["k"], d["q"], d["a"], d["p"], z, gate, skip]

    def fused():
        ins = [t.detach().requires_grad_(True) for t in leaves]
        y, yv, _ = kla_b200.kla_scan_b200(*ins[:6], epilogue=dict(z=ins[6], gate=ins[7], lambda_skip=ins[8]))
        return torch.autograd.grad([y, yv], ins, [d["dy"], d["dyvar"]])

    def eager():
        ins = [t.detach().requires_grad_(True) for t in leaves]
        y, yv, _ = kla_b200.kla_scan_b200(*ins[:6])
        y = y + ins[8] * ins[6]
        gg = F.silu(ins[7])
        y, yv = y * gg, yv * gg.pow(2)
        return torch.autograd.grad([y, yv], ins, [d["dy"], d["dyvar"]])

    gf, ge = fused(), eager()
    diff = max(float((a_ - b_).abs().max() / (b_.abs().max() + 1e-12)) for a_, b_ in zip(gf, ge))
    sync = torch.cuda.synchronize
    ms_f = _event_time(fused, args.steps, max(args.warmup, 3), sync)
    ms_e = _event_time(eager, args.steps, max(args.warmup, 3), sync)
    print(json.dumps({
        "metric": "KLA scan fwd+bwd with fused skip/gate epilogue, tokens/s", "value": B * T / (ms_f * 1e-3), "unit": UNIT,
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_f, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"raw KLA scan fwd+bwd through autograd, B={B} T={T} M={M} S={S}, with y += skip*z, y *= silu(gate), "
                               "y_var *= silu(gate)^2 and the gradients of z, gate, skip",
                   "ms_fused": ms_f, "ms_eager_epilogue": ms_e, "speedup_vs_eager_epilogue": ms_e / ms_f,
                   "max_rel_diff_of_gradients": diff},
    }), flush=True)


def run_conv(args):
    """Secondary line: the layer's causal depthwise convolution with its activation, forward + backward, at the
    training step's shape (B=16, L=2048, D=1536, 4 taps, silu, bfloat16) through ``causal_conv_b200`` beside the same
    operation as the reference module issues it (transpose, cat with the carried window, conv1d, activation, transpose
    back; src/kla/layers/common.py:87-96) with torch autograd's backward."""
    import torch
    import torch.nn.functional as F
    import kla_b200

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, L, D, K = (args.batch or 16), 2048, 1536, 4
    g = torch.Generator().manual_seed(0)
    x = torch.randn(B, L, D, generator=g).to(dev, torch.bfloat16)
    w = (0.5 * torch.randn(D, 1, K, generator=g)).to(dev)
    bias = torch.randn(D, generator=g).to(dev)
    dz = torch.randn(B, L, D, generator=g).to(dev, torch.bfloat16)

    def ours():
        ins = [t.detach().requires_grad_(True) for t in (x, w, bias)]
        z, _ = kla_b200.layer.causal_conv_b200(*ins, None, "silu")
        return torch.autograd.grad(z, ins, dz)

    def module_math():
        ins = [t.detach().requires_grad_(True) for t in (x, w, bias)]
        x_t = ins[0].transpose(1, 2)
        x_pad = torch.cat((torch.zeros(B, D, K - 1, device=dev, dtype=x_t.dtype), x_t), dim=-1)
        z = F.silu(F.conv1d(x_pad, ins[1].to(x_t.dtype), ins[2].to(x_t.dtype), groups=D)).transpose(1, 2)
        return torch.autograd.grad(z, ins, dz)

    go, gm = ours(), module_math()
    diff = max(float((a_.float() - b_.float()).abs().max() / (b_.float().abs().max() + 1e-12)) for a_, b_ in zip(go, gm))
    sync = torch.cuda.synchronize
    ms_o = _event_time(ours, args.steps, max(args.warmup, 3), sync)
    ms_m = _event_time(module_math, args.steps, max(args.warmup, 3), sync)
    print(json.dumps({
        "metric": "causal depthwise conv + activation fwd+bwd, tokens/s", "value": B * L / (ms_o * 1e-3), "unit": UNIT,
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_o, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"CausalConv1d forward + backward, B={B} L={L} D={D} K={K}, silu, [B, L, D] layout",
                   "ms_b200": ms_o, "ms_torch_module_math": ms_m, "speedup": ms_m / ms_o,
                   "max_rel_diff_of_gradients_bf16": diff},
    }), flush=True)


def run_generate(args):
    """Secondary line: prompt prefill and token-by-token decode of a whole model -- the reference's
    ``SequenceModel(ModelConfig(vocab 50304, d_model 768, 12 layers), KLAConfig(d_state=16))``, bf16, batch 32, a prompt of
    512 tokens and 128 generated ones, greedy -- through ``ModelDecoder`` (fused decode kernels per layer, the token loop
    one CUDA graph) beside the reference's own ``SequenceModel.generate`` on its torch backend."""
    import torch

    if reference_dir() is None:
        print(json.dumps({"workload": "generate", "unavailable": "the reference is not installed under baseline/_ref"}))
        return
    sys.path.insert(0, reference_dir())
    import kla_b200
    from kla import KLAConfig, ModelConfig, SequenceModel

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, LP, NEW, V = (args.batch or 32), 512, 128, 50304
    torch.manual_seed(0)
    model = SequenceModel(ModelConfig(vocab_size=V, d_model=768, n_layers=12), KLAConfig(d_state=16, backend="torch"))
    model = model.to(dev).to(torch.bfloat16).eval()
    ids = torch.randint(0, V, (B, LP), device=dev, generator=torch.Generator(device=dev).manual_seed(1))
    dec = kla_b200.ModelDecoder.from_model(model)

    def timed(fn, n):
        fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            out = fn()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / n, out

    n = max(1, min(args.steps, 3))
    t_dec, out = timed(lambda: dec.generate(ids, NEW), n)
    t_pre, _ = timed(lambda: dec.prefill(ids), n)
    t_ref, ref = timed(lambda: model.generate(ids, NEW, temperature=0.0), 1)
    same = float((out[:, LP:] == ref[:, LP:]).float().mean())
    first = float((out[:, LP] == ref[:, LP]).float().mean())
    per_tok = (t_dec - t_pre) / (NEW - 1)
    print(json.dumps({
        "workload": "generate", "metric": "decode tokens/s (whole model)", "value": B / per_tok, "unit": "tokens/s", "n_gpus": 1,
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"SequenceModel(vocab 50304, d_model 768, 12 layers, d_state 16) bf16, batch {B}, prompt {LP}, "
                               f"{NEW} new tokens, greedy"},
        "ms_generate": 1e3 * t_dec, "ms_prefill": 1e3 * t_pre, "us_per_token_step": 1e6 * per_tok,
        "reference_generate_ms": 1e3 * t_ref, "speedup_vs_reference_generate": t_ref / t_dec,
        "first_generated_token_equal_to_reference": first, "all_generated_tokens_equal_to_reference": same,
        "note": "a random-weight model's logits are nearly flat, so in bf16 the greedy choice flips where two logits are within "
                "one rounding step and the sequences part from there; the float32 test demands equal tokens",
    }), flush=True)


def run_inference(args):
    """Secondary line: the inference route of one layer at the decode configuration (batch 32,
    d_model 1024 -> M = 2048, S = 16, bf16): a prompt of 8192 tokens through LayerDecoder.prefill
    (projections and conv as library calls, the scan with sensor prologue and skip/gate epilogue
    inside), then 256 tokens decoded one by one from the state it leaves (CUDA graph of 64 tokens)."""
    import torch

    dec_mod = __import__("importlib").import_module("kalman-linear-attention_b200.decode")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, DM, S, K, LP, NTOK = (args.batch or 32), 1024, 16, 4, 8192, 64
    M = 2 * DM
    dt = torch.bfloat16
    g = torch.Generator(device="cpu").manual_seed(0)
    rn = lambda *sh, scale=1.0: (torch.randn(*sh, generator=g) * scale)
    weights = {
        "in_proj.weight": rn(2 * M, DM, scale=DM ** -0.5).to(dt), "sensor_proj.weight": rn(2 * M + 2 * S, M, scale=M ** -0.5).to(dt),
        "out_proj.weight": rn(DM, M, scale=M ** -0.5).to(dt), "conv.weight": rn(M, 1, K, scale=0.5), "conv.bias": torch.zeros(M),
        "delta": rn(M, S) - 4.0, "lambda_log": rn(M, S, scale=0.1), "process_noise": torch.full((M, S), 0.01),
        "lambda_skip": torch.tensor(-1.0),
    }
    config = dict(d_state=S, discretization="ou", zero_process_noise=False, clip_value=None, obs_var_min=1e-4,
                  obs_var_max=None, value_rank="full", qk_norm=True, use_conv=True, conv_kernel_size=K,
                  conv_activation="silu", use_gating=True, gating_activation="silu", use_lambda_skip=True,
                  return_variance=False, decode_from_prior=False)
    dec = dec_mod.LayerDecoder(weights, config).to(dev)
    prompt = torch.randn(B, LP, DM, device=dev, dtype=dt)
    xs = torch.randn(NTOK, B, DM, device=dev, dtype=dt)
    lib = __import__("importlib").import_module("kalman-linear-attention_b200._lib")

    def timed(fn, n):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    n_pre = max(1, min(args.steps, 10))
    state_box = {}

    def prefill():
        state_box["out"], state_box["state"] = dec.prefill(prompt)

    ms_pre = timed(prefill, n_pre)
    # the scan alone, on tensors of the same shapes and types
    v = torch.randn(B, LP, M, device=dev, dtype=dt)
    k = torch.nn.functional.normalize(torch.randn(B, LP, S, device=dev), dim=-1).to(dt)
    import kla_b200
    with torch.no_grad():
        ms_scan = timed(lambda: kla_b200.kla_scan_b200(
            v, v, k, k, dec.a_bar, dec.p_bar, out_dtype=dt, log_variance=(1e-4, None),
            epilogue=dict(z=v, lambda_skip=dec.skip, gate=v, gate_activation="silu")), n_pre)
    state = state_box["state"]
    dec.step(xs[0], state)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for t in range(NTOK):
                out = dec.step(xs[t], state)
    torch.cuda.current_stream().wait_stream(s)
    us_tok = timed(gr.replay, max(args.steps, 4)) * 1e3 / NTOK
    total_ms = ms_pre + 256 * us_tok * 1e-3
    esz = 2
    scan_bytes = B * LP * esz * (6 * M + 2 * S)  # v, log-variance, z, gate in; y, y_var out; k, q
    peak, src = peaks()
    print(json.dumps({
        "metric": "KLA layer inference tokens/s (prefill 8192 + 256 decoded, one layer)",
        "value": B * (LP + 256) / (total_ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": n_pre,
        "warmup": max(args.warmup, 3), "ms_per_step": total_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 activations and projections, f32 filter state", "data": "synthetic",
        "config": {"workload": f"one KLA layer, B={B} d_model={DM} M={M} S={S}: prefill of {LP} tokens, then 256 tokens "
                               "decoded one at a time (64-token CUDA graph)",
                   "prefill_ms": ms_pre, "prefill_tokens_per_s": B * LP / (ms_pre * 1e-3),
                   "scan_only_ms": ms_scan, "decode_us_per_token": us_tok, "finite": bool(torch.isfinite(out.float()).all())},
        "roofline": {"bound": "hbm", "kernel": "kla_fwd_kernel<bf16, bf16> with prologue and epilogue (prefill)",
                     "achieved": scan_bytes / (ms_scan * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": scan_bytes / (ms_scan * 1e-3) / 1e9 / peak, "traffic": None, "peak_source": src,
                     "algorithmic_bytes": scan_bytes, "ms": ms_scan},
    }), flush=True)


def run_reference_gpu(args):
    """Secondary workload: the reference's OWN GPU backends on this GPU, on the headline raw-op shape, forward +
    backward through ``kla.ops.kla_scan(..., backend=...)`` (unmodified copy under baseline/_ref): ``triton`` (its
    tiled Moebius and affine scans composed with torch operations, src/kla/ops/triton_backend.py:125-171) and ``cuda``
    (its fused CUDA kernel, JIT-compiled on first use, src/kla/ops/cuda_backend.py:158-236; its gradients through the
    precision scan are approximate by design). One JSON line per backend, ``impl: reference-<backend>``; a backend
    that cannot run here prints ``unavailable`` with the reason. Each runs in a child process with a time limit, so a
    build or a kernel that goes wrong there ends that child only."""
    if reference_dir() is None:
        print(json.dumps({"impl": "reference-gpu", "unavailable": "the reference is not installed under baseline/_ref"}))
        return
    for backend in ("triton", "cuda"):
        cmd = [sys.executable, os.path.abspath(__file__), "--workload", "_reference_gpu_child", "--backend", backend,
               "--steps", str(min(args.steps, 10)), "--warmup", str(args.warmup)]
        try:
            res = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
            lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
            if res.returncode == 0 and lines:
                print(lines[-1], flush=True)
            else:
                tail = (res.stderr or res.stdout).strip().splitlines()[-1:] or ["no output"]
                print(json.dumps({"impl": f"reference-{backend}", "unavailable": f"exit {res.returncode}: {tail[0][:300]}"}), flush=True)
        except subprocess.TimeoutExpired:
            print(json.dumps({"impl": f"reference-{backend}", "unavailable": "no result within 900 s"}), flush=True)


def run_reference_gpu_child(args):
    import torch

    sys.path.insert(0, reference_dir())
    from kla.ops import kla_scan

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B = WORK["B"]
    while True:
        try:
            host = make_inputs(seed=0, **{**WORK, "B": B})
            d = {n: t.to(dev) for n, t in host.items()}
            ins = [d[n].requires_grad_(True) for n in ("v", "lambda_v", "k", "q", "a", "p")]

            def step():
                y, y_var, _ = kla_scan(*ins, backend=args.backend)
                return torch.autograd.grad([y, y_var], ins, [d["dy"], d["dyvar"]])

            step()
            break
        except torch.OutOfMemoryError:
            del d, ins
            torch.cuda.empty_cache()
            if B == 1:
                raise
            B //= 2
    for _ in range(max(args.warmup, 1)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({
        "impl": f"reference-{args.backend}", "metric": METRIC, "value": B * WORK["L"] / (ms * 1e-3), "unit": UNIT,
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"raw KLA scan fwd+bwd through the reference's kla_scan(backend='{args.backend}'), B={B} "
                               f"T=4096 M=1024 S=16, fp32" + ("" if B == WORK["B"] else " (largest batch that fits its temporaries)"),
                   **{**WORK, "B": B}},
        "peak_memory_gb": torch.cuda.max_memory_allocated() / 1e9,
    }), flush=True)


def run_train_step(args):
    """Secondary workload: the reference's ``SequenceModel(ModelConfig(vocab 50304, d_model 768, 12 layers),
    KLAConfig(d_state=16))`` training step (forward + backward, bf16 autocast, random weights, uniform random token
    ids, batch 16 x T=2048 split over the ranks, DistributedDataParallel over NCCL) with the scan on the ``b200``
    backend; the layers, the model and DDP are the reference's and torch's own. ``--backend triton`` runs the same step
    on the reference's Triton backend for comparison (at the largest per-GPU batch its temporaries fit)."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    if reference_dir() is None:
        print(json.dumps({"workload": "train_step", "unavailable": "the reference is not installed under baseline/_ref"}))
        return
    sys.path.insert(0, reference_dir())
    import kla_b200
    from kla import KLAConfig, ModelConfig, SequenceModel

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    backend = args.backend or "b200"
    if backend == "b200":
        kla_b200.register(fuse_layer=args.fused_layer)
    GB, T, V = 16, 2048, 50304
    Bl = max(1, GB // world)
    if args.batch:
        Bl = args.batch
    torch.manual_seed(0)
    model = SequenceModel(ModelConfig(vocab_size=V, d_model=768, n_layers=12), KLAConfig(d_state=16, backend=backend)).to(dev)
    net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local]) if world > 1 else model
    ids = torch.randint(0, V, (Bl, T + 1), device=dev, generator=torch.Generator(device=dev).manual_seed(1 + rank))
    lib = __import__("importlib").import_module("kalman-linear-attention_b200._lib")

    def step():
        net.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = net(ids[:, :-1])
        loss = F.cross_entropy(logits.reshape(-1, V).float(), ids[:, 1:].reshape(-1))
        loss.backward()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    loss = step()
    n0 = lib.load().kla_b200_launch_count()
    ms = _event_time(step, args.steps, max(args.warmup, 2), barrier)
    launches = (lib.load().kla_b200_launch_count() - n0) / (args.steps + max(args.warmup, 2))
    tm = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    ms = tm.item()
    if rank == 0:
        print(json.dumps({
            "workload": "train_step", "metric": "SequenceModel training step tokens/s", "value": Bl * world * T / (ms * 1e-3),
            "unit": UNIT, "n_gpus": world, "steps": args.steps, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong" if not args.batch else "weak", "dtype": "bf16 autocast, float32 scan", "data": "synthetic",
            "config": {"workload": f"SequenceModel(vocab 50304, d_model 768, 12 layers, d_state 16) fwd+bwd, batch {Bl} per GPU x "
                                   f"T={T}, scan backend '{backend}'" + (", KLALayer.forward through the fused route "
                                   "(sensor prologue and skip/gate epilogue inside the scan kernels)" if args.fused_layer else "")
                                   + f", DDP over {world} rank(s)",
                       "global_batch": Bl * world, "seq_len": T, "parallelism": f"dp{world}"},
            "loss": float(loss), "scan_kernel_launches_per_step": launches,
            "peak_memory_gb": torch.cuda.max_memory_allocated() / 1e9,
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--profile-batch", type=int, default=0,
                    help="profiling aid: run exactly one forward and one backward launch at this batch size "
                         "(same T, M, S) and exit without timing; for captures under ncu")
    ap.add_argument("--profile-chunks", type=int, default=0,
                    help="with --profile-batch: run that one forward + backward through the time-parallel path "
                         "with this many time chunks (aggregate and fold kernels included)")
    ap.add_argument("--batch", type=int, default=0,
                    help="raw workload only: batch size per GPU instead of 8, for the occupancy sweep "
                         "(B=4 leaves one CTA per SM, B=16 fills every SM); the headline stays B=8")
    ap.add_argument("--fused-layer", action="store_true",
                    help="train_step: route KLALayer.forward through the package's fused layer forward")
    ap.add_argument("--backend", default="", help="reference_gpu child / train_step: the scan backend to run")
    ap.add_argument("--workload", default="raw", choices=["raw", "seqshard", "decode", "rawpair", "decode_layer", "prologue", "epilogue", "inference", "conv",
                                                          "reference_gpu", "_reference_gpu_child", "train_step", "generate"],
                    help="raw = the headline raw-op workload (default); seqshard = the long-sequence, "
                         "time-sharded workload (secondary line)")
    args = ap.parse_args()
    if args.workload == "reference_gpu":
        return run_reference_gpu(args)
    if args.workload == "_reference_gpu_child":
        return run_reference_gpu_child(args)
    if args.workload == "train_step":
        return run_train_step(args)
    if args.workload == "generate":
        return run_generate(args)
    if args.batch > 0:
        WORK["B"] = args.batch
    if args.workload == "seqshard" and args.impl != "reference":
        return run_seqshard(args)
    if args.workload == "decode" and args.impl != "reference":
        return run_decode(args)
    if args.workload == "rawpair" and args.impl != "reference":
        return run_rawpair(args)
    if args.workload == "decode_layer" and args.impl != "reference":
        return run_decode_layer(args)
    if args.workload == "prologue" and args.impl != "reference":
        return run_prologue(args)
    if args.workload == "epilogue" and args.impl != "reference":
        return run_epilogue(args)
    if args.workload == "inference" and args.impl != "reference":
        return run_inference(args)
    if args.workload == "conv" and args.impl != "reference":
        return run_conv(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
