"""Token-by-token decode of one KLA layer on the B200 kernels.

The reference layer's decode route (``KLALayer.forward`` with a state and ``L == 1``,
src/kla/layers/kla_layer.py:295-345) is three projections with elementwise work between
them. ``LayerDecoder.step`` keeps the projections as library GEMMs and runs the rest as two
kernels: ``kla_b200_conv_step`` (``CausalConv1d`` advanced by one token,
src/kla/layers/common.py:87-96) and ``kla_b200_step_layer`` (sensor post-processing, the
filter step, skip path and gate; kla_layer.py:199-231, 277-293, 329-338).

A decoder is built from plain tensors and a plain config dict, so it does not need the
reference package at run time; ``LayerDecoder.from_layer`` reads both off a reference
``KLALayer``. All state is updated in place, which makes a step capturable in a CUDA graph.
"""

from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib
from .ops import kla_scan_b200

CONFIG_KEYS = (
    "d_state", "discretization", "zero_process_noise", "clip_value", "obs_var_min", "obs_var_max",
    "value_rank", "qk_norm", "use_conv", "conv_kernel_size", "conv_activation", "use_gating",
    "gating_activation", "use_lambda_skip", "return_variance", "decode_from_prior",
)


def discretize(weights: dict, config: dict):
    """Discrete (a_bar, p_bar), each [M, S]: the reference's ``KLALayer._compute_aq``
    (src/kla/layers/kla_layer.py:164-190) restated on plain tensors."""
    a = -torch.exp(weights["lambda_log"].float())
    p = weights["process_noise"].float()
    if config["zero_process_noise"]:
        p = p + 1e-12
    else:
        p = p.clamp_min(1e-7)
        if config["clip_value"] is not None:
            p = p.clamp_max(config["clip_value"])
    delta = F.softplus(weights["delta"].float()) + 1e-7
    a_bar = torch.exp(delta * a)
    if config["discretization"] == "ou":
        lam_pos = a.abs().clamp_min(1e-8)
        p_bar = (p / (2.0 * lam_pos)) * (-torch.expm1(-2.0 * lam_pos * delta))
    else:
        p_bar = p * delta
    return a_bar.contiguous(), p_bar.contiguous()


class LayerDecoder:
    def __init__(self, weights: dict, config: dict):
        missing = [k for k in CONFIG_KEYS if k not in config]
        if missing:
            raise ValueError(f"decode config lacks {missing}")
        self.w = weights
        self.cfg = dict(config)
        self.M, self.S = weights["delta"].shape
        if self.S > _lib.MAX_DSTATE:
            raise NotImplementedError(f"The b200 decode kernels support d_state <= {_lib.MAX_DSTATE}; use backend='torch'.")
        if config["use_conv"] and config["conv_kernel_size"] > _lib.MAX_CONV_TAPS:
            raise NotImplementedError(f"The b200 conv step supports up to {_lib.MAX_CONV_TAPS} taps; use backend='torch'.")
        self.a_bar, self.p_bar = discretize(weights, config)
        sensor_out = weights["sensor_proj.weight"].shape[0]
        self.w_value = 0 if config["value_rank"] == "conv" else (
            weights["value_expand.weight"].shape[1] if "value_expand.weight" in weights else self.M)
        self.w_var = sensor_out - self.w_value - 2 * self.S
        skip = weights.get("lambda_skip") if config["use_lambda_skip"] else None
        self.skip = None if skip is None else skip.detach().float().reshape(-1).contiguous()
        self.conv_w = None
        if config["use_conv"]:
            self.conv_w = weights["conv.weight"].detach().float().reshape(self.M, -1).contiguous()
            cb = weights.get("conv.bias")
            self.conv_b = None if cb is None else cb.detach().float().contiguous()

    @classmethod
    def from_layer(cls, layer) -> "LayerDecoder":
        """Read weights and config off a reference ``kla.KLALayer``."""
        weights = {k: v.detach() for k, v in layer.state_dict().items()}
        config = {k: getattr(layer.config, k) for k in CONFIG_KEYS}
        return cls(weights, config)

    def to(self, device) -> "LayerDecoder":
        out = LayerDecoder.__new__(LayerDecoder)
        out.__dict__.update(self.__dict__)
        out.w = {k: v.to(device) for k, v in self.w.items()}
        for name in ("a_bar", "p_bar", "skip", "conv_w", "conv_b"):
            t = getattr(self, name, None)
            setattr(out, name, None if t is None else t.to(device))
        return out

    def init_state(self, batch: int, device, dtype=torch.float32):
        """(conv window [B, M, K-1] or None, lam [B, M, S], eta [B, M, S]) -- kla_layer.py:152-160."""
        conv = None
        if self.cfg["use_conv"]:
            conv = torch.zeros(batch, self.M, self.cfg["conv_kernel_size"] - 1, device=device, dtype=dtype)
        lam = torch.ones(batch, self.M, self.S, device=device, dtype=torch.float32)
        return conv, lam, torch.zeros_like(lam)

    def _linear(self, x, name):
        return F.linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))

    def _sensors(self, z, sens):
        """Split the sensor projection as ``KLALayer._project_sensors`` does (kla_layer.py:199-216), raw."""
        cfg, M, S = self.cfg, self.M, self.S
        o = 0
        if cfg["value_rank"] == "conv":
            v = z
        else:
            v = sens[..., o:o + self.w_value]
            o += self.w_value
            if "value_expand.weight" in self.w:
                v = self._linear(v, "value_expand")
        ls = sens[..., o:o + self.w_var]
        o += self.w_var
        if "var_expand.weight" in self.w:
            ls = self._linear(ls, "var_expand")
        return v, ls, sens[..., o:o + S], sens[..., o + S:o + 2 * S]

    @torch.no_grad()
    def prefill(self, x: torch.Tensor, state=None):
        """A whole prompt: the layer's ``forward(x, state)`` for ``L > 1`` in inference
        (kla_layer.py:295-345). ``x``: [B, L, d_model]. The projections are library GEMMs; the causal
        convolution runs in ``kla_b200_conv_seq``; the scan runs with the sensor prologue and the skip/gate epilogue inside
        (``kla_scan_b200(log_variance=, epilogue=)``). Returns ``(out, state)`` -- or ``((out, out_var),
        state)`` -- with ``state`` ready for ``step``."""
        if not x.is_cuda:
            raise NotImplementedError("The b200 kernels need CUDA tensors; use the reference layer on this device.")
        cfg, M = self.cfg, self.M
        B, L, _ = x.shape
        if state is None:
            state = self.init_state(B, x.device, x.dtype)
        conv_state, lam, eta = state
        projected = self._linear(x, "in_proj")
        z, gate = (projected[..., :M], projected[..., M:]) if cfg["use_gating"] else (projected, None)
        if cfg["use_conv"]:
            # the causal convolution over the prompt, in place of cat + transpose + conv1d + activation + transpose
            zc = torch.empty(B, L, M, device=x.device, dtype=x.dtype)
            new_window = torch.empty_like(conv_state)
            dt = _lib.F32 if x.dtype == torch.float32 else _lib.BF16
            P = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
            ca = _lib.ConvSeqArgs(B=B, L=L, D=M, K=cfg["conv_kernel_size"], dtype=dt,
                                  activation=_lib.ACT[cfg["conv_activation"]],
                                  x=_lib.Tensor3(z.data_ptr(), z.stride(0), z.stride(1)), weight=P(self.conv_w),
                                  bias=P(self.conv_b), state=P(conv_state), state_out=P(new_window),
                                  z=_lib.Tensor3(zc.data_ptr(), zc.stride(0), zc.stride(1)))
            with torch.cuda.device(x.device):
                _lib.check(_lib.load().kla_b200_conv_seq(ctypes.byref(ca), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
            conv_state.copy_(new_window)
            z = zc
        v, ls, k, q = self._sensors(z, self._linear(z, "sensor_proj"))
        if cfg["qk_norm"]:  # [B, L, S]: small next to the [B, L, M] tensors, left to torch
            k = k / k.norm(dim=-1, keepdim=True).clamp_min(1e-12)
            q = q / q.norm(dim=-1, keepdim=True).clamp_min(1e-12)
        if cfg["clip_value"] is not None:
            k, q = k.clamp(-cfg["clip_value"], cfg["clip_value"]), q.clamp(-cfg["clip_value"], cfg["clip_value"])
        epi = {}
        if self.skip is not None:
            epi.update(z=z, lambda_skip=self.skip)
        if gate is not None:
            epi.update(gate=gate, gate_activation=cfg["gating_activation"])
        y, y_var, st = kla_scan_b200(
            v, ls, k, q, self.a_bar, self.p_bar, initial_state=(lam, eta), decode_from_prior=cfg["decode_from_prior"],
            out_dtype=x.dtype if x.dtype == torch.bfloat16 else None,
            log_variance=(cfg["obs_var_min"], cfg["obs_var_max"]), epilogue=epi or None)
        lam.copy_(st.lam)
        eta.copy_(st.eta)
        y, y_var = y.to(x.dtype), y_var.to(x.dtype)
        out = self._linear(y, "out_proj")
        if cfg["return_variance"]:
            return (out, F.linear(y_var, self.w["out_proj.weight"].pow(2))), state
        return out, state

    def step(self, x: torch.Tensor, state):
        """One token. ``x``: [B, d_model]; ``state``: the tuple of ``init_state``, updated in place.
        Returns ``out`` [B, d_model], or ``(out, out_var)`` when the config returns variances."""
        if not x.is_cuda:
            raise NotImplementedError("The b200 decode kernels need CUDA tensors; use the reference layer on this device.")
        if x.dtype not in (torch.float32, torch.bfloat16):
            raise NotImplementedError(f"The b200 decode kernels take float32 or bfloat16 activations, not {x.dtype}.")
        cfg, M, S = self.cfg, self.M, self.S
        conv_state, lam, eta = state
        B = x.shape[0]
        dt = _lib.F32 if x.dtype == torch.float32 else _lib.BF16
        lib = _lib.load()
        P = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
        with torch.cuda.device(x.device):
            stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            projected = self._linear(x, "in_proj")
            z, gate = (projected[:, :M], projected[:, M:]) if cfg["use_gating"] else (projected, None)
            if cfg["use_conv"]:
                zc = torch.empty(B, M, device=x.device, dtype=x.dtype)
                ca = _lib.ConvStepArgs(B=B, D=M, K=cfg["conv_kernel_size"], dtype=dt,
                                       activation=_lib.ACT[cfg["conv_activation"]], x=P(z), x_stride_b=z.stride(0),
                                       weight=P(self.conv_w), bias=P(self.conv_b), state=P(conv_state), z=P(zc))
                _lib.check(lib.kla_b200_conv_step(ctypes.byref(ca), stream))
                z = zc
            sens = self._linear(z, "sensor_proj")
            v, ls, k, q = self._sensors(z, sens)
            y = torch.empty(B, M, device=x.device, dtype=x.dtype)
            y_var = torch.empty_like(y)
            sa = _lib.StepLayerArgs(
                B=B, M=M, S=S, in_dtype=dt, out_dtype=dt, decode_from_prior=int(cfg["decode_from_prior"]),
                qk_norm=int(cfg["qk_norm"]), gate_activation=_lib.ACT[cfg["gating_activation"] if gate is not None else None],
                lambda_skip_len=0 if self.skip is None else self.skip.numel(),
                obs_var_min=cfg["obs_var_min"], obs_var_max=cfg["obs_var_max"] or 0.0, clip_value=cfg["clip_value"] or 0.0,
                v=P(v), log_sigma_v=P(ls), v_stride_b=v.stride(0), log_sigma_v_stride_b=ls.stride(0),
                k=P(k), q=P(q), k_stride_b=k.stride(0), q_stride_b=q.stride(0),
                z=P(z), gate=P(gate), z_stride_b=z.stride(0), gate_stride_b=0 if gate is None else gate.stride(0),
                lambda_skip=P(self.skip), a=P(self.a_bar), p=P(self.p_bar), lam=P(lam), eta=P(eta),
                y=P(y), y_var=P(y_var), lam_out=P(lam), eta_out=P(eta))
            _lib.check(lib.kla_b200_step_layer(ctypes.byref(sa), stream))
            out = self._linear(y, "out_proj")
            if cfg["return_variance"]:
                return out, F.linear(y_var, self.w["out_proj.weight"].pow(2))
            return out


MODEL_KEYS = ("n_layers", "norm_eps", "mlp", "logit_softcap")


class ModelDecoder:
    """Prompt prefill and token-by-token decode of a whole stack of KLA blocks on the B200 kernels: the
    reference's ``SequenceModel.forward`` with a state and ``SequenceModel.generate``
    (src/kla/models/sequence_model.py:150-173, 200-220).

    A block is ``x += mixer(norm(x))`` then ``x += mlp(norm(x))`` (sequence_model.py:47-98). The mixers run
    through :class:`LayerDecoder` (two fused kernels per layer and token, the scan kernels for the prompt); the
    norms, the channel MLPs, the embedding and the LM head are a handful of library calls each and stay torch
    operations. One decoded token is a fixed sequence of launches over state that is updated in place, so
    ``generate`` captures it once in a CUDA graph and replays it: a token then costs no host work but one replay,
    where the reference's loop issues several hundred small launches per token from Python.

    Built from plain tensors (``SequenceModel.state_dict()``) and plain config dicts; ``from_model`` reads them
    off a reference model. The reference package is not needed at run time."""

    def __init__(self, weights: dict, layer_configs, model_config: dict):
        missing = [k for k in MODEL_KEYS if k not in model_config]
        if missing:
            raise ValueError(f"model config lacks {missing}")
        self.cfg = dict(model_config)
        self.w = weights
        n = self.cfg["n_layers"]
        if len(layer_configs) != n:
            raise ValueError(f"got {len(layer_configs)} layer configs for {n} layers")
        self.layers = []
        for i in range(n):
            pre = f"blocks.{i}.mixer."
            lw = {k[len(pre):]: v for k, v in weights.items() if k.startswith(pre)}
            self.layers.append(LayerDecoder(lw, layer_configs[i]))
        self._graph = None

    @classmethod
    def from_model(cls, model) -> "ModelDecoder":
        """Read weights and configs off a reference ``kla.SequenceModel`` whose mixers are all KLA layers."""
        weights = {k: v.detach() for k, v in model.state_dict().items()}
        layer_configs = [{k: getattr(blk.mixer.config, k) for k in CONFIG_KEYS} for blk in model.blocks]
        model_config = {k: getattr(model.config, k) for k in MODEL_KEYS}
        dec = cls(weights, layer_configs, model_config)
        dev = model.embedding.weight.device
        return dec.to(dev) if dev.type == "cuda" else dec

    def to(self, device) -> "ModelDecoder":
        out = ModelDecoder.__new__(ModelDecoder)
        out.__dict__.update(self.__dict__)
        out.w = {k: v.to(device) for k, v in self.w.items()}
        out.layers = [layer.to(device) for layer in self.layers]
        out._graph = None
        return out

    def init_state(self, batch: int, device, dtype=torch.float32):
        return [layer.init_state(batch, device, dtype) for layer in self.layers]

    def _norm(self, x, name):  # RMSNorm, src/kla/layers/common.py:45-55
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + self.cfg["norm_eps"])
        return (xf * self.w[name + ".weight"].float()).to(x.dtype)

    def _mlp(self, i, x):  # src/kla/layers/common.py:99-122
        pre = f"blocks.{i}.mlp."
        if self.cfg["mlp"] == "swiglu":
            gate, up = F.linear(x, self.w[pre + "w12.weight"], self.w.get(pre + "w12.bias")).chunk(2, dim=-1)
            return F.linear(F.silu(gate) * up, self.w[pre + "w3.weight"], self.w.get(pre + "w3.bias"))
        return F.linear(F.gelu(F.linear(x, self.w[pre + "w1.weight"], self.w.get(pre + "w1.bias"))),
                        self.w[pre + "w2.weight"], self.w.get(pre + "w2.bias"))

    def _head(self, x):
        logits = F.linear(self._norm(x, "norm_f"), self.w["lm_head.weight"])
        cap = self.cfg["logit_softcap"]
        return logits if cap is None else cap * torch.tanh(logits / cap)

    def _blocks(self, x, state, prompt: bool):
        for i, layer in enumerate(self.layers):
            h = self._norm(x, f"blocks.{i}.mixer_norm")
            mixed = layer.prefill(h, state[i])[0] if prompt else layer.step(h, state[i])
            if isinstance(mixed, tuple):  # a layer that returns variances: the mean path (sequence_model.py:85-86)
                mixed = mixed[0]
            x = x + mixed
            if self.cfg["mlp"] != "none":
                x = x + self._mlp(i, self._norm(x, f"blocks.{i}.mlp_norm"))
        return x

    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, state=None):
        """A prompt: ``input_ids`` [B, L] -> (logits [B, L, vocab], state ready for ``step``)."""
        x = F.embedding(input_ids, self.w["embedding.weight"])
        if state is None:
            state = self.init_state(x.shape[0], x.device, x.dtype)
        return self._head(self._blocks(x, state, prompt=True)), state

    @torch.no_grad()
    def step(self, token: torch.Tensor, state):
        """One token per sequence: ``token`` [B] -> logits [B, vocab]; ``state`` is updated in place."""
        x = F.embedding(token, self.w["embedding.weight"])
        return self._head(self._blocks(x, state, prompt=False))

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int, temperature: float = 0.0, top_k=None,
                 use_graph: bool = True) -> torch.Tensor:
        """``SequenceModel.generate`` (sequence_model.py:200-220): prefill, then one token at a time from the
        recurrent state. ``temperature <= 0`` is greedy. With ``use_graph`` the per-token work of all layers is
        one CUDA graph replay; sampling happens between replays, on the device."""
        logits, state = self.prefill(input_ids)
        token = self._sample(logits[:, -1], temperature, top_k)
        out = [input_ids, token]
        if max_new_tokens <= 1:
            return torch.cat(out, dim=1)
        tok_buf = token[:, 0].clone()
        graph = None
        if use_graph:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            snapshot = [[None if t is None else t.clone() for t in st] for st in state]
            with torch.cuda.stream(side):  # warm-up on a side stream, as graph capture requires
                for _ in range(2):
                    self.step(tok_buf, state)
            torch.cuda.current_stream().wait_stream(side)
            for st, snap in zip(state, snapshot):  # the warm-up advanced the state: put it back
                for t, s_ in zip(st, snap):
                    if t is not None:
                        t.copy_(s_)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                logits_buf = self.step(tok_buf, state)
        for _ in range(max_new_tokens - 1):
            if graph is not None:
                graph.replay()
                logits = logits_buf
            else:
                logits = self.step(tok_buf, state)
            token = self._sample(logits, temperature, top_k)
            tok_buf.copy_(token[:, 0])
            out.append(token)
        return torch.cat(out, dim=1)

    @staticmethod
    def _sample(logits, temperature, top_k):  # sequence_model.py:222-234
        if temperature <= 0:
            return logits.argmax(dim=-1, keepdim=True)
        logits = logits / temperature
        if top_k is not None:
            kth = torch.topk(logits, top_k, dim=-1).values[..., -1, None]
            logits = logits.masked_fill(logits < kth, float("-inf"))
        return torch.multinomial(torch.softmax(logits.float(), dim=-1), num_samples=1)
