"""Generate tests/golden/decode_*.npz: the reference layer decoding token by token.

    PYTHONPATH=<reference>/src python tests/golden/make_golden_decode.py

Each case builds a reference ``kla.KLALayer`` on CPU in float32 (backend="torch"), prefills a
few tokens, then decodes three tokens one at a time through the layer's own decode route
(``layer(x_t, state=state)``, src/kla/layers/kla_layer.py:295-345). Stored: the layer's
state_dict, the config fields the decode path reads, the discretised (a_bar, p_bar) of
``_compute_aq``, the prefill input and output, the state after the prefill, the three inputs,
and after every decoded token the layer output(s) and the full state.
"""

import os

import numpy as np
import torch

import kla

HERE = os.path.dirname(os.path.abspath(__file__))
CONFIG_KEYS = (
    "d_state", "discretization", "zero_process_noise", "clip_value", "obs_var_min", "obs_var_max",
    "value_rank", "qk_norm", "use_conv", "conv_kernel_size", "conv_activation", "use_gating",
    "gating_activation", "use_lambda_skip", "return_variance", "decode_from_prior",
)


def case(name, d_model, batch, seed, **cfg):
    torch.manual_seed(seed)
    layer = kla.KLALayer(d_model, kla.KLAConfig(backend="torch", **cfg)).eval()
    with torch.no_grad():
        for p in layer.parameters():  # move every parameter off its initial value (zeros, constants)
            p.add_(0.05 * torch.randn_like(p))
        x0 = torch.randn(batch, 5, d_model)
        xs = torch.randn(3, batch, 1, d_model)
        pre, state = layer(x0, return_state=True)
        out = {"x": xs[:, :, 0].numpy(), "x0": x0.numpy()}
        if layer.config.return_variance:
            out["pre_out"], out["pre_outvar"] = pre[0].numpy(), pre[1].numpy()
        else:
            out["pre_out"] = pre.numpy()
        for k_, v_ in layer.state_dict().items():
            out["w:" + k_] = v_.numpy()
        for k_ in CONFIG_KEYS:
            val = getattr(layer.config, k_)
            out["c:" + k_] = np.array("" if val is None else val)
        a_bar, p_bar = layer._compute_aq()
        out["a_bar"], out["p_bar"] = a_bar.numpy(), p_bar.numpy()
        if state.conv is not None:
            out["conv0"] = state.conv.numpy()
        out["lam0"], out["eta0"] = state.ssm.lam.numpy(), state.ssm.eta.numpy()
        for t in range(3):
            res, state = layer(xs[t], state=state)
            if layer.config.return_variance:
                out[f"out{t}"], out[f"outvar{t}"] = res[0][:, 0].numpy(), res[1][:, 0].numpy()
            else:
                out[f"out{t}"] = res[:, 0].numpy()
            if state.conv is not None:
                out[f"conv{t + 1}"] = state.conv.numpy()
            out[f"lam{t + 1}"], out[f"eta{t + 1}"] = state.ssm.lam.numpy(), state.ssm.eta.numpy()
    np.savez_compressed(os.path.join(HERE, f"decode_{name}.npz"), **out)
    print(name, "d_inner", layer.d_inner, "keys", len(out))


if __name__ == "__main__":
    case("default", 32, 2, 0, d_state=8)
    case("variant", 24, 3, 1, d_state=6, conv_activation="relu", gating_activation="gelu",
         lambda_skip_mode="vector", clip_value=0.8, obs_var_max=2.0, decode_from_prior=True,
         return_variance=True, var_rank=4, bias=True, discretization="zoh")
    case("bare", 16, 2, 2, d_state=4, use_conv=False, use_gating=False, use_lambda_skip=False,
         qk_norm=False, value_rank="conv")
    case("lowrank", 16, 1, 3, d_state=16, value_rank=5, conv_kernel_size=3, conv_activation="gelu")
