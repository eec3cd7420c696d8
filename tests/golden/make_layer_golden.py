"""Generates the golden vectors ``layer_*.npz`` in this folder from the REFERENCE's
own code for the two operators next to the recurrence.

    python tests/golden/make_layer_golden.py /path/to/delta-feedback-experiment

* Convolution cases call ``PreconditionedKDA._project`` on CPU (its portable
  branch: ``_causal_conv`` + ``_l2norm``, ``delta_feedback_experiment/pkda.py:197-220,
  290-316``) on a layer whose three projections are exact channel selections, so
  that the layer input IS the concatenated Q|K|V projection the fused operator
  takes.  One case passes convolution histories (``conv_state``).
* Norm-gate cases call ``PreconditionedKDA.forward`` on CPU with its collaborators
  replaced (projection, controls and recurrence return seeded tensors, the gate
  up-projection returns a seeded leaf, the output projection is the identity), so
  that the layer output IS the result of the reference's inline RMS-norm / sigmoid
  gate code (``pkda.py:543-547``) on known inputs.

* Control cases call ``PreconditionedKDA._controls`` on CPU (see ``run_controls``).
* Decode cases call ``PreconditionedKDA.forward`` on CPU for consecutive cached
  single-token steps (see ``run_decode``).

Everything is float32; gradients come from torch autograd through the
reference's code.
"""

from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name -> (B, T, H, D, taps, with_history, seed)
CONV_CASES = {
    "layer_conv_small": (2, 37, 2, 16, 4, False, 21),
    "layer_conv_d128": (1, 70, 2, 128, 4, False, 22),
    "layer_conv_taps3_history": (2, 9, 3, 8, 3, True, 23),
    "layer_conv_d64_history": (1, 5, 2, 64, 4, True, 24),
}
# name -> (B, T, H, D, seed)
GATE_CASES = {
    "layer_gate_small": (2, 5, 3, 16, 31),
    "layer_gate_d128": (1, 9, 2, 128, 32),
    "layer_gate_d64": (3, 4, 1, 64, 33),
}


def run_conv(ref_root: str, case: tuple) -> dict:
    sys.path.insert(0, ref_root)
    from delta_feedback_experiment.pkda import QK_NORM_EPS, PreconditionedKDA

    B, T, H, D, taps, with_history, seed = case
    W = H * D
    gen = torch.Generator().manual_seed(seed)
    layer = PreconditionedKDA(3 * W, num_heads=H, head_dim=D, conv_size=taps)
    eye = torch.eye(W)
    zero = torch.zeros(W, W)
    with torch.no_grad():
        layer.q_proj.weight.copy_(torch.cat((eye, zero, zero), dim=1))
        layer.k_proj.weight.copy_(torch.cat((zero, eye, zero), dim=1))
        layer.v_proj.weight.copy_(torch.cat((zero, zero, eye), dim=1))
        for conv in (layer.q_conv, layer.k_conv, layer.v_conv):
            conv.weight.copy_(torch.randn(conv.weight.shape, generator=gen) * 0.5)
    x = torch.randn(B, T, 3 * W, generator=gen).requires_grad_(True)
    state = None
    if with_history:
        state = tuple(torch.randn(B, W, taps - 1, generator=gen).requires_grad_(True) for _ in range(3))
    q, k, v, _ = layer._project(x, state, False)
    dq, dk, dv = (torch.randn(B, T, H, D, generator=gen) for _ in range(3))
    loss = (q * dq).sum() + (k * dk).sum() + (v * dv).sum()
    wrt = [x, layer.q_conv.weight, layer.k_conv.weight, layer.v_conv.weight] + list(state or ())
    grads = torch.autograd.grad(loss, wrt)
    weight = torch.cat([c.weight.squeeze(1) for c in (layer.q_conv, layer.k_conv, layer.v_conv)], dim=0)
    out = {
        "x": x.detach().numpy(), "weight": weight.detach().numpy(),
        "head_dim": np.int64(D), "norm_channels": np.int64(2 * W), "eps": np.float64(QK_NORM_EPS),
        "q": q.detach().reshape(B, T, W).numpy(), "k": k.detach().reshape(B, T, W).numpy(),
        "v": v.detach().reshape(B, T, W).numpy(),
        "dq": dq.reshape(B, T, W).numpy(), "dk": dk.reshape(B, T, W).numpy(), "dv": dv.reshape(B, T, W).numpy(),
        "dx": grads[0].numpy(),
        "dweight": torch.cat([g.squeeze(1) for g in grads[1:4]], dim=0).numpy(),
    }
    if with_history:
        # the fused operator's caller prepends the histories as rows (pkda.py:245-251)
        out["prefix"] = torch.cat([s.detach() for s in state], dim=1).transpose(1, 2).contiguous().numpy()
        out["dprefix"] = torch.cat(list(grads[4:]), dim=1).transpose(1, 2).contiguous().numpy()
    return out


def run_gate(ref_root: str, case: tuple) -> dict:
    sys.path.insert(0, ref_root)
    import delta_feedback_experiment.pkda as ref_pkda
    from delta_feedback_experiment.pkda import PreconditionedKDA

    B, T, H, D, seed = case
    W = H * D
    gen = torch.Generator().manual_seed(seed)
    layer = PreconditionedKDA(W, num_heads=H, head_dim=D)
    with torch.no_grad():
        layer.o_proj.weight.copy_(torch.eye(W))
        layer.output_norm.copy_(1.0 + 0.3 * torch.randn(D, generator=gen))
    output = (torch.randn(B, T, H, D, generator=gen) * 1.7).requires_grad_(True)
    gate_logits = (torch.randn(B, T, W, generator=gen) * 2.0).requires_grad_(True)
    dummy = torch.zeros(B, T, H, D)
    scalar = torch.zeros(B, T, H)
    hidden = torch.zeros(B, T, D)
    layer._project = lambda x, conv_state, output_final_state: (dummy, dummy, dummy, None)
    layer._controls = lambda x: (dummy, scalar, scalar, scalar, hidden)
    layer._portable_recurrence = lambda *a: (output, None, None)

    real_F = ref_pkda.F
    shim = types.SimpleNamespace(**{n: getattr(real_F, n) for n in dir(real_F) if not n.startswith("__")})

    def linear(inp, weight, bias=None):
        if inp is hidden:          # the output gate's up-projection (pkda.py:526-534)
            return gate_logits
        return real_F.linear(inp, weight, bias)

    shim.linear = linear
    ref_pkda.F = shim
    try:
        mixed = layer(torch.zeros(B, T, W))[0]
    finally:
        ref_pkda.F = real_F
    dy = torch.randn(B, T, W, generator=gen)
    grads = torch.autograd.grad((mixed * dy).sum(), [output, gate_logits, layer.output_norm])
    return {
        "x": output.detach().numpy(), "gate": gate_logits.detach().reshape(B, T, H, D).numpy(),
        "weight": layer.output_norm.detach().numpy(), "eps": np.float64(layer.norm_eps),
        "y": mixed.detach().reshape(B, T, H, D).numpy(), "dy": dy.reshape(B, T, H, D).numpy(),
        "dx": grads[0].numpy(), "dgate": grads[1].reshape(B, T, H, D).numpy(), "dweight": grads[2].numpy(),
    }


# name -> (B, H, D, taps, steps, seed)
DECODE_CASES = {
    "layer_decode_small": (2, 3, 16, 4, 3, 41),
    "layer_decode_d128": (2, 2, 128, 4, 2, 42),
    "layer_decode_taps2_d64": (3, 1, 64, 2, 2, 43),
}


def run_decode(ref_root: str, case: tuple) -> dict:
    """Cached single-token steps through the reference's ``PreconditionedKDA.forward`` on CPU
    (``state`` / ``a_state`` / ``conv_state`` given, ``output_final_state=True``): the real
    ``_project`` (history-prefixed convolution, SiLU, L2 norm), the real recurrence and the real
    norm-gate code run; the control projections and the gate up-projection return seeded tensors,
    Q|K|V projections are channel selections and the output projection is the identity."""
    sys.path.insert(0, ref_root)
    import delta_feedback_experiment.pkda as ref_pkda
    from delta_feedback_experiment.pkda import QK_NORM_EPS, PreconditionedKDA

    B, H, D, taps, steps, seed = case
    W = H * D
    gen = torch.Generator().manual_seed(seed)
    layer = PreconditionedKDA(3 * W, num_heads=H, head_dim=D, conv_size=taps)
    eye, zero = torch.eye(W), torch.zeros(W, W)
    with torch.no_grad():
        layer.q_proj.weight.copy_(torch.cat((eye, zero, zero), dim=1))
        layer.k_proj.weight.copy_(torch.cat((zero, eye, zero), dim=1))
        layer.v_proj.weight.copy_(torch.cat((zero, zero, eye), dim=1))
        for conv in (layer.q_conv, layer.k_conv, layer.v_conv):
            conv.weight.copy_(torch.randn(conv.weight.shape, generator=gen) * 0.5)
        layer.o_proj.weight.copy_(torch.cat((eye, zero, zero), dim=0))   # output = (mixed, 0, 0)
        layer.output_norm.copy_(1.0 + 0.3 * torch.randn(D, generator=gen))
        layer.A_log.copy_(torch.log(torch.empty(H).uniform_(1.0, 4.0, generator=gen)))
        layer.dt_bias.copy_(0.1 * torch.randn(W, generator=gen))
        layer.log_precond_center.copy_(-0.2 + 0.05 * torch.randn(H, generator=gen))
    state = torch.randn(B, H, D, D, generator=gen) * 0.1
    a_state = torch.rand(B, H, D, generator=gen) * 0.05
    conv_state = tuple(torch.randn(B, W, taps - 1, generator=gen) for _ in range(3))
    out = {
        "conv_weight": torch.cat([c.weight.detach().squeeze(1) for c in (layer.q_conv, layer.k_conv, layer.v_conv)], 0).numpy(),
        "A_log": layer.A_log.detach().numpy(), "dt_bias": layer.dt_bias.detach().numpy(),
        "log_atk_scale": layer.log_precond_center.detach().numpy(), "norm_weight": layer.output_norm.detach().numpy(),
        "head_dim": np.int64(D), "qk_eps": np.float64(QK_NORM_EPS), "norm_eps": np.float64(layer.norm_eps),
        "squash_x": np.float64(layer.squash_x), "squash_eps": np.float64(layer.squash_eps),
        "state0": state.numpy().copy(), "a_state0": a_state.numpy().copy(),
        "steps": np.int64(steps),
    }
    for i, s in enumerate(conv_state):
        out[f"conv0_{i}"] = s.numpy().copy()
    real_F = ref_pkda.F
    for t in range(steps):
        x = torch.randn(B, 1, 3 * W, generator=gen)
        raw = torch.randn(B, 1, H, D, generator=gen)
        beta = torch.sigmoid(torch.randn(B, 1, H, generator=gen))
        g_atk = -torch.nn.functional.softplus(torch.randn(B, 1, H, generator=gen))
        beta_atk = torch.sigmoid(torch.randn(B, 1, H, generator=gen))
        gate_logits = torch.randn(B, 1, W, generator=gen) * 2.0
        hidden = torch.zeros(B, 1, D)
        layer._controls = lambda _x, c=(raw, beta, g_atk, beta_atk, hidden): c
        shim = types.SimpleNamespace(**{n: getattr(real_F, n) for n in dir(real_F) if not n.startswith("__")})
        shim.linear = lambda inp, weight, bias=None, gl=gate_logits, hd=hidden: (
            gl if inp is hd else real_F.linear(inp, weight, bias))
        ref_pkda.F = shim
        try:
            with torch.no_grad():
                mixed, state, a_state, conv_state = layer(x, state=state, a_state=a_state, conv_state=conv_state,
                                                          output_final_state=True)
        finally:
            ref_pkda.F = real_F
        out[f"qkv_{t}"] = x[:, 0].numpy()
        out[f"g_{t}"] = raw[:, 0].numpy()
        out[f"beta_{t}"] = beta[:, 0].numpy()
        out[f"g_atk_{t}"] = g_atk[:, 0].numpy()
        out[f"beta_atk_{t}"] = beta_atk[:, 0].numpy()
        out[f"gate_{t}"] = gate_logits[:, 0].reshape(B, H, D).numpy()
        out[f"out_{t}"] = mixed[:, 0, :W].reshape(B, H, D).numpy()
        out[f"state_{t}"] = state.numpy().copy()
        out[f"a_state_{t}"] = a_state.numpy().copy()
        for i, s in enumerate(conv_state):
            out[f"conv_{t}_{i}"] = s.numpy().copy()
    return out


# name -> (B, T, H, D, seed)
CONTROL_CASES = {
    "layer_controls_small": (2, 7, 3, 16, 51),
    "layer_controls_d128": (1, 5, 4, 128, 52),
}


def run_controls(ref_root: str, case: tuple) -> dict:
    """``PreconditionedKDA._controls`` on CPU with an identity control projection (the layer
    input IS the packed row) and a decay up-projection made of identity blocks (its output is
    the decay hidden repeated per head), values and autograd gradients."""
    sys.path.insert(0, ref_root)
    from delta_feedback_experiment.pkda import PreconditionedKDA

    B, T, H, D, seed = case
    total = 2 * D + 3 * H
    gen = torch.Generator().manual_seed(seed)
    layer = PreconditionedKDA(total, num_heads=H, head_dim=D)
    with torch.no_grad():
        layer.control_proj.weight.copy_(torch.eye(total))
        layer.decay_up.weight.copy_(torch.eye(D).repeat(H, 1))
        layer.A_log_precond.copy_(torch.log(torch.empty(H).uniform_(1.0, 8.0, generator=gen)))
        layer.dt_bias_precond.copy_(0.3 * torch.randn(H, generator=gen))
    x = torch.randn(B, T, total, generator=gen).requires_grad_(True)
    raw, beta, pd, pb, gate_hidden = layer._controls(x)
    cot = [torch.randn(t.shape, generator=gen) for t in (raw, beta, pd, pb, gate_hidden)]
    loss = sum((t * c).sum() for t, c in zip((raw, beta, pd, pb, gate_hidden), cot))
    dx, dA, db = torch.autograd.grad(loss, [x, layer.A_log_precond, layer.dt_bias_precond])
    return {
        "packed": x.detach().numpy(), "A_log_precond": layer.A_log_precond.detach().numpy(),
        "dt_bias_precond": layer.dt_bias_precond.detach().numpy(), "hidden": np.int64(D),
        "decay_hidden": raw.detach()[..., 0, :].numpy(), "beta": beta.detach().numpy(),
        "g_atk": pd.detach().numpy(), "beta_atk": pb.detach().numpy(),
        "gate_hidden": gate_hidden.detach().numpy(),
        "d_decay_hidden": cot[0].sum(-2).numpy(), "d_beta": cot[1].numpy(), "d_g_atk": cot[2].numpy(),
        "d_beta_atk": cot[3].numpy(), "d_gate_hidden": cot[4].numpy(),
        "d_packed": dx.numpy(), "dA_log_precond": dA.numpy(), "ddt_bias_precond": db.numpy(),
    }


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    torch.set_num_threads(1)
    for name, case in CONV_CASES.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **run_conv(sys.argv[1], case))
        print("wrote", name)
    for name, case in GATE_CASES.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **run_gate(sys.argv[1], case))
        print("wrote", name)
    for name, case in CONTROL_CASES.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **run_controls(sys.argv[1], case))
        print("wrote", name)
    for name, case in DECODE_CASES.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **run_decode(sys.argv[1], case))
        print("wrote", name)


if __name__ == "__main__":
    main()
