"""CPU oracle for the two fused operators next to the PKDA recurrence.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file;
only the tests and the benchmark's CPU-baseline leg do, as the checker.

Independent restatements (not copies) of the reference's portable definitions:

* ``qkv_conv_oracle`` -- the short convolution, SiLU and per-head L2
  normalisation of ``delta_feedback_experiment/pkda.py:197-220`` (``_causal_conv``),
  ``:41-44`` (``_l2norm``) and ``:290-316`` (the portable branch of ``_project``),
  in the fused operator's packing (``fla_ops.py:137-170``): one input of
  concatenated Q|K|V channels, one ``[channels, taps]`` filter, three outputs.
* ``norm_gate_oracle`` -- the RMS-normed sigmoid gate of ``pkda.py:543-547``.

Parity is pinned: ``tests/golden/layer_*.npz`` hold vectors produced by running
the reference's own layer code (generator committed beside them) and
``tests/test_layer_oracle.py`` checks this file against them, values and
gradients.  Arithmetic runs in ``dtype``; gradients come from torch autograd.
"""

from __future__ import annotations

import torch


def qkv_conv_oracle(x: torch.Tensor, weight: torch.Tensor, head_dim: int, norm_channels: int,
                    eps: float, dtype: torch.dtype = torch.float32):
    """x [B,T,3W], weight [3W,taps] -> q,k,v [B,T,W].  Tap j multiplies
    x[t - (taps-1) + j]; tokens before the row start are zero."""
    x = x.to(dtype)
    weight = weight.to(dtype)
    B, T, C3 = x.shape
    taps = weight.shape[1]
    padded = torch.cat((x.new_zeros(B, taps - 1, C3), x), dim=1)
    y = x.new_zeros(B, T, C3)
    for j in range(taps):
        y = y + padded[:, j:j + T, :] * weight[:, j]
    s = y * torch.sigmoid(y)
    heads = s[..., :norm_channels].reshape(B, T, norm_channels // head_dim, head_dim)
    normed = heads * torch.rsqrt(heads.square().sum(-1, keepdim=True) + eps)
    out = torch.cat((normed.reshape(B, T, norm_channels), s[..., norm_channels:]), dim=-1)
    W = C3 // 3
    return out[..., :W], out[..., W:2 * W], out[..., 2 * W:]


def norm_gate_oracle(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float,
                     dtype: torch.dtype = torch.float32):
    """x, gate [..., D], weight [D] -> (y, rstd[rows])."""
    x = x.to(dtype)
    gate = gate.to(dtype)
    weight = weight.to(dtype)
    rstd = torch.rsqrt(x.square().mean(-1, keepdim=True) + eps)
    y = x * rstd * weight * torch.sigmoid(gate)
    return y, rstd.reshape(-1)


def decode_step_oracle(qkv, conv_state, conv_weight, g, g_atk, beta_atk, beta, A_log, dt_bias,
                       log_atk_scale, state, a_state, gate, norm_weight, head_dim: int,
                       squash_x: float = 1.5, squash_eps: float = 1e-6, qk_eps: float = 1e-6,
                       norm_eps: float = 1e-6, dtype: torch.dtype = torch.float32):
    """One cached decoding step, composed from the three oracles the way the
    reference's layer composes its operators (``pkda.py:239-288, 473-474, 539-547``
    and the cache update of ``model.py:775-787``).

    qkv [B,3W]; conv_state: three [B,W,taps-1] histories (oldest first); g [B,H,D];
    g_atk, beta_atk, beta [B,H]; state [B,H,D,D]; a_state [B,H,D]; gate [B,H,D] or None.
    Returns ``(out [B,H,D], new_state, new_a_state, new_conv_state)``.
    """
    from oracle.pkda_oracle import pkda_recurrent_oracle

    B, C3 = qkv.shape
    W = C3 // 3
    H = W // head_dim
    prefix = torch.cat([s.to(dtype) for s in conv_state], dim=1).transpose(1, 2)   # [B, taps-1, 3W]
    rows = torch.cat((prefix, qkv.to(dtype)[:, None, :]), dim=1)
    q, k, v = qkv_conv_oracle(rows, conv_weight, head_dim, 2 * W, qk_eps, dtype)
    hist = prefix.shape[1]
    new_conv = tuple(part.transpose(1, 2).contiguous()
                     for part in rows[:, rows.shape[1] - hist:].split(W, dim=-1)) if hist else conv_state
    shape = (B, 1, H, head_dim)
    o, S, A = pkda_recurrent_oracle(
        q[:, -1:].reshape(shape), k[:, -1:].reshape(shape), v[:, -1:].reshape(shape),
        g.reshape(shape), g_atk.reshape(B, 1, H), beta_atk.reshape(B, 1, H), beta.reshape(B, 1, H),
        A_log, dt_bias, log_atk_scale, initial_state=state, initial_A_state=a_state,
        squash_x=squash_x, squash_eps=squash_eps, dtype=dtype)
    o = o.reshape(B, H, head_dim)
    if gate is None:
        return o, S, A, new_conv
    y, _ = norm_gate_oracle(o, gate, norm_weight, norm_eps, dtype)
    return y, S, A, new_conv


def controls_oracle(packed, A_log_precond, dt_bias_precond, hidden: int, dtype: torch.dtype = torch.float32):
    """Packed control row -> (decay_hidden, beta, precond_decay, precond_beta, gate_hidden),
    restating ``delta_feedback_experiment/pkda.py:325-346`` (split, sigmoid, softplus)."""
    import torch.nn.functional as F
    H = A_log_precond.shape[0]
    x = packed.to(dtype)
    h0, lb, ld, lp, h1 = x.split((hidden, H, H, H, hidden), dim=-1)
    g_atk = -A_log_precond.to(dtype).exp() * F.softplus(ld + dt_bias_precond.to(dtype))
    return h0, torch.sigmoid(lb), g_atk, torch.sigmoid(lp), h1
