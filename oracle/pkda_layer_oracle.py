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
