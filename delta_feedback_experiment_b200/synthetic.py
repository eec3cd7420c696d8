"""Seeded synthetic inputs for the PKDA operator.

Two families, both generated on the CPU with a ``torch.Generator`` so that the
same seed gives the same tensors everywhere (tests, smoke check, benchmark):

* ``"unit"`` -- the benchmark configurations' distribution: ``q, k`` are
  per-head L2-normalised Gaussians, ``v ~ N(0,1)``, ``beta = sigmoid(N(0,1))``,
  raw decay ``~ N(0,1)`` with ``A_log = 0`` and ``dt_bias = 0`` so the effective
  per-channel log-decay is ``-softplus(N(0,1))``; the preconditioner gets
  ``g_atk = -softplus(N(0,1))``, ``beta_atk = sigmoid(N(0,1))`` and the
  reference's initial centre ``-0.2``
  (``delta_feedback_experiment/pkda.py:163-165``).
* ``"production"`` -- the distribution the reference's own operator benchmark
  draws (``scripts/pkda_bench.py:162-187``): SiLU-shaped activations, small
  control logits, ``exp(A_log) ~ U(1,16)`` (strong per-channel decay, up to
  about 11 nats per token) and the layer's preconditioner initialisation
  (``delta_feedback_experiment/pkda.py:184-195``).
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

INPUT_NAMES = (
    "q", "k", "v", "g", "g_atk", "beta_atk", "beta", "A_log", "dt_bias",
    "log_atk_scale",
)


def make_inputs(
    B: int,
    T: int,
    H: int,
    D: int,
    *,
    seed: int = 0,
    dist: str = "unit",
    dtype: torch.dtype = torch.bfloat16,
    n_states: Optional[int] = None,
    with_state: bool = False,
) -> dict:
    """Returns a dict with the ten operator inputs, an upstream cotangent
    ``do`` and (if ``with_state``) ``initial_state ~ N(0, 0.02)`` ``[N,H,D,D]``
    fp32 and ``initial_A_state ~ U(0, 0.02)`` ``[N,H,D]`` fp32 (non-negative:
    the recurrence takes ``log(A + eps)``).  Activations are rounded to
    ``dtype``; ``g_atk`` and the three per-head parameter vectors stay fp32, as
    the layer hands them over (``delta_feedback_experiment/pkda.py:343-345``).
    """
    gen = torch.Generator().manual_seed(seed)
    shape = (B, T, H, D)
    sc = (B, T, H)

    def rn(size):
        return torch.randn(size, generator=gen, dtype=torch.float32)

    def ru(size, lo, hi):
        return torch.rand(size, generator=gen, dtype=torch.float32) * (hi - lo) + lo

    if dist == "unit":
        q = F.normalize(rn(shape), dim=-1)
        k = F.normalize(rn(shape), dim=-1)
        v = rn(shape)
        g = rn(shape)
        beta = torch.sigmoid(rn(sc))
        beta_atk = torch.sigmoid(rn(sc))
        g_atk = -F.softplus(rn(sc))
        A_log = torch.zeros(H)
        dt_bias = torch.zeros(H * D)
    elif dist == "production":
        q = F.normalize(F.silu(rn(shape)), dim=-1)
        k = F.normalize(F.silu(rn(shape)), dim=-1)
        v = F.silu(rn(shape))
        g = rn(shape) * 0.2
        beta = torch.sigmoid(rn(sc) * 0.2)
        beta_atk = torch.sigmoid(rn(sc) * 0.2)
        A_log = ru((H,), 1.0, 16.0).log()
        dt_bias = torch.zeros(H * D)
        rate = ru((H,), 1.0, 16.0)
        dt = ru((H,), math.log(1e-3), math.log(1e-1)).exp()
        bias = dt + torch.log(-torch.expm1(-dt))
        g_atk = -rate * F.softplus(rn(sc) * 0.2 + bias)
    else:
        raise ValueError(f"unknown distribution {dist!r}")
    log_atk_scale = torch.full((H,), -0.2)
    out = {
        "q": q.to(dtype), "k": k.to(dtype), "v": v.to(dtype), "g": g.to(dtype),
        "g_atk": g_atk, "beta_atk": beta_atk.to(dtype), "beta": beta.to(dtype),
        "A_log": A_log, "dt_bias": dt_bias, "log_atk_scale": log_atk_scale,
        "do": rn((B, T, H, D)).to(dtype),
    }
    if with_state:
        N = B if n_states is None else n_states
        out["initial_state"] = rn((N, H, D, D)) * 0.02
        out["initial_A_state"] = ru((N, H, D), 0.0, 0.02)
    return out


def operator_inputs(d: dict) -> tuple:
    """The ten tensors in operator order."""
    return tuple(d[n] for n in INPUT_NAMES)


def packed_lengths(total: int, lo: int, hi: int, seed: int = 0) -> list[int]:
    """Sequence lengths drawn uniformly in ``[lo, hi]`` until they cover
    ``total`` tokens, the last one truncated; returns cumulative offsets."""
    gen = torch.Generator().manual_seed(seed)
    offs = [0]
    while offs[-1] < total:
        n = int(torch.randint(lo, hi + 1, (1,), generator=gen))
        offs.append(min(total, offs[-1] + n))
    return offs
