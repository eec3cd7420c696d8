"""CPU oracle for the PKDA (preconditioned Kimi delta attention) recurrence.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file;
only the tests, the smoke check and the benchmark's CPU-baseline leg do, and
there only as the checker or the timed CPU baseline, never as the product.

This is an independent restatement (not a copy) of the per-token recurrence the
reference defines in ``delta_feedback_experiment/pkda.py:355-410``
(``PreconditionedKDA._portable_recurrence``) and documents in
``docs/architecture.md:145-164``.  Its parity is pinned: ``tests/golden/`` holds
vectors produced by importing the reference's own function (generator script
committed beside them) and ``tests/test_oracle.py`` checks this file against
every one of them, values and gradients.

For one head and one row, with per-head parameters ``a = A_log``,
``b = dt_bias`` (a K-vector), ``c = log_atk_scale`` and constants ``x`` and
``eps``::

    g_t   = -exp(a) * softplus(raw_t + b)               (pkda.py:375-377)
    A_t   = exp(gP_t) * A_{t-1} + bP_t * k_t^2          (pkda.py:392-395)
    d_t   = log(A_t + eps) - c                          (pkda.py:396)
    w_t   = k_t * exp(-ln(x) * d_t / (1 + |d_t|))       (pkda.py:397-398)
    S'    = diag(exp(g_t)) S_{t-1}                      (pkda.py:399)
    e_t   = v_t - S'^T k_t                              (pkda.py:400)
    S_t   = S' + (beta_t * w_t) e_t^T                   (pkda.py:401-405)
    o_t   = S_t^T (scale * q_t)                         (pkda.py:372,406)

All arithmetic runs in ``dtype`` (float32 to mirror the reference, float64 to
measure the reference's own rounding floor).  Inputs may require grad; the
result is differentiable through torch autograd, which supplies the gradient
oracle.
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn.functional as F
from torch import Tensor


def pkda_recurrent_oracle(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    g: Tensor,
    g_atk: Tensor,
    beta_atk: Tensor,
    beta: Tensor,
    A_log: Tensor,
    dt_bias: Tensor,
    log_atk_scale: Tensor,
    scale: Optional[float] = None,
    squash_x: float = 1.5,
    squash_eps: float = 1e-6,
    initial_state: Optional[Tensor] = None,
    initial_A_state: Optional[Tensor] = None,
    dtype: torch.dtype = torch.float32,
) -> tuple[Tensor, Tensor, Tensor]:
    """Literal recurrence over ``[B,T,H,*]`` inputs.

    Argument order follows the operator boundary
    (``delta_feedback_experiment/fla_ops.py:255-270``): ``g`` is the raw decay
    projection ``[B,T,H,K]``, ``g_atk`` the preconditioner log-decay
    ``[B,T,H]`` (already ``<= 0``), ``beta_atk`` and ``beta`` the two update
    gates ``[B,T,H]``.  Returns ``(o [B,T,H,V] in dtype, S_T [B,H,K,V],
    A_T [B,H,K])``.
    """
    B, T, H, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    cast = lambda t: t.to(dtype)
    qs = cast(q) * scale
    kf, vf = cast(k), cast(v)
    # log-decay per key channel, natural-log domain
    log_alpha = -torch.exp(cast(A_log)).view(1, 1, H, 1) * F.softplus(
        cast(g) + cast(dt_bias).view(1, 1, H, K)
    )
    alpha = torch.exp(log_alpha)  # [B,T,H,K]
    p_decay = torch.exp(cast(g_atk))  # [B,T,H]
    p_gain = cast(beta_atk)
    w_gain = cast(beta)
    centre = cast(log_atk_scale).view(1, H, 1)
    ln_x = math.log(squash_x)

    S = (
        torch.zeros(B, H, K, V, dtype=dtype)
        if initial_state is None
        else cast(initial_state)
    )
    A = (
        torch.zeros(B, H, K, dtype=dtype)
        if initial_A_state is None
        else cast(initial_A_state)
    )
    outs = []
    for t in range(T):
        kt = kf[:, t]  # [B,H,K]
        A = p_decay[:, t, :, None] * A + p_gain[:, t, :, None] * kt * kt
        dev = torch.log(A + squash_eps) - centre
        wkey = kt * torch.exp(-ln_x * dev / (1.0 + dev.abs()))
        S = alpha[:, t, :, :, None] * S
        err = vf[:, t] - (S * kt[..., None]).sum(-2)  # [B,H,V]
        S = S + (w_gain[:, t, :, None] * wkey)[..., None] * err[:, :, None, :]
        outs.append((S * qs[:, t][..., None]).sum(-2))
    o = torch.stack(outs, dim=1) if outs else torch.zeros(B, 0, H, V, dtype=dtype)
    return o, S, A


def pkda_packed_oracle(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    g: Tensor,
    g_atk: Tensor,
    beta_atk: Tensor,
    beta: Tensor,
    A_log: Tensor,
    dt_bias: Tensor,
    log_atk_scale: Tensor,
    cu_seqlens: Sequence[int],
    scale: Optional[float] = None,
    squash_x: float = 1.5,
    squash_eps: float = 1e-6,
    initial_state: Optional[Tensor] = None,
    initial_A_state: Optional[Tensor] = None,
    dtype: torch.dtype = torch.float32,
) -> tuple[Tensor, Tensor, Tensor]:
    """Packed variable-length form: tensors are ``[1, T_total, H, *]`` and
    ``cu_seqlens`` holds ``N+1`` cumulative offsets.  The reference never packs
    (every call passes ``cu_seqlens=None``, ``fla_ops.py:296,329,429,457``);
    batch rows are independent (``tests/test_mtp.py:267-283``), so the packed
    oracle is the recurrence applied to each sequence on its own, with states
    ``[N,H,K,V]`` / ``[N,H,K]``.
    """
    offs = [int(x) for x in cu_seqlens]
    os_, Ss, As = [], [], []
    for n in range(len(offs) - 1):
        lo, hi = offs[n], offs[n + 1]
        sl = lambda t: t[:, lo:hi]
        o, S, A = pkda_recurrent_oracle(
            sl(q), sl(k), sl(v), sl(g), sl(g_atk), sl(beta_atk), sl(beta),
            A_log, dt_bias, log_atk_scale, scale, squash_x, squash_eps,
            None if initial_state is None else initial_state[n : n + 1],
            None if initial_A_state is None else initial_A_state[n : n + 1],
            dtype,
        )
        os_.append(o)
        Ss.append(S)
        As.append(A)
    return torch.cat(os_, dim=1), torch.cat(Ss, dim=0), torch.cat(As, dim=0)


INPUT_NAMES = (
    "q", "k", "v", "g", "g_atk", "beta_atk", "beta", "A_log", "dt_bias",
    "log_atk_scale",
)


def pkda_oracle_with_grads(
    inputs: Sequence[Tensor],
    do: Tensor,
    scale: Optional[float] = None,
    squash_x: float = 1.5,
    squash_eps: float = 1e-6,
    initial_state: Optional[Tensor] = None,
    initial_A_state: Optional[Tensor] = None,
    d_final_state: Optional[Tensor] = None,
    cu_seqlens: Optional[Sequence[int]] = None,
    dtype: torch.dtype = torch.float32,
) -> dict:
    """Forward plus autograd gradients of the ten operator inputs (and of the
    initial states when given) for the cotangent ``do`` (and optionally a
    cotangent on the final matrix state).  Inputs are first rounded to their own
    storage dtype (so bf16 inputs are compared on what the kernel also sees) and
    then promoted to ``dtype``."""
    leaves = [t.detach().to(dtype).clone().requires_grad_(True) for t in inputs]
    extra = []
    S0 = A0 = None
    if initial_state is not None:
        S0 = initial_state.detach().to(dtype).clone().requires_grad_(True)
        extra.append(S0)
    if initial_A_state is not None:
        A0 = initial_A_state.detach().to(dtype).clone().requires_grad_(True)
        extra.append(A0)
    if cu_seqlens is None:
        o, S, A = pkda_recurrent_oracle(
            *leaves, scale, squash_x, squash_eps, S0, A0, dtype)
    else:
        o, S, A = pkda_packed_oracle(
            *leaves, cu_seqlens, scale, squash_x, squash_eps, S0, A0, dtype)
    loss = (o * do.to(dtype)).sum()
    if d_final_state is not None:
        loss = loss + (S * d_final_state.to(dtype)).sum()
    grads = torch.autograd.grad(loss, leaves + extra, allow_unused=True)
    out = {"o": o.detach(), "final_state": S.detach(), "final_A_state": A.detach()}
    for name, gr in zip(INPUT_NAMES, grads[:10]):
        out["d" + name] = gr
    rest = list(grads[10:])
    if S0 is not None:
        out["dinitial_state"] = rest.pop(0)
    if A0 is not None:
        out["dinitial_A_state"] = rest.pop(0)
    return out
