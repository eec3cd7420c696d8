"""Host-side mirror of the PKDA layer's recurrence dispatch
(``delta_feedback_experiment/pkda.py:412-475``) and of the two stateful
operators it imports from the flash-linear-attention fork
(``pkda.py:27-34``): ``chunk_precond_kda`` and ``fused_recurrent_precond_kda``,
with the keyword signature of the call site at ``pkda.py:450-475`` plus the
packed-sequence arguments (``cu_seqlens``, ``cu_seqlens_cpu``).
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import _lib, ops
from .fla_ops import fla_ops_available, pkda_recurrence


def pkda_cuda_available() -> bool:
    """Whether the dense operators and the cached-decode kernels exist
    (reference ``pkda.py:47-53``)."""
    return fla_ops_available()


def _check_flags(use_gate_in_kernel: bool, use_qk_l2norm_in_kernel: bool) -> None:
    if not use_gate_in_kernel:
        raise NotImplementedError("the kernels always compute the decay gate from the raw projection")
    if use_qk_l2norm_in_kernel:
        raise NotImplementedError("q and k are normalised upstream (reference pkda.py:464-465)")


def fused_recurrent_precond_kda(
    q: Tensor, k: Tensor, v: Tensor, g: Tensor, g_atk: Tensor, beta_atk: Tensor, beta: Tensor,
    A_log: Tensor, dt_bias: Tensor,
    initial_state: Optional[Tensor] = None, initial_A_state: Optional[Tensor] = None,
    output_final_state: bool = False, use_gate_in_kernel: bool = True,
    use_qk_l2norm_in_kernel: bool = False, disable_recompute: bool = False,
    x: float = 1.5, eps: float = 1e-6, log_atk_scale: Optional[Tensor] = None,
    scale: Optional[float] = None, cu_seqlens: Optional[Tensor] = None,
    cu_seqlens_cpu: Optional[Tensor] = None, inplace_state: bool = False,
) -> tuple[Tensor, Optional[Tensor], Optional[Tensor]]:
    """Token-by-token recurrence (decode and short cached prefill); forward only.
    Returns ``(o, state, a_state)``.  ``inplace_state=True`` (an extension)
    updates the given fp32 states in place and returns them."""
    del disable_recompute, cu_seqlens_cpu
    _check_flags(use_gate_in_kernel, use_qk_l2norm_in_kernel)
    if log_atk_scale is None:
        raise RuntimeError("log_atk_scale is required")
    with torch.no_grad():
        return ops.recurrent_forward(
            q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale, scale, x, eps,
            initial_state, initial_A_state, cu_seqlens, output_final_state, inplace_state)


class _ChunkPKDA(torch.autograd.Function):
    """Chunked recurrence with optional initial / final state and packing."""

    @staticmethod
    def forward(ctx, q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale,
                initial_state, initial_A_state, scale, x, eps, cu_seqlens, output_final_state,
                lean):
        o, S, A, saved = ops.chunk_forward(
            q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale, scale, x, eps,
            initial_state, initial_A_state, cu_seqlens, output_final_state)
        keep = saved[:6] if lean else saved
        ctx.save_for_backward(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale,
                              initial_state, initial_A_state, cu_seqlens, *keep)
        ctx.conf = (scale, x, eps, lean)
        if S is not None:
            ctx.mark_non_differentiable(A)
            return o, S, A
        return o, None, None

    @staticmethod
    def backward(ctx, do, dS, _dA):
        t = ctx.saved_tensors
        inputs, S0, A0, cu, saved = t[:10], t[10], t[11], t[12], list(t[13:])
        scale, x, eps, lean = ctx.conf
        want = S0 is not None or A0 is not None
        grads, dS0, dA0 = ops.chunk_backward(
            *inputs, scale, x, eps, saved, do, S0, A0, cu, dS, lean, want)
        out = [gr.reshape(i.shape).to(i.dtype) for gr, i in zip(grads, inputs)]
        return (*out, dS0 if S0 is not None else None, dA0 if A0 is not None else None,
                None, None, None, None, None, None)


class _ExactPKDA(torch.autograd.Function):
    """Token-by-token kernels (exact fp32 arithmetic) with autograd: the path for
    fp32 activations and for head widths other than 128."""

    @staticmethod
    def forward(ctx, q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale,
                initial_state, initial_A_state, scale, x, eps, cu_seqlens, output_final_state):
        o, S, A = ops.recurrent_forward(
            q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale, scale, x, eps,
            initial_state, initial_A_state, cu_seqlens, output_final_state)
        ctx.save_for_backward(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale,
                              initial_state, initial_A_state, cu_seqlens)
        ctx.conf = (scale, x, eps)
        if S is not None:
            ctx.mark_non_differentiable(A)
            return o, S, A
        return o, None, None

    @staticmethod
    def backward(ctx, do, dS, _dA):
        t = ctx.saved_tensors
        inputs, S0, A0, cu = t[:10], t[10], t[11], t[12]
        scale, x, eps = ctx.conf
        want = S0 is not None or A0 is not None
        grads, dS0, dA0 = ops.recurrent_backward(*inputs, scale, x, eps, do, S0, A0, cu, dS, want)
        out = [gr.reshape(i.shape).to(i.dtype) for gr, i in zip(grads, inputs)]
        return (*out, dS0 if S0 is not None else None, dA0 if A0 is not None else None,
                None, None, None, None, None)


def chunk_precond_kda(
    q: Tensor, k: Tensor, v: Tensor, g: Tensor, g_atk: Tensor, beta_atk: Tensor, beta: Tensor,
    A_log: Tensor, dt_bias: Tensor,
    initial_state: Optional[Tensor] = None, initial_A_state: Optional[Tensor] = None,
    output_final_state: bool = False, use_gate_in_kernel: bool = True,
    use_qk_l2norm_in_kernel: bool = False, disable_recompute: bool = False,
    x: float = 1.5, eps: float = 1e-6, log_atk_scale: Optional[Tensor] = None,
    scale: Optional[float] = None, cu_seqlens: Optional[Tensor] = None,
    cu_seqlens_cpu: Optional[Tensor] = None,
) -> tuple[Tensor, Optional[Tensor], Optional[Tensor]]:
    """Chunked recurrence seeded from / returning recurrent state, with packed
    sequences (``[1, T_total, H, D]`` tensors, ``cu_seqlens`` ``[N+1]``, states
    ``[N,H,D,D]`` / ``[N,H,D]``).  bf16 activations with head width 128 take the
    chunked tensor-core kernels; fp32 activations and other head widths take the
    exact token-by-token kernels.  Both are differentiable.  ``disable_recompute=False`` (the reference's choice,
    ``pkda.py:468``) keeps only the six always-saved intermediates."""
    del cu_seqlens_cpu
    _check_flags(use_gate_in_kernel, use_qk_l2norm_in_kernel)
    if log_atk_scale is None:
        raise RuntimeError("log_atk_scale is required")
    if q.dtype == torch.bfloat16 and q.shape[-1] == 128:
        return _ChunkPKDA.apply(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale,
                                initial_state, initial_A_state, scale, x, eps, cu_seqlens,
                                output_final_state, not disable_recompute)
    return _ExactPKDA.apply(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale,
                            initial_state, initial_A_state, scale, x, eps, cu_seqlens,
                            output_final_state)


def pkda_cuda_recurrence(
    q: Tensor, k: Tensor, v: Tensor, raw_decay: Tensor, beta: Tensor, precond_decay: Tensor,
    precond_beta: Tensor, state: Optional[Tensor], a_state: Optional[Tensor],
    output_final_state: bool, *, A_log: Tensor, dt_bias: Tensor, log_precond_center: Tensor,
    head_dim: int, squash_x: float = 1.5, squash_eps: float = 1e-6, lean_recurrence: bool = True,
    training: bool = False,
) -> tuple[Tensor, Optional[Tensor], Optional[Tensor]]:
    """The dispatch of ``PreconditionedKDA._cuda_recurrence`` (reference
    ``pkda.py:412-475``) as a free function: the layer's parameters and flags
    are keyword arguments instead of ``self`` attributes."""
    if not pkda_cuda_available():
        raise RuntimeError("CUDA PKDA requires the libpkda_b200 build")
    if state is None and a_state is None and not output_final_state:
        output, _saved = pkda_recurrence(
            q, k, v, raw_decay, precond_decay, precond_beta, beta, A_log, dt_bias,
            log_precond_center, head_dim ** -0.5, squash_x, squash_eps, lean_recurrence)
        return output, None, None
    kwargs = dict(
        q=q, k=k, v=v, g=raw_decay, g_atk=precond_decay, beta_atk=precond_beta, beta=beta,
        A_log=A_log, dt_bias=dt_bias, initial_state=state, initial_A_state=a_state,
        output_final_state=output_final_state, use_gate_in_kernel=True,
        use_qk_l2norm_in_kernel=False, disable_recompute=False, x=squash_x, eps=squash_eps,
        log_atk_scale=log_precond_center)
    if output_final_state and q.shape[1] <= 64 and not training:
        return fused_recurrent_precond_kda(**kwargs)
    return chunk_precond_kda(**kwargs)


__all__ = ["chunk_precond_kda", "fused_recurrent_precond_kda", "pkda_cuda_available",
           "pkda_cuda_recurrence"]
