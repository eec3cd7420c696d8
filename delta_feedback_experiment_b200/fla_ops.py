"""Operator boundary of the PKDA recurrence, mirroring the reference's
``delta_feedback_experiment/fla_ops.py`` for this path: the same custom-op
names, signatures, saved-intermediate contract and error behaviour, with the
B200 kernels behind them instead of the Triton fork.

* ``delta_feedback::pkda_recurrence`` (reference ``fla_ops.py:252-349``)
* ``delta_feedback::pkda_recurrence_backward`` (``fla_ops.py:381-499``)

Both have fake implementations (so ``torch.compile(fullgraph=True)`` keeps them
in one graph) and an autograd registration.  Launches go to the current stream,
never synchronise and allocate only through torch, so they can be captured in
CUDA graphs.  There is no fallback: without the CUDA library the operators
raise ``RuntimeError``.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import _lib, ops

CHUNK_SIZE = 64
"""Chunk length shared by forward and backward (reference ``fla_ops.py:32``)."""

PKDA_INTERMEDIATES = ("Aqk", "Akk", "k_precond", "ac_atk", "a_atk", "sa_atk")
"""Always handed to the backward, in this order (reference ``fla_ops.py:46-53``).
Contents here: ``Aqk`` the scaled causal query-key products, ``Akk`` the inverse
UT transform, ``k_precond`` the preconditioned write keys, ``a_atk`` the
preconditioner state at every chunk start, ``sa_atk`` its per-chunk log-decay
sums, and ``ac_atk`` the main gate's per-chunk decay totals."""

PKDA_RETAINED = ("w", "kg", "v_new", "h", "qg")
"""Kept as well unless ``lean`` (reference ``fla_ops.py:57``); a lean backward
rebuilds them with the forward's own kernels, so its gradients are bitwise those
of a retaining backward."""


def fla_ops_available() -> bool:
    """True when the CUDA library loads (name kept from the reference,
    ``fla_ops.py:69-70``)."""
    return _lib.available()


def _intermediate_meta(q: Tensor, v: Tensor, lean: bool):
    return ops.intermediate_meta(q, v, lean)


def _check_intermediates(tensors, q: Tensor, v: Tensor, lean: bool) -> None:
    """The list the forward hands back must be exactly what the fake implementation
    promises to the compiler (count, and per entry shape, dtype, device, contiguity):
    a mismatch would surface far away, as a stride or shape error inside a compiled
    graph.  Same contract as the reference's check (``fla_ops.py:100-128``)."""
    names = PKDA_INTERMEDIATES + (() if lean else PKDA_RETAINED)
    promised = _intermediate_meta(q, v, lean)
    if len(tensors) != len(promised):
        raise RuntimeError(f"the PKDA forward produced {len(tensors)} intermediates where "
                           f"{len(promised)} are promised")
    for name, t, (shape, dtype) in zip(names, tensors, promised):
        found = None if t is None else (tuple(t.shape), t.dtype, t.device, t.is_contiguous())
        if found != (tuple(shape), dtype, q.device, True):
            raise RuntimeError(f"PKDA intermediate {name}: forward produced {found}, the fake "
                               f"implementation promises {(tuple(shape), dtype, q.device, True)}")


def _chunk_capable(q: Tensor) -> bool:
    return q.dtype == torch.bfloat16 and q.shape[-1] == 128


@torch.library.custom_op("delta_feedback::pkda_recurrence", mutates_args=(), device_types="cuda")
def pkda_recurrence(
    q: Tensor, k: Tensor, v: Tensor, g: Tensor, g_atk: Tensor, beta_atk: Tensor, beta: Tensor,
    A_log: Tensor, dt_bias: Tensor, log_atk_scale: Tensor,
    scale: float, squash_x: float, squash_eps: float, lean: bool,
) -> tuple[Tensor, list[Tensor]]:
    """Dense training / prefill forward without recurrent state: returns the
    output and the intermediates its backward reuses (all eleven unless
    ``lean``).  ``g`` is the raw decay projection; the gate and its chunk-local
    cumulative sum are computed inside the kernels."""
    if _chunk_capable(q):
        o, _, _, saved = ops.chunk_forward(
            q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale,
            scale, squash_x, squash_eps)
        saved = saved[:6] if lean else saved
        _check_intermediates(saved, q, v, lean)
        return o, saved
    # fp32 activations or another head width: exact token-by-token kernel.
    o, _, _ = ops.recurrent_forward(
        q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale,
        scale, squash_x, squash_eps, output_final_state=False)
    # The exact backward needs none of the intermediates; the list only keeps the
    # operator's output contract (names, shapes, dtypes), so it is left unwritten.
    saved = [torch.empty(shape, device=q.device, dtype=dt)
             for shape, dt in _intermediate_meta(q, v, lean)]
    _check_intermediates(saved, q, v, lean)
    return o, saved


@pkda_recurrence.register_fake
def _pkda_recurrence_fake(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale,
                          scale, squash_x, squash_eps, lean):
    output = torch.empty((*q.shape[:3], v.shape[-1]), device=q.device, dtype=q.dtype)
    saved = [torch.empty(shape, device=q.device, dtype=dt)
             for shape, dt in _intermediate_meta(q, v, lean)]
    return output, saved


@torch.library.custom_op("delta_feedback::pkda_recurrence_backward", mutates_args=(),
                         device_types="cuda")
def _pkda_recurrence_backward(
    q: Tensor, k: Tensor, v: Tensor, g: Tensor, g_atk: Tensor, beta_atk: Tensor, beta: Tensor,
    A_log: Tensor, dt_bias: Tensor, log_atk_scale: Tensor, saved: list[Tensor], do: Tensor,
    scale: float, squash_x: float, squash_eps: float,
    autocast_dtype: Optional[torch.dtype], lean: bool,
) -> list[Tensor]:
    """Ten input gradients, each in its input's dtype (``g_atk``, ``A_log``,
    ``dt_bias``, ``log_atk_scale`` stay fp32).  ``autocast_dtype`` is accepted
    for signature parity; the kernels fix their own arithmetic (bf16 operands,
    fp32 accumulation) and do not consult autocast."""
    del autocast_dtype
    expected = len(PKDA_INTERMEDIATES) + (0 if lean else len(PKDA_RETAINED))
    if len(saved) != expected:
        raise RuntimeError(
            f"PKDA backward received {len(saved)} intermediates, not {expected}")
    if not _chunk_capable(q):
        # fp32 activations or another head width: exact backward (ignores ``saved``)
        grads, _, _ = ops.recurrent_backward(
            q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale,
            scale, squash_x, squash_eps, do)
        inputs = (q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale)
        return [gr.reshape(t.shape).to(t.dtype) for gr, t in zip(grads, inputs)]
    grads, _, _ = ops.chunk_backward(
        q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale,
        scale, squash_x, squash_eps, saved, do, lean=lean)
    inputs = (q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale)
    return [gr.reshape(t.shape).to(t.dtype) for gr, t in zip(grads, inputs)]


@_pkda_recurrence_backward.register_fake
def _pkda_recurrence_backward_fake(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias,
                                   log_atk_scale, saved, do, scale, squash_x, squash_eps,
                                   autocast_dtype, lean):
    # the real operator returns fresh contiguous tensors whatever the inputs' strides
    return [t.new_empty(t.shape) for t in
            (q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale)]


def _recurrence_setup_context(ctx, inputs, output) -> None:
    *tensors, scale, squash_x, squash_eps, lean = inputs
    _o, saved = output
    ctx.save_for_backward(*tensors, *saved)
    ctx.scalars = (scale, squash_x, squash_eps, lean)
    ctx.autocast_dtype = (
        torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else None)
    ctx.mark_non_differentiable(*saved)


def _recurrence_backward(ctx, do, _dsaved):
    tensors = ctx.saved_tensors  # unpacked exactly once (checkpoint replays allow no more)
    inputs, saved = tensors[:10], list(tensors[10:])
    scale, squash_x, squash_eps, lean = ctx.scalars
    grads = _pkda_recurrence_backward(
        *inputs, saved, do, scale, squash_x, squash_eps, ctx.autocast_dtype, lean)
    return (*grads, None, None, None, None)


pkda_recurrence.register_autograd(_recurrence_backward, setup_context=_recurrence_setup_context)

__all__ = ["CHUNK_SIZE", "PKDA_INTERMEDIATES", "PKDA_RETAINED", "fla_ops_available",
           "pkda_recurrence"]
