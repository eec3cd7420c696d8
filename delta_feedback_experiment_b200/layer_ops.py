"""The two fused operators next to the recurrence inside the PKDA layer, behind
the reference's operator names and signatures:

* ``pkda_qkv_conv(x, weight, head_dim, norm_channels, eps) -> (q, k, v)`` --
  ``delta_feedback::pkda_qkv_conv`` of the reference
  (``delta_feedback_experiment/fla_ops.py:134-249``): causal depthwise short
  convolution over the concatenated Q|K|V projection, SiLU, per-head L2
  normalisation of the first ``norm_channels`` channels, three output slabs.
* ``pkda_norm_gate(x, gate, weight, eps) -> (y, rstd)`` --
  ``delta_feedback::pkda_norm_gate`` (``fla_ops.py:572-657``): per-head RMS
  normalisation times a learned weight times ``sigmoid(gate)``.

Both are registered as ``torch.library.custom_op`` with fake implementations and
autograd, as the reference registers them, and both call the C ABI of
``libpkda_b200.so``; there is no other implementation behind them.
"""

from __future__ import annotations

import ctypes as C

import torch
from torch import Tensor

from . import _lib, ops

_DTYPES = {torch.bfloat16: _lib.PKDA_BF16, torch.float32: _lib.PKDA_F32}


def _dtype_code(t: Tensor) -> int:
    if t.dtype not in _DTYPES:
        raise RuntimeError(f"PKDA layer operators take bf16 or fp32 activations, got {t.dtype}")
    return _DTYPES[t.dtype]


def _workspace(nbytes: int, device) -> Tensor:
    return torch.empty((max(int(nbytes), 16),), device=device, dtype=torch.uint8)


# ----------------------------------------------------------------- convolution
def _conv_args(x: Tensor, weight: Tensor, head_dim: int, norm_channels: int, eps: float):
    if x.dim() != 3 or weight.dim() != 2 or weight.shape[0] != x.shape[-1] or x.shape[-1] % 3:
        raise RuntimeError("pkda_qkv_conv expects x [B,T,3W] and weight [3W,taps]")
    a = _lib.QkvConvArgs()
    a.batch, a.seq_len, a.channels = x.shape
    a.taps = weight.shape[1]
    a.head_dim, a.norm_channels, a.eps = int(head_dim), int(norm_channels), float(eps)
    a.dtype = _dtype_code(x)
    return a


@ops._on_tensor_device
def qkv_conv_forward(x: Tensor, weight: Tensor, head_dim: int, norm_channels: int, eps: float):
    ops._require_cuda(x, weight)
    lib = _lib.load()
    x = x.contiguous()
    w32 = weight.detach().to(torch.float32).contiguous()
    a = _conv_args(x, w32, head_dim, norm_channels, eps)
    B, T, C3 = x.shape
    q, k, v = (torch.empty((B, T, C3 // 3), device=x.device, dtype=x.dtype) for _ in range(3))
    a.x, a.weight = x.data_ptr(), w32.data_ptr()
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    _lib.check(lib.pkda_qkv_conv_fwd(C.byref(a), _lib.current_stream()), "pkda_qkv_conv_fwd")
    ops._count(lib)
    return q, k, v


@ops._on_tensor_device
def qkv_conv_backward(x: Tensor, weight: Tensor, dq: Tensor, dk: Tensor, dv: Tensor, head_dim: int,
                      norm_channels: int, eps: float):
    ops._require_cuda(x, weight, dq, dk, dv)
    lib = _lib.load()
    x = x.contiguous()
    w32 = weight.detach().to(torch.float32).contiguous()
    dq, dk, dv = (t.to(x.dtype).contiguous() for t in (dq, dk, dv))
    a = _conv_args(x, w32, head_dim, norm_channels, eps)
    dx = torch.empty_like(x)
    dw = torch.empty_like(w32)
    a.x, a.weight = x.data_ptr(), w32.data_ptr()
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.dx, a.dweight = dx.data_ptr(), dw.data_ptr()
    nbytes = lib.pkda_qkv_conv_bwd_workspace_bytes(C.byref(a))
    ws = _workspace(nbytes, x.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
    _lib.check(lib.pkda_qkv_conv_bwd(C.byref(a), _lib.current_stream()), "pkda_qkv_conv_bwd")
    ops._count(lib)
    return dx, dw.to(weight.dtype)


@torch.library.custom_op("delta_feedback::pkda_qkv_conv", mutates_args=(), device_types="cuda")
def pkda_qkv_conv(x: Tensor, weight: Tensor, head_dim: int, norm_channels: int,
                  eps: float) -> tuple[Tensor, Tensor, Tensor]:
    """Signature and meaning of the reference's operator (``fla_ops.py:137-170``)."""
    return qkv_conv_forward(x, weight, head_dim, norm_channels, eps)


@pkda_qkv_conv.register_fake
def _pkda_qkv_conv_fake(x, weight, head_dim, norm_channels, eps):
    batch, length, _ = x.shape
    width = weight.shape[0] // 3
    return tuple(x.new_empty(batch, length, width) for _ in range(3))


@torch.library.custom_op("delta_feedback::pkda_qkv_conv_backward", mutates_args=(),
                         device_types="cuda")
def _pkda_qkv_conv_backward(x: Tensor, weight: Tensor, dq: Tensor, dk: Tensor, dv: Tensor,
                            head_dim: int, norm_channels: int, eps: float) -> tuple[Tensor, Tensor]:
    return qkv_conv_backward(x, weight, dq, dk, dv, head_dim, norm_channels, eps)


@_pkda_qkv_conv_backward.register_fake
def _pkda_qkv_conv_backward_fake(x, weight, dq, dk, dv, head_dim, norm_channels, eps):
    # the real operators return contiguous tensors whatever the inputs' strides
    return x.new_empty(x.shape), weight.new_empty(weight.shape)


def _conv_setup_context(ctx, inputs, output) -> None:
    x, weight, head_dim, norm_channels, eps = inputs
    ctx.save_for_backward(x, weight)
    ctx.geometry = (head_dim, norm_channels, eps)


def _conv_backward(ctx, dq, dk, dv):
    x, weight = ctx.saved_tensors
    head_dim, norm_channels, eps = ctx.geometry
    dx, dw = _pkda_qkv_conv_backward(x, weight, dq, dk, dv, head_dim, norm_channels, eps)
    return dx, dw, None, None, None


pkda_qkv_conv.register_autograd(_conv_backward, setup_context=_conv_setup_context)


# ------------------------------------------------------------------- norm gate
def _ng_args(x: Tensor, gate: Tensor, weight: Tensor, eps: float):
    if gate.shape != x.shape or weight.dim() != 1 or weight.shape[0] != x.shape[-1]:
        raise RuntimeError("pkda_norm_gate expects x, gate [..., D] and weight [D]")
    a = _lib.NormGateArgs()
    a.dim = x.shape[-1]
    a.rows = x.numel() // x.shape[-1]
    a.dtype = _dtype_code(x)
    a.eps = float(eps)
    return a


@ops._on_tensor_device
def norm_gate_forward(x: Tensor, gate: Tensor, weight: Tensor, eps: float):
    ops._require_cuda(x, gate, weight)
    lib = _lib.load()
    x = x.contiguous()
    gate = gate.to(x.dtype).contiguous()
    w32 = weight.detach().to(torch.float32).contiguous()
    a = _ng_args(x, gate, w32, eps)
    y = torch.empty_like(x)
    rstd = torch.empty((a.rows,), device=x.device, dtype=torch.float32)
    a.x, a.gate, a.weight = x.data_ptr(), gate.data_ptr(), w32.data_ptr()
    a.y, a.rstd = y.data_ptr(), rstd.data_ptr()
    _lib.check(lib.pkda_norm_gate_fwd(C.byref(a), _lib.current_stream()), "pkda_norm_gate_fwd")
    ops._count(lib)
    return y, rstd


@ops._on_tensor_device
def norm_gate_backward(x: Tensor, gate: Tensor, weight: Tensor, rstd: Tensor, dy: Tensor, eps: float):
    ops._require_cuda(x, gate, weight, rstd, dy)
    lib = _lib.load()
    x = x.contiguous()
    gate_c = gate.to(x.dtype).contiguous()
    dy = dy.to(x.dtype).contiguous()
    w32 = weight.detach().to(torch.float32).contiguous()
    rstd = rstd.to(torch.float32).contiguous()
    a = _ng_args(x, gate_c, w32, eps)
    dx, dg = torch.empty_like(x), torch.empty_like(x)
    dw = torch.empty_like(w32)
    a.x, a.gate, a.weight = x.data_ptr(), gate_c.data_ptr(), w32.data_ptr()
    a.rstd, a.dy = rstd.data_ptr(), dy.data_ptr()
    a.dx, a.dgate, a.dweight = dx.data_ptr(), dg.data_ptr(), dw.data_ptr()
    nbytes = lib.pkda_norm_gate_bwd_workspace_bytes(C.byref(a))
    ws = _workspace(nbytes, x.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
    _lib.check(lib.pkda_norm_gate_bwd(C.byref(a), _lib.current_stream()), "pkda_norm_gate_bwd")
    ops._count(lib)
    return dx, dg.to(gate.dtype), dw.to(weight.dtype)


@torch.library.custom_op("delta_feedback::pkda_norm_gate", mutates_args=(), device_types="cuda")
def pkda_norm_gate(x: Tensor, gate: Tensor, weight: Tensor, eps: float) -> tuple[Tensor, Tensor]:
    """Signature and meaning of the reference's operator (``fla_ops.py:575-593``);
    ``rstd`` has one fp32 entry per row and feeds the backward."""
    return norm_gate_forward(x, gate, weight, eps)


@pkda_norm_gate.register_fake
def _pkda_norm_gate_fake(x, gate, weight, eps):
    rows = x.numel() // x.shape[-1]
    return x.new_empty(x.shape), torch.empty((rows,), device=x.device, dtype=torch.float32)


@torch.library.custom_op("delta_feedback::pkda_norm_gate_backward", mutates_args=(),
                         device_types="cuda")
def _pkda_norm_gate_backward(x: Tensor, gate: Tensor, weight: Tensor, rstd: Tensor, dy: Tensor,
                             eps: float) -> tuple[Tensor, Tensor, Tensor]:
    return norm_gate_backward(x, gate, weight, rstd, dy, eps)


@_pkda_norm_gate_backward.register_fake
def _pkda_norm_gate_backward_fake(x, gate, weight, rstd, dy, eps):
    return x.new_empty(x.shape), gate.new_empty(gate.shape), weight.new_empty(weight.shape)


def _norm_gate_setup_context(ctx, inputs, output) -> None:
    x, gate, weight, eps = inputs
    _y, rstd = output
    ctx.save_for_backward(x, gate, weight, rstd)
    ctx.eps = eps
    ctx.mark_non_differentiable(rstd)


def _norm_gate_backward(ctx, dy, _drstd):
    x, gate, weight, rstd = ctx.saved_tensors
    dx, dg, dw = _pkda_norm_gate_backward(x, gate, weight, rstd, dy, ctx.eps)
    return dx, dg, dw, None


pkda_norm_gate.register_autograd(_norm_gate_backward, setup_context=_norm_gate_setup_context)

# ----------------------------------------------------------------- decode step
@ops._on_tensor_device
def pkda_decode_step(qkv: Tensor, conv_state, conv_weight: Tensor, g: Tensor, g_atk: Tensor,
                     beta_atk: Tensor, beta: Tensor, A_log: Tensor, dt_bias: Tensor,
                     log_atk_scale: Tensor, state: Tensor, a_state: Tensor, gate, norm_weight,
                     head_dim: int, scale=None, squash_x: float = 1.5, squash_eps: float = 1e-6,
                     qk_eps: float = 1e-6, norm_eps: float = 1e-6) -> Tensor:
    """One cached decoding step of the layer's token mixer in one launch: the
    history-prefixed Q|K|V convolution, one recurrence step and the RMS-norm gate
    (reference: ``pkda.py:239-288, 473-474, 539-541`` and the cache update of
    ``model.py:775-787``).  ``conv_state`` (three ``[B, W, taps-1]`` tensors), ``state``
    (``[B,H,D,D]`` fp32) and ``a_state`` (``[B,H,D]`` fp32) are the decode cache and are
    UPDATED IN PLACE.  ``qkv`` is the new projection row ``[B, 3W]``; ``g`` the raw decay
    ``[B,H,D]``; ``g_atk`` (fp32), ``beta_atk``, ``beta`` are ``[B,H]``; ``gate`` the
    output-gate logits ``[B,H,D]`` or None (the result is then the recurrence output).
    Returns ``[B,H,D]``."""
    ops._require_cuda(qkv, conv_weight, g, g_atk, beta_atk, beta, state, a_state, *conv_state, A_log, dt_bias,
                      log_atk_scale, gate, norm_weight)
    lib = _lib.load()
    B, C3 = qkv.shape
    W = C3 // 3
    H = W // head_dim
    taps = conv_weight.shape[1]
    act = qkv.dtype
    cache = [state, a_state, *conv_state]
    if state.dtype != torch.float32 or a_state.dtype != torch.float32 or not all(t.is_contiguous() for t in cache):
        raise RuntimeError("the decode cache (state, a_state fp32; conv histories) must be contiguous: "
                           "it is updated in place")
    if any(c.dtype != act or tuple(c.shape) != (B, W, taps - 1) for c in conv_state):
        raise RuntimeError("conv_state must be three [B, W, taps-1] tensors of the activation dtype")
    a = _lib.DecodeStepArgs()
    a.batch, a.heads, a.head_dim, a.taps = B, H, int(head_dim), int(taps)
    a.dtype = _dtype_code(qkv)
    a.scale = float(head_dim ** -0.5 if scale is None else scale)
    a.squash_x, a.squash_eps, a.qk_eps, a.norm_eps = float(squash_x), float(squash_eps), float(qk_eps), float(norm_eps)
    keep = [qkv.contiguous(), conv_weight.detach().float().contiguous(), g.to(act).contiguous(),
            g_atk.float().contiguous(), beta_atk.to(act).contiguous(), beta.to(act).contiguous(),
            A_log.detach().float().contiguous(), dt_bias.detach().float().contiguous(),
            log_atk_scale.detach().float().contiguous()]
    (a.qkv, a.conv_weight, a.g, a.g_atk, a.beta_atk, a.beta, a.A_log, a.dt_bias,
     a.log_atk_scale) = [t.data_ptr() for t in keep]
    a.conv_q, a.conv_k, a.conv_v = [c.data_ptr() for c in conv_state]
    a.state, a.a_state = state.data_ptr(), a_state.data_ptr()
    out = torch.empty((B, H, head_dim), device=qkv.device, dtype=act)
    if gate is not None:
        keep += [gate.to(act).contiguous(), norm_weight.detach().float().contiguous()]
        a.gate, a.norm_weight = keep[-2].data_ptr(), keep[-1].data_ptr()
    a.out = out.data_ptr()
    _lib.check(lib.pkda_decode_step(C.byref(a), _lib.current_stream()), "pkda_decode_step")
    ops._count(lib)
    return out


# ------------------------------------------------------------ control epilogue
def pack_control_gradients(gradients) -> Tensor:
    """The reference's ``pack_control_gradients`` (``cuda_kernels.py:1529-1535``): five
    contiguous slices with a common leading shape -> one row-major packed tensor."""
    if len(gradients) != 5:
        raise ValueError("PKDA has exactly five packed control gradients")
    g0 = gradients[0]
    ops._require_cuda(*gradients)
    prefix = g0.shape[:-1]
    if any(g.shape[:-1] != prefix or g.dtype != g0.dtype for g in gradients[1:]):
        raise ValueError("control gradients must share their leading shape and dtype")
    if any(not g.is_contiguous() for g in gradients):
        raise ValueError("control gradients must be contiguous")
    lib = _lib.load()
    return _pack_on_device(g0, lib, gradients, prefix)


@ops._on_tensor_device
def _pack_on_device(g0, lib, gradients, prefix) -> Tensor:
    a = _lib.PackControlArgs()
    a.rows = g0.numel() // max(g0.shape[-1], 1) if g0.shape[-1] else (gradients[1].numel() // max(gradients[1].shape[-1], 1))
    total = 0
    for i, g in enumerate(gradients):
        a.sizes[i] = g.shape[-1]
        a.grads[i] = g.data_ptr()
        total += g.shape[-1]
    a.dtype = _dtype_code(g0)
    out = torch.empty((*prefix, total), device=g0.device, dtype=g0.dtype)
    a.out = out.data_ptr()
    _lib.check(lib.pkda_pack_control_gradients(C.byref(a), _lib.current_stream()), "pkda_pack_control_gradients")
    ops._count(lib)
    return out


@torch.library.custom_op("delta_feedback::pack_control_gradients", mutates_args=(), device_types="cuda")
def _pack_control_gradients_op(grad0: Tensor, grad1: Tensor, grad2: Tensor, grad3: Tensor,
                               grad4: Tensor) -> Tensor:
    """Name and signature of the reference's operator (``cuda_kernels.py:1493-1506``)."""
    return pack_control_gradients((grad0, grad1, grad2, grad3, grad4))


@_pack_control_gradients_op.register_fake
def _pack_control_gradients_fake(grad0, grad1, grad2, grad3, grad4):
    total = sum(g.shape[-1] for g in (grad0, grad1, grad2, grad3, grad4))
    return torch.empty((*grad0.shape[:-1], total), device=grad0.device, dtype=grad0.dtype)


def _controls_args(packed: Tensor, A_log_precond: Tensor, dt_bias_precond: Tensor, hidden: int):
    H = A_log_precond.shape[0]
    if packed.shape[-1] != 2 * hidden + 3 * H:
        raise RuntimeError("packed control row must be [hidden | H | H | H | hidden]")
    a = _lib.ControlsArgs()
    a.rows = packed.numel() // packed.shape[-1]
    a.heads, a.hidden, a.dtype = H, int(hidden), _dtype_code(packed)
    return a


class _Controls(torch.autograd.Function):
    """Split of the packed control projection with the three per-head activations fused in
    (forward) and the packed gradient written in one pass (backward)."""

    @staticmethod
    def forward(ctx, packed: Tensor, A_log_precond: Tensor, dt_bias_precond: Tensor, hidden: int):
        ops._require_cuda(packed, A_log_precond, dt_bias_precond)
        with torch.cuda.device(packed.device):
            return _Controls._forward(ctx, packed, A_log_precond, dt_bias_precond, hidden)

    @staticmethod
    def _forward(ctx, packed, A_log_precond, dt_bias_precond, hidden):
        lib = _lib.load()
        packed = packed.contiguous()
        a32 = A_log_precond.detach().float().contiguous()
        b32 = dt_bias_precond.detach().float().contiguous()
        a = _controls_args(packed, a32, b32, hidden)
        H = a.heads
        lead = packed.shape[:-1]
        beta = torch.empty((*lead, H), device=packed.device, dtype=packed.dtype)
        beta_atk = torch.empty_like(beta)
        g_atk = torch.empty((*lead, H), device=packed.device, dtype=torch.float32)
        a.packed, a.A_log_precond, a.dt_bias_precond = packed.data_ptr(), a32.data_ptr(), b32.data_ptr()
        a.beta, a.g_atk, a.beta_atk = beta.data_ptr(), g_atk.data_ptr(), beta_atk.data_ptr()
        _lib.check(lib.pkda_controls_fwd(C.byref(a), _lib.current_stream()), "pkda_controls_fwd")
        ops._count(lib)
        ctx.save_for_backward(packed, A_log_precond, dt_bias_precond)
        ctx.hidden = hidden
        return packed[..., :hidden], beta, g_atk, beta_atk, packed[..., hidden + 3 * H:]

    @staticmethod
    def backward(ctx, d_h0, d_beta, d_g_atk, d_beta_atk, d_h1):
        saved = ctx.saved_tensors  # unpacked exactly once (checkpoint replays allow no more)
        with torch.cuda.device(saved[0].device):
            return _Controls._backward(ctx, saved, d_h0, d_beta, d_g_atk, d_beta_atk, d_h1)

    @staticmethod
    def _backward(ctx, saved, d_h0, d_beta, d_g_atk, d_beta_atk, d_h1):
        packed, A_log_precond, dt_bias_precond = saved
        lib = _lib.load()
        a32 = A_log_precond.detach().float().contiguous()
        b32 = dt_bias_precond.detach().float().contiguous()
        a = _controls_args(packed, a32, b32, ctx.hidden)
        act = packed.dtype
        keep = [None if g is None else g.to(torch.float32 if i == 2 else act).contiguous()
                for i, g in enumerate((d_h0, d_beta, d_g_atk, d_beta_atk, d_h1))]
        d_packed = torch.empty_like(packed)
        dA = torch.empty_like(a32)
        db = torch.empty_like(b32)
        a.packed, a.A_log_precond, a.dt_bias_precond = packed.data_ptr(), a32.data_ptr(), b32.data_ptr()
        (a.d_decay_hidden, a.d_beta, a.d_g_atk, a.d_beta_atk, a.d_gate_hidden) = [
            None if t is None else t.data_ptr() for t in keep]
        a.d_packed, a.dA_log_precond, a.ddt_bias_precond = d_packed.data_ptr(), dA.data_ptr(), db.data_ptr()
        nbytes = lib.pkda_controls_bwd_workspace_bytes(C.byref(a))
        ws = _workspace(nbytes, packed.device)
        a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
        _lib.check(lib.pkda_controls_bwd(C.byref(a), _lib.current_stream()), "pkda_controls_bwd")
        ops._count(lib)
        return d_packed, dA.to(A_log_precond.dtype), db.to(dt_bias_precond.dtype), None


def pkda_controls(packed: Tensor, A_log_precond: Tensor, dt_bias_precond: Tensor, hidden: int):
    """``(decay_hidden, beta, precond_decay, precond_beta, output_gate_hidden)`` from the packed
    control projection ``[..., hidden + 3H + hidden]`` -- the middle of the reference's
    ``PreconditionedKDA._controls`` (``pkda.py:318-353``) with its backward packing
    (``pkda.py:56-74``).  The two hidden pieces are views of ``packed``."""
    return _Controls.apply(packed, A_log_precond, dt_bias_precond, hidden)


__all__ = ["pkda_controls", "pack_control_gradients", "pkda_decode_step", "pkda_qkv_conv", "pkda_norm_gate", "qkv_conv_forward", "qkv_conv_backward",
           "norm_gate_forward", "norm_gate_backward"]
