"""Low-level launchers: allocate outputs with torch, fill the C structs, call
the C ABI on the current CUDA stream.  No arithmetic happens in Python.
"""

from __future__ import annotations

import ctypes as C
import functools
from typing import Optional, Sequence

import torch
from torch import Tensor

from . import _lib

CHUNK_SIZE = _lib.CHUNK

LAUNCHES = 0
"""Kernels enqueued through this module since import (launch accounting)."""


_TRACK_STATUS = False
_LAST_STATUS = None
_LAST_BWD_STATUS = None


def track_device_status(enable: bool) -> None:
    """Debugging aid.  While enabled, every chunked forward / backward copies its
    device status word (4 bytes, one extra copy on the launch stream) into a tensor
    of its own that ``last_device_status`` / ``last_backward_status`` read.  Off by
    default: production callers learn of a device-side failure through the NaN the
    library writes over the head of the outputs, without any read-back."""
    global _TRACK_STATUS, _LAST_STATUS, _LAST_BWD_STATUS
    _TRACK_STATUS = bool(enable)
    _LAST_STATUS = _LAST_BWD_STATUS = None


def last_device_status() -> int:
    """Status word the most recent chunked forward's kernels left on the device
    (0 = ok, 1 = a bounded wait inside a kernel gave up and its CTA skipped its
    stores); 0 when tracking is off.  Synchronises; meant for tests and debugging."""
    if _LAST_STATUS is None:
        return 0
    if isinstance(_LAST_STATUS, tuple):   # (device address inside the library's static array, device)
        address, device = _LAST_STATUS
        with torch.cuda.device(device):
            return int(torch.as_tensor(_DeviceWord(address), device=device).item())
    return int(_LAST_STATUS.view(torch.int32).item())


def last_backward_status() -> int:
    """The same for the most recent chunked backward (its results are void if a
    bounded wait gave up)."""
    if _LAST_BWD_STATUS is None:
        return 0
    return int(_LAST_BWD_STATUS.view(torch.int32).item())


def _status_copy(ws: Tensor, offset: int) -> Optional[Tensor]:
    """A 4-byte copy of the status word (so that the workspace itself can go back
    to the allocator when the call returns)."""
    if not _TRACK_STATUS:
        return None
    return ws[offset:offset + 4].clone()


def _count(lib) -> None:
    global LAUNCHES
    LAUNCHES += int(lib.pkda_last_launch_count())


_DTYPES = {torch.bfloat16: _lib.PKDA_BF16, torch.float32: _lib.PKDA_F32}


def _require_cuda(*tensors: Optional[Tensor]) -> None:
    """Every given tensor must live on one and the same CUDA device (the kernels
    run on a single device and dereference every pointer there)."""
    device = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("PKDA CUDA operators need CUDA tensors; there is no CPU path")
        if device is None:
            device = t.device
        elif t.device != device:
            raise RuntimeError(
                f"PKDA operator arguments live on different devices ({device} and {t.device})")


def _on_tensor_device(fn):
    """Runs a launcher with its first tensor's device current, so that the library
    launches (and encodes its tensor maps) on the device that owns the data and
    torch's current stream of THAT device is the one used, whatever device the
    caller had current (the reference's kernels guard the same way)."""
    @functools.wraps(fn)
    def wrapper(first, *args, **kwargs):
        if not getattr(first, "is_cuda", False):
            raise RuntimeError("PKDA CUDA operators need CUDA tensors; there is no CPU path")
        with torch.cuda.device(first.device):
            return fn(first, *args, **kwargs)
    return wrapper


def _problem(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale, scale, x, eps,
             initial_state, initial_A_state, cu_seqlens, keep) -> _lib.Problem:
    """Builds the shared problem struct; ``keep`` collects every tensor whose
    storage must outlive the launch call (contiguous copies, casts)."""
    B, T, H, D = q.shape
    if q.dtype not in _DTYPES:
        raise RuntimeError(f"PKDA supports bf16 and fp32 activations, not {q.dtype}")
    act = q.dtype
    _require_cuda(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale,
                  initial_state, initial_A_state)

    def act_c(t, shape):
        if tuple(t.shape) != tuple(shape):
            raise RuntimeError(f"PKDA input has shape {tuple(t.shape)}, expected {tuple(shape)}")
        t = t.to(act).contiguous()
        keep.append(t)
        return t

    def f32_c(t, numel):
        if t.numel() != numel:
            raise RuntimeError(f"PKDA parameter has {t.numel()} elements, expected {numel}")
        t = t.detach().to(torch.float32).contiguous()
        keep.append(t)
        return t

    q_, k_, v_, g_ = (act_c(t, (B, T, H, D)) for t in (q, k, v, g))
    g_atk_ = f32_c(g_atk, B * T * H)
    beta_atk_, beta_ = act_c(beta_atk, (B, T, H)), act_c(beta, (B, T, H))
    p = _lib.Problem()
    if cu_seqlens is not None:
        if B != 1:
            raise RuntimeError("packed input (cu_seqlens) needs batch size 1")
        cu = cu_seqlens.to(device=q.device, dtype=torch.int32).contiguous()
        keep.append(cu)
        p.n_seqs = cu.numel() - 1
        p.seq_len = 0
        p.cu_seqlens = cu.data_ptr()
    else:
        p.n_seqs = B
        p.seq_len = T
        p.cu_seqlens = None
    N = p.n_seqs
    p.total_tokens = B * T
    p.heads, p.head_dim = H, D
    p.dtype = _DTYPES[act]
    p.scale = float(D ** -0.5 if scale is None else scale)
    p.squash_x, p.squash_eps = float(x), float(eps)
    p.q, p.k, p.v, p.g = q_.data_ptr(), k_.data_ptr(), v_.data_ptr(), g_.data_ptr()
    p.g_atk, p.beta_atk, p.beta = g_atk_.data_ptr(), beta_atk_.data_ptr(), beta_.data_ptr()
    p.A_log = f32_c(A_log, H).data_ptr()
    p.dt_bias = f32_c(dt_bias, H * D).data_ptr()
    p.log_atk_scale = f32_c(log_atk_scale, H).data_ptr()
    if initial_state is not None:
        p.initial_state = f32_c(initial_state, N * H * D * D).data_ptr()
    if initial_A_state is not None:
        p.initial_A_state = f32_c(initial_A_state, N * H * D).data_ptr()
    return p


def n_chunks(B: int, T: int, cu_seqlens: Optional[Tensor]) -> int:
    """Length of the flat chunk axis (an upper bound for packed input, whose
    exact count would need a device read-back)."""
    if cu_seqlens is None:
        return B * (-(-T // CHUNK_SIZE))
    return (B * T) // CHUNK_SIZE + (cu_seqlens.numel() - 1)


@_on_tensor_device
def recurrent_forward(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale, scale,
                      x, eps, initial_state=None, initial_A_state=None, cu_seqlens=None,
                      output_final_state=True, inplace_state=False):
    """Token-by-token kernel.  Returns ``(o, S, A)`` (states ``None`` unless
    requested).  ``inplace_state`` writes the new states over the given fp32
    contiguous initial states and returns those same tensors."""
    _require_cuda(q, k, v, g, g_atk, beta_atk, beta)
    lib = _lib.load()
    keep: list = []
    p = _problem(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale, scale, x, eps,
                 initial_state, initial_A_state, cu_seqlens, keep)
    B, T, H, D = q.shape
    N = p.n_seqs
    args = _lib.RecurrentArgs()
    args.p = p
    o = torch.empty((B, T, H, v.shape[-1]), device=q.device, dtype=q.dtype)
    args.o = o.data_ptr()
    S = A = None
    if output_final_state:
        if inplace_state:
            ok = all(t is not None and t.dtype == torch.float32 and t.is_contiguous()
                     for t in (initial_state, initial_A_state))
            if not ok:
                raise RuntimeError("in-place decode needs contiguous fp32 initial states")
            S, A = initial_state, initial_A_state
        else:
            S = torch.empty((N, H, D, D), device=q.device, dtype=torch.float32)
            A = torch.empty((N, H, D), device=q.device, dtype=torch.float32)
        args.final_state, args.final_A_state = S.data_ptr(), A.data_ptr()
    _lib.check(lib.pkda_recurrent_fwd(C.byref(args), _lib.current_stream()), "pkda_recurrent_fwd")
    _count(lib)
    return o, S, A


def intermediate_meta(q: Tensor, v: Tensor, lean: bool, chunks_flat: Optional[int] = None):
    """Shapes and dtypes of the saved intermediates, in the reference's order
    (``delta_feedback_experiment/fla_ops.py:73-97``)."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    NT = -(-T // CHUNK_SIZE) if chunks_flat is None else chunks_flat
    act = q.dtype
    meta = [
        ((B, T, H, CHUNK_SIZE), act), ((B, T, H, CHUNK_SIZE), act), ((B, T, H, K), act),
        ((B, NT, H, K), torch.float32), ((B, NT, H, K), torch.float32),
        ((B, NT, H), torch.float32),
    ]
    if not lean:
        meta += [((B, T, H, K), act), ((B, T, H, K), act), ((B, T, H, V), act),
                 ((B, NT, H, K, V), act), ((B, T, H, K), act)]
    return tuple(meta)


@_on_tensor_device
def chunk_forward(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale, scale, x,
                  eps, initial_state=None, initial_A_state=None, cu_seqlens=None,
                  output_final_state=False):
    """Chunked forward (bf16, D = 128).  Returns ``(o, S_T, A_T, saved)`` where
    ``saved`` is the full list of eleven intermediates."""
    _require_cuda(q, k, v, g, g_atk, beta_atk, beta)
    lib = _lib.load()
    keep: list = []
    p = _problem(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale, scale, x, eps,
                 initial_state, initial_A_state, cu_seqlens, keep)
    B, T, H, D = q.shape
    N = p.n_seqs
    dev = q.device
    chunks = n_chunks(B, T, cu_seqlens) if cu_seqlens is not None else None
    saved = [torch.empty(shape, device=dev, dtype=dt)
             for shape, dt in intermediate_meta(q, v, False, chunks)]
    o = torch.empty((B, T, H, D), device=dev, dtype=q.dtype)
    args = _lib.ChunkFwdArgs()
    args.p = p
    args.o = o.data_ptr()
    S = A = None
    if output_final_state:
        S = torch.empty((N, H, D, D), device=dev, dtype=torch.float32)
        A = torch.empty((N, H, D), device=dev, dtype=torch.float32)
        args.final_state, args.final_A_state = S.data_ptr(), A.data_ptr()
    (args.Aqk, args.Akk, args.k_precond, args.ac_atk, args.a_atk, args.sa_atk, args.w, args.kg,
     args.v_new, args.h, args.qg) = [t.data_ptr() for t in saved]
    nbytes = lib.pkda_chunk_fwd_workspace_bytes(C.byref(p))
    ws = torch.empty((max(nbytes, 16),), device=dev, dtype=torch.uint8)
    args.workspace, args.workspace_bytes = ws.data_ptr(), nbytes
    _lib.check(lib.pkda_chunk_fwd(C.byref(args), _lib.current_stream()), "pkda_chunk_fwd")
    _count(lib)
    global _LAST_STATUS
    _LAST_STATUS = _status_copy(ws, int(lib.pkda_chunk_fwd_status_offset(C.byref(p))))
    return o, S, A, saved


@_on_tensor_device
def chunk_backward(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale, scale, x,
                   eps, saved: Sequence[Tensor], do, initial_state=None, initial_A_state=None,
                   cu_seqlens=None, d_final_state=None, lean=False, want_state_grads=False):
    """Chunked backward.  ``saved`` holds the six always-kept intermediates and,
    unless ``lean``, the five retained ones.  Returns the ten gradients (plus
    ``dS0, dA0`` when ``want_state_grads``)."""
    _require_cuda(q, k, v, g, g_atk, beta_atk, beta, do, d_final_state)
    lib = _lib.load()
    keep: list = []
    p = _problem(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale, scale, x, eps,
                 initial_state, initial_A_state, cu_seqlens, keep)
    B, T, H, D = q.shape
    N = p.n_seqs
    dev, act = q.device, q.dtype
    chunks = n_chunks(B, T, cu_seqlens) if cu_seqlens is not None else None
    meta = intermediate_meta(q, v, False, chunks)
    saved = list(saved)
    if lean:
        saved = saved[:6] + [torch.empty(shape, device=dev, dtype=dt) for shape, dt in meta[6:]]
    if len(saved) != 11:
        raise RuntimeError(f"PKDA backward got {len(saved)} intermediates, not 11")
    args = _lib.ChunkBwdArgs()
    args.p = p
    do_c = do.to(act).contiguous()
    args.d_o = do_c.data_ptr()
    if d_final_state is not None:
        dST = d_final_state.to(torch.float32).contiguous()
        keep.append(dST)
        args.d_final_state = dST.data_ptr()
    args.recompute = 1 if lean else 0
    (args.Aqk, args.Akk, args.k_precond, args.ac_atk, args.a_atk, args.sa_atk, args.w, args.kg,
     args.v_new, args.h, args.qg) = [t.data_ptr() for t in saved]
    dq, dk, dv, dg = (torch.empty((B, T, H, D), device=dev, dtype=act) for _ in range(4))
    dg_atk = torch.empty((B, T, H), device=dev, dtype=torch.float32)
    dbeta_atk = torch.empty((B, T, H), device=dev, dtype=act)
    dbeta = torch.empty((B, T, H), device=dev, dtype=act)
    dA_log = torch.empty((H,), device=dev, dtype=torch.float32)
    ddt_bias = torch.empty((H * D,), device=dev, dtype=torch.float32)
    dcentre = torch.empty((H,), device=dev, dtype=torch.float32)
    args.dq, args.dk, args.dv, args.dg = (t.data_ptr() for t in (dq, dk, dv, dg))
    args.dg_atk, args.dbeta_atk, args.dbeta = dg_atk.data_ptr(), dbeta_atk.data_ptr(), dbeta.data_ptr()
    args.dA_log, args.ddt_bias, args.dlog_atk_scale = (
        dA_log.data_ptr(), ddt_bias.data_ptr(), dcentre.data_ptr())
    dS0 = dA0 = None
    if want_state_grads:
        dS0 = torch.empty((N, H, D, D), device=dev, dtype=torch.float32)
        dA0 = torch.empty((N, H, D), device=dev, dtype=torch.float32)
        args.d_initial_state, args.d_initial_A_state = dS0.data_ptr(), dA0.data_ptr()
    nbytes = lib.pkda_chunk_bwd_workspace_bytes(C.byref(p))
    ws = torch.empty((max(nbytes, 16),), device=dev, dtype=torch.uint8)
    args.workspace, args.workspace_bytes = ws.data_ptr(), nbytes
    _lib.check(lib.pkda_chunk_bwd(C.byref(args), _lib.current_stream()), "pkda_chunk_bwd")
    _count(lib)
    global _LAST_BWD_STATUS
    _LAST_BWD_STATUS = _status_copy(ws, int(lib.pkda_chunk_bwd_status_offset(C.byref(p))))
    grads = [dq, dk, dv, dg, dg_atk, dbeta_atk, dbeta, dA_log, ddt_bias, dcentre]
    return grads, dS0, dA0


@_on_tensor_device
def recurrent_backward(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale, scale, x,
                       eps, do, initial_state=None, initial_A_state=None, cu_seqlens=None,
                       d_final_state=None, want_state_grads=False):
    """Exact fp32 backward of the recurrence (any supported head width, bf16 or
    fp32 activations); needs no saved intermediates.  Returns the ten gradients
    (plus ``dS0, dA0`` when ``want_state_grads``)."""
    _require_cuda(q, k, v, g, g_atk, beta_atk, beta, do, d_final_state)
    lib = _lib.load()
    keep: list = []
    p = _problem(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale, scale, x, eps,
                 initial_state, initial_A_state, cu_seqlens, keep)
    B, T, H, D = q.shape
    N = p.n_seqs
    dev, act = q.device, q.dtype
    args = _lib.RecurrentBwdArgs()
    args.p = p
    do_c = do.to(act).contiguous()
    args.d_o = do_c.data_ptr()
    if d_final_state is not None:
        dST = d_final_state.to(torch.float32).contiguous()
        keep.append(dST)
        args.d_final_state = dST.data_ptr()
    dq, dk, dv, dg = (torch.empty((B, T, H, D), device=dev, dtype=act) for _ in range(4))
    dg_atk = torch.empty((B, T, H), device=dev, dtype=torch.float32)
    dbeta_atk = torch.empty((B, T, H), device=dev, dtype=act)
    dbeta = torch.empty((B, T, H), device=dev, dtype=act)
    dA_log = torch.empty((H,), device=dev, dtype=torch.float32)
    ddt_bias = torch.empty((H * D,), device=dev, dtype=torch.float32)
    dcentre = torch.empty((H,), device=dev, dtype=torch.float32)
    args.dq, args.dk, args.dv, args.dg = (t.data_ptr() for t in (dq, dk, dv, dg))
    args.dg_atk, args.dbeta_atk, args.dbeta = dg_atk.data_ptr(), dbeta_atk.data_ptr(), dbeta.data_ptr()
    args.dA_log, args.ddt_bias, args.dlog_atk_scale = (
        dA_log.data_ptr(), ddt_bias.data_ptr(), dcentre.data_ptr())
    dS0 = dA0 = None
    if want_state_grads:
        dS0 = torch.empty((N, H, D, D), device=dev, dtype=torch.float32)
        dA0 = torch.empty((N, H, D), device=dev, dtype=torch.float32)
        args.d_initial_state, args.d_initial_A_state = dS0.data_ptr(), dA0.data_ptr()
    nbytes = lib.pkda_recurrent_bwd_workspace_bytes(C.byref(p))
    ws = torch.empty((max(nbytes, 16),), device=dev, dtype=torch.uint8)
    args.workspace, args.workspace_bytes = ws.data_ptr(), nbytes
    _lib.check(lib.pkda_recurrent_bwd(C.byref(args), _lib.current_stream()), "pkda_recurrent_bwd")
    _count(lib)
    grads = [dq, dk, dv, dg, dg_atk, dbeta_atk, dbeta, dA_log, ddt_bias, dcentre]
    return grads, dS0, dA0


def static_scratch_bytes() -> int:
    return int(_lib.load().pkda_static_scratch_bytes())


@_on_tensor_device
def chunk_forward_static(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale, scale,
                         x, eps, o, saved, initial_state=None, initial_A_state=None,
                         final_state=None, final_A_state=None):
    """Chunked forward through ``pkda_chunk_fwd_static``: for hosts that must not
    allocate device memory while the operator runs.  The caller supplies every
    buffer -- contiguous bf16 inputs, the output ``o`` and the eleven
    intermediates ``saved`` (shapes of ``intermediate_meta``), optionally the
    fp32 final-state buffers -- and the library takes its scratch from the fixed
    array built into it, so nothing is allocated here or below.  Raises
    ``RuntimeError`` when the problem needs more scratch than that array has
    (``static_scratch_bytes()``).  Calls share the array: do not let two of them
    overlap on the GPU, and make the first call on a device outside stream
    capture."""
    _require_cuda(q, k, v, g, g_atk, beta_atk, beta, o)
    lib = _lib.load()
    tensors = (q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale)
    if not all(t.is_contiguous() for t in tensors) or g_atk.dtype != torch.float32:
        raise RuntimeError("the no-allocation entry point needs contiguous inputs (fp32 g_atk)")
    keep: list = []
    p = _problem(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, log_atk_scale, scale, x, eps,
                 initial_state, initial_A_state, None, keep)
    if len(saved) != 11:
        raise RuntimeError("eleven intermediate buffers are required")
    args = _lib.ChunkFwdArgs()
    args.p = p
    args.o = o.data_ptr()
    if final_state is not None:
        args.final_state, args.final_A_state = final_state.data_ptr(), final_A_state.data_ptr()
    (args.Aqk, args.Akk, args.k_precond, args.ac_atk, args.a_atk, args.sa_atk, args.w, args.kg,
     args.v_new, args.h, args.qg) = [t.data_ptr() for t in saved]
    _lib.check(lib.pkda_chunk_fwd_static(C.byref(args), _lib.current_stream()),
               "pkda_chunk_fwd_static")
    _count(lib)
    if _TRACK_STATUS:
        global _LAST_STATUS
        _LAST_STATUS = _static_status_view(lib, p)
    return o


class _DeviceWord:
    """Presents a raw device address as a one-element int32 array to
    ``torch.as_tensor``."""

    def __init__(self, address: int):
        self.__cuda_array_interface__ = {
            "shape": (1,), "typestr": "<i4", "data": (int(address), False), "version": 2}


def _static_status_view(lib, p):
    """Where the static-scratch forward keeps its status word: the device address
    inside the library's own array and the device (nothing is allocated or copied
    here; ``last_device_status`` reads the word, before the next such call
    overwrites it)."""
    addr = C.c_void_p()
    _lib.check(lib.pkda_static_status_ptr(C.byref(p), C.byref(addr)), "pkda_static_status_ptr")
    return int(addr.value), torch.device("cuda", torch.cuda.current_device())
