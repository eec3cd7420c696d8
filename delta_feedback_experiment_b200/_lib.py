"""ctypes binding of ``libpkda_b200.so`` (declared in ``include/pkda_b200.h``).

The library is the product; this module only loads it, mirrors its argument
structs and turns status codes into ``RuntimeError``.  There is no fallback: if
the shared library is missing or does not load, every operator raises.
"""

from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libpkda_b200.so")

PKDA_BF16, PKDA_F32 = 0, 1
ABI_VERSION = 1
CHUNK = 64


class Problem(C.Structure):
    _fields_ = [
        ("n_seqs", C.c_int32), ("seq_len", C.c_int32), ("total_tokens", C.c_int32),
        ("heads", C.c_int32), ("head_dim", C.c_int32), ("dtype", C.c_int32),
        ("scale", C.c_float), ("squash_x", C.c_float), ("squash_eps", C.c_float),
        ("reserved0", C.c_int32),
        ("cu_seqlens", C.c_void_p),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("g", C.c_void_p),
        ("g_atk", C.c_void_p), ("beta_atk", C.c_void_p), ("beta", C.c_void_p),
        ("A_log", C.c_void_p), ("dt_bias", C.c_void_p), ("log_atk_scale", C.c_void_p),
        ("initial_state", C.c_void_p), ("initial_A_state", C.c_void_p),
    ]


class RecurrentArgs(C.Structure):
    _fields_ = [("p", Problem), ("o", C.c_void_p), ("final_state", C.c_void_p),
                ("final_A_state", C.c_void_p)]


class ChunkFwdArgs(C.Structure):
    _fields_ = [
        ("p", Problem), ("o", C.c_void_p), ("final_state", C.c_void_p),
        ("final_A_state", C.c_void_p),
        ("Aqk", C.c_void_p), ("Akk", C.c_void_p), ("k_precond", C.c_void_p),
        ("ac_atk", C.c_void_p), ("a_atk", C.c_void_p), ("sa_atk", C.c_void_p),
        ("w", C.c_void_p), ("kg", C.c_void_p), ("v_new", C.c_void_p), ("h", C.c_void_p),
        ("qg", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class ChunkBwdArgs(C.Structure):
    _fields_ = [
        ("p", Problem), ("d_o", C.c_void_p), ("d_final_state", C.c_void_p),
        ("recompute", C.c_int32), ("reserved1", C.c_int32),
        ("Aqk", C.c_void_p), ("Akk", C.c_void_p), ("k_precond", C.c_void_p),
        ("ac_atk", C.c_void_p), ("a_atk", C.c_void_p), ("sa_atk", C.c_void_p),
        ("w", C.c_void_p), ("kg", C.c_void_p), ("v_new", C.c_void_p), ("h", C.c_void_p),
        ("qg", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p), ("dg", C.c_void_p),
        ("dg_atk", C.c_void_p), ("dbeta_atk", C.c_void_p), ("dbeta", C.c_void_p),
        ("dA_log", C.c_void_p), ("ddt_bias", C.c_void_p), ("dlog_atk_scale", C.c_void_p),
        ("d_initial_state", C.c_void_p), ("d_initial_A_state", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class RecurrentBwdArgs(C.Structure):
    _fields_ = [
        ("p", Problem), ("d_o", C.c_void_p), ("d_final_state", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p), ("dg", C.c_void_p),
        ("dg_atk", C.c_void_p), ("dbeta_atk", C.c_void_p), ("dbeta", C.c_void_p),
        ("dA_log", C.c_void_p), ("ddt_bias", C.c_void_p), ("dlog_atk_scale", C.c_void_p),
        ("d_initial_state", C.c_void_p), ("d_initial_A_state", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class QkvConvArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("seq_len", C.c_int32), ("channels", C.c_int32), ("taps", C.c_int32),
        ("head_dim", C.c_int32), ("norm_channels", C.c_int32), ("dtype", C.c_int32), ("eps", C.c_float),
        ("x", C.c_void_p), ("weight", C.c_void_p),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("dx", C.c_void_p), ("dweight", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class NormGateArgs(C.Structure):
    _fields_ = [
        ("rows", C.c_longlong), ("dim", C.c_int32), ("dtype", C.c_int32), ("eps", C.c_float),
        ("x", C.c_void_p), ("gate", C.c_void_p), ("weight", C.c_void_p),
        ("y", C.c_void_p), ("rstd", C.c_void_p), ("dy", C.c_void_p),
        ("dx", C.c_void_p), ("dgate", C.c_void_p), ("dweight", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class DecodeStepArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32), ("taps", C.c_int32),
        ("dtype", C.c_int32),
        ("scale", C.c_float), ("squash_x", C.c_float), ("squash_eps", C.c_float), ("qk_eps", C.c_float),
        ("norm_eps", C.c_float),
        ("qkv", C.c_void_p), ("conv_q", C.c_void_p), ("conv_k", C.c_void_p), ("conv_v", C.c_void_p),
        ("conv_weight", C.c_void_p), ("g", C.c_void_p), ("g_atk", C.c_void_p),
        ("beta_atk", C.c_void_p), ("beta", C.c_void_p),
        ("A_log", C.c_void_p), ("dt_bias", C.c_void_p), ("log_atk_scale", C.c_void_p),
        ("state", C.c_void_p), ("a_state", C.c_void_p), ("gate", C.c_void_p),
        ("norm_weight", C.c_void_p), ("out", C.c_void_p),
    ]


class ControlsArgs(C.Structure):
    _fields_ = [
        ("rows", C.c_longlong), ("heads", C.c_int32), ("hidden", C.c_int32), ("dtype", C.c_int32),
        ("packed", C.c_void_p), ("A_log_precond", C.c_void_p), ("dt_bias_precond", C.c_void_p),
        ("beta", C.c_void_p), ("g_atk", C.c_void_p), ("beta_atk", C.c_void_p),
        ("d_decay_hidden", C.c_void_p), ("d_beta", C.c_void_p), ("d_g_atk", C.c_void_p),
        ("d_beta_atk", C.c_void_p), ("d_gate_hidden", C.c_void_p), ("d_packed", C.c_void_p),
        ("dA_log_precond", C.c_void_p), ("ddt_bias_precond", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class PackControlArgs(C.Structure):
    _fields_ = [
        ("rows", C.c_longlong), ("sizes", C.c_int32 * 5), ("dtype", C.c_int32),
        ("grads", C.c_void_p * 5), ("out", C.c_void_p),
    ]


EXPORTS = (
    "pkda_recurrent_fwd", "pkda_recurrent_bwd", "pkda_recurrent_bwd_workspace_bytes", "pkda_chunk_fwd_workspace_bytes", "pkda_chunk_fwd",
    "pkda_chunk_bwd_workspace_bytes", "pkda_chunk_bwd", "pkda_abi_version",
    "pkda_status_string", "pkda_sizeof_problem", "pkda_sizeof_recurrent_args",
    "pkda_sizeof_chunk_fwd_args", "pkda_sizeof_chunk_bwd_args", "pkda_last_launch_count",
    "pkda_stage_count", "pkda_stage_name", "pkda_stage_timing", "pkda_stage_timing_read",
    "pkda_static_scratch_bytes", "pkda_chunk_fwd_static", "pkda_set_direct_block_cap",
    "pkda_chunk_fwd_status_offset", "pkda_chunk_bwd_status_offset", "pkda_static_status_ptr",
    "pkda_set_variant",
    "pkda_qkv_conv_fwd", "pkda_qkv_conv_bwd_workspace_bytes", "pkda_qkv_conv_bwd",
    "pkda_norm_gate_fwd", "pkda_norm_gate_bwd_workspace_bytes", "pkda_norm_gate_bwd",
    "pkda_sizeof_qkv_conv_args", "pkda_sizeof_norm_gate_args",
    "pkda_decode_step", "pkda_sizeof_decode_step_args",
    "pkda_controls_fwd", "pkda_controls_bwd_workspace_bytes", "pkda_controls_bwd",
    "pkda_pack_control_gradients", "pkda_sizeof_controls_args", "pkda_sizeof_pack_control_args",
)

_lib: Optional[C.CDLL] = None
_load_error: Optional[str] = None


def _configure(lib: C.CDLL) -> None:
    lib.pkda_recurrent_fwd.argtypes = [C.POINTER(RecurrentArgs), C.c_void_p]
    lib.pkda_recurrent_fwd.restype = C.c_int
    lib.pkda_recurrent_bwd.argtypes = [C.POINTER(RecurrentBwdArgs), C.c_void_p]
    lib.pkda_recurrent_bwd.restype = C.c_int
    lib.pkda_recurrent_bwd_workspace_bytes.argtypes = [C.POINTER(Problem)]
    lib.pkda_recurrent_bwd_workspace_bytes.restype = C.c_size_t
    lib.pkda_chunk_fwd.argtypes = [C.POINTER(ChunkFwdArgs), C.c_void_p]
    lib.pkda_chunk_fwd.restype = C.c_int
    lib.pkda_chunk_fwd_static.argtypes = [C.POINTER(ChunkFwdArgs), C.c_void_p]
    lib.pkda_chunk_fwd_static.restype = C.c_int
    lib.pkda_static_scratch_bytes.restype = C.c_size_t
    lib.pkda_set_direct_block_cap.argtypes = [C.c_int]
    lib.pkda_set_direct_block_cap.restype = C.c_int
    lib.pkda_set_variant.argtypes = [C.c_char_p, C.c_int]
    lib.pkda_set_variant.restype = C.c_int
    lib.pkda_static_status_ptr.argtypes = [C.POINTER(Problem), C.POINTER(C.c_void_p)]
    lib.pkda_static_status_ptr.restype = C.c_int
    lib.pkda_chunk_bwd.argtypes = [C.POINTER(ChunkBwdArgs), C.c_void_p]
    lib.pkda_chunk_bwd.restype = C.c_int
    for name in ("pkda_chunk_fwd_workspace_bytes", "pkda_chunk_bwd_workspace_bytes",
                 "pkda_chunk_fwd_status_offset", "pkda_chunk_bwd_status_offset"):
        getattr(lib, name).argtypes = [C.POINTER(Problem)]
        getattr(lib, name).restype = C.c_size_t
    for name, struct in (("pkda_qkv_conv", QkvConvArgs), ("pkda_norm_gate", NormGateArgs)):
        for suffix in ("_fwd", "_bwd"):
            getattr(lib, name + suffix).argtypes = [C.POINTER(struct), C.c_void_p]
            getattr(lib, name + suffix).restype = C.c_int
        getattr(lib, name + "_bwd_workspace_bytes").argtypes = [C.POINTER(struct)]
        getattr(lib, name + "_bwd_workspace_bytes").restype = C.c_size_t
    lib.pkda_decode_step.argtypes = [C.POINTER(DecodeStepArgs), C.c_void_p]
    lib.pkda_decode_step.restype = C.c_int
    for name in ("pkda_controls_fwd", "pkda_controls_bwd"):
        getattr(lib, name).argtypes = [C.POINTER(ControlsArgs), C.c_void_p]
        getattr(lib, name).restype = C.c_int
    lib.pkda_controls_bwd_workspace_bytes.argtypes = [C.POINTER(ControlsArgs)]
    lib.pkda_controls_bwd_workspace_bytes.restype = C.c_size_t
    lib.pkda_pack_control_gradients.argtypes = [C.POINTER(PackControlArgs), C.c_void_p]
    lib.pkda_pack_control_gradients.restype = C.c_int
    lib.pkda_abi_version.restype = C.c_int
    lib.pkda_status_string.argtypes = [C.c_int]
    lib.pkda_status_string.restype = C.c_char_p
    for name in ("pkda_sizeof_problem", "pkda_sizeof_recurrent_args",
                 "pkda_sizeof_chunk_fwd_args", "pkda_sizeof_chunk_bwd_args",
                 "pkda_sizeof_qkv_conv_args", "pkda_sizeof_norm_gate_args",
                 "pkda_sizeof_decode_step_args", "pkda_sizeof_controls_args",
                 "pkda_sizeof_pack_control_args"):
        getattr(lib, name).restype = C.c_size_t
    lib.pkda_last_launch_count.restype = C.c_int
    lib.pkda_stage_count.restype = C.c_int
    lib.pkda_stage_name.argtypes = [C.c_int]
    lib.pkda_stage_name.restype = C.c_char_p
    lib.pkda_stage_timing.argtypes = [C.c_int]
    lib.pkda_stage_timing.restype = C.c_int
    lib.pkda_stage_timing_read.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_int), C.c_int]
    lib.pkda_stage_timing_read.restype = C.c_int


def load() -> C.CDLL:
    """Loads the shared library once; raises ``RuntimeError`` if that fails."""
    global _lib, _load_error
    if _lib is not None:
        return _lib
    if _load_error is not None:
        raise RuntimeError(_load_error)
    try:
        if not os.path.exists(LIB_PATH):
            raise OSError(f"{LIB_PATH} has not been built "
                          "(python -m delta_feedback_experiment_b200.build)")
        lib = C.CDLL(LIB_PATH)
        _configure(lib)
        if lib.pkda_abi_version() != ABI_VERSION:
            raise OSError("libpkda_b200.so ABI version mismatch")
        sizes = ((lib.pkda_sizeof_problem(), Problem),
                 (lib.pkda_sizeof_recurrent_args(), RecurrentArgs),
                 (lib.pkda_sizeof_chunk_fwd_args(), ChunkFwdArgs),
                 (lib.pkda_sizeof_chunk_bwd_args(), ChunkBwdArgs),
                 (lib.pkda_sizeof_qkv_conv_args(), QkvConvArgs),
                 (lib.pkda_sizeof_norm_gate_args(), NormGateArgs),
                 (lib.pkda_sizeof_decode_step_args(), DecodeStepArgs),
                 (lib.pkda_sizeof_controls_args(), ControlsArgs),
                 (lib.pkda_sizeof_pack_control_args(), PackControlArgs))
        for size, struct in sizes:
            if size != C.sizeof(struct):
                raise OSError(f"struct layout mismatch for {struct.__name__}")
    except OSError as exc:
        _load_error = f"PKDA CUDA library unavailable: {exc}"
        raise RuntimeError(_load_error) from exc
    _lib = lib
    return lib


def available() -> bool:
    try:
        load()
        return True
    except RuntimeError:
        return False


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().pkda_status_string(status).decode()
        raise RuntimeError(f"{what} failed: {msg} (status {status})")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def current_stream(device=None) -> int:
    """Raw handle of torch's current stream on ``device`` (default: the current device)."""
    return torch.cuda.current_stream(device).cuda_stream


def last_launch_count() -> int:
    return int(load().pkda_last_launch_count())


def stage_timing(enable: bool) -> None:
    check(load().pkda_stage_timing(1 if enable else 0), "pkda_stage_timing")


def stage_timing_read() -> dict:
    """``{stage name: (total ms, launches)}`` since the last read."""
    lib = load()
    n = lib.pkda_stage_count()
    ms = (C.c_float * n)()
    cnt = (C.c_int * n)()
    check(lib.pkda_stage_timing_read(ms, cnt, n), "pkda_stage_timing_read")
    return {lib.pkda_stage_name(i).decode(): (float(ms[i]), int(cnt[i])) for i in range(n) if cnt[i]}


def set_direct_block_cap(cap: int) -> None:
    """Testing aid: caps the kernels' direct block size (64 = data-driven default)."""
    check(load().pkda_set_direct_block_cap(int(cap)), "pkda_set_direct_block_cap")


def set_variant(stage: str, legacy) -> None:
    """Testing aid: pins the older mma.sync kernel of a stage (``"intra_fwd"``,
    ``"scan_fwd"``, ``"out_fwd"``, ``"scan_bwd"``, ``"intra_bwd"``) or restores the default.
    ``set_variant("out_fwd", 2)`` runs the stand-alone tcgen05 output kernel instead of
    letting the state scan produce the output."""
    check(load().pkda_set_variant(stage.encode(), int(legacy)), "pkda_set_variant")
