"""CPU checks of the C-ABI boundary: the library loads, exports every symbol the
header declares, its struct layouts match the ctypes mirror, and argument
validation answers with status codes (no kernel is launched here)."""

import ctypes as C
import os
import re

import pytest

from conftest import ROOT
from delta_feedback_experiment_b200 import _lib, build


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "pkda_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pkda_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = declared_functions()
    assert set(names) == set(_lib.EXPORTS)
    for name in names:
        assert hasattr(lib, name), name


def test_struct_layouts(lib):
    assert lib.pkda_sizeof_problem() == C.sizeof(_lib.Problem)
    assert lib.pkda_sizeof_recurrent_args() == C.sizeof(_lib.RecurrentArgs)
    assert lib.pkda_sizeof_chunk_fwd_args() == C.sizeof(_lib.ChunkFwdArgs)
    assert lib.pkda_sizeof_chunk_bwd_args() == C.sizeof(_lib.ChunkBwdArgs)
    assert lib.pkda_abi_version() == _lib.ABI_VERSION


def test_status_codes_without_launch(lib):
    args = _lib.RecurrentArgs()
    args.p.n_seqs, args.p.seq_len, args.p.total_tokens = 2, 4, 8
    args.p.heads, args.p.head_dim = 2, 128
    assert lib.pkda_recurrent_fwd(C.byref(args), None) == 1  # PKDA_ERR_NULL
    args.p.total_tokens = 7
    assert lib.pkda_recurrent_fwd(C.byref(args), None) == 2  # PKDA_ERR_SHAPE
    # empty problems are accepted and launch nothing
    args.p.n_seqs, args.p.seq_len, args.p.total_tokens = 0, 4, 0
    assert lib.pkda_recurrent_fwd(C.byref(args), None) == 0
    assert lib.pkda_last_launch_count() == 0
    cf = _lib.ChunkFwdArgs()
    cf.p.n_seqs, cf.p.seq_len, cf.p.total_tokens, cf.p.heads, cf.p.head_dim = 1, 64, 64, 1, 64
    for f in ("q", "k", "v", "g", "g_atk", "beta_atk", "beta", "A_log", "dt_bias", "log_atk_scale"):
        setattr(cf.p, f, 256)
    assert lib.pkda_chunk_fwd(C.byref(cf), None) == 2  # head_dim 64 unsupported by the chunked path
    assert b"geometry" in lib.pkda_status_string(2)
    assert _lib.load().pkda_chunk_fwd_workspace_bytes(C.byref(cf.p)) > 0


def test_operators_refuse_cpu_tensors():
    import torch
    from delta_feedback_experiment_b200 import fused_recurrent_precond_kda
    t = torch.zeros(1, 1, 1, 8)
    s = torch.zeros(1, 1, 1)
    with pytest.raises(RuntimeError, match="no CPU path"):
        fused_recurrent_precond_kda(t, t, t, t, s, s, s, torch.zeros(1), torch.zeros(8),
                                    log_atk_scale=torch.zeros(1))
