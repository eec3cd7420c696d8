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


def test_variant_switch_and_status_offsets(lib):
    """The testing switch accepts exactly the stages that have two implementations, and
    the status word sits inside the workspace the size query reports."""
    for name in (b"intra_fwd", b"scan_fwd", b"out_fwd", b"scan_bwd", b"intra_bwd"):
        assert lib.pkda_set_variant(name, 1) == 0
        assert lib.pkda_set_variant(name, 0) == 0
    assert lib.pkda_set_variant(b"atk_local", 1) == 2
    assert lib.pkda_set_variant(None, 1) == 1
    p = _lib.Problem()
    p.n_seqs, p.seq_len, p.total_tokens, p.heads, p.head_dim = 2, 130, 260, 3, 128
    for size, off in ((lib.pkda_chunk_fwd_workspace_bytes, lib.pkda_chunk_fwd_status_offset),
                      (lib.pkda_chunk_bwd_workspace_bytes, lib.pkda_chunk_bwd_status_offset)):
        total, where = size(C.byref(p)), off(C.byref(p))
        assert 0 < where and where + 4 <= total and where % 256 == 0


class _FakeTensor:
    """Stands in for a CUDA tensor where there is no GPU: only the attributes the
    device checks read."""

    def __init__(self, device):
        import torch
        self.is_cuda = device is not None
        self.device = torch.device("cuda", device) if device is not None else torch.device("cpu")


def test_arguments_on_different_devices_are_rejected_before_any_launch():
    from delta_feedback_experiment_b200 import ops
    ops._require_cuda(_FakeTensor(1), None, _FakeTensor(1))
    with pytest.raises(RuntimeError, match="different devices"):
        ops._require_cuda(_FakeTensor(0), _FakeTensor(1))
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops._require_cuda(_FakeTensor(0), _FakeTensor(None))
    calls = []
    guarded = ops._on_tensor_device(lambda first: calls.append(first))
    with pytest.raises(RuntimeError, match="no CPU path"):
        guarded(_FakeTensor(None))
    assert not calls


def test_intermediate_contract_check_names_the_offender():
    """`fla_ops._check_intermediates` compares what a forward returns with what the fake
    implementation promises (reference: fla_ops.py:100-128): count, shape, dtype, contiguity."""
    import pytest
    import torch
    from delta_feedback_experiment_b200 import fla_ops

    q = torch.empty(2, 130, 3, 128, dtype=torch.bfloat16)
    v = torch.empty(2, 130, 3, 128, dtype=torch.bfloat16)
    for lean in (True, False):
        good = [torch.empty(s, dtype=d) for s, d in fla_ops._intermediate_meta(q, v, lean)]
        fla_ops._check_intermediates(good, q, v, lean)                       # passes
        with pytest.raises(RuntimeError, match="intermediates where"):
            fla_ops._check_intermediates(good[:-1], q, v, lean)
        bad = list(good)
        bad[2] = bad[2].float()                                               # wrong dtype
        with pytest.raises(RuntimeError, match="k_precond"):
            fla_ops._check_intermediates(bad, q, v, lean)
        bad = list(good)
        bad[0] = good[0].transpose(1, 2).contiguous().transpose(1, 2)         # right shape, not contiguous
        with pytest.raises(RuntimeError, match="Aqk"):
            fla_ops._check_intermediates(bad, q, v, lean)
    assert len(fla_ops._intermediate_meta(q, v, True)) == len(fla_ops.PKDA_INTERMEDIATES)
    assert fla_ops._intermediate_meta(q, v, False)[9][0] == (2, 3, 3, 128, 128)   # h: three chunks of 64
