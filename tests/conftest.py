"""Shared test configuration: the ``gpu`` marker, import paths and helpers."""

import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True, scope="session")
def _track_device_status():
    """GPU tests read the kernels' device status word after their calls."""
    if torch.cuda.is_available():
        from delta_feedback_experiment_b200 import ops
        ops.track_device_status(True)
    yield


def load_golden(name: str) -> dict:
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as z:
        return {k: torch.from_numpy(z[k].copy()) for k in z.files}


def rel_rms(actual: torch.Tensor, expected: torch.Tensor) -> float:
    a, e = actual.detach().double().cpu(), expected.detach().double().cpu()
    return float((a - e).square().mean().sqrt() / (e.square().mean().sqrt() + 1e-30))


def assert_close(actual, expected, rtol, name="", outlier_frac=None):
    """``|a-e| <= rtol * (|e| + rms)``: the stated relative tolerance, with an RMS
    floor for entries near zero.  ``rms`` is the larger of the whole tensor's RMS
    and the RMS of the entry's own last-dimension vector (token rows differ in
    scale by an order of magnitude, e.g. the last tokens carry the final-state
    cotangent, and rounding error follows the row's scale).  For the bf16 tolerance
    (rtol >= 1e-2) a fraction of at most 1e-4 of the entries may sit in the
    rounding tail between 1x and 2x that bound; nothing may exceed 2x."""
    a, e = actual.detach().double().cpu(), expected.detach().double().cpu()
    assert a.shape == e.shape, f"{name}: shape {tuple(a.shape)} vs {tuple(e.shape)}"
    assert torch.isfinite(a).all(), f"{name}: non-finite values"
    if outlier_frac is None:
        outlier_frac = 1e-4 if rtol >= 1e-2 else 0.0
    rms = e.square().mean().sqrt()
    if e.ndim >= 2 and e.shape[-1] > 1:
        rms = torch.maximum(rms, e.square().mean(-1, keepdim=True).sqrt())
    bound = rtol * (e.abs() + rms) + 1e-30
    err = (a - e).abs()
    bad = err > bound
    worst = float((err / bound).max()) if a.numel() else 0.0
    if bad.sum() > outlier_frac * a.numel() or worst > 2.0:
        raise AssertionError(
            f"{name}: {int(bad.sum())}/{a.numel()} entries beyond rtol={rtol}; "
            f"worst {worst:.3f}x the bound; rel-rms {rel_rms(a, e):.3e}")
