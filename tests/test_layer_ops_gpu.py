"""GPU parity of the fused Q|K|V convolution and the RMS-norm gate, through the
C ABI, against the reference-made golden vectors (fp32) and the CPU oracle
(bf16, larger and ragged shapes)."""

import pytest
import torch

from conftest import assert_close, load_golden, rel_rms
from test_layer_oracle import CONV_CASES, GATE_CASES, conv_inputs

pytestmark = pytest.mark.gpu

FP32_RTOL = 1e-4   # fp32 kernels against the fp32 reference
BF16_RTOL = 2e-2   # bf16 kernels against the fp32 oracle on the same bf16-rounded inputs


def _ops():
    from delta_feedback_experiment_b200 import layer_ops
    return layer_ops


def _oracle():
    from oracle import pkda_layer_oracle
    return pkda_layer_oracle


# ------------------------------------------------------------------ convolution
@pytest.mark.parametrize("name", CONV_CASES)
def test_conv_fp32_matches_reference_golden(name):
    g = load_golden(name)
    rows, skip = conv_inputs(g)
    hd, nc, eps = int(g["head_dim"]), int(g["norm_channels"]), float(g["eps"])
    x, w = rows.cuda(), g["weight"].cuda()
    q, k, v = _ops().qkv_conv_forward(x, w, hd, nc, eps)
    for key, val in (("q", q), ("k", k), ("v", v)):
        assert_close(val[:, skip:], g[key], FP32_RTOL, f"{name}:{key}")
    pad = lambda t: torch.cat((torch.zeros(t.shape[0], skip, t.shape[2]), t), dim=1).cuda()
    dx, dw = _ops().qkv_conv_backward(x, w, pad(g["dq"]), pad(g["dk"]), pad(g["dv"]), hd, nc, eps)
    assert_close(dx[:, skip:], g["dx"], FP32_RTOL, f"{name}:dx")
    assert_close(dw, g["dweight"], FP32_RTOL, f"{name}:dweight")
    if skip:
        assert_close(dx[:, :skip], g["dprefix"], FP32_RTOL, f"{name}:dprefix")


CONV_SHAPES = [
    # B, T, H, D, taps  (ragged strips, channel counts off the 256-channel CTA width, every tap count)
    (2, 200, 4, 128, 4),
    (3, 67, 3, 32, 4),
    (1, 64, 1, 8, 1),
    (2, 129, 5, 16, 2),
    (1, 3, 2, 64, 3),
    (4, 1, 2, 128, 4),
]


@pytest.mark.parametrize("shape", CONV_SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_conv_matches_oracle(shape, dtype):
    B, T, H, D, taps = shape
    W = H * D
    gen = torch.Generator().manual_seed(100 + T)
    x = torch.randn(B, T, 3 * W, generator=gen).to(dtype)
    w = torch.randn(3 * W, taps, generator=gen) * 0.5
    grads = [torch.randn(B, T, W, generator=gen).to(dtype) for _ in range(3)]
    xo = x.float().requires_grad_(True)
    wo = w.clone().requires_grad_(True)
    ref = _oracle().qkv_conv_oracle(xo, wo, D, 2 * W, 1e-6)
    rdx, rdw = torch.autograd.grad(sum((r * d.float()).sum() for r, d in zip(ref, grads)), [xo, wo])
    got = _ops().qkv_conv_forward(x.cuda(), w.cuda(), D, 2 * W, 1e-6)
    dx, dw = _ops().qkv_conv_backward(x.cuda(), w.cuda(), *[d.cuda() for d in grads], D, 2 * W, 1e-6)
    rtol = BF16_RTOL if dtype == torch.bfloat16 else FP32_RTOL
    for key, a, e in zip("qkv", got, ref):
        assert a.dtype == dtype
        assert_close(a, e, rtol, f"{shape}:{key}")
    assert_close(dx, rdx, rtol, f"{shape}:dx")
    # dw sums B*T rounded products: bound its error against the sum's own scale
    assert rel_rms(dw, rdw) < (1e-2 if dtype == torch.bfloat16 else 1e-5), rel_rms(dw, rdw)


def test_conv_custom_op_autograd_and_determinism():
    B, T, H, D = 2, 150, 2, 128
    W = H * D
    gen = torch.Generator().manual_seed(7)
    x = torch.randn(B, T, 3 * W, generator=gen).bfloat16().cuda().requires_grad_(True)
    w = (torch.randn(3 * W, 4, generator=gen) * 0.5).cuda().requires_grad_(True)
    dq, dk, dv = (torch.randn(B, T, W, generator=gen).bfloat16().cuda() for _ in range(3))
    op = torch.ops.delta_feedback.pkda_qkv_conv
    _ops()
    runs = []
    for _ in range(2):
        q, k, v = op(x, w, D, 2 * W, 1e-6)
        dx, dw = torch.autograd.grad((q.float() * dq.float()).sum() + (k.float() * dk.float()).sum()
                                     + (v.float() * dv.float()).sum(), [x, w])
        runs.append((q, k, v, dx, dw))
    for a, b in zip(*runs):
        assert torch.equal(a, b)
    assert runs[0][4].dtype == torch.float32 and runs[0][3].dtype == torch.bfloat16
    # unit norm of every q / k head
    n = runs[0][0].float().reshape(B, T, H, D).square().sum(-1)
    assert (n - 1).abs().max() < 2e-2


def test_conv_rejects_bad_geometry():
    ops = _ops()
    x = torch.zeros(1, 4, 3 * 24, device="cuda")
    with pytest.raises(RuntimeError, match="unsupported geometry"):
        ops.qkv_conv_forward(x, torch.zeros(72, 4, device="cuda"), 24, 48, 1e-6)      # head_dim not a power of two
    with pytest.raises(RuntimeError, match="unsupported geometry"):
        ops.qkv_conv_forward(torch.zeros(1, 4, 96, device="cuda"), torch.zeros(96, 5, device="cuda"), 8, 64, 1e-6)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.qkv_conv_forward(torch.zeros(1, 4, 96), torch.zeros(96, 4), 8, 64, 1e-6)
    q, k, v = ops.qkv_conv_forward(torch.zeros(0, 4, 96, device="cuda"), torch.zeros(96, 4, device="cuda"), 8, 64, 1e-6)
    assert q.shape == (0, 4, 32)


# ------------------------------------------------------------------- norm gate
@pytest.mark.parametrize("name", GATE_CASES)
def test_norm_gate_fp32_matches_reference_golden(name):
    g = load_golden(name)
    eps = float(g["eps"])
    x, gate, w = g["x"].cuda(), g["gate"].cuda(), g["weight"].cuda()
    y, rstd = _ops().norm_gate_forward(x, gate, w, eps)
    assert_close(y, g["y"], FP32_RTOL, f"{name}:y")
    want_rstd = torch.rsqrt(g["x"].square().mean(-1) + eps).reshape(-1)
    assert_close(rstd, want_rstd, FP32_RTOL, f"{name}:rstd")
    dx, dg, dw = _ops().norm_gate_backward(x, gate, w, rstd, g["dy"].cuda(), eps)
    assert_close(dx, g["dx"], FP32_RTOL, f"{name}:dx")
    assert_close(dg, g["dgate"], FP32_RTOL, f"{name}:dgate")
    assert_close(dw, g["dweight"], FP32_RTOL, f"{name}:dweight")


@pytest.mark.parametrize("shape", [(2, 300, 16, 128), (1, 7, 3, 8), (3, 50, 2, 256), (1, 1, 1, 64), (2, 33, 5, 32)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_norm_gate_matches_oracle(shape, dtype):
    B, T, H, D = shape
    gen = torch.Generator().manual_seed(200 + T)
    x = (torch.randn(B, T, H, D, generator=gen) * 1.5).to(dtype)
    gate = (torch.randn(B, T, H, D, generator=gen) * 2).to(dtype)
    w = 1 + 0.3 * torch.randn(D, generator=gen)
    dy = torch.randn(B, T, H, D, generator=gen).to(dtype)
    xo, go, wo = (t.float().requires_grad_(True) for t in (x, gate, w))
    ry, rr = _oracle().norm_gate_oracle(xo, go, wo, 1e-6)
    rdx, rdg, rdw = torch.autograd.grad((ry * dy.float()).sum(), [xo, go, wo])
    y, rstd = _ops().norm_gate_forward(x.cuda(), gate.cuda(), w.cuda(), 1e-6)
    dx, dg, dw = _ops().norm_gate_backward(x.cuda(), gate.cuda(), w.cuda(), rstd, dy.cuda(), 1e-6)
    rtol = BF16_RTOL if dtype == torch.bfloat16 else FP32_RTOL
    assert y.dtype == dtype and rstd.dtype == torch.float32
    assert_close(y, ry, rtol, "y")
    assert_close(rstd, rr, FP32_RTOL, "rstd")
    assert_close(dx, rdx, rtol, "dx")
    assert_close(dg, rdg, rtol, "dgate")
    assert rel_rms(dw, rdw) < (1e-2 if dtype == torch.bfloat16 else 1e-5), rel_rms(dw, rdw)


def test_norm_gate_custom_op_autograd_and_determinism():
    B, T, H, D = 2, 257, 4, 128
    gen = torch.Generator().manual_seed(9)
    x = torch.randn(B, T, H, D, generator=gen).bfloat16().cuda().requires_grad_(True)
    gate = torch.randn(B, T, H, D, generator=gen).bfloat16().cuda().requires_grad_(True)
    w = (1 + 0.1 * torch.randn(D, generator=gen)).cuda().requires_grad_(True)
    dy = torch.randn(B, T, H, D, generator=gen).bfloat16().cuda()
    _ops()
    op = torch.ops.delta_feedback.pkda_norm_gate
    runs = []
    for _ in range(2):
        y, rstd = op(x, gate, w, 1e-6)
        assert rstd.shape == (B * T * H,) and not rstd.requires_grad
        runs.append((y,) + torch.autograd.grad((y.float() * dy.float()).sum(), [x, gate, w]))
    for a, b in zip(*runs):
        assert torch.equal(a, b)


def test_norm_gate_rejects_bad_geometry():
    ops = _ops()
    with pytest.raises(RuntimeError, match="unsupported geometry"):
        ops.norm_gate_forward(torch.zeros(4, 24, device="cuda"), torch.zeros(4, 24, device="cuda"),
                              torch.ones(24, device="cuda"), 1e-6)
    y, rstd = ops.norm_gate_forward(torch.zeros(0, 64, device="cuda"), torch.zeros(0, 64, device="cuda"),
                                    torch.ones(64, device="cuda"), 1e-6)
    assert y.shape == (0, 64) and rstd.shape == (0,)
