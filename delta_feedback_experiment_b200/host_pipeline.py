"""Forward + backward of the chunked PKDA operator for data that lives in host
memory.

The operators of this package take CUDA tensors, as the reference's do
(``delta_feedback_experiment/pkda.py:412-475``).  A caller whose activations sit
in pinned host memory (offloaded activations, a data-parallel shard handed over
by another process) pays two PCIe crossings per step, and those dominate the
step: at the headline shape 683 MB go each way while the kernels need about
4 ms.  Rows of the batch are independent in this operator, so the step can be
streamed: ``HostStep`` cuts the batch into row slices and overlaps the
host-to-device copy of slice i+1, the kernels of slice i and the device-to-host
copy of slice i-1 on three CUDA streams.  The result is what the un-sliced
device call returns (per-row tensors exactly, per-head parameter gradients up to
the order in which the slices are added).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch
from torch import Tensor

from .pkda import chunk_precond_kda
from .synthetic import INPUT_NAMES

ROW_INPUTS = INPUT_NAMES[:7]      # q, k, v, g, g_atk, beta_atk, beta: one leading batch axis
HEAD_PARAMS = INPUT_NAMES[7:]     # A_log, dt_bias, log_atk_scale: shared by all rows


class HostStep:
    """``HostStep(device, slices)(host, do, ...)`` runs one forward+backward.

    ``host`` maps the ten input names (``synthetic.INPUT_NAMES``) to CPU tensors,
    optionally ``initial_state`` / ``initial_A_state`` as well; ``do`` is the
    output cotangent.  Pinned tensors make the copies asynchronous.  Returns a
    dict of pinned CPU tensors: ``o``, ``d<name>`` for the ten inputs and, when
    states were given, ``dinitial_state`` / ``dinitial_A_state``.  The output
    buffers are allocated on the first call and reused afterwards.  The call
    returns once everything is enqueued; the current stream waits for the last
    copy, so a ``torch.cuda.synchronize()`` or an event on the current stream
    marks completion.
    """

    def __init__(self, device, slices: int = 4, lean: bool = False):
        self.device = torch.device(device)
        self.slices = int(slices)
        self.lean = bool(lean)
        self.s_in = torch.cuda.Stream(self.device)
        self.s_comp = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.out: Optional[Dict[str, Tensor]] = None
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def _alloc_out(self, host, do, with_state):
        out = {"o": torch.empty(do.shape, dtype=do.dtype, pin_memory=True)}
        for n in INPUT_NAMES:
            dt = torch.float32 if n in ("g_atk",) + tuple(HEAD_PARAMS) else host[n].dtype
            out["d" + n] = torch.empty(host[n].shape, dtype=dt, pin_memory=True)
        if with_state:
            for n in ("initial_state", "initial_A_state"):
                out["d" + n] = torch.empty(host[n].shape, dtype=torch.float32, pin_memory=True)
        return out

    def __call__(self, host: Dict[str, Tensor], do: Tensor) -> Dict[str, Tensor]:
        dev = self.device
        B = host["q"].shape[0]
        with_state = host.get("initial_state") is not None
        if self.out is None:
            self.out = self._alloc_out(host, do, with_state)
        out = self.out
        n_slices = max(1, min(self.slices, B))
        bounds = [(B * i) // n_slices for i in range(n_slices + 1)]
        cur = torch.cuda.current_stream(dev)
        for s in (self.s_in, self.s_comp, self.s_out):
            s.wait_stream(cur)
        self.h2d_bytes = self.d2h_bytes = 0

        def to_dev(t: Tensor) -> Tensor:
            d = torch.empty(t.shape, dtype=t.dtype, device=dev)
            d.copy_(t, non_blocking=True)
            d.record_stream(self.s_comp)
            self.h2d_bytes += t.numel() * t.element_size()
            return d

        def to_host(dst: Tensor, src: Tensor) -> None:
            src.record_stream(self.s_out)
            dst.copy_(src, non_blocking=True)
            self.d2h_bytes += src.numel() * src.element_size()

        with torch.cuda.stream(self.s_in):
            params = {n: to_dev(host[n]) for n in HEAD_PARAMS}
            params_ready = torch.cuda.Event()
            params_ready.record(self.s_in)
        param_grads = None
        staged = []
        for i in range(n_slices):
            b0, b1 = bounds[i], bounds[i + 1]
            with torch.cuda.stream(self.s_in):
                rows = {n: to_dev(host[n][b0:b1]) for n in ROW_INPUTS}
                rows["do"] = to_dev(do[b0:b1])
                if with_state:
                    rows["initial_state"] = to_dev(host["initial_state"][b0:b1])
                    rows["initial_A_state"] = to_dev(host["initial_A_state"][b0:b1])
                ready = torch.cuda.Event()
                ready.record(self.s_in)
            with torch.cuda.stream(self.s_comp):
                self.s_comp.wait_event(params_ready)
                self.s_comp.wait_event(ready)
                leaves = [rows[n].requires_grad_(True) for n in ROW_INPUTS]
                heads = [params[n].detach().requires_grad_(True) for n in HEAD_PARAMS]
                kw = dict(zip(INPUT_NAMES, leaves + heads))
                centre = kw.pop("log_atk_scale")
                S0 = A0 = None
                wrt = leaves + heads
                if with_state:
                    S0 = rows["initial_state"].requires_grad_(True)
                    A0 = rows["initial_A_state"].requires_grad_(True)
                    wrt = wrt + [S0, A0]
                o, _, _ = chunk_precond_kda(**kw, initial_state=S0, initial_A_state=A0,
                                            output_final_state=False, log_atk_scale=centre,
                                            disable_recompute=not self.lean)
                grads = torch.autograd.grad(o, wrt, rows["do"])
                head_grads = [g.float() for g in grads[7:10]]
                if param_grads is None:
                    param_grads = head_grads
                else:
                    for acc, g in zip(param_grads, head_grads):
                        acc.add_(g)
                done = torch.cuda.Event()
                done.record(self.s_comp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                to_host(out["o"][b0:b1], o.detach())
                for n, g in zip(ROW_INPUTS, grads[:7]):
                    to_host(out["d" + n][b0:b1], g)
                if with_state:
                    to_host(out["dinitial_state"][b0:b1], grads[10])
                    to_host(out["dinitial_A_state"][b0:b1], grads[11])
            staged.append((rows, o, grads))
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_stream(self.s_comp)
            for n, g in zip(HEAD_PARAMS, param_grads):
                to_host(out["d" + n], g)
        cur.wait_stream(self.s_out)
        return out
