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

Launching the twenty-odd kernels of a slice from Python costs about as much host
time as the slice's copies take on the bus, so with many slices the host becomes
the bottleneck.  When the batch divides evenly into the slices, ``HostStep``
therefore captures the forward+backward of one slice into a CUDA graph on fixed
device buffers (three sets, used in turn, so that copy-in, kernels and copy-out of
neighbouring slices overlap) and replays it per slice; the host then only enqueues
the copies and the replays.  Forward and backward are two graphs: the forward does
not need the output cotangent, so it starts while that tensor is still on its way in,
and the output leaves for the host while the backward runs; this shortens the two ends
of the pipeline, where nothing else overlaps.
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

    def __init__(self, device, slices=4, lean: bool = False, graphs: bool = True, trace: bool = False):
        """``slices``: how many equal row slices to cut the batch into, or a sequence of row
        counts (summing to the batch), e.g. ``(1, 3, 3, 1)``: small slices at both ends keep the
        un-overlapped first copy-in and last copy-out short, large ones in between keep the
        number of copies that alternate on the bus low."""
        self.device = torch.device(device)
        self.plan = None if isinstance(slices, int) else tuple(int(x) for x in slices)
        self.slices = int(slices) if isinstance(slices, int) else len(self.plan)
        self.lean = bool(lean)
        self.graphs = bool(graphs)
        self.trace = bool(trace)  # graph mode: record events around every slice's three stages (see timeline())
        self._marks = []
        self._slots = None      # graph mode: three sets of fixed device buffers with a captured step each
        self._slot_key = None
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

    # ------------------------------------------------------------------ graph mode
    def _forward(self, rows, params, with_state):
        """Forward of one slice on device tensors; returns (o, the tensors to differentiate)."""
        # (detached views: the fixed buffers themselves stay plain tensors the copies can write into)
        leaves = [rows[n].detach().requires_grad_(True) for n in ROW_INPUTS]
        heads = [params[n].detach().requires_grad_(True) for n in HEAD_PARAMS]
        kw = dict(zip(INPUT_NAMES, leaves + heads))
        centre = kw.pop("log_atk_scale")
        S0 = A0 = None
        wrt = leaves + heads
        if with_state:
            S0 = rows["initial_state"].detach().requires_grad_(True)
            A0 = rows["initial_A_state"].detach().requires_grad_(True)
            wrt = wrt + [S0, A0]
        o, _, _ = chunk_precond_kda(**kw, initial_state=S0, initial_A_state=A0,
                                    output_final_state=False, log_atk_scale=centre,
                                    disable_recompute=not self.lean)
        return o, wrt

    def _step(self, rows, params, with_state):
        """Forward + backward of one slice on device tensors; returns (o, grads)."""
        o, wrt = self._forward(rows, params, with_state)
        grads = torch.autograd.grad(o, wrt, rows["do"])
        return o.detach(), [g.detach() for g in grads]

    def _build_slots(self, host, do, with_state, rows_per):
        dev = self.device
        names = list(ROW_INPUTS) + ["do"] + (["initial_state", "initial_A_state"] if with_state else [])
        src = dict(host, do=do)
        if getattr(self, "_params", None) is None:
            self._params = {n: torch.empty(host[n].shape, dtype=host[n].dtype, device=dev) for n in HEAD_PARAMS}
        # Every graph keeps a memory pool of its own: with a shared pool the temporaries of one graph's
        # replay would land on the results of the graph captured after it, which are still being copied out.
        slots = []
        for k in range(3):
            rows = {n: torch.zeros((rows_per, *src[n].shape[1:]), dtype=src[n].dtype, device=dev) for n in names}
            with torch.cuda.stream(self.s_comp):
                if k == 0:  # one eager pass first (lazy initialisation must not happen inside a capture)
                    for n in HEAD_PARAMS:
                        self._params[n].copy_(host[n], non_blocking=True)
                    for n in names:
                        rows[n].copy_(src[n][:rows_per], non_blocking=True)
                    self._step(rows, self._params, with_state)
            self.s_comp.synchronize()
            # two graphs on one private pool (they replay in capture order): forward, then backward
            graph_f, graph_b = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph_f, stream=self.s_comp):
                o_live, wrt = self._forward(rows, self._params, with_state)
            with torch.cuda.graph(graph_b, pool=graph_f.pool(), stream=self.s_comp):
                grads = [g.detach() for g in torch.autograd.grad(o_live, wrt, rows["do"])]
            slots.append({"rows": rows, "graph_f": graph_f, "graph_b": graph_b, "o": o_live.detach(), "grads": grads,
                          "in_free": torch.cuda.Event(), "out_free": torch.cuda.Event(),
                          "ready_f": torch.cuda.Event(), "ready": torch.cuda.Event(),
                          "done_f": torch.cuda.Event(), "done": torch.cuda.Event()})
        for sl in slots:  # nothing pending on a fresh slot
            sl["in_free"].record(self.s_comp)
            sl["out_free"].record(self.s_out)
        self._names = names
        return slots

    def _call_graphs(self, host, do, with_state, plan):
        dev, out = self.device, self.out
        key = (plan, with_state, tuple(do.shape), do.dtype)
        if self._slots is None or self._slot_key != key:
            self._params = None
            # three buffer sets (and captured steps) per distinct slice size
            self._slots = {r: self._build_slots(host, do, with_state, r) for r in sorted(set(plan))}
            self._slot_key = key
        used = {r: 0 for r in self._slots}
        cur = torch.cuda.current_stream(dev)
        for s in (self.s_in, self.s_comp, self.s_out):
            s.wait_stream(cur)
        self.h2d_bytes = self.d2h_bytes = 0
        src = dict(host, do=do)
        nbytes = lambda t: t.numel() * t.element_size()
        with torch.cuda.stream(self.s_in):
            for n in HEAD_PARAMS:
                self._params[n].copy_(host[n], non_blocking=True)
                self.h2d_bytes += nbytes(host[n])
            params_ready = torch.cuda.Event()
            params_ready.record(self.s_in)
        acc = None
        b1 = 0
        self._marks = []

        def mark(stream):
            if not self.trace:
                return None
            e = torch.cuda.Event(enable_timing=True)
            e.record(stream)
            return e

        t_origin = mark(cur)
        for i, rows_per in enumerate(plan):
            sl = self._slots[rows_per][used[rows_per] % 3]
            used[rows_per] += 1
            b0, b1 = b1, b1 + rows_per
            with torch.cuda.stream(self.s_in):
                self.s_in.wait_event(sl["in_free"])       # the replay that last read these inputs is over
                m0 = mark(self.s_in)
                for n in self._names:  # the output cotangent last: only the backward waits for it
                    if n != "do":
                        sl["rows"][n].copy_(src[n][b0:b1], non_blocking=True)
                        self.h2d_bytes += nbytes(sl["rows"][n])
                sl["ready_f"].record(self.s_in)
                sl["rows"]["do"].copy_(src["do"][b0:b1], non_blocking=True)
                self.h2d_bytes += nbytes(sl["rows"]["do"])
                sl["ready"].record(self.s_in)
                m1 = mark(self.s_in)
            with torch.cuda.stream(self.s_comp):
                if i == 0:
                    self.s_comp.wait_event(params_ready)
                self.s_comp.wait_event(sl["ready_f"])
                self.s_comp.wait_event(sl["out_free"])    # the copies that last read these outputs are over
                m2 = mark(self.s_comp)
                sl["graph_f"].replay()
                sl["done_f"].record(self.s_comp)
                self.s_comp.wait_event(sl["ready"])
                sl["graph_b"].replay()
                head = sl["grads"][7:10]
                if acc is None:
                    acc = [g.float().clone() for g in head]
                else:
                    for a, g in zip(acc, head):
                        a.add_(g)
                sl["in_free"].record(self.s_comp)
                sl["done"].record(self.s_comp)
                m3 = mark(self.s_comp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(sl["done_f"])       # the output goes home while the backward runs
                m4 = mark(self.s_out)
                out["o"][b0:b1].copy_(sl["o"], non_blocking=True)
                self.d2h_bytes += nbytes(sl["o"])
                self.s_out.wait_event(sl["done"])
                pairs = [(out["d" + n][b0:b1], g) for n, g in zip(ROW_INPUTS, sl["grads"][:7])]
                if with_state:
                    pairs += [(out["dinitial_state"][b0:b1], sl["grads"][10]),
                              (out["dinitial_A_state"][b0:b1], sl["grads"][11])]
                for dst, g in pairs:
                    dst.copy_(g, non_blocking=True)
                    self.d2h_bytes += nbytes(g)
                sl["out_free"].record(self.s_out)
                if self.trace:
                    self._marks.append((t_origin, m0, m1, m2, m3, m4, mark(self.s_out)))
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_stream(self.s_comp)
            for n, g in zip(HEAD_PARAMS, acc):
                g.record_stream(self.s_out)
                out["d" + n].copy_(g, non_blocking=True)
                self.d2h_bytes += nbytes(g)
        cur.wait_stream(self.s_out)
        return out

    def timeline(self):
        """With ``trace=True``, after a synchronised call in graph mode: per slice the start and end
        (ms after the call began) of its copy-in, its kernels and its copy-out, as six numbers."""
        return [tuple(t0.elapsed_time(m) for m in rest) for t0, *rest in self._marks]

    def __call__(self, host: Dict[str, Tensor], do: Tensor) -> Dict[str, Tensor]:
        dev = self.device
        B = host["q"].shape[0]
        with_state = host.get("initial_state") is not None
        if self.out is None:
            self.out = self._alloc_out(host, do, with_state)
        out = self.out
        n_slices = max(1, min(self.slices, B))
        plan = self.plan
        if plan is not None and (sum(plan) != B or min(plan) < 1):
            raise ValueError(f"the slice plan {plan} does not add up to the batch of {B} rows")
        if plan is None and B % n_slices == 0:
            plan = (B // n_slices,) * n_slices
        if self.graphs and plan is not None:
            return self._call_graphs(host, do, with_state, plan)
        bounds = [(B * i) // n_slices for i in range(n_slices + 1)]
        if plan is not None:
            bounds = [sum(plan[:i]) for i in range(len(plan) + 1)]
            n_slices = len(plan)
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
