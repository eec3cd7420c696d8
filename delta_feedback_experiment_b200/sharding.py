"""Splitting one PKDA problem over several GPUs.

Every (batch row or packed sequence, head) pair of the operator is independent:
each owns its state ``S``, its preconditioner state ``A`` and its per-head
parameters, and no term of the recurrence couples rows
(``delta_feedback_experiment/pkda.py:390-406`` contracts over neither ``b`` nor
``h``).  A problem therefore shards with no exchange step: rows (or sequences)
first, heads when there are fewer rows than ranks.  Each rank runs the
single-GPU operator on its slice; results are concatenated, and the per-head
parameter gradients of ranks that share heads are added by the caller's
existing data-parallel reduction (they are sums over rows).

This module only does the index arithmetic and the slicing, on whatever device
the tensors live on; it launches nothing and needs no process group.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
from torch import Tensor

from .synthetic import INPUT_NAMES

ROW_INPUTS = INPUT_NAMES[:7]      # q, k, v, g, g_atk, beta_atk, beta
HEAD_PARAMS = INPUT_NAMES[7:]     # A_log [H], dt_bias [H*D], log_atk_scale [H]


@dataclass(frozen=True)
class Shard:
    """What one rank owns: rows ``[row0, row1)`` (batch rows, or sequences of a
    packed batch) and heads ``[head0, head1)``."""
    row0: int
    row1: int
    head0: int
    head1: int

    @property
    def empty(self) -> bool:
        return self.row1 <= self.row0 or self.head1 <= self.head0


def _even_split(n: int, parts: int) -> List[Tuple[int, int]]:
    return [((n * i) // parts, (n * (i + 1)) // parts) for i in range(parts)]


def _balanced_split(lengths: Sequence[int], parts: int) -> List[Tuple[int, int]]:
    """Contiguous groups of sequences with about equal token counts: group i ends
    at the first sequence boundary at or past i/parts of the total (a boundary is
    never moved backwards, so every group is contiguous and the groups cover all
    sequences; a group may be empty when one sequence is longer than a share)."""
    total = sum(lengths)
    bounds, acc, j = [0], 0, 0
    for i in range(1, parts):
        target = total * i / parts
        while j < len(lengths) and acc + lengths[j] / 2 < target:
            acc += lengths[j]
            j += 1
        bounds.append(j)
    bounds.append(len(lengths))
    return [(bounds[i], bounds[i + 1]) for i in range(parts)]


def shard_plan(n_rows: int, n_heads: int, world: int,
               seq_lengths: Optional[Sequence[int]] = None) -> List[Shard]:
    """One ``Shard`` per rank.  Rows are split first (balanced by token count when
    ``seq_lengths`` gives the lengths of a packed batch's sequences); when there
    are fewer rows than ranks, the ranks of a row split its heads (``world`` must
    then be a multiple of ``n_rows`` and the heads divisible by the ranks per row)."""
    if world < 1 or n_rows < 1 or n_heads < 1:
        raise ValueError("world, rows and heads must be positive")
    if seq_lengths is not None and len(seq_lengths) != n_rows:
        raise ValueError("one length per sequence is needed")
    if n_rows >= world:
        rows = _balanced_split(seq_lengths, world) if seq_lengths is not None else _even_split(n_rows, world)
        return [Shard(a, b, 0, n_heads) for a, b in rows]
    if world % n_rows:
        raise ValueError(f"{world} ranks cannot split {n_rows} rows evenly by heads")
    per_row = world // n_rows
    if n_heads % per_row:
        raise ValueError(f"{n_heads} heads do not divide over {per_row} ranks per row")
    hs = n_heads // per_row
    return [Shard(r // per_row, r // per_row + 1, (r % per_row) * hs, (r % per_row + 1) * hs)
            for r in range(world)]


def shard_inputs(inputs: Dict[str, Tensor], shard: Shard, head_dim: int,
                 cu_seqlens: Optional[Tensor] = None) -> Tuple[Dict[str, Tensor], Optional[Tensor]]:
    """The rank's slice of the ten operator inputs (plus ``do``, ``initial_state``,
    ``initial_A_state`` when present) and, for a packed batch, its own
    ``cu_seqlens`` (re-based to start at 0).  Row tensors are ``[B, T, H, ...]``
    (dense) or ``[1, T_total, H, ...]`` (packed); states are ``[N, H, ...]``.
    Slices are made contiguous, as the kernels require."""
    h = slice(shard.head0, shard.head1)
    out: Dict[str, Tensor] = {}
    if cu_seqlens is None:
        rows = slice(shard.row0, shard.row1)
        tok = slice(None)
    else:
        offs = cu_seqlens.tolist()
        rows = slice(0, 1)
        tok = slice(offs[shard.row0], offs[shard.row1])
    for n in (*ROW_INPUTS, "do"):
        if n in inputs and inputs[n] is not None:
            out[n] = inputs[n][rows, tok, h].contiguous()
    for n in ("initial_state", "initial_A_state"):
        if inputs.get(n) is not None:
            out[n] = inputs[n][shard.row0:shard.row1, h].contiguous()
    out["A_log"] = inputs["A_log"][h].contiguous()
    out["log_atk_scale"] = inputs["log_atk_scale"][h].contiguous()
    out["dt_bias"] = inputs["dt_bias"][shard.head0 * head_dim:shard.head1 * head_dim].contiguous()
    cu = None
    if cu_seqlens is not None:
        cu = (cu_seqlens[shard.row0:shard.row1 + 1] - cu_seqlens[shard.row0]).contiguous()
    return out, cu


def merge_row_outputs(pieces: Sequence[Tensor], plan: Sequence[Shard], packed: bool = False) -> Tensor:
    """Puts per-rank row tensors (``o``, or the gradient of a row input) back
    together: ranks that share rows are concatenated along the head axis (2),
    row groups along the batch axis (0), or the token axis (1) for a packed batch.
    State-shaped results ``[N, H, ...]`` use ``merge_state_outputs``."""
    groups: Dict[Tuple[int, int], List[Tuple[int, Tensor]]] = {}
    for t, s in zip(pieces, plan):
        if not s.empty:
            groups.setdefault((s.row0, s.row1), []).append((s.head0, t))
    merged = [torch.cat([t for _, t in sorted(g, key=lambda x: x[0])], dim=2) for _, g in sorted(groups.items())]
    return torch.cat(merged, dim=1 if packed else 0)


def merge_state_outputs(pieces: Sequence[Tensor], plan: Sequence[Shard]) -> Tensor:
    """The same for ``[N, H, ...]`` tensors (final states, initial-state gradients)."""
    groups: Dict[Tuple[int, int], List[Tuple[int, Tensor]]] = {}
    for t, s in zip(pieces, plan):
        if not s.empty:
            groups.setdefault((s.row0, s.row1), []).append((s.head0, t))
    merged = [torch.cat([t for _, t in sorted(g, key=lambda x: x[0])], dim=1) for _, g in sorted(groups.items())]
    return torch.cat(merged, dim=0)


def merge_head_grads(pieces: Sequence[Tensor], plan: Sequence[Shard], n_heads: int, per_head: int = 1) -> Tensor:
    """Adds the per-head parameter gradients of all ranks into the full vector
    (``per_head`` entries per head: 1 for ``A_log`` and ``log_atk_scale``,
    ``head_dim`` for ``dt_bias``).  Ranks are added in rank order."""
    ref = next(t for t, s in zip(pieces, plan) if not s.empty)
    out = torch.zeros((n_heads * per_head,), dtype=torch.float32, device=ref.device)
    for t, s in zip(pieces, plan):
        if not s.empty:
            out[s.head0 * per_head:s.head1 * per_head] += t.to(torch.float32)
    return out
