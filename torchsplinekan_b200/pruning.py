"""
Removal of unimportant hidden nodes from a :class:`~torchsplinekan_b200.KAN`
(API of spline_kan/pruning.py: ``PruneResult``, ``node_scores``, ``prune_nodes``).

A hidden node is scored by the strongest edge entering it and the strongest
edge leaving it, an edge's strength being ``mean_n |phi(x_n)|`` on the inputs
that layer really sees (:meth:`KANLinear.edge_l1`, which on CUDA inputs runs the
native edge-statistic kernels straight from ``x``).  Nodes whose two scores both
exceed the threshold survive; the rows / columns of the others are cut out of
the neighbouring layers' tensors and a smaller, independent network is built.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .kan import KAN
from .kan_linear import KANLinear


@dataclass
class PruneResult:
    """Outcome of :func:`prune_nodes` (spline_kan/pruning.py:30-52)."""
    model: KAN
    kept: List[List[int]]
    old_to_new: List[Dict[int, int]]
    widths_before: List[int]
    widths_after: List[int]
    params_before: int
    params_after: int
    scores_in: List[torch.Tensor] = field(repr=False, default_factory=list)
    scores_out: List[torch.Tensor] = field(repr=False, default_factory=list)
    threshold: float = 1e-2

    def summary(self) -> dict:
        names = ("widths_before", "widths_after", "params_before", "params_after", "kept", "threshold")
        return {n: getattr(self, n) for n in names}


@torch.no_grad()
def node_scores(model: KAN, x: torch.Tensor):
    """``(incoming, outgoing)``: per hidden layer one ``[width]`` tensor each
    (spline_kan/pruning.py:55-69)."""
    strengths, h = [], x
    for layer in model.layers:
        strengths.append(layer.edge_l1(h))              # [O, I] on this layer's own inputs
        h = layer(h)
    incoming = [a.amax(dim=1) for a in strengths[:-1]]  # over the edges that end in the node
    outgoing = [a.amax(dim=0) for a in strengths[1:]]   # over the edges that start at it
    return incoming, outgoing


def _cut(layer: KANLinear, rows: torch.Tensor, cols: torch.Tensor) -> KANLinear:
    """Copy of ``layer`` restricted to output nodes ``rows`` and input nodes ``cols``."""
    small = layer.make_like(in_features=int(cols.numel()), out_features=int(rows.numel()))
    pick = lambda t: t.index_select(0, rows).index_select(1, cols)
    with torch.no_grad():
        small.base_weight.copy_(pick(layer.base_weight))
        small.spline_weight.copy_(pick(layer.spline_weight))
        if layer.enable_standalone_scale_spline:
            small.spline_scaler.copy_(pick(layer.spline_scaler))
        small._copy_grid_(layer.grid.index_select(0, cols))
    small.requires_grad_(any(p.requires_grad for p in layer.parameters()))
    return small.train(layer.training)


def prune_nodes(model: KAN, x_calib: Optional[torch.Tensor] = None, threshold: float = 1e-2, *,
                keep: Optional[Sequence[Sequence[int]]] = None, min_keep: int = 1) -> PruneResult:
    """Smaller network without the hidden nodes whose incoming or outgoing score is at most
    ``threshold``; ``model`` is left untouched.  ``keep`` lists the surviving indices per hidden
    layer explicitly (no scoring then); ``min_keep`` nodes per hidden layer always survive, chosen
    by the larger ``min(incoming, outgoing)`` (spline_kan/pruning.py:86-156)."""
    hidden = len(model.layers) - 1
    scores_in: List[torch.Tensor] = []
    scores_out: List[torch.Tensor] = []
    if keep is None:
        if x_calib is None:
            raise ValueError("prune_nodes needs x_calib (or explicit keep indices)")
        scores_in, scores_out = node_scores(model, x_calib)
        keep = []
        for s_in, s_out in zip(scores_in, scores_out):
            alive = torch.nonzero((s_in > threshold) & (s_out > threshold)).flatten()
            if alive.numel() < min_keep:
                best = torch.minimum(s_in, s_out).topk(min(min_keep, s_in.numel())).indices
                alive = best.sort().values
            keep.append(alive.tolist())
    if len(keep) != hidden:
        raise ValueError(f"keep must list {hidden} hidden layers, got {len(keep)}")

    widths = model.widths
    device = model.layers[0].grid.device
    node_sets = [torch.arange(widths[0], device=device)]
    for depth, chosen in enumerate(keep, start=1):
        chosen = sorted({int(i) for i in chosen})
        if not chosen:
            raise ValueError(f"hidden layer {depth} would have no nodes")
        if chosen[0] < 0 or chosen[-1] >= widths[depth]:
            raise ValueError(f"keep indices out of range for hidden layer {depth}")
        node_sets.append(torch.tensor(chosen, device=device))
    node_sets.append(torch.arange(widths[-1], device=device))

    small = KAN.from_layers([_cut(layer, node_sets[d + 1], node_sets[d])
                             for d, layer in enumerate(model.layers)]).train(model.training)
    kept = [s.tolist() for s in node_sets[1:-1]]
    return PruneResult(model=small, kept=kept,
                       old_to_new=[{old: new for new, old in enumerate(k)} for k in kept],
                       widths_before=widths, widths_after=small.widths,
                       params_before=sum(p.numel() for p in model.parameters()),
                       params_after=sum(p.numel() for p in small.parameters()),
                       scores_in=scores_in, scores_out=scores_out, threshold=threshold)
