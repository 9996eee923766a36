"""Poon-Domingos circuits over a grid of variables (PyJuice: structures/pd.py:17-243).

Every axis-aligned hyper-rectangle reachable by cutting at the given split points is a region;
a region's sum vector mixes one product vector per (axis, split point) cut.  Regions with more
than ``max_prod_block_conns`` cuts connect every sum block to a random subset of the cuts.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple, Union

import torch

from ..nodes import BitSet, Categorical, inputs, multiply, summate, set_block_size
from .hclt import max_cdf_power_of_2


def PD(data_shape: Tuple[int, ...], num_latents: int,
       split_intervals: Optional[Union[int, Tuple[int, ...]]] = None,
       split_points: Optional[Sequence[Sequence[int]]] = None,
       max_split_depth: Optional[int] = None, max_prod_block_conns: int = 4,
       structure_type: str = "sum_dominated", num_cats: int = 256,
       tie_homogeneous_params: bool = False, block_size: Optional[int] = None):
    assert structure_type in ("sum_dominated", "prod_dominated")
    data_shape = tuple(data_shape)
    num_axes = len(data_shape)
    if block_size is None:
        block_size = min(16 if num_latents <= 32 else 32, max_cdf_power_of_2(num_latents))
    num_node_blocks = num_latents // block_size

    if split_intervals is not None:
        if isinstance(split_intervals, int):
            split_intervals = (split_intervals,) * num_axes
        split_points = [list(range(split_intervals[a], data_shape[a], split_intervals[a])) for a in range(num_axes)]
    else:
        assert split_points is not None and len(split_points) == num_axes
        for a in range(num_axes):
            assert all(0 < sp < data_shape[a] - 1 for sp in split_points[a])

    strides = [1] * num_axes
    for a in range(num_axes - 2, -1, -1):
        strides[a] = strides[a + 1] * data_shape[a + 1]

    def cube_vars(lo, hi):
        ids = torch.zeros([1], dtype=torch.long)
        for a in range(num_axes):
            ids = (ids[:, None] + torch.arange(lo[a], hi[a])[None, :] * strides[a]).reshape(-1)
        return sorted(ids.tolist())

    sources: Dict = {}
    cache: Dict = {}

    def signature(lo, hi, *ch_ns):
        return (tuple(h - l for l, h in zip(lo, hi)), tuple(len(ns.scope) for ns in ch_ns))

    def tied_or_new_sum(sig, pns, edge_ids=None):
        if not tie_homogeneous_params:
            return summate(*pns, num_node_blocks=num_node_blocks, edge_ids=edge_ids)
        if sig in sources:
            return sources[sig].duplicate(*pns, tie_params=True)
        sources[sig] = summate(*pns, num_node_blocks=num_node_blocks, edge_ids=edge_ids)
        return sources[sig]

    def leaf_region(lo, hi):
        leaves = []
        for var in cube_vars(lo, hi):
            if not tie_homogeneous_params:
                ns = inputs(var, num_node_blocks=num_node_blocks, dist=Categorical(num_cats=num_cats))
            elif "input" in sources:
                ns = sources["input"].duplicate(var, tie_params=True)
            else:
                ns = inputs(var, num_node_blocks=num_node_blocks, dist=Categorical(num_cats=num_cats))
                sources["input"] = ns
            leaves.append(ns)
        pn = multiply(*leaves)
        diag = torch.arange(0, num_node_blocks)[None, :].repeat(2, 1)
        return tied_or_new_sum(signature(lo, hi, pn), [pn], edge_ids=diag)

    root_cube = ((0,) * num_axes, data_shape)

    def build(lo, hi, depth=1):
        key = (lo, hi)
        if key in cache:
            return cache[key]
        if max_split_depth is not None and depth > max_split_depth:
            cache[key] = leaf_region(lo, hi)
            return cache[key]

        pns = []
        for a in range(num_axes):
            for sp in [p for p in split_points[a] if lo[a] < p < hi[a]]:
                left_hi = hi[:a] + (sp,) + hi[a + 1:]
                right_lo = lo[:a] + (sp,) + lo[a + 1:]
                # structures/pd.py:170-171 recurses without passing the depth on, so every
                # region below the root is built at depth 1.
                ns1 = build(lo, left_hi)
                ns2 = build(right_lo, hi)
                if structure_type == "sum_dominated":
                    pns.append(multiply(ns1, ns2))
                else:
                    pns.append(multiply(ns1.duplicate(), ns2.duplicate()))

        if len(pns) == 0:
            ns = leaf_region(lo, hi)
        elif key == root_cube:
            ns = summate(*pns, num_node_blocks=1, block_size=1)
        elif len(pns) <= max_prod_block_conns:
            ns = tied_or_new_sum(signature(lo, hi, *pns), pns)
        else:
            k = max_prod_block_conns
            picks = torch.topk(torch.rand([num_node_blocks, len(pns)]), k=k, dim=1).indices
            par_ids = torch.arange(0, num_node_blocks)[:, None, None].repeat(1, k, num_node_blocks)
            chs_ids = picks[:, :, None] * num_node_blocks + torch.arange(0, num_node_blocks)[None, None, :]
            edge_ids = torch.stack((par_ids.reshape(-1), chs_ids.reshape(-1)), dim=0)
            ns = tied_or_new_sum(signature(lo, hi, *pns), pns, edge_ids=edge_ids)
        cache[key] = ns
        return ns

    with set_block_size(block_size):
        return build(*root_cube)
