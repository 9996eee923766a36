"""Random and tensorised sum-product networks (PyJuice: structures/rat_spn.py:16-102).

``num_repetitions`` independent random binary (``num_pieces``-ary) scope splits of depth
``depth``; leaf regions are products of per-variable input vectors; one root sum over the
top products of all repetitions.  Scope shuffling uses Python's ``random`` module.
"""
from __future__ import annotations

import random
from typing import Optional

from ..nodes import Categorical, inputs, multiply, summate, set_block_size
from .hclt import max_cdf_power_of_2


def RAT_SPN(num_vars: int, num_latents: int, depth: int, num_repetitions: int, num_pieces: int = 2,
            num_cats: int = 256, block_size: Optional[int] = None):
    if block_size is None:
        block_size = min(256, max_cdf_power_of_2(num_latents))
    assert num_latents % block_size == 0, f"`num_latents` ({num_latents}) not divisible by `block_size` ({block_size})."
    num_node_blocks = num_latents // block_size

    with set_block_size(block_size):
        input_ns = [inputs(v, num_node_blocks=num_node_blocks, dist=Categorical(num_cats=num_cats))
                    for v in range(num_vars)]

        def region(scope_vars, curr_depth=0):
            # `scope_vars` is ascending, the order a scope set enumerates its variables in.
            if curr_depth >= depth or len(scope_vars) < num_pieces:
                return summate(multiply(*[input_ns[v] for v in scope_vars]), num_node_blocks=num_node_blocks)
            shuffled = list(scope_vars)
            random.shuffle(shuffled)
            q, r = divmod(len(shuffled), num_pieces)
            pieces, sid = [], 0
            for i in range(num_pieces):
                eid = sid + q + (1 if i < r else 0)
                pieces.append(sorted(shuffled[sid:eid]))
                sid = eid
            chs = [region(p, curr_depth + 1) for p in pieces]
            return summate(multiply(*chs), num_node_blocks=num_node_blocks)

        root_prods = [region(list(range(num_vars))).chs[0] for _ in range(num_repetitions)]
        return summate(*root_prods, num_node_blocks=1, block_size=1)
