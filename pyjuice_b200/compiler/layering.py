"""Depth layering of the node DAG (PyJuice: model/tensorcircuit.py:2036-2120).

Input vectors sit at depth 0; a product vector one above its deepest child; a sum vector at the
depth of its deepest child.  A sum vector with a shallower product child gets an identity
sum + product pair spliced in so that every product layer only feeds the sum layer right above
it.  The splice **mutates** ``ns.chs`` of the caller's DAG, exactly as the reference does.
"""
from __future__ import annotations

import sys
from typing import Dict, List

import torch

from ..nodes import multiply, summate


def create_node_layers(root_ns):
    depth2nodes: Dict[int, Dict[str, List]] = {}
    depth_of: Dict[int, int] = {}
    state = dict(num_layers=1, max_node_bs=0, max_ele_bs=0)

    def visit(ns):
        """Post-visit bookkeeping of one vector whose children all have depths."""
        if ns.is_input():
            depth_of[id(ns)] = 0
            depth2nodes.setdefault(0, {"input": []})["input"].append(ns)
            return
        depth = max(depth_of[id(c)] for c in ns.chs) + (1 if ns.is_prod() else 0)
        state["num_layers"] = max(depth + 1, state["num_layers"])
        depth_of[id(ns)] = depth
        if depth not in depth2nodes:
            depth2nodes[depth] = {"sum": [], "prod": []}
        if ns.is_sum():
            for k, cs in enumerate(ns.chs):
                cd = depth_of[id(cs)]
                if cd < depth:
                    eye = torch.eye(cs.block_size)[None, :, :].repeat(cs.num_node_blocks, 1, 1)
                    pass_sum = summate(cs, num_node_blocks=cs.num_node_blocks, block_size=cs.block_size,
                                       edge_ids=torch.arange(0, cs.num_node_blocks)[None, :].repeat(2, 1),
                                       params=eye)
                    pass_prod = multiply(pass_sum)
                    ns.chs[k] = pass_prod
                    depth2nodes[cd]["sum"].append(pass_sum)
                    depth_of[id(pass_sum)] = cd
                    depth_of[id(pass_prod)] = depth
            depth2nodes[depth]["sum"].append(ns)
            state["max_node_bs"] = max(state["max_node_bs"], ns.block_size)
        elif ns.is_prod():
            state["max_ele_bs"] = max(state["max_ele_bs"], ns.block_size)
        else:
            raise NotImplementedError(f"Unsupported node type {type(ns)}.")

    # iterative post-order DFS over `chs` in list order, memoised by identity
    stack = [(root_ns, 0)]
    entered = {id(root_ns)}
    while stack:
        ns, i = stack[-1]
        chs = [] if ns.is_input() else ns.chs
        if i < len(chs):
            stack[-1] = (ns, i + 1)
            cs = chs[i]
            if id(cs) not in entered:
                entered.add(id(cs))
                stack.append((cs, 0))
        else:
            visit(ns)
            stack.pop()

    claimed: Dict[int, int] = {}
    for layer in range(1, len(depth2nodes)):
        for ns in depth2nodes[layer]["sum"]:
            for cs in ns.chs:
                if cs.is_prod():
                    if id(cs) in claimed:
                        assert claimed[id(cs)] == layer, \
                            "Disallowed circumstance: a product node requested by sum nodes at different layers."
                    else:
                        depth2nodes[layer]["prod"].append(cs)
                        claimed[id(cs)] = layer
    return depth2nodes, state["num_layers"], state["max_node_bs"], state["max_ele_bs"]
