"""``inputs`` / ``multiply`` / ``summate`` / ``set_block_size``: the node-construction front door.

Same call signatures as PyJuice's helpers (src/pyjuice/nodes/construction.py:24-231), limited
to what the compiled forward/backward/EM path consumes (no external parameters, no edge-pattern
constructors).
"""
from __future__ import annotations

from typing import Optional, Sequence, Union

import torch

from .distributions import Distribution
from .nodes import CircuitNodes, InputNodes, ProdNodes, SumNodes


def _resolve_blocks(num_node_blocks: int, num_nodes: int, block_size: int):
    assert block_size == 0 or block_size & (block_size - 1) == 0, "`block_size` must be a power of 2."
    if num_nodes > 0:
        assert num_node_blocks == 0, "Only one of `num_nodes` and `num_node_blocks` can be set at the same time."
        if block_size == 0:
            block_size = CircuitNodes.DEFAULT_BLOCK_SIZE
        assert num_nodes % block_size == 0
        num_node_blocks = num_nodes // block_size
    return num_node_blocks, block_size


def inputs(var: Union[int, Sequence[int]], num_node_blocks: int = 0, dist: Optional[Distribution] = None,
           params: Optional[torch.Tensor] = None, num_nodes: int = 0, block_size: int = 0, **kwargs) -> InputNodes:
    """A vector of input nodes over variable ``var`` with leaf distribution ``dist``."""
    assert dist is not None, "`dist` must be given."
    num_node_blocks, block_size = _resolve_blocks(num_node_blocks, num_nodes, block_size)
    return InputNodes(num_node_blocks, [var] if isinstance(var, int) else list(var), dist,
                      params=params, block_size=block_size, **kwargs)


def multiply(nodes1: CircuitNodes, *args, edge_ids: Optional[torch.Tensor] = None, sparse_edges: bool = False,
             **kwargs) -> ProdNodes:
    """A vector of product nodes over children with disjoint scopes.

    ``edge_ids[i, j]`` is the block of child ``j`` that product block ``i`` multiplies; without it
    block ``i`` pairs block ``i`` of every child.
    """
    chs = [nodes1, *args]
    for c in chs:
        assert c.is_input() or c.is_sum(), "Children of product nodes must be input or sum nodes."
        assert c.block_size == nodes1.block_size, "Children of a product vector must share one block size."
    num_node_blocks, block_size = nodes1.num_node_blocks, nodes1.block_size
    if edge_ids is not None:
        if sparse_edges:
            assert edge_ids.shape[0] % block_size == 0
            num_node_blocks = edge_ids.shape[0] // block_size
        else:
            num_node_blocks = edge_ids.shape[0]
    else:
        for c in chs:
            assert c.num_node_blocks == num_node_blocks, "Children should have the same `num_node_blocks`."
    return ProdNodes(num_node_blocks, chs, edge_ids, block_size=block_size, **kwargs)


def summate(nodes1: CircuitNodes, *args, num_node_blocks: int = 0, num_nodes: int = 0,
            edge_ids: Optional[torch.Tensor] = None, block_size: int = 0, **kwargs) -> SumNodes:
    """A vector of sum nodes over children of one scope; fully connected unless ``edge_ids``
    (``[2, E]`` pairs of (sum block, child block)) says otherwise."""
    num_node_blocks, block_size = _resolve_blocks(num_node_blocks, num_nodes, block_size)
    chs = [nodes1, *args]
    for c in chs:
        assert c.is_input() or c.is_prod(), "Children of sum nodes must be input or product nodes."
    if edge_ids is not None and num_node_blocks == 0:
        num_node_blocks = int(edge_ids[0, :].max().item()) + 1
    assert num_node_blocks > 0, "Number of node blocks should be greater than 0."
    return SumNodes(num_node_blocks, chs, edge_ids, block_size=block_size, **kwargs)


class set_block_size:
    """Context manager: default ``block_size`` of nodes built inside the ``with`` body."""

    def __init__(self, block_size: int = 1):
        assert block_size & (block_size - 1) == 0, "`block_size` must be a power of 2."
        self.block_size = block_size
        self._saved = None

    def __enter__(self):
        self._saved = CircuitNodes.DEFAULT_BLOCK_SIZE
        CircuitNodes.DEFAULT_BLOCK_SIZE = self.block_size

    def __exit__(self, *exc):
        CircuitNodes.DEFAULT_BLOCK_SIZE = self._saved
        return False
