"""Node vectors of a probabilistic circuit: the DAG the layer compiler consumes.

A node vector is ``num_node_blocks`` blocks of ``block_size`` nodes that share one scope.
This is the minimal counterpart of PyJuice's ``CircuitNodes`` / ``InputNodes`` /
``ProdNodes`` / ``SumNodes`` (src/pyjuice/nodes/nodes.py:67-311, input_nodes.py:13-169,
prod_nodes.py:15-162, sum_nodes.py:17-420): the same attribute names (``chs``,
``edge_ids``, ``block_size``, ``num_node_blocks``, ``ch_block_size``, ``_params`` and the
``_output_ind_range`` / ``_param_range`` / ``_param_flow_range`` / ``_param_ids`` /
``_param_flow_ids`` / ``_inverse_param_ids`` write-backs of the compiler), so the compiler
accepts either these objects or PyJuice's own by duck typing.
"""
from __future__ import annotations

from collections import deque
from typing import Optional, Sequence, Union

import numpy as np
import torch

from .bitset import BitSet
from .distributions import Distribution

Tensor = Union[np.ndarray, torch.Tensor]


def as_bitset(scope) -> BitSet:
    """Accept a foreign scope object (anything with ``to_list``) as well as our own."""
    return scope if isinstance(scope, BitSet) else BitSet.from_array(scope.to_list())


def _dfs_postorder(root):
    """Children-first DFS over ``chs`` in list order, each vector once (nodes.py:13-38)."""
    seen, order = set(), []
    stack = [(root, 0)]
    seen.add(id(root))
    while stack:
        ns, i = stack[-1]
        if i < len(ns.chs):
            stack[-1] = (ns, i + 1)
            cs = ns.chs[i]
            if id(cs) not in seen:
                seen.add(id(cs))
                stack.append((cs, 0))
        else:
            order.append(ns)
            stack.pop()
    return order


def _parents_first(root):
    """Topological order, every vector after all of its parents (nodes.py:40-64)."""
    nparents = {}
    for ns in _dfs_postorder(root):
        for cs in ns.chs:
            nparents[id(cs)] = nparents.get(id(cs), 0) + 1
    out, queue = [], deque([root])
    while queue:
        ns = queue.popleft()
        out.append(ns)
        for cs in ns.chs:
            nparents[id(cs)] -= 1
            if nparents[id(cs)] == 0:
                queue.append(cs)
    return out


class CircuitNodes:
    DEFAULT_BLOCK_SIZE = 1

    def __init__(self, num_node_blocks: int, scope: BitSet, block_size: int = 0,
                 source_node: Optional["CircuitNodes"] = None, **kwargs):
        if block_size == 0:
            block_size = CircuitNodes.DEFAULT_BLOCK_SIZE
        assert num_node_blocks > 0
        assert block_size > 0 and (block_size & (block_size - 1)) == 0, \
            f"`block_size` must be a power of 2, but got `block_size={block_size}`."
        self.num_node_blocks = int(num_node_blocks)
        self.block_size = int(block_size)
        self.scope = scope
        self.chs = []
        self._output_ind_range = None
        self._param_ids = None
        self._params = None
        if source_node is not None:
            while source_node._source_node is not None:
                source_node = source_node._source_node
        self._source_node = source_node
        self._reverse_iter = False

    # kind predicates -----------------------------------------------------------------
    def is_sum(self):
        return False

    def is_prod(self):
        return False

    def is_input(self):
        return False

    # sizes -----------------------------------------------------------------------------
    @property
    def num_chs(self):
        return len(self.chs)

    @property
    def num_nodes(self):
        return self.num_node_blocks * self.block_size

    @property
    def num_vars(self):
        return len(self.scope)

    # tying -----------------------------------------------------------------------------
    def is_tied(self):
        return self._source_node is not None

    def get_source_ns(self):
        return self._source_node if self.is_tied() else self

    def provided(self, name):
        return getattr(self, name, None) is not None

    def has_params(self):
        src = self.get_source_ns()
        return getattr(src, "_params", None) is not None

    # traversal -------------------------------------------------------------------------
    def __iter__(self):
        order = _parents_first(self) if self._reverse_iter else _dfs_postorder(self)
        return iter(order)

    def __call__(self, reverse: bool = False):
        self._reverse_iter = reverse
        return self

    def __len__(self):
        return len(_dfs_postorder(self))

    def contains(self, ns):
        return any(n is ns for n in _dfs_postorder(self))

    def init_parameters(self, perturbation: float = 2.0, recursive: bool = True, **kwargs):
        """Random parameters for every untied vector that has none.

        Visit order is self first, then children in list order, each vector once — the order
        in which PyJuice consumes the torch RNG (sum_nodes.py:256-279, nodes.py:164-191), so
        the same seed gives the same stream.
        """
        if not recursive:
            self._init_own_parameters(perturbation, **kwargs)
            return
        seen = set()
        stack = [self]
        while stack:
            ns = stack.pop()
            # A sum vector re-draws its parameters every time it is reached, before the
            # visited check (sum_nodes.py:266-279 runs ahead of nodes.py:167-168).
            if ns.is_sum():
                ns._init_own_parameters(perturbation, **kwargs)
            if id(ns) in seen:
                continue
            seen.add(id(ns))
            if not ns.is_sum():
                ns._init_own_parameters(perturbation, **kwargs)
            stack.extend(reversed(ns.chs))

    def _init_own_parameters(self, perturbation, **kwargs):
        pass

    def _clear_tensor_circuit_hooks(self):
        for ns in _dfs_postorder(self):
            for name in ("_param_range", "_param_ids", "_inverse_param_ids", "_param_flow_range",
                         "_param_flow_ids", "_output_ind_range"):
                if hasattr(ns, name):
                    setattr(ns, name, None)


class InputNodes(CircuitNodes):
    def __init__(self, num_node_blocks: int, scope: Union[Sequence[int], BitSet], dist: Distribution,
                 params: Optional[torch.Tensor] = None, block_size: int = 0, **kwargs):
        if not isinstance(scope, BitSet):
            scope = BitSet.from_array(scope)
        super().__init__(num_node_blocks, scope, block_size=block_size, **kwargs)
        self.dist = dist
        self._param_initialized = False
        if params is not None:
            self.set_params(params)

    def is_input(self):
        return True

    @property
    def num_edges(self):
        return 0

    def has_params(self):
        return self._param_initialized

    def get_params(self):
        return self._params

    def set_params(self, params: torch.Tensor, normalize: bool = True):
        assert params.numel() == self.num_nodes * self.dist.num_parameters()
        params = params.reshape(-1).float()
        if normalize:
            params = self.dist.normalize_parameters(params)
        self._param_initialized = True
        self._params = params

    def duplicate(self, scope=None, tie_params: bool = False) -> "InputNodes":
        if scope is None:
            scope = self.scope
        elif isinstance(scope, int):
            scope = [scope]
        dist_cls, dist_kwargs = self.dist._get_constructor()
        ns = InputNodes(self.num_node_blocks, scope=scope, dist=dist_cls(**dist_kwargs),
                        block_size=self.block_size, source_node=self if tie_params else None)
        if self._params is not None and not tie_params:
            ns._params = self._params.clone()
        return ns

    def _init_own_parameters(self, perturbation, **kwargs):
        # input_nodes.py:134-160: a vector that already holds parameters keeps them.
        if not self.is_tied() and not self.has_params():
            self._params = self.dist.init_parameters(num_nodes=self.num_nodes, perturbation=perturbation,
                                                     params=self._params)

    def get_data_dtype(self):
        return self.dist.get_data_dtype()

    def __repr__(self):
        return f"InputNodes(num_node_blocks={self.num_node_blocks}, block_size={self.block_size}, dist={type(self.dist).__name__})"


class ProdNodes(CircuitNodes):
    SPARSE = 0
    BLOCK_SPARSE = 1

    def __init__(self, num_node_blocks: int, chs: Sequence[CircuitNodes], edge_ids: Optional[Tensor] = None,
                 block_size: int = 0, **kwargs):
        scope = BitSet()
        for c in chs:
            cscope = as_bitset(c.scope)
            assert not scope.contains_any(cscope), "Children of a `ProdNodes` should have disjoint scopes."
            scope = scope | cscope
        super().__init__(num_node_blocks, scope, block_size=block_size, **kwargs)
        self.chs = list(chs)
        if edge_ids is None:
            for c in self.chs:
                assert self.num_node_blocks == c.num_node_blocks and self.block_size == c.block_size, \
                    "Cannot create edges implicitly since # nodes do not match."
            edge_ids = torch.arange(self.num_node_blocks).unsqueeze(1).repeat(1, self.num_chs)
        if isinstance(edge_ids, np.ndarray):
            edge_ids = torch.from_numpy(edge_ids)
        edge_ids = edge_ids.long()
        assert edge_ids.dim() == 2 and edge_ids.size(1) == self.num_chs
        assert edge_ids.size(0) in (self.num_node_blocks, self.num_nodes), \
            f"Unexpected shape of `edge_ids`: {tuple(edge_ids.shape)}"
        per_block = edge_ids.size(0) == self.num_node_blocks
        for cid, c in enumerate(self.chs):
            limit = c.num_node_blocks if per_block else c.num_nodes
            assert bool((edge_ids[:, cid] >= 0).all()) and bool((edge_ids[:, cid] < limit).all()), "Edge index out of range."
        self.edge_ids = edge_ids

    def is_prod(self):
        return True

    @property
    def num_edges(self):
        return self.num_nodes * self.num_chs

    def is_block_sparse(self):
        return self.edge_ids.size(0) == self.num_node_blocks

    def is_sparse(self):
        return not self.is_block_sparse()

    def duplicate(self, *args, tie_params: bool = False):
        chs = list(args) if len(args) > 0 else self.chs
        assert len(chs) == self.num_chs
        return ProdNodes(self.num_node_blocks, chs, self.edge_ids.clone(), block_size=self.block_size,
                         source_node=self if tie_params else None)

    def __repr__(self):
        return f"ProdNodes(num_node_blocks={self.num_node_blocks}, block_size={self.block_size}, num_chs={self.num_chs})"


def normalize_ns_parameters(params: torch.Tensor, node_block_ids: torch.Tensor, pseudocount: float = 0.0,
                            ch_block_size: int = 1):
    """In place: make the parameters of every sum node sum to one.

    ``params`` is ``[E, block_size, ch_block_size]`` and ``node_block_ids[e]`` names the node
    block of block-edge ``e``; node ``(i, m)`` owns ``params[e, m, :]`` for all ``e`` with
    ``node_block_ids[e] == i`` (same result as nodes/backend/normalize.py:71-129 up to
    floating-point summation order).
    """
    nb = int(node_block_ids.max().item()) + 1
    per_edge = params.sum(dim=2)                                     # [E, bs]
    totals = torch.zeros(nb, params.size(1), dtype=params.dtype)
    totals.index_add_(0, node_block_ids, per_edge)
    if pseudocount == 0.0:
        params /= totals[node_block_ids].unsqueeze(2)
    else:
        nchs = torch.bincount(node_block_ids, minlength=nb).to(params.dtype) * ch_block_size
        scale = (per_edge + pseudocount / nchs[node_block_ids].unsqueeze(1)) / (totals[node_block_ids] + pseudocount)
        params *= (scale / torch.where(per_edge == 0.0, torch.full_like(per_edge, 1e-12), per_edge)).unsqueeze(2)


class SumNodes(CircuitNodes):
    def __init__(self, num_node_blocks: int, chs: Sequence[CircuitNodes], edge_ids: Optional[Tensor] = None,
                 params: Optional[torch.Tensor] = None, block_size: int = 0, **kwargs):
        assert len(chs) > 0, "`SumNodes` must have at least one child."
        for c in chs[1:]:
            assert c.block_size == chs[0].block_size, "`block_size` of the children of a `SumNodes` should be the same."
            assert as_bitset(c.scope) == as_bitset(chs[0].scope), "Children of a `SumNodes` should have the same scope."
        super().__init__(num_node_blocks, BitSet(as_bitset(chs[0].scope).mask), block_size=block_size, **kwargs)

        # sum_nodes.py:358-372: an input child is wrapped into a one-child product vector.
        self.chs = []
        for c in chs:
            if c.is_input():
                c = ProdNodes(c.num_node_blocks, [c], torch.arange(c.num_node_blocks).reshape(-1, 1),
                              block_size=c.block_size)
            self.chs.append(c)
        self.num_ch_node_blocks = sum(c.num_node_blocks for c in self.chs)
        self.ch_block_size = self.chs[0].block_size
        self._construct_edges(edge_ids)
        if params is not None:
            self.set_params(params, pseudocount=0.0)

    def is_sum(self):
        return True

    @property
    def num_edges(self):
        return self.edge_ids.size(1) * self.block_size * self.ch_block_size

    @property
    def num_ch_nodes(self):
        return self.num_ch_node_blocks * self.ch_block_size

    def _construct_edges(self, edge_ids):
        nb, ncb = self.num_node_blocks, self.num_ch_node_blocks
        if edge_ids is None:
            edge_ids = torch.stack((torch.arange(nb).repeat_interleave(ncb), torch.arange(ncb).repeat(nb)), dim=0)
        if isinstance(edge_ids, np.ndarray):
            edge_ids = torch.from_numpy(edge_ids)
        if edge_ids.dtype == torch.bool:
            assert edge_ids.shape == (nb, ncb)
            x, y = torch.where(edge_ids)
            edge_ids = torch.stack((x, y), dim=0)
        edge_ids = edge_ids.long()
        assert edge_ids.dim() == 2 and edge_ids.size(0) == 2, "Expect `edge_ids.size(0) == 2`."
        assert bool((edge_ids >= 0).all()), "Edge index underflow."
        assert bool((edge_ids[0] < nb).all()) and bool((edge_ids[1] < ncb).all()), "Edge index overflow."
        assert torch.unique(edge_ids[0]).numel() == nb, "Some node has no edge."
        self.edge_ids = edge_ids

    def get_params(self):
        return self._params

    def set_params(self, params: torch.Tensor, normalize: bool = True, pseudocount: float = 0.0):
        """Accepts ``[E]`` (blocks of 1), ``[num_nodes, num_ch_nodes]``, ``[E, bs, ch_bs]`` or
        ``[num_node_blocks, num_ch_node_blocks, bs, ch_bs]`` (sum_nodes.py:183-228)."""
        if self._source_node is not None:
            return self._source_node.set_params(params, normalize=normalize, pseudocount=pseudocount)
        bs, cbs, nb, ncb = self.block_size, self.ch_block_size, self.num_node_blocks, self.num_ch_node_blocks
        params = params.float()
        if params.dim() == 1:
            assert bs == 1 and cbs == 1 and params.size(0) == self.edge_ids.size(1)
            p = params.clone().view(-1, 1, 1)
        elif params.dim() == 2:
            assert params.shape == (self.num_nodes, ncb * cbs)
            full = params.reshape(nb, bs, ncb, cbs).permute(0, 2, 1, 3)
            p = full[self.edge_ids[0], self.edge_ids[1]].clone().contiguous()
        elif params.dim() == 3:
            assert params.shape == (self.edge_ids.size(1), bs, cbs)
            p = params.clone()
        elif params.dim() == 4:
            assert params.shape == (nb, ncb, bs, cbs)
            p = params[self.edge_ids[0], self.edge_ids[1]].clone().contiguous()
        else:
            raise ValueError("Unsupported parameter input.")
        if normalize:
            normalize_ns_parameters(p, self.edge_ids[0], pseudocount=pseudocount, ch_block_size=cbs)
        self._params = p

    def _init_own_parameters(self, perturbation, **kwargs):
        if self._source_node is None:
            self._params = torch.exp(torch.rand([self.edge_ids.size(1), self.block_size, self.ch_block_size]) * -perturbation)
            normalize_ns_parameters(self._params, self.edge_ids[0], ch_block_size=self.ch_block_size)
        else:
            self._params = None

    def duplicate(self, *args, tie_params: bool = False) -> "SumNodes":
        chs = list(args) if len(args) > 0 else self.chs
        assert len(chs) == self.num_chs, f"Number of new children ({len(chs)}) must match the number of original children ({self.num_chs})."
        for old_c, new_c in zip(self.chs, chs):
            assert old_c.num_node_blocks == new_c.num_node_blocks and old_c.block_size == new_c.block_size, "Child node size not match."
        params = self._params.clone() if (self._params is not None and not tie_params) else None
        return SumNodes(self.num_node_blocks, chs, self.edge_ids.clone(), params=params, block_size=self.block_size,
                        source_node=self if tie_params else None)

    # parameter exchange with a compiled circuit (sum_nodes.py:283-350) ------------------
    def update_parameters(self, params: torch.Tensor, clone: bool = True):
        assert self.provided("_param_range"), "The `SumNodes` has not been compiled into a `TensorCircuit`."
        if self.is_tied():
            return
        s, e = self._param_range
        flat = params[s:e].detach().cpu()
        flat = flat.clone() if clone else flat
        local = (self._param_ids - s) // (self.block_size * self.ch_block_size)
        self._params = flat.reshape(local.size(0), self.ch_block_size, self.block_size)[local].permute(0, 2, 1)

    def update_param_flows(self, param_flows: torch.Tensor, origin_ns_only: bool = True, clone: bool = True):
        assert self.provided("_param_flow_range"), "The `SumNodes` has not been compiled into a `TensorCircuit`."
        if origin_ns_only and self.is_tied():
            return
        s, e = self._param_flow_range
        flat = param_flows[s:e].detach().cpu()
        flat = flat.clone() if clone else flat
        local = (self._param_flow_ids - s) // (self.block_size * self.ch_block_size)
        self._param_flows = flat.reshape(local.size(0), self.ch_block_size, self.block_size)[local].permute(0, 2, 1)

    def gather_parameters(self, params: torch.Tensor):
        assert self.provided("_param_range"), "The `SumNodes` has not been compiled into a `TensorCircuit`."
        if self.is_tied() or not self.has_params():
            return
        s, e = self._param_range
        params[s:e] = self._params[self._inverse_param_ids].permute(0, 2, 1).reshape(-1).to(params.device)

    def __repr__(self):
        return (f"SumNodes(num_node_blocks={self.num_node_blocks}, block_size={self.block_size}, "
                f"num_chs={self.num_chs}, num_edges={self.num_edges})")
