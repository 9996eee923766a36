"""``TensorCircuit``: a compiled probabilistic circuit and the driver of its forward / backward / EM passes.

Public surface and semantics follow PyJuice's ``TensorCircuit`` / ``compile``
(model/tensorcircuit.py:201-471 forward, 473-687 backward, 1346-1387 mini_batch_em,
1394-1471 flows init / DDP sync, 1479-1654 accessors, 1801-2030 layer construction and parameter
initialisation).  What differs is underneath: layers launch hand-written CUDA kernels through a C
ABI, the inner-layer loops of forward and backward are replayed from CUDA graphs, buffers are
initialised once instead of being memset on every pass, and the DDP synchronisation is a single
all-reduce over one packed flow arena.

Buffers (fp32, batch innermost):
    node_mars      [num_nodes, B]     log-values of input and sum nodes; rows < num_dummy_nodes stay 0
    element_mars   [num_elements, B]  log-values of product nodes, shared by all product layers; dummy rows -inf
    node_flows     [num_nodes, B]     log-flows; reset to -inf at the start of every backward pass
    element_flows  [num_elements, B]  log-flows of product nodes
"""
from __future__ import annotations

import contextlib
import functools
import os
from functools import partial
from typing import Optional, Sequence, Union

import numpy as np
import torch
import torch.nn as nn

from . import _lib
from .compiler import _IdDict, compile_cum_par_flows, compile_par_update, create_node_layers
from .layers import InputLayer, LayerGroup, ParamPacker, ProdLayer, SumLayer, _alg_of, _fill, _scale, _unsupported
from .flows import FlowArena
from .nodes import as_bitset

NEG_INF = float("-inf")


def _pc_model_backward_hook(grad, pc, inputs, **kwargs):
    """Autograd hook on the returned log-likelihoods: ``lls.mean().backward()`` (or any other scalar
    loss) triggers the circuit's own backward pass with per-sample weights grad / sum(grad) * B
    (model/tensorcircuit.py:28-41)."""
    grad = grad.permute(1, 0)
    pc.backward(inputs=inputs, ll_weights=grad / grad.sum() * grad.size(1),
                compute_param_flows=pc._optim_hyperparams["compute_param_flows"],
                flows_memory=pc._optim_hyperparams["flows_memory"], **kwargs)
    return None


def _in_own_mode(fn):
    """Run a public method in the circuit's own arithmetic mode (``self.sum_mode``; None = the process default).
    A pass under another propagation rule ("MPE", "GeneralLL") runs on the plain fp32 kernels (mode 0: nothing is
    folded or fused), with the rule kept in ``self._alg`` for the duration of the call."""
    @functools.wraps(fn)
    def wrapper(self, *args, **kwargs):
        mode, prev = self.sum_mode, self._alg
        if fn.__name__ in ("forward", "backward"):
            name = kwargs.get("propagation_alg")
            if name is None:
                name = self.default_propagation_alg if fn.__name__ == "forward" else "LL"
                if fn.__name__ == "forward":
                    kwargs = {**self.propagation_alg_kwargs, **kwargs}
            if not isinstance(name, str):
                raise NotImplementedError("one propagation rule per layer is outside the compiled path")
            self._alg = _alg_of(name, kwargs)
            kwargs["propagation_alg"] = name
            if self._alg[0] != 0:
                mode = 0
        try:
            if mode is None:
                return fn(self, *args, **kwargs)
            with _lib.use_sum_mode(mode):
                return fn(self, *args, **kwargs)
        finally:
            self._alg = prev
    return wrapper


class TensorCircuit(nn.Module):
    def __init__(self, root_ns, layer_sparsity_tol: float = 0.5, max_num_partitions: Optional[int] = None,
                 disable_gpu_compilation: bool = False, force_gpu_compilation: bool = False,
                 max_tied_ns_per_parflow_block: int = 32, device=None, verbose: bool = True):
        super().__init__()
        self.root_ns = root_ns
        self.device = torch.device("cpu")
        scope = as_bitset(root_ns.scope).to_list()
        self.num_vars = (max(scope) + 1) if scope else 0

        self.node_mars = self.element_mars = self.node_flows = self.element_flows = None
        self.param_flows = None
        self._init_layers(layer_sparsity_tol, max_num_partitions, max_tied_ns_per_parflow_block)

        self._optim_hyperparams = {"compute_param_flows": True, "flows_memory": 1.0}
        self._graphs = {}
        self.use_cuda_graphs = True
        self.use_dataflow_launch = True       # runs of folded depths as one launch (tiles wait on counters)
        self.use_side_stream = True           # independent kernels of a step share the device (two streams)
        self.debug_poison = False             # fill value / flow buffers with NaN before every pass (see `assert_no_poison`)
        self.use_nvtx = bool(os.environ.get("PCX_B200_NVTX"))     # NVTX ranges around the phases of a step (profilers)
        self.sum_mode = None                  # this circuit's arithmetic (0, 1 or 2 as `_lib.set_sum_mode`); None = default
        self.chain_tile = None                # tile width of that launch in samples (16 / 32 / 64); None = choose
        self.dense_par_max_bytes = 16 << 30   # operand buffers of the dense parameter-flow product (all groups)
        self.default_propagation_alg = "LL"        # "LL", "MPE" or "GeneralLL" (see `set_propagation_alg`)
        self.propagation_alg_kwargs = dict()
        self._alg = (0, 0.0)                        # rule of the pass in progress: (id, alpha)
        self._run_params = {}
        self._cum_flow_host = 0.0
        self._cum_flow_dev = None
        self._eflow_mode = 1
        self._reference_compat = False

    @property
    def reference_compat(self) -> bool:
        """False (default): flows are the exact gradients.  True: reproduce two behaviours of the reference's kernels
        that change results beyond rounding.  (1) A product node without a sum parent at its depth (block-sparse sum
        vectors, e.g. Poon-Domingos circuits) hands down whatever its row of the shared element-flow buffer holds —
        the flow of a product with the same element id at a depth processed earlier in the pass, or nothing — because
        the reference clears that buffer once per backward pass only (model/tensorcircuit.py:526-528) while its
        backward tables skip child blocks without parents (layer/sum_layer.py:273-275).  (2) The tied-flow fusing
        kernel adds ``param_flows[0:n]`` once per padding slot when a tied sum vector owns a number of flow
        accumulators that is not a power of two (model/backend/parflow_fusing.py:50, 86-87).  In this mode the backward
        sweep keeps product layers as kernels of their own (element flows go through the shared buffer)."""
        return self._reference_compat

    @reference_compat.setter
    def reference_compat(self, on: bool):
        self._reference_compat = bool(on)
        self._graphs = {}
        self._chain_cache, self._par_job_cache, self._dense_par_cache = {}, {}, {}
        for group in self.inner_layer_groups:
            if group.is_prod():
                for layer in group:
                    layer._raw_backward_tables = bool(on)

    # ------------------------------------------------------------------------------------------
    # construction
    # ------------------------------------------------------------------------------------------
    def _init_layers(self, layer_sparsity_tol, max_num_partitions, max_tied):
        self.root_ns._clear_tensor_circuit_hooks()
        pc_num_vars = len(as_bitset(self.root_ns.scope))
        depth2nodes, num_layers, max_node_bs, max_ele_bs = create_node_layers(self.root_ns)

        self.num_dummy_nodes = max_ele_bs
        self.num_dummy_eles = max_node_bs
        self.num_dummy_params = max_node_bs * max_ele_bs
        num_nodes, num_edges, num_elements = self.num_dummy_nodes, 0, self.num_dummy_eles
        num_params, num_param_flows = self.num_dummy_params, 0
        node2tiednodes = _IdDict()

        self.input_layer_group = None
        self.inner_layer_groups = []
        layer_id = 0
        for depth in range(num_layers):
            if depth == 0:
                by_sig = {}
                for ns in depth2nodes[0]["input"]:
                    by_sig.setdefault(ns.dist.get_signature(), []).append(ns)
                layers = []
                for nodes in by_sig.values():
                    layer = InputLayer(nodes, cum_nodes=num_nodes, pc_num_vars=pc_num_vars,
                                       max_tied_ns_per_parflow_block=max_tied)
                    num_nodes += layer.num_nodes
                    layers.append(layer)
                self.input_layer_group = LayerGroup(layers)
                continue

            assert len(depth2nodes[depth]["prod"]) > 0 and len(depth2nodes[depth]["sum"]) > 0, \
                f"Depth {depth}: (# prod nodes: {len(depth2nodes[depth]['prod'])}, # sum nodes: {len(depth2nodes[depth]['sum'])})"

            by_bs = {}
            for ns in depth2nodes[depth]["prod"]:
                by_bs.setdefault(ns.block_size, []).append(ns)
            layer_num_elements = max_node_bs          # element ids restart at every depth
            prod_layers = []
            for nodes in by_bs.values():
                layer = ProdLayer(nodes, global_nid_start=layer_num_elements, layer_sparsity_tol=layer_sparsity_tol,
                                  max_num_partitions=max_num_partitions)
                layer_num_elements += layer.num_nodes
                num_edges += layer.num_edges
                prod_layers.append(layer)
            group = LayerGroup(prod_layers)
            self.inner_layer_groups.append(group)
            self.add_module(f"prod_layer_{layer_id}", group)
            num_elements = max(num_elements, layer_num_elements)

            by_bs = {}
            for ns in depth2nodes[depth]["sum"]:
                by_bs.setdefault(ns.block_size, []).append(ns)
            sum_layers = []
            for nodes in by_bs.values():
                layer = SumLayer(nodes, global_nid_start=num_nodes, global_pid_start=num_params,
                                 global_pfid_start=num_param_flows, node2tiednodes=node2tiednodes,
                                 layer_sparsity_tol=layer_sparsity_tol, max_num_partitions=max_num_partitions,
                                 max_tied_ns_per_parflow_block=max_tied)
                num_nodes += layer.num_nodes
                num_edges += layer.num_edges
                num_params += layer.num_parameters
                num_param_flows += layer.num_param_flows
                sum_layers.append(layer)
            group = LayerGroup(sum_layers)
            self.inner_layer_groups.append(group)
            self.add_module(f"sum_layer_{layer_id}", group)
            layer_id += 1

        self.num_nodes, self.num_edges, self.num_elements = num_nodes, num_edges, num_elements
        self.num_sum_params, self.num_param_flows = num_params, num_param_flows
        self.parflow_fusing_kwargs = compile_cum_par_flows(node2tiednodes)
        # (first flow, length, accumulator starts) of every tied sum source that owns more than one accumulator
        self._tied_sum_groups = [(src._param_flow_range[0], src._param_flow_range[1] - src._param_flow_range[0],
                                  [c._param_flow_range[0] for c in item[0]])
                                 for src, item in node2tiednodes.items() if len(item[0]) > 1]
        self.par_update_kwargs = compile_par_update(self.root_ns)
        self._em_blocks = self._compile_em_blocks()
        self._parentless = self._find_parentless_products()
        self.num_root_nodes = self.root_ns.num_nodes
        self._root_node_range = (self.num_nodes - self.num_root_nodes, self.num_nodes)
        self._init_parameters()

    def _find_parentless_products(self):
        """Element ranges of the product groups that hold a node without any sum parent in the group above.

        Block-sparse sum vectors (e.g. PD with a cap on connections per block) may list a product vector as a child
        without connecting every one of its blocks.  Such a product has flow zero, but its row of the shared
        ``element_flows`` buffer is never written by the element-flow kernels of that depth, and the product backward
        pass, whose tables list every product of the layer (layer/compilation.py:980-1040), would hand the row's
        stale content — the flow of another depth's product with the same element id — down to the children.  The
        reference resets the buffer once per backward pass only (model/tensorcircuit.py:526-528), so it has this
        defect; here the kernels' copies of the product backward tables skip such products (and `get_node_flows`
        resets their rows before reading), which makes the flows the true gradients (checked against autograd in
        tests/test_oracle_pins.py)."""
        out = {}
        groups = self.inner_layer_groups
        for gi in range(0, len(groups) - 1, 2):
            lo = min(l._layer_nid_range[0] for l in groups[gi])
            hi = max(l._layer_nid_range[1] for l in groups[gi])
            has_parent = torch.zeros(hi, dtype=torch.bool)
            for layer in groups[gi + 1]:
                for chids, cbs in zip(layer.partitioned_chids, layer.cs_block_sizes):
                    rows = (chids.cpu()[:, None] + torch.arange(cbs)[None, :]).reshape(-1)
                    has_parent[rows] = True
            exists = torch.zeros(hi, dtype=torch.bool)
            for layer in groups[gi]:
                for nids in layer.partitioned_nids:
                    rows = (nids.cpu()[:, None] + torch.arange(layer.block_size)[None, :]).reshape(-1)
                    exists[rows] = True
            orphan = exists & ~has_parent
            if bool(orphan.any()):
                out[gi] = (lo, hi, orphan)
        return out

    def _reset_parentless(self, prod_gi: int, logspace_flows: bool):
        rng = self._parentless.get(prod_gi)
        if rng is not None:
            _fill(self.element_flows[rng[0]:rng[1]], NEG_INF if logspace_flows else 0.0)

    def _mask_parentless_in_device_tables(self):
        """The kernels' copies of the product layers' backward tables skip parentless products (id 0 = padding), so
        the backward sweep needs no reset of the element-flow buffer; the public tables stay as compiled."""
        for gi, (lo, hi, orphan) in self._parentless.items():
            for layer in self.inner_layer_groups[gi]:
                if layer._dev is None:
                    continue
                bk = []
                layer._dev["bk_raw"] = list(layer._dev["bk"])          # as compiled (`reference_compat`)
                for u_cids, parids in layer._dev["bk"]:
                    p = parids.long().cpu()
                    dead = orphan[p.clamp(max=hi - 1)] & (p != 0)
                    bk.append((u_cids, torch.where(dead, torch.zeros_like(p), p).to(torch.int32).to(parids.device)))
                layer._dev["bk"] = bk

    def _compile_em_blocks(self):
        """Per node block of every untied sum vector: first parameter, first flow, real fan-in, block size —
        the compact form of the per-(node, 32-edge chunk) items of ``par_update_kwargs`` that the EM kernel
        walks (flows are read through the vector's own flow range, i.e. the source accumulator)."""
        par, flow, fan, bsz = [], [], [], []
        for ns in self.root_ns:
            if not ns.is_sum() or ns.is_tied():
                continue
            cnt = torch.bincount(ns.edge_ids[0], minlength=ns.num_node_blocks) * ns.ch_block_size
            off = torch.cumsum(cnt * ns.block_size, 0) - cnt * ns.block_size
            par.append(ns._param_range[0] + off)
            flow.append(ns._param_flow_range[0] + off)
            fan.append(cnt)
            bsz.append(torch.full_like(cnt, ns.block_size))
        cat = lambda lst, dt: torch.cat(lst).to(dt).contiguous()
        return dict(par=cat(par, torch.int64), flow=cat(flow, torch.int64), fan=cat(fan, torch.int32),
                    bs=cat(bsz, torch.int32), max_bs=int(max(int(b.max()) for b in bsz)))

    def _init_parameters(self, perturbation: float = 4.0, pseudocount: float = 0.0):
        """Sum parameters start as exp(-perturbation * U) unless the node vectors carry parameters; then they are
        normalised per sum node (model/tensorcircuit.py:2008-2030, model/backend/normalize.py:103-154)."""
        for ns in self.root_ns:
            if not ns.is_tied() and (ns.is_sum() or ns.is_input()) and not ns.has_params():
                ns.init_parameters(perturbation=perturbation, recursive=False)
        params = torch.exp(torch.rand([self.num_sum_params]) * -perturbation)
        params[:self.num_dummy_params] = 0.0
        for ns in self.root_ns:
            if ns.is_sum() and not ns.is_tied() and ns.has_params():
                ns.gather_parameters(params)
        self._normalize_parameters(params, pseudocount)
        self.params = nn.Parameter(params, requires_grad=False)
        for layer in self.input_layer_group:
            layer._init_parameters(perturbation)

    def _normalize_parameters(self, params: torch.Tensor, pseudocount: float = 0.0):
        eb = self._em_blocks
        for i in range(eb["par"].numel()):
            p0, fan, bs = int(eb["par"][i]), int(eb["fan"][i]), int(eb["bs"][i])
            tile = params[p0:p0 + fan * bs].view(fan, bs)
            tile.copy_((tile + pseudocount / fan) / (tile.sum(dim=0, keepdim=True) + pseudocount))

    # ------------------------------------------------------------------------------------------
    # device placement and buffers
    # ------------------------------------------------------------------------------------------
    def to(self, device):
        device = torch.device(f"cuda:{device}") if isinstance(device, int) else torch.device(device)
        if device.type == "cuda":
            _lib.load()                                   # fail here, loudly, if the kernels are not built
        nn.Module.to(self, device)
        self.input_layer_group.to(device)
        self._packer = ParamPacker(device) if device.type == "cuda" else None
        for group in self.inner_layer_groups:
            if group.is_sum():
                group.to(device, packer=self._packer)
            else:
                group.to(device)
        self.device = device
        self.parflow_fusing_kwargs = [[a.to(device), b.to(device), c.to(device), G, M]
                                      for a, b, c, G, M in self.parflow_fusing_kwargs]
        self.par_update_kwargs = [t.to(device) if isinstance(t, torch.Tensor) else t for t in self.par_update_kwargs]
        self._em_dev = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in self._em_blocks.items()}
        self._fusing_dev = [(start, n, torch.tensor(accs, dtype=torch.int64, device=device))
                            for start, n, accs in self._tied_sum_groups]
        for name in ("node_mars", "element_mars", "node_flows", "element_flows", "param_flows"):
            setattr(self, name, None)
        if device.type == "cuda":
            self._mask_parentless_in_device_tables()
        self._setup_fusion()
        self._side_stream = torch.cuda.Stream(device=device) if device.type == "cuda" else None
        self._bk_par_pending = {}
        self._graphs = {}
        self._par_job_cache = {}
        self._chain_cache = {}
        self._dense_par_cache = {}
        self._cum_flow_dev = None
        return self

    def _setup_fusion(self):
        """Decide, per depth, whether the product layer can be folded into the sum kernels above it.

        Folding needs: every sum layer of the depth on the tensor-core path (block size a multiple of 128), at most 8
        children per product node, and little duplication (an element read by few row tiles — otherwise the product
        kernel, which computes each element once, is cheaper).  `direct` additionally requires every child row of the
        depth's products to have exactly one parent product in the whole circuit: then the element-flow kernel can
        store flows straight into node_flows and the product backward kernel disappears as well."""
        self._fused = {}
        self.fuse_product_layers = getattr(self, "fuse_product_layers", True)
        if self.device.type != "cuda":
            return
        dev = self.device
        parents = torch.zeros(self.num_nodes + 1, dtype=torch.int32)
        for group in self.inner_layer_groups:
            if group.is_prod():
                for layer in group:
                    j = torch.arange(layer.block_size)
                    for cids in layer.partitioned_cids:
                        c = cids.cpu()
                        rows = (c[c != 0][:, None] + j[None, :]).reshape(-1)
                        parents.index_add_(0, rows, torch.ones_like(rows, dtype=torch.int32))
        for gi in range(1, len(self.inner_layer_groups), 2):
            pgroup, sgroup = self.inner_layer_groups[gi - 1], self.inner_layer_groups[gi]
            big = all(l.block_size % 128 == 0 and l._packer is not None and all(b is not None for b in l._packed_fw)
                      and all(b is not None for b in l._packed_bk) for l in sgroup)
            # small blocks (sample-major tiles): products of at most two children can be folded in as well
            small = (not big) and all(l._packer is not None and getattr(l, "_sm_fw", None) is not None
                                      and all(t is not None for t in l._sm_fw) and all(t is not None for t in l._sm_bk)
                                      for l in sgroup)
            if not (big or small):
                continue
            C = max(int((c != 0).sum(dim=1).max()) for l in pgroup for c in l.partitioned_cids)
            if C > (8 if big else 2):
                continue
            fc = 2 if small else (4 if C <= 4 else 8)
            n_ele = max(l._layer_nid_range[1] for l in pgroup)
            children = torch.zeros(n_ele, fc, dtype=torch.int32)
            for layer in pgroup:
                j = torch.arange(layer.block_size)
                for nids, cids in zip(layer.partitioned_nids, layer.partitioned_cids):
                    nids, cids = nids.cpu(), cids.cpu()
                    rows = (nids[:, None] + j[None, :]).reshape(-1)                      # element ids
                    if cids.size(1) < fc:
                        cids = torch.nn.functional.pad(cids, (0, fc - cids.size(1)))
                    ch = (cids[:, None, :fc] + j[None, :, None]) * (cids[:, None, :fc] != 0)
                    children[rows] = ch.reshape(-1, fc).to(torch.int32)
            used = (children != 0).any(dim=1).sum().item()
            if big:
                reads = sum(int(l.block_size // 128) * int((c != 0).sum()) for l in sgroup for c in l.partitioned_cids)
            else:                                           # every merged row gathers each of its entries once per tile
                reads = sum(int((c.cpu()[first.long().cpu()] != 0).sum()) for l in sgroup
                            for c, lists in zip(l.partitioned_cids, l._sm_fw) for _, first, _, _ in lists)
            # deep tables run on the wide-tile dense kernels, whose operand pre-pass computes every product once per
            # group of rows: folding costs them nothing, whatever the duplication
            lo_d, hi_d = SumLayer.DENSE_MIN_DEPTH, SumLayer.DENSE_WIDE_MAX_DEPTH
            dense = big and all(lo_d <= c.size(1) <= hi_d for l in sgroup for c in l.partitioned_cids) and \
                all(lo_d <= pr.size(1) * l.block_size <= hi_d for l in sgroup for pr in l.partitioned_parids)
            if used == 0 or (reads > 2 * used and not dense):
                continue
            dense = dense and reads > 2 * used              # tables the tile-at-a-time kernels handle well stay there
            ch_rows = children[children != 0].long()
            direct = big and bool((parents[ch_rows] == 1).all())
            for layer in sgroup:
                fw = [children[c.cpu()].contiguous().to(dev) for c in layer.partitioned_cids]
                bk = []
                for chids, cbs in zip(layer.partitioned_chids, layer.cs_block_sizes):
                    rows = chids.cpu()[:, None] + torch.arange(cbs)[None, :]
                    bk.append(children[rows].contiguous().to(dev))
                layer._fusion = dict(fc=fc, fw=fw, bk=bk, direct=direct, sm=small, dense=dense)
            self._fused[gi] = dict(fc=fc, direct=direct, sm=small, dense=dense,
                                   child_rows=torch.unique(ch_rows) if not direct else None)
        # rows of node_flows that still need the -inf / 0 reset each pass: children of every depth that is not
        # handled by direct stores (those are accumulated into with logaddexp)
        need = torch.zeros(self.num_nodes + 1, dtype=torch.bool)
        for gi in range(0, len(self.inner_layer_groups), 2):
            if self._fused.get(gi + 1, {}).get("direct", False):
                continue
            for layer in self.inner_layer_groups[gi]:
                j = torch.arange(layer.block_size)
                for u in layer.partitioned_u_cids:
                    need[(u.cpu()[:, None] + j[None, :]).reshape(-1)] = True
        idx = torch.nonzero(need).reshape(-1)
        self._flow_reset_ranges = None
        if idx.numel() > 0:
            breaks = torch.nonzero(idx[1:] != idx[:-1] + 1).reshape(-1) + 1
            starts = torch.cat([idx[:1], idx[breaks]])
            ends = torch.cat([idx[breaks - 1], idx[-1:]]) + 1
            if starts.numel() <= 16:
                self._flow_reset_ranges = list(zip(starts.tolist(), ends.tolist()))
        else:
            self._flow_reset_ranges = []
        covered = torch.zeros(self.num_nodes + 1, dtype=torch.bool)
        for gi, info in self._fused.items():
            if info["direct"]:
                for layer in self.inner_layer_groups[gi]:
                    for t in layer._fusion["bk"]:
                        covered[t.cpu().long().reshape(-1)] = True
        r0, r1 = self._root_node_range
        covered[r0:r1] = True
        covered[:self.num_dummy_nodes] = True
        covered[self.num_nodes] = True
        # a full reset can only be skipped when every row is either rewritten by a direct store or reset explicitly
        if self._flow_reset_ranges is not None and not bool((covered | need).all()):
            self._flow_reset_ranges = None

    def _require_cuda(self):
        if self.device.type != "cuda":
            raise NotImplementedError("the compiled circuit runs on CUDA only; call `pc.to('cuda:0')` first "
                                      "(there is no CPU path)")

    def _ensure_buffers(self, B: int, backward: bool = False):
        """(Re)allocate the value buffers when the batch size changes.  Dummy rows are written here once:
        every other row is fully overwritten by the layer that owns it on each pass."""
        if self.node_mars is None or self.node_mars.size(1) != B:
            self.node_mars = torch.zeros(self.num_nodes, B, device=self.device)
            self.element_mars = torch.full((self.num_elements, B), NEG_INF, device=self.device)
            self.node_flows = self.element_flows = None
            self._graphs = {}
        if backward and (self.node_flows is None or self.node_flows.size(1) != B):
            self.node_flows = torch.empty(self.num_nodes, B, device=self.device)
            self.element_flows = torch.full((self.num_elements, B), NEG_INF, device=self.device)
            self._eflow_mode = 1
            self._graphs = {k: g for k, g in self._graphs.items() if k[0] != "bk"}

    def _init_buffer(self, name: str, shape, set_value: Optional[float] = None):
        t = getattr(self, name, None)
        if not isinstance(t, torch.Tensor) or tuple(t.shape) != tuple(shape) or t.device != self.device:
            t = torch.zeros(shape, device=self.device)
            setattr(self, name, t)
        if set_value is not None:
            _fill(t, set_value)

    # ------------------------------------------------------------------------------------------
    # forward
    # ------------------------------------------------------------------------------------------
    def _prepare_inputs(self, inputs: torch.Tensor) -> torch.Tensor:
        assert inputs.dim() == 2 and inputs.size(1) >= self.num_vars
        if inputs.is_floating_point():
            raise TypeError("categorical inputs must be an integer tensor")
        if inputs.dtype not in (torch.uint8, torch.int16, torch.int32, torch.int64):
            inputs = inputs.long()
        return inputs.to(self.device, non_blocking=True).t().contiguous()       # [V, B]

    def _run_inner(self, key, fn):
        """Run ``fn`` (a sequence of launches on the current stream) — from a CUDA graph after the first call."""
        if not self.use_cuda_graphs:
            return fn()
        entry = self._graphs.get(key)
        if entry is None:                      # first call: run eagerly (also warms up every kernel)
            fn()
            self._graphs[key] = "warm"
        elif entry == "warm":
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            self._graphs[key] = g
            g.replay()
        else:
            entry.replay()

    def _fusion_on(self, gi: int, backward: bool = False) -> bool:
        """Whether depth `gi` (a sum group) runs with its product layer folded in.  The folded parameter-flow kernel
        reads eight samples per vector load, so the backward sweep only folds when the batch is a multiple of 8."""
        if not (self.fuse_product_layers and _lib.sum_mode() != 0 and gi in self._fused):
            return False
        if self._fused[gi]["sm"] and not SumLayer.use_sample_major:
            return False
        if backward and self._reference_compat:
            return False
        if self._fused[gi].get("dense") and not (SumLayer.use_dense_kernels and SumLayer.use_wide_dense
                                                 and self.node_mars is not None and self.node_mars.size(1) % 8 == 0):
            return False
        return (not backward) or self.node_mars.size(1) % 8 == 0

    def _launch_cfg(self):
        """Everything that changes which kernels a pass launches (part of the key of a captured graph)."""
        return (_lib.sum_mode(), self.fuse_product_layers, self.use_dataflow_launch, self.chain_tile,
                SumLayer.use_dense_kernels, SumLayer.use_wide_dense, SumLayer.use_sample_major,
                getattr(self._packer, "grown", 0),
                self._reference_compat, self._alg)

    def _chain_plan(self, B: int, mode: int):
        """Job table of the dataflow launch (one launch for a run of consecutive depths) for the forward pass
        (mode 0) or the element flows (mode 1), or None when fewer than two consecutive depths qualify.

        A depth qualifies when its product layer is folded into the sum kernels (for mode 1 also: flows are stored
        directly into the children's rows); the longest run of qualifying depths with one child-table width is used,
        the other depths keep their per-layer launches."""
        key = (B, mode, self._launch_cfg())
        cache = self.__dict__.setdefault("_chain_cache", {})
        if key in cache:
            return cache[key]
        groups = self.inner_layer_groups
        plan = None
        if self.use_dataflow_launch:
            def ok(gi):
                return (self._fusion_on(gi, backward=(mode == 1)) and not self._fused[gi]["sm"]
                        and not self._fused[gi].get("dense") and (mode == 0 or self._fused[gi]["direct"]))
            runs, cur = [], []
            for gi in range(1, len(groups), 2):
                if ok(gi) and (not cur or self._fused[cur[-1]]["fc"] == self._fused[gi]["fc"]):
                    cur.append(gi)
                else:
                    if cur:
                        runs.append(cur)
                    cur = [gi] if ok(gi) else []
            if cur:
                runs.append(cur)
            run = max(runs, key=len) if runs else []
            if len(run) >= 2:
                fc = self._fused[run[0]]["fc"]
                levels = run if mode == 0 else run[::-1]
                jobs = []                                   # (packed, rows, kids, fkids, K, row_block, par_block, n_rowtiles, level)
                for level, gi in enumerate(levels):
                    for layer in groups[gi]:
                        f = layer._fusion
                        if mode == 0:
                            for p, (nids, cids, _, _) in enumerate(layer._dev["fw"]):
                                jobs.append((layer._packed_fw[p], nids, cids, f["fw"][p], cids.size(1), layer.block_size, 1,
                                             nids.numel() * (layer.block_size // 128), level))
                        else:
                            for p, ((chids, parids, _), cbs) in enumerate(zip(layer._dev["bk"], layer.cs_block_sizes)):
                                jobs.append((layer._packed_bk[p], chids, parids, f["bk"][p], parids.size(1), cbs,
                                             layer.block_size, chids.numel() * (cbs // 128), level))
                level_tiles = [0] * len(levels)
                for j in jobs:
                    level_tiles[j[8]] += j[7]
                tn = self.chain_tile
                if tn is None:                               # widest tile that keeps about two tiles per SM in flight
                    mean_tiles = sum(level_tiles) / len(levels)
                    tn = next((t for t in (64, 32) if mean_tiles * (-(-B // t)) >= 296), 16)
                n_ct = -(-B // tn)
                rec = np.dtype([("packed", "<u8"), ("rows", "<u8"), ("kids", "<u8"), ("fkids", "<u8"), ("item_begin", "<i8"),
                                ("K", "<i4"), ("row_block", "<i4"), ("par_block", "<i4"), ("n_rowtiles", "<i4"),
                                ("level", "<i4"), ("prev_total", "<i4")])
                table = np.zeros(len(jobs), dtype=rec)
                begin = 0
                for r, (packed, rows, kids, fk, K, rb, pb, nrt, level) in zip(table, jobs):
                    r["packed"], r["rows"], r["kids"], r["fkids"] = (t.data_ptr() for t in (packed, rows, kids, fk))
                    r["item_begin"], r["K"], r["row_block"], r["par_block"], r["n_rowtiles"] = begin, K, rb, pb, nrt
                    r["level"], r["prev_total"] = level, (level_tiles[level - 1] if level > 0 else 0)
                    begin += nrt * n_ct
                plan = dict(lo=run[0], hi=run[-1], fc=fc, tn=tn, n_levels=len(levels), n_jobs=len(jobs), n_items=begin,
                            jobs=torch.from_numpy(table.view(np.uint8)).to(self.device),
                            ctrl=torch.zeros(64 + len(levels) * n_ct, dtype=torch.int32, device=self.device))
        cache[key] = plan
        return plan

    def _launch_chain(self, plan, mode: int, logspace_flows: bool = True):
        _lib.call("pcx_sum_chain", mode, self.node_mars, self.node_flows if mode == 1 else None, plan["jobs"],
                  plan["n_jobs"], plan["n_items"], plan["n_levels"], plan["tn"], plan["fc"], self.node_mars.size(1),
                  int(bool(logspace_flows)), plan["ctrl"], plan["ctrl"].numel())

    def _forward_inner(self):
        groups = self.inner_layer_groups
        plan = self._chain_plan(self.node_mars.size(1), 0)
        for gi, group in enumerate(groups):
            if plan is not None and plan["lo"] - 1 <= gi <= plan["hi"]:
                if gi == plan["lo"]:
                    self._launch_chain(plan, 0)
                continue
            if group.is_prod():
                if not self._fusion_on(gi + 1):
                    group.forward(self.node_mars, self.element_mars)
            elif self._fusion_on(gi):
                for layer in group:
                    layer.forward_fused(self.node_mars)
            else:
                group.forward(self.node_mars, self.element_mars, self.params.data, **self._alg_kwargs())

    def _alg_kwargs(self) -> dict:
        names = ("LL", "MPE", "GeneralLL")
        return dict(propagation_alg=names[self._alg[0]], **({"alpha": self._alg[1]} if self._alg[0] == 2 else {}))

    def set_propagation_alg(self, propagation_alg: str, **kwargs):
        """Default propagation rule of `forward` ("LL", "MPE", or "GeneralLL" with ``alpha``), as
        model/tensorcircuit.py:293-317."""
        _alg_of(propagation_alg, kwargs)
        self.default_propagation_alg = propagation_alg
        self.propagation_alg_kwargs = {"alpha": kwargs["alpha"]} if propagation_alg == "GeneralLL" else {}

    def forward_ll(self, *args, **kwargs):
        return self.forward(*args, propagation_alg="LL", **kwargs)

    def forward_mpe(self, *args, **kwargs):
        return self.forward(*args, propagation_alg="MPE", **kwargs)

    def forward_general_ll(self, *args, **kwargs):
        return self.forward(*args, propagation_alg="GeneralLL", **kwargs)

    @_in_own_mode
    def forward(self, inputs: torch.Tensor, input_layer_fn=None, cache=None, return_cache: bool = False,
                propagation_alg: Optional[str] = None, pflow_temperature: float = 1.0, **kwargs):
        """Per-sample log-likelihoods ``[B, num_roots]`` of ``inputs`` (``[B, num_vars]``, integer)."""
        self._require_cuda()
        _unsupported(input_layer_fn=input_layer_fn is not None, cache=cache is not None, return_cache=return_cache,
                     pflow_temperature=abs(pflow_temperature - 1.0) > 1e-6,
                     missing_mask=kwargs.get("missing_mask") is not None)
        origin_inputs = inputs
        with torch.no_grad():
            B = inputs.size(0)
            data = self._prepare_inputs(inputs)
            self._ensure_buffers(B)
            if self.debug_poison:               # every row must be rewritten by the layer that owns it
                _fill(self.node_mars[self.num_dummy_nodes:], float("nan"))
            self._last_data, self._last_inputs = data, origin_inputs
            # the operand tiles of the tensor-core kernels are re-packed (when the parameters changed) on a second
            # stream, beside the input layer: neither reads what the other writes
            cur = torch.cuda.current_stream(self.device)
            forked = _lib.sum_mode() != 0 and self.use_side_stream
            if forked:
                self._side_stream.wait_stream(cur)
                with torch.cuda.stream(self._side_stream):
                    self._packer.refresh(self.params.data)   # outside any graph capture
            elif _lib.sum_mode() != 0:
                self._packer.refresh(self.params.data)
            with self._nvtx("pcx forward: input layers"):
                for layer in self.input_layer_group:
                    layer.forward(data, self.node_mars)
            if forked:
                cur.wait_stream(self._side_stream)
            with self._nvtx("pcx forward: inner layers"):
                self._run_inner(("fw", B, self._launch_cfg(), self.params.data_ptr()), self._forward_inner)
            lls = self.node_mars[self._root_node_range[0]:self._root_node_range[1], :].permute(1, 0).clone()
        if torch.is_grad_enabled():
            lls.requires_grad = True
            lls.register_hook(partial(_pc_model_backward_hook, pc=self, inputs=origin_inputs, **self._alg_kwargs()))
        return lls

    # ------------------------------------------------------------------------------------------
    # backward
    # ------------------------------------------------------------------------------------------
    def _par_jobs(self, B: int):
        """Device job tables (one per child-table width) that let ONE launch compute the parameter flows of every
        depth whose product layer is folded in; cached per batch size."""
        key = (B, _lib.sum_mode(), self.fuse_product_layers)
        cache = self.__dict__.setdefault("_par_job_cache", {})
        if key in cache:
            return cache[key]
        rec = np.dtype([("nids", "<u8"), ("cids", "<u8"), ("pids", "<u8"), ("pfids", "<u8"), ("fkids", "<u8"),
                        ("item_begin", "<i8"), ("K", "<i4"), ("block_size", "<i4"), ("e_tiles", "<i4"), ("splits", "<i4")])
        per_fc = {}
        for gi, group in enumerate(self.inner_layer_groups):
            if (group.is_sum() and self._fusion_on(gi, True) and not self._fused[gi]["sm"]
                    and not self._fused[gi].get("dense")):
                for layer in group:
                    f = layer._fusion
                    for p, (nids, cids, pids, pfids) in enumerate(layer._dev["fw"]):
                        K = cids.size(1)
                        per_fc.setdefault(f["fc"], []).append(
                            (nids, cids, pids, pfids, f["fw"][p], K, layer.block_size,
                             nids.numel() * (layer.block_size // 128) * ((K + 63) // 64)))
        total_chunks = (B + 31) // 32                                        # the kernel works on 32-sample slices
        out = []
        for fc, jobs in per_fc.items():
            base = sum(j[-1] for j in jobs)
            splits = max(1, min(total_chunks, -(-8 * 148 // base)))          # at least two waves of four CTAs per SM
            chunks_per_cta = -(-total_chunks // splits)
            splits = -(-total_chunks // chunks_per_cta)
            table = np.zeros(len(jobs), dtype=rec)
            begin = 0
            for r, (nids, cids, pids, pfids, fk, K, bs, items) in zip(table, jobs):
                r["nids"], r["cids"], r["pids"], r["pfids"], r["fkids"] = (t.data_ptr() for t in (nids, cids, pids, pfids, fk))
                r["item_begin"], r["K"], r["block_size"], r["e_tiles"], r["splits"] = begin, K, bs, (K + 63) // 64, splits
                begin += items * splits
            dev = torch.from_numpy(table.view(np.uint8)).to(self.device)
            out.append((fc, dev, len(jobs), begin, chunks_per_cta))
        cache[key] = out
        return out

    def _dense_par_plan(self, B: int):
        """Tables whose parameter flows come from the dense product (include/pcx_b200.h): deep tables whose rows all
        list the same children, grouped by shared parameters — tied layers are contracted together, their batches
        concatenated.  Returns {(id(layer), partition): (group, slot)} and the groups, or None when nothing qualifies."""
        key = (B, self._launch_cfg())
        cache = self.__dict__.setdefault("_dense_par_cache", {})
        if key in cache:
            return cache[key]
        groups, where = {}, {}
        cpl = -(-B // 64)
        for gi in range(len(self.inner_layer_groups) - 1, -1, -1):
            group = self.inner_layer_groups[gi]
            if not group.is_sum():
                continue
            folded = self._fusion_on(gi, True)
            if folded and not self._fused[gi].get("dense"):
                continue
            for layer in group:
                if layer._packer is None:
                    continue
                for p, (nids, cids, pids, pfids) in enumerate(layer._dev["fw"]):
                    wide = layer._wide_ok(p, B, False) and nids.numel() * layer.block_size <= SumLayer.DENSE_WIDE_MAX_DEPTH
                    if not ((wide or layer._dense_ok(p, B, False)) and layer._groups_fw[p][2] == 1):
                        assert not folded, "a dense-folded table must qualify for the dense parameter-flow product"
                        continue
                    g = groups.setdefault((layer._packed_fw[p].data_ptr(), wide),
                                          dict(members=[], tables=(cids, pids, pfids), n_blocks=nids.numel(),
                                               K=cids.size(1), block_size=layer.block_size, wide=wide))
                    where[(id(layer), p)] = (g, len(g["members"]))
                    g["members"].append((layer, p))
        plan = None
        total = 0
        for g in groups.values():
            row_tiles = g["n_blocks"] * (g["block_size"] // 128)
            if g["wide"]:                                   # samples of consecutive layers packed back to back
                g["n_chunks"] = -(-len(g["members"]) * B // 64)
                g["y_bytes"] = -(-g["K"] // 256) * g["n_chunks"] * 65536
            else:
                g["n_chunks"] = len(g["members"]) * cpl
                g["y_bytes"] = -(-g["K"] // 64) * g["n_chunks"] * 16384
            g["x_bytes"] = row_tiles * g["n_chunks"] * 32768
            total += g["x_bytes"] + g["y_bytes"]
        if groups and total <= self.dense_par_max_bytes:
            for g in groups.values():
                g["x"] = torch.zeros(g["x_bytes"], dtype=torch.uint8, device=self.device)
                g["y"] = torch.zeros(g["y_bytes"], dtype=torch.uint8, device=self.device)
            rows = max(g["n_blocks"] * g["block_size"] for g in groups.values())
            plan = dict(where=where, groups=list(groups.values()),
                        work=torch.empty((-(-rows // 64) + 1) * B, dtype=torch.float32, device=self.device))
        elif groups:
            assert not any(self._fused.get(gi, {}).get("dense") for gi in self._fused), \
                "`dense_par_max_bytes` is too small for the operands of the dense parameter-flow product"
        cache[key] = plan
        return plan

    def _backward_inner(self, compute_param_flows: bool, logspace_flows: bool):
        """Reverse sweep over the inner layers.  Parameter flows of the depths whose product layer is folded in only
        read node values and node flows, and tiles of different layers are independent: they all run as ONE launch
        once the dependent chain of element-flow kernels has produced every node flow (`_launch_batched_par`, issued
        by `backward` so that it can share the device with the input layer's backward pass)."""
        pf = self.param_flows if compute_param_flows else None
        groups = self.inner_layer_groups
        any_fused = False
        dense = self._dense_par_plan(self.node_mars.size(1)) if (pf is not None and self._alg[0] == 0) else None

        def dense_stage(layer, p, node_flows, node_mars, element_mars, ls):
            hit = dense["where"].get((id(layer), p))
            if hit is None:
                return False
            g, slot = hit
            nids, cids, _, _ = layer._dev["fw"][p]
            if g["wide"]:
                f = getattr(layer, "_fusion", None)
                fk = f["fw"][p] if (f is not None and f.get("dense") and element_mars is None) else None
                _lib.call("pcx_sum_par_dense2_stage", g["x"], g["y"], node_flows, node_mars, element_mars, nids, cids,
                          fk, f["fc"] if fk is not None else 0, nids.numel(), cids.size(1), layer.block_size,
                          node_flows.size(1), g["n_chunks"], slot, ls)
            else:
                _lib.call("pcx_sum_par_dense_stage", g["x"], g["y"], dense["work"], node_flows, node_mars, element_mars,
                          nids, cids, nids.numel(), cids.size(1), layer.block_size, node_flows.size(1), g["n_chunks"],
                          slot, ls)
            return True

        plan = self._chain_plan(self.node_mars.size(1), 1)
        cur = torch.cuda.current_stream(self.device)
        side = self._side_stream if self.use_side_stream else None
        forked = False
        for gi in range(len(groups) - 1, -1, -1):
            group = groups[gi]
            if plan is not None and plan["lo"] - 1 <= gi <= plan["hi"]:
                any_fused = True
                if gi == plan["hi"]:
                    self._launch_chain(plan, 1, logspace_flows)
                continue
            if group.is_prod():
                if not (self._fusion_on(gi + 1, True) and self._fused[gi + 1]["direct"]):
                    group.backward(self.node_flows, self.element_flows, logspace_flows=logspace_flows)
            elif self._fusion_on(gi, True) and self._fused[gi].get("dense"):
                # The operands of the (tied) parameter-flow product only read this depth's node flows and values, which
                # are final by now; the element flows below read the same rows and write the children's.  The two are
                # independent, so the operand staging goes to the second stream and shares the device with the chain
                # of element-flow kernels (which are short and leave SMs idle between them).
                if pf is not None:
                    if side is not None:
                        side.wait_stream(cur)
                    with torch.cuda.stream(side if side is not None else cur):
                        for layer in group:
                            for p in range(layer.num_fw_partitions):
                                ok = dense is not None and dense_stage(layer, p, self.node_flows, self.node_mars, None,
                                                                       int(bool(logspace_flows)))
                                assert ok, "a dense-folded table must have a slot in the dense parameter-flow product"
                    forked = forked or side is not None
                for layer in group:
                    layer.backward_ele_fused(self.node_flows, self.element_flows, self.node_mars, logspace_flows)
            elif self._fusion_on(gi, True):
                any_fused = any_fused or not self._fused[gi]["sm"]
                for layer in group:
                    if self._fused[gi]["sm"] and pf is not None:       # (the 128-row kernels do this in one launch below)
                        layer.backward_par_fused(self.node_flows, self.node_mars, self.params.data, pf, logspace_flows)
                    layer.backward_ele_fused(self.node_flows, self.element_flows, self.node_mars, logspace_flows)
            else:
                # the shared element buffer holds another depth by now: recompute this depth's products
                groups[gi - 1].forward(self.node_mars, self.element_mars, _for_backward=True)
                group.backward(self.node_flows, self.element_flows, self.node_mars, self.element_mars,
                               self.params.data, param_flows=pf, logspace_flows=logspace_flows,
                               dense_par_stage=dense_stage if dense is not None else None, **self._alg_kwargs())
        if dense is not None:
            if forked:
                side.wait_stream(cur)                        # operands staged on the main stream are complete too
            with torch.cuda.stream(side if forked else cur):
                for g in dense["groups"]:
                    cids, pids, pfids = g["tables"]
                    _lib.call("pcx_sum_par_dense2_gemm" if g["wide"] else "pcx_sum_par_dense_gemm", pf, self.params.data,
                              g["x"], g["y"], cids, pids, pfids, g["n_blocks"], g["K"], g["block_size"], g["n_chunks"])
        if forked:
            cur.wait_stream(side)
        self._batched_par_pending = any_fused and pf is not None     # launched by `backward`, after this sweep

    def _launch_batched_par(self, logspace_flows: bool):
        B = self.node_flows.size(1)
        for fc, jobs, n_jobs, n_items, chunks_per_cta in self._par_jobs(B):
            _lib.call("pcx_sum_bwd_par_batched", self.param_flows, self.node_flows, self.node_mars, self.params.data,
                      jobs, n_jobs, n_items, fc, B, chunks_per_cta, int(bool(logspace_flows)))

    @_in_own_mode
    def backward(self, inputs: Optional[torch.Tensor] = None, ll_weights: Optional[torch.Tensor] = None,
                 compute_param_flows: bool = True, flows_memory: float = 1.0, input_layer_fn=None, cache=None,
                 return_cache: bool = False, allow_modify_flows: bool = False, propagation_alg: str = "LL",
                 logspace_flows: bool = True, negate_pflows: bool = False, pflow_temperature: float = 1.0, **kwargs):
        """Node / element flows and (accumulated) parameter flows of the last forward pass.

        ``logspace_flows`` selects whether the flow buffers hold log-flows (default) or linear flows; the
        parameter flows are the same either way."""
        self._require_cuda()
        # `allow_modify_flows` only permits the reference to overwrite node flows in place (linear flows only,
        # layer/sum_layer.py:442-455); the kernels here never need to, so it is accepted and changes nothing
        assert not (allow_modify_flows and logspace_flows), \
            "`allow_modify_flows` should be set to `False` when using `logspace_flows`."
        _unsupported(input_layer_fn=input_layer_fn is not None, cache=cache is not None, return_cache=return_cache,
                     negate_pflows=negate_pflows, pflow_temperature=abs(pflow_temperature - 1.0) > 1e-6,
                     missing_mask=kwargs.get("missing_mask") is not None)
        assert self.node_mars is not None and self.element_mars is not None, "Should run forward path first."
        self._run_params = dict(logspace_flows=logspace_flows, propagation_alg=propagation_alg)
        with torch.no_grad():
            B = self.node_mars.size(1)
            if inputs is None or inputs is getattr(self, "_last_inputs", None):
                data = self._last_data
            else:
                assert inputs.dim() == 2 and inputs.size(0) == B
                data = self._prepare_inputs(inputs)
            self._ensure_buffers(B, backward=True)
            ls = int(bool(logspace_flows))
            reset = NEG_INF if logspace_flows else 0.0
            if self.debug_poison:               # rows outside the reset ranges must be rewritten by direct stores
                _fill(self.node_flows, float("nan"))
            # the partial reset is only valid while every depth that was counted as "stores flows directly" does so
            rkey = (B, self._launch_cfg())
            if getattr(self, "_reset_key", None) != rkey:            # (a hundred depths: decided once per configuration)
                self._reset_key = rkey
                self._reset_partial = (B % 8 == 0 and not self._reference_compat
                                       and all(self._fusion_on(gi, True) for gi in self._fused))
            ranges = self._flow_reset_ranges if self._reset_partial else None
            if ranges is None:
                _fill(self.node_flows, reset)
            else:                                            # every other row is rewritten by a direct store
                for a0, a1 in ranges:
                    _fill(self.node_flows[a0:a1], reset)
            if self._eflow_mode != ls or self._reference_compat:
                # dummy / parentless element rows: -inf in log space, 0 linearly (`reference_compat`: the buffer is
                # cleared once per pass, as the reference does, and rows without a writer keep an earlier depth's flow)
                _fill(self.element_flows, NEG_INF if logspace_flows else 0.0)
                self._eflow_mode = ls

            if compute_param_flows:                          # decay (or clear) the accumulators and the flow total first
                self.init_param_flows(flows_memory=flows_memory)
            r0, r1 = self._root_node_range
            if ll_weights is None:
                _lib.call("pcx_set_root_flows", self.node_flows, None, r0, r1 - r0, B, ls)
                if compute_param_flows:
                    self._cum_flow_host += (r1 - r0) * B
            else:
                w = ll_weights.to(self.device, torch.float32)
                w = w.unsqueeze(0) if w.dim() == 1 else w
                assert w.size(0) == self.num_root_nodes and w.size(1) == B
                w = w.contiguous()
                _lib.call("pcx_set_root_flows", self.node_flows, w, r0, r1 - r0, B, ls)
                if compute_param_flows:
                    s = w.sum(dtype=torch.float64)
                    self._cum_flow_dev = s if self._cum_flow_dev is None else self._cum_flow_dev + s

            if _lib.sum_mode() != 0:
                self._packer.refresh(self.params.data)
            key = ("bk", B, bool(compute_param_flows), ls, self._launch_cfg(), self.params.data_ptr(),
                   self.param_flows.data_ptr() if compute_param_flows else 0)
            self._batched_par_pending = self._bk_par_pending.get(key, False)
            with self._nvtx("pcx backward: inner layers"):
                self._run_inner(key, partial(self._backward_inner, compute_param_flows, bool(logspace_flows)))
            self._bk_par_pending[key] = self._batched_par_pending

            if compute_param_flows:
                # The parameter flows of the sum layers and of the input layer are independent once every node flow
                # exists.  One rank: both run together, on two streams.  Data-parallel ranks with the overlapped
                # all-reduce: the input layer first, then the all-reduce of its flows (the larger part of the
                # arena) beside the sum layers' parameter-flow kernel.
                cur = torch.cuda.current_stream(self.device)
                if self._batched_par_pending and self.use_side_stream and not self._overlap_ready():
                    self._side_stream.wait_stream(cur)
                    with torch.cuda.stream(self._side_stream):
                        for layer in self.input_layer_group:
                            layer.backward(data, self.node_flows, self.node_mars, logspace_flows=bool(logspace_flows))
                    self._launch_batched_par(logspace_flows)
                    cur.wait_stream(self._side_stream)
                else:
                    for layer in self.input_layer_group:
                        layer.backward(data, self.node_flows, self.node_mars, logspace_flows=bool(logspace_flows))
                    self._start_early_flow_sync()
                    if self._batched_par_pending:
                        self._launch_batched_par(logspace_flows)
        return None

    # ---- data-parallel flow synchronisation overlapped with the tail of the step ---------------------------------
    def enable_flow_sync_overlap(self, group=None, dtype: Optional[torch.dtype] = None):
        """Called by an optimizer that synchronises after EVERY backward pass (``ddp=True``, one mini-batch per
        update, fp32): the all-reduce is then split in two and overlapped — the input-layer flows are reduced while
        the sum layers' parameter flows are computed, the sum-layer flows (and the flow total in the arena header)
        while the input-layer parameters are updated."""
        self._overlap_group = (group,)
        self._overlap_dtype = dtype                      # e.g. bfloat16: both parts travel in reduced precision

    def _overlap_ready(self) -> bool:
        import torch.distributed as dist
        g = getattr(self, "_overlap_group", None)
        return (g is not None and self.device.type == "cuda" and dist.is_available() and dist.is_initialized()
                and dist.get_world_size(g[0]) > 1)

    def _input_reduce_end(self) -> int:
        """Arena offset up to which the input-layer flows take part in the all-reduce: replica accumulators of tied
        input vectors are folded into their source range first and, when they form the tail of the arena, left out."""
        arena, layers = self._flow_arena, list(self.input_layer_group)
        last = layers[-1]
        if self.device.type == "cuda":
            for layer in layers:
                layer._flush_shadow()                       # flows still held in a transposed shadow table
            if last.tied2source_nids:
                last.fold_tied_flows()
        if last.tied2source_nids and getattr(last, "_tied_folded", False):
            return arena.segment_end(len(layers), last.num_untied_param_flows)
        return arena.total

    def _start_early_flow_sync(self):
        """First part of the overlapped all-reduce: the input-layer flows, as soon as the input layer's backward pass
        is enqueued."""
        if not self._overlap_ready():
            return
        if getattr(self, "_early_sync", None) is not None:
            # the input-layer flows of the previous pass are already summed over the ranks; this pass has just added
            # local flows on top of them, and no later collective can separate the two
            raise RuntimeError("two backward passes that compute parameter flows ran without an optimizer step in "
                               "between while the overlapped flow synchronisation is on (MiniBatchEM(ddp=True), one "
                               "mini-batch per update); use `niters_per_update` to accumulate over several batches")
        self._finish_late_sync()
        arena = self._flow_arena
        group, dtype = self._overlap_group[0], getattr(self, "_overlap_dtype", None)
        layers = list(self.input_layer_group)
        if all(layer._shadow is not None and layer._shadow["dirty"] and layer._arena_zero for layer in layers):
            # every input-layer flow of this update sits in a transposed shadow table and the accumulators proper are
            # empty: exchange the shadow tables themselves, so that the update can go on straight from them
            from .flows import _Works, all_reduce_async
            works = []
            for layer in layers:
                sh = layer._shadow
                works.append(all_reduce_async(sh["flows"], group=group, dtype=dtype))
                sh["touched"].fill_(1)                   # the peers' categories arrive: a later move-over skips nothing
            self._early_sync = _Works(works)
            return
        self._early_sync = arena.all_reduce_range_async(arena.offsets[1], self._input_reduce_end(),
                                                        group=group, dtype=dtype)

    def _finish_late_sync(self):
        """Make the current stream wait for the second part of the overlapped all-reduce (header + sum-layer flows)
        and pick up the summed flow total."""
        late = getattr(self, "_late_sync", None)
        if late is None:
            return
        late.wait()
        self._late_sync = None
        if self._late_head:
            self._cum_flow_host, self._cum_flow_dev = 0.0, None
            self._cum_flow_head = self._flow_arena.buf[:2].clone()

    @property
    def _cum_flow(self) -> float:
        self._finish_late_sync()
        if getattr(self, "_cum_flow_head", None) is not None:          # total left behind by the last flow sync
            self._cum_flow_host += FlowArena.decode_total(self._cum_flow_head)
            self._cum_flow_head = None
        if self._cum_flow_dev is not None:
            self._cum_flow_host += float(self._cum_flow_dev.item())
            self._cum_flow_dev = None
            _lib.check_status(self.device)                  # the host has just synchronised: a cheap place to look
        return self._cum_flow_host

    @_cum_flow.setter
    def _cum_flow(self, v: float):
        self._cum_flow_host = float(v)
        self._cum_flow_dev = None
        self._cum_flow_head = None

    # ------------------------------------------------------------------------------------------
    # parameter flows and EM
    # ------------------------------------------------------------------------------------------
    def init_param_flows(self, flows_memory: float = 1.0, batch_size: Optional[int] = None):
        assert 0.0 <= flows_memory <= 1.0, "`flows_memory` should be in [0.0, 1.0]"
        _unsupported(batch_size=batch_size is not None)
        self._require_cuda()
        self._finish_late_sync()
        if self.param_flows is None or self.param_flows.device != self.device:
            # all accumulators are views into one arena: a single all-reduce synchronises data-parallel ranks
            self._flow_arena = FlowArena([self.num_param_flows] + [l.num_param_flows for l in self.input_layer_group],
                                         self.device)
            self.param_flows = self._flow_arena.views[0]
            for layer, view in zip(self.input_layer_group, self._flow_arena.views[1:]):
                layer.param_flows = view
                layer._arena_zero = True
            self._graphs = {k: g for k, g in self._graphs.items() if k[0] != "bk"}
        elif flows_memory == 0.0:
            # Input layers whose accumulators are known to be empty still (all their flows went to the transposed
            # shadow and were consumed from there, nothing read or wrote the accumulators proper) need no clearing:
            # on configs[4] that is 2.1 GB of replica accumulators per step.
            arena, layers = self._flow_arena, list(self.input_layer_group)
            clean = [bool(getattr(layer, "_arena_zero", False)) for layer in layers]
            for layer in layers:
                layer._zero_shadow()
            if all(clean):
                _fill(arena.buf[:arena.segment_end(0)], 0.0)
            else:
                _fill(arena.buf, 0.0)
            for layer in layers:
                layer._arena_zero = True
        elif flows_memory != 1.0:
            for layer in self.input_layer_group:
                layer._flush_shadow()
            _scale(self._flow_arena.buf, flows_memory)
        # The running flow total decays with the flows it normalises.  (The reference only clears it when the
        # rescaled EM update consumes it, model/tensorcircuit.py:1363-1374, so that under data parallelism, where every
        # synchronisation replaces it by the sum over ranks, it doubles per step; here it stays the total of the
        # current accumulation window.)
        if flows_memory != 1.0:
            if flows_memory == 0.0:
                self._cum_flow_host, self._cum_flow_dev, self._cum_flow_head = 0.0, None, None
            else:
                self._cum_flow = self._cum_flow * flows_memory

    def zero_param_flows(self):
        self.init_param_flows(flows_memory=0.0)

    @_in_own_mode
    def eval_top_down_probs(self, update_pflow: bool = True, scale: float = 1.0):
        """Top-down probability of every node of a normalised circuit — the probability that a top-down sample passes
        through it: 1 for the root, parameter-weighted through sum nodes, copied through product nodes — and, with
        ``update_pflow``, ``scale * td(n) * theta(n, c)`` added to every parameter flow
        (model/backend/top_down_prob.py:290-402).

        This is the backward pass of a circuit whose every node has value one (log-value 0), with linear flows and a
        root flow of ``scale``, so it runs on the same kernels: eight identical columns (the tensor-core tiles want a
        batch that is a multiple of eight) that carry ``scale / 8`` each.  Returns the top-down probabilities
        ``[num_nodes]`` (times ``scale``)."""
        self._require_cuda()
        COLS = 8
        with torch.no_grad():
            t = self.__dict__.get("_tdp")
            if t is None:
                em = torch.zeros(self.num_elements, COLS, device=self.device)
                em[:self.num_dummy_eles] = NEG_INF
                t = dict(nm=torch.zeros(self.num_nodes, COLS, device=self.device), em=em,
                         nf=torch.empty(self.num_nodes, COLS, device=self.device),
                         ef=torch.empty(self.num_elements, COLS, device=self.device),
                         w=torch.empty(self.num_root_nodes, COLS, device=self.device))
                self._tdp = t
            if self.param_flows is None:
                self.init_param_flows()
            saved = (self.node_mars, self.element_mars, self.node_flows, self.element_flows, self._eflow_mode)
            self.node_mars, self.element_mars, self.node_flows, self.element_flows = t["nm"], t["em"], t["nf"], t["ef"]
            try:
                _fill(self.node_flows, 0.0)
                _fill(self.element_flows, 0.0)
                t["w"].fill_(float(scale) / COLS)
                r0, r1 = self._root_node_range
                _lib.call("pcx_set_root_flows", self.node_flows, t["w"], r0, r1 - r0, COLS, 0)
                if _lib.sum_mode() != 0:
                    self._packer.refresh(self.params.data)
                key = ("bk-tdp", COLS, bool(update_pflow), 0, self._launch_cfg(), self.params.data_ptr(),
                       self.param_flows.data_ptr() if update_pflow else 0)
                self._batched_par_pending = self._bk_par_pending.get(key, False)
                self._run_inner(key, partial(self._backward_inner, bool(update_pflow), False))
                self._bk_par_pending[key] = self._batched_par_pending
                if update_pflow and self._batched_par_pending:
                    self._launch_batched_par(False)
                td = self.node_flows.sum(dim=1)
                if update_pflow:
                    for layer in self.input_layer_group:
                        layer.add_missing_flows(td, scale=1.0)       # `td` already carries the scale
            finally:
                self.node_mars, self.element_mars, self.node_flows, self.element_flows, self._eflow_mode = saved
        return td

    @_in_own_mode
    def mini_batch_em(self, step_size: float, pseudocount: float = 0.0, keep_zero_params: bool = False,
                      step_size_rescaling: bool = False, **kwargs):
        """theta <- (1 - step_size) theta + step_size * (F + pseudocount / nch) / (sum F + pseudocount), for every
        sum node and every categorical leaf, from the accumulated flows F.

        ``step_size_rescaling`` (model/tensorcircuit.py:1363-1375): the flows are first scaled to
        ``step_size / (total flow of the window)``, the current parameters enter as ``(1 - step_size)`` times their
        top-down probabilities, and the update is then made with step size one."""
        assert 0.0 < step_size <= 1.0, "`step_size` should be between 0 and 1."
        self._require_cuda()
        if step_size_rescaling:
            cum = self._cum_flow
            assert cum > 0.0, "Please perform a backward pass before calling `mini_batch_em`."
            self.init_param_flows(flows_memory=step_size / cum)
            self.eval_top_down_probs(update_pflow=True, scale=1.0 - step_size)
            self._cum_flow = 0.0
            step_size = 1.0
        with torch.no_grad():
            def sum_update():
                head = self.param_flows[:2048].clone() if (self._reference_compat and self._fusing_dev) else None
                for start, n, chs in self._fusing_dev:
                    _lib.call("pcx_tied_accum", self.param_flows, start, n, chs, int(chs.numel()))
                if head is not None:
                    for tgt, sizes, ch, G, M in self.parflow_fusing_kwargs:
                        pads = ((ch == 0).sum(dim=1) - (ch[:, 0] == 0).long()).tolist()
                        for t, n, pad in zip(tgt.tolist(), sizes.tolist(), pads):
                            if pad > 0:
                                self.param_flows[t:t + n].add_(head[:n], alpha=float(pad))
                e = self._em_dev
                _lib.call("pcx_em_sum", self.params.data, self.param_flows, e["par"], e["flow"], e["fan"], e["bs"],
                          int(e["par"].numel()), e["max_bs"], float(step_size), float(pseudocount),
                          int(bool(keep_zero_params)))
                self._packer.invalidate()

            def input_update():
                for layer in self.input_layer_group:
                    layer.mini_batch_em(step_size=step_size, pseudocount=pseudocount, keep_zero_params=keep_zero_params)

            # sum parameters and input-layer parameters are disjoint
            cur = torch.cuda.current_stream(self.device)
            if getattr(self, "_late_sync", None) is not None:
                input_update()                              # beside the all-reduce of the sum-layer flows
                self._finish_late_sync()
                sum_update()
            elif self.use_side_stream:                      # the two updates run on two streams
                self._side_stream.wait_stream(cur)
                with torch.cuda.stream(self._side_stream):
                    sum_update()
                input_update()
                cur.wait_stream(self._side_stream)
            else:
                sum_update()
                input_update()

    def sync_param_flows(self, dtype: Optional[torch.dtype] = None, op=None, group=None, sync_cum_flow: bool = True,
                         _lazy: bool = False):
        """Sum the parameter flows (and the running flow total) of all data-parallel ranks with ONE all-reduce over
        the flow arena; no-op outside an initialised process group of more than one rank.

        Replica accumulators of tied input vectors are folded into their source range first and left out of the
        collective when they form the tail of the arena (a homogeneous HMM sends one emission-flow table instead of
        one per accumulator).  ``_lazy`` (optimizers): with the overlapped all-reduce, return once the input-layer
        flows are in and let `mini_batch_em` wait for the sum-layer flows."""
        import torch.distributed as dist
        if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) <= 1:
            return None
        if self.param_flows is None:
            self.init_param_flows()
        arena = self._flow_arena
        early = getattr(self, "_early_sync", None)
        if early is not None:
            # the input-layer flows are already being reduced: start the header + sum-layer part, then let the
            # current stream wait for the first part only (the input-layer update overlaps the second)
            self._early_sync = None
            if getattr(self, "_cum_flow_head", None) is not None:
                _ = self._cum_flow                          # fold a pending total of an earlier sync into the host part
            total = self._cum_flow_host if self._cum_flow_dev is None else self._cum_flow_dev + self._cum_flow_host
            arena.write_total(total)
            self._late_sync = arena.all_reduce_range_async(0, arena.segment_end(0), group=group,
                                                           dtype=getattr(self, "_overlap_dtype", None))
            self._late_head = bool(sync_cum_flow)
            early.wait()
            if not _lazy:
                self._finish_late_sync()
            return None
        self._finish_late_sync()
        end = self._input_reduce_end()
        reduce_len = None if end == arena.total else end
        if getattr(self, "_cum_flow_head", None) is not None:
            _ = self._cum_flow                              # fold a pending total of an earlier sync into the host part
        total = self._cum_flow_host if self._cum_flow_dev is None else self._cum_flow_dev + self._cum_flow_host
        head = arena.all_reduce(total, group=group, dtype=dtype, reduce_len=reduce_len, op=op)
        if sync_cum_flow:
            self._cum_flow_host, self._cum_flow_dev, self._cum_flow_head = 0.0, None, head
        return None

    def average_params(self, dtype: Optional[torch.dtype] = None, group=None):
        """Replace the sum parameters and every input layer's parameters by their mean over the data-parallel ranks
        (the exchange step of Local-SGD, PyJuice: optim/optim.py:99-124): the all-reduces are issued together and
        waited for once; no-op outside an initialised process group of more than one rank."""
        import torch.distributed as dist
        if not dist.is_available() or not dist.is_initialized():
            return None
        ws = dist.get_world_size(group)
        if ws <= 1:
            return None
        tensors = [self.params.data] + [l.params.data for l in self.input_layer_group if getattr(l, "params", None) is not None]
        with torch.no_grad():
            bufs = [t if dtype is None or t.dtype == dtype else t.to(dtype) for t in tensors]
            works = [dist.all_reduce(b, op=dist.ReduceOp.SUM, group=group, async_op=True) for b in bufs]
            for t, b, w in zip(tensors, bufs, works):
                w.wait()
                if b is not t:
                    t.copy_(b)
                t.mul_(1.0 / ws)
        if getattr(self, "_packer", None) is not None:
            self._packer.invalidate()                       # the tensor-core operand tiles are derived from the parameters
        return None

    # ------------------------------------------------------------------------------------------
    # accessors
    # ------------------------------------------------------------------------------------------
    @_in_own_mode
    def _nvtx(self, name: str):
        return torch.cuda.nvtx.range(name) if self.use_nvtx else contextlib.nullcontext()

    # ---- debugging aids ---------------------------------------------------------------------------------------------
    def assert_no_poison(self, backward: bool = False):
        """With ``debug_poison`` on, the value buffer (and, after a backward pass, the flow buffer) was NaN before the
        pass: a NaN that is still there marks a row no kernel wrote — a tile skipped by a grid computation, a
        wrong range.  Raises with the number of such values and the first rows."""
        bufs = [("node_mars", self.node_mars)] + ([("node_flows", self.node_flows)] if backward else [])
        for name, buf in bufs:
            bad = torch.isnan(buf[self.num_dummy_nodes:])
            if bool(bad.any()):
                rows = torch.nonzero(bad.any(dim=1)).reshape(-1)[:8] + self.num_dummy_nodes
                raise AssertionError(f"{name}: {int(bad.sum())} values were not written (first rows {rows.tolist()})")

    def validate_tables(self) -> dict:
        """Bounds check of every compiled index table against the buffers it indexes (node / element rows, parameter
        and flow offsets, variables): the static half of what a sanitizer run would check, on the host.  Category
        ids, the only data-dependent indices, are clamped by the leaf kernels.  Returns the number of indices checked
        per kind; raises ValueError on the first violations."""
        errs, counts = [], {}

        def cpu(t):
            return torch.as_tensor(t).detach().cpu().long()

        def check(what, idx, width, limit, skip_zero=False):
            idx = cpu(idx).reshape(-1)
            if skip_zero:
                idx = idx[idx != 0]
            counts[what] = counts.get(what, 0) + int(idx.numel())
            if idx.numel() and (int(idx.min()) < 0 or int(idx.max()) + width > limit):
                errs.append(f"{what}: index range [{int(idx.min())}, {int(idx.max())} + {width}) exceeds [0, {limit})")

        n_par, n_pf = int(self.params.numel()), int(self.num_param_flows)
        for layer in self.input_layer_group:
            check("input vids", layer.vids, 1, self.num_vars)
            cats = cpu(layer.node_cats)
            check("input s_pids", cpu(layer.s_pids) + cats, 0, int(layer.params.numel()) + 1)
            check("input s_pfids", cpu(layer.s_pfids) + cats, 0, int(layer.num_param_flows) + 1)
            check("input rows", torch.tensor(layer._output_ind_range), 0, self.num_nodes + 1)
        for group in self.inner_layer_groups:
            for layer in group:
                bs = layer.block_size
                if group.is_prod():
                    for nids, cids in zip(layer.partitioned_nids, layer.partitioned_cids):
                        check("prod nids", nids, bs, self.num_elements)
                        check("prod cids", cids, bs, self.num_nodes, skip_zero=True)
                    for u, par in zip(layer.partitioned_u_cids, layer.partitioned_parids):
                        check("prod u_cids", u, bs, self.num_nodes)
                        check("prod parids", par, bs, self.num_elements, skip_zero=True)
                    continue
                for nids, cids, pids, pfids in zip(layer.partitioned_nids, layer.partitioned_cids,
                                                   layer.partitioned_pids, layer.partitioned_pfids):
                    live = cpu(cids) != 0
                    check("sum nids", nids, bs, self.num_nodes)
                    check("sum cids", cids, 1, self.num_elements)
                    check("sum pids", cpu(pids)[live], bs, n_par)
                    check("sum pfids", cpu(pfids)[live], bs, n_pf)
                for chids, parids, parpids, cbs in zip(layer.partitioned_chids, layer.partitioned_parids,
                                                       layer.partitioned_parpids, layer.cs_block_sizes):
                    live = cpu(parids) != 0
                    check("sum chids", chids, cbs, self.num_elements)
                    check("sum parids", parids, bs, self.num_nodes, skip_zero=True)
                    check("sum parpids", cpu(parpids)[live], cbs * bs, n_par)
                f = getattr(layer, "_fusion", None)
                if f:                                                       # child rows of folded product layers
                    for t in list(f.get("fw", [])) + list(f.get("bk", [])):
                        if t is not None:
                            check("folded child rows", t, 1, self.num_nodes)
        if errs:
            raise ValueError("index tables out of bounds: " + "; ".join(errs[:6]))
        return counts

    def update_parameters(self, clone: bool = True):
        if self.device.type == "cuda":
            _lib.check_status(self.device)                  # parameters computed after a timed-out wait are wrong
        params = self.params.detach().cpu()
        for ns in self.root_ns:
            if ns.is_sum() and not ns.is_tied():
                ns.update_parameters(params, clone=clone)
        for layer in self.input_layer_group:
            layer.update_parameters()

    def update_param_flows(self, clone: bool = True, origin_ns_only: bool = True):
        flows = self.param_flows.detach().cpu()
        for ns in self.root_ns:
            if ns.is_sum() and not ns.is_tied():
                ns.update_param_flows(flows, clone=clone, origin_ns_only=origin_ns_only)

    def _prod_layer_of(self, ns):
        for gi, group in enumerate(self.inner_layer_groups):
            if group.is_prod():
                for layer in group:
                    if any(n is ns for n in layer.nodes):
                        return gi
        raise ValueError("node vector not found in this circuit")

    def get_node_mars(self, ns):
        s, e = ns._output_ind_range
        if ns.is_sum() or ns.is_input():
            return self.node_mars[s:e, :].detach()
        gi = self._prod_layer_of(ns)
        self.inner_layer_groups[gi].forward(self.node_mars, self.element_mars)
        return self.element_mars[s:e, :].detach()

    def get_node_flows(self, ns, **kwargs):
        s, e = ns._output_ind_range
        if ns.is_sum() or ns.is_input():
            return self.node_flows[s:e, :].detach()
        gi = self._prod_layer_of(ns)
        self.inner_layer_groups[gi].forward(self.node_mars, self.element_mars, _for_backward=True)
        self._reset_parentless(gi, self._run_params.get("logspace_flows", True))
        self.inner_layer_groups[gi + 1].backward(self.node_flows, self.element_flows, self.node_mars, self.element_mars,
                                                 self.params.data, param_flows=None,
                                                 logspace_flows=self._run_params.get("logspace_flows", True))
        return self.element_flows[s:e, :].detach()

    def get_node_params(self, ns, clone: bool = True, **kwargs):
        if not ns.is_sum() or ns.is_tied():
            return None
        s, e = ns._param_range
        flat = self.params[s:e].detach()
        flat = flat.clone() if clone else flat
        local = ((ns._param_ids - s) // (ns.block_size * ns.ch_block_size)).to(flat.device)
        return flat.reshape(local.size(0), ns.ch_block_size, ns.block_size)[local].permute(0, 2, 1)

    def get_node_param_flows(self, ns, clone: bool = True, **kwargs):
        if not ns.is_sum() or ns.is_tied():
            return None
        s, e = ns._param_flow_range
        flat = self.param_flows[s:e].detach()
        flat = flat.clone() if clone else flat
        local = ((ns._param_flow_ids - s) // (ns.block_size * ns.ch_block_size)).to(flat.device)
        return flat.reshape(local.size(0), ns.ch_block_size, ns.block_size)[local].permute(0, 2, 1)

    def layers(self, reverse: bool = False, ret_layer_groups: bool = False, ignore_input_layers: bool = False):
        groups = ([] if ignore_input_layers else [self.input_layer_group]) + list(self.inner_layer_groups)
        if reverse:
            groups = groups[::-1]
        for g in groups:
            if ret_layer_groups:
                yield g
            else:
                for layer in g:
                    yield layer

    def print_statistics(self):
        print(f"> Number of nodes: {self.num_nodes}")
        print(f"> Number of edges: {self.num_edges}")
        print(f"> Number of sum parameters: {self.num_sum_params}")
        print(f"> Number of input parameters: {sum(l.params.numel() for l in self.input_layer_group)}")


def compile(ns, layer_sparsity_tol: float = 0.5, max_num_partitions: Optional[int] = None,
            disable_gpu_compilation: bool = False, force_gpu_compilation: bool = False,
            max_tied_ns_per_parflow_block: int = 32, device=None, verbose: bool = True) -> TensorCircuit:
    """Compile the node DAG rooted at ``ns`` into a :class:`TensorCircuit` (model/tensorcircuit.py:2138-2175).
    Table compilation runs on the host; the two ``*_gpu_compilation`` switches are accepted and ignored."""
    return TensorCircuit(ns, layer_sparsity_tol=layer_sparsity_tol, max_num_partitions=max_num_partitions,
                         max_tied_ns_per_parflow_block=max_tied_ns_per_parflow_block, device=device, verbose=verbose)
