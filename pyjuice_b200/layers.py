"""Layer objects of a compiled circuit: index tables plus the launches that evaluate them.

The classes keep PyJuice's per-layer interface — ``layer(node_mars, element_mars[, params])`` and
``layer.backward(...)`` with the same positional arguments, ``partitioned_*`` table lists,
``LayerGroup`` iteration (layer/input_layer.py:35-604, layer/prod_layer.py:28-238,
layer/sum_layer.py:130-543, layer/layer_group.py:14-113) — but every computation is one call into
the CUDA library per partition; there is no Triton, no autotuning and no CPU path.

Tables live twice: the int64 CPU/any-device tensors that are the (bit-exact) compiler output, and
int32 device copies that the kernels read.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.nn as nn

from . import _lib
from .compiler import (compile_input, compile_prod, compile_sum_backward, compile_sum_forward,
                       reorder_input_nodes)
from .nodes import BitSet, as_bitset

_I32_MAX = 2 ** 31 - 1


def _dev_i32(t: torch.Tensor, device) -> torch.Tensor:
    if t.numel() > 0 and int(t.max()) > _I32_MAX:
        raise ValueError("index table exceeds the 32-bit range the kernels address with")
    return t.to(device=device, dtype=torch.int32).contiguous()


ALG_IDS = {"LL": 0, "MPE": 1, "GeneralLL": 2}


def _alg_of(propagation_alg, kwargs):
    """(id, alpha) of a propagation rule given by name (layer/sum_layer.py: `propagation_alg_mapping`)."""
    if propagation_alg not in ALG_IDS:
        raise NotImplementedError(f"Unknown propagation algorithm {propagation_alg}.")
    alg = ALG_IDS[propagation_alg]
    alpha = float(kwargs.get("alpha", 0.0)) if alg == 2 else 0.0
    if alg == 2 and not alpha > 0.0:
        raise ValueError("`propagation_alg='GeneralLL'` needs `alpha` > 0")
    return alg, alpha


def _unsupported(**flags):
    bad = [k for k, v in flags.items() if v]
    if bad:
        raise NotImplementedError(f"option(s) {bad} are outside the compiled LL forward/backward/EM path")


class ParamPacker:
    """Keeps the pre-split (bf16 hi/lo) parameter tiles of the tensor-core sum kernels in step with ``params``.

    Sum layers register the tables they need tiles for; layers whose tables are identical (tied parameters, e.g.
    the transition layers of a homogeneous HMM) share one buffer.  ``refresh`` re-runs the packing kernels when the
    parameter tensor was replaced, modified through torch, or updated by an EM step (``invalidate``)."""
    TILE_BYTES = 32768

    def __init__(self, device):
        self.device = device
        self.entries = {}
        self.sm_entries = {}
        self._stamp = None
        self._epoch = 0

    def register(self, key, n_rows, K, row_block, par_block, mode, kids, kpar):
        entry = self.entries.get(key)
        if entry is None:
            tiles = int(_lib.load().pcx_packed_tile_count(n_rows, K, row_block, par_block, mode))
            buf = torch.empty(tiles * self.TILE_BYTES, dtype=torch.uint8, device=self.device)
            contraction = K if mode == 0 else K * par_block
            entry = dict(buf=buf, tiles=tiles, kids=kids, kpar=kpar, K=K, row_block=row_block,
                         par_block=par_block if mode == 1 else 1, n_chunks=(contraction + 63) // 64, mode=mode)
            self.entries[key] = entry
            self._stamp = None
            self._jobs = None
        return entry["buf"]

    def invalidate(self):
        self._epoch += 1

    def _job_table(self):
        """Device array of PcxPackJob records (include/pcx_b200.h), one per registered table."""
        import numpy as np
        dt = np.dtype([("out", "<u8"), ("kids", "<u8"), ("kpar", "<u8"), ("vec_begin", "<i8"), ("K", "<i4"),
                       ("row_block", "<i4"), ("par_block", "<i4"), ("n_chunks", "<i4"), ("mode", "<i4"), ("pad", "<i4")])
        rec = np.zeros(len(self.entries), dtype=dt)
        vec = 0
        for j, e in enumerate(self.entries.values()):
            rec[j] = (e["buf"].data_ptr(), e["kids"].data_ptr(), e["kpar"].data_ptr(), vec, e["K"], e["row_block"],
                      e["par_block"], e["n_chunks"], e["mode"], 0)
            vec += e["tiles"] * 1024
        jobs = torch.from_numpy(rec.view(np.uint8).copy()).to(self.device)
        return jobs, len(self.entries), vec

    def register_sm(self, key, first_row, kids, kpar, n_merged, nb, block, K, par_block, mode):
        """Parameter tiles of a sample-major table (small node blocks); identical tables share one buffer."""
        entry = self.sm_entries.get(key)
        if entry is None:
            depth = K if mode == 0 else K * par_block
            nbytes = int(_lib.load().pcx_sm_packed_bytes(n_merged, depth, nb))
            entry = dict(buf=torch.empty(nbytes, dtype=torch.uint8, device=self.device),
                         args=(first_row, kids, kpar, n_merged, nb, block, K, par_block, mode))
            self.sm_entries[key] = entry
            self._stamp = None
            self._sm_jobs = None
        return entry["buf"]

    def refresh(self, params: torch.Tensor):
        stamp = (params.data_ptr(), params._version, self._epoch)
        if stamp == self._stamp or not (self.entries or self.sm_entries):
            return
        if self.entries:
            if getattr(self, "_jobs", None) is None:
                self._jobs = self._job_table()
            jobs, n_jobs, n_vec = self._jobs
            _lib.call("pcx_pack_sum_params", jobs, n_jobs, n_vec, params)
        if self.sm_entries:
            if getattr(self, "_sm_jobs", None) is None:
                self._sm_jobs = self._sm_job_table()
            jobs, n_jobs, n_vec = self._sm_jobs
            _lib.call("pcx_pack_sm_jobs", jobs, n_jobs, n_vec, params)
        self._stamp = stamp

    def _sm_job_table(self):
        """Device array of PcxSmPackJob records (include/pcx_b200.h), one per sample-major table."""
        import numpy as np
        dt = np.dtype([("out", "<u8"), ("first_row", "<u8"), ("kids", "<u8"), ("kpar", "<u8"), ("vec_begin", "<i8"),
                       ("nb", "<i4"), ("block", "<i4"), ("K", "<i4"), ("par_block", "<i4"), ("n_chunks", "<i4"), ("mode", "<i4")])
        rec = np.zeros(len(self.sm_entries), dtype=dt)
        vec = 0
        for j, e in enumerate(self.sm_entries.values()):
            first_row, kids, kpar, n_merged, nb, block, K, par_block, mode = e["args"]
            n_chunks = ((K if mode == 0 else K * par_block) + 63) // 64
            rec[j] = (e["buf"].data_ptr(), first_row.data_ptr(), kids.data_ptr(), kpar.data_ptr(), vec, nb, block, K,
                      par_block, n_chunks, mode)
            vec += n_merged * n_chunks * 8 * nb
        jobs = torch.from_numpy(rec.view(np.uint8).copy()).to(self.device)
        return jobs, len(self.sm_entries), vec

    @property
    def nbytes(self):
        return sum(e["buf"].numel() for e in self.entries.values())

    def scratch(self, nbytes: int) -> torch.Tensor:
        """Operand scratch of the dense sum kernels: one buffer, shared by all layers (they run one after the other);
        ``grown`` counts re-allocations, so that captured CUDA graphs that hold the old address can be dropped."""
        buf = getattr(self, "_scratch", None)
        if buf is None or buf.numel() < nbytes:
            self._scratch = buf = torch.empty(int(nbytes), dtype=torch.uint8, device=self.device)
            self.grown = getattr(self, "grown", 0) + 1
        return buf


class Layer:
    def __init__(self, nodes):
        self.nodes = nodes
        self.device = torch.device("cpu")

    def is_input(self):
        return False

    def is_prod(self):
        return False

    def is_sum(self):
        return False

    def provided(self, name):
        return getattr(self, name, None) is not None


class InputLayer(Layer, nn.Module):
    """All input vectors of one distribution family (categorical only)."""

    def __init__(self, nodes, cum_nodes: int = 0, pc_num_vars: int = 0, max_tied_ns_per_parflow_block: int = 4):
        nn.Module.__init__(self)
        nodes = reorder_input_nodes(list(nodes))
        Layer.__init__(self, nodes)
        for ns in nodes:
            if ns.dist.get_signature() != "Categorical":
                raise NotImplementedError("only Categorical input distributions are on the compiled path")
        self.pc_num_vars = pc_num_vars
        self.dist_signature = "Categorical"
        t = compile_input(nodes, cum_nodes, max_tied_ns_per_parflow_block)
        for name in ("vids", "s_pids", "s_pfids", "s_mids", "nids", "source_nids", "node_id2source_id", "metadata"):
            self.register_buffer(name, t[name])
        self.tied2source_nids = t["tied2source_nids"]
        self.num_nodes = t["num_nodes"]
        self.num_parameters = t["num_parameters"]
        self.num_param_flows = t["num_param_flows"]
        self._output_ind_range = t["output_ind_range"]
        self.num_vars_per_node = self.vids.size(1)
        assert self.num_vars_per_node == 1, "categorical leaves are univariate"
        self.node_cats = self.metadata[self.s_mids].to(torch.int64)       # categories of every node
        self.max_cats = int(self.node_cats.max().item())
        self.params = nn.Parameter(torch.empty([max(self.num_parameters, 1)], dtype=torch.float32), requires_grad=False)
        self._shadow = None
        self._param_epoch = 0
        self._arena_zero = False                 # True while the [row, category] flow accumulators are known to be all zero
        self.param_flows = None
        self._dev = {}

    def is_input(self):
        return True

    # Tables with more categories than the staged kernels can hold in shared memory are looked up through a transposed
    # shadow ([category, row] instead of [row, category]); flows are accumulated in the same layout and moved into
    # `param_flows` (the reference's layout) whenever that tensor is read.
    SHADOW_MIN_CATS = 8193
    use_fused_shadow_em = True

    @property
    def param_flows(self):
        self._flush_shadow()
        self._arena_zero = False                 # the caller may write through the tensor
        return self._param_flows

    @param_flows.setter
    def param_flows(self, value):
        self._param_flows = value
        self._arena_zero = False                 # unknown content (whoever hands over a cleared buffer says so)

    def _setup_shadow(self, device):
        self._shadow = None
        C = self.max_cats
        if device.type != "cuda" or C < self.SHADOW_MIN_CATS or int(self.node_cats.min()) != C:
            return
        s_pids = self.s_pids.cpu()
        if self.num_parameters % C != 0 or bool((s_pids % C != 0).any()):
            return
        R = self.num_parameters // C
        src = self.source_nids.cpu()
        row_pfid = torch.full((R,), -1, dtype=torch.int64)
        row_pfid[s_pids[src] // C] = self.s_pfids.cpu()[src]
        if bool((row_pfid < 0).any()):
            return
        self._shadow = dict(R=R, C=C, prow=_dev_i32(s_pids // C, device), row_pfid=row_pfid.to(device), logp=None,
                            flows=None, stamp=None, dirty=False)

    def _shadow_ok(self, B: int) -> bool:
        return self._shadow is not None and B % 4 == 0

    def _flush_shadow(self):
        """Move the flows accumulated in the transposed shadow into `param_flows` (source rows) and clear the shadow."""
        sh = self._shadow
        if sh is None or not sh["dirty"] or self._param_flows is None:
            return
        _lib.call("pcx_input_cat_flush_t", self._param_flows, sh["flows"], sh["touched"], sh["row_pfid"], sh["R"], sh["C"])
        sh["dirty"] = False
        self._arena_zero = False

    def _zero_shadow(self):
        sh = self._shadow
        if sh is not None and sh["dirty"]:
            _fill(sh["flows"], 0.0)
            sh["touched"].zero_()
            sh["dirty"] = False

    def to(self, device):
        device = torch.device(f"cuda:{device}") if isinstance(device, int) else torch.device(device)
        nn.Module.to(self, device)
        for item in self.tied2source_nids:
            item[2] = item[2].to(device)
        if self.param_flows is not None:
            self.param_flows = self.param_flows.to(device)
        self.device = device
        self._dev = {}
        if device.type == "cuda":
            self._dev = dict(vids=_dev_i32(self.vids[:, 0], device), s_pids=_dev_i32(self.s_pids, device),
                             s_pfids=_dev_i32(self.s_pfids, device), source_nids=_dev_i32(self.source_nids, device),
                             node_cats=_dev_i32(self.node_cats, device))
        self._setup_shadow(device)
        return self

    def _init_parameters(self, perturbation: float):
        """Copy (or draw) the parameters of every untied vector, in layer order (layer/input_layer.py:1131-1143)."""
        p0 = 0
        params = torch.empty_like(self.params.data, device="cpu")
        for ns in self.nodes:
            if ns.is_tied():
                continue
            p1 = p0 + ns.num_nodes * ns.dist.num_parameters()
            if not ns.has_params():
                ns.init_parameters(perturbation=perturbation, recursive=False)
            params[p0:p1] = ns._params.reshape(-1)
            p0 = p1
        self.params.data = params.to(self.device)

    def init_param_flows(self, flows_memory: float = 1.0):
        """Stand-alone use only: inside a `TensorCircuit` the flows are a view into the circuit's flow arena."""
        if self._param_flows is None or self._param_flows.device != self.device:
            self.param_flows = torch.zeros([self.num_param_flows], dtype=torch.float32, device=self.device)
            self._zero_shadow()
        elif flows_memory == 0.0:
            self._zero_shadow()
            _fill(self._param_flows, 0.0)
            self._arena_zero = True
        elif flows_memory < 1.0:
            _scale(self.param_flows, flows_memory)            # (reading the property moves shadow flows in first)
        self._tied_folded = False

    def _require_cuda(self):
        if self.device.type != "cuda":
            raise NotImplementedError("input layers run on CUDA only (no CPU path)")

    def forward(self, data: torch.Tensor, node_mars: torch.Tensor, params=None, missing_mask=None, **kwargs):
        """``data`` is ``[num_vars, B]`` (variables outermost), integer."""
        _unsupported(params=params is not None, missing_mask=missing_mask is not None)
        self._require_cuda()
        data = data.contiguous()
        B = node_mars.size(1)
        if self._shadow_ok(B):
            sh = self._shadow
            stamp = (self.params.data_ptr(), self.params._version, self._param_epoch)
            if sh["logp"] is None:
                sh["logp"] = torch.empty(sh["R"] * sh["C"], dtype=torch.float32, device=self.device)
            if sh["stamp"] != stamp:                        # parameters changed: transpose and take logarithms once
                _lib.call("pcx_input_cat_shadow", sh["logp"], self.params.data, sh["R"], sh["C"])
                sh["stamp"] = stamp
            _lib.call("pcx_input_cat_fwd_t", node_mars, sh["logp"], data, data.element_size(), self._dev["vids"],
                      sh["prow"], sh["R"], sh["C"], self.num_nodes, self._output_ind_range[0], B)
            return
        _lib.call("pcx_input_cat_fwd", node_mars, self.params.data, data, data.element_size(),
                  self._dev["vids"], self._dev["s_pids"], self._dev["node_cats"], self.max_cats,
                  self.num_nodes, self._output_ind_range[0], B)

    def backward(self, data: torch.Tensor, node_flows: torch.Tensor, node_mars: torch.Tensor, params=None,
                 logspace_flows: bool = False, missing_mask=None, **kwargs):
        """Adds the (linear) flow of every (node, sample) to the flow of the observed category."""
        _unsupported(params=params is not None, missing_mask=missing_mask is not None)
        self._require_cuda()
        if self._param_flows is None:
            self.init_param_flows()
        data = data.contiguous()
        B = node_flows.size(1)
        if self._shadow_ok(B):
            sh = self._shadow
            if sh["flows"] is None:
                sh["flows"] = torch.zeros(sh["R"] * sh["C"], dtype=torch.float32, device=self.device)
                sh["touched"] = torch.zeros(sh["C"], dtype=torch.int32, device=self.device)
            _lib.call("pcx_input_cat_bwd_t", sh["flows"], sh["touched"], node_flows, data, data.element_size(), self._dev["vids"],
                      sh["prow"], sh["R"], sh["C"], self.num_nodes, self._output_ind_range[0], B,
                      int(bool(logspace_flows)))
            sh["dirty"] = True                            # every flow lands in its source row: replicas stay as they are
            return
        self._tied_folded = False                         # replica accumulators receive new flows
        self._arena_zero = False
        _lib.call("pcx_input_cat_bwd", self._param_flows, node_flows, data, data.element_size(),
                  self._dev["vids"], self._dev["s_pfids"], self._dev["node_cats"], self.max_cats,
                  self.num_nodes, self._output_ind_range[0], B, int(bool(logspace_flows)))

    @property
    def num_untied_param_flows(self) -> int:
        """Flows of the untied vectors: they come first in the layer's flow range, replicas of tied vectors after."""
        return int(sum(ns.num_nodes * ns.dist.num_param_flows() for ns in self.nodes if not ns.is_tied()))

    def fold_tied_flows(self):
        """Move the flows of every tied group's replica accumulators into its source range: source += replicas,
        replicas = 0 (layer/input_layer.py:755-783, 1391-1411 computes the same sum).  Because the replicas are cleared
        the fold can run any number of times; the flag only saves the pass when no backward pass has run since.
        (The reference leaves the replicas in place, so that with `flows_memory` in (0, 1) their decayed content is
        added to the source again at the next update; that double count is not reproduced.)"""
        self._flush_shadow()
        if getattr(self, "_tied_folded", False):
            return
        for start, n, ch_pfids in self.tied2source_nids:
            _lib.call("pcx_tied_accum", self._param_flows, int(start), int(n), ch_pfids, int(ch_pfids.numel()))
        self._tied_folded = True

    def mini_batch_em(self, step_size: float, pseudocount: float = 0.0, keep_zero_params: bool = False):
        self._require_cuda()
        sh = self._shadow
        if (sh is not None and sh["dirty"] and self._arena_zero and not keep_zero_params and sh["logp"] is not None
                and self.use_fused_shadow_em):
            # every flow of this update sits in the transposed shadow and the accumulators proper are empty: update
            # the parameters and the transposed log-parameter table straight from it.  The flows stay in
            # the shadow (still "dirty"): whoever reads `param_flows` later gets them moved over as usual.
            self._param_epoch += 1
            if sh.get("totals") is None:
                sh["totals"] = torch.zeros(16 * sh["R"], dtype=torch.float32, device=self.device)
            _lib.call("pcx_em_input_cat_t", self.params.data, sh["logp"], sh["flows"], sh["totals"], sh["R"], sh["C"],
                      float(step_size), float(pseudocount))
            sh["stamp"] = (self.params.data_ptr(), self.params._version, self._param_epoch)
            return
        self.fold_tied_flows()
        self._param_epoch += 1                            # the kernel below writes the parameters behind torch's back
        _lib.call("pcx_em_input_cat", self.params.data, self._param_flows, self._dev["source_nids"],
                  self._dev["s_pids"], self._dev["s_pfids"], self._dev["node_cats"], int(self.source_nids.numel()), self.max_cats,
                  float(step_size), float(pseudocount), int(bool(keep_zero_params)))

    def add_missing_flows(self, node_flows: torch.Tensor, scale: float = 1.0, **kwargs):
        """``node_flows``: one LINEAR flow per node of the circuit (``[num_nodes]``).  Every leaf's flow, plus that of
        the leaves tied to it, is spread over its categories in proportion to its parameters and added to the
        parameter flows (layer/input_layer.py:894-968)."""
        self._require_cuda()
        if self._param_flows is None:
            self.init_param_flows()
        self._arena_zero = False
        s, e = self._output_ind_range
        td = node_flows[s:e].to(torch.float32)
        n2s = self.node_id2source_id.to(self.device)                # -1 for source nodes, else the source's node id
        src_flow = td.clone()
        tied = n2s >= 0
        if bool(tied.any()):
            src_flow.index_add_(0, n2s[tied], td[tied])
        src_flow = src_flow[self.source_nids.to(self.device)].contiguous()
        _lib.call("pcx_input_cat_missing", self._param_flows, self.params.data, src_flow, self._dev["source_nids"],
                  self._dev["s_pids"], self._dev["s_pfids"], self._dev["node_cats"], int(self.source_nids.numel()),
                  float(scale))

    def update_parameters(self):
        params = self.params.detach().cpu()
        for ns in self.nodes:
            if not ns.is_tied():
                s, e = ns._param_range
                ns._params = params[s:e].clone()

    def __repr__(self):
        return f"InputLayer(nid_range={self._output_ind_range}, max_cats={self.max_cats})"


class ProdLayer(Layer, nn.Module):
    def __init__(self, nodes, global_nid_start: Optional[int] = None, layer_sparsity_tol=None, max_num_partitions=None, **kwargs):
        nn.Module.__init__(self)
        Layer.__init__(self, list(nodes))
        assert len(nodes) > 0, "No input node."
        if global_nid_start is None:
            block_sparse = all((not ns.is_sparse()) and ns.block_size == nodes[0].block_size for ns in nodes)
            global_nid_start = nodes[0].block_size if block_sparse else 1
        t = compile_prod(self.nodes, global_nid_start, layer_sparsity_tol, max_num_partitions)
        self.block_size = t["block_size"]
        self.use_block_sparse_edges = t["block_sparse"]
        self.num_nodes, self.num_edges = t["num_nodes"], t["num_edges"]
        self._layer_nid_range = (global_nid_start, global_nid_start + self.num_nodes)
        self.partitioned_nids, self.partitioned_cids = t["nids"], t["cids"]
        self.partitioned_u_cids, self.partitioned_parids = t["u_cids"], t["parids"]
        self.num_fw_partitions, self.num_bk_partitions = len(t["nids"]), len(t["u_cids"])
        self._dev = None

    def is_prod(self):
        return True

    def to(self, device):
        device = torch.device(f"cuda:{device}") if isinstance(device, int) else torch.device(device)
        for name in ("partitioned_nids", "partitioned_cids", "partitioned_u_cids", "partitioned_parids"):
            setattr(self, name, [x.to(device) for x in getattr(self, name)])
        self.device = device
        self._dev = None
        if device.type == "cuda":
            self._dev = dict(fw=[(_dev_i32(n, device), _dev_i32(c, device)) for n, c in zip(self.partitioned_nids, self.partitioned_cids)],
                             bk=[(_dev_i32(u, device), _dev_i32(p, device)) for u, p in zip(self.partitioned_u_cids, self.partitioned_parids)])
        return self

    def forward(self, node_mars: torch.Tensor, element_mars: torch.Tensor, _for_backward: bool = False, **kwargs):
        if self._dev is None:
            raise NotImplementedError("product layers run on CUDA only (no CPU path)")
        B = node_mars.size(1)
        for nids, cids in self._dev["fw"]:
            _lib.call("pcx_prod_fwd", element_mars, node_mars, nids, cids, nids.numel(), cids.size(1), self.block_size, B)

    __call__ = forward

    def backward(self, node_flows: torch.Tensor, element_flows: torch.Tensor, logspace_flows: bool = False, **kwargs):
        if self._dev is None:
            raise NotImplementedError("product layers run on CUDA only (no CPU path)")
        B = node_flows.size(1)
        raw = getattr(self, "_raw_backward_tables", False) and "bk_raw" in self._dev
        for u_cids, parids in self._dev["bk_raw" if raw else "bk"]:
            _lib.call("pcx_prod_bwd", node_flows, element_flows, u_cids, parids, u_cids.numel(), parids.size(1),
                      self.block_size, B, int(bool(logspace_flows)))

    def __repr__(self):
        return f"ProdLayer(nid_range={self._layer_nid_range}, num_nodes={self.num_nodes}, num_edges={self.num_edges})"


class SumLayer(Layer, nn.Module):
    def __init__(self, nodes, global_nid_start: int, global_pid_start: int, global_pfid_start: int, node2tiednodes,
                 layer_sparsity_tol=None, max_num_partitions=None, max_tied_ns_per_parflow_block: int = 8, **kwargs):
        nn.Module.__init__(self)
        Layer.__init__(self, list(nodes))
        assert len(nodes) > 0, "No input node."
        for ns in nodes:
            assert ns.block_size == nodes[0].block_size, "`block_size` of nodes in the same layer must be identical."
        self.block_size = nodes[0].block_size
        fw = compile_sum_forward(self.nodes, global_nid_start, global_pid_start, global_pfid_start, node2tiednodes,
                                 layer_sparsity_tol, max_num_partitions, max_tied_ns_per_parflow_block)
        self.num_nodes, self.num_edges = fw["num_nodes"], fw["num_edges"]
        self.partitioned_nids, self.partitioned_cids = fw["nids"], fw["cids"]
        self.partitioned_pids, self.partitioned_pfids = fw["pids"], fw["pfids"]
        self.num_fw_partitions = len(fw["nids"])
        self._layer_nid_range = (global_nid_start, global_nid_start + self.num_nodes)
        self._layer_pid_range = (global_pid_start, fw["pid_end"])
        self._layer_pfid_range = (global_pfid_start, fw["pfid_end"])
        self.num_parameters = fw["pid_end"] - global_pid_start
        self.num_param_flows = fw["pfid_end"] - global_pfid_start
        bk = compile_sum_backward(self.nodes, layer_sparsity_tol, max_num_partitions)
        self.partitioned_chids, self.partitioned_parids = bk["chids"], bk["parids"]
        self.partitioned_parpids, self.cs_block_sizes = bk["parpids"], bk["cs_block_sizes"]
        self.num_bk_partitions = len(bk["chids"])
        self._dev = None

    def is_sum(self):
        return True

    _TABLES = ("partitioned_nids", "partitioned_cids", "partitioned_pids", "partitioned_pfids",
               "partitioned_chids", "partitioned_parids", "partitioned_parpids")

    def to(self, device, packer: Optional[ParamPacker] = None):
        device = torch.device(f"cuda:{device}") if isinstance(device, int) else torch.device(device)
        cpu_tables = {name: [x.cpu() for x in getattr(self, name)] for name in self._TABLES}
        for name in self._TABLES:
            setattr(self, name, [x.to(device) for x in getattr(self, name)])
        self.device = device
        self._dev = None
        self._packer = None
        if device.type == "cuda":
            c = lambda t: _dev_i32(t, device)
            self._dev = dict(
                fw=[tuple(map(c, q)) for q in zip(self.partitioned_nids, self.partitioned_cids, self.partitioned_pids, self.partitioned_pfids)],
                bk=[tuple(map(c, q)) for q in zip(self.partitioned_chids, self.partitioned_parids, self.partitioned_parpids)])
            self._packed_fw = [None] * self.num_fw_partitions
            self._packed_bk = [None] * self.num_bk_partitions
            if packer is not None:
                self._packer = packer
                bs = self.block_size
                if bs % 128 == 0:
                    for p, (nids, cids, pids, _) in enumerate(self._dev["fw"]):
                        key = ("fw", bs, tuple(pids.shape), cpu_tables["partitioned_pids"][p].numpy().tobytes())
                        self._packed_fw[p] = packer.register(key, nids.numel(), cids.size(1), bs, 1, 0, cids, pids)
                for p, ((chids, parids, parpids), cbs) in enumerate(zip(self._dev["bk"], self.cs_block_sizes)):
                    if cbs % 128 == 0 and bs % 8 == 0:
                        key = ("bk", bs, cbs, tuple(parids.shape), cpu_tables["partitioned_parpids"][p].numpy().tobytes(),
                               (cpu_tables["partitioned_parids"][p] != 0).numpy().tobytes())
                        self._packed_bk[p] = packer.register(key, chids.numel(), parids.size(1), cbs, bs, 1, parids, parpids)
                # small blocks: sample-major tiles of one block, or of two consecutive blocks that list the same children
                def merged_rows(table, ids, block):
                    """[(nb, first_row tensor)]: pairs of consecutive, identical rows (nb = 2 * block <= 64), then singles."""
                    if block not in (32, 64) or table.size(0) == 0:
                        return None
                    n = table.size(0)
                    pair = torch.zeros(n, dtype=torch.bool)
                    if block == 32 and n > 1:
                        same = ((table[1:] == table[:-1]).all(dim=1) & (ids[1:] == ids[:-1] + block)).tolist()
                        i = 0
                        while i < n - 1:
                            if same[i]:
                                pair[i] = True
                                i += 2
                            else:
                                i += 1
                    second = torch.zeros(n, dtype=torch.bool)
                    second[1:] = pair[:-1]
                    out = []
                    if bool(pair.any()):
                        out.append((2 * block, torch.nonzero(pair).reshape(-1)))
                    single = torch.nonzero(~pair & ~second).reshape(-1)
                    if single.numel() > 0:
                        out.append((block, single))
                    return out

                self._sm_fw = [None] * self.num_fw_partitions
                self._sm_bk = [None] * self.num_bk_partitions
                for p, (nids, cids, pids, _) in enumerate(self._dev["fw"]):
                    groups = merged_rows(cpu_tables["partitioned_cids"][p], cpu_tables["partitioned_nids"][p], bs)
                    if groups is not None:
                        self._sm_fw[p] = []
                        for nb, first in groups:
                            key = ("smfw", bs, nb, tuple(pids.shape), cpu_tables["partitioned_pids"][p].numpy().tobytes(),
                                   first.numpy().tobytes())
                            fr = _dev_i32(first, device)
                            buf = packer.register_sm(key, fr, cids, pids, first.numel(), nb, bs, cids.size(1), 1, 0)
                            self._sm_fw[p].append((nb, fr, first.numel(), buf))
                for p, ((chids, parids, parpids), cbs) in enumerate(zip(self._dev["bk"], self.cs_block_sizes)):
                    if bs % 8 != 0 or (bs & (bs - 1)) != 0:
                        continue
                    groups = merged_rows(cpu_tables["partitioned_parids"][p], cpu_tables["partitioned_chids"][p], cbs)
                    if groups is not None:
                        self._sm_bk[p] = []
                        for nb, first in groups:
                            # two child blocks can only share a tile if their parameter tiles line up as well
                            key = ("smbk", bs, cbs, nb, tuple(parids.shape), cpu_tables["partitioned_parpids"][p].numpy().tobytes(),
                                   (cpu_tables["partitioned_parids"][p] != 0).numpy().tobytes(), first.numpy().tobytes())
                            fr = _dev_i32(first, device)
                            buf = packer.register_sm(key, fr, parids, parpids, first.numel(), nb, cbs, parids.size(1), bs, 1)
                            self._sm_bk[p].append((nb, fr, first.numel(), buf))
            # rows of a table that list the same children (parents) share one tensor-core operand in the dense kernels
            def groups_of(table):
                uniq, inverse = torch.unique(table, dim=0, return_inverse=True)
                first = torch.full((uniq.size(0),), table.size(0), dtype=torch.int64)
                first.scatter_reduce_(0, inverse, torch.arange(table.size(0)), reduce="amin")
                return _dev_i32(inverse, device), _dev_i32(first, device), int(uniq.size(0))
            self._groups_fw = [groups_of(t) for t in cpu_tables["partitioned_cids"]]
            self._groups_bk = [groups_of(t) for t in cpu_tables["partitioned_parids"]]
        return self

    # Tables at least this deep take the two-step dense path (operand pre-pass + GEMM over pre-tiled operands).
    DENSE_MIN_DEPTH = 512

    def _dense_ok(self, p: int, B: int, backward: bool) -> bool:
        if not self.use_dense_kernels or B % 64 != 0 or _lib.sum_mode() == 0:
            return False
        if backward:
            return self._packed_bk[p] is not None and self._dev["bk"][p][1].size(1) * self.block_size >= self.DENSE_MIN_DEPTH
        return self._packed_fw[p] is not None and self._dev["fw"][p][1].size(1) >= self.DENSE_MIN_DEPTH

    def _dense_scratch(self, n_groups: int, depth: int, B: int) -> torch.Tensor:
        return self._packer.scratch(int(_lib.load().pcx_dense_scratch_bytes(n_groups, depth, B)))

    # The wide-tile dense kernels (128 rows x up to 256 samples, contraction split over CTAs) hold all operand rows of
    # eight samples in shared memory during their pre-pass: at most this many rows.
    DENSE_WIDE_MAX_DEPTH = 6144
    use_wide_dense = True

    def _wide_ok(self, p: int, B: int, backward: bool) -> bool:
        if not (self.use_dense_kernels and self.use_wide_dense) or B % 8 != 0 or _lib.sum_mode() == 0 or self._packer is None:
            return False
        if backward:
            depth = self._dev["bk"][p][1].size(1) * self.block_size
            return self._packed_bk[p] is not None and self.DENSE_MIN_DEPTH <= depth <= self.DENSE_WIDE_MAX_DEPTH
        depth = self._dev["fw"][p][1].size(1)
        return self._packed_fw[p] is not None and self.DENSE_MIN_DEPTH <= depth <= self.DENSE_WIDE_MAX_DEPTH

    def _wide_scratch(self, n_groups: int, depth: int, B: int):
        """Operand scratch of one wide-tile launch, shared by all layers (they run one after the other)."""
        scratch = self._packer.scratch(int(_lib.load().pcx_dense2_scratch_bytes(n_groups, depth, B)))
        return scratch, scratch.numel()

    def _forward_wide(self, p: int, node_mars, element_mars, fkids, fc: int):
        nids, cids, _, _ = self._dev["fw"][p]
        B = node_mars.size(1)
        row_group, group_row, n_groups = self._groups_fw[p]
        scratch, nbytes = self._wide_scratch(n_groups, cids.size(1), B)
        _lib.call("pcx_sum_fwd_dense2", node_mars, element_mars, self._packed_fw[p], nids, cids, fkids, fc, row_group,
                  group_row, n_groups, scratch, nbytes, nids.numel(), cids.size(1), self.block_size, B)

    def _backward_ele_wide(self, p: int, node_flows, element_flows, node_mars, element_mars, fkids, fc: int, direct: bool,
                           logspace_flows: bool):
        chids, parids, _ = self._dev["bk"][p]
        cbs = self.cs_block_sizes[p]
        B = node_flows.size(1)
        row_group, group_row, n_groups = self._groups_bk[p]
        scratch, nbytes = self._wide_scratch(n_groups, parids.size(1) * self.block_size, B)
        _lib.call("pcx_sum_bwd_ele_dense2", element_flows, element_mars, node_flows, node_mars, self._packed_bk[p], chids,
                  parids, fkids, fc, int(bool(direct)), row_group, group_row, n_groups, scratch, nbytes,
                  chids.numel(), parids.size(1), self.block_size, cbs, B, int(bool(logspace_flows)))

    use_dense_kernels = True
    use_sample_major = True          # tensor-core tiles of 128 samples x 32/64 nodes for small node blocks

    def _use_packed(self, params):
        if self._packer is None or _lib.sum_mode() == 0:
            return False
        self._packer.refresh(params)
        return True

    def _require_cuda(self):
        if self._dev is None:
            raise NotImplementedError("sum layers run on CUDA only (no CPU path)")

    def forward(self, node_mars: torch.Tensor, element_mars: torch.Tensor, params: torch.Tensor,
                propagation_alg: str = "LL", pflow_temperature: float = 1.0, **kwargs):
        self._require_cuda()
        _unsupported(pflow_temperature=abs(pflow_temperature - 1.0) > 1e-6)
        B = node_mars.size(1)
        alg, alpha = _alg_of(propagation_alg, kwargs)
        if alg != 0:                                      # "MPE" / "GeneralLL": plain fp32 kernels
            for nids, cids, pids, _ in self._dev["fw"]:
                _lib.call("pcx_sum_fwd_alg", node_mars, element_mars, params, nids, cids, pids, nids.numel(),
                          cids.size(1), self.block_size, B, alg, alpha)
            return
        packed = self._use_packed(params)
        for p, (nids, cids, pids, _) in enumerate(self._dev["fw"]):
            if packed and self._wide_ok(p, B, False):
                self._forward_wide(p, node_mars, element_mars, None, 0)
            elif packed and self._dense_ok(p, B, False):
                row_group, group_row, n_groups = self._groups_fw[p]
                scratch = self._dense_scratch(n_groups, cids.size(1), B)
                _lib.call("pcx_sum_fwd_dense", node_mars, element_mars, self._packed_fw[p], nids, cids, row_group,
                          group_row, n_groups, scratch, scratch.numel(), nids.numel(), cids.size(1), self.block_size, B)
            elif packed and self._packed_fw[p] is not None:
                _lib.call("pcx_sum_fwd_packed", node_mars, element_mars, self._packed_fw[p], nids, cids,
                          nids.numel(), cids.size(1), self.block_size, B)
            elif packed and self.use_sample_major and self._sm_fw[p] is not None:
                for nb, first_row, n_merged, buf in self._sm_fw[p]:
                    _lib.call("pcx_sum_fwd_sm", node_mars, element_mars, buf, first_row, nids, cids, None, n_merged, nb,
                              cids.size(1), B)
            else:
                _lib.call("pcx_sum_fwd", node_mars, element_mars, params, nids, cids, pids,
                          nids.numel(), cids.size(1), self.block_size, B)

    __call__ = forward

    # ---- product layer folded in (tables prepared by TensorCircuit._setup_fusion) ------------------------------
    def forward_fused(self, node_mars: torch.Tensor):
        B, f = node_mars.size(1), self._fusion
        if f.get("sm"):                                   # small blocks: sample-major tiles, products of two children
            for p, (nids, cids, _, _) in enumerate(self._dev["fw"]):
                for nb, first_row, n_merged, buf in self._sm_fw[p]:
                    _lib.call("pcx_sum_fwd_sm", node_mars, None, buf, first_row, nids, cids, f["fw"][p], n_merged, nb,
                              cids.size(1), B)
            return
        if f.get("dense"):                                # deep tables: the wide-tile dense kernels gather the products
            for p in range(self.num_fw_partitions):
                self._forward_wide(p, node_mars, None, f["fw"][p], f["fc"])
            return
        for p, (nids, cids, _, _) in enumerate(self._dev["fw"]):
            _lib.call("pcx_sum_fwd_fused", node_mars, self._packed_fw[p], nids, cids, f["fw"][p], f["fc"],
                      nids.numel(), cids.size(1), self.block_size, B)

    def backward_ele_fused(self, node_flows, element_flows, node_mars, logspace_flows: bool):
        B, f = node_flows.size(1), self._fusion
        if f.get("sm"):
            for p, ((chids, parids, _), cbs) in enumerate(zip(self._dev["bk"], self.cs_block_sizes)):
                for nb, first_row, n_merged, buf in self._sm_bk[p]:
                    _lib.call("pcx_sum_bwd_ele_sm", element_flows, None, node_flows, node_mars, buf, first_row, chids,
                              parids, f["bk"][p], cbs, n_merged, nb, parids.size(1), self.block_size, B,
                              int(bool(logspace_flows)))
            return
        if f.get("dense"):
            for p in range(self.num_bk_partitions):
                self._backward_ele_wide(p, node_flows, None if f["direct"] else element_flows, node_mars, None,
                                        f["bk"][p], f["fc"], f["direct"], logspace_flows)
            return
        for p, ((chids, parids, _), cbs) in enumerate(zip(self._dev["bk"], self.cs_block_sizes)):
            _lib.call("pcx_sum_bwd_ele_fused", element_flows, node_flows, node_mars, self._packed_bk[p], chids, parids,
                      f["bk"][p], f["fc"], int(f["direct"]), chids.numel(), parids.size(1), self.block_size, cbs, B,
                      int(bool(logspace_flows)))

    def backward_par_fused(self, node_flows, node_mars, params, param_flows, logspace_flows: bool):
        B, f = node_flows.size(1), self._fusion
        if f.get("sm"):
            for p, (nids, cids, pids, pfids) in enumerate(self._dev["fw"]):
                for nb, first_row, n_merged, _ in self._sm_fw[p]:
                    _lib.call("pcx_sum_bwd_par_sm", param_flows, node_flows, node_mars, None, params, first_row, nids,
                              cids, pids, pfids, f["fw"][p], n_merged, nb, self.block_size, cids.size(1), B,
                              int(bool(logspace_flows)))
            return
        for p, (nids, cids, pids, pfids) in enumerate(self._dev["fw"]):
            _lib.call("pcx_sum_bwd_par_fused", param_flows, node_flows, node_mars, params, nids, cids, pids, pfids,
                      f["fw"][p], f["fc"], nids.numel(), cids.size(1), self.block_size, B, int(bool(logspace_flows)))

    def backward(self, node_flows: torch.Tensor, element_flows: torch.Tensor, node_mars: torch.Tensor,
                 element_mars: torch.Tensor, params: torch.Tensor, param_flows: Optional[torch.Tensor] = None,
                 allow_modify_flows: bool = False, propagation_alg: str = "LL", logspace_flows: bool = False,
                 negate_pflows: bool = False, accumulate_ch_flows: bool = False, allow_neg_flows: bool = False,
                 pflow_temperature: float = 1.0, temper_eflow: bool = False, **kwargs):
        self._require_cuda()
        _unsupported(allow_modify_flows=allow_modify_flows,
                     negate_pflows=negate_pflows, accumulate_ch_flows=accumulate_ch_flows, allow_neg_flows=allow_neg_flows,
                     pflow_temperature=abs(pflow_temperature - 1.0) > 1e-6, temper_eflow=temper_eflow)
        B = node_flows.size(1)
        ls = int(bool(logspace_flows))
        alg, alpha = _alg_of(propagation_alg, kwargs)
        if alg != 0:                                      # "MPE" / "GeneralLL": plain fp32 kernels
            for (chids, parids, parpids), cbs in zip(self._dev["bk"], self.cs_block_sizes):
                _lib.call("pcx_sum_bwd_ele_alg", element_flows, element_mars, node_flows, node_mars, params, chids, parids,
                          parpids, chids.numel(), parids.size(1), self.block_size, cbs, B, ls, alg, alpha)
            if param_flows is not None:
                for nids, cids, pids, pfids in self._dev["fw"]:
                    _lib.call("pcx_sum_bwd_par_alg", param_flows, node_flows, node_mars, element_mars, params, nids, cids,
                              pids, pfids, nids.numel(), cids.size(1), self.block_size, B, ls, alg, alpha)
            return
        packed = self._use_packed(params)
        for p, ((chids, parids, parpids), cbs) in enumerate(zip(self._dev["bk"], self.cs_block_sizes)):
            if packed and self._wide_ok(p, B, True):
                self._backward_ele_wide(p, node_flows, element_flows, node_mars, element_mars, None, 0, False, ls)
            elif packed and self._dense_ok(p, B, True):
                row_group, group_row, n_groups = self._groups_bk[p]
                scratch = self._dense_scratch(n_groups, parids.size(1) * self.block_size, B)
                _lib.call("pcx_sum_bwd_ele_dense", element_flows, element_mars, node_flows, node_mars, self._packed_bk[p],
                          chids, parids, row_group, group_row, n_groups, scratch, scratch.numel(), chids.numel(),
                          parids.size(1), self.block_size, cbs, B, ls)
            elif packed and self._packed_bk[p] is not None:
                _lib.call("pcx_sum_bwd_ele_packed", element_flows, element_mars, node_flows, node_mars, self._packed_bk[p],
                          chids, parids, chids.numel(), parids.size(1), self.block_size, cbs, B, ls)
            elif packed and self.use_sample_major and self._sm_bk[p] is not None:
                for nb, first_row, n_merged, buf in self._sm_bk[p]:
                    _lib.call("pcx_sum_bwd_ele_sm", element_flows, element_mars, node_flows, node_mars, buf, first_row,
                              chids, parids, None, cbs, n_merged, nb, parids.size(1), self.block_size, B, ls)
            else:
                _lib.call("pcx_sum_bwd_ele", element_flows, element_mars, node_flows, node_mars, params,
                          chids, parids, parpids, chids.numel(), parids.size(1), self.block_size, cbs, B, ls)
        if param_flows is not None:
            stage = kwargs.get("dense_par_stage")
            for p, (nids, cids, pids, pfids) in enumerate(self._dev["fw"]):
                if (stage is not None and packed and (self._dense_ok(p, B, False) or self._wide_ok(p, B, False))
                        and self._groups_fw[p][2] == 1 and stage(self, p, node_flows, node_mars, element_mars, ls)):
                    continue                       # this table's flows come out of one product over all staged layers
                if (packed and self.use_sample_major and self._packed_fw[p] is None and self._sm_fw[p] is not None
                        and B % 8 == 0):
                    for nb, first_row, n_merged, _ in self._sm_fw[p]:
                        _lib.call("pcx_sum_bwd_par_sm", param_flows, node_flows, node_mars, element_mars, params,
                                  first_row, nids, cids, pids, pfids, None, n_merged, nb, self.block_size, cids.size(1), B, ls)
                    continue
                _lib.call("pcx_sum_bwd_par", param_flows, node_flows, node_mars, element_mars, params,
                          nids, cids, pids, pfids, nids.numel(), cids.size(1), self.block_size, B, ls)

    def __repr__(self):
        return f"SumLayer(nid_range={self._layer_nid_range}, num_nodes={self.num_nodes}, num_edges={self.num_edges})"


class LayerGroup(nn.Module):
    """Layers of one kind at one depth, evaluated one after the other (layer/layer_group.py:14-113)."""

    def __init__(self, layers: Sequence[Layer]):
        super().__init__()
        assert len(layers) >= 1, "A `LayerGroup` must contains at least 1 layer."
        first = layers[0]
        self.layer_type = "input" if first.is_input() else ("prod" if first.is_prod() else "sum")
        self.num_layers = len(layers)
        self.layers = list(layers)
        for i, layer in enumerate(self.layers):
            self.add_module(f"layer_{i}", layer)

    def to(self, device, **kwargs):
        for layer in self.layers:
            layer.to(device, **kwargs)
        return self

    def forward(self, *args, **kwargs):
        for layer in self.layers:
            layer.forward(*args, **kwargs)

    __call__ = forward

    def backward(self, *args, **kwargs):
        for layer in self.layers:
            layer.backward(*args, **kwargs)

    def is_input(self):
        return self.layer_type == "input"

    def is_prod(self):
        return self.layer_type == "prod"

    def is_sum(self):
        return self.layer_type == "sum"

    def __len__(self):
        return self.num_layers

    def __getitem__(self, idx):
        return self.layers[idx]

    def __iter__(self):
        return iter(self.layers)


def _fill(t: torch.Tensor, v: float):
    if t.is_cuda:
        _lib.call("pcx_fill_f32", t, t.numel(), float(v))
    else:
        t.fill_(v)


def _scale(t: torch.Tensor, v: float):
    if t.is_cuda:
        _lib.call("pcx_scale_f32", t, t.numel(), float(v))
    else:
        t.mul_(v)
