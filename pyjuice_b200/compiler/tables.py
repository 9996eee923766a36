"""Index-table builders for sum, product and input layers.

Every function here restates, with NumPy, what PyJuice's layer compiler emits
(layer/compilation.py, layer/sum_layer.py:139-306, layer/prod_layer.py:31-159,
layer/input_layer.py:38-246).  The tables are int64 and must come out bit-identical: they fix
the memory layout of parameters and flows that every kernel and every accessor relies on.

Conventions (shared with the kernels):
  * id 0 in any child / parent / parameter table means "padding"; row 0.. of the value buffers
    and parameter 0.. are dummies that make padded entries contribute nothing;
  * ``pids[row, e]`` addresses the ``block_size`` consecutive parameters (node index fastest) of
    child node ``e`` of node block ``row``; a (node block, child block) pair is a contiguous
    ``[ch_block_size, block_size]`` tile starting at ``parpids``.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np
import torch

from .partition import assign_partitions, partition_maxima


def _np(t) -> np.ndarray:
    return t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else np.asarray(t)


def _rank_within_group(keys: np.ndarray, num_groups: int) -> np.ndarray:
    """rank[k] = number of earlier positions with the same key (order of appearance)."""
    order = np.argsort(keys, kind="stable")
    sorted_keys = keys[order]
    starts = np.zeros(num_groups + 1, dtype=np.int64)
    np.add.at(starts, sorted_keys + 1, 1)
    starts = np.cumsum(starts)
    rank = np.empty(keys.shape[0], dtype=np.int64)
    rank[order] = np.arange(keys.shape[0], dtype=np.int64) - starts[sorted_keys]
    return rank


class _IdDict:
    """Insertion-ordered mapping keyed by object identity (node vectors are compared by identity)."""

    def __init__(self):
        self._keys, self._vals = {}, {}

    def __contains__(self, k):
        return id(k) in self._keys

    def __getitem__(self, k):
        return self._vals[id(k)]

    def __setitem__(self, k, v):
        self._keys[id(k)] = k
        self._vals[id(k)] = v

    def items(self):
        return [(self._keys[i], self._vals[i]) for i in self._keys]

    def __len__(self):
        return len(self._keys)


# --------------------------------------------------------------------------------------------
# Sum layers
# --------------------------------------------------------------------------------------------

def _assign_sum_ranges(nodes, pid_start, pfid_start, node2tiednodes: _IdDict, max_tied: int):
    """Parameter / flow ranges of every vector of the layer, in list order
    (layer/compilation.py:312-391).  Returns per-vector (ns_pid_start, ns_pfid_start,
    add_params, add_flows) plus the advanced global counters."""
    out = []
    local_counts = _IdDict()     # per-layer occupancy of every flow accumulator of a source
    untied_idx = []
    for idx, ns in enumerate(nodes):
        if not ns.is_tied():
            if getattr(ns, "_param_range", None) is None:
                ns._param_range = (pid_start, pid_start + ns.num_edges)
                pid_start += ns.num_edges
                ns._param_flow_range = (pfid_start, pfid_start + ns.num_edges)
                pfid_start += ns.num_edges
                add_p = add_f = True
            else:
                assert getattr(ns, "_param_flow_range", None) is not None
                add_p = add_f = False
            untied_idx.append(idx)
            out.append((ns._param_range[0], ns._param_flow_range[0], add_p, add_f))
            continue

        src = ns.get_source_ns()
        if getattr(src, "_param_range", None) is None:
            ns._param_range = (pid_start, pid_start + ns.num_edges)
            ns._param_flow_range = (pfid_start, pfid_start + ns.num_edges)
            src._param_range = tuple(ns._param_range)
            src._param_flow_range = tuple(ns._param_flow_range)
            pid_start += ns.num_edges
            pfid_start += ns.num_edges
            add_p = add_f = True
        else:
            ns._param_range = tuple(src._param_range)
            add_p = add_f = False

        if src not in node2tiednodes:
            node2tiednodes[src] = [[src], [src._param_flow_range]]
            local_counts[src] = [1]
        elif src not in local_counts:
            local_counts[src] = [0] * len(node2tiednodes[src][0])

        if getattr(ns, "_param_flow_range", None) is None:
            counts = local_counts[src]
            if all(c >= max_tied for c in counts):
                ns._param_flow_range = (pfid_start, pfid_start + ns.num_edges)
                pfid_start += ns.num_edges
                node2tiednodes[src][1].append(ns._param_flow_range)
                node2tiednodes[src][0].append(ns)
                counts.append(1)
                add_f = True
            else:
                target = min(range(len(counts)), key=lambda i: counts[i])
                ns._param_flow_range = tuple(node2tiednodes[src][1][target])
                counts[target] += 1
                add_f = False
        out.append((src._param_range[0], ns._param_flow_range[0], add_p, add_f))
    return out, untied_idx, pid_start, pfid_start


def compile_sum_forward(nodes, global_nid_start: int, pid_start: int, pfid_start: int, node2tiednodes: _IdDict,
                        layer_sparsity_tol, max_num_partitions, max_tied: int):
    """Forward tables of one sum layer.

    Returns dict(nids, cids, pids, pfids: lists of torch int64 tensors per partition;
    num_nodes, num_edges, pid_end, pfid_end).  Side effects on the vectors: ``_output_ind_range``,
    ``_param_range``, ``_param_flow_range``, ``_param_ids``, ``_param_flow_ids``,
    ``_inverse_param_ids``.
    """
    bs = nodes[0].block_size
    # node ids and fan-ins (layer/compilation.py:107-126)
    fan_in = []
    nid = global_nid_start
    num_edges = 0
    for ns in nodes:
        cnt = np.bincount(_np(ns.edge_ids[0]), minlength=ns.num_node_blocks).astype(np.int64)
        fan_in.append(cnt * ns.ch_block_size)
        ns._output_ind_range = (nid, nid + ns.num_nodes)
        nid += ns.num_nodes
        num_edges += ns.num_edges
    n_chs = np.concatenate(fan_in)
    num_blocks = n_chs.shape[0]

    maxima = partition_maxima(n_chs, max_num_partitions, layer_sparsity_tol)
    part, rank, sizes = assign_partitions(n_chs, maxima, first_min=1)

    nids = [np.zeros(int(sizes[p]), dtype=np.int64) for p in range(len(maxima))]
    cids = [np.zeros((int(sizes[p]), int(maxima[p])), dtype=np.int64) for p in range(len(maxima))]
    pids = [np.zeros_like(c) for c in cids]
    pfids = [np.zeros_like(c) for c in cids]

    ranges, untied_idx, pid_end, pfid_end = _assign_sum_ranges(nodes, pid_start, pfid_start, node2tiednodes, max_tied)

    blk0 = 0
    param_ids: Dict[int, np.ndarray] = {}
    flow_ids: Dict[int, np.ndarray] = {}
    for idx, ns in enumerate(nodes):
        ns_pid, ns_pfid, add_p, add_f = ranges[idx]
        cbs = ns.ch_block_size
        eb = _np(ns.edge_ids).astype(np.int64)                      # [2, Eb] block edges
        nb = ns.num_node_blocks
        cnt = np.bincount(eb[0], minlength=nb).astype(np.int64)
        brank = _rank_within_group(eb[0], nb)                        # block-level column of each edge
        cum_nodes = np.zeros(nb, dtype=np.int64)                     # child nodes before block i
        cum_nodes[1:] = np.cumsum(cnt[:-1] * cbs)

        # which child vector each block edge points into, and that vector's first element id
        ch_blocks = np.array([c.num_node_blocks for c in ns.chs], dtype=np.int64)
        ch_block_end = np.cumsum(ch_blocks)
        ch_block_beg = ch_block_end - ch_blocks
        ch_first = np.array([c._output_ind_range[0] for c in ns.chs], dtype=np.int64)
        which = np.searchsorted(ch_block_end, eb[1], side="right")
        child_first_node = ch_first[which] + (eb[1] - ch_block_beg[which]) * cbs   # [Eb]

        # expand to child nodes: column = brank * cbs + j
        j = np.arange(cbs, dtype=np.int64)
        cols = (brank[:, None] * cbs + j[None, :])                    # [Eb, cbs]
        node_cids = child_first_node[:, None] + j[None, :]
        gp = (cum_nodes[eb[0]][:, None] + cols) * bs                  # offset from the vector's start
        p_of = part[blk0 + eb[0]]
        r_of = rank[blk0 + eb[0]]
        for p in np.unique(p_of):
            sel = p_of == p
            rr = np.broadcast_to(r_of[sel][:, None], cols[sel].shape)
            cids[p][rr, cols[sel]] = node_cids[sel]
            pids[p][rr, cols[sel]] = ns_pid + gp[sel]
            pfids[p][rr, cols[sel]] = ns_pfid + gp[sel]
        blocks = np.arange(nb, dtype=np.int64)
        for p in np.unique(part[blk0:blk0 + nb]):
            sel = part[blk0:blk0 + nb] == p
            nids[p][rank[blk0:blk0 + nb][sel]] = ns._output_ind_range[0] + blocks[sel] * bs

        if add_p:
            param_ids[idx] = ns_pid + gp[:, 0]
        if add_f:
            flow_ids[idx] = ns_pfid + gp[:, 0]
        blk0 += nb

    for idx, ids in param_ids.items():
        tgt = nodes[idx].get_source_ns() if nodes[idx].is_tied() else nodes[idx]
        tgt._param_ids = torch.from_numpy(ids.copy())
    for idx, ids in flow_ids.items():
        nodes[idx]._param_flow_ids = torch.from_numpy(ids.copy())
    for idx in untied_idx:
        nodes[idx]._inverse_param_ids = torch.argsort(nodes[idx]._param_ids)

    to_t = lambda lst: [torch.from_numpy(a) for a in lst]
    return dict(nids=to_t(nids), cids=to_t(cids), pids=to_t(pids), pfids=to_t(pfids),
                num_nodes=num_blocks * bs, num_edges=num_edges, pid_end=pid_end, pfid_end=pfid_end)


def compile_sum_backward(nodes, layer_sparsity_tol, max_num_partitions):
    """Backward (child-major) tables of one sum layer: per child block, its parent node blocks and
    the parameter tile of each (layer/compilation.py:129-174, 696-858; sum_layer.py:241-306)."""
    # child vectors grouped by block size, first-seen order; parents per child, first-seen order
    groups: Dict[int, List] = {}
    parents = _IdDict()
    for ns in nodes:
        for cs in ns.chs:
            g = groups.setdefault(cs.block_size, [])
            if not any(c is cs for c in g):
                g.append(cs)
            if cs not in parents:
                parents[cs] = []
            if not any(p is ns for p in parents[cs]):
                parents[cs].append(ns)

    per_ns = _IdDict()   # block-level rank / cumulative edge counts of every parent vector

    def ns_stats(ns):
        if ns not in per_ns:
            eb = _np(ns.edge_ids).astype(np.int64)
            cnt = np.bincount(eb[0], minlength=ns.num_node_blocks).astype(np.int64)
            cum = np.zeros(ns.num_node_blocks, dtype=np.int64)
            cum[1:] = np.cumsum(cnt[:-1])
            per_ns[ns] = (eb, _rank_within_group(eb[0], ns.num_node_blocks), cum)
        return per_ns[ns]

    chids_all, parids_all, parpids_all, cs_sizes = [], [], [], []
    for cbs, chs in groups.items():
        # gather, per child vector, the block edges of every parent that point into it
        gathered = []
        n_pargs = []
        for cs in chs:
            items = []
            counts = np.zeros(cs.num_node_blocks, dtype=np.int64)
            for ns in parents[cs]:
                eb, brank, cum = ns_stats(ns)
                k = [i for i, c in enumerate(ns.chs) if c is cs][0]
                beg = sum(c.num_node_blocks for c in ns.chs[:k])
                sel = (eb[1] >= beg) & (eb[1] < beg + cs.num_node_blocks)
                par_blk = eb[0][sel]
                ch_blk = eb[1][sel] - beg
                counts += np.bincount(ch_blk, minlength=cs.num_node_blocks)
                items.append((ns, par_blk, ch_blk, cum[par_blk] + brank[sel]))
            gathered.append(items)
            n_pargs.append(counts)
        n_pargs_cat = np.concatenate(n_pargs)

        maxima = partition_maxima(n_pargs_cat, max_num_partitions, layer_sparsity_tol)
        part, rank, sizes = assign_partitions(n_pargs_cat, maxima, first_min=1)
        chids = [np.zeros(int(sizes[p]), dtype=np.int64) for p in range(len(maxima))]
        parids = [np.zeros((int(sizes[p]), int(maxima[p])), dtype=np.int64) for p in range(len(maxima))]
        parpids = [np.zeros_like(a) for a in parids]

        blk0 = 0
        for cs, items in zip(chs, gathered):
            ncb = cs.num_node_blocks
            # column of every (parent edge -> child block): order over (parent vector, edge order)
            all_ch = np.concatenate([it[2] for it in items]) if items else np.zeros(0, dtype=np.int64)
            col_all = _rank_within_group(all_ch, ncb)
            off = 0
            for ns, par_blk, ch_blk, tile_idx in items:
                n = par_blk.shape[0]
                col = col_all[off:off + n]
                off += n
                ns_pid = (ns.get_source_ns() if ns.is_tied() else ns)._param_range[0]
                p_of = part[blk0 + ch_blk]
                r_of = rank[blk0 + ch_blk]
                for p in np.unique(p_of):
                    sel = p_of == p
                    chids[p][r_of[sel]] = cs._output_ind_range[0] + ch_blk[sel] * cbs
                    parids[p][r_of[sel], col[sel]] = ns._output_ind_range[0] + par_blk[sel] * ns.block_size
                    parpids[p][r_of[sel], col[sel]] = ns_pid + tile_idx[sel] * ns.block_size * cbs
            blk0 += ncb

        chids_all += chids
        parids_all += parids
        parpids_all += parpids
        cs_sizes += [cbs] * len(maxima)

    to_t = lambda lst: [torch.from_numpy(a) for a in lst]
    return dict(chids=to_t(chids_all), parids=to_t(parids_all), parpids=to_t(parpids_all), cs_block_sizes=cs_sizes)


# --------------------------------------------------------------------------------------------
# Product layers
# --------------------------------------------------------------------------------------------

def compile_prod(nodes, global_nid_start: int, layer_sparsity_tol, max_num_partitions):
    """Forward and backward tables of one product layer (layer/prod_layer.py:31-159,
    layer/compilation.py:863-1185)."""
    block_sparse = all((not ns.is_sparse()) and ns.block_size == nodes[0].block_size for ns in nodes)
    bs = nodes[0].block_size if block_sparse else 1

    # element ids, per-row fan-in
    n_chgs = []
    eid = global_nid_start
    num_edges = 0
    for ns in nodes:
        rows = ns.num_node_blocks if block_sparse else ns.num_nodes
        n_chgs.append(np.full(rows, ns.num_chs, dtype=np.int64))
        ns._output_ind_range = (eid, eid + ns.num_nodes)
        eid += ns.num_nodes
        num_edges += ns.num_nodes * ns.num_chs
    n_chgs = np.concatenate(n_chgs)
    num_rows = n_chgs.shape[0]

    maxima = partition_maxima(n_chgs, max_num_partitions, layer_sparsity_tol)
    sizes = np.zeros(len(maxima), dtype=np.int64)
    placement = []
    for ns in nodes:
        p = int((ns.num_chs > maxima).sum())
        placement.append((p, int(sizes[p])))
        sizes[p] += ns.num_node_blocks if block_sparse else ns.num_nodes

    nids = [np.zeros(int(sizes[p]), dtype=np.int64) for p in range(len(maxima))]
    cids = [np.zeros((int(sizes[p]), int(maxima[p])), dtype=np.int64) for p in range(len(maxima))]
    for ns, (p, r0) in zip(nodes, placement):
        first = ns._output_ind_range[0]
        eb = _np(ns.edge_ids).astype(np.int64)
        if block_sparse:
            r1 = r0 + ns.num_node_blocks
            nids[p][r0:r1] = first + np.arange(0, ns.num_nodes, bs, dtype=np.int64)
            for k, cs in enumerate(ns.chs):
                cids[p][r0:r1, k] = eb[:, k] * bs + cs._output_ind_range[0]
        else:
            r1 = r0 + ns.num_nodes
            nids[p][r0:r1] = first + np.arange(0, ns.num_nodes, dtype=np.int64)
            if not ns.is_sparse():
                j = np.arange(ns.block_size, dtype=np.int64)
                eb = (eb[:, None, :] * ns.block_size + j[None, :, None]).reshape(-1, eb.shape[1])
            for k, cs in enumerate(ns.chs):
                cids[p][r0:r1, k] = eb[:, k] + cs._output_ind_range[0]

    # backward: unique children with their parents, in order of appearance over the flattened
    # forward tables (partition-major, row-major)
    flat_cids = np.concatenate([c.reshape(-1) for c in cids])
    flat_par = np.concatenate([np.repeat(n, c.shape[1]) for n, c in zip(nids, cids)])
    u_cids, par_counts = np.unique(flat_cids, return_counts=True)
    keep = u_cids >= global_nid_start          # prod_layer.py:117 / compilation.py:980-993
    below = np.nonzero(~keep)[0]
    if below.size > 0:
        cut = int(below.max()) + 1
        u_cids, par_counts = u_cids[cut:], par_counts[cut:]

    bk_maxima = partition_maxima(par_counts, max_num_partitions, layer_sparsity_tol)
    bpart, brank, bsizes = assign_partitions(par_counts, bk_maxima, first_min=0)
    out_u = [np.zeros(int(bsizes[p]), dtype=np.int64) for p in range(len(bk_maxima))]
    out_par = [np.zeros((int(bsizes[p]), int(bk_maxima[p])), dtype=np.int64) for p in range(len(bk_maxima))]
    for p in range(len(bk_maxima)):
        sel = bpart == p
        out_u[p][brank[sel]] = u_cids[sel]
    # k-th parent of a child = k-th occurrence of the child in flat_cids
    pos = np.searchsorted(u_cids, flat_cids)
    pos_ok = (pos < u_cids.shape[0])
    pos_c = np.where(pos_ok, pos, 0)
    valid = pos_ok & (u_cids[pos_c] == flat_cids) if u_cids.shape[0] > 0 else np.zeros_like(pos_ok)
    vpos = pos[valid]
    occ = _rank_within_group(vpos, max(int(u_cids.shape[0]), 1))
    vpar = flat_par[valid]
    for p in range(len(bk_maxima)):
        sel = bpart[vpos] == p
        out_par[p][brank[vpos[sel]], occ[sel]] = vpar[sel]

    to_t = lambda lst: [torch.from_numpy(a) for a in lst]
    return dict(block_size=bs, block_sparse=block_sparse, num_nodes=num_rows * bs, num_edges=num_edges,
                nids=to_t(nids), cids=to_t(cids), u_cids=to_t(out_u), parids=to_t(out_par))


# --------------------------------------------------------------------------------------------
# Input layers
# --------------------------------------------------------------------------------------------

def reorder_input_nodes(nodes):
    """Untied vectors first (a tied vector pulls its source forward if needed), tied ones after,
    otherwise keeping the given order (layer/input_layer.py:1101-1129)."""
    in_layer = {id(ns) for ns in nodes}
    added = set()
    untied, tied = [], []
    for ns in nodes:
        if id(ns) in added:
            continue
        if not ns.is_tied():
            untied.append(ns)
            added.add(id(ns))
            continue
        src = ns.get_source_ns()
        if id(src) in added:
            tied.append(ns)
            added.add(id(ns))
        elif id(src) in in_layer:
            untied.append(src)
            tied.append(ns)
            added.update((id(ns), id(src)))
        else:
            raise ValueError("A tied `InputNodes` should be in the same layer with its source nodes.")
    out = untied + tied
    assert len(out) == len(nodes), "Total node length should not change after reordering."
    return out


def compile_input(nodes, cum_nodes: int, max_tied: int):
    """Per-node tables of one input layer (layer/input_layer.py:66-246).  ``nodes`` must already be
    reordered.  Returns a dict of torch tensors plus the tied-accumulator list."""
    layer_first = cum_nodes
    cum_params = cum_flows = cum_sources = 0
    accum = _IdDict()     # source -> [vectors that opened an accumulator, users of the current one, current range]
    for ns in nodes:
        ns._output_ind_range = (cum_nodes, cum_nodes + ns.num_nodes)
        cum_nodes += ns.num_nodes
        npar, nflow = ns.dist.num_parameters(), ns.dist.num_param_flows()
        if not ns.is_tied():
            ns._param_range = (cum_params, cum_params + ns.num_nodes * npar)
            cum_params += ns.num_nodes * npar
            ns._param_flow_range = (cum_flows, cum_flows + ns.num_nodes * nflow)
            cum_flows += ns.num_nodes * nflow
            cum_sources += ns.num_nodes
        else:
            src = ns.get_source_ns()
            ns._param_range = tuple(src._param_range)
            if src not in accum:
                accum[src] = [[src], 1, src._param_flow_range]
            entry = accum[src]
            if entry[1] >= max_tied:
                ns._param_flow_range = (cum_flows, cum_flows + ns.num_nodes * nflow)
                cum_flows += ns.num_nodes * nflow
                entry[2] = ns._param_flow_range
                entry[0].append(ns)
                entry[1] = 1
            else:
                ns._param_flow_range = tuple(entry[2])
                entry[1] += 1
    num_nodes = cum_nodes - layer_first

    num_vars = len(nodes[0].scope.to_list())
    vids = np.empty((num_nodes, num_vars), dtype=np.int64)
    s_pids = np.empty(num_nodes, dtype=np.int64)
    s_pfids = np.empty(num_nodes, dtype=np.int64)
    s_mids = np.empty(num_nodes, dtype=np.int64)
    nids = np.zeros(num_nodes, dtype=np.int64)
    source_nids = np.empty(cum_sources, dtype=np.int64)
    node_id2source_id = np.empty(num_nodes, dtype=np.int64)
    metadata: List[float] = []
    n0 = s0 = 0
    var_seen: Dict[int, int] = {}
    local_range = _IdDict()
    for ns in nodes:
        n1 = n0 + ns.num_nodes
        local_range[ns] = (n0, n1)
        scope_vars = ns.scope.to_list()
        assert len(scope_vars) == num_vars
        vids[n0:n1, :] = np.asarray(scope_vars, dtype=np.int64)[None, :]
        npar, nflow = ns.dist.num_parameters(), ns.dist.num_param_flows()
        s_pids[n0:n1] = ns._param_range[0] + np.arange(ns.num_nodes, dtype=np.int64) * npar if npar > 0 else 0
        s_pfids[n0:n1] = ns._param_flow_range[0] + np.arange(ns.num_nodes, dtype=np.int64) * nflow if nflow > 0 else 0
        if not ns.is_tied():
            source_nids[s0:s0 + ns.num_nodes] = np.arange(n0, n1)
            s0 += ns.num_nodes
            node_id2source_id[n0:n1] = -1
        else:
            a, b = local_range[ns.get_source_ns()]
            node_id2source_id[n0:n1] = np.arange(a, b)
        s_mids[n0:n1] = len(metadata)
        metadata.extend(ns.dist.get_metadata())
        if num_vars == 1:
            v = scope_vars[0]
            nids[n0:n1] = np.arange(n1 - n0) + var_seen.get(v, 0)
            var_seen[v] = var_seen.get(v, 0) + (n1 - n0)
        n0 = n1

    tied2source = []
    for src, entry in accum.items():
        if len(entry[0]) > 1:
            ch = torch.tensor([c._param_flow_range[0] for c in entry[0]], dtype=torch.long)
            tied2source.append([src._param_flow_range[0], src._param_flow_range[1] - src._param_flow_range[0], ch])

    t = torch.from_numpy
    return dict(vids=t(vids), s_pids=t(s_pids), s_pfids=t(s_pfids), s_mids=t(s_mids), nids=t(nids),
                source_nids=t(source_nids), node_id2source_id=t(node_id2source_id),
                metadata=torch.tensor(metadata).float(), tied2source_nids=tied2source,
                num_nodes=num_nodes, num_parameters=cum_params, num_param_flows=cum_flows,
                output_ind_range=(layer_first, cum_nodes))


# --------------------------------------------------------------------------------------------
# EM work items and tied-flow fusing tables
# --------------------------------------------------------------------------------------------

def compile_par_update(root_ns, BLOCK_SIZE: int = 32):
    """One work item per (sum node, chunk of <= BLOCK_SIZE child nodes) of every untied sum vector,
    in DFS post-order (model/backend/par_update.py:15-45, 48-154).  Returns the six int64 tables
    ``[par_start_ids, pflow_start_ids, blk_sizes, blk_intervals, global_nids, nchs]``, a zeroed
    ``cum_pflows`` and the metadata dict."""
    cols = [[] for _ in range(6)]
    global_nid = 0
    for ns in root_ns:
        if not ns.is_sum() or ns.is_tied():
            continue
        bs, cbs = ns.block_size, ns.ch_block_size
        cnt = np.bincount(_np(ns.edge_ids[0]), minlength=ns.num_node_blocks).astype(np.int64)
        fan = cnt * cbs
        blk_par0 = ns._param_range[0] + np.concatenate(([0], np.cumsum(fan[:-1] * bs)))
        blk_flow0 = ns._param_flow_range[0] + np.concatenate(([0], np.cumsum(fan[:-1] * bs)))
        g = np.arange(bs, dtype=np.int64)
        for i in range(ns.num_node_blocks):
            f = int(fan[i])
            sid = np.arange(0, f, BLOCK_SIZE, dtype=np.int64)
            size = np.minimum(sid + BLOCK_SIZE, f) - sid
            shape = (sid.shape[0], bs)
            cols[0].append((blk_par0[i] + sid[:, None] * bs + g[None, :]).reshape(-1))
            cols[1].append((blk_flow0[i] + sid[:, None] * bs + g[None, :]).reshape(-1))
            cols[2].append(np.broadcast_to(size[:, None], shape).reshape(-1))
            cols[3].append(np.full(shape[0] * bs, bs, dtype=np.int64))
            cols[4].append(np.broadcast_to((global_nid + g)[None, :], shape).reshape(-1))
            cols[5].append(np.full(shape[0] * bs, f, dtype=np.int64))
            global_nid += bs
    tables = [torch.from_numpy(np.ascontiguousarray(np.concatenate(c).astype(np.int64))) for c in cols]
    tot = int(tables[4][-1].item()) + 1
    return tables + [torch.zeros([tot], dtype=torch.float32), {"tot_num_nodes": tot, "BLOCK_SIZE": BLOCK_SIZE}]


def compile_cum_par_flows(node2tiednodes: _IdDict, MAX_NBLOCKS: int = 2048, BLOCK_SIZE: int = 2048):
    """Tables that add the flow accumulators of a tied sum vector into its source's range
    (model/backend/parflow_fusing.py:11-62).  One entry per power-of-two accumulator count:
    ``[target_pfids, block_sizes, child_pfids, BLOCK_G, BLOCK_M]``; ``child_pfids`` rows are padded
    with 0 up to ``BLOCK_G``."""
    specs: Dict[int, list] = {}
    for src, item in node2tiednodes.items():
        if len(item[0]) <= 1:
            continue
        assert len(item[0]) <= MAX_NBLOCKS
        nblock = 1 << (len(item[0]) - 1).bit_length()
        specs.setdefault(nblock, []).append(
            (src._param_flow_range[0], src._param_flow_range[1] - src._param_flow_range[0],
             [c._param_flow_range[0] for c in item[0]]))
    out = []
    for G, lst in specs.items():
        M = BLOCK_SIZE // G
        tgt, sizes, chs = [], [], []
        for start, n, ch_starts in lst:
            for b0 in range(0, n, M):
                tgt.append(start + b0)
                sizes.append(min(b0 + M, n) - b0)
                chs.append([c + b0 for c in ch_starts] + [0] * (G - len(ch_starts)))
        out.append([torch.tensor(tgt), torch.tensor(sizes), torch.tensor(chs), G, M])
    return out
