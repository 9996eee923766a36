"""CPU oracle for the compiled probabilistic-circuit forward / backward / mini-batch-EM path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file; it exists so that
tests, the smoke check and the CPU-baseline leg of the benchmark have an independent statement of
what the CUDA kernels must compute.  It is a plain PyTorch (CPU, float64 by default) restatement
of PyJuice's algorithm, driven purely by the compiled index tables:

  * input forward    log p[s_pids[n] + x[vids[n], b]]                nodes/distributions/categorical.py:82-91
  * product forward  sum of child rows                                layer/prod_layer.py:161-166, layer/kernels/prod.py:156-226
  * sum forward      log sum_e theta[pids+m] exp(emars[cids])         layer/sum_layer.py:1077-1082, layer/kernels/sum_forward_block_sparse.py:79-124
  * root flows / driver order                                         model/tensorcircuit.py:355-441, 527-674
  * element flows    emars + log sum_n theta exp(nflow - nmar)        layer/sum_layer.py:2679-2692, layer/kernels/sum_backward_element_block_sparse.py:86-190
  * parameter flows  theta * sum_b exp(nflow - nmar + emar)           layer/sum_layer.py:2712-2722, layer/kernels/sum_backward_param_block_sparse.py:64-142
  * product backward logaddexp-accumulate of parent flows             layer/prod_layer.py:207-238, layer/kernels/prod.py:192-226
  * input backward   flows[s_pfids[n] + x] += exp(node_flows)         nodes/distributions/categorical.py:93-100
  * tied accumulate  source range := sum of accumulators              model/backend/parflow_fusing.py:80-99, layer/input_layer.py:1391-1411
  * EM update        (1-eta) theta + eta (F + alpha/nch)/(sum F + alpha)   model/backend/par_update.py:173-256, categorical.py:191-228

Pinning.  Tables: the compiled tables the oracle is driven by are checked bit-for-bit against the reference
compiler's output (tests/golden/*.npz, tests/test_tables_golden.py).  Values: tests/golden/values_<case>.npz hold
what the reference ITSELF computes on a B200 (its Triton path through its public API: log-likelihoods, node values,
node flows, parameter flows, post-EM parameters; written by tests/golden/make_values.py), and
tests/test_reference_values.py checks every function below against them.  tests/test_oracle_pins.py adds the
closed-form dense restatements that the reference's own tests assert (tests/model/simple_model_test.py:191-528,
tests/structures/hmm_correctness_test.py) and an autograd evaluator that shares no code with this file.

Two behaviours of the reference's kernels that change results beyond rounding are reproduced only when
``reference_compat=True`` is passed (product nodes without a sum parent; padding slots of the tied-flow fusing
kernel); by default flows are the exact gradients of the log-likelihood.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

NEG_INF = float("-inf")


class OracleState:
    """All buffers of one forward/backward/EM pass, named as in ``TensorCircuit``."""

    def __init__(self):
        self.node_mars = self.element_mars = self.node_flows = self.element_flows = None
        self.param_flows = None
        self.input_param_flows = []
        self.cache = {}                 # parameter blocks gathered per distinct index table (see `_gathered`)


def _tables(pc):
    """Pull the index tables out of a compiled circuit (ours or the reference's) as CPU tensors."""
    t = dict(num_nodes=pc.num_nodes, num_elements=pc.num_elements, root=tuple(pc._root_node_range),
             num_param_flows=pc.num_param_flows, inputs=[], inner=[])
    for layer in pc.input_layer_group:
        t["inputs"].append(dict(
            vids=layer.vids.cpu(), s_pids=layer.s_pids.cpu(), s_pfids=layer.s_pfids.cpu(),
            source_nids=layer.source_nids.cpu(), metadata=layer.metadata.cpu(), s_mids=layer.s_mids.cpu(),
            rng=tuple(layer._output_ind_range), num_param_flows=layer.num_param_flows,
            tied=[(a, b, c.cpu()) for a, b, c in layer.tied2source_nids]))
    for group in pc.inner_layer_groups:
        layers = []
        for layer in group:
            if group.is_prod():
                layers.append(dict(kind="prod", bs=layer.block_size,
                                   nids=[x.cpu() for x in layer.partitioned_nids], cids=[x.cpu() for x in layer.partitioned_cids],
                                   u_cids=[x.cpu() for x in layer.partitioned_u_cids], parids=[x.cpu() for x in layer.partitioned_parids]))
            else:
                layers.append(dict(kind="sum", bs=layer.block_size,
                                   nids=[x.cpu() for x in layer.partitioned_nids], cids=[x.cpu() for x in layer.partitioned_cids],
                                   pids=[x.cpu() for x in layer.partitioned_pids], pfids=[x.cpu() for x in layer.partitioned_pfids],
                                   chids=[x.cpu() for x in layer.partitioned_chids], parids=[x.cpu() for x in layer.partitioned_parids],
                                   parpids=[x.cpu() for x in layer.partitioned_parpids], cs_block_sizes=list(layer.cs_block_sizes)))
        t["inner"].append(("prod" if group.is_prod() else "sum", layers))
    return t


def _lse(x, dim):
    m = x.max(dim=dim, keepdim=True).values
    m = torch.where(torch.isinf(m) & (m < 0), torch.zeros_like(m), m)
    return (x - m).exp().sum(dim=dim).log() + m.squeeze(dim)


def _prod_forward(layer, node_mars, element_mars):
    j = torch.arange(layer["bs"])
    for nids, cids in zip(layer["nids"], layer["cids"]):
        rows = (cids[:, :, None] + j[None, None, :])                 # [n, C, bs]
        vals = node_mars[rows]                                       # [n, C, bs, B]
        vals = torch.where((cids == 0)[:, :, None, None], torch.zeros_like(vals), vals)
        element_mars[(nids[:, None] + j[None, :]).reshape(-1)] = vals.sum(dim=1).reshape(-1, vals.size(-1))


def _row_chunks(n_rows, per_row_elems, budget=32_000_000):
    step = max(1, budget // max(per_row_elems, 1))
    for r0 in range(0, n_rows, step):
        yield r0, min(r0 + step, n_rows)


def _neg_inf_like(x):
    return torch.full_like(x, NEG_INF)


def _table_key(*tables):
    """Identity of index tables by content: layers with tied parameters carry equal tables."""
    return tuple((tuple(t.shape), hash(t.numpy().tobytes())) for t in tables)


def _gathered(cache, key, make):
    """Parameter blocks gathered through an index table, computed once per distinct table (tied layers share them)."""
    if cache is None:
        return make()
    if key not in cache:
        cache[key] = make()
    return cache[key]


def _sum_forward(layer, node_mars, element_mars, params, cache=None):
    m = torch.arange(layer["bs"])
    B = node_mars.size(1)
    for nids, cids, pids in zip(layer["nids"], layer["cids"], layer["pids"]):
        K = cids.size(1)
        pkey = _table_key(pids) if cache is not None else None
        for r0, r1 in _row_chunks(nids.numel(), K * (B + layer["bs"])):
            em = element_mars[cids[r0:r1]]                           # [n, K, B]
            th = _gathered(cache, ("fw", pkey, r0, r1),
                           lambda: params[pids[r0:r1, :, None] + m[None, None, :]])     # [n, K, bs]
            mx = em.max(dim=1).values                                # [n, B]
            dead = torch.isinf(mx) & (mx < 0)
            mx0 = torch.where(dead, torch.zeros_like(mx), mx)
            acc = torch.bmm(th.transpose(1, 2), (em - mx0[:, None, :]).exp())   # [n, bs, B]
            out = acc.log() + mx0[:, None, :]
            out = torch.where(dead[:, None, :], _neg_inf_like(out), out)
            node_mars[(nids[r0:r1, None] + m[None, :]).reshape(-1)] = out.reshape(-1, B)


def _sum_backward(layer, st, params, compute_param_flows, cache=None, pending=None):
    bs = layer["bs"]
    n = torch.arange(bs)
    B = st.node_mars.size(1)
    # element flows
    for chids, parids, parpids, cbs in zip(layer["chids"], layer["parids"], layer["parpids"], layer["cs_block_sizes"]):
        c = torch.arange(cbs)
        P = parids.size(1)
        bkey = _table_key(parpids) if cache is not None else None
        for r0, r1 in _row_chunks(chids.numel(), P * bs * (2 * B + cbs)):
            pr, pp = parids[r0:r1], parpids[r0:r1]                   # [r, P]
            rows = (pr[:, :, None] + n[None, None, :]).reshape(pr.size(0), -1)          # [r, P*bs]
            nf, nm = st.node_flows[rows], st.node_mars[rows]         # [r, P*bs, B]
            lnf = torch.where(torch.isinf(nm) & (nm < 0), _neg_inf_like(nf), nf - nm)
            pad = (pr == 0)[:, :, None].expand(-1, -1, bs).reshape(pr.size(0), -1)
            lnf = torch.where(pad[:, :, None], _neg_inf_like(lnf), lnf)
            th = _gathered(cache, ("bk", bkey, cbs, r0, r1), lambda: params[
                pp[:, :, None, None] + c[None, None, :, None] * bs + n[None, None, None, :]]     # [r, P, cbs, bs]
                .permute(0, 2, 1, 3).reshape(pr.size(0), cbs, -1))                                # [r, cbs, P*bs]
            mx = lnf.max(dim=1).values
            dead = torch.isinf(mx) & (mx < 0)
            mx0 = torch.where(dead, torch.zeros_like(mx), mx)
            acc = torch.bmm(th, (lnf - mx0[:, None, :]).exp())       # [r, cbs, B]
            tgt = (chids[r0:r1, None] + c[None, :]).reshape(-1)
            em = st.element_mars[tgt].reshape(pr.size(0), cbs, B)
            out = acc.log() + mx0[:, None, :] + em
            kill = dead[:, None, :] | (torch.isinf(em) & (em < 0)) | (acc <= 0)
            st.element_flows[tgt] = torch.where(kill, _neg_inf_like(out), out).reshape(-1, B)
    if not compute_param_flows:
        return
    # parameter flows
    for nids, cids, pids, pfids in zip(layer["nids"], layer["cids"], layer["pids"], layer["pfids"]):
        K = cids.size(1)
        fkey = _table_key(pids, pfids) if pending is not None else None
        for r0, r1 in _row_chunks(nids.numel(), (K + 2 * bs) * B + 2 * K * bs):
            rows = (nids[r0:r1, None] + n[None, :])                  # [r, bs]
            nf, nm = st.node_flows[rows], st.node_mars[rows]         # [r, bs, B]
            lnf = torch.where(torch.isinf(nm) & (nm < 0), _neg_inf_like(nf), nf - nm)
            em = st.element_mars[cids[r0:r1]]                        # [r, K, B]  (padding -> row 0 = -inf)
            shift = lnf.max(dim=1).values
            shift = torch.where(torch.isinf(shift), torch.zeros_like(shift), shift)
            acc = torch.bmm((lnf - shift[:, None, :]).exp(), (em + shift[:, None, :]).exp().transpose(1, 2))   # [r, bs, K]
            if pending is not None:
                # layers with the same parameter and flow tables (tied): sum their contractions, scatter once at the end
                slot = pending.setdefault((fkey, r0, r1), dict(pids=pids[r0:r1], pfids=pfids[r0:r1], bs=bs, acc=None))
                slot["acc"] = acc if slot["acc"] is None else slot["acc"] + acc
                continue
            th = params[pids[r0:r1, None, :] + n[None, :, None]]     # [r, bs, K]
            idx = (pfids[r0:r1, None, :] + n[None, :, None]).reshape(-1)
            st.param_flows.index_add_(0, idx, (th * acc).reshape(-1))


ALG_IDS = {"LL": 0, "MPE": 1, "GeneralLL": 2}


def _sum_forward_alg(layer, node_mars, element_mars, params, alg, alpha):
    """The reference's other propagation rules (layer/sum_layer.py:1079-1090): "MPE": max_k (log theta + child),
    "GeneralLL": (1 / alpha) log sum_k (theta exp(child))^alpha."""
    m = torch.arange(layer["bs"])
    B = node_mars.size(1)
    for nids, cids, pids in zip(layer["nids"], layer["cids"], layer["pids"]):
        K = cids.size(1)
        for r0, r1 in _row_chunks(nids.numel(), K * layer["bs"] * B):
            em = element_mars[cids[r0:r1]]                           # [n, K, B]
            lth = params[pids[r0:r1, :, None] + m[None, None, :]].log()                 # [n, K, bs]
            lth = torch.where((cids[r0:r1] == 0)[:, :, None], _neg_inf_like(lth), lth)
            val = lth.permute(0, 2, 1)[:, :, :, None] + em[:, None, :, :]               # [n, bs, K, B]
            out = val.max(dim=2).values if alg == 1 else _lse(alpha * val, 2) / alpha
            node_mars[(nids[r0:r1, None] + m[None, :]).reshape(-1)] = out.reshape(-1, B)


def _sum_backward_alg(layer, st, params, compute_param_flows, alg, alpha):
    """Flows under "MPE" (a parent's flow goes to the children and parameters that attain its maximum, within 1e-6:
    layer/kernels/sum_backward_element_block_sparse.py:89-94, sum_backward_param_block_sparse.py:69-77) and
    "GeneralLL" (element flows weighted by theta^alpha exp(alpha (child - value)), parameter flows by the ordinary
    theta exp(child - value): sum_backward_element_block_sparse.py:113-139, sum_backward_param_block_sparse.py:79-134
    and tests/layer/propagation_algs_test.py:198-236)."""
    bs = layer["bs"]
    n = torch.arange(bs)
    B = st.node_mars.size(1)

    def weight(lth, em, nm, a):                     # log weight of (parent, element): shapes broadcast
        lw = lth + em - nm
        lw = torch.where(torch.isnan(lw), _neg_inf_like(lw), lw)
        if alg == 1:
            return torch.where(lw.abs() < 1e-6, torch.zeros_like(lw), _neg_inf_like(lw))
        return a * lw

    for chids, parids, parpids, cbs in zip(layer["chids"], layer["parids"], layer["parpids"], layer["cs_block_sizes"]):
        c = torch.arange(cbs)
        P = parids.size(1)
        for r0, r1 in _row_chunks(chids.numel(), P * bs * cbs * B):
            pr, pp = parids[r0:r1], parpids[r0:r1]
            rows = (pr[:, :, None] + n[None, None, :]).reshape(pr.size(0), -1)          # [r, P*bs]
            nf, nm = st.node_flows[rows], st.node_mars[rows]                            # [r, P*bs, B]
            pad = (pr == 0)[:, :, None].expand(-1, -1, bs).reshape(pr.size(0), -1)
            nf = torch.where(pad[:, :, None], _neg_inf_like(nf), nf)
            lth = params[pp[:, :, None, None] + c[None, None, :, None] * bs + n[None, None, None, :]] \
                .permute(0, 2, 1, 3).reshape(pr.size(0), cbs, -1).log()                 # [r, cbs, P*bs]
            tgt = (chids[r0:r1, None] + c[None, :]).reshape(-1)
            em = st.element_mars[tgt].reshape(pr.size(0), cbs, B)
            lw = weight(lth[:, :, :, None], em[:, :, None, :], nm[:, None, :, :], alpha)           # [r, cbs, P*bs, B]
            tot = nf[:, None, :, :] + lw
            tot = torch.where(torch.isnan(tot), _neg_inf_like(tot), tot)
            st.element_flows[tgt] = _lse(tot, 2).reshape(-1, B)
    if not compute_param_flows:
        return
    for nids, cids, pids, pfids in zip(layer["nids"], layer["cids"], layer["pids"], layer["pfids"]):
        K = cids.size(1)
        for r0, r1 in _row_chunks(nids.numel(), K * bs * B):
            rows = (nids[r0:r1, None] + n[None, :])
            nf, nm = st.node_flows[rows], st.node_mars[rows]                            # [r, bs, B]
            em = st.element_mars[cids[r0:r1]]                                           # [r, K, B]
            lth = params[pids[r0:r1, None, :] + n[None, :, None]].log()                 # [r, bs, K]
            lth = torch.where((cids[r0:r1] == 0)[:, None, :], _neg_inf_like(lth), lth)
            lw = weight(lth[:, :, :, None], em[:, None, :, :], nm[:, :, None, :], 1.0)  # [r, bs, K, B]
            tot = nf[:, :, None, :] + lw
            tot = torch.where(torch.isnan(tot), _neg_inf_like(tot), tot)
            idx = (pfids[r0:r1, None, :] + n[None, :, None]).reshape(-1)
            st.param_flows.index_add_(0, idx, tot.exp().sum(dim=3).reshape(-1))


def _flush_pending_param_flows(pending, st, params):
    for slot in pending.values():
        n = torch.arange(slot["bs"])
        th = params[slot["pids"][:, None, :] + n[None, :, None]]
        idx = (slot["pfids"][:, None, :] + n[None, :, None]).reshape(-1)
        st.param_flows.index_add_(0, idx, (th * slot["acc"]).reshape(-1))


def _prod_backward(layer, st):
    j = torch.arange(layer["bs"])
    for u_cids, parids in zip(layer["u_cids"], layer["parids"]):
        rows = (parids[:, :, None] + j[None, None, :])               # [n, P, bs]
        ef = st.element_flows[rows]                                  # [n, P, bs, B]
        ef = torch.where((parids == 0)[:, :, None, None], torch.full_like(ef, NEG_INF), ef)
        inc = _lse(ef, dim=1)                                        # [n, bs, B]
        tgt = (u_cids[:, None] + j[None, :]).reshape(-1)
        st.node_flows[tgt] = torch.logaddexp(st.node_flows[tgt], inc.reshape(tgt.numel(), -1))


def forward(pc, x: torch.Tensor, params: torch.Tensor, input_params, dtype=torch.float64, tables=None,
            state: Optional[OracleState] = None, propagation_alg: str = "LL", alpha: float = 0.0):
    """Per-sample log-likelihoods ``[B, num_roots]``; fills ``state.node_mars / element_mars``.

    ``x`` is ``[B, V]`` integer, ``params`` the flat sum-parameter vector, ``input_params`` one flat
    vector per input layer."""
    t = tables or _tables(pc)
    st = state or OracleState()
    B = x.size(0)
    xt = x.t().long().cpu()
    st.node_mars = torch.zeros(t["num_nodes"], B, dtype=dtype)
    st.element_mars = torch.full((t["num_elements"], B), NEG_INF, dtype=dtype)
    params = params.detach().cpu().to(dtype)
    for lt, ip in zip(t["inputs"], input_params):
        ip = ip.detach().cpu().to(dtype)
        vals = xt[lt["vids"][:, 0]]                                  # [N, B]
        st.node_mars[lt["rng"][0]:lt["rng"][1]] = ip[lt["s_pids"][:, None] + vals].log()
    for kind, layers in t["inner"]:
        for layer in layers:
            if kind == "prod":
                _prod_forward(layer, st.node_mars, st.element_mars)
            elif ALG_IDS[propagation_alg] != 0:
                _sum_forward_alg(layer, st.node_mars, st.element_mars, params, ALG_IDS[propagation_alg], alpha)
            else:
                _sum_forward(layer, st.node_mars, st.element_mars, params, cache=st.cache)
    st.tables = t
    return st.node_mars[t["root"][0]:t["root"][1]].t().clone(), st


def backward(pc, x: torch.Tensor, params: torch.Tensor, input_params, st: OracleState,
             ll_weights: Optional[torch.Tensor] = None, compute_param_flows: bool = True,
             param_flows: Optional[torch.Tensor] = None, input_param_flows=None, reference_compat: bool = False,
             propagation_alg: str = "LL", alpha: float = 0.0):
    """Log-space node/element flows and (accumulated) parameter flows.  ``st`` comes from
    :func:`forward` on the same inputs.  Existing ``param_flows`` are added to, as the reference does.

    ``reference_compat`` reproduces the reference's handling of product nodes without a sum parent (see the
    comment in the loop below) instead of giving them zero flow."""
    t = st.tables
    dtype = st.node_mars.dtype
    B = x.size(0)
    xt = x.t().long().cpu()
    params = params.detach().cpu().to(dtype)
    st.node_flows = torch.full((t["num_nodes"], B), NEG_INF, dtype=dtype)
    st.element_flows = torch.full((t["num_elements"], B), NEG_INF, dtype=dtype)
    r0, r1 = t["root"]
    st.node_flows[r0:r1] = 0.0 if ll_weights is None else ll_weights.to(dtype).reshape(-1, B).log()
    st.param_flows = torch.zeros(t["num_param_flows"], dtype=dtype) if param_flows is None else param_flows.detach().cpu().to(dtype).clone()
    inner = t["inner"]
    pending = {}
    for gi in range(len(inner) - 1, -1, -1):
        kind, layers = inner[gi]
        if kind == "prod":
            for layer in layers:
                _prod_backward(layer, st)
        else:
            for layer in inner[gi - 1][1]:                           # recompute the product layer below
                _prod_forward(layer, st.node_mars, st.element_mars)
            # A product node without a sum parent at this depth has flow zero.  Its row of the shared buffer is not
            # written below, so clear the buffer per depth (the reference clears it once per pass only,
            # model/tensorcircuit.py:526-528, and lets such a row keep another depth's flow; that defect is
            # deliberately not reproduced: the flows here are the true gradients, see tests/test_oracle_pins.py).
            if not reference_compat:
                st.element_flows.fill_(NEG_INF)
            for layer in layers:
                if ALG_IDS[propagation_alg] != 0:
                    _sum_backward_alg(layer, st, params, compute_param_flows, ALG_IDS[propagation_alg], alpha)
                else:
                    _sum_backward(layer, st, params, compute_param_flows, cache=st.cache, pending=pending)
    _flush_pending_param_flows(pending, st, params)
    st.input_param_flows = []
    for li, lt in enumerate(t["inputs"]):
        pf = torch.zeros(lt["num_param_flows"], dtype=dtype)
        if input_param_flows is not None and input_param_flows[li] is not None:
            pf = input_param_flows[li].detach().cpu().to(dtype).clone()
        if compute_param_flows:
            vals = xt[lt["vids"][:, 0]]
            idx = (lt["s_pfids"][:, None] + vals).reshape(-1)
            pf.index_add_(0, idx, st.node_flows[lt["rng"][0]:lt["rng"][1]].exp().reshape(-1))
        st.input_param_flows.append(pf)
    return st


def top_down(pc, params: torch.Tensor, input_params, scale: float = 1.0, tables=None, dtype=torch.float64):
    """Top-down probabilities of a normalised circuit and the parameter flows they induce
    (model/backend/top_down_prob.py:15-402, layer/input_layer.py:894-968): td(root) = scale; an element receives
    sum_n td(n) theta(n, e); a node the sum of its parent elements; parameter flow theta(n, e) td(n); a leaf's td,
    plus that of the leaves tied to it, spreads over its categories in proportion to its parameters.
    Returns (td [num_nodes], sum parameter flows, [input parameter flows])."""
    t = tables or _tables(pc)
    params = params.detach().cpu().to(dtype)
    nn_, ne_ = t["num_nodes"], t["num_elements"]
    td = torch.zeros(nn_, dtype=dtype)
    td[t["root"][0]:t["root"][1]] = scale
    pf = torch.zeros(t["num_param_flows"], dtype=dtype)
    inner = t["inner"]
    for gi in range(len(inner) - 1, -1, -1):
        kind, layers = inner[gi]
        if kind == "prod":
            for layer in layers:
                j = torch.arange(layer["bs"])
                for u_cids, parids in zip(layer["u_cids"], layer["parids"]):
                    rows = parids[:, :, None] + j[None, None, :]
                    inc = torch.where((parids == 0)[:, :, None], torch.zeros((), dtype=dtype), etd[rows]).sum(dim=1)
                    tgt = (u_cids[:, None] + j[None, :]).reshape(-1)
                    td[tgt] += inc.reshape(-1)
        else:
            etd = torch.zeros(ne_, dtype=dtype)
            for layer in layers:
                m = torch.arange(layer["bs"])
                for nids, cids, pids, pfids in zip(layer["nids"], layer["cids"], layer["pids"], layer["pfids"]):
                    th = params[pids[:, :, None] + m[None, None, :]]                    # [n, K, bs]
                    flow = th * td[nids[:, None] + m[None, :]][:, None, :]               # theta(n, e) td(n)
                    flow = torch.where((cids == 0)[:, :, None], torch.zeros((), dtype=dtype), flow)
                    etd.index_add_(0, cids.reshape(-1), flow.sum(dim=2).reshape(-1))
                    pf.index_add_(0, (pfids[:, :, None] + m[None, None, :]).reshape(-1), flow.reshape(-1))
            etd[0] = 0.0
    ipfs = []
    for lt, ip in zip(t["inputs"], input_params):
        ip = ip.detach().cpu().to(dtype)
        out = torch.zeros(lt["num_param_flows"], dtype=dtype)
        r0, r1 = lt["rng"]
        flow = td[r0:r1].clone()
        n2s = pc.input_layer_group[len(ipfs)].node_id2source_id.cpu()
        tied = n2s >= 0
        flow.index_add_(0, n2s[tied], td[r0:r1][tied])
        for n in lt["source_nids"].tolist():
            C = int(lt["metadata"][lt["s_mids"][n]])
            a, b = int(lt["s_pids"][n]), int(lt["s_pfids"][n])
            out[b:b + C] += flow[n] * ip[a:a + C]
        ipfs.append(out)
    return td, pf, ipfs


def em_update_rescaled(pc, params, input_params, st: OracleState, step_size: float, pseudocount: float, cum_flow: float):
    """The rescaled mini-batch EM update (model/tensorcircuit.py:1363-1387): flows * step_size / cum_flow, plus the
    top-down flows of the current parameters at (1 - step_size), then the update with step size one."""
    _, pf, ipfs = top_down(pc, params, input_params, scale=1.0 - step_size, tables=st.tables, dtype=st.param_flows.dtype)
    st2 = OracleState()
    st2.tables = st.tables
    st2.param_flows = st.param_flows * (step_size / cum_flow) + pf
    st2.input_param_flows = [a * (step_size / cum_flow) + b for a, b in zip(st.input_param_flows, ipfs)]
    return em_update(pc, params, input_params, st2, 1.0, pseudocount)


def em_update(pc, params: torch.Tensor, input_params, st: OracleState, step_size: float, pseudocount: float = 0.0,
              reference_compat: bool = False):
    """Returns ``(new_params, [new_input_params])``; flows are taken from ``st``.

    ``reference_compat`` reproduces the reference's tied-flow fusing kernel on padding slots (see below)."""
    dtype = st.param_flows.dtype
    new_inputs = []
    for lt, ip, pf in zip(st.tables["inputs"], input_params, st.input_param_flows):
        ip = ip.detach().cpu().to(dtype).clone()
        pf = pf.clone()
        for start, n, ch in lt["tied"]:
            pf[start:start + n] = sum(pf[int(c):int(c) + n] for c in ch)
        src = lt["source_nids"]
        cats = lt["metadata"][lt["s_mids"][src]].long()
        for C in torch.unique(cats).tolist():                        # all nodes with C categories at once
            sel = src[cats == C]
            c = torch.arange(C)
            pidx = lt["s_pids"][sel][:, None] + c[None, :]
            flow = pf[lt["s_pfids"][sel][:, None] + c[None, :]]
            ip[pidx] = (1.0 - step_size) * ip[pidx] + step_size * (flow + pseudocount / C) / (flow.sum(dim=1, keepdim=True) + pseudocount)
        new_inputs.append(ip)

    params = params.detach().cpu().to(dtype).clone()
    pf = st.param_flows.clone()
    head = pf.clone()          # what the reference's kernel reads through a padding slot: param_flows[0 : n]
    for tgt, sizes, chs, G, M in pc.parflow_fusing_kwargs:
        for i in range(tgt.numel()):
            n = int(sizes[i])
            # Slots after the first that hold 0 are padding up to the power-of-two group width.  (The
            # reference kernel's mask `offs >= 0`, parflow_fusing.py:86-87, lets such padding slots add
            # param_flows[0:n] as well; that is a defect for non-power-of-two accumulator counts and is
            # deliberately not reproduced.)
            real = [int(c) for k, c in enumerate(chs[i].tolist()) if k == 0 or c != 0]
            total = sum(pf[c:c + n] for c in real)
            if reference_compat:
                total = total + (chs[i].numel() - len(real)) * head[:n]
            pf[int(tgt[i]):int(tgt[i]) + n] = total
    par_start, pflow_start, blk_sizes, blk_int, gnids, nchs = [a.cpu() for a in pc.par_update_kwargs[:6]]
    tot = int(gnids.max().item()) + 1
    j = torch.arange(int(blk_sizes.max().item()))
    mask = j[None, :] < blk_sizes[:, None]
    fidx = pflow_start[:, None] + j[None, :] * blk_int[:, None]
    pidx = par_start[:, None] + j[None, :] * blk_int[:, None]
    flows = torch.where(mask, pf[torch.where(mask, fidx, torch.zeros_like(fidx))], torch.zeros((), dtype=dtype))
    node_tot = torch.zeros(tot, dtype=dtype).index_add_(0, gnids, flows.sum(dim=1))
    new = (flows + pseudocount / nchs[:, None].to(dtype)) / (node_tot[gnids][:, None] + pseudocount)
    old = params[torch.where(mask, pidx, torch.zeros_like(pidx))]
    upd = (1.0 - step_size) * old + step_size * new
    params[pidx[mask]] = upd[mask]
    return params, new_inputs
