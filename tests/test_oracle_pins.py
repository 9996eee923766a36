"""Pins the CPU oracle (oracle/pc_oracle.py) to what the reference's own tests assert.

The reference cannot run this path without a GPU, so its tests' closed-form dense restatements are the
golden statements available: tests/model/simple_model_test.py:191-528 (forward, flows, parameter flows, EM)
is transcribed below on the same circuit, and a homogeneous HMM is checked against the textbook
forward-backward recursions (what tests/structures/hmm_correctness_test.py and
tests/model/homogeneous_hmm_test.py:98-212 verify).  The tables driving the oracle are the ones checked
bit-for-bit against the reference compiler in test_tables_golden.py.
"""
import numpy as np
import pytest
import torch

import pyjuice_b200 as pj
from cases import OursApi, simple_model
from oracle import pc_oracle as orc


def _run_oracle(pc, x, step=None, pseudo=0.0):
    iparams = [l.params.data for l in pc.input_layer_group]
    lls, st = orc.forward(pc, x, pc.params.data, iparams)
    orc.backward(pc, x, pc.params.data, iparams, st)
    new = orc.em_update(pc, pc.params.data, iparams, st, step, pseudo) if step is not None else None
    return lls, st, new


def test_simple_model_dense_restatement():
    torch.manual_seed(82392)
    api = OursApi()
    ns, kw = simple_model(api, block_size=16)
    ns.init_parameters()
    pc = api.compile(ns, **kw)
    B = 64
    data = torch.randint(0, 4, [B, 4])
    lls, st, (new_params, _) = _run_oracle(pc, data, step=0.25, pseudo=0.01)
    nm, nf, pf = st.node_mars, st.node_flows.exp(), st.param_flows

    np4, np5, np6 = ns.chs
    ns0, ni2, ni3 = np4.chs
    ns1, ni0, ni1 = np5.chs
    ns2 = np6.chs[0]
    rng = lambda n: slice(*n._output_ind_range)
    d = torch.float64

    # leaves (simple_model_test.py:203-217)
    leaf = {}
    for ni, v, c in ((ni0, 0, 4), (ni1, 1, 4), (ni2, 2, 6), (ni3, 3, 6)):
        leaf[v] = ni._params.reshape(-1, c)[:, data[:, v]].log().to(d)
        assert torch.allclose(nm[rng(ni)], leaf[v], atol=1e-6)
    np0_l = np3_l = leaf[0] + leaf[1]
    np1_l, np2_l = leaf[2] + leaf[3], leaf[1] + leaf[2]

    # first sum layer (:238-256); node-level parameter matrices as the test builds them
    e0 = ns0._params.reshape(2, 4, 16, 16).permute(0, 2, 1, 3).reshape(32, 64).to(d)
    e1 = ns1._params.reshape(2, 2, 16, 16).permute(0, 2, 1, 3).reshape(32, 32).to(d)
    e2 = ns2._params.reshape(2, 2, 16, 16).permute(0, 2, 1, 3).reshape(32, 32).to(d)
    ch0 = torch.cat((np0_l, np3_l), dim=0)
    ns0_l = (e0 @ ch0.exp()).log()
    ns1_l = (e1 @ np1_l.exp()).log()
    ns2_l = (e2 @ np2_l.exp()).log()
    assert torch.allclose(nm[rng(ns0)], ns0_l, atol=1e-5)
    assert torch.allclose(nm[rng(ns1)], ns1_l, atol=1e-5)
    assert torch.allclose(nm[rng(ns2)], ns2_l, atol=1e-5)

    # root (:258-277)
    np4_l, np5_l, np6_l = ns0_l + leaf[2] + leaf[3], ns1_l + leaf[0] + leaf[1], ns2_l + leaf[0] + leaf[3]
    chr_ = torch.cat((np4_l, np5_l, np6_l), dim=0)
    er = ns._params.reshape(1, 6, 1, 16).permute(0, 2, 1, 3).reshape(1, 96).to(d)
    ns_l = (er @ chr_.exp()).log()
    assert torch.allclose(nm[rng(ns)], ns_l, atol=1e-5)
    assert torch.allclose(lls[:, 0], ns_l[0], atol=1e-5)

    # backward (:279-424): root flow 1, element flows of the root, then the three lower sums
    assert torch.allclose(nf[rng(ns)], torch.ones(1, B, dtype=d))
    eflows = er.reshape(96, 1) * (chr_ - ns_l).exp()
    np4_f, np5_f, np6_f = eflows[0:32], eflows[32:64], eflows[64:96]
    assert torch.allclose(nf[rng(ns0)], np4_f, atol=1e-7)
    assert torch.allclose(nf[rng(ns1)], np5_f, atol=1e-7)
    assert torch.allclose(nf[rng(ns2)], np6_f, atol=1e-7)
    ps, pe = ns._param_flow_range
    assert torch.allclose(pf[ps:pe], eflows.sum(dim=1), atol=1e-6 * B)

    def lower(e, ch_l, n_l, n_f):
        ratio = n_f / n_l.exp()
        return ch_l.exp() * (e.t() @ ratio), e * (ratio @ ch_l.exp().t())

    f0, p0 = lower(e0, ch0, ns0_l, np4_f)
    f1, p1 = lower(e1, np1_l, ns1_l, np5_f)
    f2, p2 = lower(e2, np2_l, ns2_l, np6_f)
    np0_f, np3_f = f0[0:32], f0[32:64]
    for nsx, pref, cols in ((ns0, p0, 64), (ns1, p1, 32), (ns2, p2, 32)):
        a, b = nsx._param_flow_range
        got = pf[a:b].reshape(2, cols, 16).permute(0, 2, 1).reshape(32, cols)
        assert torch.allclose(got, pref, atol=1e-6 * B)

    # leaf flows (:376-390) and their histograms (:392-424)
    exp_leaf = {0: np0_f + np3_f + np5_f + np6_f, 1: np0_f + f2 + np3_f + np5_f, 2: f1 + f2 + np4_f, 3: f1 + np4_f + np6_f}
    ipf = st.input_param_flows[0]
    for ni, v, c in ((ni0, 0, 4), (ni1, 1, 4), (ni2, 2, 6), (ni3, 3, 6)):
        assert torch.allclose(nf[rng(ni)], exp_leaf[v], atol=1e-6)
        ref = torch.zeros(32, c, dtype=d)
        for b in range(B):
            ref[:, data[b, v]] += exp_leaf[v][:, b]
        a, e = ni._param_flow_range
        assert torch.allclose(ipf[a:e].reshape(32, c), ref, atol=1e-6)

    # EM (:426-528)
    step, pseudo = 0.25, 0.01
    for nsx, e_old, pflow, cols in ((ns0, e0, p0, 64), (ns1, e1, p1, 32), (ns2, e2, p2, 32)):
        target = (1 - step) * e_old + step * (pflow + pseudo / cols) / (pflow.sum(dim=1, keepdim=True) + pseudo)
        a, b = nsx._param_range
        got = new_params[a:b].reshape(2, cols, 16).permute(0, 2, 1).reshape(32, cols)
        assert torch.allclose(got, target, atol=1e-7)
    rp = eflows.sum(dim=1)
    target = (1 - step) * er.reshape(96) + step * (rp + pseudo / 96) / (rp.sum() + pseudo)
    a, b = ns._param_range
    assert torch.allclose(new_params[a:b], target, atol=1e-7)


def test_hmm_matches_forward_backward_recursions():
    torch.manual_seed(7)
    L, V, T, B = 8, 11, 6, 32
    alpha = torch.rand(L, L).double() + 0.05
    alpha /= alpha.sum(dim=1, keepdim=True)                  # alpha[z_t, z_{t+1}]
    beta = torch.rand(L, V).double() + 0.05
    beta /= beta.sum(dim=1, keepdim=True)
    gamma = torch.rand(L).double() + 0.05
    gamma /= gamma.sum()
    ns = pj.structures.HMM(seq_length=T, num_latents=L, num_emits=V, homogeneous=True, block_size=4,
                           alpha=alpha.float(), beta=beta.float(), gamma=gamma.float())
    pc = pj.compile(ns)
    x = torch.randint(0, V, (B, T))
    lls, st, _ = _run_oracle(pc, x)
    a, bmat, g = alpha.float().double(), beta.float().double(), gamma.float().double()
    a, bmat, g = a / a.sum(1, keepdim=True), bmat / bmat.sum(1, keepdim=True), g / g.sum()

    # backward messages m_t[z] = p(x_t.. | z_t = z); the circuit's sum vector at position t holds
    # sum_{z'} alpha[z, z'] m_{t+1}[z']
    m = bmat[:, x[:, T - 1]]                                  # [L, B]
    msgs = {T - 1: m}
    for t in range(T - 2, -1, -1):
        m = bmat[:, x[:, t]] * (a @ m)
        msgs[t] = m
    ll = (g[:, None] * msgs[0]).sum(dim=0).log()
    assert torch.allclose(lls[:, 0], ll, atol=1e-6)

    # expected transition counts = tied transition parameter flows; expected emission counts = tied leaf flows
    fwd = g[:, None].expand(L, B).clone()                     # p(x_<t, z_t)
    xi = torch.zeros(L, L, dtype=torch.float64)
    em = torch.zeros(L, V, dtype=torch.float64)
    px = ll.exp()
    for t in range(T):
        post = fwd * msgs[t] / px                             # p(z_t | x)
        for b in range(B):
            em[:, x[b, t]] += post[:, b]
        if t < T - 1:
            joint = fwd * bmat[:, x[:, t]]                    # p(x_<=t, z_t)
            xi += torch.einsum("ib,ij,jb->ij", joint / px, a, msgs[t + 1])
            fwd = a.t() @ joint
    trans_ns = [n for n in ns if n.is_sum() and not n.is_tied() and n.block_size == 4][0]
    s, e = trans_ns._param_flow_range
    got = st.param_flows[s:e]
    local = (trans_ns._param_flow_ids - s) // 16
    got = got.reshape(local.numel(), 4, 4)[local].permute(0, 2, 1)                  # [E, bs, ch_bs]
    dense = torch.zeros(L, L, dtype=torch.float64)
    for k in range(trans_ns.edge_ids.size(1)):
        i, j = trans_ns.edge_ids[:, k].tolist()
        dense[i * 4:(i + 1) * 4, j * 4:(j + 1) * 4] = got[k]
    assert torch.allclose(dense, xi, atol=1e-6)

    layer = pc.input_layer_group[0]
    ipf = st.input_param_flows[0].clone()
    for start, n, ch in layer.tied2source_nids:
        ipf[start:start + n] = sum(ipf[int(c):int(c) + n] for c in ch)
    src = [n for n in ns if n.is_input() and not n.is_tied()][0]
    s, e = src._param_flow_range
    assert torch.allclose(ipf[s:e].reshape(L, V), em, atol=1e-6)


def test_flow_invariants_on_cfg0_shape():
    from cases import hclt_cfg0
    from pyjuice_b200.data import tree_bn_samples
    api = OursApi()
    torch.manual_seed(0)
    ns, kw = hclt_cfg0(api)
    ns.init_parameters()
    pc = api.compile(ns, **kw)
    x = torch.from_numpy(tree_bn_samples(4096, 32, 4, seed=0))[:64]
    lls, st, (new_params, new_inputs) = _run_oracle(pc, x, step=0.1, pseudo=0.1)
    assert torch.isfinite(lls).all()
    B = x.size(0)
    nfl = st.node_flows.exp()
    layer = pc.input_layer_group[0]
    # every variable's leaves carry unit flow per sample; every sum node's parameter flows add up to its node flow
    r0, r1 = layer._output_ind_range
    per_var = torch.zeros(32, B, dtype=torch.float64).index_add_(0, layer.vids[:, 0], nfl[r0:r1])
    assert torch.allclose(per_var, torch.ones_like(per_var), atol=1e-9)
    s, e = pc.root_ns._param_flow_range
    assert abs(st.param_flows[s:e].sum().item() - B) < 1e-8
    for nsx in pc.root_ns:
        if nsx.is_sum() and not nsx.is_tied():
            a, b = nsx._param_range
            fan = nsx.edge_ids.size(1) // nsx.num_node_blocks * nsx.ch_block_size
            sums = new_params[a:b].reshape(nsx.num_node_blocks, fan, nsx.block_size).sum(dim=1)
            assert torch.allclose(sums, torch.ones_like(sums), atol=1e-6)
    ip = new_inputs[0].reshape(-1, 4).sum(dim=1)
    assert torch.allclose(ip, torch.ones_like(ip), atol=1e-6)


@pytest.mark.parametrize("case", ["pd_parentless", "hclt", "hmm", "rat"])
def test_oracle_flows_are_the_gradients_of_the_log_likelihood(case):
    """Pin the oracle's backward pass against a second evaluator that shares no code with it: a recursive walk of
    the node DAG with torch autograd (tests/dag_autograd.py).  Flow of a node = d log p(x) / d log value(node).

    ``pd_parentless`` is a Poon-Domingos circuit in which block-sparse sum vectors leave some product blocks
    without a parent.  The reference hands the stale content of their rows of the shared element-flow buffer down
    to the children (it clears the buffer once per backward pass, model/tensorcircuit.py:526-528, while its
    backward tables skip child blocks without parents, layer/sum_layer.py:273-275); the oracle and the CUDA path
    deliberately do not: such a product has flow zero.  Also checked: the leaves of every variable receive a total
    flow of exactly one per sample."""
    import random
    from dag_autograd import true_flows
    torch.manual_seed(0)
    random.seed(0)
    if case == "pd_parentless":
        ns = pj.structures.PD((8, 8), num_latents=2, split_points=[[2, 4, 6], [2, 4, 6]], num_cats=4)
    elif case == "hclt":
        x0 = torch.randint(0, 4, (200, 10))
        ns = pj.structures.HCLT(x0.float(), num_latents=4, num_cats=4)
    elif case == "hmm":
        ns = pj.structures.HMM(seq_length=6, num_latents=8, num_emits=5, homogeneous=True)
    else:
        ns = pj.structures.RAT_SPN(num_vars=12, num_latents=4, depth=2, num_repetitions=3, num_cats=4)
    ns.init_parameters()
    pc = pj.compile(ns)
    layer = pc.input_layer_group[0]
    cats = int(layer.node_cats.min())
    x = torch.randint(0, cats, (3, pc.num_vars))
    params = pc.params.data.double()
    iparams = [l.params.data.double() for l in pc.input_layer_group]
    lls, st = orc.forward(pc, x, params, iparams)
    orc.backward(pc, x, params, iparams, st)

    ref_lls, flows, order = true_flows(pc, ns, st.node_mars)
    assert torch.allclose(ref_lls.reshape(-1), lls.reshape(-1).double(), atol=1e-9)
    if case == "pd_parentless":
        assert len(pc._parentless) > 0, "the case is meant to contain product blocks without a parent"
    for n in order:
        if id(n) in flows:
            s, e = n._output_ind_range
            assert torch.allclose(st.node_flows[s:e].exp().double(), flows[id(n)], atol=1e-9), (case, s, e)
    s, e = layer._output_ind_range
    per_var = torch.zeros(pc.num_vars, x.size(0), dtype=torch.float64)
    per_var.index_add_(0, layer.vids[:, 0], st.node_flows[s:e].exp().double())
    assert torch.allclose(per_var, torch.ones_like(per_var), atol=1e-9)
