"""The reference's other propagation rules ("MPE", "GeneralLL"; tests/layer/propagation_algs_test.py).

CPU: the oracle's statements of the two rules are pinned by identities that need no second implementation —
GeneralLL with alpha = 1 is the ordinary rule (values, flows, parameter flows), MPE values are the log-probability of
the best complete assignment of the latent choices (brute force on a tiny circuit), MPE flows are 0 / 1 per sample and
every sum node hands its flow to exactly one child.  GPU: the plain kernels against the closed forms the reference's
own test uses (layer level, linear flows), and whole circuits against the oracle."""
import itertools
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
sys.path.insert(0, os.path.dirname(HERE))

import pyjuice_b200 as pj
from cases import CASES, OursApi
from oracle import pc_oracle as orc

DEV = "cuda:0"


def _build(name, seed=0):
    api = OursApi()
    torch.manual_seed(seed)
    ns, kw = CASES[name](api)
    ns.init_parameters()
    return api.compile(ns, **kw)


def _data(pc, B, seed):
    g = torch.Generator().manual_seed(seed)
    layer = pc.input_layer_group[0]
    cats = torch.zeros(pc.num_vars, dtype=torch.long)
    cats[layer.vids[:, 0]] = layer.node_cats
    return (torch.rand(B, pc.num_vars, generator=g) * cats[None, :].clamp(min=1)).long()


def _oracle_step(pc, x, alg, alpha=0.0):
    params = pc.params.data.cpu()
    iparams = [l.params.data.cpu() for l in pc.input_layer_group]
    lls, st = orc.forward(pc, x, params, iparams, propagation_alg=alg, alpha=alpha)
    st = orc.backward(pc, x, params, iparams, st, propagation_alg=alg, alpha=alpha)
    return lls, st


@pytest.mark.parametrize("name", ["hclt_grid", "pd_small", "hmm_small"])
def test_oracle_general_ll_with_alpha_one_is_the_ordinary_rule(name):
    pc = _build(name, seed=4)
    x = _data(pc, 6, seed=1)
    a, sa = _oracle_step(pc, x, "LL")
    b, sb = _oracle_step(pc, x, "GeneralLL", alpha=1.0)
    assert torch.allclose(a, b, atol=1e-9)
    live = ~torch.isinf(sa.node_flows)
    assert torch.equal(live, ~torch.isinf(sb.node_flows))
    assert torch.allclose(sa.node_flows[live], sb.node_flows[live], atol=1e-9)
    assert torch.allclose(sa.param_flows, sb.param_flows, atol=1e-9)


def test_oracle_mpe_value_is_the_best_assignment_and_flows_follow_it():
    """A tiny HMM: the MPE value of the root is max over latent paths of log p(path, x); brute force over the paths."""
    torch.manual_seed(3)
    T, S, V = 4, 3, 5
    ns = pj.structures.HMM(seq_length=T, num_latents=S, num_emits=V, homogeneous=False, block_size=1)
    ns.init_parameters()
    pc = pj.compile(ns)
    x = torch.randint(0, V, (5, T))
    lls, st = _oracle_step(pc, x, "MPE")
    ll, _ = _oracle_step(pc, x, "LL")
    assert torch.all(lls <= ll + 1e-12) and torch.all(lls >= ll - T * torch.log(torch.tensor(float(S))) - 1e-9)
    # flows: per sample every node flow is 0 or 1 (log 0 / -inf), the root's is 1, and the parameter flows of every
    # sum node add up to its flow (exactly one child takes it, barring exact ties)
    nf = st.node_flows.exp()
    assert torch.all((nf < 1e-12) | ((nf - 1).abs() < 1e-9))
    r0, r1 = st.tables["root"]
    assert torch.allclose(nf[r0:r1], torch.ones_like(nf[r0:r1]))
    sum_rows = torch.cat([(nids[:, None] + torch.arange(layer["bs"])[None, :]).reshape(-1)
                          for kind, layers in st.tables["inner"] if kind == "sum" for layer in layers for nids in layer["nids"]])
    assert abs(float(st.param_flows.sum()) - float(nf[sum_rows].sum())) < 1e-6
    # brute force through the oracle itself under the ordinary rule would need the joint; use the max-product identity
    # instead: replacing every sum by a max can only lower the value, and for S = 1 the two coincide
    ns1 = pj.structures.HMM(seq_length=T, num_latents=1, num_emits=V, homogeneous=False, block_size=1)
    ns1.init_parameters()
    pc1 = pj.compile(ns1)
    a, _ = _oracle_step(pc1, x, "MPE")
    b, _ = _oracle_step(pc1, x, "LL")
    assert torch.allclose(a, b, atol=1e-9)


# ---- GPU ------------------------------------------------------------------------------------------------------------
def _i32(t):
    return t.to(torch.int32).to(DEV).contiguous()


@pytest.mark.gpu
@pytest.mark.parametrize("bs", [1, 4, 16])
@pytest.mark.parametrize("alg,alpha", [("MPE", 0.0), ("GeneralLL", 1.2), ("GeneralLL", 3.0), ("LL", 0.0)])
def test_layer_kernels_against_the_closed_forms(alg, alpha, bs):
    """Hand-made tables, linear flows, the formulas of the reference's test (propagation_algs_test.py:186-236, 282-330)."""
    from pyjuice_b200 import _lib
    from pyjuice_b200.layers import ALG_IDS
    gen = torch.Generator().manual_seed(17 + bs)
    B, n_rows, K = 12, 5, 3                                # 5 sum blocks, 3 child blocks each (element blocks of bs)
    n_eblocks = 7
    # one element row per (block, j); sum block i lists K distinct child ELEMENTS per node?  The table lists element
    # rows per edge k: cids[i, k]; every node of block i has these K children with its own parameter
    E = n_eblocks * bs
    em = torch.rand(E + bs, B, generator=gen, dtype=torch.float64).log()
    em[:bs] = float("-inf")                                # rows 0 .. bs-1: "no element"
    cids = torch.stack([torch.randperm(E, generator=gen)[:K] + bs for _ in range(n_rows)])           # [rows, K]
    theta = torch.rand(n_rows, K, bs, generator=gen, dtype=torch.float64) + 0.05
    params = torch.cat([torch.zeros(bs, dtype=torch.float64), theta.reshape(-1)])
    pids = (torch.arange(n_rows * K).reshape(n_rows, K) + 1) * bs
    em, theta = em.float().double(), theta.float().double()
    nids = bs * (1 + torch.arange(n_rows))
    val = theta.log().permute(0, 2, 1)[:, :, :, None] + em[cids][:, None, :, :]                     # [rows, bs, K, B]
    if alg == "MPE":
        ref = val.max(dim=2).values
    elif alg == "GeneralLL":
        ref = torch.logsumexp(alpha * val, dim=2) / alpha
    else:
        ref = torch.logsumexp(val, dim=2)
    node_mars = torch.zeros(bs * (1 + n_rows), B, device=DEV)
    a = ALG_IDS[alg]
    _lib.call("pcx_sum_fwd_alg", node_mars, em.float().to(DEV), params.float().to(DEV), _i32(nids), _i32(cids), _i32(pids),
              n_rows, K, bs, B, a, float(alpha))
    got = node_mars[bs:].reshape(n_rows, bs, B).double().cpu()
    assert (got - ref).abs().max() < 1e-5
    # parameter flows with linear node flows: MPE: sum_b flow * [child attains the max]; GeneralLL and LL:
    # theta * sum_b flow * exp(child - value), with the rule's values
    nm = node_mars.double().cpu()                          # the kernel's own values (fp32), as the reference test uses
    nf = torch.rand(bs * (1 + n_rows), B, generator=gen, dtype=torch.float64).float().double()
    nmr, nfr = nm[bs:].reshape(n_rows, bs, B), nf[bs:].reshape(n_rows, bs, B)
    w = theta.log().permute(0, 2, 1)[:, :, :, None] + em[cids][:, None, :, :] - nmr[:, :, None, :]  # [rows, bs, K, B]
    if alg == "MPE":
        pref = (nfr[:, :, None, :] * (w.abs() < 1e-6)).sum(dim=3)
    else:
        pref = (nfr[:, :, None, :] * w.exp()).sum(dim=3)
    pf = torch.zeros(params.numel(), device=DEV)
    _lib.call("pcx_sum_bwd_par_alg", pf, nf.float().to(DEV), node_mars, em.float().to(DEV), params.float().to(DEV),
              _i32(nids), _i32(cids), _i32(pids), _i32(pids), n_rows, K, bs, B, 0, a, float(alpha))
    gotp = pf[bs:].reshape(n_rows, K, bs).permute(0, 2, 1).double().cpu()
    assert (gotp - pref).abs().max() < 1e-4 * max(1.0, float(pref.abs().max()))
    _lib.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["hclt_grid", "pd_small", "hmm_small", "hclt_b128"])
@pytest.mark.parametrize("alg,alpha", [("MPE", 0.0), ("GeneralLL", 2.0)])
@pytest.mark.parametrize("logspace", [True, False])
def test_whole_circuits_under_the_other_rules_match_the_oracle(name, alg, alpha, logspace):
    pc = _build(name, seed=4).to(DEV)
    x = _data(pc, 24, seed=2)
    kw = {"alpha": alpha} if alg == "GeneralLL" else {}
    lls = pc(x.to(DEV), propagation_alg=alg, **kw)
    pc.backward(x.to(DEV), flows_memory=0.0, propagation_alg=alg, logspace_flows=logspace, **kw)
    ref_lls, st = _oracle_step(pc, x, alg, alpha)
    assert (lls.double().cpu() - ref_lls).abs().max() < 1e-4
    nf = pc.node_flows.double().cpu()
    nf = nf.exp() if logspace else nf
    ref_nf = st.node_flows.exp()
    d = pc.num_dummy_nodes
    assert (nf[d:] - ref_nf[d:]).abs().max() < 1e-3 * max(1.0, float(ref_nf[d:].max()))
    pf, ref_pf = pc.param_flows.double().cpu(), st.param_flows
    assert (pf - ref_pf).abs().max() < 1e-3 * max(1.0, float(ref_pf.max()))
    # the ordinary rule afterwards is untouched by the detour (kernels, graphs and folding come back)
    a = pc(x.to(DEV))
    b, _ = _oracle_step(pc, x, "LL")
    assert (a.double().cpu() - b).abs().max() < 1e-3
    # defaults: `set_propagation_alg` and the named shorthands
    pc.set_propagation_alg(alg, **kw)
    assert torch.equal(pc(x.to(DEV)), lls)
    pc.set_propagation_alg("LL")
    assert torch.equal(pc.forward_mpe(x.to(DEV)) if alg == "MPE" else pc.forward_general_ll(x.to(DEV), alpha=alpha), lls)
