"""Update schedules of the EM optimizers on the GPU against the CPU oracle carried through the same schedule:
`FullBatchEM` (flows accumulated over several batches, one exact M-step), `MiniBatchEM(niters_per_update=3)`,
and decaying flows (`flows_memory = 0.5`) on circuits with tied leaves and tied sums.

Reference behaviour followed: optim/full_batch_em.py:21-27, optim/mini_batch_em.py:44-56,
model/tensorcircuit.py:1394-1418 (flow decay).
"""
import pytest
import torch

import pyjuice_b200 as pj
from pyjuice_b200 import _lib
from cases import CASES, OursApi, data_for
from helpers import LL_ATOL, OracleTrainer

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _build(name, seed=0):
    api = OursApi()
    torch.manual_seed(seed)
    ns, kw = CASES[name](api)
    ns.init_parameters()
    return api.compile(ns, **kw)


@pytest.mark.parametrize("name", ["hclt_grid", "hmm_blocks"])
def test_full_batch_em_accumulates_then_makes_one_exact_m_step(name):
    pc = _build(name, seed=11).to(DEV)
    ref = OracleTrainer(pc)
    opt = pj.optim.FullBatchEM(pc, pseudocount=0.1)
    for epoch in range(2):
        for i in range(3):
            x = data_for(pc, 48, seed=100 * epoch + i)
            lls = pc(x.to(DEV))
            lls.mean().backward()
            ref_lls = ref.accumulate(x)
            assert (lls.detach().double().cpu() - ref_lls).abs().max().item() <= LL_ATOL
        opt.step()
        ref.update(1.0, 0.1)
        print(name, epoch, ref.check_params(pc))
    _lib.check_status(DEV)


@pytest.mark.parametrize("name", ["simple_model", "tied_sums"])
def test_mini_batch_em_updates_every_third_batch(name):
    pc = _build(name, seed=12).to(DEV)
    ref = OracleTrainer(pc)
    opt = pj.optim.MiniBatchEM(pc, step_size=0.2, niters_per_update=3, pseudocount=0.05)
    for i in range(7):
        x = data_for(pc, 40, seed=i)
        lls = pc(x.to(DEV))
        lls.mean().backward()
        before = pc.params.data.clone()
        opt.step()
        ref.accumulate(x)
        if (i + 1) % 3 == 0:
            ref.update(0.2, 0.05)
            assert not torch.equal(before, pc.params.data)
        else:
            assert torch.equal(before, pc.params.data), "parameters moved between updates"
        ref.check_params(pc)


@pytest.mark.parametrize("name", ["hmm_blocks", "tied_sums", "hclt_b128"])
def test_decaying_flows_over_several_steps(name):
    """`backward(flows_memory=0.5)` halves what the accumulators hold and adds the new flows; the update then uses the
    decayed sum.  hmm_blocks has tied leaves with several replica accumulators: their flows must reach the update on
    every step, not only on the first."""
    pc = _build(name, seed=13).to(DEV)
    ref = OracleTrainer(pc)
    pc.init_param_flows(flows_memory=0.0)
    for i in range(4):
        x = data_for(pc, 32, seed=50 + i)
        pc(x.to(DEV))
        pc.backward(x.to(DEV), flows_memory=0.5)
        pc.mini_batch_em(step_size=0.3, pseudocount=0.1)
        ref.accumulate(x, flows_memory=0.5)
        ref.update(0.3, 0.1, zero_flows=False)
        print(name, i, ref.check_params(pc))
    assert abs(pc._cum_flow - 32 * (1 + 0.5 + 0.25 + 0.125)) < 1e-3


@pytest.mark.parametrize("name", ["simple_model", "hmm_blocks", "tied_sums", "hclt_b128", "pd_small", "hmm_b128"])
def test_top_down_probabilities_and_rescaled_update(name):
    """`eval_top_down_probs` against the oracle's recursion, and `mini_batch_em(step_size_rescaling=True)`
    (flows * step / total flow + (1 - step) * top-down flows, then an update with step one) against the same
    schedule on the CPU.  Reference: model/backend/top_down_prob.py:290-402, model/tensorcircuit.py:1363-1387."""
    from oracle import pc_oracle as orc
    from helpers import oracle_step, rel_close
    pc = _build(name, seed=14).to(DEV)
    p0 = pc.params.data.double().cpu()
    ip0 = [l.params.data.double().cpu() for l in pc.input_layer_group]
    td_ref, _, _ = orc.top_down(pc, p0, ip0, 1.0)
    td = pc.eval_top_down_probs(update_pflow=False, scale=1.0)
    ok, err = rel_close(td[pc.num_dummy_nodes:], td_ref[pc.num_dummy_nodes:])
    assert ok, f"top-down probabilities rel err {err}"

    x = data_for(pc, 40, seed=3)
    for rep in range(2):                                     # second round: captured / replayed launches
        p0 = pc.params.data.double().cpu()
        ip0 = [l.params.data.double().cpu() for l in pc.input_layer_group]
        _, st, _ = oracle_step(pc, x, None, params=p0, input_params=ip0)
        ref_p, ref_ip = orc.em_update_rescaled(pc, p0, ip0, st, 0.25, 0.1, cum_flow=40.0)
        pc.init_param_flows(flows_memory=0.0)
        pc(x.to(DEV))
        pc.backward(x.to(DEV))
        pc.mini_batch_em(step_size=0.25, pseudocount=0.1, step_size_rescaling=True)
        assert pc._cum_flow == 0.0
        ok, err = rel_close(pc.params.data[pc.num_dummy_params:], ref_p[pc.num_dummy_params:])
        assert ok, f"rescaled update, sum parameters rel err {err}"
        for layer, ref in zip(pc.input_layer_group, ref_ip):
            ok, err = rel_close(layer.params.data, ref)
            assert ok, f"rescaled update, input parameters rel err {err}"
    _lib.check_status(DEV)
