"""GPU parity: the CUDA path (through the C ABI) against the CPU oracle on seeded circuits and inputs.

Tolerances (fp32 kernels vs the fp64 oracle): per-sample log-likelihood within 1e-3 nats absolute; node
flows, parameter flows and post-EM parameters within 1e-3 relative.
"""
import numpy as np
import pytest
import torch

import pyjuice_b200 as pj
from cases import CASES, OursApi
from helpers import check_against_oracle, oracle_step, rel_close, LL_ATOL

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _data_for(pc, B, seed=0):
    g = torch.Generator().manual_seed(seed)
    layer = pc.input_layer_group[0]
    cats = torch.zeros(pc.num_vars, dtype=torch.long)
    cats[layer.vids[:, 0].cpu()] = layer.node_cats.cpu()
    return (torch.rand(B, pc.num_vars, generator=g) * cats[None, :].clamp(min=1)).long()


def _build(name, seed=0):
    api = OursApi()
    torch.manual_seed(seed)
    ns, kw = CASES[name](api)
    ns.init_parameters()
    return api.compile(ns, **kw)


@pytest.mark.parametrize("name", sorted(CASES))
def test_step_matches_oracle(name):
    pc = _build(name).to(DEV)
    errs = check_against_oracle(pc, _data_for(pc, 64))
    print(name, errs)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("B", [5, 128, 200])
@pytest.mark.parametrize("name", ["hclt_b128", "hmm_b128"])
def test_sum_arithmetic_modes(name, B, mode):
    """fp32 CUDA-core kernels (mode 0) and the tcgen05 kernels with split-bf16 operands (mode 1) both meet the bar."""
    from pyjuice_b200 import _lib
    _lib.set_sum_mode(mode)
    try:
        pc = _build(name, seed=7).to(DEV)
        errs = check_against_oracle(pc, _data_for(pc, B, seed=B))
        print(name, B, mode, errs)
        _lib.check_status()
    finally:
        _lib.set_sum_mode(1)


@pytest.mark.parametrize("B", [1, 3, 33, 100, 256])
@pytest.mark.parametrize("name", ["simple_model", "simple_model_bs1", "hclt_grid", "hmm_blocks", "pd_small"])
def test_ragged_batch_sizes(name, B):
    pc = _build(name, seed=1).to(DEV)
    check_against_oracle(pc, _data_for(pc, B, seed=B))


@pytest.mark.parametrize("name", ["simple_model", "simple_model_bs4", "hmm_small", "rat_small"])
def test_linear_space_flows(name):
    pc = _build(name, seed=2).to(DEV)
    check_against_oracle(pc, _data_for(pc, 48), logspace_flows=False)


def test_graph_replay_equals_eager_and_accumulates():
    pc = _build("hclt_grid", seed=3).to(DEV)
    x = _data_for(pc, 128)
    ref_lls, st, _ = oracle_step(pc, x)
    pc.init_param_flows(flows_memory=0.0)
    for it in range(4):                     # eager, warm, captured, replayed
        lls = pc(x.to(DEV))
        pc.backward(x.to(DEV))
        assert (lls.double().cpu() - ref_lls).abs().max().item() <= LL_ATOL
    ok, err = rel_close(pc.param_flows, 4 * st.param_flows)
    assert ok, f"accumulated flows rel err {err}"
    pc.use_cuda_graphs = False
    pc.init_param_flows(flows_memory=0.0)
    lls2 = pc(x.to(DEV))
    pc.backward(x.to(DEV))
    assert torch.equal(lls, lls2)
    ok, err = rel_close(pc.param_flows, st.param_flows)
    assert ok


def test_autograd_hook_and_optimizer_increase_ll():
    pc = _build("hclt_cfg0", seed=4).to(DEV)
    from pyjuice_b200.data import tree_bn_samples
    data = torch.from_numpy(tree_bn_samples(4096, 32, 4, seed=0))
    opt = pj.optim.MiniBatchEM(pc, step_size=0.1, pseudocount=0.1)
    first = last = None
    for epoch in range(3):
        tot = 0.0
        for i in range(0, 4096, 256):
            x = data[i:i + 256].to(DEV)
            lls = pc(x)
            lls.mean().backward()
            opt.step()
            tot += lls.mean().item()
        first = tot if first is None else first
        last = tot
    assert last > first, f"EM did not improve the log-likelihood: {first} -> {last}"


def test_weighted_backward_matches_oracle():
    pc = _build("simple_model", seed=5).to(DEV)
    x = _data_for(pc, 40)
    w = torch.rand(40) + 0.5
    ref_lls, st, _ = oracle_step(pc, x, ll_weights=w)
    pc.init_param_flows(flows_memory=0.0)
    pc(x.to(DEV))
    pc.backward(x.to(DEV), ll_weights=w.to(DEV))
    ok, err = rel_close(pc.param_flows, st.param_flows)
    assert ok, err
    assert abs(pc._cum_flow - w.sum().item()) < 1e-3


def test_layer_level_calls_and_accessors():
    """Drive layers one by one, as the reference's tests do (simple_model_test.py:225-289)."""
    pc = _build("simple_model", seed=6).to(DEV)
    x = _data_for(pc, 32)
    ref_lls, st, _ = oracle_step(pc, x)
    pc.use_cuda_graphs = False
    pc(x.to(DEV))
    pc.backward(x.to(DEV), logspace_flows=False)
    ns = pc.root_ns
    np4 = ns.chs[0]
    got = pc.get_node_mars(np4).double().cpu()
    pc.inner_layer_groups[2][0].forward(pc.node_mars, pc.element_mars)
    s, e = np4._output_ind_range
    assert torch.allclose(pc.element_mars[s:e].double().cpu(), got)
    pc.inner_layer_groups[3][0].backward(pc.node_flows, pc.element_flows, pc.node_mars, pc.element_mars, pc.params,
                                         None, logspace_flows=False)
    ref = st.element_flows   # oracle leaves the last-processed (deepest-first) layer; recompute through node flows
    ns0 = np4.chs[0]
    a, b = ns0._output_ind_range
    assert torch.allclose(pc.element_flows[s:e].double().cpu(), pc.node_flows[a:b].double().cpu(), rtol=1e-4, atol=1e-7)
    p = pc.get_node_params(ns0)
    assert p.shape == ns0._params.shape and torch.allclose(p.cpu(), ns0._params, atol=1e-6)


@pytest.mark.parametrize("name", ["hclt_b128", "hmm_b128"])
def test_folded_product_layers_match_separate_kernels(name):
    """Folding the product layers into the sum kernels (and storing flows straight into node_flows) must not change
    any result; the two circuits exercise the direct-store case (tree) and shared children (HMM)."""
    pc = _build(name, seed=9).to(DEV)
    assert len(pc._fused) > 0, "expected the 128-block depths to be foldable"
    x = _data_for(pc, 64, seed=2).to(DEV)
    out = {}
    for fuse in (True, False):
        pc.fuse_product_layers = fuse
        pc.init_param_flows(flows_memory=0.0)
        lls = pc(x)
        pc.backward(x)
        torch.cuda.synchronize()
        out[fuse] = (lls.clone(), pc.node_flows[pc.num_dummy_nodes:].exp().clone(), pc.param_flows.clone(),
                     pc.input_layer_group[0].param_flows.clone())
    for a, b in zip(out[True], out[False]):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-6), (a - b).abs().max()


@pytest.mark.parametrize("name,batch", [("hclt_b128", 64), ("hclt_b128", 200), ("hmm_b128", 72)])
@pytest.mark.parametrize("tile", [None, 16, 32, 64])
def test_dataflow_launch_matches_per_layer_launches(name, batch, tile):
    """A run of depths executed as ONE launch whose tiles wait on counters must give exactly what the per-layer
    launches give (same tiles, same arithmetic), for every tile width, with and without CUDA graphs, repeatedly
    (the counters are cleared by every call)."""
    pc = _build(name, seed=11).to(DEV)
    x = _data_for(pc, batch, seed=3).to(DEV)
    out = {}
    for dataflow in (False, True):
        pc.use_dataflow_launch = dataflow
        pc.chain_tile = tile if dataflow else None
        for rep in range(3 if dataflow else 1):              # eager, captured, replayed
            pc.init_param_flows(flows_memory=0.0)
            lls = pc(x)
            pc.backward(x)
            torch.cuda.synchronize()
        out[dataflow] = (lls.clone(), pc.node_flows[pc.num_dummy_nodes:].exp().clone(), pc.param_flows.clone(),
                         pc.input_layer_group[0].param_flows.clone())
    if batch % 8 == 0:
        assert pc._chain_plan(batch, 0) is not None and pc._chain_plan(batch, 1) is not None
    for a, b in zip(out[True], out[False]):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-7), (a - b).abs().max()


@pytest.mark.parametrize("latents", [2, 8, 64])
def test_products_without_a_parent_receive_no_flow(latents):
    """Block-sparse sum vectors can leave product blocks without a parent (Poon-Domingos circuits do).  Their rows
    of the shared element-flow buffer are not written by the element-flow kernels; they must read as "no flow" on
    every pass — eager, captured and replayed — not as whatever another depth or the previous pass left there."""
    import random
    torch.manual_seed(0)
    random.seed(0)
    ns = pj.structures.PD((8, 8), num_latents=latents, split_points=[[2, 4, 6], [2, 4, 6]], num_cats=4)
    ns.init_parameters()
    pc = pj.compile(ns).to(DEV)
    x = torch.randint(0, 4, (64, pc.num_vars))
    if latents == 2:
        assert len(pc._parentless) > 0
    for rep in range(4):
        errs = check_against_oracle(pc, x, step=0.05, pseudo=0.1)
    layer = pc.input_layer_group[0]
    s, e = layer._output_ind_range
    per_var = torch.zeros(pc.num_vars, 64, device=DEV)
    per_var.index_add_(0, layer.vids[:, 0].to(DEV), pc.node_flows[s:e].exp())
    assert (per_var - 1.0).abs().max().item() < 1e-4


def test_no_kernel_reported_a_failed_wait():
    from pyjuice_b200 import _lib
    torch.cuda.synchronize()
    _lib.check_status()


def test_cpu_use_fails_loudly():
    pc = _build("simple_model_bs1")
    with pytest.raises(NotImplementedError):
        pc(torch.zeros(4, 4, dtype=torch.long))


def test_c_abi_direct_calls():
    """Call entry points with raw pointers, as a non-Python host would."""
    from pyjuice_b200 import _lib
    lib = _lib.load()
    assert lib.pcx_build_arch() == 100
    n = 100003
    t = torch.empty(n, device=DEV)
    _lib.call("pcx_fill_f32", t, n, 2.5)
    _lib.call("pcx_scale_f32", t, n, 2.0)
    assert torch.all(t == 5.0)
    # product forward on a hand-made table: 3 row blocks of 4 nodes, up to 2 children, B = 20
    B, bs = 20, 4
    nm = torch.randn(40, B, device=DEV)
    em = torch.full((16, B), float("-inf"), device=DEV)
    nids = torch.tensor([4, 8, 12], dtype=torch.int32, device=DEV)
    cids = torch.tensor([[4, 8], [12, 0], [20, 36]], dtype=torch.int32, device=DEV)
    _lib.call("pcx_prod_fwd", em, nm, nids, cids, 3, 2, bs, B)
    ref = torch.stack([nm[4:8] + nm[8:12], nm[12:16], nm[20:24] + nm[36:40]]).reshape(12, B)
    assert torch.allclose(em[4:16], ref, atol=1e-6)
    assert torch.isinf(em[:4]).all()


@pytest.mark.parametrize("homogeneous", [True, False])
@pytest.mark.parametrize("B", [32, 64, 192, 256, 320])
def test_dense_layers_match_oracle_and_tiled_kernels(B, homogeneous):
    """Deep tables (here 1024 x 1024 transition blocks) take the two-step dense path: operand pre-pass plus a GEMM
    over pre-tiled operands, parameter flows of tied layers in one product over their concatenated batches.  The
    wide-tile kernels (128 rows x up to 256 samples, split contraction, product layer folded in, flows stored directly
    into the children's rows) are checked against the oracle, against the first-generation dense kernels (batches
    that are multiples of 64) and against the tile-at-a-time kernels, over repeated (eager, captured, replayed) steps."""
    from pyjuice_b200.layers import SumLayer
    torch.manual_seed(3)
    ns = pj.structures.HMM(seq_length=5, num_latents=1024, num_emits=16, homogeneous=homogeneous)
    ns.init_parameters()
    pc = pj.compile(ns).to(DEV)
    x = torch.randint(0, 16, (B, 5))
    assert any(l._wide_ok(0, B, False) for g in pc.inner_layer_groups if g.is_sum() for l in g), "expected dense tables"
    assert any(f.get("dense") for f in pc._fused.values()), "expected depths with the product layer folded into the dense kernels"
    for rep in range(3):
        check_against_oracle(pc, x, step=0.05, pseudo=0.1)
    check_against_oracle(pc, x, step=0.05, pseudo=0.1, logspace_flows=False)
    out = {}
    try:
        for mode, (dense, wide) in {"wide": (True, True), "dense": (True, False), "tiled": (False, False)}.items():
            SumLayer.use_dense_kernels, SumLayer.use_wide_dense = dense, wide
            pc.init_param_flows(flows_memory=0.0)
            lls = pc(x.to(DEV))
            pc.backward(x.to(DEV))
            torch.cuda.synchronize()
            out[mode] = (lls.clone(), pc.node_flows[pc.num_dummy_nodes:].exp().clone(), pc.param_flows.clone())
    finally:
        SumLayer.use_dense_kernels, SumLayer.use_wide_dense = True, True
    for other in ("dense", "tiled"):
        for a, b in zip(out["wide"], out[other]):
            assert torch.allclose(a, b, rtol=2e-4, atol=1e-6), (other, (a - b).abs().max())
    # two runs of the split contraction give bit-equal results: partial tiles are added in a fixed order
    pc.init_param_flows(flows_memory=0.0)
    lls2 = pc(x.to(DEV))
    assert torch.equal(lls2, out["wide"][0])
    _lib_status()


def test_wide_dense_kernels_without_folding_and_with_weights():
    """The wide-tile kernels behind the per-layer interface (element_mars / element_flows in use, no folding), and a
    weighted backward pass."""
    torch.manual_seed(4)
    ns = pj.structures.HMM(seq_length=4, num_latents=1024, num_emits=12, homogeneous=True)
    ns.init_parameters()
    pc = pj.compile(ns).to(DEV)
    pc.fuse_product_layers = False
    x = torch.randint(0, 12, (72, 4))
    check_against_oracle(pc, x, step=0.1, pseudo=0.1)
    pc.fuse_product_layers = True
    w = torch.rand(72) + 0.5
    ref_lls, st, _ = oracle_step(pc, x, ll_weights=w)
    pc.init_param_flows(flows_memory=0.0)
    pc(x.to(DEV))
    pc.backward(x.to(DEV), ll_weights=w.to(DEV))
    ok, err = rel_close(pc.param_flows, st.param_flows)
    assert ok, err
    _lib_status()


@pytest.mark.parametrize("B", [64, 100, 30])
@pytest.mark.parametrize("homogeneous", [True, False])
def test_large_vocabulary_leaves_use_the_transposed_shadow(B, homogeneous):
    """Categorical leaves with more categories than the staged kernels hold (here 9000) are looked up through a
    transposed copy of the parameter table and accumulate their flows in the same layout; flows of tied replicas are
    reported in the source range.  Batches that are not multiples of 4 take the general kernels instead."""
    torch.manual_seed(8)
    ns = pj.structures.HMM(seq_length=6, num_latents=32, num_emits=9000, homogeneous=homogeneous, block_size=8)
    ns.init_parameters()
    pc = pj.compile(ns, max_tied_ns_per_parflow_block=2).to(DEV)
    layer = pc.input_layer_group[0]
    assert layer._shadow is not None
    assert layer._shadow_ok(B) == (B % 4 == 0)
    x = torch.randint(0, 9000, (B, 6))
    x[:, 0] = torch.arange(B) % 7                       # repeated tokens: several samples add to one row of flows
    for rep in range(3):
        errs = check_against_oracle(pc, x, step=0.2, pseudo=0.1, fold_input_flows=True)
    print(B, homogeneous, errs)
    # decaying flows over several steps, shadow flows included
    from helpers import OracleTrainer
    ref = OracleTrainer(pc)
    pc.init_param_flows(flows_memory=0.0)
    for i in range(3):
        xi = torch.randint(0, 9000, (B, 6))
        pc(xi.to(DEV))
        pc.backward(xi.to(DEV), flows_memory=0.5)
        pc.mini_batch_em(step_size=0.3, pseudocount=0.1)
        ref.accumulate(xi, flows_memory=0.5)
        ref.update(0.3, 0.1, zero_flows=False)
        ref.check_params(pc)
    _lib_status()


def _lib_status():
    from pyjuice_b200 import _lib
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("B", [64, 36])
@pytest.mark.parametrize("homogeneous", [True, False])
def test_em_straight_from_the_transposed_shadow(B, homogeneous, monkeypatch):
    """When all flows of an update sit in the transposed shadow (nobody read `param_flows`, no data-parallel
    exchange), the leaf parameters and the transposed log-parameter table are updated straight from it.  Same
    parameters, same likelihoods afterwards and the same flows on a later read as the three-kernel path (move the
    flows, update, rebuild the shadow), and as the oracle."""
    from pyjuice_b200 import _lib
    from helpers import OracleTrainer
    calls = []
    orig = _lib.call
    monkeypatch.setattr(_lib, "call", lambda name, *a: (calls.append(name), orig(name, *a))[1])
    pcs = []
    for fused in (True, False):
        torch.manual_seed(8)
        ns = pj.structures.HMM(seq_length=6, num_latents=32, num_emits=9000, homogeneous=homogeneous, block_size=8)
        ns.init_parameters()
        pc = pj.compile(ns, max_tied_ns_per_parflow_block=2).to(DEV)
        pc.input_layer_group[0].use_fused_shadow_em = fused
        pcs.append(pc)
    ref = OracleTrainer(pcs[0])
    opts = [pj.optim.MiniBatchEM(pc, step_size=0.3, pseudocount=0.1) for pc in pcs]
    for i in range(3):
        xi = torch.randint(0, 9000, (B, 6))
        xi[:, 0] = torch.arange(B) % 5
        for pc, opt in zip(pcs, opts):
            calls.clear()
            pc(xi.to(DEV)).mean().backward()
            opt.step()
            fused = pc.input_layer_group[0].use_fused_shadow_em
            assert ("pcx_em_input_cat_t" in calls) == fused and ("pcx_input_cat_flush_t" in calls) == (not fused)
        ref.accumulate(xi, flows_memory=0.0)
        ref.update(0.3, 0.1, zero_flows=True)
        ref.check_params(pcs[0])
        a, b = (pc.input_layer_group[0].params.data for pc in pcs)
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-9), (a - b).abs().max()
    x = torch.randint(0, 9000, (B, 6)).to(DEV)
    lls = [pc(x) for pc in pcs]
    assert torch.allclose(lls[0], lls[1], rtol=0, atol=1e-4)
    # the flows of an update stay readable after the update from the shadow
    flows = []
    for pc in pcs:
        pc.init_param_flows(flows_memory=0.0)
        pc(x)
        pc.backward(x)
        pc.mini_batch_em(step_size=0.3, pseudocount=0.1)
        flows.append(pc.input_layer_group[0].param_flows.clone())
    assert torch.allclose(flows[0], flows[1], rtol=1e-5, atol=1e-7) and float(flows[0].sum()) > 0
    _lib_status()


@pytest.mark.parametrize("B", [64, 100, 256])
@pytest.mark.parametrize("case", ["pd", "rat", "hmm64", "hmm32_tied"])
def test_small_blocks_on_tensor_cores_match_oracle_and_cuda_core_kernels(case, B):
    """Node blocks of 32 / 64 run as sample-major tensor-core tiles (128 samples x 32 / 64 nodes; pairs of blocks that
    list the same children share a tile).  Checked against the oracle, against the fp32 CUDA-core kernels, over
    repeated steps, with ragged batches."""
    import random
    from pyjuice_b200.layers import SumLayer
    torch.manual_seed(5)
    random.seed(5)
    if case == "pd":
        ns = pj.structures.PD((8, 8), num_latents=64, split_points=[[2, 4, 6], [4]], num_cats=6)
    elif case == "rat":
        ns = pj.structures.RAT_SPN(num_vars=24, num_latents=32, depth=3, num_repetitions=4, num_cats=6)
    elif case == "hmm64":
        ns = pj.structures.HMM(seq_length=6, num_latents=64, num_emits=6, homogeneous=False)
    else:
        ns = pj.structures.HMM(seq_length=7, num_latents=32, num_emits=6, homogeneous=True)
    ns.init_parameters()
    pc = pj.compile(ns).to(DEV)
    used = [l for g in pc.inner_layer_groups if g.is_sum() for l in g
            if any(t is not None for t in getattr(l, "_sm_fw", [None]))]
    assert used, "expected layers with sample-major tables"
    x = torch.randint(0, 6, (B, pc.num_vars))
    for rep in range(3):
        check_against_oracle(pc, x, step=0.05, pseudo=0.1)
    check_against_oracle(pc, x, step=0.05, pseudo=0.1, logspace_flows=False)
    out = {}
    try:
        for sm in (True, False):
            SumLayer.use_sample_major = sm
            pc.init_param_flows(flows_memory=0.0)
            lls = pc(x.to(DEV))
            pc.backward(x.to(DEV))
            torch.cuda.synchronize()
            out[sm] = (lls.clone(), pc.node_flows[pc.num_dummy_nodes:].exp().clone(), pc.param_flows.clone())
    finally:
        SumLayer.use_sample_major = True
    for a, b in zip(out[True], out[False]):
        assert torch.allclose(a, b, rtol=2e-4, atol=1e-6), (a - b).abs().max()
    _lib_status()


@pytest.mark.parametrize("name", ["hmm_blocks", "hclt_b128"])
def test_checkpoint_of_a_trained_circuit_reloads_to_the_same_likelihoods(name, tmp_path):
    """Train a few EM steps on the device, save the compiled circuit, load and compile the file: the new circuit
    gives the same log-likelihoods (its parameters pass through one more host-side normalisation: 1e-4 nats)."""
    pc = _build(name).to(DEV)
    x = _data_for(pc, 64).to(DEV)
    opt = pj.optim.MiniBatchEM(pc, step_size=0.3, pseudocount=0.05)
    before = pc(x).clone()
    for _ in range(3):
        pc(x).mean().backward()
        opt.step()
    after = pc(x).clone()
    assert (after.mean() > before.mean()).item()
    pj.save(str(tmp_path / "trained.jpc"), pc)
    pc2 = pj.compile(pj.load(str(tmp_path / "trained.jpc"))).to(DEV)
    assert torch.allclose(pc2.params.data, pc.params.data, rtol=1e-5, atol=1e-9)
    assert torch.allclose(pc2(x), after, rtol=0, atol=1e-4)


def test_allow_modify_flows_is_accepted_and_changes_nothing():
    """The flag only permits overwriting node flows in place (linear flows); results are those without it, and it
    is rejected together with log-space flows as in the reference (layer/sum_layer.py:442)."""
    pc = _build("hclt_cfg0", seed=3).to(DEV)
    x = _data_for(pc, 32).to(DEV)
    pc(x)
    pc.backward(x, logspace_flows=False, flows_memory=0.0)
    want = pc.param_flows.clone()
    pc.backward(x, logspace_flows=False, flows_memory=0.0, allow_modify_flows=True)
    assert torch.equal(pc.param_flows, want)
    with pytest.raises(AssertionError):
        pc.backward(x, logspace_flows=True, allow_modify_flows=True)


def test_arithmetic_mode_belongs_to_the_circuit_and_the_calling_thread():
    """Two circuits in one process keep their own arithmetic (`pc.sum_mode`): interleaved steps of an fp32
    CUDA-core circuit and a tensor-core circuit give what each gives alone, and a step driven from a second host
    thread under another process default does not change the first thread's results."""
    import threading
    from pyjuice_b200 import _lib
    pc_a, pc_b, pc_c = (_build("hmm_b128", seed=3).to(DEV) for _ in range(3))
    x = _data_for(pc_a, 64, seed=3).to(DEV)
    pc_a.sum_mode, pc_b.sum_mode = 0, 2

    def step(pc):
        lls = pc(x)
        pc.backward(x, flows_memory=0.0)
        return lls.clone(), pc.param_flows.clone()

    alone_a, alone_b = step(pc_a), step(pc_b)
    assert not torch.equal(alone_a[0], alone_b[0]), "fp32 and single-bf16 arithmetic must differ somewhere"
    for _ in range(2):                                   # interleaved: graphs and launch plans are keyed by the mode
        got_b, got_a = step(pc_b), step(pc_a)
        # likelihoods bit for bit; parameter flows are sums of float atomics, equal up to their order
        assert torch.equal(got_a[0], alone_a[0]) and torch.allclose(got_a[1], alone_a[1], rtol=1e-5, atol=1e-7)
        assert torch.equal(got_b[0], alone_b[0]) and torch.allclose(got_b[1], alone_b[1], rtol=1e-5, atol=1e-7)
    ref_c = step(pc_c)                                   # the process default (split bf16)
    out = {}

    def other_thread():
        with _lib.use_sum_mode(0):
            out["c_fp32"] = step(pc_c)
        out["c_default"] = step(pc_c)

    t = threading.Thread(target=other_thread)
    t.start()
    t.join()
    torch.cuda.synchronize()
    assert torch.equal(out["c_fp32"][0], alone_a[0]) and torch.equal(out["c_default"][0], ref_c[0])
    assert torch.equal(step(pc_c)[0], ref_c[0]) and _lib.sum_mode() == 1


@pytest.mark.parametrize("B", [24, 33, 128])
@pytest.mark.parametrize("name", ["hclt_b128", "hmm_b128", "pd_small", "rat_small", "hclt_grid", "tied_sums", "sparse_sum"])
def test_every_row_is_written_and_runs_repeat_bit_for_bit(name, B):
    """Race / coverage checks that need no sanitizer.  (a) The value buffer and the flow buffer are filled with NaN
    before each pass (`debug_poison`): every row must be rewritten by the kernel that owns it, whichever kernel family,
    fold and tile shape the table takes — a NaN that survives is a tile nobody computed.  (b) Likelihoods, values and
    node flows involve no atomics: two runs on the same inputs are equal bit for bit (eager, captured, replayed), and
    equal to the run without poison.  Parameter flows are sums of float atomics: equal up to their order."""
    pc = _build(name, seed=5).to(DEV)
    pc.validate_tables()
    x = _data_for(pc, B, seed=B).to(DEV)
    runs = []
    for poison in (False, True, True, True):
        pc.debug_poison = poison
        pc.init_param_flows(flows_memory=0.0)
        lls = pc(x)
        pc.backward(x)
        torch.cuda.synchronize()
        if poison:
            pc.assert_no_poison(backward=True)
        runs.append((lls.clone(), pc.node_mars.clone(), pc.node_flows.clone(), pc.param_flows.clone()))
    nd = pc.num_dummy_nodes
    for r in runs[1:]:
        assert torch.equal(r[0], runs[0][0]) and torch.equal(r[1][nd:], runs[0][1][nd:])
        assert torch.equal(r[2][nd:], runs[0][2][nd:])
        assert torch.allclose(r[3], runs[0][3], rtol=1e-5, atol=1e-7)
    _lib_status()
