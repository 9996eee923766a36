"""Checkpoints (`.jpc`): a circuit survives save -> load with its structure, tying and parameters intact; a file
written by the reference's own `save` (tests/golden/ref_hmm_blocks.jpc, made by tests/golden/make_golden.py) loads
and compiles to the reference compiler's tables; leaf distributions are recorded under the class path the reference
unpickles; records that name anything but NumPy helpers and leaf distributions are refused."""
import os
import pickle

import numpy as np
import pytest
import torch

import pyjuice_b200 as pj
from pyjuice_b200 import io as pio
from cases import CASES, OursApi, dump_tables

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _small():
    with pj.set_block_size(4):
        leaves = [pj.inputs(v, 2, pj.Categorical(num_cats=5)) for v in (0, 0, 1, 1)]
        m0, m1 = pj.multiply(leaves[0], leaves[2]), pj.multiply(leaves[1], leaves[3])
        return pj.summate(m0, m1, num_node_blocks=2)


def _same(a, b, params=True):
    va, vb = list(a), list(b)
    assert len(va) == len(vb)
    ia, ib = {id(n): i for i, n in enumerate(va)}, {id(n): i for i, n in enumerate(vb)}
    for x, y in zip(va, vb):
        assert (x.is_input(), x.is_prod(), x.is_sum()) == (y.is_input(), y.is_prod(), y.is_sum())
        assert (x.num_node_blocks, x.block_size) == (y.num_node_blocks, y.block_size)
        assert [ia[id(c)] for c in x.chs] == [ib[id(c)] for c in y.chs]
        assert x.is_tied() == y.is_tied()
        if x.is_tied():
            assert ia[id(x.get_source_ns())] == ib[id(y.get_source_ns())]
        if x.is_input():
            assert x.scope == y.scope and x.dist.num_cats == y.dist.num_cats
        else:
            assert torch.equal(x.edge_ids, y.edge_ids)
        if params:
            assert (x._params is None) == (y._params is None)
            if x._params is not None:
                assert torch.equal(x._params, y._params)


def test_structure_round_trip(tmp_path):
    ns = _small()
    pj.save(str(tmp_path / "a.jpc"), ns)
    _same(ns, pj.load(str(tmp_path / "a.jpc")))
    with pytest.raises(ValueError):
        pj.save(str(tmp_path / "a.bin"), ns)
    with pytest.raises(ValueError):
        pj.load(str(tmp_path / "a.bin"))


def test_parameters_and_tying_round_trip(tmp_path):
    torch.manual_seed(2)
    ns = pj.structures.HMM(seq_length=6, num_latents=8, num_emits=13)
    ns.init_parameters()
    pj.save(str(tmp_path / "hmm.jpc"), ns)
    back = pj.load(str(tmp_path / "hmm.jpc"))
    _same(ns, back)
    pa, pb = pj.compile(ns), pj.compile(back)                     # and the compiled parameter vectors agree
    assert torch.equal(pa.params.data, pb.params.data)
    assert torch.equal(pa.input_layer_group[0].params.data, pb.input_layer_group[0].params.data)


def test_saving_a_compiled_circuit_writes_its_current_parameters(tmp_path):
    torch.manual_seed(4)
    ns = _small()
    ns.init_parameters()
    pc = pj.compile(ns)
    initial = pc.params.data.clone()
    with torch.no_grad():                                         # stand-in for training: new normalised parameters
        pc.params.data.mul_(torch.rand_like(pc.params.data) + 0.5)
        pc._normalize_parameters(pc.params.data)
        leaf = pc.input_layer_group[0].params.data
        leaf.copy_(torch.softmax(torch.randn(leaf.numel() // 5, 5), dim=1).reshape(-1))
    pj.save(str(tmp_path / "pc.jpc"), pc)
    back = pj.compile(pj.load(str(tmp_path / "pc.jpc")))
    assert torch.equal(back.input_layer_group[0].params.data, pc.input_layer_group[0].params.data)
    assert not torch.allclose(back.params.data, initial, rtol=1e-3)      # not the initial ones
    assert torch.allclose(back.params.data, pc.params.data, rtol=1e-6, atol=1e-9)   # compile normalises once more


def test_reference_written_checkpoint_loads_and_compiles_to_the_golden_tables():
    ns = pj.load(os.path.join(GOLDEN, "ref_hmm_blocks.jpc"))
    api = OursApi()
    built, kw = CASES["hmm_blocks"](api)
    _same(built, ns, params=False)
    for v in ns:
        if not v.is_prod() and not v.is_tied():
            assert v._params is not None and torch.isfinite(v._params).all()
    ours = dump_tables(api.compile(ns, **kw))
    ref = np.load(os.path.join(GOLDEN, "hmm_blocks.npz"))
    assert sorted(ours) == sorted(ref.files)
    for key in ref.files:
        assert np.array_equal(np.asarray(ours[key]), ref[key]), key


def test_leaf_distribution_record_names_the_reference_class(tmp_path):
    blob = pio._dump_dist(pj.Categorical(num_cats=7))
    assert b"pyjuice.nodes.distributions.categorical\nCategorical\n" in blob
    d = pio._load_dist(blob)
    assert isinstance(d, pj.Categorical) and d.num_cats == 7 and d.get_metadata() == [7]


def test_foreign_globals_are_refused(tmp_path):
    import subprocess
    evil = pickle.dumps([{"type": "Input", "num_node_blocks": 1, "block_size": 1, "chs": (), "scope": [0],
                          "dist": pickle.dumps(subprocess.Popen)}])
    (tmp_path / "evil.jpc").write_bytes(evil)
    with pytest.raises(pickle.UnpicklingError):
        pj.load(str(tmp_path / "evil.jpc"))
    (tmp_path / "evil2.jpc").write_bytes(pickle.dumps([subprocess.Popen]))
    with pytest.raises(pickle.UnpicklingError):
        pj.load(str(tmp_path / "evil2.jpc"))
