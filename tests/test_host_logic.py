"""CPU-side checks: the shared library and its header agree, structure generators and data generators behave,
and unsupported options are rejected instead of being silently ignored."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import pyjuice_b200 as pj
from pyjuice_b200 import _lib
from pyjuice_b200.compiler import partition_nodes_by_n_edges
from pyjuice_b200.structures import Tree, minimum_spanning_tree

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "pcx_b200.h")).read()
    return sorted(set(re.findall(r"^\s*(?:int|int64_t)\s+(pcx_\w+)\s*\(", text, flags=re.M)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared_symbols()
    assert len(names) >= 14
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/pcx_b200.h but not exported"
    assert set(_lib.SIGNATURES) | set(_lib.PLAIN) == set(names), "ctypes prototypes and header disagree"
    assert lib.pcx_build_arch() == 100


def test_chow_liu_matches_networkx():
    nx = pytest.importorskip("networkx")
    rng = np.random.default_rng(0)
    for n in (5, 17, 40):
        mi = rng.random((n, n)).astype(np.float32)
        mi = (mi + mi.T) / 2
        g = nx.Graph()
        for v in range(n):
            g.add_node(v)
            for u in range(v):
                g.add_edge(u, v, weight=-mi[u, v])
        t_ref = nx.minimum_spanning_tree(g)
        t = minimum_spanning_tree(-mi.astype(np.float64))
        assert [tuple(e) for e in t_ref.edges()] == [tuple(e) for e in _edges_in_nx_order(t)]
        root = nx.center(t_ref)[0]
        assert root == t.center()
        assert list(nx.dfs_postorder_nodes(t_ref, root)) == t.dfs_postorder(root)
        clt = nx.bfs_tree(t_ref, root)
        ch = t.rooted_children(root)
        for v in range(n):
            assert list(clt.successors(v)) == ch[v]


def _edges_in_nx_order(t: Tree):
    seen, out = set(), []
    for u in range(t.n):
        for v in t.adj[u]:
            if v not in seen:
                out.append((u, v))
        seen.add(u)
    return out


def test_partition_examples():
    # one value -> one group; widely spread values split until the padded work is within (1 + tol) of the real work
    assert partition_nodes_by_n_edges(np.array([8, 8, 8]), sparsity_tolerance=0.5).tolist() == [8]
    out = partition_nodes_by_n_edges(np.array([1] * 50 + [64] * 2), sparsity_tolerance=0.1)
    assert out.tolist() == [1, 64]
    assert partition_nodes_by_n_edges(np.array([3, 5, 9]), max_num_partitions=1).tolist() == [9]


def test_data_generators_are_seeded_and_in_range():
    from pyjuice_b200 import data
    a = data.tree_bn_samples(256, 32, 4, seed=0)
    b = data.tree_bn_samples(256, 32, 4, seed=0)
    assert np.array_equal(a, b) and a.min() >= 0 and a.max() < 4 and a.shape == (256, 32)
    x, tree, root = data.grid_gaussian_bn_samples(128, 6, 6, seed=1, num_cats=64)
    assert x.shape == (128, 36) and x.max() < 64 and len(tree.edges) == 35
    m = data.mixture_samples(64, 20, 16, seed=3)
    assert m.shape == (64, 20) and m.max() < 16
    h = data.hmm_samples(32, 10, vocab=500, seed=4, num_states=16)
    assert h.shape == (32, 10) and h.max() < 500


def test_unsupported_options_raise():
    ns = pj.structures.HMM(seq_length=4, num_latents=4, num_emits=5)
    pc = pj.compile(ns)
    with pytest.raises(NotImplementedError):
        pc.forward(torch.zeros(2, 4, dtype=torch.long))           # no CPU path
    with pytest.raises(AssertionError):
        pj.optim.MiniBatchEM(pc, sync_every=0)


def test_parameters_are_normalised_after_compile():
    torch.manual_seed(0)
    ns = pj.structures.RAT_SPN(num_vars=12, num_latents=8, depth=2, num_repetitions=2, num_cats=5, block_size=4)
    pc = pj.compile(ns)
    eb = pc._em_blocks
    for i in range(eb["par"].numel()):
        p0, fan, bs = int(eb["par"][i]), int(eb["fan"][i]), int(eb["bs"][i])
        s = pc.params.data[p0:p0 + fan * bs].view(fan, bs).sum(dim=0)
        assert torch.allclose(s, torch.ones_like(s), atol=1e-5)
    assert torch.all(pc.params.data[:pc.num_dummy_params] == 0)


def test_patch_pyjuice_rebinds_the_front_door(monkeypatch):
    """`patch_pyjuice` swaps the compiled path of an installed PyJuice for this engine (a stand-in module here)."""
    import sys
    import types
    import pyjuice_b200 as pj
    fake = types.ModuleType("pyjuice")
    fake.model = types.ModuleType("pyjuice.model")
    fake.optim = types.ModuleType("pyjuice.optim")
    fake.compile = fake.TensorCircuit = fake.model.compile = fake.model.TensorCircuit = None
    monkeypatch.setitem(sys.modules, "pyjuice", fake)
    out = pj.patch_pyjuice()
    assert out is fake
    assert fake.compile is pj.compile and fake.model.TensorCircuit is pj.TensorCircuit
    assert fake.optim.MiniBatchEM is pj.optim.MiniBatchEM and fake.optim.FullBatchEM is pj.optim.FullBatchEM


def test_table_validation_accepts_compiled_circuits_and_names_a_bad_index():
    """`validate_tables` checks every compiled index against the buffer it indexes (the static part of what a
    sanitizer run would check); a corrupted entry is reported with its table."""
    import sys, os
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    from cases import CASES, OursApi
    import pytest
    api = OursApi()
    for name in ("hclt_grid", "pd_small", "hmm_blocks", "sparse_sum", "tied_sums"):
        torch.manual_seed(0)
        ns, kw = CASES[name](api)
        ns.init_parameters()
        pc = api.compile(ns, **kw)
        counts = pc.validate_tables()
        assert counts["sum cids"] > 0 and counts["prod cids"] > 0 and counts["input vids"] > 0
    layer = [l for g in pc.inner_layer_groups for l in g if not g.is_prod()][0]
    saved = layer.partitioned_cids[0][0, 0].item()
    layer.partitioned_cids[0][0, 0] = pc.num_elements + 5
    with pytest.raises(ValueError, match="sum cids"):
        pc.validate_tables()
    layer.partitioned_cids[0][0, 0] = saved
    layer.partitioned_pids[0][0, 0] = pc.params.numel()
    with pytest.raises(ValueError, match="sum pids"):
        pc.validate_tables()


def test_public_header_is_plain_c():
    """`include/pcx_b200.h` is the boundary a non-Python host binds: it must compile as C99 on its own (no C++, no
    torch or CUDA types in the signatures)."""
    import os, shutil, subprocess, tempfile
    import pytest
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "h.c")
        open(src, "w").write('#include "include/pcx_b200.h"\nint main(void) { return 0; }\n')
        r = subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", "-I", root, src],
                           capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
