"""Circuit definitions shared by the golden-table generator and the parity tests.

Every case is a function ``build(api) -> (root_ns, compile_kwargs)`` where ``api`` is a thin adapter over
either this package or the reference PyJuice, so that one definition produces the same node DAG through
both front doors.  Cases mirror the reference's own test circuits
(tests/model/simple_model_test.py:17-50, tests/model/homogeneous_hmm_test.py,
tests/model/parameter_tying_test.py, tests/layer/sum_layer_test.py) and scaled-down versions of the five
benchmark configurations.
"""
from __future__ import annotations

import random

import numpy as np
import torch


class OursApi:
    """Adapter over ``pyjuice_b200``."""
    name = "ours"

    def __init__(self):
        import pyjuice_b200 as pj
        self.pj = pj
        self.inputs, self.multiply, self.summate = pj.inputs, pj.multiply, pj.summate
        self.set_block_size = pj.set_block_size

    def cat(self, n):
        return self.pj.Categorical(num_cats=n)

    def compile(self, ns, **kw):
        return self.pj.compile(ns, verbose=False, **kw)

    def hmm(self, **kw):
        return self.pj.structures.HMM(**kw)

    def pd(self, data_shape, num_latents, num_cats, **kw):
        return self.pj.structures.PD(data_shape, num_latents, num_cats=num_cats, **kw)

    def rat_spn(self, num_cats, **kw):
        return self.pj.structures.RAT_SPN(num_cats=num_cats, **kw)

    def hclt_from_tree(self, edges, n, root, num_latents, num_cats, **kw):
        tree = self.pj.structures.Tree(n, edges)
        return self.pj.structures.tree_to_hidden_circuit(tree, root, num_latents, num_cats, **kw)

    def hclt_from_data(self, x, num_latents, num_cats, **kw):
        return self.pj.structures.HCLT(x.float(), num_latents, num_cats=num_cats, **kw)


class RefApi:
    """Adapter over the reference ``pyjuice`` (must already be importable)."""
    name = "ref"

    def __init__(self):
        import pyjuice as juice
        import pyjuice.nodes.distributions as dists
        self.juice, self.dists = juice, dists
        self.inputs, self.multiply, self.summate = juice.inputs, juice.multiply, juice.summate
        self.set_block_size = juice.set_block_size

    def cat(self, n):
        return self.dists.Categorical(num_cats=n)

    def compile(self, ns, **kw):
        return self.juice.compile(ns, disable_gpu_compilation=True, verbose=False, **kw)

    def hmm(self, **kw):
        return self.juice.structures.HMM(**kw)

    def pd(self, data_shape, num_latents, num_cats, **kw):
        return self.juice.structures.PD(data_shape, num_latents, input_node_params={"num_cats": num_cats}, **kw)

    def rat_spn(self, num_cats, **kw):
        return self.juice.structures.RAT_SPN(input_node_params={"num_cats": num_cats}, **kw)

    def hclt_from_tree(self, edges, n, root, num_latents, num_cats, **kw):
        import networkx as nx
        from pyjuice.structures.compilation import BayesianTreeToHiddenRegionGraph
        g = nx.Graph()
        g.add_nodes_from(range(n))
        g.add_edges_from(edges)
        return BayesianTreeToHiddenRegionGraph(g, root, num_latents, self.dists.Categorical, {"num_cats": num_cats}, **kw)

    def hclt_from_data(self, x, num_latents, num_cats, **kw):
        return self.juice.structures.HCLT(x.float(), num_latents, input_node_params={"num_cats": num_cats}, **kw)


def _seed(s):
    torch.manual_seed(s)
    random.seed(s)
    np.random.seed(s)


# ---- the reference's own test circuits -----------------------------------------------------------

def simple_model(api, block_size=16):
    """tests/model/simple_model_test.py:17-50 (mixed category counts, shared inputs, 1-node root)."""
    with api.set_block_size(block_size):
        ni0 = api.inputs(0, num_node_blocks=2, dist=api.cat(4))
        ni1 = api.inputs(1, num_node_blocks=2, dist=api.cat(4))
        ni2 = api.inputs(2, num_node_blocks=2, dist=api.cat(6))
        ni3 = api.inputs(3, num_node_blocks=2, dist=api.cat(6))
        np0, np1 = api.multiply(ni0, ni1), api.multiply(ni2, ni3)
        np2, np3 = api.multiply(ni1, ni2), api.multiply(ni0, ni1)
        ns0 = api.summate(np0, np3, num_node_blocks=2)
        ns1 = api.summate(np1, num_node_blocks=2)
        ns2 = api.summate(np2, num_node_blocks=2)
        np4, np5, np6 = api.multiply(ns0, ni2, ni3), api.multiply(ns1, ni0, ni1), api.multiply(ns2, ni0, ni3)
        ns = api.summate(np4, np5, np6, num_node_blocks=1, block_size=1)
    return ns, dict(layer_sparsity_tol=0.1)


def simple_model_bs1(api):
    return simple_model(api, block_size=1)


def simple_model_bs4(api):
    return simple_model(api, block_size=4)


def sparse_sum(api):
    """A sum layer with explicit, uneven block edges (several forward and backward partitions)."""
    with api.set_block_size(8):
        ni = [api.inputs(v, num_node_blocks=4, dist=api.cat(5)) for v in range(4)]
        np0 = api.multiply(ni[0], ni[1])
        np1 = api.multiply(ni[0], ni[1], edge_ids=torch.tensor([[0, 1], [1, 2], [2, 3], [3, 0], [0, 0], [3, 3]]))
        e = torch.tensor([[0, 0, 0, 0, 0, 0, 1, 1, 2, 2, 2, 3, 4, 4, 4, 4, 4, 4, 4, 4, 4],
                          [0, 1, 2, 3, 4, 5, 1, 9, 0, 5, 7, 6, 0, 1, 2, 3, 4, 5, 6, 8, 9]])
        ns0 = api.summate(np0, np1, num_node_blocks=5, edge_ids=e)
        np2 = api.multiply(ni[2], ni[3])
        ns1 = api.summate(np2, num_node_blocks=5)
        np3 = api.multiply(ns0, ns1)
        ns = api.summate(np3, num_node_blocks=1, block_size=1)
    return ns, dict(layer_sparsity_tol=0.1, max_num_partitions=4)


def passthrough(api):
    """A sum vector with children of different depth: the compiler splices in an identity sum/product pair."""
    with api.set_block_size(4):
        ni = [api.inputs(v, num_node_blocks=2, dist=api.cat(3)) for v in range(3)]
        s01 = api.summate(api.multiply(ni[0], ni[1]), num_node_blocks=2)
        deep = api.multiply(s01, ni[2])
        shallow = api.multiply(ni[0], ni[1], ni[2])
        mid = api.summate(deep, shallow, num_node_blocks=2)
        ns = api.summate(api.multiply(mid), num_node_blocks=1, block_size=1)
    return ns, dict()


def tied_sums(api):
    """Tied sum vectors spread over layers with a small accumulator capacity (several flow accumulators)."""
    with api.set_block_size(4):
        ni = [api.inputs(v, num_node_blocks=2, dist=api.cat(4)) for v in range(6)]
        leaves = [api.summate(api.multiply(ni[v]), num_node_blocks=2) for v in range(6)]
        src = api.summate(api.multiply(leaves[0], leaves[1]), num_node_blocks=2)
        dup1 = src.duplicate(api.multiply(leaves[2], leaves[3]), tie_params=True)
        dup2 = src.duplicate(api.multiply(leaves[4], leaves[5]), tie_params=True)
        top_src = api.summate(api.multiply(src, dup1), num_node_blocks=2)
        ns = api.summate(api.multiply(top_src, dup2), num_node_blocks=1, block_size=1)
    return ns, dict(max_tied_ns_per_parflow_block=1)


def hmm_small(api):
    return api.hmm(seq_length=8, num_latents=16, num_emits=20, homogeneous=True), dict()


def hmm_blocks(api):
    """Homogeneous HMM with several node blocks and accumulator capacity 2 (replicated flow ranges)."""
    return (api.hmm(seq_length=7, num_latents=32, num_emits=12, homogeneous=True, block_size=8),
            dict(max_tied_ns_per_parflow_block=2))


def hmm_inhomogeneous(api):
    return api.hmm(seq_length=5, num_latents=8, num_emits=6, homogeneous=False), dict()


# ---- scaled-down benchmark configurations -------------------------------------------------------------

def _grid_tree(h, w, seed):
    from pyjuice_b200.structures import random_grid_spanning_tree
    t = random_grid_spanning_tree(h, w, np.random.default_rng(seed))
    return t.edges, h * w


def hclt_grid(api):
    """Hidden tree over a random spanning tree of a 5x5 grid, 4 node blocks of 8 (cfg1 in small)."""
    edges, n = _grid_tree(5, 5, 1)
    from pyjuice_b200.structures import Tree
    root = Tree(n, edges).center()
    return api.hclt_from_tree(edges, n, root, num_latents=32, num_cats=16, block_size=8), dict()


def hclt_cfg0(api):
    """configs[0]: HCLT over 32 variables with 4 categories, 8 latents, tree learnt from the seeded samples."""
    from pyjuice_b200.data import tree_bn_samples
    x = torch.from_numpy(tree_bn_samples(num_samples=4096, num_vars=32, num_cats=4, seed=0))
    return api.hclt_from_data(x, num_latents=8, num_cats=4), dict()


def hclt_b128(api):
    """Hidden tree with 128-node blocks (the tile shape of the tensor-core kernels), two blocks per vector."""
    edges, n = _grid_tree(3, 4, 5)
    from pyjuice_b200.structures import Tree
    root = Tree(n, edges).center()
    return api.hclt_from_tree(edges, n, root, num_latents=256, num_cats=12, block_size=128), dict()


def hmm_b128(api):
    """Homogeneous HMM with 256 states in blocks of 128 (dense 256 x 256 tied transitions)."""
    return api.hmm(seq_length=6, num_latents=256, num_emits=40, homogeneous=True, block_size=128), dict()


def pd_small(api):
    """Poon-Domingos over an 8x8 grid with two scales of splits (random block connections included)."""
    _seed(2)
    pts = sorted(set(range(2, 8, 2)) | set(range(4, 8, 4)))
    return api.pd((8, 8), 32, 16, split_points=[pts, pts], block_size=8), dict()


def pd_parentless(api):
    """Poon-Domingos over an 8x8 grid, 2 node blocks of 8 per region: block-sparse sum vectors leave some product
    blocks without any sum parent (the case in which the reference's backward pass hands stale element flows down)."""
    _seed(0)
    return api.pd((8, 8), 16, 4, split_points=[[2, 4, 6], [2, 4, 6]], block_size=8), dict()


def rat_small(api):
    _seed(3)
    return api.rat_spn(8, num_vars=24, num_latents=16, depth=3, num_repetitions=4, block_size=8), dict()


CASES = {
    "simple_model": simple_model,
    "simple_model_bs1": simple_model_bs1,
    "simple_model_bs4": simple_model_bs4,
    "sparse_sum": sparse_sum,
    "passthrough": passthrough,
    "tied_sums": tied_sums,
    "hmm_small": hmm_small,
    "hmm_blocks": hmm_blocks,
    "hmm_inhomogeneous": hmm_inhomogeneous,
    "hclt_grid": hclt_grid,
    "hclt_cfg0": hclt_cfg0,
    "hclt_b128": hclt_b128,
    "hmm_b128": hmm_b128,
    "pd_small": pd_small,
    "pd_parentless": pd_parentless,
    "rat_small": rat_small,
}


def data_for(pc, B, seed=0):
    """Seeded categorical inputs ``[B, num_vars]`` (int64) within every variable's category count; works on a circuit
    compiled by this package or by the reference (both expose ``vids``, ``metadata`` and ``s_mids``)."""
    g = torch.Generator().manual_seed(seed)
    cats = torch.zeros(pc.num_vars, dtype=torch.long)
    for layer in pc.input_layer_group:
        node_cats = layer.metadata.cpu()[layer.s_mids.cpu()].long()
        cats[layer.vids[:, 0].cpu()] = node_cats
    return (torch.rand(B, pc.num_vars, generator=g) * cats[None, :].clamp(min=1)).long()


def dump_tables(pc) -> dict:
    """Every compiled table and scalar of the parity set, flattened into name -> numpy array."""
    out = {}
    put = lambda k, v: out.__setitem__(k, np.asarray(v.detach().cpu().numpy() if isinstance(v, torch.Tensor) else v))
    for name in ("num_nodes", "num_elements", "num_edges", "num_sum_params", "num_param_flows",
                 "num_dummy_nodes", "num_dummy_eles", "num_dummy_params"):
        put(f"scalar/{name}", np.int64(getattr(pc, name)))
    put("scalar/root_range", np.asarray(pc._root_node_range, dtype=np.int64))
    for li, layer in enumerate(pc.input_layer_group):
        for name in ("vids", "s_pids", "s_pfids", "s_mids", "nids", "source_nids", "node_id2source_id", "metadata"):
            put(f"input{li}/{name}", getattr(layer, name))
        for ti, (a, b, c) in enumerate(layer.tied2source_nids):
            put(f"input{li}/tied{ti}", np.concatenate([[a, b], c.cpu().numpy()]).astype(np.int64))
        put(f"input{li}/num_tied", np.int64(len(layer.tied2source_nids)))
    for gi, group in enumerate(pc.inner_layer_groups):
        for li, layer in enumerate(group):
            names = (("nids", "cids", "u_cids", "parids") if group.is_prod()
                     else ("nids", "cids", "pids", "pfids", "chids", "parids", "parpids"))
            for name in names:
                lst = getattr(layer, f"partitioned_{name}")
                put(f"g{gi}l{li}/{name}/count", np.int64(len(lst)))
                for pi, t in enumerate(lst):
                    put(f"g{gi}l{li}/{name}/{pi}", t)
            if not group.is_prod():
                put(f"g{gi}l{li}/cs_block_sizes", np.asarray(layer.cs_block_sizes, dtype=np.int64))
    for i, t in enumerate(pc.par_update_kwargs[:6]):
        put(f"par_update/{i}", t)
    for i, (a, b, c, G, M) in enumerate(pc.parflow_fusing_kwargs):
        put(f"fusing{i}/target_pfids", a)
        put(f"fusing{i}/block_sizes", b)
        put(f"fusing{i}/child_pfids", c)
        put(f"fusing{i}/GM", np.asarray([G, M], dtype=np.int64))
    put("fusing/count", np.int64(len(pc.parflow_fusing_kwargs)))
    # per-vector write-backs, in DFS post-order
    for ni, ns in enumerate(pc.root_ns):
        if getattr(ns, "_output_ind_range", None) is not None:
            put(f"ns{ni}/out", np.asarray(ns._output_ind_range, dtype=np.int64))
        if ns.is_sum() or ns.is_input():
            for name in ("_param_range", "_param_flow_range"):
                if getattr(ns, name, None) is not None:
                    put(f"ns{ni}/{name}", np.asarray(getattr(ns, name), dtype=np.int64))
        if ns.is_sum():
            for name in ("_param_ids", "_param_flow_ids", "_inverse_param_ids"):
                if getattr(ns, name, None) is not None:
                    put(f"ns{ni}/{name}", getattr(ns, name))
    return out


def tables_digest(pc):
    """(number of arrays, SHA-256 over names, dtypes, shapes and bytes of every compiled table of the parity set)."""
    import hashlib
    tables = dump_tables(pc)
    h = hashlib.sha256()
    for key in sorted(tables):
        a = np.ascontiguousarray(tables[key])
        h.update(key.encode())
        h.update(str(a.dtype).encode())
        h.update(str(a.shape).encode())
        h.update(a.tobytes())
    return len(tables), h.hexdigest()
