"""Generates ``tests/golden/<case>.npz``: the index tables the REFERENCE compiler emits for every case of
``cases.py``.  Run in a container that has the reference checkout:

    python tests/golden/make_golden.py <path to the PyJuice checkout>/src

The reference imports matplotlib (absent here) and touches CUDA in three places while compiling; both are
neutralised below, in this script only, so that its table compiler runs on the host
(``disable_gpu_compilation=True``).  Nothing else of the reference is modified, and the fixtures are plain
NumPy archives of int64 tables.  It also writes one checkpoint with the reference's own ``save``
(``ref_hmm_blocks.jpc``) for the loader test, and, with ``--full``, ``full_tables.json``: a SHA-256 over all tables the
reference compiler emits for the benchmark configurations 1-4 at FULL size (too large to store as arrays).
"""
import contextlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
if len(sys.argv) < 2:
    sys.exit("usage: python make_golden.py <path to the PyJuice checkout>/src")
REF_SRC = sys.argv[1]


def load_reference():
    for name in ("matplotlib", "matplotlib.pyplot", "matplotlib.patches"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.path.insert(0, REF_SRC)
    torch.cuda.current_device = lambda: 0

    class _NoDevice(contextlib.AbstractContextManager):
        def __init__(self, *a, **k):
            pass

        def __exit__(self, *a):
            return False

    torch.cuda.device = _NoDevice
    import pyjuice  # noqa: F401
    import pyjuice.layer.input_layer as il
    il.InputLayer._get_num_nodes_gcd = lambda self: 1      # uses `.cuda()`; only feeds a launch heuristic
    return pyjuice


def main():
    load_reference()
    from cases import CASES, RefApi, dump_tables
    api = RefApi()
    for name, build in CASES.items():
        ns, kw = build(api)
        pc = api.compile(ns, **kw)
        tables = dump_tables(pc)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **tables)
        print(f"{name}: {len(tables)} arrays, num_nodes={pc.num_nodes}, num_edges={pc.num_edges}")
    checkpoint_fixture(api)
    if "--full" in sys.argv:
        full_size_digests()


def full_size_digests():
    import json
    import pyjuice as juice
    import bench
    from cases import tables_digest
    out = {}
    for cfg in ("cfg1", "cfg2", "cfg3", "cfg4"):
        ns, _ = bench.build_workload(cfg, 8, lib=bench.ReferenceStructures(juice))
        pc = juice.compile(ns, disable_gpu_compilation=True, verbose=False)
        n, digest = tables_digest(pc)
        out[cfg] = {"arrays": n, "sha256": digest, "num_nodes": int(pc.num_nodes), "num_edges": int(pc.num_edges)}
        print(cfg, out[cfg], flush=True)
    with open(os.path.join(HERE, "full_tables.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)


def checkpoint_fixture(api):
    """``ref_hmm_blocks.jpc``: a checkpoint written by the reference's own ``save`` (tied sums, tied leaves, random
    parameters).  The other direction is checked here, once: the reference's ``load`` reads a file this package
    wrote and finds the same vectors and parameters."""
    import tempfile
    from cases import CASES
    from pyjuice.io import load, save
    import pyjuice_b200 as ours
    torch.manual_seed(7)
    ns, _ = CASES["hmm_blocks"](api)
    ns.init_parameters()
    save(os.path.join(HERE, "ref_hmm_blocks.jpc"), ns)
    mine = ours.load(os.path.join(HERE, "ref_hmm_blocks.jpc"))
    with tempfile.TemporaryDirectory() as d:
        ours.save(os.path.join(d, "ours.jpc"), mine)
        back = load(os.path.join(d, "ours.jpc"))
    a, b = list(ns), list(back)
    assert len(a) == len(b)
    for x, y in zip(a, b):
        assert (x.num_node_blocks, x.block_size, x.is_tied()) == (y.num_node_blocks, y.block_size, y.is_tied())
        if x._params is not None:        # the reference renormalises sum parameters when it loads them
            assert torch.allclose(x._params, y._params, rtol=1e-6, atol=1e-8)
    print(f"ref_hmm_blocks.jpc: {len(a)} vectors; the reference loads this package's file")


if __name__ == "__main__":
    sys.path.insert(0, HERE)
    main()
