"""Generates ``tests/golden/<case>.npz``: the index tables the REFERENCE compiler emits for every case of
``cases.py``.  Run in a container that has the reference checkout:

    python tests/golden/make_golden.py <path to the PyJuice checkout>/src

The reference imports matplotlib (absent here) and touches CUDA in three places while compiling; both are
neutralised below, in this script only, so that its table compiler runs on the host
(``disable_gpu_compilation=True``).  Nothing else of the reference is modified, and the fixtures are plain
NumPy archives of int64 tables.
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


if __name__ == "__main__":
    sys.path.insert(0, HERE)
    main()
