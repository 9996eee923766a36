"""Bit-exact parity of the compiled index tables with the reference compiler's output.

``tests/golden/<case>.npz`` were produced by ``tests/golden/make_golden.py`` from the reference's own
compiler; here the same circuits are built through this package's front door and compiled by this
package's compiler, and every table, scalar and per-vector write-back must be identical.
"""
import os

import numpy as np
import pytest

from cases import CASES, OursApi, dump_tables

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", sorted(CASES))
def test_tables_match_reference(name):
    ref = np.load(os.path.join(GOLDEN, f"{name}.npz"))
    api = OursApi()
    ns, kw = CASES[name](api)
    pc = api.compile(ns, **kw)
    ours = dump_tables(pc)
    assert sorted(ours.keys()) == sorted(ref.files), (
        f"table sets differ: only ours {sorted(set(ours) - set(ref.files))[:8]}, only ref {sorted(set(ref.files) - set(ours))[:8]}")
    for key in ref.files:
        a, b = np.asarray(ours[key]), ref[key]
        assert a.shape == b.shape, f"{name}:{key} shape {a.shape} != {b.shape}"
        assert a.dtype == b.dtype, f"{name}:{key} dtype {a.dtype} != {b.dtype}"
        assert np.array_equal(a, b), f"{name}:{key} differs at {np.argwhere(a != b)[:4].tolist()}"
