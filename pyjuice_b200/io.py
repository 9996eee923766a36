"""Checkpoints: ``save`` / ``load`` of a circuit as a ``.jpc`` file, in PyJuice's own record format
(src/pyjuice/io/io.py:13-51, src/pyjuice/io/serialization.py:11-126), so files move both ways between the two
engines.

A ``.jpc`` file is a pickled list with one dict per node vector, children before parents: ``type`` ("Input" /
"Product" / "Sum"), ``num_node_blocks``, ``block_size``, ``chs`` (indices into the list), ``edge_ids`` and ``params``
as NumPy arrays, ``scope`` and the pickled leaf distribution for inputs, ``source_node`` for tied vectors.  Saving a
compiled circuit first copies the trained parameters from the device back into the node vectors
(``TensorCircuit.update_parameters``).

Two things differ from a plain ``pickle.load``: leaf distributions are written under the class path PyJuice
unpickles (``pyjuice.nodes.distributions...``) and read back through an unpickler that maps that path, or this
package's, onto this package's classes; and both unpicklers refuse every global that a checkpoint has no business
naming (a ``.jpc`` file from an untrusted source cannot run code here).
"""
from __future__ import annotations

import io as _io
import pickle
from typing import Sequence, Union

import numpy as np
import torch

from .nodes import CircuitNodes, inputs, multiply, summate
from .nodes import distributions as _dists

# class name -> module the reference keeps it in (what its unpickler imports)
_REF_DIST_MODULE = {"Categorical": "pyjuice.nodes.distributions.categorical"}
# instance attributes the reference's base class sets (nodes/distributions/distributions.py:9-12)
_REF_DIST_BASE_STATE = {"post_fw_fns": [], "post_bp_fns": [], "sampling_fns": []}


def _dump_dist(dist) -> bytes:
    """Protocol-2 pickle of a leaf distribution, naming the reference's class: GLOBAL, EMPTY_TUPLE, NEWOBJ,
    <state dict>, BUILD, STOP."""
    name = type(dist).__name__
    if name not in _REF_DIST_MODULE:
        raise NotImplementedError(f"leaf distribution `{name}` has no checkpoint record")
    state = dict(_REF_DIST_BASE_STATE, **{k: v for k, v in vars(dist).items()})
    body = pickle.dumps(state, protocol=2)
    assert body[:2] == b"\x80\x02" and body[-1:] == b"."
    return (b"\x80\x02c" + _REF_DIST_MODULE[name].encode() + b"\n" + name.encode() + b"\n)\x81"
            + body[2:-1] + b"b.")


class _DistUnpickler(pickle.Unpickler):
    def find_class(self, module, name):
        if module.startswith("pyjuice.nodes.distributions") or module.startswith(_dists.__name__):
            cls = getattr(_dists, name, None)
            if isinstance(cls, type) and issubclass(cls, _dists.Distribution):
                return cls
            raise NotImplementedError(f"leaf distribution `{name}` is not on the compiled path")
        raise pickle.UnpicklingError(f"a leaf-distribution record names `{module}.{name}`")


def _load_dist(blob: bytes):
    return _DistUnpickler(_io.BytesIO(blob)).load()


class _RecordUnpickler(pickle.Unpickler):
    """Node records hold ints, strings, tuples, bytes and NumPy arrays: only NumPy's own reconstruction helpers may
    be named."""
    _ALLOWED = {("numpy", "dtype"), ("numpy", "ndarray"),
                ("numpy.core.multiarray", "_reconstruct"), ("numpy._core.multiarray", "_reconstruct"),
                ("numpy.core.multiarray", "scalar"), ("numpy._core.multiarray", "scalar"),
                ("numpy.core.numeric", "_frombuffer"), ("numpy._core.numeric", "_frombuffer")}

    def find_class(self, module, name):
        if (module, name) in self._ALLOWED:
            return super().find_class(module, name)
        raise pickle.UnpicklingError(f"a node record names `{module}.{name}`")


def serialize_nodes(root_ns: CircuitNodes):
    """One record per node vector, children first (io/serialization.py:11-54)."""
    records, index = [], {}
    for ns in root_ns:
        rec = {"type": "Input" if ns.is_input() else ("Product" if ns.is_prod() else "Sum"),
               "num_node_blocks": ns.num_node_blocks, "block_size": ns.block_size,
               "chs": tuple(index[id(c)] for c in ns.chs)}
        if not ns.is_input():
            rec["edge_ids"] = ns.edge_ids.detach().cpu().numpy().copy()
        if getattr(ns, "_params", None) is not None:
            rec["params"] = ns._params.detach().cpu().numpy().copy()
        if ns.is_input():
            rec["scope"] = ns.scope.to_list()
            rec["dist"] = _dump_dist(ns.dist)
        index[id(ns)] = len(records)
        records.append(rec)
    for ns in root_ns:
        if ns.is_tied():
            records[index[id(ns)]]["source_node"] = index[id(ns._source_node)]
    return records


def deserialize_nodes(records: Sequence[dict]) -> CircuitNodes:
    """Rebuild the node DAG from its records; returns the last vector (the root).  Older files name the block
    fields ``num_node_groups`` / ``group_size`` or only ``num_nodes`` (io/serialization.py:57-126)."""
    built = {}
    for i, rec in enumerate(records):
        if "num_node_blocks" in rec:
            nb, bs = rec["num_node_blocks"], rec["block_size"]
        elif "num_node_groups" in rec:
            nb, bs = rec["num_node_groups"], rec["group_size"]
        else:
            nb, bs = rec["num_nodes"], 1
        for key in ("external_params", "zero_param_mask"):
            if rec.get(key) is not None:
                raise NotImplementedError(f"`{key}` records are not on the compiled path")
        chs = [built[c] for c in rec["chs"]]
        if rec["type"] == "Input":
            ns = inputs(rec["scope"], nb, _load_dist(rec["dist"]), block_size=bs)
            if "params" in rec:
                ns.set_params(torch.from_numpy(np.array(rec["params"])), normalize=False)
        elif rec["type"] == "Product":
            edge_ids = torch.from_numpy(np.array(rec["edge_ids"]))
            ns = multiply(*chs, edge_ids=edge_ids, sparse_edges=edge_ids.size(0) != chs[0].num_node_blocks)
        else:
            assert rec["type"] == "Sum"
            ns = summate(*chs, edge_ids=torch.from_numpy(np.array(rec["edge_ids"])), block_size=bs)
            assert ns.num_node_blocks == nb
            if "params" in rec:
                ns.set_params(torch.from_numpy(np.array(rec["params"])), normalize=False)
        built[i] = ns
    for i, rec in enumerate(records):
        if "source_node" in rec:
            built[i]._source_node = built[rec["source_node"]]
    return built[len(records) - 1]


def save(fname: str, model: Union[CircuitNodes, "TensorCircuit"]):
    """Write an uncompiled (node DAG) or compiled circuit to ``fname`` (must end with ``.jpc``)."""
    from .model import TensorCircuit
    if not fname.endswith(".jpc"):
        raise ValueError(f"Unknown file type `.{fname.split('.')[-1]}`.")
    if isinstance(model, TensorCircuit):
        model.update_parameters()
        root_ns = model.root_ns
    else:
        root_ns = model
    with open(fname, "wb") as f:
        pickle.dump(serialize_nodes(root_ns), f)


def load(fname: str) -> CircuitNodes:
    """Read a ``.jpc`` file written by this package or by PyJuice; returns the root node vector."""
    if not fname.endswith(".jpc"):
        raise ValueError(f"Unknown file type `.{fname.split('.')[-1]}`.")
    with open(fname, "rb") as f:
        records = _RecordUnpickler(f).load()
    return deserialize_nodes(records)
