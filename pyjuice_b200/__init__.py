"""B200-native engine for the compiled probabilistic-circuit forward / backward / mini-batch-EM path.

Front door mirrors PyJuice: ``inputs`` / ``multiply`` / ``summate`` build the node DAG, ``compile`` turns it
into a :class:`TensorCircuit`, ``optim.MiniBatchEM`` drives EM.  Computation happens in hand-written sm_100a
CUDA kernels behind the C ABI of ``include/pcx_b200.h``; there is no CPU or Triton path.
"""
from . import nodes, structures, optim, io
from .nodes import inputs, multiply, summate, set_block_size, Categorical, BitSet
from .nodes import distributions
from .model import TensorCircuit, compile
from .io import save, load
from .layers import InputLayer, ProdLayer, SumLayer, LayerGroup

__version__ = "0.1.0"


def patch_pyjuice():
    """Point an installed PyJuice at this engine: ``pyjuice.compile``, ``pyjuice.TensorCircuit`` (also under
    ``pyjuice.model``) and ``pyjuice.optim.MiniBatchEM / FullBatchEM / CircuitOptimizer`` are rebound, so that an
    unmodified PyJuice script builds its node DAG with PyJuice and runs the compiled forward / backward / EM path here
    (``compile`` reads PyJuice's node vectors by duck typing).  Returns the patched module; raises ImportError when
    PyJuice is not importable."""
    import importlib
    pj = importlib.import_module("pyjuice")
    pj.compile, pj.TensorCircuit = compile, TensorCircuit
    model = getattr(pj, "model", None)
    if model is not None:
        model.compile, model.TensorCircuit = compile, TensorCircuit
    ref_optim = getattr(pj, "optim", None)
    if ref_optim is not None:
        for name in ("CircuitOptimizer", "MiniBatchEM", "FullBatchEM"):
            setattr(ref_optim, name, getattr(optim, name))
    return pj
