"""B200-native engine for the compiled probabilistic-circuit forward / backward / mini-batch-EM path.

Front door mirrors PyJuice: ``inputs`` / ``multiply`` / ``summate`` build the node DAG, ``compile`` turns it
into a :class:`TensorCircuit`, ``optim.MiniBatchEM`` drives EM.  Computation happens in hand-written sm_100a
CUDA kernels behind the C ABI of ``include/pcx_b200.h``; there is no CPU or Triton path.
"""
from . import nodes, structures, optim
from .nodes import inputs, multiply, summate, set_block_size, Categorical, BitSet
from .nodes import distributions
from .model import TensorCircuit, compile
from .layers import InputLayer, ProdLayer, SumLayer, LayerGroup

__version__ = "0.1.0"
