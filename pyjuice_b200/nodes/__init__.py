from .bitset import BitSet
from .distributions import Categorical, Distribution
from .nodes import CircuitNodes, InputNodes, ProdNodes, SumNodes, as_bitset, normalize_ns_parameters
from .construction import inputs, multiply, summate, set_block_size
from . import distributions
