from .trees import Tree, minimum_spanning_tree, random_grid_spanning_tree, random_spanning_tree
from .hclt import HCLT, tree_to_hidden_circuit, chow_liu_tree, mutual_information_chunked
from .hmm import HMM
from .pd import PD
from .rat_spn import RAT_SPN
