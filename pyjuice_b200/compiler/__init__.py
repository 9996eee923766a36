from .partition import partition_nodes_by_n_edges, partition_maxima, next_power_of_2
from .layering import create_node_layers
from .tables import (compile_sum_forward, compile_sum_backward, compile_prod, compile_input, reorder_input_nodes,
                     compile_par_update, compile_cum_par_flows, _IdDict)
