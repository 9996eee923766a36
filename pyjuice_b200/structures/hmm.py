"""Hidden Markov models as circuits (PyJuice: structures/hmm.py:16-91).

One input vector per position (emissions), one sum vector per transition, chained from the
last position to the first; with ``homogeneous=True`` every emission vector is tied to the
first one built and every transition vector to the first transition.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..nodes import Categorical, inputs, multiply, summate, set_block_size
from .hclt import max_cdf_power_of_2


def HMM(seq_length: int, num_latents: int, num_emits: int, homogeneous: bool = True, block_size: Optional[int] = None,
        alpha: Optional[torch.Tensor] = None, beta: Optional[torch.Tensor] = None, gamma: Optional[torch.Tensor] = None):
    """``alpha`` ``[L, L]`` transitions, ``beta`` ``[L, num_emits]`` emissions, ``gamma`` ``[L]`` initial."""
    if block_size is None:
        block_size = min(max_cdf_power_of_2(num_latents), 1024)
    num_node_blocks = num_latents // block_size

    with set_block_size(block_size):
        ns_input = inputs(seq_length - 1, num_node_blocks=num_node_blocks, dist=Categorical(num_cats=num_emits))
        if beta is not None:
            assert beta.shape == (num_latents, num_emits)
            ns_input.set_params(beta)

        ns_sum = None
        curr_zs = ns_input
        for var in range(seq_length - 2, -1, -1):
            curr_xs = ns_input.duplicate(var, tie_params=homogeneous)
            if ns_sum is None:
                ns = summate(curr_zs, num_node_blocks=num_node_blocks)
                if alpha is not None:
                    assert alpha.shape == (num_latents, num_latents)
                    ns.set_params(alpha)
                ns_sum = ns
            else:
                ns = ns_sum.duplicate(curr_zs, tie_params=homogeneous)
            curr_zs = multiply(curr_xs, ns)

        ns = summate(curr_zs, num_node_blocks=1, block_size=1)
        if gamma is not None:
            assert gamma.dim() == 1 and gamma.size(0) == num_latents
            ns.set_params(gamma.unsqueeze(0))
    return ns
