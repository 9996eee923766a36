"""Leaf distributions.  Only ``Categorical`` is on the compiled forward/backward/EM path.

Mirrors the host-side part of PyJuice's ``Categorical``
(src/pyjuice/nodes/distributions/categorical.py:12-73): signature, metadata, parameter
counts and random initialisation.  The device math (log-prob gather, flow scatter, EM) lives
in the CUDA library, not here.
"""
from __future__ import annotations

from typing import Optional

import torch


class Distribution:
    need_meta_parameters = False

    def get_signature(self):
        raise NotImplementedError

    def get_metadata(self):
        return []

    def num_parameters(self) -> int:
        raise NotImplementedError

    def num_param_flows(self) -> int:
        raise NotImplementedError

    def requires_external_inputs(self) -> bool:
        return False


class Categorical(Distribution):
    """``num_cats``-way categorical leaf; parameters are the ``num_cats`` probabilities."""

    def __init__(self, num_cats: int):
        self.num_cats = int(num_cats)

    def get_signature(self):
        return "Categorical"

    def get_metadata(self):
        return [self.num_cats]

    def num_parameters(self) -> int:
        return self.num_cats

    def num_param_flows(self) -> int:
        return self.num_cats

    def normalize_parameters(self, params: torch.Tensor) -> torch.Tensor:
        params = params.reshape(-1, self.num_cats)
        params = params / params.sum(dim=1, keepdim=True)
        return params.reshape(-1)

    def init_parameters(self, num_nodes: int, perturbation: float = 2.0,
                        params: Optional[torch.Tensor] = None, **kwargs) -> torch.Tensor:
        # categorical.py:54-67: existing parameters are returned untouched; otherwise
        # exp(-perturbation * U[0,1)) rows, normalised.
        if params is not None:
            assert params.numel() == num_nodes * self.num_cats
            return params
        p = torch.exp(torch.rand([num_nodes, self.num_cats]) * -perturbation)
        p /= p.sum(dim=1, keepdim=True)
        return p.reshape(-1)

    def get_data_dtype(self):
        return torch.long

    def _get_constructor(self):
        return Categorical, {"num_cats": self.num_cats}
