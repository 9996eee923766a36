"""Hidden Chow-Liu tree circuits.

``tree_to_hidden_circuit`` turns a tree Bayesian network over the observed variables into the
circuit of the latent-tree model in which every variable ``x_v`` hangs off a latent ``z_v`` with
``num_latents`` states (PyJuice: structures/compilation.py:12-107).  ``HCLT`` first estimates
the tree from data by pairwise mutual information and a maximum spanning tree
(structures/hclt.py:13-132).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..nodes import Categorical, inputs, multiply, summate, set_block_size
from .trees import Tree, minimum_spanning_tree


def max_cdf_power_of_2(val: int) -> int:
    """Largest power of two dividing ``val`` (utils/util.py:6-18)."""
    return val & (-val)


def tree_to_hidden_circuit(tree: Tree, root: int, num_latents: int, num_cats: int, num_root_ns: int = 1,
                           block_size: Optional[int] = None, tie_input_params: bool = False):
    if block_size is None:
        block_size = min(1024, max_cdf_power_of_2(num_latents))
    num_node_blocks = num_latents // block_size
    children = tree.rooted_children(root)

    template = None

    def leaf(v):
        nonlocal template
        if not tie_input_params:
            return inputs(v, num_node_blocks=num_node_blocks, dist=Categorical(num_cats=num_cats))
        if template is None:
            template = inputs(v, num_node_blocks=num_node_blocks, dist=Categorical(num_cats=num_cats))
            return template
        return template.duplicate(v, tie_params=True)

    var2ns = {}
    with set_block_size(block_size):
        for v in tree.dfs_postorder(root):
            chs = children[v]
            if len(chs) == 0:
                var2ns[v] = leaf(v)
                continue
            prod = multiply(*[var2ns[c] for c in chs], leaf(v))
            if v == root:
                if num_root_ns == 1:
                    var2ns[v] = summate(prod, num_node_blocks=1, block_size=1)
                else:
                    var2ns[v] = summate(prod, num_node_blocks=num_root_ns // block_size, block_size=block_size)
            else:
                var2ns[v] = summate(prod, num_node_blocks=num_node_blocks)
    return var2ns[root]


def mutual_information(x1: torch.Tensor, x2: torch.Tensor, num_bins: int, sigma: float) -> torch.Tensor:
    """Soft-binned pairwise mutual information between the columns of ``x1`` and ``x2``
    (Gaussian kernel of width ``sigma`` around ``num_bins`` centres on [0, 1])."""
    B, K1 = x1.shape
    K2 = x2.size(1)
    x1 = (x1 - x1.min()) / (x1.max() - x1.min() + 1e-8)
    x2 = (x2 - x2.min()) / (x2.max() - x2.min() + 1e-8)
    bins = torch.linspace(0, 1, num_bins, device=x1.device)
    p1 = torch.exp(-0.5 * (x1.unsqueeze(2) - bins.view(1, 1, -1)).pow(2) / sigma ** 2)
    p2 = torch.exp(-0.5 * (x2.unsqueeze(2) - bins.view(1, 1, -1)).pow(2) / sigma ** 2)
    joint = torch.einsum("bia,baj->ij", p1.reshape(B, K1 * num_bins, 1), p2.reshape(B, 1, K2 * num_bins))
    joint = joint.reshape(K1, num_bins, K2, num_bins) / B
    m1 = (p1 / p1.sum(dim=2, keepdim=True)).mean(dim=0)
    m2 = (p2 / p2.sum(dim=2, keepdim=True)).mean(dim=0)
    joint = joint / joint.sum(dim=(1, 3), keepdim=True)
    h1 = -(m1 * torch.log(m1 + 1e-4)).sum(dim=1)
    h2 = -(m2 * torch.log(m2 + 1e-4)).sum(dim=1)
    h12 = -(joint * torch.log(joint + 1e-4)).sum(dim=(1, 3))
    return h1.unsqueeze(1) + h2.unsqueeze(0) - h12


def mutual_information_chunked(x: torch.Tensor, num_bins: int, sigma: float, chunk_size: int) -> torch.Tensor:
    K = x.size(1)
    mi = torch.zeros([K, K])
    for xs in range(0, K, chunk_size):
        xe = min(xs + chunk_size, K)
        for ys in range(0, K, chunk_size):
            ye = min(ys + chunk_size, K)
            mi[xs:xe, ys:ye] = mutual_information(x[:, xs:xe], x[:, ys:ye], num_bins, sigma)
    return mi


def chow_liu_tree(mi: np.ndarray) -> Tree:
    return minimum_spanning_tree(-np.asarray(mi, dtype=np.float64))


def HCLT(x: torch.Tensor, num_latents: int, num_bins: int = 32, sigma: float = 0.5 / 32, chunk_size: int = 64,
         num_root_ns: int = 1, block_size: Optional[int] = None, num_cats: int = 256,
         tie_input_params: bool = False, tree: Optional[Tree] = None, root: Optional[int] = None):
    """Hidden Chow-Liu tree over the columns of ``x`` (``[num_samples, num_vars]``, float).

    ``tree`` (and optionally ``root``) bypasses the data-driven structure search and uses the given
    backbone instead.
    """
    if tree is None:
        mi = mutual_information_chunked(x.float(), num_bins, sigma, chunk_size).detach().cpu().numpy()
        tree = chow_liu_tree(mi)
    if root is None:
        root = tree.center()
    return tree_to_hidden_circuit(tree, root, num_latents, num_cats, num_root_ns=num_root_ns,
                                  block_size=block_size, tie_input_params=tie_input_params)
