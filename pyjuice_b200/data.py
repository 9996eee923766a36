"""Seeded synthetic data sets with the shapes and value distributions of the five benchmark configurations.

They stand in for the image / text corpora the reference's training tests download: integer matrices
``[num_samples, num_vars]`` (int64) drawn from small generative models, so that circuits see structured
rather than uniform data.  Everything is NumPy on the host and a function of the seed only.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np

from .structures.trees import Tree, random_grid_spanning_tree, random_spanning_tree


def _sample_rows(cdf: np.ndarray, row: np.ndarray, u: np.ndarray) -> np.ndarray:
    """For every i draw a category from the distribution whose CDF is ``cdf[row[i]]`` using the uniform
    ``u[i]``: one binary search over the row-offset, flattened CDF table."""
    R, C = cdf.shape
    flat = (cdf + np.arange(R)[:, None]).reshape(-1)
    flat[C - 1::C] = np.arange(1, R + 1)                     # each row ends exactly at row + 1
    pos = np.searchsorted(flat, row + u, side="right")
    return np.minimum(pos - row * C, C - 1).astype(np.int64)


def _ancestral(tree: Tree, root: int, root_cdf: np.ndarray, cpt_cdf_of, num_samples: int, rng) -> np.ndarray:
    children = tree.rooted_children(root)
    x = np.zeros((num_samples, tree.n), dtype=np.int64)
    x[:, root] = _sample_rows(root_cdf[None, :], np.zeros(num_samples, dtype=np.int64), rng.random(num_samples))
    queue = [root]
    for v in queue:
        for c in children[v]:
            x[:, c] = _sample_rows(cpt_cdf_of(c), x[:, v], rng.random(num_samples))
            queue.append(c)
    return x


def tree_bn_samples(num_samples: int, num_vars: int, num_cats: int, seed: int, alpha: float = 0.5,
                    return_tree: bool = False):
    """Samples of a random tree-structured Bayesian network: uniform random labelled tree, root marginal and
    every conditional row ~ Dirichlet(alpha)."""
    rng = np.random.default_rng(seed)
    tree = random_spanning_tree(num_vars, rng)
    root_cdf = np.cumsum(rng.dirichlet(np.full(num_cats, alpha)))
    cpts = {v: np.cumsum(rng.dirichlet(np.full(num_cats, alpha), size=num_cats), axis=1) for v in range(num_vars)}
    x = _ancestral(tree, 0, root_cdf, lambda v: cpts[v], num_samples, rng)
    return (x, tree) if return_tree else x


def _disc_gaussian_rows(centres: np.ndarray, sigma: float, num_cats: int) -> np.ndarray:
    k = np.arange(num_cats)[None, :]
    p = np.exp(-0.5 * ((k - centres[:, None]) / sigma) ** 2) + 1e-12
    return p / p.sum(axis=1, keepdims=True)


def grid_gaussian_bn_samples(num_samples: int, height: int, width: int, seed: int, num_cats: int = 256,
                             shift_std: float = 20.0, sigma: float = 25.0) -> Tuple[np.ndarray, Tree, int]:
    """Samples of a tree Bayesian network over a ``height x width`` grid of ``num_cats``-valued variables.

    The tree is a random spanning tree of the 4-neighbour grid.  Variable ``v`` with parent value ``p`` follows a
    discretised Gaussian over ``0..num_cats-1`` centred at ``p + d_v`` with standard deviation ``sigma``, where the
    per-variable shift ``d_v ~ N(0, shift_std)``.  The root is a discretised Gaussian centred mid-range with
    standard deviation ``num_cats / 4``.  Returns ``(x, tree, root)``."""
    rng = np.random.default_rng(seed)
    tree = random_grid_spanning_tree(height, width, rng)
    root = tree.center()
    shifts = rng.normal(0.0, shift_std, size=tree.n)
    root_cdf = np.cumsum(_disc_gaussian_rows(np.array([num_cats / 2.0]), num_cats / 4.0, num_cats)[0])
    parents = np.arange(num_cats, dtype=np.float64)

    def cpt_cdf(v):
        return np.cumsum(_disc_gaussian_rows(parents + shifts[v], sigma, num_cats), axis=1)

    return _ancestral(tree, root, root_cdf, cpt_cdf, num_samples, rng), tree, root


def mixture_samples(num_samples: int, num_vars: int, num_cats: int, seed: int, num_components: int = 10,
                    alpha: float = 0.3) -> np.ndarray:
    """I.i.d. samples of a uniform mixture of ``num_components`` products of categoricals; every component's
    per-variable distribution ~ Dirichlet(alpha)."""
    rng = np.random.default_rng(seed)
    z = rng.integers(0, num_components, size=num_samples)
    x = np.zeros((num_samples, num_vars), dtype=np.int64)
    for v in range(num_vars):
        cdf = np.cumsum(rng.dirichlet(np.full(num_cats, alpha), size=num_components), axis=1)
        x[:, v] = _sample_rows(cdf, z, rng.random(num_samples))
    return x


def hmm_samples(num_samples: int, seq_length: int, vocab: int, seed: int, num_states: int = 256,
                trans_alpha: float = 0.05, emit_alpha: float = 0.01) -> np.ndarray:
    """Token sequences from a ground-truth HMM: transition rows ~ Dirichlet(trans_alpha), emission rows ~
    Dirichlet(emit_alpha), uniform initial state."""
    rng = np.random.default_rng(seed)
    trans = np.cumsum(rng.dirichlet(np.full(num_states, trans_alpha), size=num_states), axis=1)
    g = rng.standard_gamma(emit_alpha, size=(num_states, vocab)) + 1e-300
    emit = np.cumsum(g / g.sum(axis=1, keepdims=True), axis=1)
    z = rng.integers(0, num_states, size=num_samples)
    x = np.zeros((num_samples, seq_length), dtype=np.int64)
    for t in range(seq_length):
        x[:, t] = _sample_rows(emit, z, rng.random(num_samples))
        z = _sample_rows(trans, z, rng.random(num_samples))
    return x
