"""Small tree utilities used by the structure generators (no graph library needed).

``Tree`` keeps, per vertex, its neighbours in edge-insertion order.  Traversal orders follow
the conventions PyJuice obtains from networkx on a graph built with the same edge insertion
order (structures/compilation.py:50-73 uses ``bfs_tree`` successors and
``dfs_postorder_nodes``; structures/hclt.py:54-64, 118-120 uses Kruskal's minimum spanning
tree and the first graph centre), so the generated node DAG — and hence every compiled
index table — comes out identical.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Sequence, Tuple

import numpy as np


class Tree:
    def __init__(self, num_vertices: int, edges: Iterable[Tuple[int, int]]):
        self.n = int(num_vertices)
        self.adj: Dict[int, List[int]] = {v: [] for v in range(self.n)}
        self.edges: List[Tuple[int, int]] = []
        for u, v in edges:
            u, v = int(u), int(v)
            self.adj[u].append(v)
            self.adj[v].append(u)
            self.edges.append((u, v))
        assert len(self.edges) == self.n - 1, "a tree over n vertices has n - 1 edges"

    def rooted_children(self, root: int) -> Dict[int, List[int]]:
        """Children of every vertex when the tree hangs from ``root`` (adjacency order)."""
        children = {v: [] for v in range(self.n)}
        seen = {root}
        queue = [root]
        for v in queue:
            for w in self.adj[v]:
                if w not in seen:
                    seen.add(w)
                    children[v].append(w)
                    queue.append(w)
        assert len(seen) == self.n, "graph is not connected"
        return children

    def dfs_postorder(self, root: int) -> List[int]:
        order, seen = [], {root}
        stack = [(root, iter(self.adj[root]))]
        while stack:
            v, it = stack[-1]
            advanced = False
            for w in it:
                if w not in seen:
                    seen.add(w)
                    stack.append((w, iter(self.adj[w])))
                    advanced = True
                    break
            if not advanced:
                order.append(v)
                stack.pop()
        return order

    def eccentricities(self) -> List[int]:
        ecc = []
        for s in range(self.n):
            dist = {s: 0}
            queue = [s]
            for v in queue:
                for w in self.adj[v]:
                    if w not in dist:
                        dist[w] = dist[v] + 1
                        queue.append(w)
            ecc.append(max(dist.values()))
        return ecc

    def center(self) -> int:
        """First vertex (lowest id) of minimum eccentricity."""
        ecc = self.eccentricities()
        return int(np.argmin(np.asarray(ecc)))


def minimum_spanning_tree(weights: np.ndarray) -> Tree:
    """Kruskal on the complete graph with symmetric ``weights[u, v]``.

    Candidate edges are enumerated as (u, v), u < v, in lexicographic order and sorted by
    weight with a stable sort, so ties resolve to the lexicographically first edge.
    """
    n = weights.shape[0]
    iu, iv = np.triu_indices(n, k=1)
    order = np.argsort(weights[iu, iv], kind="stable")
    parent = list(range(n))

    def find(x):
        while parent[x] != x:
            parent[x] = parent[parent[x]]
            x = parent[x]
        return x

    picked = []
    for k in order:
        u, v = int(iu[k]), int(iv[k])
        ru, rv = find(u), find(v)
        if ru != rv:
            parent[ru] = rv
            picked.append((u, v))
            if len(picked) == n - 1:
                break
    return Tree(n, picked)


def random_grid_spanning_tree(height: int, width: int, rng: np.random.Generator) -> Tree:
    """A random spanning tree of the 4-neighbour ``height x width`` grid (vertex = row * width + col):
    Kruskal over the grid edges with i.i.d. uniform weights."""
    edges = []
    for r in range(height):
        for c in range(width):
            v = r * width + c
            if c + 1 < width:
                edges.append((v, v + 1))
            if r + 1 < height:
                edges.append((v, v + width))
    w = rng.random(len(edges))
    order = np.argsort(w, kind="stable")
    n = height * width
    parent = list(range(n))

    def find(x):
        while parent[x] != x:
            parent[x] = parent[parent[x]]
            x = parent[x]
        return x

    picked = []
    for k in order:
        u, v = edges[k]
        ru, rv = find(u), find(v)
        if ru != rv:
            parent[ru] = rv
            picked.append((u, v))
    return Tree(n, picked)


def random_spanning_tree(n: int, rng: np.random.Generator) -> Tree:
    """A uniformly random labelled tree over ``n`` vertices, decoded from a random Pruefer sequence."""
    if n == 1:
        return Tree(1, [])
    if n == 2:
        return Tree(2, [(0, 1)])
    seq = rng.integers(0, n, size=n - 2)
    degree = np.ones(n, dtype=np.int64)
    for s in seq:
        degree[s] += 1
    edges = []
    import heapq
    leaves = [v for v in range(n) if degree[v] == 1]
    heapq.heapify(leaves)
    for s in seq:
        leaf = heapq.heappop(leaves)
        edges.append((int(leaf), int(s)))
        degree[s] -= 1
        if degree[s] == 1:
            heapq.heappush(leaves, int(s))
    u = heapq.heappop(leaves)
    v = heapq.heappop(leaves)
    edges.append((int(u), int(v)))
    return Tree(n, edges)
