"""A second, independent evaluator of a circuit: it walks the node DAG (not the compiled tables) in log space with
torch autograd, so the flow of every node is simply d log p(x) / d log value(node).  It shares no code with the
oracle or the compiler and is used to pin the oracle's flows (tests/test_oracle_pins.py)."""
import torch


def collect(root):
    order, seen, stack = [], set(), [root]
    while stack:
        n = stack.pop()
        if id(n) in seen:
            continue
        seen.add(id(n))
        order.append(n)
        stack += list(getattr(n, "chs", []))
    return order


def evaluate(pc, root, leaf_values):
    """``leaf_values``: {id(input vector): [num_nodes, B] log-values (requires_grad)}.  Returns the root's values and
    {id(vector): values} with gradients retained."""
    cache = {}

    def val(ns):
        k = id(ns)
        if k in cache:
            return cache[k]
        if ns.is_input():
            v = leaf_values[k]
        elif ns.is_prod():
            bs = ns.block_size
            child_vals = [val(c) for c in ns.chs]
            rows = []
            for i in range(ns.num_node_blocks):
                acc = 0
                for c, cv in enumerate(child_vals):
                    b = int(ns.edge_ids[i, c])
                    acc = acc + cv[b * bs:(b + 1) * bs]
                rows.append(acc)
            v = torch.cat(rows, 0)
        else:
            cbs = ns.ch_block_size
            cat = torch.cat([val(c) for c in ns.chs], 0)
            src = ns.get_source_ns() if ns.is_tied() else ns      # tied vectors read their source's parameters
            P = pc.get_node_params(src).double()                   # [edges, block_size, ch_block_size]
            e = ns.edge_ids
            rows = []
            for i in range(ns.num_node_blocks):
                terms = [torch.log(P[k])[:, :, None] + cat[int(e[1, k]) * cbs:(int(e[1, k]) + 1) * cbs][None, :, :]
                         for k in torch.nonzero(e[0] == i)[:, 0].tolist()]
                rows.append(torch.logsumexp(torch.cat(terms, 1), dim=1))
            v = torch.cat(rows, 0)
        if v.requires_grad and not v.is_leaf:
            v.retain_grad()
        cache[k] = v
        return v

    return val(root), cache


def true_flows(pc, root, node_mars):
    """Log-likelihoods and {id(vector): flows} of all input and sum vectors, leaves taken from ``node_mars``."""
    order = collect(root)
    leaves = {}
    for n in order:
        if n.is_input():
            s, e = n._output_ind_range
            leaves[id(n)] = node_mars[s:e].clone().double().requires_grad_(True)
    out, cache = evaluate(pc, root, leaves)
    out.sum().backward()
    flows = {id(n): cache[id(n)].grad for n in order if not n.is_prod() and cache[id(n)].grad is not None}
    return out.detach(), flows, order
