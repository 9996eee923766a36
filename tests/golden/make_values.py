"""Generates ``tests/golden/values_<case>.npz``: what the REFERENCE itself computes on a GPU for the cases of
``cases.py`` — per-sample log-likelihoods, node values, node flows, parameter flows of the sum layers and of the
input layers, and the parameters after one mini-batch EM step.

    python tests/golden/make_values.py <dir that holds the installed `pyjuice` package> [--out DIR] [--cases a,b]

It needs a CUDA device: the reference's leaf and product layers exist as Triton kernels only.  The reference runs
unmodified through its public API (``compile``, ``pc(x)``, ``pc.backward``, ``pc.mini_batch_em``) on its Triton
path: its optional CuTe kernels are switched off with the reference's own environment switches
(``PYJUICE_DISABLE_CUDA_KERNELS=1``; their barrier waits are unbounded, layer/kernels/c/tlmm_forward_sum.cu:55-61)
and so is autotuning (``PYJUICE_AUTOTUNE=0``).  Two precisions are recorded: ``force_use_fp32=True`` (the parity
target; note that the reference's Triton kernels multiply fp32 operands in TF32 even then, ``tl.dot``'s default) and
the reference's default precision (bf16 forward), of which only the log-likelihoods (``lls_default``) and the
worst relative differences of flows and parameters (``default_dev``) are kept, so the fixtures also tell how far the
reference is from itself.

Protocol shared with the parity tests: seed, build the node DAG, ``init_parameters()`` on it, compile; the
compiled parameter vectors and the inputs are stored in the fixture, so nothing depends on random-number streams
lining up between the two implementations.
"""
import argparse
import os
import sys
import types

os.environ.setdefault("PYJUICE_DISABLE_CUDA_KERNELS", "1")
os.environ.setdefault("PYJUICE_DISABLE_DIST_CUDA_KERNELS", "1")
os.environ.setdefault("PYJUICE_AUTOTUNE", "0")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, HERE)

STEP_SIZE, PSEUDOCOUNT = 0.1, 0.1
# The rescaled update (`step_size_rescaling=True`) is recorded for these cases only: on `sparse_sum` the reference's
# own top-down pass made an illegal memory access on a B200 (the CUDA context is lost after it), so it is not run
# again there, nor on the cases after it that were never reached.
RESCALED_CASES = ("hclt_cfg0", "simple_model", "simple_model_bs1", "simple_model_bs4")
# case -> (seed, batch)
VALUE_CASES = {
    "hclt_cfg0": (0, 256), "simple_model": (0, 64), "simple_model_bs1": (0, 33), "simple_model_bs4": (0, 64),
    "sparse_sum": (0, 64), "passthrough": (0, 64), "tied_sums": (0, 64), "hmm_small": (0, 64), "hmm_blocks": (0, 64),
    "hmm_inhomogeneous": (0, 64), "hclt_grid": (0, 32), "hclt_b128": (0, 16), "hmm_b128": (0, 16), "pd_small": (0, 8),
    "pd_parentless": (0, 32), "rat_small": (0, 32),
}


def load_reference(pkg_dir):
    for name in ("matplotlib", "matplotlib.pyplot", "matplotlib.patches"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.path.insert(0, pkg_dir)
    import pyjuice
    return pyjuice


def run_case(api, name, seed, B, dev):
    from cases import CASES, data_for
    torch.manual_seed(seed)
    ns, kw = CASES[name](api)
    ns.init_parameters()
    pc = api.compile(ns, **kw)
    pc.to(dev)
    x = data_for(pc, B, seed=seed)
    xd = x.to(dev)
    out = {"x": x.numpy(), "params0": pc.params.detach().cpu().numpy(),
           "step_size": np.float64(STEP_SIZE), "pseudocount": np.float64(PSEUDOCOUNT)}
    for i, layer in enumerate(pc.input_layer_group):
        out[f"iparams0_{i}"] = layer.params.detach().cpu().numpy()
    p0 = pc.params.detach().clone()
    ip0 = [layer.params.detach().clone() for layer in pc.input_layer_group]
    for suffix, fp32 in (("", True), ("_default", False)):
        pc.params.data.copy_(p0)
        for layer, p in zip(pc.input_layer_group, ip0):
            layer.params.data.copy_(p)
        pc.init_param_flows(flows_memory=0.0)
        with torch.no_grad():
            lls = pc(xd, force_use_fp32=fp32)
        pc.backward(xd, flows_memory=1.0, force_use_fp32=fp32)
        torch.cuda.synchronize()
        out["lls" + suffix] = lls.detach().cpu().numpy()
        cur = {"param_flows": pc.param_flows.detach().cpu().numpy()}
        for i, layer in enumerate(pc.input_layer_group):
            cur[f"iparam_flows_{i}"] = layer.param_flows.detach().cpu().numpy()
        if fp32:
            out["node_mars"] = pc.node_mars.detach().cpu().numpy()
            out["node_flows"] = pc.node_flows.detach().cpu().numpy()
        pc.mini_batch_em(step_size=STEP_SIZE, pseudocount=PSEUDOCOUNT)
        torch.cuda.synchronize()
        cur["params1"] = pc.params.detach().cpu().numpy()
        for i, layer in enumerate(pc.input_layer_group):
            cur[f"iparams1_{i}"] = layer.params.detach().cpu().numpy()
        if fp32:
            out.update(cur)
        else:                       # worst |default - fp32| / max(|fp32|, 1e-6 * max|fp32|) per quantity
            dev = []
            for k, v in cur.items():
                ref = out[k].astype(np.float64)
                floor = 1e-6 * max(np.abs(ref).max(), 1e-30)
                dev.append(float((np.abs(v - ref) / np.maximum(np.abs(ref), floor)).max()))
            out["default_dev"] = np.asarray(dev)
    if name not in RESCALED_CASES:
        return out
    # the rescaled update (model/tensorcircuit.py:1363-1375): flows * step / total + (1 - step) * top-down flows
    pc.params.data.copy_(p0)
    for layer, p in zip(pc.input_layer_group, ip0):
        layer.params.data.copy_(p)
    pc.init_param_flows(flows_memory=0.0)
    pc._cum_flow = 0.0
    with torch.no_grad():
        pc(xd, force_use_fp32=True)
    pc.backward(xd, flows_memory=1.0, force_use_fp32=True)
    pc.mini_batch_em(step_size=0.25, pseudocount=PSEUDOCOUNT, step_size_rescaling=True)
    torch.cuda.synchronize()
    out["params1_rescaled"] = pc.params.detach().cpu().numpy()
    for i, layer in enumerate(pc.input_layer_group):
        out[f"iparams1_rescaled_{i}"] = layer.params.detach().cpu().numpy()
    # the other propagation rules (model/tensorcircuit.py:322-347, 485-509): values and flows from the initial parameters
    pc.params.data.copy_(p0)
    for layer, p in zip(pc.input_layer_group, ip0):
        layer.params.data.copy_(p)
    for tag, kw in (("mpe", dict(propagation_alg="MPE")), ("gll2", dict(propagation_alg="GeneralLL", alpha=2.0))):
        pc.init_param_flows(flows_memory=0.0)
        with torch.no_grad():
            lls = pc(xd, force_use_fp32=True, **kw)
        # linear flows: under "MPE" the reference's log-space element-flow kernel adds log-flows within a tile
        # (layer/kernels/sum_backward_element_block_sparse.py:94), which is not a quantity to pin anything to
        pc.backward(xd, flows_memory=1.0, force_use_fp32=True, logspace_flows=False, **kw)
        torch.cuda.synchronize()
        out["lls_" + tag] = lls.detach().cpu().numpy()
        out["param_flows_" + tag] = pc.param_flows.detach().cpu().numpy()
        out["node_flows_" + tag] = pc.node_flows.detach().cpu().numpy()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("pkg_dir")
    ap.add_argument("--out", default=HERE)
    ap.add_argument("--cases", default=",".join(VALUE_CASES))
    args = ap.parse_args()
    assert torch.cuda.is_available(), "the reference's forward/backward/EM path needs a CUDA device"
    load_reference(args.pkg_dir)
    from cases import RefApi
    api = RefApi()
    os.makedirs(args.out, exist_ok=True)
    for name in args.cases.split(","):
        seed, B = VALUE_CASES[name]
        try:
            out = run_case(api, name, seed, B, torch.device("cuda:0"))
        except Exception as e:                                  # keep going: one case must not lose the others
            print(f"{name}: FAILED {type(e).__name__}: {e}", flush=True)
            continue
        np.savez_compressed(os.path.join(args.out, f"values_{name}.npz"), **out)
        d = np.abs(out["lls"] - out["lls_default"]).max()
        print(f"{name}: B={B} mean LL {out['lls'].mean():.6f}; default precision differs by {d:.2e} nats", flush=True)


if __name__ == "__main__":
    main()
