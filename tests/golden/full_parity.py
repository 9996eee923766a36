"""Measures, on a GPU box, how far this package's CUDA path is from the REFERENCE's own GPU path on the five
benchmark configurations at full circuit size, and writes the figures to a JSON file.

    python tests/golden/full_parity.py <dir that holds the installed `pyjuice` package> [--out FILE] [--configs cfg1,cfg3]

For every configuration both implementations compile the same seeded node DAG (built through the reference's own
structure generators and through this package's), the reference's compiled parameters are copied into this
package's circuit, and one forward + backward + mini-batch-EM step (step 0.1, pseudocount 0.1) runs on the same
batch.  Recorded per configuration: worst |LL difference| in nats, worst relative difference of node flows,
sum-layer parameter flows, input-layer parameter flows (tied accumulators summed) and post-EM parameters, for the
reference at ``force_use_fp32=True`` and at its default precision, and the same figures against the fp64 CPU
oracle where the oracle is fast enough.  The reference runs its Triton kernels only (see make_values.py).
"""
import argparse
import json
import os
import sys
import time

os.environ.setdefault("PYJUICE_DISABLE_CUDA_KERNELS", "1")
os.environ.setdefault("PYJUICE_DISABLE_DIST_CUDA_KERNELS", "1")
os.environ.setdefault("PYJUICE_AUTOTUNE", "0")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.join(HERE, "..", "..")
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(ROOT, "tests"))

BATCH = {"cfg0": 256, "cfg1": 64, "cfg2": 32, "cfg3": 64, "cfg4": 64}


def rel_err(got, ref, floor=1e-6):
    got, ref = got.double(), ref.double().to(got.device)
    scale = max(ref.abs().max().item(), 1e-30)
    return ((got - ref).abs() / torch.clamp(ref.abs(), min=floor * scale)).max().item()


def folded_input_flows(layer, flows):
    """Input-layer flows with every tied group's accumulators summed into its source range (replicas dropped)."""
    f = flows.detach().clone().double()
    for start, n, ch in layer.tied2source_nids:
        start, n = int(start), int(n)
        tot = sum(f[int(c):int(c) + n].clone() for c in ch)
        for c in ch:
            f[int(c):int(c) + n] = 0.0
        f[start:start + n] = tot
    return f


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("pkg_dir")
    ap.add_argument("--out", default=os.path.join(HERE, "full_parity.json"))
    ap.add_argument("--configs", default="cfg0,cfg1,cfg2,cfg3,cfg4")
    ap.add_argument("--compat", action="store_true", help="run this package with `reference_compat = True`")
    args = ap.parse_args()
    from make_values import load_reference
    juice = load_reference(args.pkg_dir)
    import bench
    import pyjuice_b200 as pj
    dev = torch.device("cuda:0")
    results = {}
    for cfg in args.configs.split(","):
        B = BATCH[cfg]
        t0 = time.time()
        ns_ref, x = bench.build_workload(cfg, B, lib=bench.ReferenceStructures(juice))
        ref = juice.compile(ns_ref, verbose=False)
        ref.to(dev)
        ns, _ = bench.build_workload(cfg, B)
        pc = pj.compile(ns).to(dev)
        pc.reference_compat = bool(args.compat)
        assert pc.num_nodes == ref.num_nodes and pc.num_sum_params == ref.num_sum_params
        p0 = ref.params.detach().clone()
        ip0 = [l.params.detach().clone() for l in ref.input_layer_group]
        xd = torch.from_numpy(x).to(dev)
        rec = {"batch": B, "parentless_product_groups": len(pc._parentless)}
        for label, kw in (("fp32", {"force_use_fp32": True}), ("default", {})):
            ref.params.data.copy_(p0)
            for l, p in zip(ref.input_layer_group, ip0):
                l.params.data.copy_(p)
            pc.params.data.copy_(p0)
            pc._packer.invalidate()
            for l, p in zip(pc.input_layer_group, ip0):
                l.params.data.copy_(p)
            ref.init_param_flows(flows_memory=0.0)
            with torch.no_grad():
                lls_ref = ref(xd, **kw)
            ref.backward(xd, flows_memory=1.0, **kw)
            pc.init_param_flows(flows_memory=0.0)
            lls = pc(xd)
            pc.backward(xd)
            torch.cuda.synchronize()
            r = {"ll_abs": (lls.double() - lls_ref.double()).abs().max().item(), "ll_magnitude": lls_ref.abs().max().item(),
                 "node_flows_rel": rel_err(pc.node_flows[pc.num_dummy_nodes:].exp(), ref.node_flows[pc.num_dummy_nodes:].exp()),
                 "param_flows_rel": rel_err(pc.param_flows, ref.param_flows),
                 "input_flows_rel": max(rel_err(folded_input_flows(a, a.param_flows), folded_input_flows(b, b.param_flows))
                                        for a, b in zip(pc.input_layer_group, ref.input_layer_group))}
            ref.mini_batch_em(step_size=0.1, pseudocount=0.1)
            pc.mini_batch_em(step_size=0.1, pseudocount=0.1)
            torch.cuda.synchronize()
            r["params_rel"] = rel_err(pc.params.data[pc.num_dummy_params:], ref.params.data[pc.num_dummy_params:])
            r["input_params_rel"] = max(rel_err(a.params.data, b.params.data)
                                        for a, b in zip(pc.input_layer_group, ref.input_layer_group))
            rec["vs_reference_" + label] = r
        rec["seconds"] = round(time.time() - t0, 1)
        results[cfg] = rec
        print(cfg, json.dumps(rec), flush=True)
        del ref, pc
        torch.cuda.empty_cache()
    with open(args.out, "w") as f:
        json.dump(results, f, indent=1, sort_keys=True)


if __name__ == "__main__":
    main()
