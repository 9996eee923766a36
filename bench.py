"""Benchmark of the compiled probabilistic-circuit training step (forward + backward + mini-batch EM).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config cfg4] [--others cfg1,cfg2,cfg3]
                    [--impl ours|reference|triton]

One "step" is one mini-batch of the named configuration through ``pc(x)``, ``lls.mean().backward()`` and
``MiniBatchEM.step()``.  The headline workload is configs[4] (the homogeneous HMM: the largest single-GPU
configuration and the one whose sum layers are bound by the tensor cores); the other benchmark configurations
are measured in the same run and reported under ``other_configs``.  Rank 0 prints ONE JSON line:

  value         samples/s over all ranks, inputs already resident in HBM, timed with CUDA events
  e2e           the same metric with each step's batch copied from pinned host memory inside the timed region
                and the mean log-likelihood read back to the host
  roofline      the dominant kernel family, timed per launch with CUDA events in a separate instrumented pass
  cpu_baseline  the CPU oracle (fp32, all host threads) on a bounded sample of the same workload
  other_configs {cfgN: {value, ms_per_step, e2e, roofline, sum_layers}} at the same number of GPUs

Data parallelism is STRONG scaling: the configuration's stated global batch is split over the ranks (batch / N
samples each); every rank holds the whole circuit, and parameter flows are all-reduced once per EM step.

``--impl reference`` times the CPU oracle alone (the reference has no runnable CPU implementation of this path;
the oracle is its restatement) and prints the same line with ``"impl": "reference"``.  ``--impl triton`` times
the reference's own GPU path (its Triton kernels, through its public API) on one GPU when the reference package
is installed under ``baseline/_ref``: the number to beat on the same box.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import pyjuice_b200 as pj  # noqa: E402
from pyjuice_b200 import data as pdata  # noqa: E402

STEP_SIZE, PSEUDOCOUNT = 0.1, 0.1
L2_BYTES = 126e6

CONFIGS = {
    # name: (description, global batch)
    "cfg0": ("HCLT-32 4cats K=8", 256),
    "cfg1": ("HCLT-784 grid28x28 256cats K=128", 512),
    "cfg2": ("PD-28x28 256cats K=64 splits[4,7,14]", 512),
    "cfg3": ("RAT-SPN-784 256cats depth5 rep16 K=32", 1024),
    "cfg4": ("HMM 4096 states vocab32768 T=128 tied", 256),
    # profiling case: the layer shape of cfg4 (4096 x 4096 tied transitions, 256 samples) in a circuit small enough
    # for multi-pass profiler captures (8 tokens, 2048-word vocabulary: well under 1 GB on the device)
    "cfg4-short": ("HMM 4096 states vocab2048 T=8 tied (profiling case)", 256),
    # profiling case: the circuit of cfg2 at a quarter of its batch (a few GB on the device instead of 15)
    "cfg2-b128": ("PD-28x28 256cats K=64 splits[4,7,14] (profiling case: batch 128)", 128),
}


class OurStructures:
    """Structure builders of this package under one calling convention (see `ReferenceStructures`)."""

    def hclt_from_data(self, x, num_latents, num_cats):
        return pj.structures.HCLT(torch.from_numpy(x).float(), num_latents=num_latents, num_cats=num_cats)

    def hclt_from_tree(self, tree, root, num_latents, num_cats):
        return pj.structures.tree_to_hidden_circuit(tree, root, num_latents=num_latents, num_cats=num_cats)

    def pd(self, shape, num_latents, split_points, num_cats):
        return pj.structures.PD(shape, num_latents=num_latents, split_points=split_points, num_cats=num_cats)

    def rat_spn(self, num_vars, num_latents, depth, num_repetitions, num_cats):
        return pj.structures.RAT_SPN(num_vars=num_vars, num_latents=num_latents, depth=depth,
                                     num_repetitions=num_repetitions, num_cats=num_cats)

    def hmm(self, seq_length, num_latents, num_emits):
        return pj.structures.HMM(seq_length=seq_length, num_latents=num_latents, num_emits=num_emits, homogeneous=True)


class ReferenceStructures:
    """The same five builders over the reference package (``--impl triton`` only)."""

    def __init__(self, juice):
        self.juice = juice
        import pyjuice.nodes.distributions as dists
        self.dists = dists

    def hclt_from_data(self, x, num_latents, num_cats):
        return self.juice.structures.HCLT(torch.from_numpy(x).float(), num_latents,
                                          input_node_params={"num_cats": num_cats})

    def hclt_from_tree(self, tree, root, num_latents, num_cats):
        import networkx as nx
        from pyjuice.structures.compilation import BayesianTreeToHiddenRegionGraph
        g = nx.Graph()
        g.add_nodes_from(range(tree.n))
        g.add_edges_from(tree.edges)
        return BayesianTreeToHiddenRegionGraph(g, root, num_latents, self.dists.Categorical, {"num_cats": num_cats})

    def pd(self, shape, num_latents, split_points, num_cats):
        return self.juice.structures.PD(shape, num_latents, split_points=split_points,
                                        input_node_params={"num_cats": num_cats})

    def rat_spn(self, num_vars, num_latents, depth, num_repetitions, num_cats):
        return self.juice.structures.RAT_SPN(num_vars=num_vars, num_latents=num_latents, depth=depth,
                                             num_repetitions=num_repetitions, input_node_params={"num_cats": num_cats})

    def hmm(self, seq_length, num_latents, num_emits):
        return self.juice.structures.HMM(seq_length=seq_length, num_latents=num_latents, num_emits=num_emits,
                                         homogeneous=True)


def build_workload(name: str, num_samples: int, lib=None):
    """Returns (root_ns, data[num_samples, V] as a numpy int64 array); both depend on the configuration's seed only."""
    import random
    lib = lib or OurStructures()
    if name == "cfg0":
        torch.manual_seed(0)
        x = pdata.tree_bn_samples(4096, 32, 4, seed=0)
        ns = lib.hclt_from_data(x, 8, 4)
        x = x[np.arange(num_samples) % 4096]
    elif name == "cfg1":
        torch.manual_seed(1)
        x, tree, root = pdata.grid_gaussian_bn_samples(num_samples, 28, 28, seed=1)
        ns = lib.hclt_from_tree(tree, root, 128, 256)
    elif name in ("cfg2", "cfg2-b128"):
        torch.manual_seed(2)
        random.seed(2)
        pts = sorted(set(range(4, 28, 4)) | set(range(7, 28, 7)) | set(range(14, 28, 14)))
        ns = lib.pd((28, 28), 64, [pts, pts], 256)
        x, _, _ = pdata.grid_gaussian_bn_samples(num_samples, 28, 28, seed=2)
    elif name == "cfg3":
        torch.manual_seed(3)
        random.seed(3)
        ns = lib.rat_spn(784, 32, 5, 16, 256)
        x = pdata.mixture_samples(num_samples, 784, 256, seed=3)
    elif name == "cfg4":
        torch.manual_seed(4)
        ns = lib.hmm(128, 4096, 32768)
        x = pdata.hmm_samples(num_samples, 128, 32768, seed=4)
    elif name == "cfg4-short":
        torch.manual_seed(4)
        ns = lib.hmm(8, 4096, 2048)
        x = pdata.hmm_samples(num_samples, 8, 2048, seed=4)
    else:
        raise ValueError(name)
    ns.init_parameters()
    return ns, x


def circuit_stats(pc, B):
    """Algorithmic work per sample and per step (the figures every roofline number is computed from).

    Product layers: a forward launch must read every DISTINCT child row once and write every product row once; a
    backward launch reads every product row's flow once and reads and writes every distinct child row's flow."""
    e_sum = sum(l.num_edges for g in pc.inner_layer_groups if g.is_sum() for l in g)
    prod_edges = sum(l.num_edges for g in pc.inner_layer_groups if g.is_prod() for l in g)
    prod_nodes = sum(l.num_nodes for g in pc.inner_layer_groups if g.is_prod() for l in g)
    n_in = sum(l.num_nodes for l in pc.input_layer_group)
    p_in = sum(l.num_parameters for l in pc.input_layer_group)
    f_in = sum(l.num_param_flows for l in pc.input_layer_group)
    f_in_untied = sum(l.num_untied_param_flows for l in pc.input_layer_group)
    sum_rows = sum(l.num_nodes for g in pc.inner_layer_groups if g.is_sum() for l in g)
    prod_fwd = prod_bwd = 0
    groups = pc.inner_layer_groups
    for gi, g in enumerate(groups):
        if not g.is_prod():
            continue
        folded = gi + 1 < len(groups) and pc._fusion_on(gi + 1)
        folded_bk = folded and B % 8 == 0                  # the backward sweep folds for batches that are multiples of 8
        n = sum(l.num_nodes for l in g)
        u = sum(int(t.numel()) * l.block_size for l in g for t in l.partitioned_u_cids)      # distinct child rows
        prod_fwd += (0 if folded else u + n) + (0 if folded_bk else u + n)      # forward pass + recompute in backward
        if not (folded_bk and pc._fused[gi + 1]["direct"]):
            prod_bwd += n + 2 * u
    return dict(e_sum=e_sum, prod_edges=prod_edges, prod_nodes=prod_nodes, n_in=n_in, p_in=p_in, f_in=f_in,
                f_in_untied=f_in_untied, p_sum=pc.num_sum_params, f_sum=pc.num_param_flows, sum_rows=sum_rows,
                prod_fwd_launched=prod_fwd, prod_bwd_launched=prod_bwd)


def family_of(name: str) -> str:
    """Launch family of a C-ABI entry point: the variants of one operator (product layer folded in, pre-split
    parameter tiles, all layers in one launch, built-in scratch) count as that operator."""
    if name.startswith("pcx_sum_chain"):                  # the dataflow launch: forward or element flows of many layers
        return "pcx_sum_fwd" if name.endswith("_fwd") else "pcx_sum_bwd_ele"
    if name.endswith("_dense2_prep"):                     # operand pre-pass of the wide dense kernels (fwd and element flows)
        return "pcx_sum_dense_prep"
    if name.startswith("pcx_sum_par_dense"):              # operand staging + one product: the parameter flows
        return "pcx_sum_bwd_par"
    if name in ("pcx_input_cat_shadow", "pcx_input_cat_flush_t"):     # upkeep of the transposed leaf tables
        return "pcx_input_cat_upkeep"
    if name.startswith("pcx_pack_sm"):
        return "pcx_pack_sum_params"
    if name.startswith("pcx_input_cat_fwd"):
        return "pcx_input_cat_fwd"
    if name.startswith("pcx_input_cat_bwd"):
        return "pcx_input_cat_bwd"
    for suffix in ("_fused", "_packed", "_batched", "_noalloc", "_dense2", "_dense", "_sm", "_t"):
        if name.endswith(suffix):
            name = name[:-len(suffix)]
    return name


# Algorithmic work of one launch family per STEP (batch B): (binding roofline, amount in bytes or flops, flops).
# Sum layers: 2 * E_sum * B flops per pass against the minimum bytes of the pass -- every child row read once,
# every output row written once (fp32), parameters once.  With B in the hundreds that is 15-30 flop/byte, far
# below the ridge (about 250 flop/byte at the measured peaks) unless a node block is large: HBM binds them, and
# the tensor-core figure is reported beside it.
def family_work(stats, B, elsize):
    s = stats
    flops = 2.0 * s["e_sum"] * B
    child_rows = s["prod_nodes"] if s["prod_nodes"] else s["sum_rows"]
    intensity = flops / (4.0 * B * (child_rows + s["sum_rows"]) + 4.0 * s["p_sum"])
    sum_bound = "tensor" if intensity > 250.0 else "hbm"

    def sum_family(nbytes):
        return (sum_bound, flops if sum_bound == "tensor" else nbytes, flops)

    return {
        "pcx_sum_fwd": sum_family(4.0 * B * (child_rows + s["sum_rows"]) + 4.0 * s["p_sum"]),
        # reads flows and values of the parents and values of the children, writes the children's flows
        "pcx_sum_bwd_ele": sum_family(4.0 * B * (2 * s["sum_rows"] + 2 * child_rows) + 4.0 * s["p_sum"]),
        # reads flows and values of the parents and values of the children; parameters read, flows read-modify-write
        "pcx_sum_bwd_par": sum_family(4.0 * B * (2 * s["sum_rows"] + child_rows) + 4.0 * s["p_sum"] + 8.0 * s["f_sum"]),
        # product layers that are not folded into the sum kernels: forward, once more inside the backward pass
        "pcx_prod_fwd": ("hbm", 4.0 * s["prod_fwd_launched"] * B, 0.0),
        "pcx_prod_bwd": ("hbm", 4.0 * s["prod_bwd_launched"] * B, 0.0),
        "pcx_input_cat_fwd": ("hbm", 4.0 * s["n_in"] * B, 0.0),
        # flows of every (node, sample) read; one flow cell per (node, sample) read and written
        "pcx_input_cat_bwd": ("hbm", 4.0 * s["n_in"] * B + 8.0 * min(s["f_in"], s["n_in"] * B), 0.0),
        "pcx_em_input_cat": ("hbm", 12.0 * s["p_in"], 0.0),
        "pcx_em_sum": ("hbm", 12.0 * s["p_sum"], 0.0),
        "pcx_fill_f32": ("hbm", 4.0 * (s["f_sum"] + s["f_in"]), 0.0),
        "pcx_pack_sum_params": ("hbm", 4.0 * s["p_sum"] + 2 * 4.0 * s["p_sum"], 0.0),
    }


# DRAM bytes (read + write) of ONE launch of the named family's dominant kernel, from `ncu` captures of the same
# kernels on one B200 (dram__bytes_read.sum + dram__bytes_write.sum); None = not captured.  (config, family) -> bytes
# Sources: profiles/ncu_full_cfg1_chain_par.md, profiles/ncu_full_cfg4_wide_gemm.md, profiles/launch_list_cfg2_pd_b512.md,
# profiles/traffic_cfg3_rat_spn_b1024.md
TRAFFIC_PER_LAUNCH = {
    # configs[1], B = 512: one dataflow launch each for the forward pass and the element flows, one batched launch
    # for the parameter flows
    ("cfg1", "pcx_sum_fwd"): 389.0e6,
    ("cfg1", "pcx_sum_bwd_ele"): 801.4e6,
    ("cfg1", "pcx_sum_bwd_par"): 636.3e6,
    # configs[4], B = 256: the GEMM of one 4096 x 4096 transition layer (captured without cache flushes between
    # kernels: the tied parameter tiles stay in L2 from layer to layer); parameter flows: the capture of a 7-layer
    # circuit scaled to the 127 layers of the one product (traffic grows with the contraction depth)
    ("cfg4", "pcx_sum_fwd"): 31.7e6,
    ("cfg4", "pcx_sum_bwd_ele"): 51.0e6,
    ("cfg4", "pcx_sum_bwd_par"): 449.2e6 * 127 / 7,
    # configs[2], B = 512: mean over the 29 parameter-flow launches of a step, captured at B = 128 and scaled by 4
    # (every operand is a row of B samples)
    ("cfg2", "pcx_sum_bwd_par"): 1536.0e6 * 4 / 29,
    # configs[3], B = 1024: mean over the product-backward launches of the capture
    ("cfg3", "pcx_prod_bwd"): (2569.6e6 + 503.2e6) / 29,
}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi.  It is started well before the timed
    regions (its start-up disturbs the GPU for a moment); only the samples that fall inside them are reported."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.windows = [], None, []
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def window(self, t0: float, t1: float):
        self.windows.append((t0, t1))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        ok = [r for t, r in self.rows if len(r) >= 6 and any(a - 0.05 <= t <= b + 0.05 for a, b in self.windows)]
        sm = [float(r[0]) for r in ok if r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in ok if r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in ok for n, v in zip(names, r[2:6]) if v.lower() == "active"})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm": p["hbm_gbs"], "tensor": p["bf16_tflops"], "source": "measured"}
    return {"hbm": 6650.0, "tensor": 1590.0, "source": "fallback"}


def host_threads() -> int:
    """Host cores this process may use.  Launchers such as torchrun export OMP_NUM_THREADS=1; the CPU arm sets the
    thread count itself so that it is the same however the script was started."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(n)
    return torch.get_num_threads()


def oracle_step_time(pc, x_cpu: torch.Tensor, repeats: int = 1):
    """Seconds per forward + backward + EM step of the fp32 CPU oracle on ``x_cpu``."""
    from oracle import pc_oracle as orc
    tables = orc._tables(pc)
    params = pc.params.data.detach().cpu()
    iparams = [l.params.data.detach().cpu() for l in pc.input_layer_group]
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        _, st = orc.forward(pc, x_cpu, params, iparams, dtype=torch.float32, tables=tables)
        orc.backward(pc, x_cpu, params, iparams, st)
        orc.em_update(pc, params, iparams, st, STEP_SIZE, PSEUDOCOUNT)
        best = min(best, time.perf_counter() - t0)
    return best


def cpu_sample_size(config: str, B: int, requested: int) -> int:
    """Samples per CPU step (configs[4] is 12.8 GFLOP per sample plus half a minute of per-step table work on the host)."""
    return min(B, requested, 128 if config.startswith("cfg4") else requested)


def run_reference(args, rank):
    """CPU arm: the oracle restatement of the reference algorithm on the host cores, one bounded sample per step."""
    if rank != 0:
        return
    cores = host_threads()
    desc, B = CONFIGS[args.config]
    sample = cpu_sample_size(args.config, B, args.cpu_sample)
    ns, x = build_workload(args.config, sample)
    pc = pj.compile(ns)
    xc = torch.from_numpy(x)
    # one step at the full sample size (also the warm-up) tells how many fit into about two minutes; a step that is
    # itself longer shrinks the sample (for most circuits this CPU path is close to linear in the number of samples)
    t_one = oracle_step_time(pc, xc)
    budget = 120.0
    if t_one > budget and sample > 8:
        sample = max(8, int(sample * budget / t_one) // 8 * 8)
        xc = xc[:sample]
        t_one = oracle_step_time(pc, xc)
    steps = max(1, min(args.steps, int(budget // max(t_one, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle_step_time(pc, xc)
    dt = (time.perf_counter() - t0) / steps
    value = sample / dt
    what = (f"{sample} samples per step (of the {B}-sample batch), fwd+bwd+EM, fp32 torch CPU, {cores} threads, "
            f"{steps} timed steps")
    print(json.dumps({
        "impl": "reference", "metric": "samples/sec fwd+bwd+EM", "value": value, "unit": "samples/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.config, max(args.gpus, 1)),
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": cores, "kind": "port", "sample": what},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(config: str, world: int) -> dict:
    desc, B = CONFIGS[config]
    return {"workload": f"{config}: {desc}", "global_batch": B, "batch_per_gpu": B // world, "parallelism": f"dp{world}",
            "em": {"step_size": STEP_SIZE, "pseudocount": PSEUDOCOUNT}}


def run_triton(args, rank):
    """The reference's own GPU path (Triton kernels, public API, stock code) on one GPU: the number to beat."""
    if rank != 0:
        return
    import types
    pkg = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(pkg, "pyjuice")):
        print(json.dumps({"impl": "triton", "unavailable": "the reference package is not installed under baseline/_ref"}))
        return
    os.environ.setdefault("PYJUICE_DISABLE_CUDA_KERNELS", "1")      # its CuTe kernels wait on barriers without a bound
    os.environ.setdefault("PYJUICE_DISABLE_DIST_CUDA_KERNELS", "1")
    os.environ.setdefault("PYJUICE_AUTOTUNE", "0")
    for name in ("matplotlib", "matplotlib.pyplot", "matplotlib.patches"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.path.insert(0, pkg)
    import pyjuice as juice
    dev = torch.device("cuda:0")
    desc, B = CONFIGS[args.config]
    n_batches = 4
    ns, x = build_workload(args.config, B * n_batches, lib=ReferenceStructures(juice))
    pc = juice.compile(ns, verbose=False)
    pc.to(dev)
    xs = [torch.from_numpy(x[i * B:(i + 1) * B]).to(dev) for i in range(n_batches)]
    opt = juice.optim.MiniBatchEM(pc, step_size=STEP_SIZE, pseudocount=PSEUDOCOUNT)
    results = {}
    for mode, kw in (("eager", {}), ("cudagraph", {"record_cudagraph": True}),
                     ("fp32", {"force_use_fp32": True})):
        def step(xb):
            lls = pc(xb, **kw)
            lls.mean().backward()
            opt.step()
            return lls
        try:
            for i in range(max(args.warmup, 3)):
                step(xs[i % n_batches])
            torch.cuda.synchronize()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            for i in range(args.steps):
                step(xs[i % n_batches])
            ev1.record()
            torch.cuda.synchronize()
            results[mode] = ev0.elapsed_time(ev1) / args.steps
        except Exception as e:                               # one variant must not lose the others
            results[mode] = f"{type(e).__name__}: {e}"[:200]
    ok = {k: v for k, v in results.items() if isinstance(v, float) and k != "fp32"}
    best = min(ok.values()) if ok else None
    print(json.dumps({
        "impl": "triton", "metric": "samples/sec fwd+bwd+EM", "value": B / (best * 1e-3) if best else None,
        "unit": "samples/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": best,
        "higher_is_better": True, "dtype": "reference default (bf16 forward, tf32 backward tensor cores)",
        "data": "synthetic", "config": workload_config(args.config, 1),
        "ms_per_step_by_variant": results,
        "note": "reference 2.6.3, Triton kernels only (CuTe kernels and autotuning switched off by its own env flags)",
    }), flush=True)


def measure_ours(config: str, args, rank: int, world: int, dev, K: int, W: int, sampler, with_cpu: bool):
    """Build one configuration on this rank, time it, and return the fields of its result (rank 0) or None."""
    import torch.distributed as dist
    from pyjuice_b200 import _lib
    desc, B = CONFIGS[config]
    assert B % world == 0, f"the global batch {B} does not split over {world} ranks"
    Bl = B // world
    n_batches = 4
    ns, x = build_workload(config, B * n_batches)
    pc = pj.compile(ns).to(dev)
    pc.use_cuda_graphs = not args.no_graphs
    pc.use_dataflow_launch = not args.no_dataflow
    if args.no_fold:
        pc.fuse_product_layers = False
    pc.use_side_stream = not args.no_side_stream
    pc.chain_tile = args.chain_tile
    max_cats = max(l.max_cats for l in pc.input_layer_group)
    np_dtype, elsize = (np.uint8, 1) if max_cats <= 256 else (np.int32, 4)
    shard = lambda i: x[i * B + rank * Bl:i * B + (rank + 1) * Bl]
    host = [torch.from_numpy(shard(i).astype(np_dtype)).pin_memory() for i in range(n_batches)]
    resident = [h.to(dev) for h in host]
    opt = pj.optim.MiniBatchEM(pc, step_size=STEP_SIZE, pseudocount=PSEUDOCOUNT, ddp=world > 1)

    def step(xb):
        lls = pc(xb)
        lls.mean().backward()
        opt.step()
        return lls

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(W):
        step(resident[i % n_batches])
    barrier()
    stats = circuit_stats(pc, Bl)          # after the first steps: which depths fold their product layer depends on the batch

    # launches per step, counted on an eager step (graph replays launch the same kernels)
    pc.use_cuda_graphs = False
    _lib.COUNT = 0
    step(resident[0])
    launches_per_step = _lib.COUNT
    pc.use_cuda_graphs = not args.no_graphs
    barrier()

    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.time()
    ev0.record()
    for i in range(K):
        step(resident[i % n_batches])
    ev1.record()
    barrier()
    ms_dev = ev0.elapsed_time(ev1)
    if sampler:
        sampler.window(t0, time.time())

    barrier()
    t0 = time.time()
    ev0.record()
    last = 0.0
    for i in range(K):
        xb = host[i % n_batches].to(dev, non_blocking=True)
        last = step(xb).mean().item()
    ev1.record()
    barrier()
    ms_e2e = ev0.elapsed_time(ev1)
    if sampler:
        sampler.window(t0, time.time())
    _lib.check_status(dev)                 # a bounded device wait that ran out would have produced wrong numbers

    t = torch.tensor([ms_dev, ms_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_dev, ms_e2e = t.tolist()

    # instrumented pass: per-family device time with CUDA events around every launch (eager, outside the timed region)
    # (every rank takes the steps — they contain the flow all-reduce — but only rank 0 records)
    fam = {}
    pc.use_cuda_graphs = False
    pc.use_side_stream = False            # one stream: every launch is timed alone
    for rep in range(3):
        _lib.PROFILE = [] if (rep == 2 and rank == 0) else None
        _lib.PROFILE_BYTES.clear()
        step(resident[0])
        torch.cuda.synchronize()
    if rank == 0:
        for name, a, b in _lib.PROFILE:
            d = fam.setdefault(family_of(name), [0, 0.0])
            d[0] += 1
            d[1] += a.elapsed_time(b)
    _lib.PROFILE = None
    _lib.check_status(dev)
    if world > 1:
        dist.barrier()
    if rank != 0:
        return None

    peaks = measured_peaks()
    work = family_work(stats, Bl, elsize)
    if "pcx_fill_f32" in _lib.PROFILE_BYTES:               # what the step actually cleared (untouched accumulators are skipped)
        work["pcx_fill_f32"] = ("hbm", float(_lib.PROFILE_BYTES["pcx_fill_f32"]), 0.0)
    fam_ms = {k: round(v[1], 4) for k, v in sorted(fam.items(), key=lambda kv: -kv[1][1])}
    top = max(fam, key=lambda k: fam[k][1])
    bound, amount, fam_flops = work.get(top, ("hbm", 0.0, 0.0))
    n_launch, tot_ms = fam[top]
    achieved = amount / (tot_ms * 1e-3) / (1e12 if bound == "tensor" else 1e9)

    def frac_of(k, v):
        """Fraction of the binding roofline, or None when one launch moves less than the L2 holds (then the bytes
        need not come from HBM and the HBM roofline does not apply)."""
        b, amt, _ = work[k]
        if b == "hbm" and amt / max(v[0], 1) < L2_BYTES:
            return None
        return round(amt / (v[1] * 1e-3) / (1e12 if b == "tensor" else 1e9) / peaks[b], 4)

    roofline = {"kernel": top, "bound": bound, "achieved": achieved, "peak": peaks[bound],
                "unit": "TFLOP/s" if bound == "tensor" else "GB/s", "frac": achieved / peaks[bound],
                "traffic": TRAFFIC_PER_LAUNCH.get((config, top)), "peak_source": peaks["source"],
                "launches_per_step": n_launch, "ms_per_step_in_kernel": tot_ms,
                "algorithmic_bytes_or_flops_per_step": amount,
                "tensor_tflops": fam_flops / (tot_ms * 1e-3) / 1e12 if fam_flops else None,
                "family_ms_per_step": fam_ms,
                "family_frac": {k: frac_of(k, v) for k, v in fam.items() if k in work and v[1] > 0}}
    sum_ms = sum(fam[k][1] for k in ("pcx_sum_fwd", "pcx_sum_bwd_ele", "pcx_sum_bwd_par", "pcx_sum_dense_prep") if k in fam)
    sum_tflops = 6.0 * stats["e_sum"] * Bl / (sum_ms * 1e-3) / 1e12 if sum_ms > 0 else None

    cpu = None
    if with_cpu:
        cores = host_threads()
        sample = cpu_sample_size(config, B, args.cpu_sample)
        sec = oracle_step_time(pc, torch.from_numpy(x[:sample]))
        cpu = {"value": sample / sec, "unit": "samples/s", "cores": cores, "kind": "port",
               "sample": f"one fwd+bwd+EM step on {sample} samples, fp32 torch CPU oracle, {cores} threads, {sec:.2f} s"}

    total = B * K
    cfg = workload_config(config, world)
    cfg.update({"input_dtype": np.dtype(np_dtype).name, "cuda_graphs": not args.no_graphs,
                "l2": "value buffers (%.2f GB per GPU) exceed the 126 MB L2; no explicit flush" %
                      (4.0 * Bl * 2 * (pc.num_nodes + pc.num_elements) / 1e9),
                "circuit": {k: int(v) for k, v in stats.items()}})
    out = {
        "value": total / (ms_dev * 1e-3), "ms_per_step": ms_dev / K, "steps": K, "warmup": W, "config": cfg,
        "e2e": {"value": total / (ms_e2e * 1e-3), "unit": "samples/s", "ms_per_step": ms_e2e / K,
                "h2d_bytes_per_step": int(B * pc.num_vars * elsize), "d2h_bytes_per_step": 4 * world,
                "last_mean_ll": last},
        "gpu_launches": launches_per_step * K,
        "roofline": roofline,
        # tflops: algorithmic flops (6 * edges * samples) over the sum-layer time of the instrumented pass (eager, one
        # stream, an event between every two kernels); tflops_whole_step: the same flops over the live step, leaves
        # and EM included — a lower bound that needs no instrumentation
        "sum_layers": {"tflops": sum_tflops, "ms_per_step": sum_ms,
                       "tflops_whole_step": 6.0 * stats["e_sum"] * Bl / (ms_dev / K * 1e-3) / 1e12,
                       "frac_of_bf16_peak": (sum_tflops or 0) / peaks["tensor"],
                       "arith": ["fp32 FMA (CUDA cores)",
                                 "tcgen05 bf16 hi/lo split x3, fp32 accumulate (fwd, element flows, parameter flows)",
                                 "tcgen05 single bf16, fp32 accumulate (fwd, element flows, parameter flows)"][args.sum_mode]},
        "cpu_baseline": cpu,
    }
    del pc, opt, resident, host
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="cfg4", choices=sorted(CONFIGS))
    ap.add_argument("--others", default=None,
                    help="comma-separated configurations measured in the same run (default: cfg1,cfg2,cfg3 beside cfg4)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "triton"])
    ap.add_argument("--cpu-sample", type=int, default=512, help="samples per CPU-baseline step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--no-fold", action="store_true", help="product layers as kernels of their own (not folded into the sum kernels)")
    ap.add_argument("--no-dataflow", action="store_true", help="per-layer launches instead of one launch per run of layers")
    ap.add_argument("--no-side-stream", action="store_true", help="every kernel of a step on one stream")
    ap.add_argument("--no-dependent-launch", action="store_true",
                    help="plain stream order between the dense kernels (no programmatic dependent launch)")
    ap.add_argument("--chain-tile", type=int, default=None, choices=[16, 32, 64], help="tile width of the dataflow launch")
    ap.add_argument("--sum-mode", type=int, default=1, choices=[0, 1, 2],
                    help="0 fp32 CUDA cores, 1 tensor cores with split-bf16 operands, 2 tensor cores single bf16")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        return run_reference(args, rank)
    if args.impl == "triton":
        return run_triton(args, rank)

    import torch.distributed as dist
    from pyjuice_b200 import _lib
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device(f"cuda:{local_rank}")
    if world > 1:
        import datetime
        # NCCL's kernels on a high-priority stream: the all-reduce of the input-layer flows runs beside the
        # parameter-flow kernel, whose 2000+ CTAs would otherwise keep the collective's few CTAs waiting for an SM
        opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120), pg_options=opts)
    W, K = max(args.warmup, 3), args.steps
    _lib.set_sum_mode(args.sum_mode)
    _lib.load().pcx_set_dependent_launch(0 if args.no_dependent_launch else 1)
    others = args.others if args.others is not None else ("cfg1,cfg2,cfg3" if args.config == "cfg4" else "")
    others = [c for c in others.split(",") if c and c != args.config]

    sampler = ClockSampler(local_rank) if rank == 0 else None      # started early: see the class comment
    head = measure_ours(args.config, args, rank, world, dev, K, W, sampler,
                        with_cpu=not args.no_cpu_baseline and world == 1 and rank == 0)
    other_out = {}
    for c in others:
        r = measure_ours(c, args, rank, world, dev, min(K, 30), 3, sampler, with_cpu=False)
        if r is not None:
            other_out[c] = {"value": r["value"], "unit": "samples/s", "ms_per_step": r["ms_per_step"], "steps": r["steps"],
                            "global_batch": r["config"]["global_batch"], "e2e": r["e2e"], "gpu_launches": r["gpu_launches"],
                            "roofline": {k: r["roofline"][k] for k in ("kernel", "bound", "achieved", "peak", "unit", "frac",
                                                                        "traffic", "family_ms_per_step", "family_frac")},
                            "sum_layers": r["sum_layers"]}
    clocks = sampler.stop() if sampler else None
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    out = {"metric": "samples/sec fwd+bwd+EM", "value": head["value"], "unit": "samples/s", "n_gpus": world,
           "steps": K, "warmup": W, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong",
           "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": head["config"], "e2e": head["e2e"],
           "gpu_launches": head["gpu_launches"], "roofline": head["roofline"], "sum_layers": head["sum_layers"],
           "cpu_baseline": head["cpu_baseline"], "other_configs": other_out, "clocks": clocks}
    sys.stderr.flush()
    print(json.dumps(out), flush=True)                 # the one JSON line, last thing on stdout


if __name__ == "__main__":
    main()
