"""Benchmark of the compiled probabilistic-circuit training step (forward + backward + mini-batch EM).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config cfg1] [--impl ours|reference]

One "step" is one mini-batch of the named configuration through ``pc(x)``, ``lls.mean().backward()`` and
``MiniBatchEM.step()``.  Rank 0 prints ONE JSON line:

  value        samples/s over all ranks, inputs already resident in HBM, timed with CUDA events
  e2e          the same metric with each step's batch copied from pinned host memory inside the timed region
               and the mean log-likelihood read back to the host
  roofline     the dominant kernel family, timed per launch with CUDA events in a separate instrumented pass
  cpu_baseline the CPU oracle (fp32, all host threads) on a bounded sample of the same workload

``--impl reference`` times that CPU oracle alone (the reference has no runnable CPU implementation of this
path; the oracle is its restatement) and prints the same line with ``"impl": "reference"``.

Under torchrun every rank holds the full circuit and its own shard of the batch (weak scaling: the per-GPU
batch is fixed); parameter flows are all-reduced once per EM step.
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

CONFIGS = {
    # name: (description, per-GPU batch)
    "cfg0": ("HCLT-32 4cats K=8", 256),
    "cfg1": ("HCLT-784 grid28x28 256cats K=128", 512),
    "cfg2": ("PD-28x28 256cats K=64 splits[4,7,14]", 512),
    "cfg3": ("RAT-SPN-784 256cats depth5 rep16 K=32", 1024),
    "cfg4": ("HMM 4096 states vocab32768 T=128 tied", 256),
}


def build_workload(name: str, num_samples: int, seed_offset: int = 0):
    """Returns (root_ns, data[num_samples, V] as a numpy int64 array).  Circuit structure and parameters depend
    on the configuration's seed only; ``seed_offset`` (the rank) only changes which samples are drawn."""
    if name == "cfg0":
        torch.manual_seed(0)
        x = pdata.tree_bn_samples(4096, 32, 4, seed=0)
        ns = pj.structures.HCLT(torch.from_numpy(x).float(), num_latents=8, num_cats=4)
        x = x[(np.arange(num_samples) + seed_offset * num_samples) % 4096]
    elif name == "cfg1":
        torch.manual_seed(1)
        _, tree, root = pdata.grid_gaussian_bn_samples(16, 28, 28, seed=1)
        ns = pj.structures.tree_to_hidden_circuit(tree, root, num_latents=128, num_cats=256)
        x, _, _ = pdata.grid_gaussian_bn_samples(num_samples * (seed_offset + 1), 28, 28, seed=1)
        x = x[-num_samples:]
    elif name == "cfg2":
        import random
        torch.manual_seed(2)
        random.seed(2)
        pts = sorted(set(range(4, 28, 4)) | set(range(7, 28, 7)) | set(range(14, 28, 14)))
        ns = pj.structures.PD((28, 28), num_latents=64, split_points=[pts, pts], num_cats=256)
        x, _, _ = pdata.grid_gaussian_bn_samples(num_samples * (seed_offset + 1), 28, 28, seed=2)
        x = x[-num_samples:]
    elif name == "cfg3":
        import random
        torch.manual_seed(3)
        random.seed(3)
        ns = pj.structures.RAT_SPN(num_vars=784, num_latents=32, depth=5, num_repetitions=16, num_cats=256)
        x = pdata.mixture_samples(num_samples * (seed_offset + 1), 784, 256, seed=3)[-num_samples:]
    elif name == "cfg4":
        torch.manual_seed(4)
        ns = pj.structures.HMM(seq_length=128, num_latents=4096, num_emits=32768, homogeneous=True)
        x = pdata.hmm_samples(num_samples * (seed_offset + 1), 128, 32768, seed=4)[-num_samples:]
    else:
        raise ValueError(name)
    ns.init_parameters()
    return ns, x


def circuit_stats(pc, B):
    """Algorithmic work per sample and per step (the figures every roofline number is computed from)."""
    e_sum = sum(l.num_edges for g in pc.inner_layer_groups if g.is_sum() for l in g)
    prod_edges = sum(l.num_edges for g in pc.inner_layer_groups if g.is_prod() for l in g)
    prod_nodes = sum(l.num_nodes for g in pc.inner_layer_groups if g.is_prod() for l in g)
    n_in = sum(l.num_nodes for l in pc.input_layer_group)
    p_in = sum(l.num_parameters for l in pc.input_layer_group)
    f_in = sum(l.num_param_flows for l in pc.input_layer_group)
    sum_rows = sum(l.num_nodes for g in pc.inner_layer_groups if g.is_sum() for l in g)
    # product layers that still run as kernels of their own (the others are folded into the sum kernels):
    # (edges + nodes) per forward launch, (edges + 2 nodes) per backward launch, summed over the launches of a step
    prod_fwd = prod_bwd = 0
    groups = pc.inner_layer_groups
    for gi, g in enumerate(groups):
        if not g.is_prod():
            continue
        folded = gi + 1 < len(groups) and pc._fusion_on(gi + 1)
        folded_bk = folded and B % 8 == 0                  # the backward sweep folds for batches that are multiples of 8
        e, n = sum(l.num_edges for l in g), sum(l.num_nodes for l in g)
        prod_fwd += (0 if folded else e + n) + (0 if folded_bk else e + n)      # forward pass + recompute in backward
        if not (folded_bk and pc._fused[gi + 1]["direct"]):
            prod_bwd += e + 2 * n
    return dict(e_sum=e_sum, prod_edges=prod_edges, prod_nodes=prod_nodes, n_in=n_in, p_in=p_in, f_in=f_in,
                p_sum=pc.num_sum_params, f_sum=pc.num_param_flows, sum_rows=sum_rows,
                prod_fwd_launched=prod_fwd, prod_bwd_launched=prod_bwd)


def family_of(name: str) -> str:
    """Launch family of a C-ABI entry point: the variants of one operator (product layer folded in, pre-split
    parameter tiles, all layers in one launch, built-in scratch) count as that operator."""
    if name.startswith("pcx_sum_chain"):                  # the dataflow launch: forward or element flows of many layers
        return "pcx_sum_fwd" if name.endswith("_fwd") else "pcx_sum_bwd_ele"
    if name.startswith("pcx_sum_par_dense"):              # operand staging + one product: the parameter flows
        return "pcx_sum_bwd_par"
    if name.startswith("pcx_pack_sm"):
        return "pcx_pack_sum_params"
    for suffix in ("_fused", "_packed", "_batched", "_noalloc", "_dense", "_sm"):
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
        "pcx_input_cat_bwd": ("hbm", 4.0 * s["n_in"] * B + 8.0 * s["f_in"], 0.0),
        "pcx_em_input_cat": ("hbm", 12.0 * s["p_in"], 0.0),
        "pcx_em_sum": ("hbm", 12.0 * s["p_sum"], 0.0),
        "pcx_fill_f32": ("hbm", 4.0 * (s["f_sum"] + s["f_in"]), 0.0),
        "pcx_pack_sum_params": ("hbm", 4.0 * s["p_sum"] + 2 * 4.0 * s["p_sum"], 0.0),
    }


# DRAM bytes per step (read + write) of a launch family, from ncu captures of the same kernels; None = not captured
TRAFFIC_PER_STEP = {
    # configs[1], B = 512: one dataflow launch each for the forward pass and the element flows, one batched launch
    # for the parameter flows (profiles/ncu_full_cfg1_chain_par.md)
    ("cfg1", "pcx_sum_fwd"): 389.0e6,
    ("cfg1", "pcx_sum_bwd_ele"): 801.4e6,
    ("cfg1", "pcx_sum_bwd_par"): 636.3e6,
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


def run_reference(args, rank):
    """CPU arm: the oracle restatement of the reference algorithm on the host cores, one bounded sample per step."""
    if rank != 0:
        return
    desc, B = CONFIGS[args.config]
    sample = min(B, args.cpu_sample)
    ns, x = build_workload(args.config, sample)
    pc = pj.compile(ns)
    xc = torch.from_numpy(x)
    cores = torch.get_num_threads()
    # one step at the full sample size tells how long K of them would take; the sample shrinks until the whole
    # run fits in about two minutes (throughput of this CPU path is close to linear in the number of samples)
    t_one = oracle_step_time(pc, xc)
    budget = 120.0
    if t_one * args.steps > budget and sample > 8:
        sample = max(8, int(sample * budget / (t_one * args.steps)) // 8 * 8)
        xc = xc[:sample]
        oracle_step_time(pc, xc)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle_step_time(pc, xc)
    dt = (time.perf_counter() - t0) / args.steps
    value = sample / dt
    what = f"{sample} samples per step (of the {B}-sample batch), fwd+bwd+EM, fp32 torch CPU, {cores} threads"
    print(json.dumps({
        "impl": "reference", "metric": "samples/sec fwd+bwd+EM", "value": value, "unit": "samples/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.config}: {desc}", "batch_per_gpu": B},
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": cores, "kind": "port", "sample": what},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--config", default="cfg1", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-sample", type=int, default=512, help="samples per CPU-baseline step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--no-dataflow", action="store_true", help="per-layer launches instead of one launch per run of layers")
    ap.add_argument("--no-side-stream", action="store_true", help="every kernel of a step on one stream")
    ap.add_argument("--chain-tile", type=int, default=None, choices=[16, 32, 64], help="tile width of the dataflow launch")
    ap.add_argument("--sum-mode", type=int, default=1, choices=[0, 1, 2],
                    help="0 fp32 CUDA cores, 1 tensor cores with split-bf16 operands, 2 tensor cores single bf16")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        return run_reference(args, rank)

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
    desc, B = CONFIGS[args.config]
    _lib.set_sum_mode(args.sum_mode)

    sampler = ClockSampler(local_rank) if rank == 0 else None      # started early: see the class comment
    n_batches = 4
    ns, x = build_workload(args.config, B * n_batches, seed_offset=rank)
    pc = pj.compile(ns).to(dev)
    pc.use_cuda_graphs = not args.no_graphs
    pc.use_dataflow_launch = not args.no_dataflow
    pc.use_side_stream = not args.no_side_stream
    pc.chain_tile = args.chain_tile
    stats = circuit_stats(pc, B)
    max_cats = max(l.max_cats for l in pc.input_layer_group)
    np_dtype, elsize = (np.uint8, 1) if max_cats <= 256 else (np.int32, 4)
    host = [torch.from_numpy(x[i * B:(i + 1) * B].astype(np_dtype)).pin_memory() for i in range(n_batches)]
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
    clocks = sampler.stop() if sampler else None

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
        step(resident[0])
        torch.cuda.synchronize()
    if rank == 0:
        for name, a, b in _lib.PROFILE:
            d = fam.setdefault(family_of(name), [0, 0.0])
            d[0] += 1
            d[1] += a.elapsed_time(b)
    _lib.PROFILE = None
    pc.use_cuda_graphs = not args.no_graphs
    pc.use_side_stream = not args.no_side_stream

    if world > 1:
        dist.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    work = family_work(stats, B, elsize)
    fam_ms = {k: round(v[1], 4) for k, v in sorted(fam.items(), key=lambda kv: -kv[1][1])}
    top = max(fam, key=lambda k: fam[k][1])
    bound, amount, fam_flops = work.get(top, ("hbm", 0.0, 0.0))
    n_launch, tot_ms = fam[top]
    achieved = amount / (tot_ms * 1e-3) / (1e12 if bound == "tensor" else 1e9)
    roofline = {"kernel": top, "bound": bound, "achieved": achieved, "peak": peaks[bound],
                "unit": "TFLOP/s" if bound == "tensor" else "GB/s", "frac": achieved / peaks[bound],
                "traffic": TRAFFIC_PER_STEP.get((args.config, top)), "peak_source": peaks["source"],
                "launches_per_step": n_launch, "ms_per_step_in_kernel": tot_ms,
                "algorithmic_bytes_or_flops_per_step": amount,
                "tensor_tflops": fam_flops / (tot_ms * 1e-3) / 1e12 if fam_flops else None,
                "family_ms_per_step": fam_ms,
                "family_frac": {k: round(work[k][1] / (v[1] * 1e-3) / (1e12 if work[k][0] == "tensor" else 1e9)
                                         / peaks[work[k][0]], 4) for k, v in fam.items() if k in work and v[1] > 0}}
    sum_ms = sum(fam[k][1] for k in ("pcx_sum_fwd", "pcx_sum_bwd_ele", "pcx_sum_bwd_par") if k in fam)
    sum_tflops = 6.0 * stats["e_sum"] * B / (sum_ms * 1e-3) / 1e12 if sum_ms > 0 else None

    cpu = None
    if not args.no_cpu_baseline and world == 1:            # the CPU baseline is reported by the single-GPU run only
        sample = min(B, args.cpu_sample)
        sec = oracle_step_time(pc, torch.from_numpy(x[:sample]))
        cores = torch.get_num_threads()
        cpu = {"value": sample / sec, "unit": "samples/s", "cores": cores, "kind": "port",
               "sample": f"one fwd+bwd+EM step on {sample} samples, fp32 torch CPU oracle, {cores} threads, {sec:.2f} s"}

    total = B * world * K
    out = {
        "metric": "samples/sec fwd+bwd+EM", "value": total / (ms_dev * 1e-3), "unit": "samples/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_dev / K, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.config}: {desc}", "batch_per_gpu": B, "global_batch": B * world,
                   "parallelism": f"dp{world}", "em": {"step_size": STEP_SIZE, "pseudocount": PSEUDOCOUNT},
                   "input_dtype": np.dtype(np_dtype).name, "cuda_graphs": not args.no_graphs,
                   "l2": "value buffers (%.2f GB) exceed the 126 MB L2; no explicit flush" %
                         (4.0 * B * 2 * (pc.num_nodes + pc.num_elements) / 1e9),
                   "circuit": {k: int(v) for k, v in stats.items()}},
        "e2e": {"value": total / (ms_e2e * 1e-3), "unit": "samples/s", "ms_per_step": ms_e2e / K,
                "h2d_bytes_per_step": int(B * pc.num_vars * elsize), "d2h_bytes_per_step": 4, "last_mean_ll": last},
        "gpu_launches": launches_per_step * K,
        "roofline": roofline,
        "sum_layers": {"tflops": sum_tflops, "ms_per_step": sum_ms, "frac_of_bf16_peak": (sum_tflops or 0) / peaks["tensor"],
                       "arith": ["fp32 FMA (CUDA cores)",
                                 "tcgen05 bf16 hi/lo split x3, fp32 accumulate (fwd, element flows, parameter flows)",
                                 "tcgen05 single bf16, fp32 accumulate (fwd, element flows, parameter flows)"][args.sum_mode]},
        "cpu_baseline": cpu,
        "clocks": clocks,
    }
    if world > 1:
        dist.destroy_process_group()
    sys.stderr.flush()
    print(json.dumps(out), flush=True)                 # the one JSON line, last thing on stdout


if __name__ == "__main__":
    main()
