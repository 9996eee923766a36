"""The five benchmark configurations at FULL circuit size on the GPU.

* configs[0..3]: one forward + backward + EM step against the (fp64) CPU oracle on a batch the oracle finishes in
  seconds.  Log-likelihood within 1e-3 nats.  Flows and parameters within 1e-3 relative PLUS the rounding of the
  value buffers themselves: a flow is the exponential of a difference of fp32 log-values, and at |log-value| = 3500
  (784 variables with 256 categories) fp32 numbers are 2.4e-4 apart, so every rounding of a stored value moves a
  flow by up to 1.2e-4 relative, whoever computes it (the reference keeps the same fp32 buffers).  The allowance is
  four spacings: rtol = 1e-3 + 4 * eps_fp32 * max|log-likelihood|;
* all five, at the benchmark's own batch size, through properties that need no oracle:
  - flow conservation: in a smooth and decomposable circuit the flows of the leaves of one variable sum to the
    root flow (1) for every sample;
  - the tensor-core kernels (bf16 hi/lo split) and the fp32 CUDA-core kernels give the same log-likelihoods;
  - categorical leaf parameters stay normalised after the EM update.
"""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402
import pyjuice_b200 as pj  # noqa: E402
from pyjuice_b200 import _lib  # noqa: E402
from helpers import check_against_oracle, LL_ATOL  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _to_tensor(x):
    return torch.from_numpy(x).long()


@pytest.mark.parametrize("cfg,batch", [("cfg0", 256), ("cfg1", 64), ("cfg2", 16), ("cfg3", 64)])
def test_full_size_step_matches_oracle(cfg, batch):
    ns, x = bench.build_workload(cfg, batch)
    pc = pj.compile(ns).to(DEV)
    magnitude = pc(_to_tensor(x).to(DEV)).abs().max().item()
    errs = check_against_oracle(pc, _to_tensor(x), rtol=1e-3 + 4 * 1.1920929e-07 * magnitude)
    print("full size", cfg, f"max |LL| {magnitude:.0f}", {k: f"{v:.2e}" for k, v in errs.items()})
    _lib.check_status()


def test_cfg4_layer_shape_matches_oracle():
    """configs[4] at its full WIDTH (4096 states in blocks of 1024, 32768 tokens: the wide dense kernels with folded
    products and direct flow stores, the transposed leaf tables, tied parameters) on a sequence short enough for the
    fp64 oracle: log-likelihood within 1e-3 nats, flows and post-EM parameters within 1e-3 relative."""
    import numpy as np
    torch.manual_seed(4)
    ns = pj.structures.HMM(seq_length=4, num_latents=4096, num_emits=32768, homogeneous=True)
    ns.init_parameters()
    pc = pj.compile(ns).to(DEV)
    assert any(f.get("dense") for f in pc._fused.values()) and pc.input_layer_group[0]._shadow is not None
    x = torch.from_numpy(np.random.default_rng(4).integers(0, 32768, size=(64, 4)))
    x[:, 0] = x[0, 0]                                    # one token shared by all samples: many flows into one row
    for rep in range(2):
        errs = check_against_oracle(pc, x, fold_input_flows=True)
    print("cfg4 width", {k: f"{v:.2e}" for k, v in errs.items()})
    _lib.check_status()


@pytest.mark.parametrize("cfg", ["cfg0", "cfg1", "cfg2", "cfg3", "cfg4"])
def test_full_size_properties(cfg):
    _, B = bench.CONFIGS[cfg]
    ns, x = bench.build_workload(cfg, B)
    pc = pj.compile(ns).to(DEV)
    xb = _to_tensor(x).to(DEV)
    try:
        pc.init_param_flows(flows_memory=0.0)
        lls = pc(xb).clone()
        pc.backward(xb)
        assert torch.isfinite(lls).all()

        # flow conservation per variable and sample
        layer = pc.input_layer_group[0]
        s, e = layer._output_ind_range
        flows = pc.node_flows[s:e].exp()
        per_var = torch.zeros(pc.num_vars, B, device=DEV)
        per_var.index_add_(0, layer.vids[:, 0].to(DEV), flows)
        assert (per_var - 1.0).abs().max().item() < 2e-3, (per_var - 1.0).abs().max().item()

        # EM keeps every categorical distribution normalised
        pc.mini_batch_em(step_size=0.1, pseudocount=0.1)
        cats = layer.max_cats
        if int(layer.node_cats.min()) == cats:
            sums = layer.params.data.view(-1, cats).sum(dim=1)
            assert (sums - 1.0).abs().max().item() < 1e-4
        _lib.check_status()

        # same log-likelihoods from the fp32 CUDA-core kernels (fresh circuit: parameters as before the update)
        _lib.set_sum_mode(0)
        torch.manual_seed(0)
        ns2, _ = bench.build_workload(cfg, B)
        pc2 = pj.compile(ns2).to(DEV)
        lls2 = pc2(xb)
        assert (lls2 - lls).abs().max().item() <= LL_ATOL, (lls2 - lls).abs().max().item()
    finally:
        _lib.set_sum_mode(1)
