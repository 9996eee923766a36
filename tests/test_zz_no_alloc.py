"""The allocation-free forward entry point (``pcx_sum_fwd_noalloc``) against the regular tensor-core entry point.

Some hosts of this library cannot hand it device memory when they need a sum-layer forward: code that runs where
``cudaMalloc`` is off limits (it synchronises the whole device, which a latency-critical serving loop or a stream
capture cannot tolerate), or a plugin inside a process whose memory pool belongs to another framework.  For them
the library carries a fixed scratch array for the pre-split parameter tiles; this test checks that the entry point
built on it gives the same numbers as ``pcx_sum_fwd_packed`` with a caller-owned buffer, twice in a row (the second
call reuses the scratch the first one filled, with a different table), and that an oversized table is refused.

The file name sorts last on purpose: if this fails under ``pytest -x``, every other test has already run.
"""
import pytest
import torch

from cases import CASES, OursApi
from oracle import pc_oracle as orc
from pyjuice_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _circuit(dev=DEV):
    api = OursApi()
    torch.manual_seed(11)
    ns, kw = CASES["hclt_b128"](api)
    ns.init_parameters()
    return api.compile(ns, **kw).to(dev)


def test_noalloc_forward_matches_packed_entry_point_twice():
    _check_twice(DEV)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_noalloc_forward_on_a_second_device():
    """The scratch array exists once per GPU and its address is looked up per device: the same check on cuda:1 while
    cuda:0 stays the current device."""
    assert torch.cuda.current_device() == 0
    _check_twice("cuda:1")
    _check_twice(DEV)                                          # and the first device's address is still its own


def _check_twice(DEV):
    pc = _circuit(DEV)
    B = 96
    g = torch.Generator().manual_seed(3)
    x = (torch.rand(B, pc.num_vars, generator=g) * 12).long()
    pc(x.to(DEV))                                              # fills node_mars / element_mars, packs the tiles
    _, oracle = orc.forward(pc, x, pc.params.data.double().cpu(), [l.params.data.double().cpu() for l in pc.input_layer_group])
    sum_groups = [(gi, grp) for gi, grp in enumerate(pc.inner_layer_groups) if grp.is_sum() and grp[0].block_size % 128 == 0]
    assert len(sum_groups) >= 2
    checked = 0
    for gi, grp in sum_groups[:2]:                             # two different tables, back to back
        layer = grp[0]
        pc.inner_layer_groups[gi - 1].forward(pc.node_mars, pc.element_mars)      # this depth's products
        nids, cids, pids, _ = layer._dev["fw"][0]
        args = (nids.numel(), cids.size(1), layer.block_size, B)
        ref = pc.node_mars.clone()
        _lib.call("pcx_sum_fwd_packed", ref, pc.element_mars, layer._packed_fw[0], nids, cids, *args)
        out = torch.full_like(pc.node_mars, float("nan"))
        _lib.call("pcx_sum_fwd_noalloc", out, pc.element_mars, pc.params.data, nids, cids, pids, *args)
        torch.cuda.synchronize(DEV)
        s, e = layer._layer_nid_range
        assert torch.isfinite(out[s:e]).all()
        # same kernel, same tiles: the tolerance of the parity tests (1e-3 nats) is met with room to spare
        assert (out[s:e] - ref[s:e]).abs().max().item() <= 1e-3
        assert torch.equal(out[s:e], ref[s:e])
        # and against the CPU oracle's values of the same rows
        assert (out[s:e].double().cpu() - oracle.node_mars[s:e]).abs().max().item() <= 1e-3
        checked += 1
    assert checked == 2
    _lib.check_status(DEV)


def test_noalloc_rejects_tables_beyond_the_builtin_scratch():
    pc = _circuit()
    layer = [grp[0] for grp in pc.inner_layer_groups if grp.is_sum() and grp[0].block_size % 128 == 0][0]
    nids, cids, pids, _ = layer._dev["fw"][0]
    B = 8
    nm = torch.zeros(pc.num_nodes, B, device=DEV)
    em = torch.zeros(pc.num_elements, B, device=DEV)
    # 300 table rows, each needing at least one tile per 64-deep slice, exceed the 256 built-in tiles:
    # the call is refused before anything is launched
    big_nids = nids[:1].repeat(300).contiguous()
    big_cids = cids[:1].repeat(300, 1).contiguous()
    big_pids = pids[:1].repeat(300, 1).contiguous()
    with pytest.raises(_lib.PcxError, match="built-in scratch"):
        _lib.call("pcx_sum_fwd_noalloc", nm, em, pc.params.data, big_nids, big_cids, big_pids,
                  300, cids.size(1), layer.block_size, B)
    torch.cuda.synchronize()
