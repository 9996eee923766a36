"""The give-up branch of the bounded device waits, exercised without faulting, trapping or hanging the GPU.

Every mbarrier wait and counter poll of the tensor-core kernels has an iteration limit; on expiry the kernel
records a code in a per-device status word and returns (the reference's kernels spin without a bound,
layer/kernels/c/tlmm_forward_sum.cu:55-61).  `pcx_probe_bounded_wait` launches one warp that waits on something
nobody ever signals, with a small explicit limit, so the branch runs in a few milliseconds.
"""
import pytest
import torch

import pyjuice_b200 as pj
from pyjuice_b200 import _lib
from cases import CASES, OursApi, data_for
from helpers import check_against_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("which", [0, 1])
def test_bounded_wait_runs_out_and_is_reported(which):
    torch.cuda.synchronize()
    _lib.clear_status(DEV)
    assert _lib.get_status(DEV) == 0
    _lib.call("pcx_probe_bounded_wait", which, 2000)
    assert _lib.get_status(DEV) == 900 + which           # the kernel returned through its give-up branch
    with pytest.raises(_lib.PcxError):
        _lib.check_status(DEV)                           # raises once and clears the word
    assert _lib.get_status(DEV) == 0
    _lib.check_status(DEV)

    # the context is still usable: a normal step afterwards matches the oracle
    api = OursApi()
    torch.manual_seed(0)
    ns, kw = CASES["hclt_b128"](api)
    ns.init_parameters()
    pc = api.compile(ns, **kw).to(DEV)
    check_against_oracle(pc, data_for(pc, 64))
    _lib.check_status(DEV)


def test_probe_rejects_unbounded_limits():
    with pytest.raises(_lib.PcxError):
        _lib.call("pcx_probe_bounded_wait", 0, 1 << 20)
    with pytest.raises(_lib.PcxError):
        _lib.call("pcx_probe_bounded_wait", 2, 100)
