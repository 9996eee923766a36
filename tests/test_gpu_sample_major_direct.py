"""Direct calls of the sample-major entry points (32-node blocks on the tensor cores) with hand-made tables, checked
against fp64 torch arithmetic: the single-pass forward of deep tables (every 64-entry chunk scaled by its own
per-sample maximum, chunks folded into a running sum) on values whose chunks lie hundreds of nats apart or hold no
mass at all, and the parameter flows of shallow tables, four of which share one 128 x 128 product.
Reference kernels: layer/sum_layer.py:367-412 (forward), 520-541 (parameter flows)."""
import pytest
import torch

from pyjuice_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NB = 32                                     # nodes per block


def _i32(t):
    return t.to(torch.int32).to(DEV).contiguous()


def _tables(n_rows, K, n_elems, pad_last, gen):
    """cids [n_rows, K] into element rows 1..n_elems (0 = no child; the last `pad_last` columns of odd rows), params
    theta[i, n, k] = params[pids[i, k] + n], one flow slot per parameter."""
    cids = torch.randint(1, n_elems + 1, (n_rows, K), generator=gen)
    if pad_last:
        cids[1::2, K - pad_last:] = 0
    theta = torch.rand(n_rows, K, NB, generator=gen, dtype=torch.float64) + 0.05
    theta = theta * (cids != 0)[:, :, None]
    theta = theta / theta.sum(dim=1, keepdim=True)
    theta = theta.float().double()                      # the reference arithmetic starts from the fp32 values
    params = torch.cat([torch.zeros(NB, dtype=torch.float64), theta.reshape(-1)])       # slot 0..31: dummy
    pids = (torch.arange(n_rows * K).reshape(n_rows, K) + 1) * NB
    return cids, theta, params.float(), pids


@pytest.mark.parametrize("B", [128, 40, 200])
@pytest.mark.parametrize("K,pad", [(65, 0), (100, 7), (256, 0), (300, 40), (64, 3), (24, 5)])
def test_forward_of_32_node_blocks_against_fp64(K, pad, B):
    gen = torch.Generator().manual_seed(K * 1000 + B)
    n_rows, n_elems = 5, 400
    cids, theta, params, pids = _tables(n_rows, K, n_elems, pad, gen)
    em = torch.randn(n_elems + 1, B, generator=gen, dtype=torch.float64) * 3.0
    # chunks of the table far apart: elements are shifted by a per-element offset of up to +-300 nats, some samples
    # see whole stretches of the table without mass, one sample has no mass anywhere
    em += (torch.randint(0, 4, (n_elems + 1, 1), generator=gen).double() - 2.0) * 150.0
    em[torch.rand(n_elems + 1, B, generator=gen) < 0.1] = float("-inf")
    em[: n_elems // 2, 1] = float("-inf")
    em[:, 3] = float("-inf")
    em[0] = float("-inf")                                           # row 0: "no element"
    em = em.float().double()
    ref = torch.logsumexp(torch.log(theta)[:, :, :, None] + em[cids][:, :, None, :], dim=1)       # [rows, NB, B]

    node_mars = torch.zeros(1 + n_rows * NB, B, device=DEV)
    nids = _i32(1 + NB * torch.arange(n_rows))
    first_row = _i32(torch.arange(n_rows))
    packed = torch.empty(int(_lib.load().pcx_sm_packed_bytes(n_rows, K, NB)), dtype=torch.uint8, device=DEV)
    params_d, cids_d, pids_d = params.to(DEV), _i32(cids), _i32(pids)
    _lib.call("pcx_pack_sm_params", packed, params_d, first_row, cids_d, pids_d, n_rows, NB, NB, K, 1, 0)
    _lib.call("pcx_sum_fwd_sm", node_mars, em.float().to(DEV).contiguous(), packed, first_row, nids, cids_d, None,
              n_rows, NB, K, B)
    torch.cuda.synchronize()
    _lib.check_status()
    got = node_mars[1:].reshape(n_rows, NB, B).double().cpu()
    dead = torch.isinf(ref)
    assert torch.equal(torch.isinf(got) & (got < 0), dead), "samples without mass must give -inf, all others a value"
    err = (got[~dead] - ref[~dead]).abs().max().item()
    print(f"K={K} B={B}: worst |log-value error| {err:.2e} at magnitudes up to {ref[~dead].abs().max():.0f}")
    assert err < 1e-4                                               # fp32 inputs at |value| ~ 300: 3e-5 of spacing


@pytest.mark.parametrize("B", [8, 40, 128])
@pytest.mark.parametrize("n_rows", [1, 5, 8])
@pytest.mark.parametrize("K,pad", [(32, 0), (24, 5), (8, 0), (40, 3)])
def test_parameter_flows_of_32_node_blocks_against_fp64(K, pad, n_rows, B):
    """K <= 32: four tables per 128 x 128 product (the tail group of `n_rows` = 1, 5 is partly empty); K = 40: one
    table per tile.  Element values far apart between samples exercise the per-sample shift."""
    gen = torch.Generator().manual_seed(K * 100 + n_rows * 10 + B)
    n_elems = 90
    cids, theta, params, pids = _tables(n_rows, K, n_elems, pad, gen)
    em = torch.randn(n_elems + 1, B, generator=gen, dtype=torch.float64) * 2.0 - 40.0 * torch.rand(1, B, generator=gen).double()
    em[0] = float("-inf")
    nm = torch.randn(1 + n_rows * NB, B, generator=gen, dtype=torch.float64) * 2.0 - 30.0
    nf = nm + torch.randn(1 + n_rows * NB, B, generator=gen, dtype=torch.float64) * 3.0 + 40.0 * torch.rand(1, B, generator=gen).double()
    nf[:, 2] = float("-inf")                                        # a sample that carries no flow at all
    em, nm, nf = em.float().double(), nm.float().double(), nf.float().double()
    ratio = torch.exp(nf - nm)[1:].reshape(n_rows, NB, B)           # flow / value of every node
    ref = theta * torch.einsum("inb,ikb->ikn", ratio, torch.exp(em[cids]))             # [rows, K, NB]

    pf = torch.zeros(params.numel(), device=DEV)
    nids = _i32(1 + NB * torch.arange(n_rows))
    first_row = _i32(torch.arange(n_rows))
    _lib.call("pcx_sum_bwd_par_sm", pf, nf.float().to(DEV).contiguous(), nm.float().to(DEV).contiguous(),
              em.float().to(DEV).contiguous(), params.to(DEV), first_row, nids, _i32(cids), _i32(pids), _i32(pids), None,
              n_rows, NB, NB, K, B, 1)
    torch.cuda.synchronize()
    _lib.check_status()
    got = pf[NB:].reshape(n_rows, K, NB).double().cpu()
    assert float(pf[:NB].abs().max()) == 0.0, "absent children add no flow"
    scale = ref.abs().max()
    err = ((got - ref).abs() / (ref.abs() + 1e-6 * scale)).max().item()
    print(f"K={K} rows={n_rows} B={B}: worst relative flow error {err:.2e}")
    assert err < 1e-3
