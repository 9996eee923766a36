"""Two data-parallel ranks on two GPUs (NCCL): after `sync_param_flows` every rank holds the flows of the whole
batch, and the EM update leaves identical parameters on both ranks, equal to a single-GPU step on the full batch.
Local-SGD (`sync_every > 1`) is checked against two single-GPU circuits averaged on the host.
Skipped on boxes with fewer than two GPUs."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build():
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    from cases import CASES, OursApi
    api = OursApi()
    torch.manual_seed(21)
    ns, kw = CASES["hmm_blocks"](api)             # tied sums and tied leaves with several flow accumulators
    ns.init_parameters()
    return api.compile(ns, **kw)


def _data(pc, B):
    g = torch.Generator().manual_seed(5)
    return (torch.rand(B, pc.num_vars, generator=g) * 12).long()


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device(f"cuda:{rank}"))
    try:
        import pyjuice_b200 as pj
        pc = _build().to(f"cuda:{rank}")
        x = _data(pc, 64)
        shard = x[rank * 32:(rank + 1) * 32].to(f"cuda:{rank}")
        opt = pj.optim.MiniBatchEM(pc, step_size=0.2, pseudocount=0.1, ddp=True)
        lls = pc(shard)
        lls.mean().backward()
        pc.sync_param_flows()
        flows = pc.param_flows.clone().cpu()
        cum = pc._cum_flow                                # flow total of the window, summed over the ranks
        opt.ddp = False                                   # already synchronised above
        opt.step()
        torch.cuda.synchronize()
        first = dict(flows=flows, params=pc.params.data.cpu(), iparams=pc.input_layer_group[0].params.data.cpu(), cum=cum)
        # many more steps through the optimizer's own (overlapped, two-part) synchronisation
        opt.ddp = True
        for _ in range(60):
            pc(shard).mean().backward()
            opt.step()
        torch.cuda.synchronize()
        torch.save(dict(first, params_after=pc.params.data.cpu(), iparams_after=pc.input_layer_group[0].params.data.cpu(),
                        cum_after=pc._cum_flow), os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_step_equals_single_gpu_step(tmp_path):
    import torch.multiprocessing as mp
    import pyjuice_b200 as pj
    port = 29700 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = (torch.load(tmp_path / f"rank{r}.pt") for r in range(2))
    assert torch.equal(r0["flows"], r1["flows"]) and torch.equal(r0["params"], r1["params"])
    assert torch.equal(r0["iparams"], r1["iparams"])
    assert abs(r0["cum"] - 64.0) < 1e-3

    pc = _build().to("cuda:0")
    x = _data(pc, 64).to("cuda:0")
    opt = pj.optim.MiniBatchEM(pc, step_size=0.2, pseudocount=0.1)
    pc(x).mean().backward()
    flows = pc.param_flows.clone().cpu()
    opt.step()
    assert torch.allclose(r0["flows"], flows, rtol=1e-4, atol=1e-5)
    assert torch.allclose(r0["params"], pc.params.data.cpu(), rtol=1e-4, atol=1e-7)
    assert torch.allclose(r0["iparams"], pc.input_layer_group[0].params.data.cpu(), rtol=1e-4, atol=1e-7)

    # sixty more steps: ranks stay identical and finite, the flow total stays that of one window, and the result is
    # that of sixty single-GPU steps on the full batch
    assert torch.equal(r0["params_after"], r1["params_after"]) and torch.equal(r0["iparams_after"], r1["iparams_after"])
    assert torch.isfinite(r0["params_after"]).all() and r0["cum_after"] == 0.0
    for _ in range(60):
        pc(x).mean().backward()
        opt.step()
    assert torch.allclose(r0["params_after"], pc.params.data.cpu(), rtol=2e-3, atol=1e-6)
    assert torch.allclose(r0["iparams_after"], pc.input_layer_group[0].params.data.cpu(), rtol=2e-3, atol=1e-6)


def _local_sgd_worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = f"cuda:{rank}"
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device(dev))
    try:
        import pyjuice_b200 as pj
        pc = _build().to(dev)
        x = _data(pc, 64)
        shard = x[rank * 32:(rank + 1) * 32].to(dev)
        opt = pj.optim.MiniBatchEM(pc, step_size=0.5, pseudocount=0.1, ddp=True, sync_every=2)
        snaps = []
        for _ in range(4):                                 # updates 1 and 3 are local, 2 and 4 end with the average
            pc(shard).mean().backward()
            opt.step()
            snaps.append((pc.params.data.cpu().clone(), pc.input_layer_group[0].params.data.cpu().clone()))
        lls = pc(shard)                                    # the operand tiles must follow the averaged parameters
        torch.cuda.synchronize()
        torch.save(dict(snaps=snaps, lls=lls.cpu()), os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_local_sgd_two_ranks(tmp_path):
    """`sync_every=2`: each rank updates on its own shard's flows, every second update is followed by the average
    of the parameters; checked against two single-GPU circuits stepped on the shards and averaged on the host."""
    import torch.multiprocessing as mp
    import pyjuice_b200 as pj
    port = 33700 + (os.getpid() % 2000)
    mp.spawn(_local_sgd_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r = [torch.load(tmp_path / f"rank{k}.pt") for k in range(2)]
    for step, same in enumerate([False, True, False, True]):
        for a, b in zip(r[0]["snaps"][step], r[1]["snaps"][step]):
            assert torch.equal(a, b) == same, f"update {step + 1}: ranks {'differ' if same else 'agree'}"

    pcs = [_build().to("cuda:0") for _ in range(2)]
    x = _data(pcs[0], 64).to("cuda:0")
    opts = [pj.optim.MiniBatchEM(pc, step_size=0.5, pseudocount=0.1) for pc in pcs]
    for step in range(4):
        for k in range(2):
            pcs[k](x[k * 32:(k + 1) * 32]).mean().backward()
            opts[k].step()
        if step % 2 == 1:
            for get in (lambda pc: pc.params.data, lambda pc: pc.input_layer_group[0].params.data):
                mean = (get(pcs[0]) + get(pcs[1])) / 2
                for pc in pcs:
                    get(pc).copy_(mean)
                    pc._packer.invalidate()
        for k in range(2):
            assert torch.allclose(r[k]["snaps"][step][0], pcs[k].params.data.cpu(), rtol=1e-4, atol=1e-7)
            assert torch.allclose(r[k]["snaps"][step][1], pcs[k].input_layer_group[0].params.data.cpu(), rtol=1e-4, atol=1e-7)
    for k in range(2):
        assert torch.allclose(r[k]["lls"], pcs[k](x[k * 32:(k + 1) * 32]).cpu(), rtol=1e-5, atol=1e-4)


def _bf16_worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = f"cuda:{rank}"
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device(dev))
    try:
        import pyjuice_b200 as pj
        pc = _build().to(dev)
        x = _data(pc, 64)
        shard = x[rank * 32:(rank + 1) * 32].to(dev)
        opt = pj.optim.MiniBatchEM(pc, step_size=0.2, pseudocount=0.1, ddp=True, ddp_dtype=torch.bfloat16)
        assert pc._overlap_ready(), "a reduced-precision exchange keeps the overlapped two-part all-reduce"
        for _ in range(5):
            pc(shard).mean().backward()
            opt.step()
        torch.cuda.synchronize()
        torch.save(dict(params=pc.params.data.cpu(), iparams=pc.input_layer_group[0].params.data.cpu()),
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_bf16_flow_exchange_two_ranks(tmp_path):
    """`ddp_dtype=torch.bfloat16` (the reference's `sync_param_flows(dtype=...)`, model/tensorcircuit.py:1456-1460):
    the flows cross the link in bf16, through the same overlapped two-part all-reduce as fp32; the ranks stay
    identical and the parameters stay within bf16's 2^-8 relative rounding of the fp32 single-GPU result."""
    import torch.multiprocessing as mp
    import pyjuice_b200 as pj
    port = 37700 + (os.getpid() % 2000)
    mp.spawn(_bf16_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = (torch.load(tmp_path / f"rank{r}.pt") for r in range(2))
    assert torch.equal(r0["params"], r1["params"]) and torch.equal(r0["iparams"], r1["iparams"])
    pc = _build().to("cuda:0")
    x = _data(pc, 64).to("cuda:0")
    opt = pj.optim.MiniBatchEM(pc, step_size=0.2, pseudocount=0.1)
    for _ in range(5):
        pc(x).mean().backward()
        opt.step()
    err = ((r0["params"] - pc.params.data.cpu()).abs() / pc.params.data.cpu().clamp_min(1e-3)).max().item()
    ierr = (r0["iparams"] - pc.input_layer_group[0].params.data.cpu()).abs().max().item()
    print(f"bf16 exchange: worst relative parameter difference {err:.2e}, leaf parameters {ierr:.2e}")
    assert err < 2e-2 and ierr < 2e-2


def _big_vocab():
    import pyjuice_b200 as pj
    torch.manual_seed(8)
    ns = pj.structures.HMM(seq_length=6, num_latents=32, num_emits=9000, homogeneous=True, block_size=8)
    ns.init_parameters()
    return pj.compile(ns, max_tied_ns_per_parflow_block=2)


def _shadow_worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = f"cuda:{rank}"
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device(dev))
    try:
        import pyjuice_b200 as pj
        from pyjuice_b200 import _lib
        calls = []
        orig = _lib.call
        _lib.call = lambda name, *a: (calls.append(name), orig(name, *a))[1]
        pc = _big_vocab().to(dev)
        g = torch.Generator().manual_seed(5)
        x = torch.randint(0, 9000, (64, 6), generator=g)
        shard = x[rank * 32:(rank + 1) * 32].to(dev)
        opt = pj.optim.MiniBatchEM(pc, step_size=0.3, pseudocount=0.1, ddp=True)
        for _ in range(4):
            pc(shard).mean().backward()
            opt.step()
        torch.cuda.synchronize()
        torch.save(dict(params=pc.params.data.cpu(), iparams=pc.input_layer_group[0].params.data.cpu(),
                        fused="pcx_em_input_cat_t" in calls, flushed="pcx_input_cat_flush_t" in calls),
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_large_vocabulary_flows_are_exchanged_in_their_transposed_table(tmp_path):
    """Leaves with more than 8192 categories keep their flows in a transposed shadow table.  Under the overlapped
    data-parallel exchange that table itself is all-reduced (no move into the `[row, category]` accumulators) and the
    EM update runs straight from it on every rank; the result equals single-GPU training on the full batch."""
    import torch.multiprocessing as mp
    import pyjuice_b200 as pj
    port = 39700 + (os.getpid() % 2000)
    mp.spawn(_shadow_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = (torch.load(tmp_path / f"rank{r}.pt") for r in range(2))
    assert r0["fused"] and r1["fused"] and not r0["flushed"] and not r1["flushed"]
    assert torch.equal(r0["params"], r1["params"]) and torch.equal(r0["iparams"], r1["iparams"])
    pc = _big_vocab().to("cuda:0")
    g = torch.Generator().manual_seed(5)
    x = torch.randint(0, 9000, (64, 6), generator=g).to("cuda:0")
    opt = pj.optim.MiniBatchEM(pc, step_size=0.3, pseudocount=0.1)
    for _ in range(4):
        pc(x).mean().backward()
        opt.step()
    assert torch.allclose(r0["params"], pc.params.data.cpu(), rtol=1e-3, atol=1e-7)
    assert torch.allclose(r0["iparams"], pc.input_layer_group[0].params.data.cpu(), rtol=1e-3, atol=1e-9)
