"""World-size-2 data-parallel logic on CPU (gloo): the flow arena's single all-reduce sums every accumulator and the
running flow total exactly, leaves the excluded tail alone, and is a no-op without a process group; the Local-SGD
exchange step averages the parameters of the ranks every `sync_every` updates."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    from pyjuice_b200.flows import FlowArena
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        arena = FlowArena([1000, 37, 300], "cpu")
        for i, v in enumerate(arena.views):
            v.copy_(torch.arange(v.numel(), dtype=torch.float32) * (rank + 1) + i)
        before_tail = arena.views[2][100:].clone()
        reduce_len = arena.segment_end(2, 100)                     # last segment: only its first 100 floats
        head = arena.all_reduce(5000.0 * (rank + 1) + 0.25, reduce_len=reduce_len)
        total = FlowArena.decode_total(head)
        ok = abs(total - (5000.0 * 3 + 0.5)) < 1e-3
        for i, v in enumerate(arena.views):
            n = v.numel() if i < 2 else 100
            exp = torch.arange(v.numel(), dtype=torch.float32)[:n] * 3 + 2 * i
            ok = ok and torch.equal(v[:n], exp)
        ok = ok and torch.equal(arena.views[2][100:], before_tail)
        # device-scalar form of the flow total
        head = arena.all_reduce(torch.tensor(123456789.0, dtype=torch.float64), reduce_len=64)
        ok = ok and abs(FlowArena.decode_total(head) - 2 * 123456789.0) < 1.0
        open(os.path.join(out_dir, f"rank{rank}.txt"), "w").write("ok" if ok else "bad")
    finally:
        dist.destroy_process_group()


def test_flow_arena_allreduce_world2(tmp_path):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok"


def _avg_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import pyjuice_b200 as pj
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        torch.manual_seed(100 + rank)                              # rank-specific parameters
        ns = pj.structures.HMM(seq_length=5, num_latents=8, num_emits=11)
        ns.init_parameters(perturbation=2.0)
        pc = pj.compile(ns)
        mine = [pc.params.data.clone()] + [l.params.data.clone() for l in pc.input_layer_group]
        exp = []
        for t in mine:
            e = t.clone()
            dist.all_reduce(e)
            exp.append(e / world)
        opt = pj.optim.MiniBatchEM.__new__(pj.optim.MiniBatchEM)   # the optimizer's exchange step alone (no device)
        opt.pc, opt.ddp, opt.ddp_dtype, opt.ddp_group, opt.sync_every, opt._update_count = pc, True, None, None, 3, 0
        opt._post_update_sync(); opt._post_update_sync()           # updates 1 and 2 stay local
        ok = all(torch.equal(a, b) for a, b in zip(mine, [pc.params.data] + [l.params.data for l in pc.input_layer_group]))
        opt._post_update_sync()                                    # update 3: parameters are averaged
        got = [pc.params.data] + [l.params.data for l in pc.input_layer_group]
        ok = ok and all(torch.allclose(a, b, rtol=1e-6, atol=1e-8) for a, b in zip(got, exp))
        ok = ok and not torch.equal(got[0], mine[0])
        eb = pc._em_blocks                                         # a mean of normalised vectors is normalised
        for i in range(eb["par"].numel()):
            p0, fan, bs = int(eb["par"][i]), int(eb["fan"][i]), int(eb["bs"][i])
            sm = pc.params.data[p0:p0 + fan * bs].view(fan, bs).sum(dim=0)
            ok = ok and torch.allclose(sm, torch.ones_like(sm), atol=1e-5)
        open(os.path.join(out_dir, f"rank{rank}.txt"), "w").write("ok" if ok else "bad")
    finally:
        dist.destroy_process_group()


def test_local_sgd_parameter_average_world2(tmp_path):
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_avg_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok"


def test_sync_is_noop_without_process_group():
    import pyjuice_b200 as pj
    ns = pj.structures.HMM(seq_length=4, num_latents=4, num_emits=5)
    pc = pj.compile(ns)
    assert pc.sync_param_flows() is None


def test_arena_layout():
    from pyjuice_b200.flows import FlowArena
    a = FlowArena([10, 70, 5], "cpu")
    assert a.offsets == [64, 128, 256] and a.total == 320
    assert all(v.data_ptr() % 256 == a.buf.data_ptr() % 256 for v in a.views)
    a.views[1].fill_(2.0)
    assert a.buf[128:198].sum().item() == 140.0 and a.buf[:128].sum().item() == 0.0


def _leaver_worker(rank, world, port, out_dir):
    """Rank 1 takes part in the first exchange and then leaves between steps; rank 0 goes on to the next exchange."""
    import datetime
    import time
    sys.path.insert(0, ROOT)
    from pyjuice_b200.flows import FlowArena
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=8))
    arena = FlowArena([256, 64], "cpu")
    for v in arena.views:
        v.fill_(float(rank + 1))
    arena.all_reduce(1.0)                                          # step 1: both ranks
    first_ok = bool(torch.all(arena.views[0] == 3.0))
    if rank == 1:
        open(os.path.join(out_dir, "rank1.txt"), "w").write("left")
        os._exit(0)                                                # leaves without a word, between steps
    before = arena.buf.clone()
    t0 = time.time()
    try:
        arena.all_reduce(1.0)                                      # step 2: the peer is gone
        outcome = "no error"
    except Exception as e:                                         # gloo: connection reset, or the group's timeout
        outcome = f"error:{type(e).__name__}"
    dt = time.time() - t0
    open(os.path.join(out_dir, "rank0.txt"), "w").write(f"{first_ok}|{outcome}|{dt:.1f}|{bool(torch.isfinite(arena.buf).all())}|"
                                                        f"{arena.buf.numel() == before.numel()}")
    os._exit(0)                                                    # the group cannot be torn down collectively any more


def test_a_rank_that_left_ends_the_next_exchange_with_an_error_not_a_hang(tmp_path):
    """Failure detection on the host: a data-parallel rank that exits between steps makes the survivor's next flow
    exchange raise (connection reset, or the process group's timeout at the latest) instead of waiting forever; the
    survivor keeps its flow arena."""
    port = 31500 + (os.getpid() % 2000)
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_leaver_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
        assert not p.is_alive(), "a rank is still waiting for the one that left"
    assert open(tmp_path / "rank1.txt").read() == "left"
    first_ok, outcome, dt, finite, same = open(tmp_path / "rank0.txt").read().split("|")
    assert first_ok == "True" and outcome.startswith("error:"), outcome
    assert float(dt) < 60.0 and finite == "True" and same == "True"
