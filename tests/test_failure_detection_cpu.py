"""Failure detection without touching a GPU: gloo ranks on the CPU, failures made on the host
(a rank that raises, a rank that leaves, a rank that never joins, mismatched signatures)."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, world, port, timeout_s=20):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s))


def _raising_worker(rank, world, port, store_port, out):
    from rl_kernel_b200.distributed.algorithms.collectives import TorchDistributedDeterministicCollective
    from rl_kernel_b200.distributed.health import PeerFailure, PeerMonitor

    _init(rank, world, port)
    store = dist.TCPStore("127.0.0.1", store_port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20))
    mon = PeerMonitor(store, rank, world, timeout_s=10, max_lag=0)
    coll = TorchDistributedDeterministicCollective()
    seen = None
    try:
        for step in range(4):
            with mon.step(step):
                x = torch.full((4,), float(rank + step))
                coll.all_reduce_(x)
                if rank == 1 and step == 2:
                    # the step's collective is done, nothing is in flight: fail on the host
                    raise RuntimeError("injected host failure")
    except PeerFailure as e:
        seen = ("peer", e.rank, e.reason)
    except RuntimeError as e:
        seen = ("self", rank, str(e))
    torch.save(seen, f"{out}.{rank}")
    time_to_linger = 0.5                      # keep the store's host alive until the peer has read it
    import time
    time.sleep(time_to_linger)
    dist.destroy_process_group()


def test_rank_that_raises_is_seen_by_its_peer_before_the_next_collective(tmp_path):
    out = str(tmp_path / "r")
    mp.spawn(_raising_worker, args=(2, _port(), _port(), out), nprocs=2, join=True)
    r0, r1 = torch.load(f"{out}.0"), torch.load(f"{out}.1")
    assert r1[0] == "self" and "injected" in r1[2]
    assert r0[0] == "peer" and r0[1] == 1 and "injected host failure" in r0[2]


def _leaving_worker(rank, world, port, store_port, out):
    from rl_kernel_b200.distributed.health import PeerFailure, PeerMonitor

    _init(rank, world, port)
    store = dist.TCPStore("127.0.0.1", store_port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20))
    mon = PeerMonitor(store, rank, world, timeout_s=1.0, max_lag=0)
    seen = "none"
    import time
    try:
        for step in range(3):
            if rank == 1 and step == 1:
                mon.leave("scaled down")
                break
            with mon.step(step):
                pass
    except PeerFailure as e:
        seen = e.reason
    torch.save(seen, f"{out}.{rank}")
    time.sleep(0.5)
    dist.destroy_process_group()


def test_rank_that_leaves_between_steps_is_reported(tmp_path):
    out = str(tmp_path / "l")
    mp.spawn(_leaving_worker, args=(2, _port(), _port(), out), nprocs=2, join=True)
    assert "left" in torch.load(f"{out}.0") and "scaled down" in torch.load(f"{out}.0")


def _stalled_worker(rank, world, port, store_port, out):
    from rl_kernel_b200.distributed.health import PeerFailure, PeerMonitor

    _init(rank, world, port)
    store = dist.TCPStore("127.0.0.1", store_port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20))
    mon = PeerMonitor(store, rank, world, timeout_s=0.6, max_lag=0)
    import time
    seen = "none"
    try:
        with mon.step(0):
            pass
        if rank == 1:
            time.sleep(2.0)                   # never reaches step 1 in time
        else:
            with mon.step(1):
                pass
            with mon.step(2):
                pass
    except PeerFailure as e:
        seen = e.reason
    torch.save(seen, f"{out}.{rank}")
    time.sleep(0.3 if rank == 1 else 2.0)
    dist.destroy_process_group()


def test_stalled_rank_times_out_on_the_host(tmp_path):
    out = str(tmp_path / "s")
    mp.spawn(_stalled_worker, args=(2, _port(), _port(), out), nprocs=2, join=True)
    assert "no progress" in torch.load(f"{out}.0")


def _mismatch_worker(rank, world, port, out):
    from rl_kernel_b200.distributed.algorithms.collectives import TorchDistributedDeterministicCollective

    _init(rank, world, port)
    coll = TorchDistributedDeterministicCollective()
    err = ""
    try:
        coll.all_reduce_(torch.zeros(4 if rank == 0 else 8))
    except ValueError as e:
        err = str(e)
    torch.save(err, f"{out}.{rank}")
    dist.destroy_process_group()


def test_signature_mismatch_fails_closed_on_every_rank(tmp_path):
    out = str(tmp_path / "m")
    mp.spawn(_mismatch_worker, args=(2, _port(), out), nprocs=2, join=True)
    for r in range(2):
        assert "signature mismatch" in torch.load(f"{out}.{r}")


def _absent_worker(rank, world, port, out):
    """Rank 1 never joins the collective: the short process-group timeout ends rank 0's call with
    an error instead of a hang."""
    _init(rank, world, port, timeout_s=2)
    err = "none"
    if rank == 0:
        try:
            dist.all_reduce(torch.zeros(4))
        except Exception as e:       # gloo raises a RuntimeError subclass with a timeout message
            err = type(e).__name__
    else:
        import time
        time.sleep(4.0)
    torch.save(err, f"{out}.{rank}")
    os._exit(0)                      # the group is broken by design; skip the orderly teardown


def test_collective_with_an_absent_rank_ends_with_an_error(tmp_path):
    out = str(tmp_path / "a")
    mp.spawn(_absent_worker, args=(2, _port(), out), nprocs=2, join=True)
    assert torch.load(f"{out}.0") != "none"
