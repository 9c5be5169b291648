"""Failure detection and signalling-protocol checks.  All failures are made on the host (CPU ranks, a dropped
message in the protocol model); no GPU is faulted."""
import os
import time

import pytest
import torch
import torch.distributed as dist

from dist_utils import run_ranks
from hybrid_model_factory_b200.parallel import protocol_model as pm
from hybrid_model_factory_b200.utils.health import Heartbeat, PeerFailure


@pytest.mark.parametrize("world", [2, 4])
def test_protocols_have_no_premature_overwrite_or_deadlock(world):
    for make in (pm.sp_chain_program, pm.gemm_allreduce_program):
        res = pm.simulate([make(r, world, 4) for r in range(world)], trials=100)
        assert res.ok and not res.timeouts, res.violations[:3]


def test_dropped_flag_ends_in_bounded_timeouts_not_a_hang():
    progs = [pm.sp_chain_program(r, 3, 2) for r in range(3)]
    res = pm.simulate(progs, trials=20, drop=(0, 0))       # rank 0 never signals its first state
    assert res.timeouts and all(ev[0] == "wait" for _, ev in res.timeouts)


def test_single_buffered_allreduce_would_be_caught():
    def bad(rank, world, epochs):          # same protocol without the parity double-buffer
        return [(k, n.split(".")[0] + ".x" if k in ("write", "read") else n, e)
                for k, n, e in pm.gemm_allreduce_program(rank, world, epochs)]
    res = pm.simulate([bad(r, 2, 3) for r in range(2)], trials=300)
    assert not res.ok


def _hb_worker(rank, world, mode):
    from torch.distributed.distributed_c10d import _get_default_store
    hb = Heartbeat(_get_default_store(), rank, world, timeout_s=2.0)
    x = torch.ones(4)
    for step in range(1, 4):
        if mode == "raise" and rank == 1 and step == 2:
            hb.fail("exception in step 2")
            return                          # leaves between steps, nothing in flight
        if mode == "vanish" and rank == 1 and step == 2:
            return                          # exits silently: no heartbeat any more
        hb.beat(step)
        try:
            hb.wait_for_peers(step)
        except PeerFailure as e:
            assert e.ranks == [1] and rank == 0 and step == 2
            return
        dist.all_reduce(x)
    assert mode == "ok"


@pytest.mark.parametrize("mode", ["ok", "raise", "vanish"])
def test_heartbeat_detects_a_lost_rank_before_the_next_collective(mode):
    # the surviving rank must not enter the collective of the step the peer never reached
    run_ranks(_hb_worker_nobarrier, 2, mode, timeout=60)


def _hb_worker_nobarrier(rank, world, mode):
    _hb_worker(rank, world, mode)
    if mode != "ok":
        os._exit(0)         # skip the helper's final barrier: one rank is gone by design


@pytest.mark.gpu
def test_device_wait_runs_out_and_reports_status():
    """A device-side wait on a flag that nothing sets ends by its time limit with an error status; a later
    launch on the same context works."""
    import ctypes
    from hybrid_model_factory_b200.ops import _lib
    K = _lib.kernels()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    res = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    _lib.read_status(reset=True)
    t0 = time.time()
    _lib.check(K.hmf_wait_probe(_lib.ptr(flag), ctypes.c_uint(1), ctypes.c_ulonglong(50_000_000), _lib.ptr(res),
                                _lib.stream_ptr(flag.device)), "wait_probe")
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0 and int(res) == 0
    code, _, detail, count = _lib.read_status(reset=True)
    assert code == 2 and detail == 0x900 and count == 1          # kFlagTimeout at the probe's wait site
    flag.fill_(3)
    _lib.check(K.hmf_wait_probe(_lib.ptr(flag), ctypes.c_uint(1), ctypes.c_ulonglong(50_000_000), _lib.ptr(res),
                                _lib.stream_ptr(flag.device)), "wait_probe")
    torch.cuda.synchronize()
    assert int(res) == 1 and _lib.read_status()[0] == 0
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0
