"""Helpers to run a function on several CPU ranks (gloo) inside a test."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, errq, backend="gloo"):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"], os.environ["WORLD_SIZE"] = str(rank), str(world)
    os.environ["LOCAL_RANK"] = str(rank)
    torch.set_num_threads(2)
    dump_after = float(os.environ.get("HMF_TEST_DUMP_AFTER_S", "0"))
    if dump_after > 0:          # a rank still running by then prints every thread's stack (shows where it waits)
        import faulthandler
        faulthandler.dump_traceback_later(dump_after, exit=False)
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
            import datetime
            # a rank that failed never joins the others' next collective: let that collective give up in minutes
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                                    timeout=datetime.timedelta(seconds=180))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
        fn(rank, world, *args)
        dist.barrier()
    except Exception:
        errq.put((rank, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_ranks(fn, world: int, *args, timeout: float = 300.0, backend: str = "gloo"):
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, errq, backend)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
    errors = []
    while not errq.empty():
        errors.append(errq.get())
    # a rank that failed leaves the others waiting in their next collective: show its error with the timeout
    assert not alive, f"{len(alive)} rank(s) timed out" + "".join(f"\n[rank {r}]\n{tb}" for r, tb in errors)
    assert not errors, "\n".join(f"[rank {r}]\n{tb}" for r, tb in errors)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
