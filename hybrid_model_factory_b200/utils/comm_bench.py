"""Micro-benchmarks of the fused compute + communication kernels against their NCCL formulations.

    torchrun --nproc-per-node N -m hybrid_model_factory_b200.utils.comm_bench [gemm_ar] [cp_attn] [moe]
    python -m hybrid_model_factory_b200.utils.comm_bench single [gemm_ar] [moe] [sp_scan] [cp_attn]

The ``single`` form runs the same kernels on one GPU with every peer address pointing at that GPU's own buffers
(profiling and smoke testing).

Every number is a CUDA-event time on the launching stream after warm-up, maximum over ranks, inputs larger than L2
or an L2 flush between iterations.  Rank 0 prints one line per case with the roofline bound
``max(FLOPs / measured GEMM peak, NVLink bytes / 770 GB/s)``.
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

LINK_GBS = 770.0     # measured peer copy bandwidth per direction per GPU on this pool


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p["bf16_tflops"], p["hbm_gbs"], "measured"
    except Exception:
        return 1590.0, 6650.0, "fallback"


_flush = None


def timed_graph(fn, reps=20, iters=5):
    """Small ops: ``reps`` calls captured in one CUDA graph, replayed ``iters`` times; returns ms per call (max over
    ranks).  Removes host launch latency from the measurement."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for _ in range(reps):
            fn()
    total = 0.0
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    t = torch.tensor([total / iters / reps], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def timed(fn, iters=10, warmup=3, flush=True):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    total = 0.0
    for _ in range(iters):
        if flush:
            _flush.zero_()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    t = torch.tensor([total / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def report(name, ms_fused, ms_nccl, flops, link_bytes):
    tf, _, src = _peaks()
    bound_ms = max(flops / (tf * 1e9), link_bytes / (LINK_GBS * 1e6))
    if dist.get_rank() == 0:
        print(f"{name}: fused {ms_fused * 1e3:.1f} us, NCCL formulation {ms_nccl * 1e3:.1f} us "
              f"({ms_nccl / ms_fused:.2f}x), roofline bound {bound_ms * 1e3:.1f} us "
              f"({bound_ms / ms_fused:.2f} of {src} bound)", flush=True)


def bench_gemm_ar():
    from ..parallel.tp import TPContext
    tp = TPContext(dist.group.WORLD)
    tp.enable_fused_gemm(max_m=256, max_n=4096)
    n = tp.size
    for M, N, K in ((64, 4096, 4096), (64, 4096, 12288), (16, 4096, 12288), (256, 4096, 4096)):
        Ks = K // n
        x = torch.randn(M, Ks, device="cuda").bfloat16()
        w = (torch.randn(N, Ks, device="cuda") * 0.02).bfloat16()

        def nccl():
            y = F.linear(x, w)
            dist.all_reduce(y)
            return y
        fused = timed_graph(lambda: tp.linear_allreduce(x, w))
        base = timed_graph(nccl)
        # every rank reads the other ranks' bf16 partials of the whole [M, N] result once
        report(f"gemm+all-reduce M={M} N={N} K={K}/{n}", fused, base, 2.0 * M * N * Ks, (n - 1) * M * N * 2.0)


def bench_gemm_rs_ag():
    """GEMM -> reduce-scatter and all-gather -> GEMM (one kernel each) against F.linear + NCCL collectives."""
    from ..ops.fused_comm import PeerAllGatherGemm, PeerGemmAllReduce
    n, rank = dist.get_world_size(), dist.get_rank()
    rs = PeerGemmAllReduce(dist.group.WORLD, max_m=256, max_n=4096)
    ag = PeerAllGatherGemm(dist.group.WORLD, max_m=256, max_ks=4096, max_n=12288)
    os.environ["HMF_TP_NVLS"] = "1"
    nv = PeerGemmAllReduce(dist.group.WORLD, max_m=256, max_n=4096)
    os.environ["HMF_TP_NVLS"] = "0"
    for M, N, K in ((64, 4096, 4096), (64, 4096, 12288), (256, 4096, 4096)):
        Ks = K // n
        x = torch.randn(M, Ks, device="cuda").bfloat16()
        w = (torch.randn(N, Ks, device="cuda") * 0.02).bfloat16()
        out = torch.empty(M, N // n, device="cuda", dtype=torch.bfloat16)

        def nccl_rs():
            y = F.linear(x, w)
            dist.reduce_scatter_tensor(out, y.view(M, n, N // n).transpose(0, 1).contiguous())
            return out
        fused = timed_graph(lambda: rs.reduce_scatter(x, w))
        base = timed_graph(nccl_rs)
        if nv.use_nvls:
            t_nv = timed_graph(lambda: nv(x, w))
            t_nvrs = timed_graph(lambda: nv.reduce_scatter(x, w))
            if rank == 0:
                print(f"  NVLS (multimem.ld_reduce) M={M} N={N} K={K}/{n}: all-reduce {t_nv * 1e3:.1f} us, "
                      f"reduce-scatter {t_nvrs * 1e3:.1f} us", flush=True)
        # every rank reads the other ranks' bf16 partials of its own N / n columns once
        report(f"gemm+reduce-scatter M={M} N={N} K={K}/{n}", fused, base, 2.0 * M * N * Ks, (n - 1) * M * (N // n) * 2.0)
    for M, N, K in ((64, 12288, 4096), (64, 4096, 4096), (256, 12288, 4096)):
        Ks, Nl = K // n, N // n
        xs = torch.randn(M, Ks, device="cuda").bfloat16()
        w = (torch.randn(Nl, K, device="cuda") * 0.02).bfloat16()
        gathered = torch.empty(n, M, Ks, device="cuda", dtype=torch.bfloat16)

        def nccl_ag():
            dist.all_gather_into_tensor(gathered, xs)
            return F.linear(gathered.permute(1, 0, 2).reshape(M, K), w)
        fused = timed(lambda: ag(xs, w), iters=20, flush=False)
        base = timed(nccl_ag, iters=20, flush=False)
        report(f"all-gather+gemm M={M} N={N}/{n} K={K}", fused, base, 2.0 * M * Nl * K, (n - 1) * M * Ks * 2.0)


def bench_cp_attn():
    from ..parallel.cp_attention import cp_attention
    from ..parallel.peer import enable_peer_kv
    from ..parallel.sp import init_sp_group
    n = dist.get_world_size()
    sp = init_sp_group(n)
    T, H, Hkv, D = int(os.environ.get("HMF_CP_TOKENS", 131072)) // n, 32, 8, 128
    q = torch.randn(1, T, H, D, device="cuda").bfloat16()
    k = torch.randn(1, T, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(1, T, Hkv, D, device="cuda").bfloat16()
    with torch.no_grad():
        base = timed(lambda: cp_attention(q, k, v, sp), iters=5)
        enable_peer_kv(sp, k.numel() * 2)
        fused = timed(lambda: cp_attention(q, k, v, sp), iters=5)
    Tg = T * n
    flops = 4.0 * Tg * Tg / 2 * H * D / n                       # causal, this rank's share (zig-zag balanced)
    link = (n - 1) / n * Tg * Hkv * D * 2 * 2.0                  # remote K and V read once
    report(f"context-parallel attention fwd, {Tg} tokens over {n} GPUs", fused, base, flops, link)


def bench_moe():
    from ..ops import reference as R
    from ..parallel.ep import EPContext, ep_experts_forward
    from ..parallel.ep_fused import FusedExpertParallel
    n, rank = dist.get_world_size(), dist.get_rank()
    E, Dm, Fi, T, k = 64, 2048, 768, 8192, 8
    per = E // n
    g = torch.Generator().manual_seed(0)
    wgu = (torch.randn(per, 2 * Fi, Dm, generator=g) * 0.02).bfloat16().cuda()
    wd = (torch.randn(per, Dm, Fi, generator=g) * 0.02).bfloat16().cuda()
    x = torch.randn(T, Dm, device="cuda").bfloat16()
    w, idx = R.moe_router(torch.randn(T, E, device="cuda"), k)
    ep = EPContext.from_group(dist.group.WORLD)
    fe = FusedExpertParallel(dist.group.WORLD, per, Dm, Fi, max_send_rows=T * k, capacity_rows=2 * T * k)
    with torch.no_grad():
        base = timed(lambda: ep_experts_forward(x, wgu, wd, w.to(x.dtype), idx, ep), iters=5)
        fused = timed(lambda: fe.forward(x, w, idx, wgu, wd), iters=5)
    flops = 2.0 * T * k * Dm * Fi * 3
    link = (n - 1) / n * T * k * Dm * 2 * 2.0                     # dispatch + combine
    report(f"MoE layer E={E} top-{k} T={T} Dm={Dm} F={Fi}, EP={n}", fused, base, flops, link)


CASES = {"gemm_ar": bench_gemm_ar, "gemm_rs_ag": bench_gemm_rs_ag, "cp_attn": bench_cp_attn, "moe": bench_moe}


# -- one GPU: every "peer" address is one of this GPU's own buffers ---------------------------------------------------
# Same kernels, same flag protocol, no NVLink traffic: the mode the kernels are profiled in (a profiler replays each
# launch many times, which a kernel that waits for another process cannot survive) and a smoke test of each path.
def _event_ms(fn, iters=5, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def single_gemm_ar():
    from ..ops.fused_comm import PeerGemmAllReduce
    op = PeerGemmAllReduce(None, max_m=256, max_n=4096)
    M, N, K = 64, 4096, 12288
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
    ms = _event_ms(lambda: op(x, w))
    err = float((op(x, w).float() - x.float() @ w.float().t()).abs().max())
    print(f"single-GPU gemm+all-reduce M={M} N={N} K={K}: {ms * 1e3:.1f} us, max abs err {err:.3g} "
          f"({N * K * 2 / ms / 1e6:.0f} GB/s of weights)", flush=True)


def single_moe():
    from ..ops import reference as R
    from ..parallel.ep_fused import FusedExpertParallel
    E, Dm, Fi, T, k = 64, 2048, 768, 8192, 8
    g = torch.Generator().manual_seed(0)
    wgu = (torch.randn(E, 2 * Fi, Dm, generator=g) * 0.02).bfloat16().cuda()
    wd = (torch.randn(E, Dm, Fi, generator=g) * 0.02).bfloat16().cuda()
    x = torch.randn(T, Dm, device="cuda").bfloat16()
    w, idx = R.moe_router(torch.randn(T, E, device="cuda"), k)
    fe = FusedExpertParallel(None, E, Dm, Fi, max_send_rows=T * k, capacity_rows=T * k)
    with torch.no_grad():
        ms = _event_ms(lambda: fe.forward(x, w, idx, wgu, wd))
    flops = 2.0 * T * k * Dm * Fi * 3
    print(f"single-GPU MoE layer E={E} top-{k} T={T} Dm={Dm} F={Fi}: {ms:.3f} ms ({flops / ms / 1e9:.0f} TFLOP/s over "
          f"the whole layer, routing tables included)", flush=True)


def single_sp_scan():
    """Two launches of the GDN scan standing for SP ranks 0 and 1: the first pushes its final state and raises the
    per-(batch, head) flags in a buffer, the second starts from that buffer after seeing the flags."""
    from ..ops.gdn_cuda import GDNChunkCore
    from ..parallel.peer import PeerIO
    B, T, H, D = 1, 16384, 32, 128
    q, k, v = (torch.randn(B, T, H, D, device="cuda").bfloat16() for _ in range(3))
    g = -torch.rand(B, T, H, device="cuda") * 0.1
    beta = torch.rand(B, T, H, device="cuda")
    core = GDNChunkCore(scale=D ** -0.5)
    buf = torch.zeros(B, H, D, D, device="cuda", dtype=torch.float32)
    flags = torch.zeros(B * H, device="cuda", dtype=torch.int32)
    epoch = [0]

    def chain():
        epoch[0] += 1
        o0, (h_mid,), _, _ = core.forward((q, k, v, g, beta), None,
                                          PeerIO(None, None, buf.data_ptr(), flags.data_ptr(), epoch[0]))
        o1, (h_end,), _, _ = core.forward((q, k, v, g, beta), None, PeerIO(buf, flags, 0, 0, epoch[0]))
        return o0, o1, h_mid, h_end
    with torch.no_grad():
        ms = _event_ms(chain)
        o0, o1, h_mid, h_end = chain()
        ref1, (ref_end,), _, _ = core.forward((q, k, v, g, beta), (h_mid,), None)
    err = float((o1.float() - ref1.float()).abs().max())
    print(f"single-GPU SP scan chain (2 segments of {T} tokens, {H} heads): {ms:.3f} ms for both launches, pushed "
          f"state vs local state: max abs diff of the outputs {err:.3g}", flush=True)


def single_cp_attn():
    from ..ops import cuda_ops
    from ..parallel.peer import PeerKVExchange
    T, H, Hkv, D = 16384, 32, 8, 128
    q = torch.randn(1, T, H, D, device="cuda").bfloat16()
    k = torch.randn(1, T, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(1, T, Hkv, D, device="cuda").bfloat16()
    kv = PeerKVExchange(None, 0, 1, k.numel() * 2)
    Lc = T // 2

    def run():
        kv.publish(k, v)
        return kv.attention(q[:, Lc:], 1, D ** -0.5, 0, 2 ** 31 - 1)
    with torch.no_grad():
        ms = _event_ms(run)
        o, _ = run()
        ref = cuda_ops.attention(q, k, v, causal=True)[:, Lc:]
    err = float((o.float() - ref.float()).abs().max())
    flops = 4.0 * Lc * (Lc + Lc / 2) * H * D
    print(f"single-GPU CP attention (second half of {T} tokens, K/V fetched through the exchange buffers): {ms:.3f} ms "
          f"({flops / ms / 1e9:.0f} TFLOP/s), max abs err vs the plain kernel {err:.3g}", flush=True)


SINGLE = {"gemm_ar": single_gemm_ar, "moe": single_moe, "sp_scan": single_sp_scan, "cp_attn": single_cp_attn}


def main(argv=None) -> int:
    args = list(argv if argv is not None else sys.argv[1:])
    if "single" in args:
        from ..ops import _lib
        torch.cuda.set_device(0)
        for name in [a for a in args if a in SINGLE] or list(SINGLE):
            SINGLE[name]()
        torch.cuda.synchronize()
        print("kernel status", _lib.read_status())
        return 0
    names = [a for a in args if a in CASES] or list(CASES)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    for name in names:
        CASES[name]()
    from ..ops import _lib
    torch.cuda.synchronize()
    if dist.get_rank() == 0:
        print("kernel status", _lib.read_status())
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
