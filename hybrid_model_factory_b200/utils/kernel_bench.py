"""Kernel microbenchmarks with roofline fractions.

    python -m hybrid_model_factory_b200.utils.kernel_bench attention_fwd --seq 16384
    python -m hybrid_model_factory_b200.utils.kernel_bench all

Each case is timed with CUDA events on the launching stream after warm-up (inputs are larger
than the 126 MB L2, or an L2-sized buffer is rewritten between iterations), and reported as
achieved TFLOP/s or GB/s and as a fraction of the measured peaks of this machine
(``MEASURED_PEAKS.json`` at the repository root when present, else the documented fallback of
6.65 TB/s and 1.59 PFLOP/s).  The same commands are what the ``profiles/`` summaries were
captured from under ``ncu``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "src": "fallback"}


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def time_fn(fn, iters=5, warmup=3, flush=True):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def report(name, ms, flops=None, bytes_=None):
    pk = peaks()
    line = f"{name}: {ms:.3f} ms"
    if flops:
        tf = flops / ms / 1e9
        line += f"  {tf:.0f} TFLOP/s ({tf / pk['tflops']:.2f} of {pk['src']} cuBLAS bf16 peak)"
    if bytes_:
        gbs = bytes_ / ms / 1e6
        line += f"  {gbs:.0f} GB/s ({gbs / pk['hbm_gbs']:.2f} of {pk['src']} copy bandwidth)"
    print(line, flush=True)


def bench_gemm_skinny(args):
    """Decode-sized projections: the swap-AB kernel against the vendor library, weights cold in L2 (flushed between
    iterations; the weight read is the algorithmic traffic)."""
    import torch.nn.functional as F
    from ..ops.gemm import skinny_gemm
    shapes = ((4096, 4096), (6144, 4096), (10368, 4096), (24576, 4096), (4096, 12288), (151936, 4096))
    rows = (1, 16, 64)
    if args.skinny_shape:                  # "N,K,M": one case (profiler captures)
        n, k, m = (int(v) for v in args.skinny_shape.split(","))
        shapes, rows = ((n, k),), (m,)
    for N, K in shapes:
        w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
        for M in rows:
            x = torch.randn(M, K, device="cuda").bfloat16()
            ms = time_fn(lambda: skinny_gemm(x, w), iters=10)
            ms_lib = time_fn(lambda: F.linear(x, w), iters=10)
            report(f"skinny gemm M={M} N={N} K={K}", ms, bytes_=2.0 * N * K)
            report(f"  library     M={M} N={N} K={K}", ms_lib, bytes_=2.0 * N * K)
        del w


def bench_gka_prep(args):
    """GKA input preparation (q / k normalisation, beta gate): fused kernels against the eager formulation."""
    from ..ops import cuda_ops
    from ..ops import reference as R
    T, H, D = args.seq, args.heads, 128
    q, k, v = (torch.randn(1, T, H, D, device="cuda").bfloat16() for _ in range(3))
    beta = torch.rand(1, T, H, device="cuda").bfloat16()
    nbytes = 6.0 * T * H * D * 2
    ms = time_fn(lambda: cuda_ops.gka_prepare(q, k, v, beta, 1e-6), iters=10)
    report(f"gka_prepare kernel T={T} H={H} D={D}", ms, bytes_=nbytes)
    ms = time_fn(lambda: R.gka_prepare(q, k, v, beta, 1e-6), iters=5)
    report(f"gka_prepare eager PyTorch T={T} H={H} D={D}", ms, bytes_=nbytes)
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    outs = cuda_ops.gka_prepare(qg, kg, vg, beta, 1e-6)
    gs = [torch.randn_like(o) for o in outs]
    ms = time_fn(lambda: torch.autograd.grad(outs, (qg, kg, vg), gs, retain_graph=True), iters=10)
    report(f"gka_prepare backward kernel T={T} H={H} D={D}", ms, bytes_=9.0 * T * H * D * 2)


def bench_gemm(args):
    from ..ops.gemm import gemm
    M = N = K = args.size
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    report(f"gemm_bf16 {M}^3 (one CTA per tile)", time_fn(lambda: gemm(a, b, out=out, pair=False)), flops=2.0 * M * N * K)
    report(f"gemm_bf16 {M}^3 (CTA pair per tile)", time_fn(lambda: gemm(a, b, out=out, pair=True)), flops=2.0 * M * N * K)
    report(f"torch.matmul (cuBLAS) {M}^3", time_fn(lambda: torch.matmul(a, b.t(), out=out)), flops=2.0 * M * N * K)


def bench_gemm_step(args):
    """The projection GEMMs of one Qwen3-8B decoder layer at ``--seq`` tokens: forward, input gradient and weight
    gradient of [hidden 4096 -> 4096], [4096 -> 12288], [12288 -> 4096], [4096 -> 1024], own kernel against cuBLAS."""
    from ..ops.gemm import gemm
    T = args.seq
    for n_out, k_in in ((4096, 4096), (12288, 4096), (4096, 12288), (1024, 4096)):
        x = torch.randn(T, k_in, device="cuda").bfloat16()
        w = torch.randn(n_out, k_in, device="cuda").bfloat16()
        dy = torch.randn(T, n_out, device="cuda").bfloat16()
        fl = 2.0 * T * n_out * k_in
        cases = (("fwd  ", lambda: gemm(x, w), lambda: torch.matmul(x, w.t())),
                 ("dgrad", lambda: gemm(dy, w, b_mn_major=True), lambda: torch.matmul(dy, w)),
                 ("wgrad", lambda: gemm(dy, x, a_mn_major=True, b_mn_major=True), lambda: torch.matmul(dy.t(), x)))
        for name, own, lib in cases:
            a, b = time_fn(own, flush=False), time_fn(lib, flush=False)
            os.environ["HMF_GEMM_PAIR"] = "0"
            a1 = time_fn(own, flush=False)
            os.environ["HMF_GEMM_PAIR"] = "1"
            name = f"{name} [1-CTA {a1:.3f} ms]"
            tf = fl / a / 1e9
            print(f"gemm {name} T={T} {k_in}->{n_out}: own {a:.3f} ms ({tf:.0f} TFLOP/s)  cuBLAS {b:.3f} ms "
                  f"({fl / b / 1e9:.0f} TFLOP/s)  own/cuBLAS time {a / b:.2f}", flush=True)


def bench_gemm_fp8(args):
    """Row-wise scaled float8 GEMM and its quantisers against the bf16 CTA-pair GEMM, layer shapes at ``--seq`` tokens."""
    from ..ops import fp8
    from ..ops.gemm import gemm
    T = args.seq
    for n_out, k_in in ((4096, 4096), (12288, 4096), (4096, 12288)):
        x = torch.randn(T, k_in, device="cuda").bfloat16()
        w = torch.randn(n_out, k_in, device="cuda").bfloat16()
        xq, sx = fp8.quant_rows(x)
        wq, sw = fp8.quant_rows(w)
        a = time_fn(lambda: fp8.gemm_fp8(xq, sx, wq, sw), flush=False)
        b = time_fn(lambda: gemm(x, w), flush=False)
        q = time_fn(lambda: fp8.quant_rows(x), flush=False)
        qt = time_fn(lambda: fp8.quant_cols_t(x), flush=False)
        fl = 2.0 * T * n_out * k_in
        print(f"fp8 gemm T={T} {k_in}->{n_out}: {a:.3f} ms ({fl / a / 1e9:.0f} TFLOP/s)  bf16 pair gemm {b:.3f} ms "
              f"({fl / b / 1e9:.0f} TFLOP/s)  quant_rows(x) {q:.3f} ms  quant_cols_t(x) {qt:.3f} ms", flush=True)


def _qkv(T, H, Hkv, D):
    q = torch.randn(1, T, H, D, device="cuda").bfloat16()
    k = torch.randn(1, T, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(1, T, Hkv, D, device="cuda").bfloat16()
    return q, k, v


def bench_attention_fwd(args):
    from ..ops import cuda_ops
    T, H, Hkv, D = args.seq, args.heads, args.kv_heads, 128
    q, k, v = _qkv(T, H, Hkv, D)
    ms = time_fn(lambda: cuda_ops.attention_fwd_raw(q, k, v, D ** -0.5, 0, 2 ** 31 - 1, 0), flush=False)
    report(f"attention_fwd causal T={T} H={H}/{Hkv} D={D}", ms, flops=4.0 * T * T * H * D / 2)


def bench_attention_bwd(args):
    from ..ops import cuda_ops
    T, H, Hkv, D = args.seq, args.heads, args.kv_heads, 128
    q, k, v = _qkv(T, H, Hkv, D)
    o, lse = cuda_ops.attention_fwd_raw(q, k, v, D ** -0.5, 0, 2 ** 31 - 1, 0)
    do = torch.randn_like(o)
    for det, name in ((False, "fused kernel"), (True, "dQ + dK/dV kernels")):
        ms = time_fn(lambda: cuda_ops.attention_bwd_raw(q, k, v, o, do, lse, D ** -0.5, 0, 2 ** 31 - 1, 0,
                                                        deterministic=det), flush=False)
        report(f"attention_bwd {name} causal T={T} H={H}/{Hkv} D={D} (5-GEMM flop count)", ms,
               flops=10.0 * T * T * H * D / 2)


def _gdn_inputs(T, H):
    q = torch.randn(1, T, H, 128, device="cuda").bfloat16()
    k = torch.randn(1, T, H, 128, device="cuda").bfloat16()
    v = torch.randn(1, T, H, 128, device="cuda").bfloat16()
    g = -torch.rand(1, T, H, device="cuda") * 0.1
    beta = torch.rand(1, T, H, device="cuda")
    return q, k, v, g, beta


def bench_gdn_fwd(args):
    from ..ops import mixers
    T, H = args.seq, args.heads
    q, k, v, g, beta = _gdn_inputs(T, H)
    with torch.no_grad():
        ms = time_fn(lambda: mixers.gated_delta_rule(q, k, v, g, beta), flush=False)
    io = 4 * T * H * 128 * 2  # q, k, v in; o out
    report(f"gdn_fwd (prep + scan) T={T} H={H}", ms, bytes_=io)


def bench_gdn_fwd_bwd(args):
    from ..ops import mixers
    T, H = args.seq, args.heads
    leaves = [t.requires_grad_(True) for t in _gdn_inputs(T, H)]

    def step():
        o, _ = mixers.gated_delta_rule(*leaves)
        o.backward(torch.ones_like(o))
    report(f"gdn_fwd_bwd T={T} H={H}", time_fn(step, flush=False))


def bench_gka_cheb(args):
    """Chebyshev ridge solve of Gated KalmaNet: the one-kernel solve and the batched fp32 PyTorch formulation."""
    from ..ops import gka_parallel as GP
    T, H, D = args.seq, args.heads, 128
    q = torch.randn(1, T, H, D, device="cuda").bfloat16()
    k = torch.nn.functional.normalize(torch.randn(1, T, H, D, device="cuda"), dim=-1).bfloat16()
    gk = -torch.rand(1, T, H, device="cuda") * 0.1
    iters = 30
    flops = 2.0 * T * H * iters * (64 * 128 + 64 * 128 + 128 * 128)
    with torch.no_grad():
        ms = time_fn(lambda: GP.chebyshev_chunk_parallel(q, k, gk, num_iter=iters), flush=False)
        report(f"gka_cheb kernel T={T} H={H} iters={iters}", ms, flops=flops)
        qf, kf = q.float(), k.float()
        ms = time_fn(lambda: GP.chebyshev_chunk_parallel(qf, kf, gk, num_iter=iters), iters=2, warmup=1, flush=False)
        report(f"gka_cheb batched PyTorch fp32 T={T} H={H} iters={iters}", ms, flops=flops)


def bench_rmsnorm(args):
    from ..ops import functional as F_ops
    N, D = args.seq * 8, 4096
    x = torch.randn(N, D, device="cuda").bfloat16()
    w = torch.ones(D, device="cuda").bfloat16()
    with torch.no_grad():
        ms = time_fn(lambda: F_ops.rms_norm(x, w, 1e-6))
    report(f"rms_norm [{N}, {D}]", ms, bytes_=2.0 * N * D * 2)


def bench_swiglu(args):
    from ..ops import functional as F_ops
    N, D = args.seq, 12288
    g = torch.randn(N, D, device="cuda").bfloat16()
    u = torch.randn(N, D, device="cuda").bfloat16()
    with torch.no_grad():
        ms = time_fn(lambda: F_ops.swiglu(g, u))
    report(f"swiglu [{N}, {D}]", ms, bytes_=3.0 * N * D * 2)


def bench_conv1d(args):
    from ..ops import functional as F_ops
    T, Cc = args.seq, 6144
    x = torch.randn(1, T, Cc, device="cuda").bfloat16()
    w = torch.randn(Cc, 4, device="cuda").bfloat16()
    with torch.no_grad():
        ms = time_fn(lambda: F_ops.causal_conv1d(x, w, None, "silu"))
    report(f"causal_conv1d+silu [1, {T}, {Cc}]", ms, bytes_=2.0 * T * Cc * 2)


def bench_paged_decode(args):
    """Decode-step paged attention: ``--batch`` requests of ``--seq`` cached tokens each, block size 64."""
    import ctypes as ct
    from ..ops import _lib
    K = _lib.kernels()
    Rn, H, Hkv, D, bs, L = args.batch, args.heads, args.kv_heads, 128, 64, args.seq
    mb = (L + bs - 1) // bs
    nb = Rn * mb
    kc = torch.randn(nb, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(nb, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    bt = torch.randperm(nb, device="cuda").to(torch.int32).view(Rn, mb).contiguous()
    lens = torch.full((Rn,), L, dtype=torch.int32, device="cuda")
    q = torch.randn(Rn, H, D, device="cuda", dtype=torch.bfloat16)
    o = torch.empty_like(q)
    for splits in (1, 2, 4, 8, 16):
        po = torch.empty(Rn, H, splits, D, device="cuda", dtype=torch.float32)
        pml = torch.empty(Rn, H, splits, 2, device="cuda", dtype=torch.float32)

        def run():
            _lib.check(K.hmf_paged_attention_decode_tc(
                _lib.ptr(q), _lib.ptr(kc), _lib.ptr(vc), _lib.ptr(bt), _lib.ptr(lens), _lib.ptr(o), _lib.ptr(po),
                _lib.ptr(pml), ct.c_int(Rn), ct.c_int(H), ct.c_int(Hkv), ct.c_int(D), ct.c_int(bs), ct.c_int(nb),
                ct.c_int(mb), ct.c_int(splits), ct.c_int(0), ct.c_float(D ** -0.5), _lib.stream_ptr(q.device)), "pa")
        ms = time_fn(run, flush=(kc.numel() * 4 < (256 << 20)))
        report(f"paged_attention_decode_tc R={Rn} L={L} Hq={H} Hkv={Hkv} splits={splits}", ms,
               bytes_=2.0 * Rn * L * Hkv * D * 2)


CASES = {"gka_prep": bench_gka_prep, "gemm_skinny": bench_gemm_skinny, "gemm_step": bench_gemm_step, "gemm_fp8": bench_gemm_fp8, "gka_cheb": bench_gka_cheb, "paged_decode": bench_paged_decode, "gemm": bench_gemm, "attention_fwd": bench_attention_fwd, "attention_bwd": bench_attention_bwd,
         "gdn_fwd": bench_gdn_fwd, "gdn_fwd_bwd": bench_gdn_fwd_bwd, "rmsnorm": bench_rmsnorm, "swiglu": bench_swiglu,
         "conv1d": bench_conv1d}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=list(CASES) + ["all"])
    ap.add_argument("--seq", type=int, default=16384)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--size", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--skinny-shape", default=None, help="gemm_skinny: N,K,M of a single case")
    args = ap.parse_args(argv)
    names = list(CASES) if args.case == "all" else [args.case]
    for n in names:
        CASES[n](args)
    from ..ops import _lib
    print("kernel status", _lib.read_status())


if __name__ == "__main__":
    sys.exit(main())
