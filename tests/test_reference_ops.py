"""Chunk-parallel reference forms agree with their token-by-token definitions (CPU, fp32)."""
import torch

from hybrid_model_factory_b200.ops import reference as R


def _rand(B=2, T=150, H=3, D=16, Dv=16):
    q = torch.randn(B, T, H, D)
    k = torch.randn(B, T, H, D)
    v = torch.randn(B, T, H, Dv)
    g = -torch.rand(B, T, H) * 0.2
    beta = torch.rand(B, T, H)
    return q, k, v, g, beta


def test_gdn_chunk_matches_recurrent():
    q, k, v, g, beta = _rand()
    h0 = torch.randn(2, 3, 16, 16) * 0.1
    o1, s1 = R.gated_delta_rule_recurrent(q, k, v, g, beta, initial_state=h0)
    o2, s2 = R.gated_delta_rule_chunk(q, k, v, g, beta, initial_state=h0, chunk_size=64)
    torch.testing.assert_close(o1, o2, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(s1, s2, rtol=1e-4, atol=1e-5)


def test_gdn_state_split_equals_full():
    q, k, v, g, beta = _rand(T=128)
    o, s = R.gated_delta_rule_chunk(q, k, v, g, beta)
    o_a, s_a = R.gated_delta_rule_chunk(q[:, :64], k[:, :64], v[:, :64], g[:, :64], beta[:, :64])
    o_b, s_b = R.gated_delta_rule_chunk(q[:, 64:], k[:, 64:], v[:, 64:], g[:, 64:], beta[:, 64:], initial_state=s_a)
    torch.testing.assert_close(torch.cat([o_a, o_b], 1), o, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(s_b, s, rtol=1e-4, atol=1e-5)


def test_gla_chunk_matches_recurrent():
    q, k, v, g, _ = _rand()
    o1, s1 = R.simple_gla_recurrent(q, k, v, g)
    o2, s2 = R.simple_gla_chunk(q, k, v, g, chunk_size=64)
    torch.testing.assert_close(o1, o2, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(s1, s2, rtol=1e-4, atol=1e-4)


def test_gka_chunk_matches_recurrent_and_solves():
    q, k, v, g, _ = _rand(T=100)
    q, k = R.l2_norm(q), R.l2_norm(k)
    x1, h1 = R.gka_chebyshev_recurrent(q, k, g, num_iter=30)
    x2, h2 = R.gka_chebyshev_chunk(q, k, g, num_iter=30, chunk_size=64)
    torch.testing.assert_close(x1, x2, rtol=1e-3, atol=1e-4)
    torch.testing.assert_close(h1, h2, rtol=1e-4, atol=1e-5)
    # the last row solves (H_T + lambda I) x = q_T
    fro = h1.pow(2).sum((-1, -2)).sqrt()
    lam = 0.02 * fro
    res = torch.einsum("bhij,bhj->bhi", h1, x1[:, -1]) + lam[..., None] * x1[:, -1] - q[:, -1]
    assert res.abs().max() < 1e-3


def test_ssd_chunk_matches_recurrent():
    B, T, H, P, G, N = 2, 130, 4, 8, 2, 16
    x = torch.randn(B, T, H, P)
    dt = torch.rand(B, T, H) * 0.5
    A = -torch.rand(H)
    Bm, Cm = torch.randn(B, T, G, N), torch.randn(B, T, G, N)
    D = torch.randn(H)
    h0 = torch.randn(B, H, P, N) * 0.1
    y1, s1 = R.ssd_recurrent(x, dt, A, Bm, Cm, D, initial_state=h0)
    y2, s2 = R.ssd_chunk(x, dt, A, Bm, Cm, D, initial_state=h0, chunk_size=64)
    torch.testing.assert_close(y1, y2, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(s1, s2, rtol=1e-4, atol=1e-4)


def test_attention_masks_and_merge():
    B, T, Hq, Hkv, D, w = 1, 40, 4, 2, 8, 6
    q, k, v = torch.randn(B, T, Hq, D), torch.randn(B, T, Hkv, D), torch.randn(B, T, Hkv, D)
    # window 2w = in-window part + hollow part, merged exactly
    o_full, _ = R.attention(q, k, v, window=2 * w, return_lse=True)
    o_s, l_s = R.attention(q, k, v, window=w, return_lse=True)
    o_c, l_c = R.attention(q, k, v, hollow=w, return_lse=True)
    o_m, _ = R.merge_attention_states(o_s, l_s, o_c, l_c)
    torch.testing.assert_close(o_m, o_full, rtol=1e-5, atol=1e-5)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.repeat_interleave(2, 2).transpose(1, 2), v.repeat_interleave(2, 2).transpose(1, 2),
        is_causal=True).transpose(1, 2)
    torch.testing.assert_close(R.attention(q, k, v), ref, rtol=1e-5, atol=1e-5)


def test_conv_state_and_update():
    B, T, C, K = 2, 20, 6, 4
    x, w, b = torch.randn(B, T, C), torch.randn(C, K), torch.randn(C)
    y, st = R.causal_conv1d(x, w, b, return_final_state=True)
    y1, st1 = R.causal_conv1d(x[:, :12], w, b, return_final_state=True)
    y2 = R.causal_conv1d(x[:, 12:], w, b, initial_state=st1)
    torch.testing.assert_close(torch.cat([y1, y2], 1), y)
    yt, st2 = R.causal_conv1d_update(x[:, 12], st1, w, b)
    torch.testing.assert_close(yt, y[:, 12], rtol=1e-5, atol=1e-6)


def test_rope_and_norms():
    x = torch.randn(2, 5, 3, 8)
    pos = torch.arange(5).expand(2, 5)
    cos, sin = R.rope_tables(pos, 8, 1e4)
    y = R.apply_rope(x, cos, sin)
    torch.testing.assert_close(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5, atol=1e-5)
    n = R.rms_norm(x, torch.ones(8))
    torch.testing.assert_close(n.pow(2).mean(-1), torch.ones(2, 5, 3), rtol=1e-3, atol=1e-3)


def test_linear_ce_and_moe():
    h, w = torch.randn(10, 8), torch.randn(32, 8)
    y = torch.randint(0, 32, (10,))
    y[3] = -100
    loss, n = R.linear_cross_entropy(h, w, y, chunk=4)
    ref = torch.nn.functional.cross_entropy(h @ w.t(), y, ignore_index=-100, reduction="sum")
    torch.testing.assert_close(loss, ref)
    assert n.item() == 9
    x = torch.randn(12, 8)
    wgu, wd = torch.randn(4, 12, 8), torch.randn(4, 8, 6)
    wts, idx = R.moe_router(torch.randn(12, 4), 2)
    out = R.moe_experts(x, wgu, wd, wts, idx)
    ref = torch.zeros(12, 8)
    for t in range(12):
        for j in range(2):
            e = idx[t, j]
            g, u = (x[t] @ wgu[e].t()).chunk(2)
            ref[t] += wts[t, j] * ((torch.nn.functional.silu(g) * u) @ wd[e].t())
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-4)


def test_gka_implicit_backward_equals_autograd_through_the_converged_iteration():
    """``ChebyshevCore.backward`` (adjoint solve, GLA form of ``dH``, closed form of ``|H|_F``) against autograd
    through the iteration itself, on CPU where both use the same PyTorch forward."""
    import torch
    from hybrid_model_factory_b200.ops import gka_parallel as GP
    from hybrid_model_factory_b200.ops.scan import ssm_scan
    torch.manual_seed(0)
    B, T, H, D = 1, 40, 2, 8
    q = torch.randn(B, T, H, D)
    k = torch.nn.functional.normalize(torch.randn(B, T, H, D), dim=-1)
    gk = -torch.rand(B, T, H) * 0.2
    a = torch.randn(B, H, D, 4) * 0.3
    h0 = a @ a.transpose(-1, -2)
    w = torch.randn(B, T, H, D)
    wh = torch.randn(B, H, D, D) * 0.01
    wh = wh + wh.transpose(-1, -2)
    ref = [t.clone().requires_grad_(True) for t in (q, k, gk, h0)]
    x_r, hT_r = GP.chebyshev_chunk_parallel(ref[0], ref[1], ref[2], ridge_ratio=0.05, num_iter=200,
                                            initial_state=ref[3], chunk_size=16)
    ((x_r * w).sum() + (hT_r * wh).sum()).backward()
    mine = [t.clone().requires_grad_(True) for t in (q, k, gk, h0)]
    core = GP.ChebyshevCore(0.05, 200, chunk_size=16)
    x_k, (hT_k,) = ssm_scan(core, mine[:3], (mine[3],), None)
    ((x_k * w).sum() + (hT_k * wh).sum()).backward()
    assert torch.allclose(x_k, x_r, atol=1e-5)
    for a_, b_, name in zip(mine, ref, ("dq", "dk", "dgk", "dh0")):
        err = float((a_.grad - b_.grad).norm() / b_.grad.norm())
        assert err < 1e-4, (name, err)
