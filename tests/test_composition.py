"""State composition: coefficient identities and end-to-end consistency of the composed cache."""
import itertools

import torch

from hybrid_model_factory_b200.models import composition as C
from hybrid_model_factory_b200.models.configuration import HybridConfig
from hybrid_model_factory_b200.models.modeling_hybrid import build_model


def test_scalar_coefficients_are_the_permutation_average():
    torch.manual_seed(0)
    N = 4
    A = torch.rand(N, 3)
    s = torch.randn(N, 3)
    total = torch.zeros(3)
    perms = list(itertools.permutations(range(N)))
    for perm in perms:
        state = torch.zeros(3)
        for i in perm:                      # sequential composition: state <- A_i * state + s_i
            state = A[i] * state + s[i]
        total += state
    ref = total / len(perms)
    c = C.picaso_coefficients(A)
    assert torch.allclose((c * s).sum(0), ref, atol=1e-5)
    assert torch.allclose(torch.exp(C.picaso_log_coefficients(torch.log(A))), c, atol=1e-5)


def test_matrix_coefficients_reduce_to_scalar_case():
    torch.manual_seed(0)
    a = torch.rand(3, 2)
    Phi = a[..., None, None] * torch.eye(4)
    cm = C.picaso_matrix_coefficients(Phi)
    cs = C.picaso_coefficients(a)
    assert torch.allclose(cm, cs[..., None, None] * torch.eye(4), atol=1e-5)


def _model(pattern):
    cfg = HybridConfig("hybrid_qwen3", vocab_size=128, hidden_size=64, intermediate_size=128,
                       num_hidden_layers=len(pattern.split("-")), num_attention_heads=4, num_key_value_heads=2,
                       head_dim=16, hybrid_override_pattern=pattern)
    torch.manual_seed(0)
    return build_model(cfg).eval()


def test_single_chunk_composition_equals_plain_prefill():
    model = _model("*-GDN-M2-GKA")
    ctx = torch.randint(0, 128, (1, 24))
    q = torch.randint(0, 128, (1, 5))
    ref = model.generate(torch.cat([ctx, q], 1), max_new_tokens=6)[:, 29:]
    for ct in ("concat_fuse", "concat_soup", "full_fuse"):
        out = C.generate_composed(model, ctx, q, num_chunks=1, compose_type=ct, max_new_tokens=6)
        assert torch.equal(out, ref), ct


def test_all_nine_modes_run_and_gdn_transition_matches_linearity():
    model = _model("*-GDN-M2-GKA")
    ctx = torch.randint(0, 128, (1, 32))
    q = torch.randint(0, 128, (1, 4))
    for kv in C.KV_MODES:
        for ssm in C.SSM_MODES:
            out = C.generate_composed(model, ctx, q, num_chunks=3, compose_type=f"{kv}_{ssm}", max_new_tokens=3,
                                      prefix=torch.randint(0, 128, (1, 4)))
            assert out.shape == (1, 3)
    # the transition trick: state(chunk | S0) == Phi @ S0 + state(chunk | 0) with Phi = state(v = 0 | I)
    from hybrid_model_factory_b200.ops import mixers
    B, T, H, D = 1, 40, 2, 16
    qq, kk, vv = (torch.randn(B, T, H, D) for _ in range(3))
    g, beta = -torch.rand(B, T, H) * 0.2, torch.rand(B, T, H)
    S0 = torch.randn(B, H, D, D) * 0.3
    eye = torch.eye(D).expand(B, H, D, D).contiguous()
    _, Phi = mixers.gated_delta_rule(qq, kk, torch.zeros_like(vv), g, beta, initial_state=eye)
    _, s_zero = mixers.gated_delta_rule(qq, kk, vv, g, beta)
    _, s_inj = mixers.gated_delta_rule(qq, kk, vv, g, beta, initial_state=S0)
    assert torch.allclose(s_inj, Phi @ S0 + s_zero, atol=2e-4)
