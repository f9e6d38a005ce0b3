"""Host logic of the layer shell around the operator (CPU) and the shell end to end (GPU).

The reference pins the same behaviour for its shell in tests/attention/ (projection shapes, rotary
embedding on q and k only, head-first contiguous tensors into the operator, one o_proj)."""

import pytest
import torch

from oal_b200 import attention_shell as shell
from oracle import oal_oracle as orc


def test_rope_tables_and_rotation_match_the_complex_form():
    n, d = 9, 8
    cos, sin = shell.rope_tables(n, d, theta=1.0e6)
    assert cos.shape == (n, d) and sin.shape == (n, d)
    g = torch.Generator().manual_seed(0)
    q = torch.randn(2, 3, n, d, generator=g, dtype=torch.float64)
    k = torch.randn(2, 1, n, d, generator=g, dtype=torch.float64)
    rq, rk = shell.apply_rotary_pos_emb(q, k, cos.double(), sin.double())
    # rotate-half convention = complex rotation of the pair (x[j], x[j + d/2]) by angle pos * theta^(-2j/d)
    inv = 1.0 / (1.0e6 ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
    ang = torch.arange(n, dtype=torch.float64)[:, None] * inv[None, :]
    z = torch.complex(q[..., : d // 2], q[..., d // 2:]) * torch.polar(torch.ones_like(ang), ang)
    torch.testing.assert_close(rq, torch.cat((z.real, z.imag), -1), atol=1e-6, rtol=1e-6)
    # position 0 is the identity; norms are preserved
    torch.testing.assert_close(rk[:, :, 0], k[:, :, 0])
    torch.testing.assert_close(rq.norm(dim=-1), q.norm(dim=-1))


def test_projection_layout_and_contract_errors():
    geo = shell.ModelGeometry(num_layers=1, hidden_size=32, num_query_heads=4, num_kv_heads=2, head_dim=8)
    lin = lambda o: torch.nn.Linear(32, o, bias=True)
    x = torch.randn(2, 5, 32)
    pe = shell.rope_tables(5, 8)
    q, k, v = shell.project_qkv_and_apply_rope(q_proj=lin(32), k_proj=lin(16), v_proj=lin(16), hidden_states=x,
                                               position_embeddings=pe, geometry=geo)
    assert q.shape == (2, 4, 5, 8) and k.shape == (2, 2, 5, 8) and v.shape == (2, 2, 5, 8)
    assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
    out = shell.restore_and_project_output(head_output=q, o_proj=torch.nn.Linear(32, 32, bias=False), geometry=geo)
    assert out.shape == (2, 5, 32)
    with pytest.raises(shell.AttentionContractError):
        shell.project_qkv_and_apply_rope(q_proj=lin(32), k_proj=lin(16), v_proj=lin(16), hidden_states=x[..., :31],
                                         position_embeddings=pe, geometry=geo)
    with pytest.raises(shell.AttentionContractError):
        shell.project_qkv_and_apply_rope(q_proj=lin(32), k_proj=lin(16), v_proj=lin(16), hidden_states=x,
                                         position_embeddings=shell.rope_tables(6, 8), geometry=geo)
    with pytest.raises(shell.AttentionContractError):
        shell.restore_and_project_output(head_output=k, o_proj=torch.nn.Linear(32, 32), geometry=geo)


def test_lora_linear_starts_as_the_base_layer_and_trains_only_the_update():
    layer = shell.LoRALinear(16, 8, rank=4, alpha=8.0, bias=True, dtype=torch.float32)
    x = torch.randn(3, 16)
    torch.testing.assert_close(layer(x), layer.base(x))            # B = 0 at initialisation
    assert [n for n, p in layer.named_parameters() if p.requires_grad] == ["lora_a", "lora_b"]
    assert layer.scaling == 2.0


@pytest.mark.gpu
def test_layer_matches_dense_oracle_and_reuses_its_prepared_call():
    torch.manual_seed(5)
    geo = shell.ModelGeometry(num_layers=1, hidden_size=4 * 64, num_query_heads=4, num_kv_heads=2, head_dim=64)
    groups = (torch.arange(64) % 4).to(torch.int32).expand(4, -1).contiguous()
    factor = torch.rand(4, 15) * 0.9 + 0.1
    cache = shell.PreparedCallCache(precision="bf16_tensorcore")
    layer = shell.OalAttentionLayer(0, groups.cuda(), factor.cuda(), cache=cache, geometry=geo, lora_rank=4,
                                    lora_alpha=8.0, dtype=torch.bfloat16, device="cuda")
    x = (torch.randn(2, 200, geo.hidden_size, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    pe = shell.rope_tables(200, 64, device="cuda", dtype=torch.bfloat16)
    y = layer(x, pe)
    y.float().square().mean().backward()
    assert y.shape == x.shape and x.grad is not None and layer.factor.grad is not None
    assert layer.q_proj.lora_b.grad is not None and layer.q_proj.base.weight.grad is None
    # the operator inside the shell against the fp64 dense statement on the same projected tensors
    with torch.no_grad():
        q, k, v = shell.project_qkv_and_apply_rope(q_proj=layer.q_proj, k_proj=layer.k_proj, v_proj=layer.v_proj,
                                                   hidden_states=x, position_embeddings=pe, geometry=geo)
        out, _, _ = cache.grouped(q, k, v, layer.dim_groups, layer.factor, cache_key="check")
        a, b, c = orc.expand_factor(layer.factor.detach().double().cpu(), 4, 1e-6)
        want, _, _ = orc.dense_forward(q.double().cpu(), k.double().cpu(), v.double().cpu(), groups, a, b, c, scale=0.125)
    assert orc.normalized_max_error(out.float().cpu(), want) < 2e-2     # bf16 io tolerance
    # a second call with the same signature reuses the prepared call of the layer
    before = len(cache._entries[0])
    layer(x.detach().requires_grad_(), pe)
    assert len(cache._entries[0]) == before == 1


@pytest.mark.gpu
def test_fused_rope_prologue_matches_the_elementwise_statement_forward_and_backward():
    torch.manual_seed(11)
    geo = shell.ModelGeometry(num_layers=1, hidden_size=6 * 64, num_query_heads=6, num_kv_heads=2, head_dim=64)
    b, n = 2, 203
    lin = lambda o: torch.nn.Linear(geo.hidden_size, o, bias=True, dtype=torch.bfloat16, device="cuda")
    qp, kp, vp = lin(384), lin(128), lin(128)
    x = (torch.randn(b, n, geo.hidden_size, device="cuda")).to(torch.bfloat16)
    pe = shell.rope_tables(n, 64, device="cuda")
    outs = {}
    for fused in (True, False):
        xi = x.clone().requires_grad_()
        q, k, v = shell.project_qkv_and_apply_rope(q_proj=qp, k_proj=kp, v_proj=vp, hidden_states=xi,
                                                   position_embeddings=pe, geometry=geo, fused=fused)
        assert q.shape == (b, 6, n, 64) and k.shape == (b, 2, n, 64) and v.shape == (b, 2, n, 64)
        assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
        g = torch.Generator(device="cuda").manual_seed(3)
        gq, gk, gv = (torch.randn(t.shape, generator=g, device="cuda").to(torch.bfloat16) for t in (q, k, v))
        torch.autograd.backward([q, k, v], [gq, gk, gv])
        outs[fused] = [t.detach().float() for t in (q, k, v, xi.grad)]
    # fp64 statement of the rotation on the same projections
    with torch.no_grad():
        qf = qp(x).double().reshape(b, n, 6, 64).transpose(1, 2)
        cos, sin = pe[0].double(), pe[1].double()
        rot = torch.cat((-qf[..., 32:], qf[..., :32]), -1)
        want_q = qf * cos + rot * sin
    err = lambda a, r: float((a.double() - r.double()).abs().max() / r.double().abs().max())
    assert err(outs[True][0], want_q) < 1e-2            # one bf16 rounding
    assert torch.equal(outs[True][2], outs[False][2])   # v is only moved
    for fused_t, plain_t in zip(outs[True], outs[False]):
        assert err(fused_t, plain_t) < 2e-2             # the element-wise path rounds to bf16 after every step


@pytest.mark.gpu
def test_token_major_output_matches_the_restore_step_forward_and_backward():
    """``output_layout="tokens_first"``: the kernels write ``out`` as ``[B, N, Hq, 64]`` and read its upstream
    gradient in that layout; values and gradients must be those of the reference's restore step
    (transpose + contiguous copy + reshape, qwen_lora_experiment/attention/common.py:575-596) applied to the
    heads-first result -- bit for bit, since only the addresses of the stores and loads change."""
    import oal_b200
    from oal_b200 import synthetic

    case = synthetic.qwen_head_case(21, batch=2, n=300, hq=6, hkv=2, g=8, bf16=True)
    dev = "cuda"
    groups = case.dim_groups.to(dev)
    dflat = torch.randn(2, 300, 6 * 64, generator=torch.Generator().manual_seed(1)).to(dev, torch.bfloat16)
    results = {}
    for layout in ("heads_first", "tokens_first"):
        q, k, v = (t.to(dev, torch.bfloat16).requires_grad_() for t in (case.q, case.k, case.v))
        factor = case.factor.to(dev).requires_grad_()
        prepared = oal_b200.prepare_grouped_hd_block_gemm(q, k, v, groups, factor, scale=case.scale,
                                                          precision="bf16_tensorcore", output_layout=layout)
        out, num, den = oal_b200.run_prepared_grouped_hd_block_gemm(prepared, q, k, v, factor)
        if layout == "heads_first":
            flat = out.transpose(1, 2).contiguous().reshape(2, 300, 6 * 64)       # the restore step
        else:
            assert out.shape == (2, 300, 6, 64) and out.is_contiguous()
            flat = out.reshape(2, 300, 6 * 64)
        flat.backward(dflat)
        results[layout] = [t.detach().clone() for t in (flat, num, den, q.grad, k.grad, v.grad, factor.grad)]
    for x, y in zip(results["heads_first"], results["tokens_first"]):
        assert torch.equal(x, y)
    with pytest.raises(ValueError, match="output_layout"):
        oal_b200.prepare_grouped_hd_block_gemm(q, k, v, groups, factor, output_layout="columns_first")


@pytest.mark.gpu
def test_layer_with_token_major_output_equals_layer_with_restore_step():
    torch.manual_seed(9)
    geo = shell.ModelGeometry(num_layers=1, hidden_size=4 * 64, num_query_heads=4, num_kv_heads=2, head_dim=64)
    groups = (torch.arange(64) % 4).to(torch.int32).expand(4, -1).contiguous()
    factor = torch.rand(4, 15) * 0.9 + 0.1
    x = (torch.randn(2, 150, geo.hidden_size, device="cuda") * 0.5).to(torch.bfloat16)
    pe = shell.rope_tables(150, 64, device="cuda", dtype=torch.bfloat16)
    outs = []
    for layout in ("heads_first", "tokens_first"):
        torch.manual_seed(3)
        cache = shell.PreparedCallCache(precision="bf16_tensorcore", output_layout=layout)
        layer = shell.OalAttentionLayer(0, groups.cuda(), factor.cuda(), cache=cache, geometry=geo, lora_rank=4,
                                        lora_alpha=8.0, dtype=torch.bfloat16, device="cuda")
        xi = x.clone().requires_grad_()
        y = layer(xi, pe)
        y.float().square().mean().backward()
        outs.append((y.detach(), xi.grad.detach(), layer.factor.grad.detach()))
    for a_, b_ in zip(*outs):
        assert torch.equal(a_, b_)
