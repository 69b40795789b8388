"""Residual add + LayerNorm kernel against the reference's LayerNorm arithmetic in fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(a, resid, scale, shift, eps):
    """model_inference.py:102-107 (mean, var(unbiased=False), eps, scale, shift) on the bf16-rounded
    sum, in fp32."""
    s = a.float() + (resid.float() if resid is not None else 0.0)
    s = s.bfloat16().float() if resid is not None else s
    mean = s.mean(dim=-1, keepdim=True)
    var = s.var(dim=-1, keepdim=True, unbiased=False)
    return s, (s - mean) / torch.sqrt(var + eps) * scale.float() + shift.float()


@pytest.mark.parametrize("cols", [8, 64, 768, 1024, 1280, 1600, 2048])
@pytest.mark.parametrize("rows", [1, 7, 1000])
@pytest.mark.parametrize("with_resid", [False, True])
def test_add_layernorm_matches_fp32(fa_lib, rows, cols, with_resid):
    from tfg_flashattention_b200.block_ops import add_layernorm
    g = torch.Generator(device="cuda").manual_seed(rows * 10000 + cols)
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g)
    a = (rnd(rows, cols) * 2 + 0.5).bfloat16()
    resid = (rnd(rows, cols) * 3 - 1).bfloat16() if with_resid else None
    scale, shift = (1 + 0.2 * rnd(cols)).bfloat16(), (0.3 * rnd(cols)).bfloat16()
    out = add_layernorm(a, resid, scale, shift, 1e-5)
    s_ref, y_ref = _reference(a, resid, scale, shift, 1e-5)
    if with_resid:
        s, y = out
        assert torch.equal(s, s_ref.bfloat16())          # the sum is bit-exact
    else:
        y = out
    # one bf16 rounding of a value of magnitude <= ~8: half an ulp of 2^-5, plus fp32 noise
    err = (y.float() - y_ref).abs()
    assert (err <= 2.0 ** -8 * y_ref.abs().clamp_min(1.0) + 1e-3).all(), err.max().item()


def test_add_layernorm_in_place_and_3d(fa_lib):
    from tfg_flashattention_b200.block_ops import add_layernorm
    torch.manual_seed(0)
    a = torch.randn(2, 5, 1600, device="cuda").bfloat16()
    x = torch.randn(2, 5, 1600, device="cuda").bfloat16()
    scale, shift = torch.ones(1600, device="cuda").bfloat16(), torch.zeros(1600, device="cuda").bfloat16()
    s0, y0 = add_layernorm(a, x, scale, shift)
    x_alias = x.clone()
    s1, y1 = add_layernorm(a, x_alias, scale, shift, sum_out=x_alias)     # residual stream updated in place
    assert s1.data_ptr() == x_alias.data_ptr()
    assert torch.equal(s0, s1) and torch.equal(y0, y1)
    # without a kept sum the row is normalised before any rounding: equal up to that rounding
    y2 = add_layernorm(a, x, scale, shift, return_sum=False)
    torch.testing.assert_close(y2.float(), y0.float(), rtol=0, atol=0.05)


def test_add_layernorm_rejects(fa_lib):
    from tfg_flashattention_b200.block_ops import add_layernorm
    ok = torch.zeros(4, 64, device="cuda").bfloat16()
    w = torch.ones(64, device="cuda").bfloat16()
    with pytest.raises(RuntimeError):
        add_layernorm(ok.float(), None, w, w)
    with pytest.raises(RuntimeError):
        add_layernorm(ok[:, :32], None, w[:32], w[:32])                    # not contiguous
    with pytest.raises(RuntimeError):
        add_layernorm(ok, ok[:2], w, w)
    bad = torch.zeros(4, 2056, device="cuda").bfloat16()
    with pytest.raises(RuntimeError, match="fa_b200"):
        add_layernorm(bad, None, torch.ones(2056, device="cuda").bfloat16(), torch.ones(2056, device="cuda").bfloat16())


def test_fused_block_path_equals_module_by_module_path(fa_lib):
    """GPTModel with the fused add+LayerNorm / GELU-epilogue path against the same bf16 model run
    block by block through torch's layer_norm, add and gelu."""
    from tfg_flashattention_b200 import gpt2
    cfg = {"vocab_size": 503, "context_length": 256, "emb_dim": 256, "n_heads": 4, "n_layers": 3,
           "drop_rate": 0.0, "qkv_bias": True, "impl_type": "cuda"}
    model = gpt2.init_random(gpt2.GPTModel(cfg, dtype=torch.bfloat16), seed=5, std=0.05).cuda().eval()
    ids = torch.randint(0, cfg["vocab_size"], (3, 200), device="cuda")
    with torch.no_grad():
        plain = model(ids).float()
        model.prepare_for_inference()
        assert model._fused_blocks
        fused = model(ids).float()
        last = model(ids, last_token_only=True).float()
    scale = plain.abs().max().item()
    assert (fused - plain).abs().max().item() <= 0.03 * scale      # bf16 rounding at different places
    assert (fused - plain).abs().mean().item() <= 0.004 * scale
    torch.testing.assert_close(last, fused[:, -1:, :], rtol=0, atol=0.02 * scale)


@pytest.mark.parametrize("M", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("N,K", [(7, 8), (64, 64), (4800, 1600), (1600, 6400), (50257, 768)])
def test_linear_small_matches_fp32(fa_lib, M, N, K):
    """y = act(x W^T + b) for a few rows: against the fp32 product of the same bf16 numbers."""
    from tfg_flashattention_b200.block_ops import linear_small
    g = torch.Generator(device="cuda").manual_seed(M * 100003 + N + K)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    b = torch.randn(N, device="cuda", generator=g).bfloat16()
    ref = x.float() @ w.float().t()
    for bias, gelu in ((None, False), (b, False), (b, True)):
        want = ref + (bias.float() if bias is not None else 0.0)
        if gelu:
            want = torch.nn.functional.gelu(want, approximate="tanh")
        got = linear_small(x, w, bias, gelu=gelu).float()
        assert got.shape == (M, N)
        # fp32 accumulation, one rounding to bf16
        assert ((got - want).abs() <= 2.0 ** -8 * want.abs() + 1e-3).all(), (got - want).abs().max().item()


def test_linear_small_strided_weight_3d_input_and_errors(fa_lib):
    from tfg_flashattention_b200.block_ops import linear_small
    torch.manual_seed(1)
    big = torch.randn(300, 512, device="cuda").bfloat16()
    w = big[:, 128:384]                                   # rows 512 apart, 256 columns used
    x = torch.randn(2, 1, 256, device="cuda").bfloat16()   # [B, 1, K] as in a decode step
    got = linear_small(x, w).float()
    assert got.shape == (2, 1, 300)
    want = x.float().view(2, 256) @ w.float().t()
    assert ((got.view(2, 300) - want).abs() <= 2.0 ** -8 * want.abs() + 1e-3).all()
    with pytest.raises(RuntimeError, match="fa_b200"):
        linear_small(torch.zeros(9, 64, device="cuda").bfloat16(), torch.zeros(8, 64, device="cuda").bfloat16())
    with pytest.raises(RuntimeError):
        linear_small(torch.zeros(2, 60, device="cuda").bfloat16(), torch.zeros(8, 60, device="cuda").bfloat16())
    with pytest.raises(RuntimeError):
        linear_small(x, w.float())


@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("K", [64, 768, 1600, 2048])
def test_linear_small_with_add_layernorm_prologue(fa_lib, M, K):
    """x' = LayerNorm(x + resid) inside the Linear kernel: equal to add_layernorm followed by the
    plain kernel (same roundings), and close to the fp32 formula."""
    from tfg_flashattention_b200.block_ops import add_layernorm, linear_small
    g = torch.Generator(device="cuda").manual_seed(M * 7919 + K)
    N = 3 * K if K <= 768 else 264
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    r = (torch.randn(M, K, device="cuda", generator=g) * 2).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    b = torch.randn(N, device="cuda", generator=g).bfloat16()
    sc = (1 + 0.2 * torch.randn(K, device="cuda", generator=g)).bfloat16()
    sh = (0.3 * torch.randn(K, device="cuda", generator=g)).bfloat16()
    # with the sum kept
    s_ref, h_ref = add_layernorm(x, r, sc, sh, 1e-5)
    y_ref = linear_small(h_ref, w, b, gelu=True)
    s, y = linear_small(x, w, b, gelu=True, resid=r, ln_scale=sc, ln_shift=sh, eps=1e-5, keep_sum=True)
    assert torch.equal(s, s_ref)
    torch.testing.assert_close(y.float(), y_ref.float(), rtol=0, atol=2e-2)
    assert (y.float() - y_ref.float()).abs().mean().item() < 1e-3
    # LayerNorm only (first block, final norm without residual) and residual only
    y1 = linear_small(x, w, b, ln_scale=sc, ln_shift=sh)
    y1_ref = linear_small(add_layernorm(x, None, sc, sh, 1e-5), w, b)
    torch.testing.assert_close(y1.float(), y1_ref.float(), rtol=0, atol=2e-2)
    y2 = linear_small(x, w, resid=r)
    y2_ref = (x.float() + r.float()) @ w.float().t()
    assert ((y2.float() - y2_ref).abs() <= 2.0 ** -7 * y2_ref.abs() + 3e-2).all()
    # fp32 formula end to end
    s32 = (x.float() + r.float()).bfloat16().float()
    h32 = torch.nn.functional.layer_norm(s32, (K,), sc.float(), sh.float(), 1e-5).bfloat16().float()
    want = torch.nn.functional.gelu(h32 @ w.float().t() + b.float(), approximate="tanh")
    assert ((y.float() - want).abs() <= 2.0 ** -6 * want.abs() + 2e-2).all()


def test_linear_small_prologue_rejects(fa_lib):
    from tfg_flashattention_b200.block_ops import linear_small
    x = torch.zeros(1, 4096, device="cuda").bfloat16()
    w = torch.zeros(8, 4096, device="cuda").bfloat16()
    one = torch.ones(4096, device="cuda").bfloat16()
    with pytest.raises(RuntimeError, match="fa_b200"):
        linear_small(x, w, ln_scale=one, ln_shift=one)            # K > 2048 with a prologue
    with pytest.raises(RuntimeError):
        linear_small(x[:, :64].contiguous(), w[:, :64].contiguous(), ln_scale=one[:64].contiguous())
