"""Parity of every kernel schedule fa_b200_fwd can dispatch, of the benchmark configurations at
their full shapes, and of the bytes around the outputs.

fa_b200_fwd picks one of four schedules per call (fa_b200_fwd_plan reports the pick).  Each test
here first asserts which schedule its shape gets, then compares the result with the CPU oracle
(the reference's manual branch, src/py/model_inference.py:68-75) at the tolerances of
test_parity_gpu.py: max-abs <= 2e-2, mean-abs <= 2e-3, LSE within 1e-3 * max(1, |LSE|) against the
oracle on the bf16-rounded inputs the kernel receives.  Ragged lengths follow the reference's
boundary test (test/py/test_cuda_implementation.py:93-117).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-2
MEAN_ABS = 2e-3


@pytest.fixture(scope="module")
def cfa(fa_lib):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from tfg_flashattention_b200 import custom_flash_attn
    assert fa_lib.fa_b200_device_ok(0) == 1, "device 0 is not compute capability 10.x"
    return custom_flash_attn


def _oracle():
    from oracle import attention_oracle
    return attention_oracle


def _check_heads_fully(o, lse, qb, kb, vb, heads, causal):
    """Every row of the listed (b, h) heads against the oracle on the same bf16 inputs."""
    orc = _oracle()
    for (b, h) in heads:
        ro, rl = orc.manual_attention(qb[b:b + 1, h:h + 1].float().cpu(), kb[b:b + 1, h:h + 1].float().cpu(),
                                      vb[b:b + 1, h:h + 1].float().cpu(), causal=causal, return_lse=True)
        d = (o[b, h].float().cpu() - ro[0, 0]).abs()
        assert d.max().item() <= MAX_ABS, f"head {(b, h)}: max-abs {d.max().item():.3e}"
        assert d.mean().item() <= MEAN_ABS, f"head {(b, h)}: mean-abs {d.mean().item():.3e}"
        dl = (lse[b, h].cpu() - rl[0, 0]).abs()
        assert (dl <= 1e-3 * rl[0, 0].abs().clamp_min(1.0)).all(), f"head {(b, h)}: LSE {dl.max().item():.3e}"


def _check_rows(o, lse, q, k, v, qb, kb, vb, heads, rows, causal, input_rounding_slack=False):
    """Sampled rows of the listed heads.  With input_rounding_slack the fp32-input oracle is
    consulted too: the kernel may add at most the tolerance to what rounding q, k, v to bf16 costs
    by itself (needed where scaled key rows make that rounding alone exceed the tolerance)."""
    orc = _oracle()
    for (b, h) in heads:
        rb, rlb = orc.manual_attention_rows(qb[b, h].float().cpu(), kb[b, h].float().cpu(),
                                            vb[b, h].float().cpu(), rows, causal=causal)
        got = o[b, h, rows.cuda()].float().cpu()
        d = (got - rb).abs()
        assert d.max().item() <= MAX_ABS, f"head {(b, h)}: max-abs {d.max().item():.3e}"
        assert d.mean().item() <= MEAN_ABS, f"head {(b, h)}: mean-abs {d.mean().item():.3e}"
        dl = (lse[b, h, rows.cuda()].cpu() - rlb).abs()
        assert (dl <= 1e-3 * rlb.abs().clamp_min(1.0)).all(), f"head {(b, h)}: LSE {dl.max().item():.3e}"
        if input_rounding_slack:
            ro, _ = orc.manual_attention_rows(q[b, h], k[b, h], v[b, h], rows, causal=causal)
            assert (got - ro).abs().max().item() <= (rb - ro).abs().max().item() + MAX_ABS
            assert (got - ro).abs().mean().item() <= (rb - ro).abs().mean().item() + MEAN_ABS


def _spread_heads(B, H, n):
    """n (batch, head) pairs spread over the flattened list, first and last included."""
    total = B * H
    idx = sorted({round(i * (total - 1) / (n - 1)) for i in range(n)})
    return [(i // H, i % H) for i in idx]


def _tile_edge_rows(N, n_random, seed):
    g = torch.Generator().manual_seed(seed)
    edges = [r for t in range(0, N, 128) for r in (t, t + 1, t + 31, t + 32, t + 126, t + 127) if r < N]
    return torch.cat([torch.randint(0, N, (n_random,), generator=g), torch.tensor(edges + [N - 1])]).unique()


# ------------------------------------------------------------- every schedule the launcher can pick

@pytest.mark.parametrize("B,H,N", [(10, 20, 512), (10, 20, 1000), (5, 40, 384)])
def test_persistent_noncausal_schedule(cfa, B, H, N):
    """Non-causal, at least 592 work items of at most 8 K/V tiles: resident CTAs loop over items
    (fa_fwd_kernel<true,false>); N = 1000 puts a ragged last K/V tile on that path.  Every row of
    every head is compared with the oracle."""
    torch.manual_seed(7000 + N)
    q, k, v = (torch.randn(B, H, N, 64) for _ in range(3))
    qb, kb, vb = (t.to("cuda", torch.bfloat16) for t in (q, k, v))
    assert cfa.plan(qb, kb, vb, causal=False)[0] == "persistent_full"
    o, lse = cfa.forward(qb, kb, vb, causal=False, return_lse=True)
    assert cfa.last_status() == 0
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    ro, rl = _oracle().manual_attention_blocked(qb.float().cpu(), kb.float().cpu(), vb.float().cpu(),
                                                causal=False, return_lse=True)
    d = (o.float().cpu() - ro).abs()
    assert d.max().item() <= MAX_ABS and d.mean().item() <= MEAN_ABS, (d.max().item(), d.mean().item())
    assert ((lse.cpu() - rl).abs() <= 1e-3 * rl.abs().clamp_min(1.0)).all()
    # the same heads computed alone take the one-CTA-per-tile schedule: identical bits
    for (b, h) in _spread_heads(B, H, 4):
        alone, alone_lse = cfa.forward(qb[b:b + 1, h:h + 1], kb[b:b + 1, h:h + 1], vb[b:b + 1, h:h + 1],
                                       causal=False, return_lse=True)
        assert torch.equal(alone[0, 0], o[b, h]) and torch.equal(alone_lse[0, 0], lse[b, h])


@pytest.mark.parametrize("B,H,N", [(8, 25, 384), (8, 25, 640), (8, 25, 600), (30, 20, 128)])
def test_persistent_rotated_causal_schedule(cfa, B, H, N):
    """Causal with an odd number of query tiles and at least 592 items: resident CTAs stride
    through single tiles whose order inside a head is rotated by the head index.  Every row of
    every head is compared with the oracle; N = 600 adds a ragged last tile."""
    torch.manual_seed(8000 + N)
    q, k, v = (torch.randn(B, H, N, 64) for _ in range(3))
    qb, kb, vb = (t.to("cuda", torch.bfloat16) for t in (q, k, v))
    assert cfa.plan(qb, kb, vb, causal=True)[0] == "persistent_rotated"
    o, lse = cfa.forward(qb, kb, vb, causal=True, return_lse=True)
    assert cfa.last_status() == 0
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    ro, rl = _oracle().manual_attention_blocked(qb.float().cpu(), kb.float().cpu(), vb.float().cpu(),
                                                causal=True, return_lse=True)
    d = (o.float().cpu() - ro).abs()
    assert d.max().item() <= MAX_ABS and d.mean().item() <= MEAN_ABS, (d.max().item(), d.mean().item())
    assert ((lse.cpu() - rl).abs() <= 1e-3 * rl.abs().clamp_min(1.0)).all()
    for (b, h) in _spread_heads(B, H, 4):
        alone = cfa.forward(qb[b:b + 1, h:h + 1], kb[b:b + 1, h:h + 1], vb[b:b + 1, h:h + 1])
        assert torch.equal(alone[0, 0], o[b, h])


@pytest.mark.parametrize("causal,N", [(True, 256), (False, 128), (True, 128)])
def test_many_items_per_cta(cfa, causal, N):
    """A persistent CTA decodes all its work items into a table of 256 entries when it starts.
    Here every CTA gets about 250 of them (generated on the device: 1-2 GB of inputs); sampled
    heads from the first to the last are compared with the oracle and with the same head computed
    alone.  One more batch entry per CTA than the table holds and the launcher takes one CTA per
    tile instead."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    per_cta = 250
    tiles = N // 128
    heads = (2 * sms * per_cta) // tiles          # items = heads * tiles = 2 * sms * per_cta
    B, H = heads // 8, 8
    g = torch.Generator(device="cuda").manual_seed(9100 + N + int(causal))
    qb, kb, vb = (torch.randn(B, H, N, 64, device="cuda", generator=g).bfloat16() for _ in range(3))
    want = {(True, 256): "persistent_paired", (True, 128): "persistent_rotated", (False, 128): "persistent_full"}
    assert cfa.plan(qb, kb, vb, causal=causal) == (want[(causal, N)], 2 * sms)
    o, lse = cfa.forward(qb, kb, vb, causal=causal, return_lse=True)
    assert cfa.last_status() == 0
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    picked = _spread_heads(B, H, 12)
    _check_heads_fully(o, lse, qb, kb, vb, picked, causal)
    for (b, h) in picked[::3]:
        alone, alone_lse = cfa.forward(qb[b:b + 1, h:h + 1], kb[b:b + 1, h:h + 1], vb[b:b + 1, h:h + 1],
                                       causal=causal, return_lse=True)
        assert torch.equal(alone[0, 0], o[b, h]) and torch.equal(alone_lse[0, 0], lse[b, h])
    # past the table: 2 * sms * 256 items fit, a few more do not
    big_b = (2 * sms * 256) // (tiles * H) + 2
    t = torch.empty(big_b, H, N, 64, device="cuda", dtype=torch.bfloat16)
    assert cfa.plan(t, t, t, causal=causal) == ("cta_per_tile", big_b * H * tiles)


def test_plan_reports_each_schedule(cfa):
    """The dispatch rule itself, on shapes of the benchmark configurations."""
    def plan(B, H, N, causal):
        t = torch.empty(B, H, N, 64, device="cuda", dtype=torch.bfloat16)
        return cfa.plan(t, t, t, causal=causal)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert plan(32, 25, 1024, True) == ("persistent_paired", 2 * sms)
    assert plan(4, 12, 1024, True)[0] == "persistent_paired"
    assert plan(16, 16, 512, False) == ("persistent_full", 2 * sms)
    assert plan(16, 16, 4096, False) == ("cta_per_tile", 16 * 16 * 32)
    assert plan(4, 25, 8192, True)[0] == "cta_per_tile"
    assert plan(2, 3, 300, True) == ("cta_per_tile", 18)
    assert plan(8, 25, 384, True)[0] == "persistent_rotated"
    assert plan(0, 4, 16, True) == ("none", 0)


# ------------------------------------------------------------- benchmark configurations, full shapes

@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("N", [512, 1024, 2048, 4096])
def test_config3_full_shape(cfa, N, causal):
    """B = 16, H = 16 (GPT-2 medium attention-only sweep), both modes: all rows of four heads at
    N <= 1024, a sample of rows (tile edges included) of four heads above, plus two properties on
    the whole tensor: rows of P sum to one (V = 1 gives O = 1) and no value is NaN or infinite."""
    from tfg_flashattention_b200.workloads import config3
    w = config3(N, causal)
    q, k, v = w.make_cpu()
    qb, kb, vb = (t.to("cuda", torch.bfloat16) for t in (q, k, v))
    o, lse = cfa.forward(qb, kb, vb, causal=causal, return_lse=True)
    assert cfa.last_status() == 0
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    heads = _spread_heads(w.B, w.H, 4)
    if N <= 1024:
        _check_heads_fully(o, lse, qb, kb, vb, heads, causal)
    else:
        _check_rows(o, lse, q, k, v, qb, kb, vb, heads, _tile_edge_rows(N, 512, N), causal)
    ones = cfa.forward(qb, kb, torch.ones_like(vb), causal=causal)
    assert cfa.last_status() == 0
    assert (ones.float() - 1.0).abs().max().item() <= 1e-2


@pytest.mark.parametrize("N", [16384, 32768])
def test_config5_long_context(cfa, N):
    """B = 4, H = 25, 1 % of the key rows scaled x4, causal (N = 8192 is covered by
    test_long_context_stress_rows): sampled rows of three heads, always including the rows right
    after a scaled key row, where a wrong lazy rescale of O would show."""
    from tfg_flashattention_b200.workloads import config5
    w = config5(N)
    q, k, v = w.make_cpu()
    qb, kb, vb = (t.to("cuda", torch.bfloat16) for t in (q, k, v))
    o, lse = cfa.forward(qb, kb, vb, return_lse=True)
    assert cfa.last_status() == 0
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    big = (k[0, 0].norm(dim=-1) > 20).nonzero().flatten()       # the scaled rows (same for every head)
    assert big.numel() == N // 100
    g = torch.Generator().manual_seed(N)
    edges = [t * 128 + r for t in (0, 1, N // 256, N // 128 - 1) for r in (0, 31, 32, 127)]
    rows = torch.cat([torch.randint(0, N, (384,), generator=g), big[:64], (big[:200] + 1).clamp_max(N - 1),
                      torch.tensor(edges)]).unique()
    _check_rows(o, lse, q, k, v, qb, kb, vb, [(0, 0), (1, 7), (3, 24)], rows, True,
                input_rounding_slack=True)


# ------------------------------------------------------------- nothing outside the outputs is written

@pytest.mark.parametrize("layout", ["bhnd", "bnhd"])
@pytest.mark.parametrize("N", [1, 65, 129, 300])
def test_outputs_stay_inside_their_buffers(cfa, N, layout):
    """O and LSE are carved out of larger buffers filled with a sentinel (the stand-in for a
    memory checker): the bytes before, after and -- for a strided O -- between the rows the kernel
    owns must be bit-identical afterwards.  O is written by TMA stores of 32-row slabs that the
    tensor map clips at row N; the LSE by plain stores guarded by row < N."""
    torch.manual_seed(9000 + N)
    B, H, d, pad = 2, 3, 64, 512
    q, k, v = (torch.randn(B, H, N, d, device="cuda").bfloat16() for _ in range(3))
    sentinel = -7.5
    if layout == "bhnd":
        n_elems = B * H * N * d
        arena = torch.full((pad + n_elems + pad,), sentinel, device="cuda", dtype=torch.bfloat16)
        out = arena[pad:pad + n_elems].view(B, H, N, d)
        owned = torch.zeros_like(arena, dtype=torch.bool)
        owned[pad:pad + n_elems] = True
    else:
        # [B, N, H, 2*d] memory: each head's row is followed by d elements that are not ours
        n_elems = B * N * H * 2 * d
        arena = torch.full((pad + n_elems + pad,), sentinel, device="cuda", dtype=torch.bfloat16)
        body = arena[pad:pad + n_elems].view(B, N, H, 2 * d)
        out = body[..., :d].permute(0, 2, 1, 3)
        owned = torch.zeros_like(arena, dtype=torch.bool)
        owned[pad:pad + n_elems].view(B, N, H, 2 * d)[..., :d] = True
    assert out.data_ptr() % 16 == 0
    lse_arena = torch.full((pad + B * H * N + pad,), sentinel, device="cuda", dtype=torch.float32)
    import ctypes
    from tfg_flashattention_b200 import _lib as lib
    p = cfa._fwd_params(q, k, v, out, lse_arena[pad:pad + B * H * N], True, None)
    rc = lib.load().fa_b200_fwd(ctypes.byref(p))
    assert rc == 0 and cfa.last_status() == 0
    assert (arena[~owned] == sentinel).all(), "bytes outside O were written"
    assert (lse_arena[:pad] == sentinel).all() and (lse_arena[pad + B * H * N:] == sentinel).all(), \
        "bytes outside LSE were written"
    ref_o, ref_lse = cfa.forward(q, k, v, return_lse=True)
    assert torch.equal(out, ref_o)
    assert torch.equal(lse_arena[pad:pad + B * H * N].view(B, H, N), ref_lse)
