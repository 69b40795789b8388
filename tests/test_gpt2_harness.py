"""The GPT-2 harness (the caller of the hot path) against the reference's own model output."""
import os

import numpy as np
import pytest
import torch

from tfg_flashattention_b200 import gpt2


def _load_tiny(golden_dir, impl):
    t = np.load(os.path.join(golden_dir, "gpt_tiny.npz"))
    cfg = {"vocab_size": 97, "context_length": 48, "emb_dim": 128, "n_heads": int(t["n_heads"]),
           "n_layers": int(t["n_layers"]), "drop_rate": 0.0, "qkv_bias": True, "impl_type": impl}
    model = gpt2.GPTModel(cfg).eval()
    # the reference's state_dict exactly as it saved it, `att.mask` buffers included
    sd = {k[3:]: torch.from_numpy(t[k]) for k in t.files if k.startswith("sd.")}
    assert any(k.endswith(".att.mask") for k in sd)
    model.load_state_dict(sd, strict=True)
    assert sorted(model.state_dict().keys()) == sorted(sd.keys())
    return model, torch.from_numpy(t["ids"]), torch.from_numpy(t["logits"])


@pytest.mark.parametrize("impl", ["manual", "functional"])
def test_harness_loads_reference_state_dict_and_matches_logits(golden_dir, impl):
    """Same parameter names as the reference GPTModel; same logits on the CPU in fp32."""
    model, ids, logits_ref = _load_tiny(golden_dir, impl)
    with torch.no_grad():
        logits = model(ids)
    torch.testing.assert_close(logits, logits_ref, rtol=1e-4, atol=2e-5)


def test_last_token_only(golden_dir):
    model, ids, logits_ref = _load_tiny(golden_dir, "manual")
    with torch.no_grad():
        last = model(ids, last_token_only=True)
    torch.testing.assert_close(last, logits_ref[:, -1:, :], rtol=1e-4, atol=2e-5)


def test_prepare_for_inference_is_a_pure_cache(golden_dir):
    """Fused QKV + padded head give the same logits and leave the state_dict untouched."""
    model, ids, logits_ref = _load_tiny(golden_dir, "manual")
    keys = sorted(model.state_dict().keys())
    model.prepare_for_inference()
    assert sorted(model.state_dict().keys()) == keys
    assert model._head_w is not None and model._head_w.shape[0] % 64 == 0   # vocab 97 -> 128
    with torch.no_grad():
        logits = model(ids)
    assert logits.shape == logits_ref.shape
    torch.testing.assert_close(logits, logits_ref, rtol=1e-4, atol=2e-5)


def test_kv_cache_forward_equals_full_forward(golden_dir):
    """Prompt in one pass, then token by token against the cache == one pass over everything
    (CPU, fp32, torch attention: checks the cache bookkeeping, positions and masks)."""
    model, ids, logits_ref = _load_tiny(golden_dir, "manual")
    caches = model.allocate_kv_cache(ids.shape[0], 48)
    with torch.no_grad():
        first = model(ids[:, :25], kv_caches=caches, pos=0)
        rest = [model(ids[:, t:t + 1], kv_caches=caches, pos=t) for t in range(25, ids.shape[1])]
    got = torch.cat([first] + rest, dim=1)
    torch.testing.assert_close(got, logits_ref, rtol=1e-4, atol=3e-5)


def test_generate_with_cache_equals_reference_style_recompute(golden_dir):
    model, ids, _ = _load_tiny(golden_dir, "manual")
    prompt = ids[:, :12]
    a = gpt2.generate(model, prompt, 8, 48, temperature=0.0)                    # cached, greedy
    b = gpt2.generate(model, prompt, 8, 48, temperature=0.0, use_cache=False)   # the reference's loop
    assert a.shape == (2, 20) and torch.equal(a, b)
    g1 = torch.Generator().manual_seed(3)
    g2 = torch.Generator().manual_seed(3)
    c = gpt2.generate(model, prompt, 5, 48, temperature=1.0, top_k=10, generator=g1)
    d = gpt2.generate(model, prompt, 5, 48, temperature=1.0, top_k=10, use_cache=False, generator=g2)
    assert torch.equal(c, d)
    # past the context length the cache cannot slide: the remaining tokens are produced as the
    # reference produces all of them, from the last context_size tokens (model_inference.py:202)
    e = gpt2.generate(model, ids, 20, 48, temperature=0.0)                       # 40 + 20 > 48
    f = gpt2.generate(model, ids, 20, 48, temperature=0.0, use_cache=False)
    assert e.shape == (2, 60) and torch.equal(e, f)
    long_prompt = torch.cat([ids, ids], dim=1)                                   # 80 > 48 from the start
    assert torch.equal(gpt2.generate(model, long_prompt, 3, 48, temperature=0.0),
                       gpt2.generate(model, long_prompt, 3, 48, temperature=0.0, use_cache=False))


def test_configs_and_flops():
    cfg = gpt2.gpt2_config("gpt2-xl")
    assert (cfg["emb_dim"], cfg["n_layers"], cfg["n_heads"]) == (1600, 48, 25)
    assert cfg["emb_dim"] // cfg["n_heads"] == 64
    assert abs(gpt2.prefill_flops_per_token(cfg, 1024) - (3.11e9 + 1.57e8)) / 3.27e9 < 0.01
    small = gpt2.gpt2_config("gpt2-small")
    assert abs(gpt2.prefill_flops_per_token(small, 1024) - (2.47e8 + 1.89e7)) / 2.66e8 < 0.01


@pytest.mark.gpu
def test_harness_with_cuda_kernel_matches_reference_logits(golden_dir, fa_lib):
    """impl_type="cuda": every layer's attention runs through the sm_100a kernel (bf16 under
    autocast, as in the reference); logits against the reference's fp32 CPU logits."""
    model, ids, logits_ref = _load_tiny(golden_dir, "cuda")
    model = model.cuda()
    with torch.no_grad():
        logits = model(ids.cuda()).float().cpu()
    from tfg_flashattention_b200 import custom_flash_attn
    assert custom_flash_attn.last_status() == 0
    # bf16 attention + bf16 projections under autocast against fp32: logits are O(1)
    assert (logits - logits_ref).abs().max().item() < 5e-2
    assert (logits - logits_ref).abs().mean().item() < 5e-3
    # and against the same model with torch's attention under the same autocast recipe
    model_f, _, _ = _load_tiny(golden_dir, "functional")
    with torch.no_grad():
        logits_f = model_f.cuda()(ids.cuda()).float().cpu()
    assert (logits - logits_f).abs().max().item() < 3e-2


@pytest.mark.gpu
def test_generation_with_decode_kernel(golden_dir, fa_lib):
    """impl_type="cuda": prompt through the prefill kernel, every new token through the decode
    kernel over the bf16 K/V cache; logits of the cached steps against the reference's fp32 logits
    and greedy tokens against the recompute loop."""
    model, ids, logits_ref = _load_tiny(golden_dir, "cuda")
    model = model.cuda()
    ids = ids.cuda()
    caches = model.allocate_kv_cache(ids.shape[0], 48)
    with torch.no_grad():
        first = model(ids[:, :25], kv_caches=caches, pos=0)
        rest = [model(ids[:, t:t + 1], kv_caches=caches, pos=t) for t in range(25, ids.shape[1])]
    got = torch.cat([first] + rest, dim=1).float().cpu()
    from tfg_flashattention_b200 import custom_flash_attn
    assert custom_flash_attn.last_status() == 0
    assert (got - logits_ref).abs().max().item() < 5e-2
    assert (got - logits_ref).abs().mean().item() < 5e-3
    a = gpt2.generate(model, ids[:, :12], 8, 48, temperature=0.0)
    b = gpt2.generate(model, ids[:, :12], 8, 48, temperature=0.0, use_cache=False)
    assert a.shape == (2, 20)
    # bf16 paths differ in rounding; greedy choices may part ways only at a near-tie
    assert (a == b).float().mean().item() >= 0.9


@pytest.mark.gpu
def test_bf16_model_prefill_small(fa_lib):
    """GPT-2 small, random init, whole model in bf16: "cuda" against "functional"."""
    cfg = gpt2.gpt2_config("gpt2-small")
    cfg["n_layers"] = 2
    m = gpt2.init_random(gpt2.GPTModel(cfg, dtype=torch.bfloat16), seed=1).cuda().eval()
    m.prepare_for_inference()
    ids = torch.randint(0, cfg["vocab_size"], (2, 1024), generator=torch.Generator().manual_seed(1)).cuda()
    with torch.no_grad():
        a = m(ids).float()
        for blk in m.trf_blocks:
            blk.att.impl_type = "functional"
        b = m(ids).float()
    assert torch.isfinite(a).all()
    assert (a - b).abs().max().item() < 5e-2


@pytest.mark.gpu
def test_decode_with_length_on_the_device(fa_lib):
    """kv_len as an int32 on the GPU: the launch is sized for the whole cache, the kernel reads the
    length when it runs; every length gives exactly what the host-side length gives."""
    from tfg_flashattention_b200 import custom_flash_attn as cfa
    torch.manual_seed(3)
    for B, H, cap in ((2, 3, 300), (32, 25, 128), (1, 1, 1000)):
        q = torch.randn(B, H, 64, device="cuda").bfloat16()
        k = torch.randn(B, H, cap, 64, device="cuda").bfloat16()
        v = torch.randn(B, H, cap, 64, device="cuda").bfloat16()
        length = torch.ones(1, dtype=torch.int32, device="cuda")
        for n in (1, 2, 63, 64, 65, cap // 2, cap - 1, cap):
            length.fill_(n)
            o_dev, lse_dev = cfa.decode(q, k, v, length, return_lse=True)
            o_host, lse_host = cfa.decode(q, k, v, n, return_lse=True)
            # the chunking differs (sized for `cap` instead of `n`): equal up to fp32 summation order
            torch.testing.assert_close(o_dev.float(), o_host.float(), rtol=0, atol=2e-2)
            torch.testing.assert_close(lse_dev, lse_host, rtol=1e-5, atol=1e-5)
        length.fill_(cap + 50)                      # clamped to the cache size
        torch.testing.assert_close(cfa.decode(q, k, v, length).float(), cfa.decode(q, k, v, cap).float(),
                                   rtol=0, atol=2e-2)
    assert cfa.last_status() == 0
    with pytest.raises(RuntimeError):
        cfa.decode(q, k, v, torch.ones(1, dtype=torch.int64, device="cuda"))


@pytest.mark.gpu
def test_generation_with_graph_replay_equals_eager_cache_path(golden_dir, fa_lib):
    """generate(cuda_graph=True): the single-token forward recorded once and replayed per token
    picks the same greedy tokens as the eager K/V-cache loop, on the fp32 and the bf16 model."""
    model, ids, _ = _load_tiny(golden_dir, "cuda")
    model = model.cuda()
    ids = ids.cuda()
    a = gpt2.generate(model, ids[:, :12], 10, 48, temperature=0.0)
    b = gpt2.generate(model, ids[:, :12], 10, 48, temperature=0.0, cuda_graph=True)
    assert torch.equal(a, b)
    cfg = {"vocab_size": 503, "context_length": 128, "emb_dim": 256, "n_heads": 4, "n_layers": 3,
           "drop_rate": 0.0, "qkv_bias": True, "impl_type": "cuda"}
    m = gpt2.init_random(gpt2.GPTModel(cfg, dtype=torch.bfloat16), seed=9, std=0.05).cuda().eval()
    m.prepare_for_inference()
    prompt = torch.randint(0, 503, (3, 40), device="cuda")
    a = gpt2.generate(m, prompt, 20, 128, temperature=0.0)
    b = gpt2.generate(m, prompt, 20, 128, temperature=0.0, cuda_graph=True)
    assert a.shape == b.shape == (3, 60)
    assert torch.equal(a, b)
    session = gpt2.GenerationSession(m, 3, 128)                 # recorded once, used for two prompts
    assert torch.equal(gpt2.generate(m, prompt, 20, 128, temperature=0.0, session=session), a)
    prompt2 = torch.randint(0, 503, (3, 17), device="cuda")
    assert torch.equal(gpt2.generate(m, prompt2, 9, 128, temperature=0.0, session=session),
                       gpt2.generate(m, prompt2, 9, 128, temperature=0.0))
    from tfg_flashattention_b200 import custom_flash_attn
    assert custom_flash_attn.last_status() == 0


@pytest.mark.gpu
def test_decode_appends_the_new_row_itself(fa_lib):
    """k_new / v_new: the kernel uses them as the newest row and writes them into the caches;
    same result as copying them in first, for host- and device-side lengths, split and unsplit."""
    from tfg_flashattention_b200 import custom_flash_attn as cfa
    torch.manual_seed(4)
    for B, H, cap, n in ((2, 3, 300, 137), (32, 25, 128, 128), (1, 2, 1000, 1), (1, 25, 1024, 700)):
        q = torch.randn(B, H, 64, device="cuda").bfloat16()
        k = torch.randn(B, H, cap, 64, device="cuda").bfloat16()
        v = torch.randn(B, H, cap, 64, device="cuda").bfloat16()
        qkv = torch.randn(B, 1, 3, H, 64, device="cuda").bfloat16()       # as the fused projection leaves them
        kn, vn = qkv[:, :, 1].transpose(1, 2), qkv[:, :, 2].transpose(1, 2)   # [B, H, 1, 64] views
        k_ref, v_ref = k.clone(), v.clone()
        k_ref[:, :, n - 1] = kn[:, :, 0]
        v_ref[:, :, n - 1] = vn[:, :, 0]
        want, lse_want = cfa.decode(q, k_ref, v_ref, n, return_lse=True)
        k1, v1 = k.clone(), v.clone()
        got, lse = cfa.decode(q, k1, v1, n, return_lse=True, k_new=kn, v_new=vn)
        assert torch.equal(got, want) and torch.equal(lse, lse_want)
        assert torch.equal(k1, k_ref) and torch.equal(v1, v_ref)        # appended, nothing else touched
        k2, v2 = k.clone(), v.clone()
        length = torch.full((1,), n, dtype=torch.int32, device="cuda")
        got2 = cfa.decode(q, k2, v2, length, k_new=kn, v_new=vn)
        assert torch.equal(k2, k_ref) and torch.equal(v2, v_ref)
        torch.testing.assert_close(got2.float(), want.float(), rtol=0, atol=2e-2)
    assert cfa.last_status() == 0
    with pytest.raises(RuntimeError):
        cfa.decode(q, k, v, 5, k_new=kn)
