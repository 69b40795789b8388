"""Loading OpenAI-layout GPT-2 parameters (the reference's load_weights_into_gpt) on the CPU."""
import os

import numpy as np
import pytest
import torch

from oracle import gpt2_oracle
from tfg_flashattention_b200 import checkpoint, gpt2

CFG = {"vocab_size": 97, "context_length": 48, "emb_dim": 128, "n_heads": 2, "n_layers": 2,
       "drop_rate": 0.0, "qkv_bias": True, "impl_type": "manual"}


def _openai_params(seed):
    """A parameter dictionary in the checkpoint's own layout ([in, out] weights, fused c_attn)."""
    rng = np.random.default_rng(seed)
    d, v, ctx = CFG["emb_dim"], CFG["vocab_size"], CFG["context_length"]
    f = lambda *shape: rng.normal(0.0, 0.05, shape).astype(np.float32)
    blocks = [{"attn": {"c_attn": {"w": f(d, 3 * d), "b": f(3 * d)}, "c_proj": {"w": f(d, d), "b": f(d)}},
               "mlp": {"c_fc": {"w": f(d, 4 * d), "b": f(4 * d)}, "c_proj": {"w": f(4 * d, d), "b": f(d)}},
               "ln_1": {"g": 1 + f(d), "b": f(d)}, "ln_2": {"g": 1 + f(d), "b": f(d)}}
              for _ in range(CFG["n_layers"])]
    return {"wte": f(v, d), "wpe": f(ctx, d), "g": 1 + f(d), "b": f(d), "blocks": blocks}


def test_loaded_model_computes_what_the_layout_means():
    """x @ c_attn.w + b cut into q|k|v, [in,out] weights, tied head: checked through the logits of
    the CPU oracle fed with the same numbers under the model's own parameter names."""
    params = _openai_params(0)
    model = gpt2.GPTModel(CFG).eval()
    checkpoint.load_weights_into_gpt(model, params)
    blk0 = params["blocks"][0]
    d = CFG["emb_dim"]
    np.testing.assert_array_equal(model.trf_blocks[0].att.W_key.weight.detach().numpy(),
                                  blk0["attn"]["c_attn"]["w"][:, d:2 * d].T)
    np.testing.assert_array_equal(model.trf_blocks[0].att.W_value.bias.detach().numpy(), blk0["attn"]["c_attn"]["b"][2 * d:])
    np.testing.assert_array_equal(model.trf_blocks[1].ff.layers[2].weight.detach().numpy(),
                                  params["blocks"][1]["mlp"]["c_proj"]["w"].T)
    np.testing.assert_array_equal(model.out_head.weight.detach().numpy(), params["wte"])
    ids = torch.randint(0, CFG["vocab_size"], (2, 33), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        logits = model(ids)
    sd = {k: v.detach() for k, v in model.state_dict().items()}
    ref = gpt2_oracle.gpt_forward(sd, ids, n_layers=CFG["n_layers"], n_heads=CFG["n_heads"])
    torch.testing.assert_close(logits, ref, rtol=1e-4, atol=2e-5)


def test_round_trip_through_npz(tmp_path):
    params = _openai_params(1)
    path = os.path.join(tmp_path, "gpt2_tiny.npz")
    checkpoint.save_params_npz(path, params)
    back = checkpoint.load_params_npz(path)
    a, b = gpt2.GPTModel(CFG).eval(), gpt2.GPTModel(CFG).eval()
    checkpoint.load_weights_into_gpt(a, params)
    checkpoint.load_weights_into_gpt(b, back)
    for (ka, va), (kb, vb) in zip(a.state_dict().items(), b.state_dict().items()):
        assert ka == kb and torch.equal(va, vb)
    again = checkpoint.params_from_gpt(a)
    np.testing.assert_array_equal(again["blocks"][1]["attn"]["c_attn"]["w"], params["blocks"][1]["attn"]["c_attn"]["w"])
    np.testing.assert_array_equal(again["blocks"][0]["mlp"]["c_fc"]["w"], params["blocks"][0]["mlp"]["c_fc"]["w"])


def test_shape_mismatch_raises_value_error_like_the_reference():
    params = _openai_params(2)
    params["blocks"][1]["mlp"]["c_fc"]["w"] = params["blocks"][1]["mlp"]["c_fc"]["w"][:, :-1]
    with pytest.raises(ValueError, match="Shape mismatch"):
        checkpoint.load_weights_into_gpt(gpt2.GPTModel(CFG), params)
    params = _openai_params(3)
    params["blocks"].pop()
    with pytest.raises(ValueError, match="Shape mismatch"):
        checkpoint.load_weights_into_gpt(gpt2.GPTModel(CFG), params)


def test_loading_drops_stale_inference_caches():
    model = gpt2.GPTModel(CFG).eval()
    checkpoint.load_weights_into_gpt(model, _openai_params(4))
    model.prepare_for_inference()
    ids = torch.arange(20).reshape(1, 20) % CFG["vocab_size"]
    checkpoint.load_weights_into_gpt(model, _openai_params(5))
    fresh = gpt2.GPTModel(CFG).eval()
    checkpoint.load_weights_into_gpt(fresh, _openai_params(5))
    with torch.no_grad():
        torch.testing.assert_close(model(ids), fresh(ids))


def test_same_state_dict_as_the_reference_loader(golden_dir, tmp_path):
    """tests/golden/loader_tiny.npz holds a parameter dictionary and the state_dict the
    reference's own load_weights_into_gpt (model_inference.py:313-376) made of it; this loader
    must produce the same state_dict bit for bit -- and the reference's dict, `att.mask` buffers
    included, must load into the harness model with strict=True."""
    t = np.load(os.path.join(golden_dir, "loader_tiny.npz"))
    cfg = {"vocab_size": 31, "context_length": 8, "emb_dim": 32, "n_heads": 2, "n_layers": 2,
           "drop_rate": 0.0, "qkv_bias": True, "impl_type": "manual"}
    flat = os.path.join(tmp_path, "flat.npz")
    np.savez(flat, **{k[2:]: t[k] for k in t.files if k.startswith("p.")})
    params = checkpoint.load_params_npz(flat)
    model = gpt2.GPTModel(cfg).eval()
    checkpoint.load_weights_into_gpt(model, params)
    ref_sd = {k[3:]: torch.from_numpy(t[k]) for k in t.files if k.startswith("sd.")}
    ours = model.state_dict()
    assert sorted(ours.keys()) == sorted(ref_sd.keys())          # incl. trf_blocks.N.att.mask
    for k, v in ref_sd.items():
        assert torch.equal(ours[k], v), k
    other = gpt2.GPTModel(cfg).eval()
    other.load_state_dict(ref_sd, strict=True)
    for k, v in ref_sd.items():
        assert torch.equal(other.state_dict()[k], v), k
