"""Generate the golden fixtures in this folder from the REFERENCE project's own Python code.

Run once in a container that has the reference sources (they do not travel to the GPU box):

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's src/py/model_inference.py unmodified.  That file imports, at module
level, packages that are only needed by its benchmark driver and are absent here (matplotlib, the
compiled `custom_flash_attn` extension, gpt_download -> tensorflow, its Triton kernel); those
names are replaced by empty stand-in modules so that the import succeeds.  None of them is touched
by the code paths used below (`MultiHeadAttention` with impl_type="manual", `GPTModel`), which run
on the CPU in fp32.

Fixtures written (all float32 / int64 numpy arrays):
  attn_manual_cases.npz  for each case c: q_c, k_c, v_c [B,H,N,64] as the reference module formed
                         them (outputs of W_query/W_key/W_value, viewed and transposed,
                         model_inference.py:60-66) and o_c [B,H,N,64], the reference's
                         `attn_weights @ values` (:75) recovered from the tensor it feeds out_proj.
  gpt_tiny.npz           a 2-layer GPTModel (emb 128, 2 heads of 64, vocab 97, ctx 48, qkv_bias
                         as the reference driver sets it, :422): every state_dict entry, the token
                         (the `att.mask` buffers included), the token ids, and the logits.
  loader_tiny.npz        a synthetic parameter dictionary in the OpenAI checkpoint layout
                         (`p.<path>` entries: wte, wpe, g, b, blocks.<i>.attn.c_attn.w ...) and the
                         state_dict (`sd.<name>`) of a reference GPTModel after the reference's own
                         load_weights_into_gpt(gpt, params) (model_inference.py:313-376) ran on it.
"""
import sys
import types

import numpy as np
import torch

CASES = [  # (B, H, N) -- the reference tests' ragged lengths (test_cuda_implementation.py:93) and a few more
    (2, 2, 10), (2, 2, 11), (1, 2, 15), (2, 2, 33), (1, 2, 63), (2, 2, 65),
    (1, 2, 128), (1, 1, 200), (1, 1, 300),
]


def import_reference(ref_root):
    for name in ("matplotlib", "matplotlib.pyplot", "custom_flash_attn", "gpt_download",
                 "triton_implementation"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["matplotlib"].use = lambda *a, **k: None
    sys.modules["matplotlib"].pyplot = sys.modules["matplotlib.pyplot"]
    sys.modules["gpt_download"].download_and_load_gpt2 = None
    sys.modules["triton_implementation"]._flash_attn_forward = None
    sys.dont_write_bytecode = True
    sys.path.insert(0, f"{ref_root}/src/py")
    import model_inference
    return model_inference


def attention_cases(mi):
    out = {}
    for c, (B, H, N) in enumerate(CASES):
        torch.manual_seed(1000 + c)
        d_model = H * 64
        mha = mi.MultiHeadAttention(d_model, d_model, 512, 0.0, H, "manual", qkv_bias=True).eval()
        with torch.no_grad():
            for lin in (mha.W_query, mha.W_key, mha.W_value):
                lin.weight.mul_(3.0)       # spread the scores so the softmax is not near-uniform
        cap = {}
        hooks = [
            mha.W_query.register_forward_hook(lambda m, i, o: cap.__setitem__("q", o.detach().clone())),
            mha.W_key.register_forward_hook(lambda m, i, o: cap.__setitem__("k", o.detach().clone())),
            mha.W_value.register_forward_hook(lambda m, i, o: cap.__setitem__("v", o.detach().clone())),
            mha.out_proj.register_forward_pre_hook(lambda m, i: cap.__setitem__("ctx", i[0].detach().clone())),
        ]
        with torch.no_grad():
            mha(torch.randn(B, N, d_model))
        for h in hooks:
            h.remove()
        to_bhnd = lambda t: t.view(B, N, H, 64).transpose(1, 2).contiguous().numpy()
        out[f"q_{c}"], out[f"k_{c}"], out[f"v_{c}"] = (to_bhnd(cap[x]) for x in "qkv")
        out[f"o_{c}"] = to_bhnd(cap["ctx"])     # ctx is [B,N,H*64] after the reference's transpose(1,2)
    out["shapes"] = np.array(CASES, dtype=np.int64)
    return out


def gpt_tiny(mi):
    cfg = {"vocab_size": 97, "context_length": 48, "emb_dim": 128, "n_heads": 2, "n_layers": 2,
           "drop_rate": 0.0, "qkv_bias": True, "impl_type": "manual"}
    torch.manual_seed(7)
    gpt = mi.GPTModel(cfg).eval()
    ids = torch.randint(0, cfg["vocab_size"], (2, 40))
    import warnings
    with torch.no_grad(), warnings.catch_warnings():
        warnings.simplefilter("ignore")   # autocast("cuda") warns on a CPU-only box and is inert
        logits = gpt(ids)
    out = {f"sd.{k}": v.detach().numpy() for k, v in gpt.state_dict().items()}   # unmodified, `att.mask` included
    out["ids"] = ids.numpy()
    out["logits"] = logits.numpy()
    out["n_layers"] = np.array(cfg["n_layers"])
    out["n_heads"] = np.array(cfg["n_heads"])
    return out


LOADER_CFG = {"vocab_size": 31, "context_length": 8, "emb_dim": 32, "n_heads": 2, "n_layers": 2,
              "drop_rate": 0.0, "qkv_bias": True, "impl_type": "manual"}


def openai_params(cfg, seed):
    """A parameter dictionary in the checkpoint's own layout ([in, out] weights, fused c_attn)."""
    rng = np.random.default_rng(seed)
    d, v, ctx = cfg["emb_dim"], cfg["vocab_size"], cfg["context_length"]
    f = lambda *shape: rng.normal(0.0, 0.05, shape).astype(np.float32)
    blocks = [{"attn": {"c_attn": {"w": f(d, 3 * d), "b": f(3 * d)}, "c_proj": {"w": f(d, d), "b": f(d)}},
               "mlp": {"c_fc": {"w": f(d, 4 * d), "b": f(4 * d)}, "c_proj": {"w": f(4 * d, d), "b": f(d)}},
               "ln_1": {"g": 1 + f(d), "b": f(d)}, "ln_2": {"g": 1 + f(d), "b": f(d)}}
              for _ in range(cfg["n_layers"])]
    return {"wte": f(v, d), "wpe": f(ctx, d), "g": 1 + f(d), "b": f(d), "blocks": blocks}


def _flatten(prefix, node, out):
    if isinstance(node, dict):
        for k, v in node.items():
            _flatten(f"{prefix}.{k}" if prefix else k, v, out)
    elif isinstance(node, list):
        for i, v in enumerate(node):
            _flatten(f"{prefix}.{i}", v, out)
    else:
        out[prefix] = node


def loader_tiny(mi):
    params = openai_params(LOADER_CFG, 5)
    torch.manual_seed(9)
    gpt = mi.GPTModel(LOADER_CFG).eval()
    mi.load_weights_into_gpt(gpt, params)           # the reference's loader, unmodified
    flat = {}
    _flatten("", params, flat)
    out = {f"p.{k}": v for k, v in flat.items()}
    out.update({f"sd.{k}": v.detach().numpy() for k, v in gpt.state_dict().items()})
    return out


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    ref_root = sys.argv[1]
    here = __file__.rsplit("/", 1)[0]
    mi = import_reference(ref_root)
    np.savez_compressed(f"{here}/attn_manual_cases.npz", **attention_cases(mi))
    np.savez_compressed(f"{here}/gpt_tiny.npz", **gpt_tiny(mi))
    np.savez_compressed(f"{here}/loader_tiny.npz", **loader_tiny(mi))
    print("wrote", f"{here}/attn_manual_cases.npz", f"{here}/gpt_tiny.npz", f"{here}/loader_tiny.npz")
