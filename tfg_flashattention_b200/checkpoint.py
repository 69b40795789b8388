"""OpenAI GPT-2 parameters -> GPTModel, without TensorFlow.

The reference fills its model from the nested dictionary that its downloader builds out of the
TensorFlow checkpoint (`load_weights_into_gpt(gpt, params)`, src/py/model_inference.py:313-376;
the dictionary comes from gpt_download.py): top-level `wte`, `wpe`, `g`, `b` and a list `blocks`
whose entries hold `attn.c_attn`, `attn.c_proj`, `mlp.c_fc`, `mlp.c_proj` (each `{w, b}`, weights
stored `[in, out]`) and `ln_1`, `ln_2` (each `{g, b}`).  Reading the TensorFlow checkpoint itself
needs TensorFlow, which the attention path has no use for; this module takes the same dictionary
from any source and adds a flat `.npz` form of it (`blocks.3.attn.c_attn.w`, ...) that numpy alone
reads and writes, so a checkpoint converted once elsewhere can be loaded from a local path.

`load_weights_into_gpt` keeps the reference's name, argument order and error behaviour (a
`ValueError` naming both shapes on any mismatch); the fused c_attn matrix is cut into the
W_query / W_key / W_value parameters the way the reference cuts it (three equal column blocks,
transposed to `[out, in]`), and the output head is tied to `wte`.
"""
from __future__ import annotations

import numpy as np
import torch

# (parameter of a TransformerBlock, path inside params["blocks"][i], stored transposed?)
_BLOCK_MAP = (
    ("att.out_proj.weight", ("attn", "c_proj", "w"), True),
    ("att.out_proj.bias", ("attn", "c_proj", "b"), False),
    ("ff.layers.0.weight", ("mlp", "c_fc", "w"), True),
    ("ff.layers.0.bias", ("mlp", "c_fc", "b"), False),
    ("ff.layers.2.weight", ("mlp", "c_proj", "w"), True),
    ("ff.layers.2.bias", ("mlp", "c_proj", "b"), False),
    ("norm1.scale", ("ln_1", "g"), False),
    ("norm1.shift", ("ln_1", "b"), False),
    ("norm2.scale", ("ln_2", "g"), False),
    ("norm2.shift", ("ln_2", "b"), False),
)
_LEAVES = (("attn", "c_attn", "w"), ("attn", "c_attn", "b")) + tuple(path for _, path, _ in _BLOCK_MAP)


def _dig(tree, path):
    for key in path:
        tree = tree[key]
    return tree


def _assign(param: torch.nn.Parameter, value, what: str) -> None:
    value = np.asarray(value)
    if tuple(param.shape) != tuple(value.shape):
        raise ValueError(f"Shape mismatch. Left: {tuple(param.shape)}, Right: {tuple(value.shape)} ({what})")
    with torch.no_grad():
        param.copy_(torch.from_numpy(np.ascontiguousarray(value)).to(param.dtype))


def load_weights_into_gpt(gpt, params) -> None:
    """Copy an OpenAI-layout parameter dictionary into `gpt` (a GPTModel), in place."""
    if len(params["blocks"]) != len(gpt.trf_blocks):
        raise ValueError(f"Shape mismatch. Left: {len(gpt.trf_blocks)} blocks, "
                         f"Right: {len(params['blocks'])} blocks")
    _assign(gpt.pos_emb.weight, params["wpe"], "wpe")
    _assign(gpt.tok_emb.weight, params["wte"], "wte")
    for i, (block, src) in enumerate(zip(gpt.trf_blocks, params["blocks"])):
        named = dict(block.named_parameters())
        w = np.asarray(_dig(src, ("attn", "c_attn", "w")))
        b = np.asarray(_dig(src, ("attn", "c_attn", "b")))
        if w.shape[-1] % 3 or b.shape[-1] % 3:
            raise ValueError(f"Shape mismatch. Left: 3 equal parts, Right: {w.shape} (blocks.{i}.attn.c_attn)")
        for name, w_part, b_part in zip(("W_query", "W_key", "W_value"),
                                        np.split(w, 3, axis=-1), np.split(b, 3, axis=-1)):
            _assign(named[f"att.{name}.weight"], w_part.T, f"blocks.{i}.{name}.weight")
            if f"att.{name}.bias" in named:
                _assign(named[f"att.{name}.bias"], b_part, f"blocks.{i}.{name}.bias")
        for target, path, transposed in _BLOCK_MAP:
            value = np.asarray(_dig(src, path))
            _assign(named[target], value.T if transposed else value, f"blocks.{i}." + ".".join(path))
    _assign(gpt.final_norm.scale, params["g"], "g")
    _assign(gpt.final_norm.shift, params["b"], "b")
    _assign(gpt.out_head.weight, params["wte"], "out_head <- wte")
    if hasattr(gpt, "invalidate_inference_cache"):
        gpt.invalidate_inference_cache()


def params_from_gpt(gpt) -> dict:
    """The inverse: a GPTModel's parameters in the OpenAI layout (the head is assumed tied)."""
    def np32(t):
        return t.detach().float().cpu().numpy()
    blocks = []
    for block in gpt.trf_blocks:
        named = dict(block.named_parameters())
        qkv_w = [np32(named[f"att.{n}.weight"]).T for n in ("W_query", "W_key", "W_value")]
        d_out = qkv_w[0].shape[1]
        qkv_b = [np32(named[f"att.{n}.bias"]) if f"att.{n}.bias" in named else np.zeros(d_out, np.float32)
                 for n in ("W_query", "W_key", "W_value")]
        tree = {"attn": {"c_attn": {"w": np.concatenate(qkv_w, axis=-1), "b": np.concatenate(qkv_b, axis=-1)},
                         "c_proj": {}}, "mlp": {"c_fc": {}, "c_proj": {}}, "ln_1": {}, "ln_2": {}}
        for target, path, transposed in _BLOCK_MAP:
            value = np32(named[target])
            _dig(tree, path[:-1])[path[-1]] = value.T.copy() if transposed else value
        blocks.append(tree)
    return {"wte": np32(gpt.tok_emb.weight), "wpe": np32(gpt.pos_emb.weight),
            "g": np32(gpt.final_norm.scale), "b": np32(gpt.final_norm.shift), "blocks": blocks}


def save_params_npz(path: str, params: dict) -> None:
    """Write the dictionary as one flat .npz (keys `wte`, `blocks.0.attn.c_attn.w`, ...)."""
    flat = {k: np.asarray(params[k]) for k in ("wte", "wpe", "g", "b")}
    for i, src in enumerate(params["blocks"]):
        for leaf in _LEAVES:
            flat[f"blocks.{i}." + ".".join(leaf)] = np.asarray(_dig(src, leaf))
    np.savez(path, **flat)


def load_params_npz(path: str) -> dict:
    """Read a file written by `save_params_npz` back into the nested dictionary."""
    with np.load(path) as data:
        params = {k: data[k] for k in ("wte", "wpe", "g", "b")}
        n_blocks = 1 + max(int(k.split(".")[1]) for k in data.files if k.startswith("blocks."))
        params["blocks"] = []
        for i in range(n_blocks):
            tree: dict = {}
            for leaf in _LEAVES:
                node = tree
                for key in leaf[:-1]:
                    node = node.setdefault(key, {})
                node[leaf[-1]] = data[f"blocks.{i}." + ".".join(leaf)]
            params["blocks"].append(tree)
    return params
