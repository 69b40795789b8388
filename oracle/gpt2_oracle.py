"""CPU oracle for the caller of the attention hot path: the reference's GPT-2 forward with its
standard-PyTorch ("manual") attention.  TEST INFRASTRUCTURE ONLY -- never imported by the product.

Restates src/py/model_inference.py:39-190 functionally (plain tensors in a dict instead of
nn.Module objects), in fp32 on the CPU:
  LayerNorm          :96-107   eps 1e-5, biased variance, scale/shift
  GELU (tanh form)   :109-117
  FeedForward        :119-128  Linear(d, 4d) -> GELU -> Linear(4d, d)
  MultiHeadAttention :57-94    separate W_query/W_key/W_value (+bias), view to [B,H,N,d],
                               manual attention (:68-75), transpose(1,2), out_proj
  TransformerBlock   :149-164  pre-LN, residuals; dropout is identity at inference
  GPTModel           :180-190  tok_emb + pos_emb -> blocks -> final_norm -> out_head (no bias)

The reference wraps attention in torch.autocast("cuda", bfloat16) (:153); on the CPU that context
is inert, so the oracle is plain fp32, which is what "the reference's standard-PyTorch attention"
computes when run on host cores.

Parameter naming matches the reference's state_dict keys (e.g. "trf_blocks.0.att.W_query.weight"),
so a state_dict of the reference GPTModel can be fed in unchanged; tests/golden/make_golden.py
does exactly that to pin this file.
"""
from __future__ import annotations

import math

import torch

from .attention_oracle import manual_attention


def layer_norm(x, scale, shift, eps=1e-5):
    mean = x.mean(dim=-1, keepdim=True)
    var = x.var(dim=-1, keepdim=True, unbiased=False)
    return (x - mean) / torch.sqrt(var + eps) * scale + shift


def gelu_tanh(x):
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def linear(x, w, b=None):
    y = x @ w.t()
    return y if b is None else y + b


def attention_block(x, sd, prefix, n_heads):
    b, n, d_model = x.shape
    hd = d_model // n_heads

    def proj(name):
        w = sd[f"{prefix}.{name}.weight"]
        bias = sd.get(f"{prefix}.{name}.bias")
        return linear(x, w, bias).view(b, n, n_heads, hd).transpose(1, 2)

    q, k, v = proj("W_query"), proj("W_key"), proj("W_value")
    ctx = manual_attention(q, k, v, causal=True).transpose(1, 2).contiguous().view(b, n, d_model)
    return linear(ctx, sd[f"{prefix}.out_proj.weight"], sd[f"{prefix}.out_proj.bias"])


def gpt_forward(sd, in_idx, n_layers, n_heads):
    """Logits [B, N, vocab] of the reference GPTModel for token ids in_idx [B, N]."""
    sd = {k: v.detach().to("cpu", torch.float32) for k, v in sd.items() if v.dtype.is_floating_point}
    b, n = in_idx.shape
    x = sd["tok_emb.weight"][in_idx] + sd["pos_emb.weight"][torch.arange(n)]
    for i in range(n_layers):
        p = f"trf_blocks.{i}"
        shortcut = x
        h = layer_norm(x, sd[f"{p}.norm1.scale"], sd[f"{p}.norm1.shift"])
        x = attention_block(h, sd, f"{p}.att", n_heads) + shortcut
        shortcut = x
        h = layer_norm(x, sd[f"{p}.norm2.scale"], sd[f"{p}.norm2.shift"])
        h = linear(h, sd[f"{p}.ff.layers.0.weight"], sd[f"{p}.ff.layers.0.bias"])
        h = gelu_tanh(h)
        h = linear(h, sd[f"{p}.ff.layers.2.weight"], sd[f"{p}.ff.layers.2.bias"])
        x = h + shortcut
    x = layer_norm(x, sd["final_norm.scale"], sd["final_norm.shift"])
    return linear(x, sd["out_head.weight"])
