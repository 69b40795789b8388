"""CPU oracle for the attention hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in fp32 on the CPU, the reference project's standard-PyTorch ("manual")
attention branch -- src/py/model_inference.py:55 (mask buffer) and :68-75 (the branch) -- which
is what the reference defines as correct for its CUDA kernel's inputs.  It is the checker for the
CUDA path; nothing in the product imports it.  Only tests/, __graft_entry__.smoke() and
bench.py's CPU-baseline / reference arm may call it.

Parity pin: tests/golden/*.npz were produced by importing the reference's own
`MultiHeadAttention` (impl_type="manual") and `GPTModel` in a container that holds the reference
sources (tests/golden/make_golden.py); tests/test_oracle.py checks this restatement against those
files, and against torch's scaled_dot_product_attention, which is what every reference test
compares with (test/py/test_cuda_implementation.py:49-52, 83, 112).
LSE and the non-causal mode have no counterpart in the reference's CUDA path; they are pinned here
against torch.logsumexp / unmasked softmax ("parity unpinned" by the reference itself for these
two outputs).  LSE follows the only definition the reference contains: m + log(l) on the scaled
scores (src/py/triton_implementation.py:129-132, 153-154).
"""
from __future__ import annotations

import math

import torch


def manual_attention(q, k, v, causal=True, softmax_scale=None, return_lse=False):
    """softmax(mask(q k^T) / sqrt(d)) v, written the way the reference writes it.

    q, k, v: [B, H, N, d] tensors (any float dtype; computed in fp32 on the CPU).
    Follows src/py/model_inference.py:68-75 statement by statement:
      :69  attn = queries @ keys.transpose(-2, -1)
      :70  mask_bool = triu(ones(ctx, ctx), diagonal=1).bool()[:N, :N]      (buffer from :55)
      :71  attn.masked_fill_(mask_bool, -inf)
      :72  attn_weights = softmax(attn / d ** 0.5, dim=-1)
      :73  dropout (p = 0 at inference: identity)
      :75  context = attn_weights @ values          (before the transpose(1, 2) of the call site)
    Returns O [B, H, N, d] fp32, and LSE [B, H, N] fp32 when asked.
    """
    q = q.detach().to("cpu", torch.float32)
    k = k.detach().to("cpu", torch.float32)
    v = v.detach().to("cpu", torch.float32)
    n, d = q.shape[-2], q.shape[-1]
    attn = q @ k.transpose(-2, -1)
    if causal:
        mask_bool = torch.triu(torch.ones(n, n), diagonal=1).bool()
        attn.masked_fill_(mask_bool, -torch.inf)
    if softmax_scale is None:
        scaled = attn / d ** 0.5
    else:
        scaled = attn * softmax_scale
    attn_weights = torch.softmax(scaled, dim=-1)
    out = attn_weights @ v
    if return_lse:
        return out, torch.logsumexp(scaled, dim=-1)
    return out


def manual_attention_rows(q, k, v, rows, causal=True, softmax_scale=None):
    """The same arithmetic for a subset of query rows of ONE head, for sequences whose full
    N x N score matrix is too large to hold (N up to 32768).

    q, k, v: [N, d];  rows: 1-D LongTensor of query indices.
    Returns (O[rows] fp32 [R, d], LSE[rows] fp32 [R]).
    """
    q = q.detach().to("cpu", torch.float32)
    k = k.detach().to("cpu", torch.float32)
    v = v.detach().to("cpu", torch.float32)
    n, d = k.shape
    scale = (1.0 / d ** 0.5) if softmax_scale is None else softmax_scale
    outs, lses = [], []
    for start in range(0, rows.numel(), 256):
        r = rows[start:start + 256]
        s = q[r] @ k.t()
        if causal:
            cols = torch.arange(n)
            s.masked_fill_(cols[None, :] > r[:, None], -torch.inf)
        s = s * scale
        outs.append(torch.softmax(s, dim=-1) @ v)
        lses.append(torch.logsumexp(s, dim=-1))
    return torch.cat(outs), torch.cat(lses)


def manual_attention_blocked(q, k, v, causal=True, softmax_scale=None, return_lse=False):
    """manual_attention evaluated one (batch, head) at a time in 256-row blocks, so that the
    score matrix held at any moment is 256 x N.  Same results, bounded memory."""
    B, H, N, d = q.shape
    out = torch.empty(B, H, N, d, dtype=torch.float32)
    lse = torch.empty(B, H, N, dtype=torch.float32)
    rows = torch.arange(N)
    for b in range(B):
        for h in range(H):
            o_, l_ = manual_attention_rows(q[b, h], k[b, h], v[b, h], rows, causal, softmax_scale)
            out[b, h] = o_
            lse[b, h] = l_
    return (out, lse) if return_lse else out


def attention_python_loops(q, k, v, causal=True):
    """Triple-loop float64 evaluation for tiny cases (an arithmetic cross-check of the tensor
    formulation above that shares no library call with it).  q, k, v: [N, d] nested lists or
    tensors of one head.  Returns (O as list of lists, LSE as list)."""
    q = [[float(x) for x in row] for row in q]
    k = [[float(x) for x in row] for row in k]
    v = [[float(x) for x in row] for row in v]
    n, d = len(q), len(q[0])
    scale = 1.0 / math.sqrt(d)
    out, lse = [], []
    for i in range(n):
        last = i if causal else n - 1
        s = [scale * sum(q[i][c] * k[j][c] for c in range(d)) for j in range(last + 1)]
        m = max(s)
        e = [math.exp(x - m) for x in s]
        z = sum(e)
        out.append([sum(e[j] * v[j][c] for j in range(last + 1)) / z for c in range(d)])
        lse.append(m + math.log(z))
    return out, lse
