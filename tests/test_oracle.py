"""The CPU oracle against (a) fixtures produced by the reference's own Python code, (b) torch's
scaled_dot_product_attention -- the comparison every reference test makes
(test/py/test_cuda_implementation.py:49-52, 83, 112) -- and (c) a float64 triple loop."""
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle.attention_oracle import (attention_python_loops, manual_attention,
                                     manual_attention_blocked, manual_attention_rows)
from oracle.gpt2_oracle import gpt_forward


def _cases(golden_dir):
    g = np.load(os.path.join(golden_dir, "attn_manual_cases.npz"))
    for c, (B, H, N) in enumerate(g["shapes"]):
        yield c, [torch.from_numpy(g[f"{x}_{c}"]) for x in "qkvo"]


def test_oracle_reproduces_reference_manual_branch(golden_dir):
    n = 0
    for c, (q, k, v, o_ref) in _cases(golden_dir):
        o = manual_attention(q, k, v, causal=True)
        assert torch.equal(o, o_ref), f"case {c}: oracle differs from the reference's manual branch"
        n += 1
    assert n == 9


def test_blocked_oracle_matches_dense(golden_dir):
    for c, (q, k, v, o_ref) in _cases(golden_dir):
        o, lse = manual_attention_blocked(q, k, v, causal=True, return_lse=True)
        _, lse_d = manual_attention(q, k, v, causal=True, return_lse=True)
        torch.testing.assert_close(o, o_ref, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(lse, lse_d, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("N", [10, 65, 128, 300])
def test_oracle_vs_torch_sdpa(N, causal):
    torch.manual_seed(N)
    q, k, v = (torch.randn(2, 3, N, 64) for _ in range(3))
    o, lse = manual_attention(q, k, v, causal=causal, return_lse=True)
    ref = F.scaled_dot_product_attention(q, k, v, is_causal=causal)
    torch.testing.assert_close(o, ref, rtol=1e-5, atol=2e-6)
    s = (q @ k.transpose(-1, -2)) / 8.0
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(N, N), 1).bool(), float("-inf"))
    torch.testing.assert_close(lse, torch.logsumexp(s, -1), rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("causal", [True, False])
def test_oracle_vs_float64_loops(causal):
    torch.manual_seed(5)
    q, k, v = (torch.randn(12, 64) for _ in range(3))
    o, lse = manual_attention(q[None, None], k[None, None], v[None, None], causal=causal, return_lse=True)
    o64, lse64 = attention_python_loops(q, k, v, causal=causal)
    torch.testing.assert_close(o[0, 0], torch.tensor(o64, dtype=torch.float32), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(lse[0, 0], torch.tensor(lse64, dtype=torch.float32), rtol=1e-5, atol=1e-6)


def test_row_subset_oracle():
    torch.manual_seed(6)
    q, k, v = (torch.randn(700, 64) for _ in range(3))
    rows = torch.tensor([0, 1, 127, 128, 255, 256, 511, 699])
    o, lse = manual_attention_rows(q, k, v, rows, causal=True)
    of, lf = manual_attention(q[None, None], k[None, None], v[None, None], return_lse=True)
    torch.testing.assert_close(o, of[0, 0, rows], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(lse, lf[0, 0, rows], rtol=1e-5, atol=1e-5)


def test_custom_scale():
    torch.manual_seed(8)
    q, k, v = (torch.randn(1, 2, 40, 64) for _ in range(3))
    o = manual_attention(q, k, v, causal=True, softmax_scale=0.2)
    ref = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=0.2)
    torch.testing.assert_close(o, ref, rtol=1e-5, atol=2e-6)


def test_gpt2_oracle_reproduces_reference_model(golden_dir):
    t = np.load(os.path.join(golden_dir, "gpt_tiny.npz"))
    sd = {k[3:]: torch.from_numpy(t[k]) for k in t.files if k.startswith("sd.")}
    logits = gpt_forward(sd, torch.from_numpy(t["ids"]), int(t["n_layers"]), int(t["n_heads"]))
    torch.testing.assert_close(logits, torch.from_numpy(t["logits"]), rtol=1e-5, atol=5e-6)
