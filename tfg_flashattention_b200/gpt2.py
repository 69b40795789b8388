"""GPT-2 prefill harness: the caller of the attention hot path.

Mirrors the reference's model (src/py/model_inference.py:39-190) module for module and parameter
name for parameter name, so a reference state_dict loads unchanged (strict=True, including the
`att.mask` buffers the reference stores, which are dropped on load and regenerated on export):

    MultiHeadAttention  :39-94    W_query / W_key / W_value / out_proj, impl_type dispatch
    LayerNorm           :96-107   scale / shift, eps 1e-5, biased variance
    GELU                :109-117  tanh form
    FeedForward         :119-128  layers.0 / layers.2
    TransformerBlock    :149-164  pre-LN, attention under bf16 autocast
    GPTModel            :180-190  tok_emb + pos_emb -> trf_blocks -> final_norm -> out_head

What differs, on purpose:
  * impl_type "cuda" calls this package's `custom_flash_attn.forward` on the strided
    `[B,N,H,d] -> transpose(1,2)` views directly.  The reference makes three `.contiguous()`
    copies first (:86-90); the kernel reads the views in place through its TMA descriptors and
    writes O in `[B,N,H,d]` memory, so the copy back is free as well.
  * the reference's "cuda" and "triton" branches forget the `transpose(1, 2)` that its "manual"
    and "functional" branches apply before `.view(b, n, d_out)` (:75, :80 against :83, :86-92),
    which scrambles heads and tokens.  Parity is defined against the "manual" branch, so the
    transpose is applied here.
  * LayerNorm and GELU call the fused torch ops (same arithmetic, one kernel each).
  * `prepare_for_inference()` builds two derived, cached tensors without touching the parameters
    (so state_dicts stay interchangeable): the three QKV projections concatenated into one
    `[3*d_model, d_model]` weight (one GEMM instead of three; q, k, v become column slices of one
    buffer, which the kernel reads in place), and the output head padded from 50257 to a
    multiple of 64 rows (an odd vocabulary size sends the logits GEMM down a slow unaligned
    cuBLAS path); the padded logits are sliced back to the vocabulary size.
  * `GPTModel(cfg, dtype=torch.bfloat16)` builds the whole model in bf16 (the prefill benchmark
    configuration); the default keeps the reference's precision recipe: fp32 everywhere, bf16
    autocast around attention only (:153-154).

  * generation keeps a K/V cache: `generate()` has the reference's signature and sampling rules
    (:199-228) but runs the prompt once through the prefill kernel and every further token
    through the single-query decode kernel, instead of re-running the whole prefix per token.
    `use_cache=False` reproduces the reference's recompute loop (for comparison).

  * `load_weights_into_gpt(gpt, params)` (:313-376) lives in `checkpoint.py`.

"manual" and "functional" branches are kept for comparison on any device; "cuda" has no fallback.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

GPT2_SIZES = {   # model_inference.py:392-397
    "gpt2-small": {"emb_dim": 768, "n_layers": 12, "n_heads": 12},
    "gpt2-medium": {"emb_dim": 1024, "n_layers": 24, "n_heads": 16},
    "gpt2-large": {"emb_dim": 1280, "n_layers": 36, "n_heads": 20},
    "gpt2-xl": {"emb_dim": 1600, "n_layers": 48, "n_heads": 25},
}


def gpt2_config(name: str, impl_type: str = "cuda", context_length: int = 1024) -> dict:
    """GPT_CONFIG_124M (:378-386) updated the way the reference driver does (:420-422)."""
    cfg = {"vocab_size": 50257, "context_length": context_length, "drop_rate": 0.0,
           "qkv_bias": True, "impl_type": impl_type}
    cfg.update(GPT2_SIZES[name])
    return cfg


def _few_rows(x, enabled, limit=1) -> bool:
    """True when `x` holds at most `limit` token rows on the bf16 GPU path: its Linear layer then
    goes through block_ops.linear_small (one pass over the weights) instead of a tiled GEMM.
    Measured on B200 against cuBLAS inside CUDA graphs: for one row the kernel is equal (QKV, first
    MLP layer) or up to 2x faster (K = 4 * d_model, d_model x d_model, the vocabulary head); from
    two rows on cuBLAS wins on the wide layers, except for the head (faster up to 8 rows)."""
    return (enabled and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0
            and x.numel() // x.shape[-1] <= limit and x.shape[-1] <= 8192)


class DevicePosition:
    """Where the next token goes, kept on the GPU so that a recorded decode step needs no host
    value: `index` (int64 [1]) addresses the cache row and the position embedding, `length`
    (int32 [1]) = index + 1 is what the decode kernel reads as the number of valid rows."""

    def __init__(self, device):
        self.index = torch.zeros(1, dtype=torch.long, device=device)
        self.length = torch.ones(1, dtype=torch.int32, device=device)

    def set(self, pos: int):
        self.index.fill_(pos)
        self.length.fill_(pos + 1)

    def advance(self):
        self.index.add_(1)
        self.length.add_(1)


class MultiHeadAttention(nn.Module):
    def __init__(self, d_in, d_out, context_length, dropout, num_heads, impl_type, qkv_bias=False):
        super().__init__()
        assert d_out % num_heads == 0, "d_out must be a multiple of num_heads"
        self.head_dim = d_out // num_heads
        self.num_heads = num_heads
        self.d_out = d_out
        self.impl_type = impl_type
        self.W_query = nn.Linear(d_in, d_out, bias=qkv_bias)
        self.W_key = nn.Linear(d_in, d_out, bias=qkv_bias)
        self.W_value = nn.Linear(d_in, d_out, bias=qkv_bias)
        self.out_proj = nn.Linear(d_out, d_out)
        self.dropout = nn.Dropout(dropout)
        self.context_length = context_length
        self._qkv_w = None      # fused [3*d_out, d_in] weight / [3*d_out] bias (inference cache)
        self._qkv_b = None
        self.small_linear = False   # set by GPTModel.prepare_for_inference on the bf16 GPU path
        # The reference registers the causal mask as a persistent buffer (model_inference.py:55),
        # so its state_dicts carry a `mask` entry per attention module.  Nothing here reads a mask
        # (the kernel masks by index), so none is stored -- context_length^2 floats per layer --
        # but state_dicts stay interchangeable in both directions: the entry is accepted and
        # dropped on load, and written (built on the fly) on export.
        self._register_load_state_dict_pre_hook(self._drop_mask_on_load)
        self._register_state_dict_hook(self._add_mask_on_export)

    @staticmethod
    def _drop_mask_on_load(state_dict, prefix, *_):
        state_dict.pop(prefix + "mask", None)

    @staticmethod
    def _add_mask_on_export(module, state_dict, prefix, _local_metadata):
        ref = module.W_query.weight
        n = module.context_length
        state_dict[prefix + "mask"] = torch.triu(torch.ones(n, n, device=ref.device), diagonal=1)

    def fuse_qkv(self):
        """Cache the concatenated projection (call again after changing the weights)."""
        with torch.no_grad():
            self._qkv_w = torch.cat([self.W_query.weight, self.W_key.weight, self.W_value.weight], 0).contiguous()
            self._qkv_b = (None if self.W_query.bias is None else
                           torch.cat([self.W_query.bias, self.W_key.bias, self.W_value.bias], 0).contiguous())

    def forward(self, x, kv_cache=None, pos=0, qkv=None):
        """x [B, n, d_in].  Without a cache: causal attention among the n tokens (prefill).  With
        kv_cache = (K, V) of shape [B, N_max, H, d]: the new keys/values are written at rows
        pos .. pos+n-1 and the queries attend rows 0 .. pos+n-1 (causally among themselves).
        `qkv` [B, n, 3*d_out]: the fused projection already computed by the caller (x is unused)."""
        h, d = self.num_heads, self.head_dim
        if qkv is not None:
            b, n = qkv.shape[:2]
            few = True
            from .block_ops import linear_small
            qkv = qkv.view(b, n, 3, h, d)
            q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        else:
            b, n, _ = x.shape
            few = _few_rows(x, self.small_linear and not self.training)
            if few:
                from .block_ops import linear_small
            if self._qkv_w is not None and not self.training:
                qkv = (linear_small(x.contiguous(), self._qkv_w, self._qkv_b) if few
                       else F.linear(x, self._qkv_w, self._qkv_b)).view(b, n, 3, h, d)
                q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
            else:
                q = self.W_query(x).view(b, n, h, d).transpose(1, 2)
                k = self.W_key(x).view(b, n, h, d).transpose(1, 2)
                v = self.W_value(x).view(b, n, h, d).transpose(1, 2)
        dev_pos = isinstance(pos, DevicePosition)   # decode step inside a CUDA graph
        if dev_pos and not (self.impl_type == "cuda" and n == 1 and kv_cache is not None):
            raise NotImplementedError("a device-side position is for single-token steps of the cuda path")
        # a single new token on the cuda path: the decode kernel appends k, v to the caches itself
        append_in_kernel = (self.impl_type == "cuda" and kv_cache is not None and n == 1
                            and k.dtype == torch.bfloat16 and kv_cache[0].dtype == torch.bfloat16)
        if kv_cache is not None:
            ck, cv = kv_cache
            if append_in_kernel:
                pass
            elif dev_pos:
                ck.index_copy_(1, pos.index, k.transpose(1, 2).to(ck.dtype))
                cv.index_copy_(1, pos.index, v.transpose(1, 2).to(cv.dtype))
            else:
                ck[:, pos:pos + n] = k.transpose(1, 2).to(ck.dtype)
                cv[:, pos:pos + n] = v.transpose(1, 2).to(cv.dtype)
        if self.impl_type == "cuda":
            from . import custom_flash_attn
            if q.dtype != torch.bfloat16:      # outside autocast: the kernel is bf16-only
                q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
            if kv_cache is not None and n == 1:
                ctx = custom_flash_attn.decode(q, ck.transpose(1, 2), cv.transpose(1, 2),
                                               pos.length if dev_pos else pos + 1,
                                               k_new=k if append_in_kernel else None,
                                               v_new=v if append_in_kernel else None)
                ctx = ctx.transpose(1, 2)                                    # [B, 1, H, d]
            elif pos == 0:
                ctx = custom_flash_attn.forward(q, k, v).transpose(1, 2)     # [B,N,H,d], dense
            else:
                raise NotImplementedError("prefill in several chunks is not supported")
        elif self.impl_type in ("manual", "functional"):
            if kv_cache is not None:
                k = ck[:, :pos + n].transpose(1, 2).to(q.dtype)
                v = cv[:, :pos + n].transpose(1, 2).to(q.dtype)
            total = pos + n if kv_cache is not None else n
            attn = q @ k.transpose(-2, -1)
            # query i (absolute position pos + i) sees keys 0 .. pos + i
            mask = torch.triu(torch.ones(n, total, device=q.device), diagonal=1 + total - n).bool()
            attn.masked_fill_(mask, -torch.inf)
            w = self.dropout(torch.softmax(attn / k.shape[-1] ** 0.5, dim=-1))
            ctx = (w @ v).transpose(1, 2)
        else:
            raise ValueError(f"unknown impl_type {self.impl_type!r}")
        ctx = ctx.reshape(b, n, self.d_out)
        if not torch.is_autocast_enabled():
            ctx = ctx.to(self.out_proj.weight.dtype)
        if few and ctx.dtype == torch.bfloat16:
            return linear_small(ctx.contiguous(), self.out_proj.weight, self.out_proj.bias)
        return self.out_proj(ctx)


class LayerNorm(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.eps = 1e-5
        self.scale = nn.Parameter(torch.ones(config["emb_dim"]))
        self.shift = nn.Parameter(torch.zeros(config["emb_dim"]))

    def forward(self, x):
        return F.layer_norm(x, x.shape[-1:], self.scale, self.shift, self.eps)


class GELU(nn.Module):
    def forward(self, x):
        return F.gelu(x, approximate="tanh")


class FeedForward(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.layers = nn.Sequential(nn.Linear(config["emb_dim"], 4 * config["emb_dim"]), GELU(),
                                    nn.Linear(4 * config["emb_dim"], config["emb_dim"]))

    small_linear = False   # set by GPTModel.prepare_for_inference on the bf16 GPU path

    def forward(self, x):
        fc, proj = self.layers[0], self.layers[2]
        if _few_rows(x, self.small_linear and not self.training) and fc.weight.dtype == x.dtype:
            from .block_ops import linear_small
            h = linear_small(x.contiguous(), fc.weight, fc.bias, gelu=True)
            return linear_small(h, proj.weight, proj.bias)
        if x.is_cuda and x.dtype == torch.bfloat16 and not self.training and fc.weight.dtype == x.dtype:
            # the tanh GELU runs in the epilogue of the first GEMM (cuBLASLt) instead of as a
            # separate pass over the [tokens, 4*d_model] activation
            h = torch._addmm_activation(fc.bias, x.reshape(-1, x.shape[-1]), fc.weight.t(), use_gelu=True)
            return proj(h).view(*x.shape[:-1], proj.out_features)
        return self.layers(x)


class TransformerBlock(nn.Module):
    def __init__(self, cfg, autocast_attention=True):
        super().__init__()
        self.att = MultiHeadAttention(cfg["emb_dim"], cfg["emb_dim"], cfg["context_length"],
                                      cfg["drop_rate"], cfg["n_heads"], cfg["impl_type"], cfg["qkv_bias"])
        self.ff = FeedForward(cfg)
        self.norm1 = LayerNorm(cfg)
        self.norm2 = LayerNorm(cfg)
        self.drop_shortcut = nn.Dropout(cfg["drop_rate"])
        self.autocast_attention = autocast_attention

    def forward(self, x, kv_cache=None, pos=0):
        shortcut = x
        h = self.norm1(x)
        if self.autocast_attention and x.is_cuda and x.dtype == torch.float32:
            with torch.autocast(device_type="cuda", dtype=torch.bfloat16):   # as the reference, :153
                h = self.att(h, kv_cache, pos)
            h = h.to(x.dtype)
        else:
            h = self.att(h, kv_cache, pos)
        x = self.drop_shortcut(h) + shortcut
        shortcut = x
        x = self.drop_shortcut(self.ff(self.norm2(x))) + shortcut
        return x


class GPTModel(nn.Module):
    def __init__(self, cfg, dtype=None):
        super().__init__()
        self.cfg = dict(cfg)
        self.tok_emb = nn.Embedding(cfg["vocab_size"], cfg["emb_dim"])
        self.pos_emb = nn.Embedding(cfg["context_length"], cfg["emb_dim"])
        self.drop_emb = nn.Dropout(cfg["drop_rate"])
        self.trf_blocks = nn.Sequential(*[TransformerBlock(cfg) for _ in range(cfg["n_layers"])])
        self.final_norm = LayerNorm(cfg)
        self.out_head = nn.Linear(cfg["emb_dim"], cfg["vocab_size"], bias=False)
        self._head_w = None     # out_head weight padded to a multiple of 64 rows (inference cache)
        self._fused_blocks = False   # residual add + LayerNorm through block_ops.add_layernorm
        if dtype is not None:
            self.to(dtype)

    def prepare_for_inference(self):
        """Build the fused QKV weights and the padded output head (derived caches; parameters and
        state_dict are untouched).  Call after loading or moving the weights."""
        for blk in self.trf_blocks:
            blk.att.fuse_qkv()
        w = self.out_head.weight
        pad = (-w.shape[0]) % 64
        with torch.no_grad():
            self._head_w = F.pad(w, (0, 0, 0, pad)).contiguous() if pad else None
        # bf16 model on a GPU with the attention kernel: every "x + branch; LayerNorm" pair of the
        # blocks becomes one kernel of the library as well
        d = self.cfg["emb_dim"]
        self._fused_blocks = (w.is_cuda and w.dtype == torch.bfloat16 and self.cfg["impl_type"] == "cuda"
                              and d % 8 == 0 and d <= 2048 and self.cfg["drop_rate"] == 0.0)
        for blk in self.trf_blocks:      # single-token steps: Linear layers as one pass over the weights
            blk.att.small_linear = blk.ff.small_linear = self._fused_blocks
        return self

    def invalidate_inference_cache(self):
        """Drop the derived tensors of `prepare_for_inference` (after the parameters changed)."""
        for blk in self.trf_blocks:
            blk.att._qkv_w = blk.att._qkv_b = None
            blk.att.small_linear = blk.ff.small_linear = False
        self._head_w = None
        self._fused_blocks = False
        return self

    def allocate_kv_cache(self, batch, max_len=None, dtype=None):
        """One (K, V) pair of [B, N_max, H, d] tensors per layer, in the model's device; bf16 when
        the attention kernel is used (it reads the cache in place)."""
        dev = self.tok_emb.weight.device
        h = self.cfg["n_heads"]
        d = self.cfg["emb_dim"] // h
        n_max = self.cfg["context_length"] if max_len is None else max_len
        if dtype is None:
            dtype = torch.bfloat16 if self.cfg["impl_type"] == "cuda" else self.tok_emb.weight.dtype
        return [(torch.zeros(batch, n_max, h, d, dtype=dtype, device=dev),
                 torch.zeros(batch, n_max, h, d, dtype=dtype, device=dev))
                for _ in range(self.cfg["n_layers"])]

    def _blocks_fused(self, x, kv_caches, pos, last_token_only):
        """The block stack and the final norm with every shortcut addition folded into the
        LayerNorm that follows it (TransformerBlock.forward computes the same values: x + att(
        norm1(x)), then x + ff(norm2(x))).  `x` is the residual stream, updated in place; `branch`
        is the output of the previous sub-layer that has not been added to it yet."""
        from .block_ops import add_layernorm
        branch = None
        for i, blk in enumerate(self.trf_blocks):
            cache = None if kv_caches is None else kv_caches[i]
            if branch is None:
                h = add_layernorm(x, None, blk.norm1.scale, blk.norm1.shift, blk.norm1.eps)
            else:
                x, h = add_layernorm(branch, x, blk.norm1.scale, blk.norm1.shift, blk.norm1.eps, sum_out=x)
            branch = blk.att(h, cache, pos)
            x, h = add_layernorm(branch, x, blk.norm2.scale, blk.norm2.shift, blk.norm2.eps, sum_out=x)
            branch = blk.ff(h)
        if last_token_only:               # what generate() consumes (model_inference.py:206)
            x, branch = x[:, -1:, :].contiguous(), (None if branch is None else branch[:, -1:, :].contiguous())
        fn = self.final_norm
        return add_layernorm(x if branch is None else branch, None if branch is None else x,
                             fn.scale, fn.shift, fn.eps, return_sum=False)

    def _blocks_one_row(self, x, kv_caches, pos):
        """The same stack for a single token row (a generation step at batch 1), returning the
        LOGITS: every Linear layer is one pass over its weights (block_ops.linear_small) and the
        "x + branch; LayerNorm" in front of the QKV projection, the first MLP layer and the head
        runs inside that layer's kernel, so a block is five launches besides the cache append."""
        from .block_ops import linear_small
        branch = None
        for i, blk in enumerate(self.trf_blocks):
            cache = None if kv_caches is None else kv_caches[i]
            att, fc, proj = blk.att, blk.ff.layers[0], blk.ff.layers[2]
            if branch is None:
                qkv = linear_small(x, att._qkv_w, att._qkv_b, ln_scale=blk.norm1.scale,
                                   ln_shift=blk.norm1.shift, eps=blk.norm1.eps)
            else:
                x, qkv = linear_small(branch, att._qkv_w, att._qkv_b, resid=x, ln_scale=blk.norm1.scale,
                                      ln_shift=blk.norm1.shift, eps=blk.norm1.eps, keep_sum=True)
            branch = att(None, cache, pos, qkv=qkv)
            x, h = linear_small(branch, fc.weight, fc.bias, gelu=True, resid=x, ln_scale=blk.norm2.scale,
                                ln_shift=blk.norm2.shift, eps=blk.norm2.eps, keep_sum=True)
            branch = linear_small(h, proj.weight, proj.bias)
        fn = self.final_norm
        if branch is None:
            return linear_small(x, self.out_head.weight, ln_scale=fn.scale, ln_shift=fn.shift, eps=fn.eps)
        return linear_small(branch, self.out_head.weight, resid=x, ln_scale=fn.scale, ln_shift=fn.shift, eps=fn.eps)

    @torch.no_grad()
    def capture_prefill(self, batch, n, last_token_only=False, warmup=3):
        """Record one prefill forward for a fixed [batch, n] shape as a CUDA graph and return
        `run(ids) -> logits`: the ~300 launches of a forward (GEMMs, attention, add+LayerNorm) are
        replayed as one graph launch, which removes the host gaps between them.  The returned
        logits live in the graph's own memory and are overwritten by the next call."""
        dev = self.tok_emb.weight.device
        static_ids = torch.zeros(batch, n, dtype=torch.long, device=dev)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):          # first calls set up library state: keep them out of the capture
            for _ in range(warmup):
                self(static_ids, last_token_only=last_token_only)
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_out = self(static_ids, last_token_only=last_token_only)

        def run(ids):
            static_ids.copy_(ids)
            graph.replay()
            return static_out
        run.graph = graph
        return run

    @torch.no_grad()
    def capture_decode_step(self, kv_caches, warmup=2):
        """Record one generation step (one new token per sequence against `kv_caches`) as a CUDA
        graph.  Returns `step(ids [B,1]) -> logits [B,1,vocab]` and the DevicePosition it advances:
        call `position.set(prompt_len)` after the prefill has filled the caches, then `step` once
        per token.  A step is then one graph launch instead of ~15 kernel launches per layer, which
        is what bounds small-batch generation.  The warm-up steps write cache row 0 and are
        overwritten by the prefill, so capture BEFORE running the prompt."""
        dev = self.tok_emb.weight.device
        batch = kv_caches[0][0].shape[0]
        position = DevicePosition(dev)
        static_ids = torch.zeros(batch, 1, dtype=torch.long, device=dev)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self(static_ids, kv_caches=kv_caches, pos=position)
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_logits = self(static_ids, kv_caches=kv_caches, pos=position)
            position.advance()

        def step(ids):
            static_ids.copy_(ids)
            graph.replay()
            return static_logits
        step.graph = graph
        return step, position

    def forward(self, in_idx, last_token_only=False, kv_caches=None, pos=0):
        _, n = in_idx.shape
        if isinstance(pos, DevicePosition):
            x = self.tok_emb(in_idx) + self.pos_emb(pos.index)
        else:
            x = self.tok_emb(in_idx) + self.pos_emb(torch.arange(pos, pos + n, device=in_idx.device))
        x = self.drop_emb(x)
        if self._fused_blocks and not self.training and x.dtype == torch.bfloat16:
            x = x.contiguous()
            if _few_rows(x, True):
                return self._blocks_one_row(x, kv_caches, pos)      # logits
            x = self._blocks_fused(x, kv_caches, pos, last_token_only)
        else:
            if kv_caches is None:
                x = self.trf_blocks(x)
            else:
                for blk, cache in zip(self.trf_blocks, kv_caches):
                    x = blk(x, cache, pos)
            x = self.final_norm(x)
            if last_token_only:           # what generate() consumes (model_inference.py:206)
                x = x[:, -1:, :]
        if _few_rows(x, self._fused_blocks and not self.training, limit=8):
            from .block_ops import linear_small
            return linear_small(x.contiguous(), self.out_head.weight)
        if self._head_w is not None and not self.training:
            return F.linear(x, self._head_w)[..., :self.out_head.weight.shape[0]]
        return self.out_head(x)


class GenerationSession:
    """K/V caches for `batch` sequences of up to `context_size` tokens plus (cuda_graph=True) the
    recorded single-token step; pass it to generate() to reuse both across prompts."""

    @torch.no_grad()
    def __init__(self, model, batch, context_size, cuda_graph=True):
        self.batch, self.context_size = batch, context_size
        self.caches = model.allocate_kv_cache(batch, context_size)
        self.step_fn = self.position = None
        if cuda_graph:
            self.step_fn, self.position = model.capture_decode_step(self.caches)


@torch.no_grad()
def generate(model, idx, max_new_tokens, context_size, temperature=1.0, top_k=None, eos_id=None,
             use_cache=True, generator=None, cuda_graph=False, session=None):
    """The reference's generate() (model_inference.py:199-228): same arguments, same top-k /
    temperature / multinomial-or-argmax rules, same stop at eos_id.  With use_cache=True the
    prompt is run once and each new token costs one single-token forward against the K/V cache;
    with use_cache=False every token re-runs `idx[:, -context_size:]` as the reference does.
    cuda_graph=True (with the cache, "cuda" attention) records the single-token forward once and
    replays it per token: one graph launch instead of ~15 kernel launches per layer.  Recording
    costs a few steps' time; `session=GenerationSession(model, batch, context_size)` keeps the
    caches and the recorded step across calls.
    The cache holds context_size rows and does not slide: once the sequence outgrows it (or if the
    prompt alone is longer), the remaining tokens are produced the reference's way, by re-running
    the last context_size tokens (:202), so a call that generates past the context length
    continues exactly as it does in the reference instead of failing."""
    caches = None
    pos = 0
    step_fn = position = None
    if use_cache and idx.shape[1] > context_size:
        use_cache = False                  # nothing of this prompt's cache would stay valid
    if use_cache:
        if session is not None:            # caches and the recorded step are reused across calls
            if session.batch != idx.shape[0] or session.context_size < min(context_size, idx.shape[1] + max_new_tokens):
                raise ValueError("the generation session was made for another batch or context size")
            context_size = min(context_size, session.context_size)
            caches, step_fn, position = session.caches, session.step_fn, session.position
        else:
            caches = model.allocate_kv_cache(idx.shape[0], context_size)
            if cuda_graph:
                step_fn, position = model.capture_decode_step(caches)
    for step in range(max_new_tokens):
        if use_cache and step > 0 and pos + 1 > context_size:
            use_cache = False              # the cache is full: recompute over the sliding window from here on
        if use_cache and step > 0 and step_fn is not None:
            logits = step_fn(idx[:, -1:])
            pos += 1
        elif use_cache:
            inp = idx if step == 0 else idx[:, -1:]
            logits = model(inp, last_token_only=True, kv_caches=caches, pos=pos)
            pos += inp.shape[1]
            if position is not None:
                position.set(pos)
        else:
            logits = model(idx[:, -context_size:], last_token_only=True)
        logits = logits[:, -1, :].float()
        if top_k is not None:
            top_logits, _ = torch.topk(logits, top_k)
            logits = torch.where(logits < top_logits[:, -1:], torch.full_like(logits, -torch.inf), logits)
        if temperature > 0.0:
            probs = torch.softmax(logits / temperature, dim=-1)
            idx_next = torch.multinomial(probs, num_samples=1, generator=generator)
        else:
            idx_next = torch.argmax(logits, dim=-1, keepdim=True)
        if eos_id is not None and idx.shape[0] == 1 and int(idx_next) == eos_id:   # as the reference, :224
            break
        idx = torch.cat((idx, idx_next), dim=1)
    return idx


def init_random(model: GPTModel, seed: int, std: float = 0.02) -> GPTModel:
    """Random-init weights N(0, std) from `seed` (LayerNorm scale 1 / shift 0, as the reference
    initialises them, :100-101); stands in for the OpenAI checkpoints, which need the network."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, prm in model.named_parameters():
            if name.endswith(".scale"):
                prm.fill_(1.0)
            elif name.endswith(".shift"):
                prm.zero_()
            else:
                prm.copy_((torch.randn(prm.shape, generator=g) * std).to(prm.dtype))
    return model


def prefill_flops_per_token(cfg: dict, n: int) -> float:
    """2*(12*L*d_model^2 + d_model*vocab) for the GEMMs + causal-adjusted attention 2*N*d_model*L."""
    L, dm, vocab = cfg["n_layers"], cfg["emb_dim"], cfg["vocab_size"]
    return 2.0 * (12.0 * L * dm * dm + dm * vocab) + 2.0 * n * dm * L
