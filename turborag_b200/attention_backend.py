"""Compressed-prefix attention inside a Hugging Face model's forward pass.

The reference serves a stored document by dequantising every layer back into an fp16
``DynamicCache`` before the question is run (cag_store.py:325-352 ``build_dynamic_cache``), so
the model's attention reads 16 bits per element again.  This module keeps the document's
turbo_mse pages as the KV cache of the prefix and registers an attention function with
``transformers.AttentionInterface`` that reads those pages directly:

* a turbo_mse document's question chunk (``Sq`` new tokens, causal inside the chunk) goes
  through ``tq_mse_prefill_paged`` -- prefix pages decoded on the fly, chunk K/V in fp16;
* everything else -- a turbo_prod document's question chunk, every generated token, a later
  chunk -- goes through ``tq_decode_paged`` over the prefix (split-KV records, the new tokens x
  query heads laid out as the GQA group of their kv head) and a causal fp32 pass over the short
  fp16 tail of new tokens, merged by their log-sum-exp weights.

Pieces:
  ``CompressedPrefixLayer``  cache layer: reports prefix + tail as its length (positions, masks),
                             stores only the fp16 tail;
  ``compressed_prefix_cache`` a ``DynamicCache`` made of such layers;
  ``install``                hangs the stored pages on the model's attention modules and selects
                             the registered attention function;
  ``turborag_mse_attention`` the attention function itself.

Requirements checked at run time: head_dim 128, batch 1, fp16, the model's softmax scale equal
to 1 / sqrt(head_dim), no sliding window.  Anything else raises; there is no fallback path.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .wrapper import TurboQuantWrapper, TQConfig

ATTENTION_NAME = "turborag_mse"
PARTIAL_STRIDE = 130


@dataclass
class LayerPrefix:
    """One layer's stored document: turbo_prod or turbo_mse pages with identity slots (page p
    holds tokens 16 p .. 16 p + 15, the order ``CAGStore.pack_document`` writes)."""
    pool: torch.Tensor          # uint8 [pages * page_size_bytes]
    num_tokens: int
    block_table: torch.Tensor   # int32 [1, pages]
    seq_lens: torch.Tensor      # int32 [1]


class _Runtime:
    """What the attention function needs besides its arguments (one per installed model)."""

    def __init__(self, tq: TurboQuantWrapper, cfg: TQConfig, layout, scheme: str = "turbo_mse") -> None:
        self.tq, self.cfg, self.layout, self.scheme = tq, cfg, layout, scheme


def _layer_base():
    from transformers.cache_utils import DynamicLayer
    return DynamicLayer


def make_layer_class():
    base = _layer_base()

    class CompressedPrefixLayer(base):
        """``DynamicLayer`` whose first ``prefix_len`` positions live in compressed pages held
        by the attention module; ``keys`` / ``values`` are the fp16 tail only."""

        def __init__(self, prefix_len: int) -> None:
            super().__init__()
            self.prefix_len = int(prefix_len)

        def get_seq_length(self) -> int:
            return self.prefix_len + super().get_seq_length()

    return CompressedPrefixLayer


def compressed_prefix_cache(prefix_len: int, num_layers: int):
    """``DynamicCache`` whose layers start at position ``prefix_len`` with an empty tail."""
    from transformers import DynamicCache
    cache = DynamicCache()
    cls = make_layer_class()
    cache.layers = [cls(prefix_len) for _ in range(num_layers)]
    return cache


def _attention_modules(model):
    mods = [m for m in model.modules() if hasattr(m, "layer_idx") and hasattr(m, "q_proj")]
    mods.sort(key=lambda m: m.layer_idx)
    return mods


def install(model, pools: list[torch.Tensor], num_tokens: int, tq: TurboQuantWrapper | None = None,
            scheme: str = "turbo_mse"):
    """Attach a stored document (``pools[l]`` = layer l's turbo_mse or turbo_prod pool as loaded
    by ``CAGStore.load_document``) to ``model`` and route its attention through this module.
    Returns the cache to pass as ``past_key_values``."""
    register()
    if scheme not in ("turbo_mse", "turbo_prod"):
        raise ValueError("compressed-prefix attention serves turbo_mse and turbo_prod documents")
    tq = tq or TurboQuantWrapper()
    mods = _attention_modules(model)
    if len(mods) != len(pools):
        raise ValueError(f"{len(pools)} stored layers for a model with {len(mods)} attention layers")
    head_dim = mods[0].head_dim
    num_kv = model.config.num_key_value_heads
    if head_dim != 128:
        raise ValueError("the compressed attention path needs head_dim 128")
    cfg = tq.default_config()
    cfg.num_kv_heads, cfg.head_dim = num_kv, head_dim
    layout = tq.layout_for_scheme(scheme, cfg)
    rt = _Runtime(tq, cfg, layout, scheme)
    pages = (num_tokens + cfg.block_size - 1) // cfg.block_size
    for m, pool in zip(mods, pools):
        if not pool.is_cuda or pool.dtype != torch.uint8 or pool.numel() != pages * layout.page_size_bytes:
            raise ValueError(f"pool is not a device-resident {scheme} pool of this document")
        if abs(m.scaling - 1.0 / math.sqrt(head_dim)) > 1e-9:
            raise ValueError("softmax scale differs from 1 / sqrt(head_dim)")
        dev = pool.device
        m._tq_prefix = LayerPrefix(pool, num_tokens,
                                   torch.arange(pages, dtype=torch.int32, device=dev).view(1, -1),
                                   torch.tensor([num_tokens], dtype=torch.int32, device=dev))
        m._tq_runtime = rt
    model.config._attn_implementation = ATTENTION_NAME
    return compressed_prefix_cache(num_tokens, len(mods))


def uninstall(model, attn_implementation: str = "eager") -> None:
    for m in _attention_modules(model):
        for name in ("_tq_prefix", "_tq_runtime"):
            if hasattr(m, name):
                delattr(m, name)
    model.config._attn_implementation = attn_implementation


def _tail_attention(query, key, value, scaling: float):
    """Causal fp32 attention of the last ``Sq`` positions over the fp16 tail: ``query``
    [Hq, Sq, D], ``key`` / ``value`` [Hkv, T, D] with the queries at tail positions T - Sq .. T - 1.
    Returns (out [Hq, Sq, D], lse [Hq, Sq])."""
    hq, sq, _ = query.shape
    hkv, t, _ = key.shape
    g = hq // hkv
    q = query.float().reshape(hkv, g * sq, -1)
    s = torch.matmul(q, key.float().transpose(1, 2)).view(hkv, g, sq, t) * scaling
    if sq > 1:
        pos = torch.arange(t - sq, t, device=query.device).view(sq, 1)
        s = s.masked_fill(torch.arange(t, device=query.device).view(1, t) > pos, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.matmul(torch.exp(s - lse.unsqueeze(-1)).view(hkv, g * sq, t), value.float())
    return o.reshape(hq, sq, -1), lse.reshape(hq, sq)


def _prefix_attention(rt: _Runtime, prefix: LayerPrefix, query, stream: int):
    """Attention of every (new token, query head) over the compressed pages alone: the Sq x G rows
    of a kv head form its GQA group in one paged decode.  ``query`` [Hq, Sq, D] fp16.  Returns
    (out [Hq, Sq, D] fp32, lse [Hq, Sq]) from the split-KV records."""
    hq, sq, d = query.shape
    hkv = rt.cfg.num_kv_heads
    g = hq // hkv
    rows = query.reshape(hkv, g * sq, d).reshape(1, hkv * g * sq, d).contiguous()  # row h * (G Sq) + (g, s)
    rec = torch.empty(1, rows.shape[1], PARTIAL_STRIDE, dtype=torch.float32, device=query.device)
    rt.tq.decode_paged(rt.scheme, rows, prefix.pool, prefix.block_table, prefix.seq_lens, rt.layout, rt.cfg,
                       partials_out=rec, stream=stream)
    out = torch.empty(rows.shape[1], d, dtype=torch.float16, device=query.device)
    rt.tq.merge_partials(rec.view(1, rows.shape[1], PARTIAL_STRIDE), out, rows.shape[1], hkv, stream=stream)
    lse = rec[0, :, 128] + torch.log(rec[0, :, 129])
    return out.float().view(hq, sq, d), lse.view(hq, sq)


def turborag_mse_attention(module, query, key, value, attention_mask=None, dropout: float = 0.0,
                           scaling: float | None = None, sliding_window=None, **kwargs):
    """``AttentionInterface`` function: ``query`` [1, Hq, Sq, 128], ``key`` / ``value`` the fp16
    tail the cache layer returned [1, Hkv, T, 128] (it ends with the Sq new tokens).  Returns
    ([1, Sq, Hq, 128], None)."""
    prefix: LayerPrefix | None = getattr(module, "_tq_prefix", None)
    rt: _Runtime | None = getattr(module, "_tq_runtime", None)
    if prefix is None or rt is None:
        raise RuntimeError("no stored document attached to this layer (attention_backend.install)")
    if query.shape[0] != 1 or query.dtype != torch.float16 or query.shape[-1] != 128:
        raise ValueError("compressed-prefix attention: batch 1, fp16, head_dim 128")
    if dropout or sliding_window is not None:
        raise ValueError("compressed-prefix attention: no dropout, no sliding window")
    if scaling is not None and abs(scaling - 1.0 / math.sqrt(128)) > 1e-9:
        raise ValueError("softmax scale differs from 1 / sqrt(head_dim)")
    _, hq, sq, d = query.shape
    tail = key.shape[2]
    if tail < sq:
        raise ValueError("the cache layer returned fewer tail positions than new tokens")
    tq, cfg, layout = rt.tq, rt.cfg, rt.layout
    stream = torch.cuda.current_stream(query.device).cuda_stream
    if sq == tail and getattr(rt, "scheme", "turbo_mse") == "turbo_mse":
        # the question chunk: causal inside the chunk, every chunk token sees the whole prefix
        q = query.transpose(1, 2).contiguous()                     # [1, Sq, Hq, D]
        ck = key.transpose(1, 2).contiguous()                      # [1, Sq, Hkv, D]
        cv = value.transpose(1, 2).contiguous()
        out = torch.empty_like(q)
        tq.mse_prefill_paged(q, prefix.pool, prefix.block_table, prefix.seq_lens, ck, cv, out,
                             layout, cfg, stream=stream)
        return out, None
    # split-KV records over the pages, causal fp32 pass over the fp16 tail, log-sum-exp merge
    o_p, lse_p = _prefix_attention(rt, prefix, query[0].contiguous(), stream)
    o_t, lse_t = _tail_attention(query[0], key[0], value[0], 1.0 / math.sqrt(d))
    w_p = torch.sigmoid(lse_p - lse_t).unsqueeze(-1)
    out = (w_p * o_p + (1.0 - w_p) * o_t).to(torch.float16)          # [Hq, Sq, D]
    return out.transpose(0, 1).unsqueeze(0).contiguous(), None


_registered = False


def register() -> None:
    """Register ``turborag_mse_attention`` under the name ``turborag_mse`` (idempotent)."""
    global _registered
    if _registered:
        return
    from transformers import AttentionInterface
    AttentionInterface.register(ATTENTION_NAME, turborag_mse_attention)
    try:  # the causal-mask builder looks the name up too; the function ignores the mask it gets
        from transformers import AttentionMaskInterface
        from transformers.masking_utils import sdpa_mask
        AttentionMaskInterface.register(ATTENTION_NAME, sdpa_mask)
    except ImportError:
        pass
    _registered = True
