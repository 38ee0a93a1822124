"""Compressed-prefix attention inside a Hugging Face model's forward pass.

The reference serves a stored document by dequantising every layer back into an fp16
``DynamicCache`` before the question is run (cag_store.py:325-352 ``build_dynamic_cache``), so
the model's attention reads 16 bits per element again.  This module keeps the document's
turbo_mse pages as the KV cache of the prefix and registers an attention function with
``transformers.AttentionInterface`` that reads those pages directly:

* the question chunk (``Sq`` new tokens, causal inside the chunk) goes through
  ``tq_mse_prefill_paged`` -- prefix pages decoded on the fly, chunk K/V in fp16;
* every generated token goes through ``tq_decode_paged`` over the prefix (a split-KV record)
  and an fp16 pass over the short tail of new tokens, merged by their log-sum-exp weights.

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
    """One layer's stored document: turbo_mse pages with identity slots (page p holds tokens
    16 p .. 16 p + 15, the order ``CAGStore.pack_document`` writes)."""
    pool: torch.Tensor          # uint8 [pages * page_size_bytes]
    num_tokens: int
    block_table: torch.Tensor   # int32 [1, pages]
    seq_lens: torch.Tensor      # int32 [1]


class _Runtime:
    """What the attention function needs besides its arguments (one per installed model)."""

    def __init__(self, tq: TurboQuantWrapper, cfg: TQConfig, layout) -> None:
        self.tq, self.cfg, self.layout = tq, cfg, layout


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


def install(model, pools: list[torch.Tensor], num_tokens: int, tq: TurboQuantWrapper | None = None):
    """Attach a stored document (``pools[l]`` = layer l's turbo_mse pool as loaded by
    ``CAGStore.load_document``) to ``model`` and route its attention through this module.
    Returns the cache to pass as ``past_key_values``."""
    register()
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
    layout = tq.make_mse_layout_for(cfg)
    rt = _Runtime(tq, cfg, layout)
    pages = (num_tokens + cfg.block_size - 1) // cfg.block_size
    for m, pool in zip(mods, pools):
        if not pool.is_cuda or pool.dtype != torch.uint8 or pool.numel() != pages * layout.page_size_bytes:
            raise ValueError("pool is not a device-resident turbo_mse pool of this document")
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
    """fp32 attention of one query token over the fp16 tail; returns (out [Hq, D], lse [Hq])."""
    hq, hkv = query.shape[0], key.shape[0]
    g = hq // hkv
    q = query.float().view(hkv, g, -1)
    s = torch.matmul(q, key.float().transpose(1, 2)) * scaling        # [Hkv, G, T]
    lse = torch.logsumexp(s, dim=-1)
    o = torch.matmul(torch.exp(s - lse.unsqueeze(-1)), value.float())  # [Hkv, G, D]
    return o.view(hq, -1), lse.view(hq)


def turborag_mse_attention(module, query, key, value, attention_mask=None, dropout: float = 0.0,
                           scaling: float | None = None, sliding_window=None, **kwargs):
    """``AttentionInterface`` function: ``query`` [1, Hq, Sq, 128], ``key`` / ``value`` the fp16
    tail the cache layer returned [1, Hkv, T, 128].  Returns ([1, Sq, Hq, 128], None)."""
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
    tq, cfg, layout = rt.tq, rt.cfg, rt.layout
    stream = torch.cuda.current_stream(query.device).cuda_stream
    if sq == tail:
        # the question chunk: causal inside the chunk, every chunk token sees the whole prefix
        q = query.transpose(1, 2).contiguous()                     # [1, Sq, Hq, D]
        ck = key.transpose(1, 2).contiguous()                      # [1, Sq, Hkv, D]
        cv = value.transpose(1, 2).contiguous()
        out = torch.empty_like(q)
        tq.mse_prefill_paged(q, prefix.pool, prefix.block_table, prefix.seq_lens, ck, cv, out,
                             layout, cfg, stream=stream)
        return out, None
    if sq == 1:
        # one generated token: split-KV record over the pages, fp16 pass over the tail
        q = query[:, :, 0, :].contiguous()                         # [1, Hq, D]
        rec = torch.empty(1, hq, PARTIAL_STRIDE, dtype=torch.float32, device=query.device)
        tq.decode_paged("turbo_mse", q, prefix.pool, prefix.block_table, prefix.seq_lens, layout, cfg,
                        partials_out=rec, stream=stream)
        o_p = torch.empty(hq, d, dtype=torch.float16, device=query.device)
        tq.merge_partials(rec.view(1, hq, PARTIAL_STRIDE), o_p, hq, cfg.num_kv_heads, stream=stream)
        lse_p = rec[0, :, 128] + torch.log(rec[0, :, 129])
        o_t, lse_t = _tail_attention(q[0], key[0], value[0], 1.0 / math.sqrt(d))
        w_p = torch.sigmoid(lse_p - lse_t).unsqueeze(-1)
        out = (w_p * o_p.float() + (1.0 - w_p) * o_t).to(torch.float16)
        return out.view(1, 1, hq, d), None
    raise NotImplementedError("a chunk after the first one (Sq > 1 with an older tail) is not supported: "
                              "run the question as one chunk, then decode token by token")


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
