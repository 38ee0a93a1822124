"""Host-side sharding for one 8-GPU box (one process per GPU, torch.distributed).

* quantize+pack / dequant: independent (layer, document) units are dealt out in
  contiguous shards, no communication;
* decode over many sequences: sequences are dealt out the same way;
* long-context decode: the KV tokens of every sequence are cut into page-aligned
  contiguous ranges, one per rank; every rank produces (acc, m, l) partials for
  its range, ONE all-gather brings all partials into local memory, and the local
  merge kernel (log-sum-exp) finishes.  The gathered buffer is plain local device
  memory; no kernel ever reads a peer's memory.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .wrapper import PARTIAL_STRIDE


def shard_range(num_units: int, rank: int, world: int) -> range:
    """Contiguous shard of ``num_units`` for ``rank``; sizes differ by at most one."""
    base, extra = divmod(num_units, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def kv_token_range(num_tokens: int, rank: int, world: int, block_size: int = 16) -> tuple[int, int]:
    """[begin, end) of the KV tokens rank ``rank`` attends to: whole pages, contiguous."""
    pages = -(-num_tokens // block_size)
    r = shard_range(pages, rank, world)
    return min(r.start * block_size, num_tokens), min(r.stop * block_size, num_tokens)


def gather_partials(partials: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather fp32 partials [rows, 130] -> [world, rows, 130] (NCCL on GPUs, gloo on CPU)."""
    assert partials.shape[-1] == PARTIAL_STRIDE and partials.dtype == torch.float32
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(partials.shape), dtype=partials.dtype, device=partials.device)
    if partials.is_cuda:
        dist.all_gather_into_tensor(out, partials.contiguous(), group=group)
    else:
        chunks = list(out.unbind(0))
        dist.all_gather(chunks, partials.contiguous(), group=group)
    return out


def decode_kv_split(tq, scheme, query, page_pool, block_tables, seq_lens, layout, cfg,
                    max_kv_tokens: int, output: torch.Tensor, group=None, workspace=None,
                    stream: int = 0) -> torch.Tensor:
    """Long-context decode with the KV sequence split across the ranks of ``group``.

    Every rank holds the pages of its own token range (``page_pool``/``block_tables`` are
    local; table entries outside the rank's range are never read).  Returns ``output``
    (fp16 [B, Hq, 128]), identical on every rank."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    b, hq, _ = query.shape
    begin, end = kv_token_range(max_kv_tokens, rank, world, cfg.block_size)
    part = torch.empty(b, hq, PARTIAL_STRIDE, dtype=torch.float32, device=query.device)
    tq.decode_paged(scheme, query, page_pool, block_tables, seq_lens, layout, cfg,
                    partials_out=part, max_kv_tokens=max_kv_tokens, kv_begin=begin, kv_end=end,
                    workspace=workspace, stream=stream)
    allp = gather_partials(part.view(b * hq, PARTIAL_STRIDE), group)
    tq.merge_partials(allp, output.view(b * hq, -1), hq, cfg.num_kv_heads, stream=stream)
    return output
