"""Host-side sharding for one 8-GPU box (one process per GPU, torch.distributed).

* quantize+pack / dequant: independent (layer, document) units are dealt out in
  contiguous shards, no communication;
* decode over many sequences: sequences are dealt out the same way;
* long-context decode: the KV tokens of every sequence are cut into page-aligned
  contiguous ranges, one per rank; every rank produces (acc, m, l) partials for
  its range and the ranks exchange them, either
  - by plain peer stores over NVLink into buffers every rank has mapped (``PeerExchange`` +
    ``decode_kv_split_peer``: one publish launch, one merge launch that waits for the peers'
    flags with a 2-second bound; no collective library call on the data path), or
  - by ONE NCCL all-gather followed by the local merge kernel (``decode_kv_split``; also the
    gloo path of the CPU tests).
  No kernel ever *reads* a peer's memory, and nothing uses multicast or TMA on peer memory.
"""
from __future__ import annotations

import ctypes as C

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


class PeerExchange:
    """One zero-initialised exchange buffer per rank, mapped into every peer of ``group``.

    Mapping: torch symmetric memory where it works, else CUDA IPC handles of an ordinary
    allocation (``how`` says which).  ``rows_cap`` = the largest sequences * num_q_heads of any
    call.  Every rank must make the same sequence of calls (the exchange number is implicit)."""

    def __init__(self, tq, rows_cap: int, device: torch.device, group=None) -> None:
        self.tq, self.group, self.rows_cap = tq, group, rows_cap
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        nbytes = tq.peer_buffer_bytes(self.world, rows_cap)
        self._keep = []
        try:
            import torch.distributed._symmetric_memory as symm
            self.buf = symm.empty(nbytes, dtype=torch.uint8, device=device)
            self.buf.zero_()
            hdl = symm.rendezvous(self.buf, group if group is not None else dist.group.WORLD)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            self._keep.append(hdl)
            self.how = "symmetric memory"
        except Exception:  # noqa: BLE001 - any failure of the optional path selects the IPC path
            self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
            mine = self.buf.untyped_storage()._share_cuda_()
            handles = [None] * self.world
            dist.all_gather_object(handles, mine, group=group)
            ptrs = []
            for q, hnd in enumerate(handles):
                if q == self.rank:
                    ptrs.append(self.buf.data_ptr())
                    continue
                st = torch.UntypedStorage._new_shared_cuda(*hnd)
                view = torch.empty(0, dtype=torch.uint8, device=device).set_(st)
                self._keep.append(view)
                ptrs.append(view.data_ptr())
            self.how = "CUDA IPC"
        self.ptr_array = (C.c_void_p * self.world)(*ptrs)
        self.local = torch.empty(rows_cap, PARTIAL_STRIDE, dtype=torch.float32, device=device)
        self.exchange = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)  # every buffer is zeroed and mapped before anyone publishes

    def publish_and_merge(self, rows: int, output: torch.Tensor, num_q_heads: int, num_kv_heads: int,
                          stream: int = 0) -> None:
        """``self.local[:rows]`` holds this rank's records; ``output`` gets fp16 [rows, 128]."""
        self.exchange += 1
        self.tq.peer_publish(self.local, self.ptr_array, self.rank, self.world, rows, self.rows_cap,
                             self.exchange, stream)
        self.tq.peer_merge(self.buf, self.world, rows, self.rows_cap, self.exchange, output,
                           num_q_heads, num_kv_heads, stream)


def decode_kv_split_peer(xchg: PeerExchange, scheme, query, page_pool, block_tables, seq_lens, layout,
                         cfg, max_kv_tokens: int, output: torch.Tensor, workspace=None,
                         stream: int = 0) -> torch.Tensor:
    """``decode_kv_split`` with the partials exchanged by peer stores instead of an all-gather:
    decode kernel, then a split merge that stores the records into every peer's buffer, waits for
    the peers' flags and merges the records that arrived here -- two launches, no collective (three
    for batches too large for that kernel's grid to be resident at once)."""
    tq = xchg.tq
    b, hq, _ = query.shape
    rows = b * hq
    begin, end = kv_token_range(max_kv_tokens, xchg.rank, xchg.world, cfg.block_size)
    xchg.exchange += 1
    tq.decode_paged_exchange(scheme, query, page_pool, block_tables, seq_lens, layout, cfg, xchg.ptr_array,
                             xchg.rank, xchg.world, xchg.rows_cap, xchg.exchange, max_kv_tokens, begin, end,
                             output, workspace=workspace, stream=stream)
    return output
