"""Per-layer compressed-KV disk store, file-compatible with the reference's
``tq_backend/cag_store.py`` (same method names, arguments and on-disk format), with the load
path rebuilt for a B200 host.

On-disk format (``tq_backend/cag_store.py:97-157``), kept bit-for-bit so stores written by either
implementation can be read by the other:
  * ``<sha256(doc_id)[:16]>_L<layer:02d>_<scheme>.bin``  -- the raw page pool
    (``ceil(N / 16) * page_size_bytes`` bytes), or for scheme ``fp16`` a ``torch.save`` of
    ``{"num_tokens", "kv", "shape"}``;
  * ``...meta``  -- ``torch.save({"num_tokens": N, "slots": arange(N, int32)})``;
  * ``manifest.json``  -- ``{"v": 1, "entries": {doc_id: {"sha256", "layers": {"<layer>::<scheme>":
    {"key", "num_tokens", "stored_at"}}}}}``, written through a temporary file and a rename.  This
    implementation adds ``head_shape`` and ``page_size_bytes`` to a layer record (the reference
    ignores fields it does not know) and refuses a load that contradicts them: the format itself
    is unversioned and stale pages would otherwise decode to garbage silently;
  * ``<sha256(doc_id)[:16]>_<scheme>.tqdoc`` (this implementation only, ``export_container``) -- all
    layers of a document in one file behind a versioned, checksummed header that states scheme,
    head shape, page geometry and token count; read front to back by ``load_container_hnd``.

What differs from the reference on the way back to the GPU (``cag_store.py:161-255``):
  * the pool file is read straight into a reusable pinned host buffer (``readinto``: no
    ``bytes -> bytearray -> frombuffer -> clone`` copies) and copied to the device on a side
    stream, so the read of layer l+1 overlaps the dequant of layer l;
  * ``build_dynamic_cache`` dequantises directly into the ``[1, H, N, D]`` layout a Hugging Face
    cache wants (``tq_dequant_kv_hnd``), instead of ``[N, H, D]`` followed by
    ``permute().contiguous()``;
  * ``fused_attention`` accepts any number of query rows per kv head (GQA) and
    ``decode_documents`` serves a batch of stored documents with one paged call.
There is no CPU fallback: every tensor operation needs the CUDA library.
"""
from __future__ import annotations

import hashlib
import json
import os
import struct
import time
import zlib
from pathlib import Path
from typing import Literal

import torch

from .wrapper import TQConfig, TurboQuantWrapper

Scheme = Literal["fp16", "turbo_prod", "turbo_mse", "qjl"]  # "qjl": not in the reference's store
_MANIFEST = "manifest.json"

# One-file-per-document container (not in the reference, whose per-layer files carry no header):
#   fixed part  "<8sIIIIQIIIIQQ": magic, version, header_bytes, scheme (0 turbo_prod, 1 turbo_mse),
#               num_layers, num_tokens, num_kv_heads, head_dim, block_size, page_size_bytes,
#               layer_bytes, layer_stride
#   then        num_layers x "<II": layer index, CRC-32 of that layer's pool
#   then        "<I": CRC-32 of every header byte before it
#   padding to header_bytes (a multiple of 4096); layer i's pool at header_bytes + i * layer_stride
#   (layer_stride = layer_bytes rounded up to 4096, so every pool starts on a page of the file).
_DOC_MAGIC = b"TQCAGDOC"
_DOC_VERSION = 1
_DOC_FIXED = struct.Struct("<8sIIIIQIIIIQQ")
_DOC_ALIGN = 4096
_READ_RING = 8      # pinned staging buffers a container load keeps in flight
_READ_THREADS = 4   # reader threads (file reads release the interpreter lock)
_SCHEME_IDS = {"turbo_prod": 0, "turbo_mse": 1, "qjl": 2}


def _align_up(x: int, a: int) -> int:
    return -(-x // a) * a


class CAGStore:
    def __init__(self, store_dir: str | Path, lib_path: str | Path | None = None) -> None:
        self.store_dir = Path(store_dir)
        self.store_dir.mkdir(parents=True, exist_ok=True)
        self.tq = TurboQuantWrapper(lib_path)
        self._manifest_path = self.store_dir / _MANIFEST
        self._pinned: list[torch.Tensor | None] = [None, None]  # staging buffers, used in turn
        self._readers = None
        self._copy_stream: torch.cuda.Stream | None = None

    # ---- names and manifest -------------------------------------------------------------------
    @staticmethod
    def _doc_hash(doc_id: str) -> str:
        return hashlib.sha256(doc_id.encode()).hexdigest()

    def _key(self, doc_id: str, layer: int, scheme: Scheme) -> str:
        return f"{self._doc_hash(doc_id)[:16]}_L{layer:02d}_{scheme}"

    def _pool_path(self, doc_id: str, layer: int, scheme: Scheme) -> Path:
        return self.store_dir / (self._key(doc_id, layer, scheme) + ".bin")

    def _meta_path(self, doc_id: str, layer: int, scheme: Scheme) -> Path:
        return self.store_dir / (self._key(doc_id, layer, scheme) + ".meta")

    def exists(self, doc_id: str, layer: int, scheme: Scheme) -> bool:
        return self._pool_path(doc_id, layer, scheme).exists()

    def _load_manifest(self) -> dict:
        try:
            return json.loads(self._manifest_path.read_text())
        except (FileNotFoundError, json.JSONDecodeError, OSError):
            return {"v": 1, "entries": {}}

    def _save_manifest(self, manifest: dict) -> None:
        tmp = self._manifest_path.with_suffix(".tmp")
        tmp.write_text(json.dumps(manifest, indent=2))
        tmp.replace(self._manifest_path)  # a torn write never replaces a good manifest

    def _update_manifest(self, doc_id: str, layer: int, scheme: Scheme, num_tokens: int,
                         head_shape: tuple[int, int] | None = None) -> None:
        manifest = self._load_manifest()
        entry = manifest.setdefault("entries", {}).setdefault(doc_id, {"sha256": "", "layers": {}})
        entry["sha256"] = self._doc_hash(doc_id)
        rec = {"key": self._key(doc_id, layer, scheme), "num_tokens": num_tokens, "stored_at": time.time()}
        if head_shape is not None:
            # Not in the reference's manifest (it ignores unknown fields): what the bytes mean, so that
            # a load with another head shape or page geometry fails instead of decoding garbage.
            rec["head_shape"] = [int(head_shape[0]), int(head_shape[1])]
            if scheme != "fp16":
                rec["page_size_bytes"] = int(self._layout(scheme, self._make_cfg_from_shape(head_shape)).page_size_bytes)
        entry.setdefault("layers", {})[f"{layer}::{scheme}"] = rec
        self._save_manifest(manifest)

    def _verify_manifest(self, doc_id: str, layer: int, scheme: Scheme,
                         head_shape: tuple[int, int] | None = None, manifest: dict | None = None) -> None:
        """RuntimeError when the manifest contradicts the file about to be read; a store without
        a manifest entry for the document is accepted (older stores have none)."""
        entry = (manifest if manifest is not None else self._load_manifest()).get("entries", {}).get(doc_id)
        if entry is None:
            return
        stored, computed = entry.get("sha256", ""), self._doc_hash(doc_id)
        if stored and stored != computed:
            raise RuntimeError(f"Manifest integrity error for doc_id={doc_id!r}: stored SHA-256 "
                               f"{stored[:8]}... != computed {computed[:8]}...")
        layer_entry = entry.get("layers", {}).get(f"{layer}::{scheme}")
        if layer_entry and layer_entry.get("key") != self._key(doc_id, layer, scheme):
            raise RuntimeError(f"Manifest key mismatch for doc_id={doc_id!r} layer={layer} scheme={scheme}: "
                               f"stored {layer_entry.get('key')!r} != computed "
                               f"{self._key(doc_id, layer, scheme)!r}")
        if layer_entry and head_shape is not None and "head_shape" in layer_entry:
            if list(layer_entry["head_shape"]) != [int(head_shape[0]), int(head_shape[1])]:
                raise RuntimeError(f"doc_id={doc_id!r} layer={layer} scheme={scheme} was stored with head shape "
                                   f"{tuple(layer_entry['head_shape'])}, asked for {tuple(head_shape)}")
            if scheme != "fp16" and "page_size_bytes" in layer_entry:
                page = int(self._layout(scheme, self._make_cfg_from_shape(head_shape)).page_size_bytes)
                if int(layer_entry["page_size_bytes"]) != page:
                    raise RuntimeError(f"doc_id={doc_id!r} layer={layer} scheme={scheme}: stored pages are "
                                       f"{layer_entry['page_size_bytes']} bytes, this build uses {page}")

    # ---- configuration ------------------------------------------------------------------------
    def _make_cfg_from_shape(self, head_shape: tuple[int, int]) -> TQConfig:
        cfg = self.tq.default_config()
        cfg.num_kv_heads, cfg.head_dim = head_shape
        return cfg

    def _make_cfg(self, key: torch.Tensor) -> TQConfig:
        return self._make_cfg_from_shape((key.shape[1], key.shape[2]))

    def _layout(self, scheme: Scheme, cfg: TQConfig):
        if scheme == "turbo_prod":
            return self.tq.make_layout_for(cfg)
        if scheme == "turbo_mse":
            return self.tq.make_mse_layout_for(cfg)
        if scheme == "qjl":
            return self.tq.make_qjl_layout_for(cfg)
        raise ValueError(f"Unknown scheme: {scheme}")

    def _pool_bytes(self, scheme: Scheme, num_tokens: int, cfg: TQConfig) -> int:
        pages = -(-num_tokens // cfg.block_size)
        return pages * self._layout(scheme, cfg).page_size_bytes

    def vram_bytes(self, scheme: Scheme, num_tokens: int, head_shape: tuple[int, int]) -> int:
        cfg = self._make_cfg_from_shape(head_shape)
        if scheme == "fp16":
            return 2 * num_tokens * cfg.num_kv_heads * cfg.head_dim * 2
        return self._pool_bytes(scheme, num_tokens, cfg)

    # ---- offline: pack ------------------------------------------------------------------------
    def pack_document(self, doc_id: str, layer: int, key: torch.Tensor, value: torch.Tensor,
                      scheme: Scheme = "turbo_prod", overwrite: bool = False) -> int:
        """Compress and save one layer's KV ([N, H, D] fp16 CUDA tensors); returns the bytes on disk."""
        pool_p, meta_p = self._pool_path(doc_id, layer, scheme), self._meta_path(doc_id, layer, scheme)
        if pool_p.exists() and not overwrite:
            return pool_p.stat().st_size
        n = key.shape[0]
        slots = torch.arange(n, dtype=torch.int32, device=key.device)
        if scheme == "fp16":
            kv = torch.cat([key.reshape(-1), value.reshape(-1)]).cpu()
            torch.save({"num_tokens": n, "kv": kv, "shape": list(key.shape)}, pool_p)
        else:
            cfg = self._make_cfg(key)
            layout = self._layout(scheme, cfg)
            pool = torch.zeros(self._pool_bytes(scheme, n, cfg), dtype=torch.uint8, device=key.device)
            {"turbo_prod": self.tq.pack, "turbo_mse": self.tq.mse_pack, "qjl": self.tq.qjl_pack}[scheme](
                key.contiguous(), value.contiguous(), slots, pool, layout, cfg, stream=self._stream(key.device))
            host = torch.empty(pool.numel(), dtype=torch.uint8, pin_memory=True)
            host.copy_(pool, non_blocking=True)
            torch.cuda.current_stream(key.device).synchronize()
            with pool_p.open("wb") as f:
                f.write(memoryview(host.numpy()))
        torch.save({"num_tokens": n, "slots": slots.cpu()}, meta_p)
        self._update_manifest(doc_id, layer, scheme, n, (key.shape[1], key.shape[2]))
        return pool_p.stat().st_size

    # ---- online: load -------------------------------------------------------------------------
    @staticmethod
    def _stream(device) -> int:
        """Handle of torch's current stream on ``device``: every library call of the store runs on it,
        so the kernels are ordered with the caller's work inside ``with torch.cuda.stream(s)`` too."""
        return torch.cuda.current_stream(device).cuda_stream

    def _copy_to_device(self, host: torch.Tensor, nbytes: int, device: torch.device):
        """Pinned buffer -> fresh device tensor on the copy stream; returns (pool, end-of-copy event).
        The copy stream first waits for the caller's stream: the block the caching allocator hands
        out may still be in use by work queued there (a previous layer's dequant).  record_stream
        keeps the allocator from recycling the pool while the copy is in flight."""
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device)
        pool = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self._copy_stream.wait_stream(torch.cuda.current_stream(device))
        done = torch.cuda.Event()
        with torch.cuda.stream(self._copy_stream):
            pool.copy_(host[:nbytes], non_blocking=True)
            done.record()
        pool.record_stream(self._copy_stream)
        return pool, done

    def _reader_pool(self):
        if self._readers is None:
            from concurrent.futures import ThreadPoolExecutor
            self._readers = ThreadPoolExecutor(max_workers=_READ_THREADS, thread_name_prefix="cagstore-read")
        return self._readers

    def _staging(self, which: int, nbytes: int) -> torch.Tensor:
        while len(self._pinned) <= which:
            self._pinned.append(None)
        buf = self._pinned[which]
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, pin_memory=True)
            self._pinned[which] = buf
        return buf

    def _read_pool(self, doc_id: str, layer: int, scheme: Scheme, cfg: TQConfig, num_tokens: int,
                   which: int, device: torch.device) -> tuple[torch.Tensor, torch.cuda.Event]:
        """File -> pinned buffer -> device on the copy stream; returns the device pool and the
        event that marks the end of the copy."""
        nbytes = self._pool_bytes(scheme, num_tokens, cfg)
        host = self._staging(which, nbytes)
        with self._pool_path(doc_id, layer, scheme).open("rb", buffering=0) as f:
            got = f.readinto(memoryview(host.numpy())[:nbytes])
        if got != nbytes:
            raise RuntimeError(f"{self._pool_path(doc_id, layer, scheme)}: {got} bytes, expected {nbytes} "
                               f"(wrong head_shape, or a stale store)")
        return self._copy_to_device(host, nbytes, device)

    def load_document(self, doc_id: str, layer: int, scheme: Scheme = "turbo_prod",
                      head_shape: tuple[int, int] = (2, 64)) -> tuple[torch.Tensor, torch.Tensor, int]:
        """Load compressed KV to CUDA.  Returns (pool or (key, value), slots, num_tokens)."""
        pool_p = self._pool_path(doc_id, layer, scheme)
        if not pool_p.exists():
            raise FileNotFoundError(f"No pre-computed KV: doc={doc_id} layer={layer} scheme={scheme}")
        self._verify_manifest(doc_id, layer, scheme, head_shape)
        meta = torch.load(self._meta_path(doc_id, layer, scheme), weights_only=False)
        n, slots = int(meta["num_tokens"]), meta["slots"]
        dev = torch.device("cuda", torch.cuda.current_device())
        if scheme == "fp16":
            kv = torch.load(pool_p, weights_only=False)["kv"].to(dev, non_blocking=True)
            h, d = head_shape
            return (kv[:n * h * d].reshape(n, h, d).contiguous(),
                    kv[n * h * d:].reshape(n, h, d).contiguous()), slots.to(dev), n
        cfg = self._make_cfg_from_shape(head_shape)
        pool, done = self._read_pool(doc_id, layer, scheme, cfg, n, 0, dev)
        torch.cuda.current_stream(dev).wait_event(done)
        # the staging buffer is reused by the next call: the copy out of it must have finished
        done.synchronize()
        return pool, slots.to(dev), n

    def load_as_kv_fp16(self, doc_id: str, layer: int, scheme: Scheme,
                        head_shape: tuple[int, int] = (2, 64)) -> tuple[torch.Tensor, torch.Tensor]:
        """Load and dequantise one layer -> (key, value), each [N, H, D] fp16 CUDA."""
        pool, slots, n = self.load_document(doc_id, layer, scheme, head_shape)
        if scheme == "fp16":
            return pool
        cfg = self._make_cfg_from_shape(head_shape)
        h, d = head_shape
        out_k = torch.empty(n, h, d, device=slots.device, dtype=torch.float16)
        out_v = torch.empty_like(out_k)
        {"turbo_prod": self.tq.dequant, "turbo_mse": self.tq.mse_dequant, "qjl": self.tq.qjl_dequant}[scheme](
            pool, slots, out_k, out_v, self._layout(scheme, cfg), cfg, stream=self._stream(slots.device))
        return out_k, out_v

    def load_layers_hnd(self, doc_id: str, num_layers: int, scheme: Scheme,
                        head_shape: tuple[int, int] = (2, 64)) -> tuple[list, int]:
        """[(layer, key, value)] with key/value [1, H, N, D] fp16 CUDA for every stored layer, and
        the document length.  The file read and host-to-device copy of the next layer run while
        the current one is dequantised."""
        dev = torch.device("cuda", torch.cuda.current_device())
        layers = [l for l in range(num_layers) if self.exists(doc_id, l, scheme)]
        out, doc_len = [], 0
        if scheme == "fp16":
            for l in layers:
                k, v = self.load_as_kv_fp16(doc_id, l, scheme, head_shape)
                out.append((l, k.permute(1, 0, 2).unsqueeze(0).contiguous(),
                            v.permute(1, 0, 2).unsqueeze(0).contiguous()))
                doc_len = doc_len or k.shape[0]
            return out, doc_len
        cfg = self._make_cfg_from_shape(head_shape)
        layout = self._layout(scheme, cfg)
        h, d = head_shape
        # one manifest read for the whole document; the token count comes from the manifest record
        # when there is one (pack_document always writes slots = arange(N), which is rebuilt on the
        # device), else from the .meta file as in the reference
        manifest = self._load_manifest()
        records = manifest.get("entries", {}).get(doc_id, {}).get("layers", {})
        metas, identity = {}, {}
        for l in layers:
            self._verify_manifest(doc_id, l, scheme, head_shape, manifest)
            rec = records.get(f"{l}::{scheme}")
            if rec and "num_tokens" in rec:
                n = int(rec["num_tokens"])
                if n not in identity:
                    identity[n] = torch.arange(n, dtype=torch.int32, device=dev)
                metas[l] = (n, identity[n])
            else:
                meta = torch.load(self._meta_path(doc_id, l, scheme), weights_only=False)
                metas[l] = (int(meta["num_tokens"]), meta["slots"].to(dev))
        pending = None
        copies_in_flight: list[torch.cuda.Event | None] = [None, None]
        for i, l in enumerate(layers):
            if pending is None:
                pending = self._read_pool(doc_id, l, scheme, cfg, metas[l][0], i & 1, dev)
                copies_in_flight[i & 1] = pending[1]
            pool, done = pending
            pending = None
            if i + 1 < len(layers):  # start the next layer's read + copy before this layer's dequant
                nxt = layers[i + 1]
                if copies_in_flight[(i + 1) & 1] is not None:
                    copies_in_flight[(i + 1) & 1].synchronize()  # its staging buffer is free again
                pending = self._read_pool(doc_id, nxt, scheme, cfg, metas[nxt][0], (i + 1) & 1, dev)
                copies_in_flight[(i + 1) & 1] = pending[1]
            n, slots = metas[l]
            torch.cuda.current_stream(dev).wait_event(done)
            k = torch.empty(1, h, n, d, device=dev, dtype=torch.float16)
            v = torch.empty_like(k)
            self.tq.dequant_hnd(scheme, pool, slots, k, v, layout, cfg, stream=self._stream(dev))
            out.append((l, k, v))
            doc_len = doc_len or n
        for ev in copies_in_flight:
            if ev is not None:
                ev.synchronize()
        return out, doc_len

    # ---- one file per document ----------------------------------------------------------------
    def container_path(self, doc_id: str, scheme: Scheme) -> Path:
        return self.store_dir / f"{self._doc_hash(doc_id)[:16]}_{scheme}.tqdoc"

    def export_container(self, doc_id: str, num_layers: int, scheme: Scheme,
                         head_shape: tuple[int, int] = (2, 64)) -> Path:
        """Gather the per-layer files of a stored document into one versioned, self-describing
        file that can be streamed front to back (layout at the top of this module).  Host only."""
        if scheme not in _SCHEME_IDS:
            raise ValueError("containers hold the compressed schemes")
        layers = [l for l in range(num_layers) if self.exists(doc_id, l, scheme)]
        if not layers:
            raise FileNotFoundError(f"No pre-computed KV: doc={doc_id} scheme={scheme}")
        cfg = self._make_cfg_from_shape(head_shape)
        page = int(self._layout(scheme, cfg).page_size_bytes)
        manifest = self._load_manifest()
        sizes = set()
        for l in layers:
            self._verify_manifest(doc_id, l, scheme, head_shape, manifest)
            sizes.add(self._pool_path(doc_id, l, scheme).stat().st_size)
        if len(sizes) != 1:
            raise RuntimeError(f"doc_id={doc_id!r}: layers of different sizes {sorted(sizes)}")
        layer_bytes = sizes.pop()
        n = int(torch.load(self._meta_path(doc_id, layers[0], scheme), weights_only=False)["num_tokens"])
        if layer_bytes != self._pool_bytes(scheme, n, cfg):
            raise RuntimeError(f"doc_id={doc_id!r}: {layer_bytes}-byte pools do not hold {n} tokens of head shape "
                               f"{tuple(head_shape)}")
        stride = _align_up(layer_bytes, _DOC_ALIGN)
        header_bytes = _align_up(_DOC_FIXED.size + 8 * len(layers) + 4, _DOC_ALIGN)
        final, tmp = self.container_path(doc_id, scheme), self.container_path(doc_id, scheme).with_suffix(".tmp")
        table = b""
        with tmp.open("wb") as f:
            f.truncate(header_bytes + stride * len(layers))
            for i, l in enumerate(layers):
                data = self._pool_path(doc_id, l, scheme).read_bytes()
                table += struct.pack("<II", l, zlib.crc32(data))
                f.seek(header_bytes + i * stride)
                f.write(data)
            head = _DOC_FIXED.pack(_DOC_MAGIC, _DOC_VERSION, header_bytes, _SCHEME_IDS[scheme], len(layers), n,
                                   cfg.num_kv_heads, cfg.head_dim, cfg.block_size, page, layer_bytes, stride) + table
            f.seek(0)
            f.write(head + struct.pack("<I", zlib.crc32(head)))
        tmp.replace(final)
        return final

    @staticmethod
    def read_container_header(f) -> dict:
        """Parse and check the header of an open container; raises RuntimeError on a file that is
        not a container of this version or whose header bytes were damaged."""
        fixed = f.read(_DOC_FIXED.size)
        if len(fixed) != _DOC_FIXED.size:
            raise RuntimeError("container: file shorter than its header")
        (magic, version, header_bytes, scheme_id, num_layers, n, h, d, block, page, layer_bytes,
         stride) = _DOC_FIXED.unpack(fixed)
        if magic != _DOC_MAGIC:
            raise RuntimeError("container: bad magic (not a document container)")
        if version != _DOC_VERSION:
            raise RuntimeError(f"container: version {version}, this build reads version {_DOC_VERSION}")
        if num_layers > (1 << 16) or header_bytes < _DOC_FIXED.size + 8 * num_layers + 4:
            raise RuntimeError("container: implausible header")
        table = f.read(8 * num_layers)
        crc = f.read(4)
        if len(table) != 8 * num_layers or len(crc) != 4 or struct.unpack("<I", crc)[0] != zlib.crc32(fixed + table):
            raise RuntimeError("container: header checksum mismatch")
        pairs = [struct.unpack_from("<II", table, 8 * i) for i in range(num_layers)]
        scheme = {v: k for k, v in _SCHEME_IDS.items()}.get(scheme_id)
        if scheme is None:
            raise RuntimeError(f"container: unknown scheme id {scheme_id}")
        return {"scheme": scheme, "num_tokens": n, "head_shape": (h, d), "block_size": block,
                "page_size_bytes": page, "layer_bytes": layer_bytes, "layer_stride": stride,
                "header_bytes": header_bytes, "layers": [p[0] for p in pairs], "crc32": [p[1] for p in pairs]}

    def _stream_container(self, doc_id: str, scheme: Scheme, head_shape, verify: bool, consume) -> int:
        """Read a container front to back: a few reader threads fill a ring of pinned buffers with
        the next layers (positional reads) while layer i goes pinned buffer -> device on the copy
        stream and ``consume(layer, pool, copied_event, header)`` runs.  Returns the document
        length."""
        path = self.container_path(doc_id, scheme)
        if not path.exists():
            raise FileNotFoundError(f"No container: doc={doc_id} scheme={scheme}")
        dev = torch.device("cuda", torch.cuda.current_device())
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(dev)
        with path.open("rb", buffering=0) as f:
            hd = self.read_container_header(f)
            cfg = self._make_cfg_from_shape(hd["head_shape"])
            page = int(self._layout(scheme, cfg).page_size_bytes)
            want = self._pool_bytes(scheme, hd["num_tokens"], cfg)
            if hd["scheme"] != scheme or (head_shape is not None and tuple(head_shape) != tuple(hd["head_shape"])):
                raise RuntimeError(f"container holds {hd['scheme']} with head shape {hd['head_shape']}, asked for "
                                   f"{scheme} {tuple(head_shape) if head_shape else ''}")
            if hd["block_size"] != cfg.block_size or hd["page_size_bytes"] != page or hd["layer_bytes"] != want:
                raise RuntimeError(f"container pages ({hd['block_size']} tokens, {hd['page_size_bytes']} bytes, "
                                   f"{hd['layer_bytes']} per layer) do not match this build "
                                   f"({cfg.block_size}, {page}, {want})")
            nbytes, fd = hd["layer_bytes"], f.fileno()
            ring = min(_READ_RING, len(hd["layers"]))
            hosts = [self._staging(j, nbytes) for j in range(ring)]

            def read_layer(i: int) -> None:
                # positional reads: the reader threads share the descriptor
                view = memoryview(hosts[i % ring].numpy())[:nbytes]
                off, got = hd["header_bytes"] + i * hd["layer_stride"], 0
                while got < nbytes:
                    k = os.preadv(fd, [view[got:]], off + got)
                    if k <= 0:
                        raise RuntimeError(f"{path}: truncated at layer {hd['layers'][i]}")
                    got += k
                if verify and zlib.crc32(view) != hd["crc32"][i]:
                    raise RuntimeError(f"{path}: checksum mismatch in layer {hd['layers'][i]}")

            readers = self._reader_pool()
            reads = {i: readers.submit(read_layer, i) for i in range(ring)}
            copied: list[torch.cuda.Event | None] = [None] * ring
            try:
                for i, l in enumerate(hd["layers"]):
                    reads.pop(i).result()
                    pool, done = self._copy_to_device(hosts[i % ring], nbytes, dev)
                    copied[i % ring] = done
                    # the buffer of the previous layer is free once its copy has finished: hand it to
                    # the reader of the layer one ring ahead of it
                    if i >= 1 and i - 1 + ring < len(hd["layers"]):
                        copied[(i - 1) % ring].synchronize()
                        reads[i - 1 + ring] = readers.submit(read_layer, i - 1 + ring)
                    consume(l, pool, done, hd)
            finally:
                for fut in reads.values():
                    fut.cancel()
                for fut in reads.values():
                    if not fut.cancelled():
                        try:
                            fut.result()
                        except Exception:
                            pass
                for ev in copied:
                    if ev is not None:
                        ev.synchronize()
        return hd["num_tokens"]

    def load_container_pools(self, doc_id: str, scheme: Scheme, head_shape: tuple[int, int] | None = None,
                             verify: bool = False) -> tuple[list, int]:
        """[(layer, pool)] on the device (pages stay compressed) and the document length."""
        out = []
        dev = torch.device("cuda", torch.cuda.current_device())

        def consume(l, pool, done, hd):
            torch.cuda.current_stream(dev).wait_event(done)
            out.append((l, pool))
        n = self._stream_container(doc_id, scheme, head_shape, verify, consume)
        return out, n

    def load_container_hnd(self, doc_id: str, scheme: Scheme, head_shape: tuple[int, int] | None = None,
                           verify: bool = False) -> tuple[list, int]:
        """``load_layers_hnd`` from a container: [(layer, key, value)] with [1, H, N, D] fp16 tensors."""
        out = []
        dev = torch.device("cuda", torch.cuda.current_device())
        state = {}

        def consume(l, pool, done, hd):
            if not state:
                h, d = hd["head_shape"]
                state["cfg"] = self._make_cfg_from_shape((h, d))
                state["layout"] = self._layout(scheme, state["cfg"])
                state["slots"] = torch.arange(hd["num_tokens"], dtype=torch.int32, device=dev)
            h, d = hd["head_shape"]
            torch.cuda.current_stream(dev).wait_event(done)
            k = torch.empty(1, h, hd["num_tokens"], d, device=dev, dtype=torch.float16)
            v = torch.empty_like(k)
            self.tq.dequant_hnd(scheme, pool, state["slots"], k, v, state["layout"], state["cfg"],
                                stream=self._stream(dev))
            out.append((l, k, v))
        n = self._stream_container(doc_id, scheme, head_shape, verify, consume)
        return out, n

    def build_dynamic_cache(self, doc_id: str, num_layers: int, scheme: Scheme,
                            head_shape: tuple[int, int] = (2, 64)):
        """Hugging Face ``DynamicCache`` from the stored layers; returns (cache, doc_num_tokens)."""
        from transformers import DynamicCache
        cache = DynamicCache()
        layers, doc_len = self.load_layers_hnd(doc_id, num_layers, scheme, head_shape)
        for l, k, v in layers:
            cache.update(k, v, l)
        return cache, doc_len

    def attach_to_model(self, model, doc_id: str, num_layers: int, head_shape: tuple[int, int] = (2, 128),
                        scheme: Scheme = "turbo_mse"):
        """Serve a stored turbo_mse / turbo_prod document to a Hugging Face model WITHOUT dequantising
        it: loads the compressed pools (from the one-file container when there is one, else from the
        per-layer files), hangs them on the model's attention layers and returns
        ``(cache, doc_num_tokens)``; pass ``cache`` as ``past_key_values`` (see
        ``turborag_b200/attention_backend.py``).  The counterpart of ``build_dynamic_cache`` for a
        model whose attention reads the pages directly."""
        from . import attention_backend
        if self.container_path(doc_id, scheme).exists():
            loaded, n = self.load_container_pools(doc_id, scheme, head_shape)
            pools = [pool for _, pool in loaded]
        else:
            pools, n = [], 0
            for l in range(num_layers):
                pool, _, n = self.load_document(doc_id, l, scheme, head_shape)
                pools.append(pool)
        return attention_backend.install(model, pools, n, self.tq, scheme), n

    # ---- attention over stored pages ------------------------------------------------------------
    def fused_attention(self, query: torch.Tensor, pool, slots: torch.Tensor, N: int, scheme: Scheme,
                        head_shape: tuple[int, int] = (2, 64)) -> torch.Tensor:
        """Compressed-KV attention; ``query`` [Q, H, D] fp16 (Q rows per kv head), returns [Q, H, D]."""
        if scheme == "fp16":
            key, value = pool
            q, k, v = query.permute(1, 0, 2).float(), key.permute(1, 0, 2).float(), value.permute(1, 0, 2).float()
            attn = torch.softmax(torch.bmm(q, k.transpose(1, 2)) * head_shape[1] ** -0.5, dim=-1)
            return torch.bmm(attn, v).permute(1, 0, 2).to(query.dtype)
        cfg = self._make_cfg_from_shape(head_shape)
        output = torch.empty_like(query)
        fn = {"turbo_prod": self.tq.fused_attn_output, "turbo_mse": self.tq.mse_fused_attn_output,
              "qjl": self.tq.qjl_fused_attn_output}[scheme]
        fn(query.contiguous(), pool, slots, output, self._layout(scheme, cfg), cfg, query.shape[0], N,
           stream=self._stream(query.device))
        return output

    def decode_documents(self, query: torch.Tensor, pools: list[torch.Tensor], lengths: list[int],
                         scheme: Scheme, head_shape: tuple[int, int] = (2, 64)) -> torch.Tensor:
        """One paged GQA decode over a batch of stored documents: ``query`` [B, Hq, D] fp16 (query
        head j belongs to kv head j // (Hq / H)), ``pools[b]`` the loaded pool of document b with
        identity slots (what ``pack_document`` writes), ``lengths[b]`` its token count."""
        if scheme == "fp16":
            raise ValueError("decode_documents serves the compressed schemes")
        cfg = self._make_cfg_from_shape(head_shape)
        layout = self._layout(scheme, cfg)
        page = layout.page_size_bytes
        pages = [p.numel() // page for p in pools]
        pool = torch.cat(pools)
        width = max(max(pages), 1)
        tables = torch.zeros(len(pools), width, dtype=torch.int32)
        first = 0
        for b, n in enumerate(pages):
            tables[b, :n] = torch.arange(first, first + n, dtype=torch.int32)
            first += n
        dev = query.device
        return self.tq.decode_paged(scheme, query.contiguous(), pool, tables.to(dev),
                                    torch.tensor(lengths, dtype=torch.int32, device=dev), layout, cfg,
                                    max_kv_tokens=max(lengths), stream=self._stream(dev))
