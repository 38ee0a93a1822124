"""Benchmark of the compressed-KV hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload decode|longctx] [--layers L --batch B --kv-tokens T]
    (--workload longctx: long-context decode with the KV sequence split across ranks and an
     NCCL all-gather + log-sum-exp merge per layer; the last three options shrink a case)

Workload: fused decode attention over turbo_prod pages — batch 32
sequences x 32768 cached tokens, 36 layers, 16 query heads / 2 kv heads, head_dim 128,
16-token pages, block tables = a seeded random permutation of each layer's pages.  One
step = one decode token for the whole batch through all 36 layers (36 launches of the
decode kernel + 36 of the merge kernel).  Synthetic data: K ~ N(0,1) with four outlier
channels x8, V ~ N(0,1), q ~ N(0,1), packed on the device by this library's pack kernel.

The JSON line carries
  value          GB/s of algorithmic bytes (compressed pages + block tables), pages resident
                 in HBM, CUDA-event time on the launch stream, max over ranks;
  e2e            the same bytes when every layer's pages start in pinned HOST memory and
                 cross PCIe inside the timed region (what the reference's load-then-attend
                 flow does), plus query H2D and output D2H;
  e2e_resident   pages resident (a serving KV cache); query, block tables and sequence
                 lengths go H2D and the outputs come back D2H every step;
  roofline       decode kernel vs the measured HBM copy bandwidth (MEASURED_PEAKS.json);
  cpu_baseline   the CPU oracle (a port of the reference's kernels; the reference has no CPU
                 implementation of this path) on the box's host cores, bounded sample;
  secondary      quantize-pack and dequant GB/s on the offline-store shape (with the CPU oracle's
                 quantiser and the reference's attention_ref_single_head timed beside them), chunk
                 prefill TFLOP/s, and three sharded workloads measured at every N:
                   decode_strong    the same 32 sequences dealt over the ranks (32/N each);
                   longctx_kvsplit  28 layers, 28 q / 4 kv heads, 8 x 131072 tokens, every sequence's
                                    KV range cut over the ranks, (acc, m, l) partials exchanged per
                                    layer by peer stores and by an NCCL all-gather, LSE merge;
                   store_sharded    36 layers x 64 documents x 8192 tokens dealt by (layer, document)
                                    unit: pack (both schemes) and dequant into [head, token, dim].
With N > 1 (torchrun) the headline runs the whole workload on every rank's own sequences (weak
scaling, no data-path collective).

--impl reference: the reference's own CUDA kernels (its only implementation of this path), driven
through its own ctypes wrapper, when oracle/_ref holds them (make -C oracle ref); otherwise the CPU
oracle port on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "fused compressed-KV decode attn GB/s"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one decode-kernel launch at the default
# per-layer shape. Captured with ncu at half the batch (141.06 MB read + 5.09 MB written for
# 140.6 MB of pages) and scaled by the pages one launch reads: every page is read once, so
# traffic grows in proportion. Only valid for the default shape; other shapes report null.
DECODE_DRAM_TRAFFIC_PER_LAUNCH = 2 * (141.06e6 + 4.15e6)
OUTLIERS = (3, 17, 64, 101)


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 50 ms.

    The query process takes a moment to come up (longer on a box with many GPUs), so it is started
    ahead of the warm-up, `begin()` / `end()` mark the loaded window, and only rows that arrive
    inside it are used.  A timed region shorter than a few sampling periods is followed by an
    untimed continuation of the same loop (`hold_load`) so that the window still holds samples
    taken under that load."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    MIN_WINDOW_MS = 400.0

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None
        self.t0 = self.t1 = None
        self.window = "timed region"

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [c.strip() for c in line.split(",")]))

    def wait_ready(self, timeout_s: float = 8.0):
        """Returns once the first row has arrived (or the time is up)."""
        t_end = time.monotonic() + timeout_s
        while self.proc is not None and not self.rows and time.monotonic() < t_end:
            time.sleep(0.02)

    def begin(self):
        self.t0 = time.monotonic()

    def end(self):
        self.t1 = time.monotonic()

    def hold_load(self, total_ms: float, ms_per_step: float, step, sync):
        """Closes the window; if the timed region was short, first keeps `step` running (untimed,
        the same count on every rank) until the window is MIN_WINDOW_MS long."""
        if self.proc is not None and total_ms < self.MIN_WINDOW_MS:
            n = int(min(5000, max(1, np.ceil((self.MIN_WINDOW_MS - total_ms) / max(ms_per_step, 1e-3)))))
            for _ in range(n):
                step()
            sync()
            self.window = f"timed region + {n} untimed steps of the same loop"
        self.end()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.t1 is None:
            self.end()
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        t0 = self.t0 if self.t0 is not None else 0.0
        for t, r in self.rows:
            if not t0 <= t <= self.t1:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm),
                "window": self.window}


def synth_kv(torch, n, h, dev, gen):
    scale = torch.ones(128, device=dev)
    scale[list(OUTLIERS)] = 8.0
    k = (torch.randn(n, h, 128, device=dev, generator=gen) * scale).to(torch.float16)
    v = torch.randn(n, h, 128, device=dev, generator=gen).to(torch.float16)
    return k, v


# -------------------------------------------------------------------------------------
# reference arm: the CPU port on host cores
# -------------------------------------------------------------------------------------

def host_threads():
    """Threads the CPU arm may use: the cores this process is allowed on.  The oracle is told the
    number explicitly -- launchers such as torchrun export OMP_NUM_THREADS=1 to every rank, which
    would otherwise turn the all-cores baseline into a single-thread one."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    from oracle import oracle as O
    O.set_threads(n)
    return n


def cpu_decode_sample(num_seqs, kv_tokens, hq, h, seed=0):
    """Build `num_seqs` packed sequences with the oracle and return a closure that runs one
    pass of oracle decode attention over them, plus the bytes it processes."""
    from oracle import oracle as O
    rng = np.random.default_rng(seed)
    cfg = O.make_config(h)
    lay = O.prod_layout(cfg)
    pages = kv_tokens // 16
    tables = rng.permutation(num_seqs * pages).astype(np.int32).reshape(num_seqs, pages)
    pool = np.zeros(num_seqs * pages * lay.page_size_bytes, np.uint8)
    t = np.arange(kv_tokens)
    for b in range(num_seqs):
        k = rng.standard_normal((kv_tokens, h, 128)).astype(np.float32)
        k[:, :, list(OUTLIERS)] *= 8
        v = rng.standard_normal((kv_tokens, h, 128)).astype(np.float32)
        O.pack("turbo_prod", k.astype(np.float16), v.astype(np.float16),
               (tables[b][t // 16] * 16 + t % 16).astype(np.int32), cfg, pool=pool)
    q = rng.standard_normal((num_seqs, hq, 128)).astype(np.float16)
    lens = np.full(num_seqs, kv_tokens, np.int32)
    nbytes = num_seqs * (kv_tokens * h * 134 + pages * 4)

    def run():
        return O.decode_paged("turbo_prod", q, pool, tables, lens, cfg)
    return run, nbytes


REF_DIR = ROOT / "oracle" / "_ref"


def reference_gpu_arm(args):
    """The reference's kernels, unmodified, through the reference's own ctypes wrapper (both built
    from the reference checkout into oracle/_ref): tq_launch_turbo_prod_pack_kv builds the pages,
    tq_launch_turbo_prod_fused_attention_output reads them, one call per sequence with the 8 query
    rows per kv head of GQA 8:1 (it has no batched entry point).  A step = a bounded sample of the
    workload's sequences for one layer.  Returns False when the reference build or a GPU is missing."""
    from oracle import ref_client
    if not ((REF_DIR / "libturboquant_ref.so").exists() and ref_client.available()):
        return False
    import torch
    if not torch.cuda.is_available():
        return False
    RefWrapper = ref_client.load()[0].TurboQuantWrapper
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    ref = RefWrapper(str(REF_DIR / "libturboquant_ref.so"))
    N, HQ, H = args.kv_tokens, args.q_heads, args.kv_heads
    G = HQ // H
    num_seqs = max(1, min(args.batch, 2))
    cfg = ref.default_config()
    cfg.num_kv_heads, cfg.head_dim = H, 128
    lay = ref.make_layout_for(cfg)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234)
    pages = N // 16
    t = torch.arange(N, device=dev)
    pools, slots_l, qs = [], [], []
    for b in range(num_seqs):
        table = torch.randperm(pages, device=dev, generator=gen).to(torch.int32)
        slots = (table[t // 16].to(torch.int64) * 16 + t % 16).to(torch.int32)
        k, v = synth_kv(torch, N, H, dev, gen)
        pool = torch.zeros(pages * lay.page_size_bytes, dtype=torch.uint8, device=dev)
        ref.pack(k, v, slots, pool, lay, cfg)
        pools.append(pool)
        slots_l.append(slots)
        # reference layout: row g of kv head h = query head h*G + g
        qs.append(torch.randn(G, H, 128, device=dev, generator=gen).to(torch.float16))
    outs = [torch.zeros_like(q) for q in qs]
    host_pools = [p_.cpu().pin_memory() for p_ in pools]
    out_host = torch.zeros(num_seqs, G, H, 128, dtype=torch.float16).pin_memory()
    torch.cuda.synchronize()

    def step():
        for b in range(num_seqs):
            ref.fused_attn_output(qs[b], pools[b], slots_l[b], outs[b], lay, cfg, G, N)

    def step_e2e():
        for b in range(num_seqs):
            pools[b].copy_(host_pools[b], non_blocking=True)
            ref.fused_attn_output(qs[b], pools[b], slots_l[b], outs[b], lay, cfg, G, N)
            out_host[b].copy_(outs[b], non_blocking=True)
        torch.cuda.synchronize()

    sampler = ClockSampler(local).start()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler.wait_ready()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.begin()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    sampler.hold_load(ms * args.steps, ms, step, torch.cuda.synchronize)
    clocks = sampler.stop()
    step_e2e()
    t0 = time.perf_counter()
    e2e_steps = max(1, min(args.steps, 5))
    for _ in range(e2e_steps):
        step_e2e()
    t_e2e = (time.perf_counter() - t0) / e2e_steps
    # slot mappings are per token in the reference API: 4 B per token instead of 4 B per page
    nbytes = num_seqs * (N * H * 134 + N * 4)
    gbs = nbytes / (ms * 1e-3) / 1e9
    sample = (f"{num_seqs} of {args.batch} sequences x {N} tokens x 1 of {args.layers} layers per step, one "
              f"tq_launch_turbo_prod_fused_attention_output call per sequence ({G} query rows x {H} kv heads)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args), "sample": sample},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": 0, "kind": "reference", "sample": sample,
                         "device": "the same B200: the reference implements this path only as CUDA kernels "
                                   "(compiled unmodified for sm_100), it has no CPU implementation"},
        "e2e": {"value": nbytes / t_e2e / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": sum(p_.numel() for p_ in host_pools),
                "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": t_e2e * 1e3,
                "note": "pages copied from pinned host memory before every call, outputs copied back"},
        "gpu_launches": args.steps * num_seqs, "clocks": clocks,
    }))
    return True


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if reference_gpu_arm(args):
        return
    cores = host_threads()
    num_seqs = max(1, min(args.batch, 8))
    run, nbytes = cpu_decode_sample(num_seqs, args.kv_tokens, args.q_heads, args.kv_heads)
    for _ in range(args.warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    dt = (time.perf_counter() - t0) / args.steps
    gbs = nbytes / dt / 1e9
    used = min(cores, num_seqs * args.q_heads)
    sample = (f"{num_seqs} of {args.batch} sequences x {args.kv_tokens} tokens x 1 of {args.layers} layers "
              f"per step, OpenMP over (sequence, query head)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args), "sample": sample},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": used, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def workload_name(args):
    kind = "longctx_kvsplit" if args.workload == "longctx" else "decode"
    return (f"{kind}_turbo_prod_b{args.batch}_kv{args.kv_tokens}_L{args.layers}"
            f"_q{args.q_heads}kv{args.kv_heads}_d128_page16")


# -------------------------------------------------------------------------------------
# long-context decode with the KV sequence split across ranks (one exchange step per layer)
# -------------------------------------------------------------------------------------

def longctx_measure(torch, dist, tq, dev, rank, world, B, N, L, HQ, H, exchanges, steps, warmup, sampler=None):
    """One measurement of the long-context decode with every sequence's KV range cut over the
    ranks (strong scaling: the total work is fixed).  Every rank holds the pages of its contiguous,
    page-aligned token range of every sequence; per layer: local split-KV decode -> (acc, m, l)
    partials, exchange (peer stores over NVLink with the final merge inside the publishing kernel:
    two launches per layer; or one NCCL all-gather and a merge launch), local log-sum-exp merge.
    Returns {exchange: dict} for every name in `exchanges` ("peer", "nccl"; same on every rank):
    whole-job GB/s, microseconds per layer, and the time of the local decode part alone (the same
    launches without the exchange) for the share spent outside it."""
    from turborag_b200.parallel import gather_partials, kv_token_range
    cfg = tq.default_config()
    cfg.num_kv_heads = H
    lay = tq.make_layout_for(cfg)
    lo, hi = kv_token_range(N, rank, world, 16)
    local_pages_per_seq = (hi - lo) // 16
    pages = B * local_pages_per_seq
    gen = torch.Generator(device=dev)
    gen.manual_seed(99 + rank)
    # block tables cover the whole sequence; entries outside [lo, hi) are never read
    tables = torch.zeros(L, B, N // 16, dtype=torch.int32, device=dev)
    pools = torch.zeros(L, pages * lay.page_size_bytes, dtype=torch.uint8, device=dev)
    tpos = torch.arange(lo, hi, device=dev)
    for l in range(L):
        perm = torch.randperm(pages, device=dev, generator=gen).to(torch.int32).view(B, local_pages_per_seq)
        tables[l, :, lo // 16:hi // 16] = perm
        for b in range(B):
            k, v = synth_kv(torch, hi - lo, H, dev, gen)
            slots = (tables[l, b][tpos // 16].to(torch.int64) * 16 + tpos % 16).to(torch.int32)
            tq.pack(k, v, slots, pools[l], lay, cfg)
    lens = torch.full((B,), N, dtype=torch.int32, device=dev)
    q = torch.randn(L, B, HQ, 128, device=dev, generator=gen).to(torch.float16)
    out = torch.zeros(L, B, HQ, 128, dtype=torch.float16, device=dev)
    part = torch.empty(B * HQ, 130, dtype=torch.float32, device=dev)
    ws = torch.empty(max(tq.decode_workspace_bytes(B, HQ, N, cfg), 16), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    xchg = None

    def step():
        for l in range(L):
            if xchg is not None:
                xchg.exchange += 1
                tq.decode_paged_exchange("turbo_prod", q[l], pools[l], tables[l], lens, lay, cfg, xchg.ptr_array,
                                         rank, world, xchg.rows_cap, xchg.exchange, N, lo, hi, out[l],
                                         workspace=ws, stream=stream)
                continue
            tq.decode_paged("turbo_prod", q[l], pools[l], tables[l], lens, lay, cfg,
                            partials_out=part.view(B, HQ, 130), max_kv_tokens=N, kv_begin=lo, kv_end=hi,
                            workspace=ws, stream=stream)
            allp = gather_partials(part) if world > 1 else part.view(1, B * HQ, 130)
            tq.merge_partials(allp, out[l].view(B * HQ, 128), HQ, H, stream=stream)

    def step_local_only():
        # the decode part of a layer alone: same kernels, partials stay on this GPU
        for l in range(L):
            tq.decode_paged("turbo_prod", q[l], pools[l], tables[l], lens, lay, cfg,
                            partials_out=part.view(B, HQ, 130), max_kv_tokens=N, kv_begin=lo, kv_end=hi,
                            workspace=ws, stream=stream)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, clocks=None):
        for _ in range(warmup):
            fn()
        if clocks is not None:
            clocks.wait_ready()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if clocks is not None:
            clocks.begin()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync_all()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total = float(t.item())
        if clocks is not None:
            clocks.hold_load(total, total / steps, fn, sync_all)
        return total / steps

    ms_local = timed(step_local_only)
    total_bytes = L * B * (N * H * 134 + (N // 16) * 4)  # whole job, all ranks together
    res = {}
    for exchange in exchanges:
        if world > 1 and exchange == "peer":
            from turborag_b200.parallel import PeerExchange
            xchg = PeerExchange(tq, B * HQ, dev)
        else:
            xchg = None
        ms_per_step = timed(step, sampler if exchange == exchanges[0] else None)
        status = tq.peer_status() if xchg is not None else 0
        res[exchange] = {
            "value": total_bytes / (ms_per_step * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": ms_per_step,
            "us_per_layer": ms_per_step * 1e3 / L, "us_per_layer_decode_only": ms_local * 1e3 / L,
            "share_outside_decode": max(0.0, 1.0 - ms_local / ms_per_step),
            "exchange": ("none (one rank)" if world == 1 else
                         f"peer stores over NVLink ({xchg.how})" if xchg is not None else "one NCCL all-gather"),
            "partials_bytes_per_rank_per_layer": B * HQ * 130 * 4, "peer_wait_status": status,
            "scaling": "strong", "shape": f"b{B}_kv{N}_L{L}_q{HQ}kv{H}"}
        if world == 1:
            break  # one rank: nothing is exchanged, one measurement serves both names
    return res


def longctx(args):
    """--workload longctx: the KV-split measurement as the headline of its own JSON line."""
    import torch
    import torch.distributed as dist

    import turborag_b200

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    tq = turborag_b200.TurboQuantWrapper()
    B, N, L, HQ, H = args.batch, args.kv_tokens, args.layers, args.q_heads, args.kv_heads
    sampler = ClockSampler(local).start()
    r = longctx_measure(torch, dist, tq, dev, rank, world, B, N, L, HQ, H, (args.exchange,), args.steps, args.warmup,
                        sampler=sampler)
    r = next(iter(r.values()))
    clocks = sampler.stop()
    peak, peak_kind = peaks()
    per_rank = r["value"] / world
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": workload_name(args), "global_batch": B, "kv_tokens": N, "layers": L,
                       "parallelism": (f"kv sequence split over {world} rank(s), {B * HQ * 130 * 4} B of partials per "
                                       f"rank per layer exchanged by {r['exchange']}, local LSE merge"),
                       "l2": "inputs larger than L2"},
            "roofline": {"bound": "hbm", "achieved": per_rank, "peak": peak, "unit": "GB/s",
                         "frac": per_rank / peak, "traffic": None, "peak_kind": peak_kind,
                         "kernel": "decode_paged16_kernel<turbo_prod> + partial exchange + merge, per rank"},
            "detail": r, "gpu_launches": args.steps * L * 3, "clocks": clocks,
        }))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# -------------------------------------------------------------------------------------
# our arm
# -------------------------------------------------------------------------------------

def ours(args):
    import torch
    import torch.distributed as dist

    import turborag_b200

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    tq = turborag_b200.TurboQuantWrapper()  # no library -> FileNotFoundError, no fallback

    B, N, L, HQ, H = args.batch, args.kv_tokens, args.layers, args.q_heads, args.kv_heads
    cfg = tq.default_config()
    cfg.num_kv_heads = H
    lay = tq.make_layout_for(cfg)
    pages_per_seq = N // 16
    pages = B * pages_per_seq
    layer_bytes = pages * lay.page_size_bytes
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)

    # ---- build the paged pools on the device with the pack kernel ---------------------
    pools = torch.zeros(L, layer_bytes, dtype=torch.uint8, device=dev)
    tables = torch.empty(L, B, pages_per_seq, dtype=torch.int32, device=dev)
    tpos = torch.arange(N, device=dev)
    for l in range(L):
        tables[l] = torch.randperm(pages, device=dev, generator=gen).to(torch.int32).view(B, pages_per_seq)
        for b in range(B):
            k, v = synth_kv(torch, N, H, dev, gen)
            slots = (tables[l, b][tpos // 16].to(torch.int64) * 16 + tpos % 16).to(torch.int32)
            tq.pack(k, v, slots, pools[l], lay, cfg)
    lens = torch.full((B,), N, dtype=torch.int32, device=dev)
    q_host = torch.randn(L, B, HQ, 128, generator=torch.Generator().manual_seed(7 + rank)).to(torch.float16).pin_memory()
    q_dev = q_host.to(dev)
    out_dev = torch.zeros(L, B, HQ, 128, dtype=torch.float16, device=dev)
    out_host = torch.zeros(L, B, HQ, 128, dtype=torch.float16).pin_memory()
    ws = torch.empty(max(tq.decode_workspace_bytes(B, HQ, N, cfg), 16), dtype=torch.uint8, device=dev)
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream

    def step_resident():
        for l in range(L):
            tq.decode_paged("turbo_prod", q_dev[l], pools[l], tables[l], lens, lay, cfg, output=out_dev[l],
                            max_kv_tokens=N, workspace=ws, stream=stream)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    bytes_per_launch = B * (N * H * 134 + pages_per_seq * 4)
    bytes_per_step = bytes_per_launch * L
    default_shape = (B, N, H, HQ) == (32, 32768, 2, 16)
    traffic = DECODE_DRAM_TRAFFIC_PER_LAUNCH if default_shape else None

    # ---- value: pages resident, device-timed ------------------------------------------
    sampler = ClockSampler(local).start()
    for _ in range(args.warmup):
        step_resident()
    sampler.wait_ready()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.begin()
    e0.record()
    for _ in range(args.steps):
        step_resident()
    e1.record()
    sync_all()
    total_ms = max_over_ranks(e0.elapsed_time(e1))
    ms_per_step = total_ms / args.steps
    sampler.hold_load(total_ms, ms_per_step, step_resident, sync_all)
    clocks = sampler.stop()
    value = world * bytes_per_step / (ms_per_step * 1e-3) / 1e9
    launch_ms = total_ms / (args.steps * L)
    achieved = bytes_per_launch / (launch_ms * 1e-3) / 1e9
    peak, peak_kind = peaks()

    # ---- e2e_resident: q / tables / lens H2D, outputs D2H every step --------------------
    tables_host = tables.cpu().pin_memory()
    lens_host = lens.cpu().pin_memory()
    tables_in = torch.empty_like(tables)
    lens_in = torch.empty_like(lens)

    def step_e2e_resident():
        q_dev.copy_(q_host, non_blocking=True)
        tables_in.copy_(tables_host, non_blocking=True)
        lens_in.copy_(lens_host, non_blocking=True)
        for l in range(L):
            tq.decode_paged("turbo_prod", q_dev[l], pools[l], tables_in[l], lens_in, lay, cfg,
                            output=out_dev[l], max_kv_tokens=N, workspace=ws, stream=stream)
        out_host.copy_(out_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def wall(fn, steps, warm):
        for _ in range(warm):
            fn()
        sync_all()
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        torch.cuda.synchronize()
        dt = max_over_ranks(time.perf_counter() - t0)
        return dt / steps

    t_res = wall(step_e2e_resident, args.steps, 1)
    h2d_res = q_host.numel() * 2 + tables_host.numel() * 4 + lens_host.numel() * 4
    d2h = out_host.numel() * 2

    # ---- e2e: every layer's pages cross PCIe from pinned host memory ------------------
    host_pool = pools[0].cpu().pin_memory()  # one layer's pages; sent once per layer per step
    staging = [torch.empty(layer_bytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=dev)
    filled = [torch.cuda.Event() for _ in range(2)]
    drained = [torch.cuda.Event() for _ in range(2)]
    main = torch.cuda.current_stream()

    def step_e2e_cold():
        q_dev.copy_(q_host, non_blocking=True)
        tables_in.copy_(tables_host, non_blocking=True)
        lens_in.copy_(lens_host, non_blocking=True)
        for l in range(L):
            s = l & 1
            with torch.cuda.stream(copy_stream):
                if l >= 2:
                    copy_stream.wait_event(drained[s])
                staging[s].copy_(host_pool, non_blocking=True)
                filled[s].record(copy_stream)
            main.wait_event(filled[s])
            tq.decode_paged("turbo_prod", q_dev[l], staging[s], tables_in[0], lens_in, lay, cfg,
                            output=out_dev[l], max_kv_tokens=N, workspace=ws, stream=stream)
            drained[s].record(main)
        out_host.copy_(out_dev, non_blocking=True)
        main.synchronize()

    step_resident()
    torch.cuda.synchronize()
    layer0_resident = out_dev[0].clone()
    cold_steps = max(1, min(args.steps, 3))
    t_cold = wall(step_e2e_cold, cold_steps, 1)
    # the cold loop sends one layer's pages (layer 0's) for every layer: its layer-0 output must be the
    # resident run's, bit for bit
    e2e_same = bool(torch.equal(out_host[0].to(dev), layer0_resident))
    h2d_cold = h2d_res + L * layer_bytes

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": workload_name(args), "global_batch": B * world, "kv_tokens": N, "layers": L,
                   "parallelism": f"sequences sharded, {world} rank(s), no collective",
                   "l2": "inputs larger than L2 (281 MB of pages per launch)",
                   "pct_of_measured_hbm": 100.0 * achieved / peak},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "frac_of_spec_8000_gbs": achieved / 8000.0, "traffic": traffic,
                     "traffic_source": "constant: one ncu capture of this kernel at half the batch, scaled by "
                                       "the pages a launch reads (profiles/decode_turbo_prod_b16_kv32768.md); "
                                       "not measured in this run",
                     "peak_kind": peak_kind, "kernel": "decode_paged16_kernel<turbo_prod,2>",
                     "algorithmic_bytes_per_launch": bytes_per_launch,
                     "launch_ms": launch_ms,
                     "note": "launch_ms = timed region / decode launches; includes the merge kernel and launch gaps"},
        "e2e": {"value": world * bytes_per_step / t_cold / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": h2d_cold, "d2h_bytes_per_step": d2h, "ms_per_step": t_cold * 1e3,
                "layer0_output_equals_resident_run": e2e_same,
                "note": "compressed pages start in pinned host memory and are copied H2D per layer "
                        "inside the timed region (double-buffered against the decode kernel)"},
        "e2e_resident": {"value": world * bytes_per_step / t_res / 1e9, "unit": UNIT,
                         "h2d_bytes_per_step": h2d_res, "d2h_bytes_per_step": d2h, "ms_per_step": t_res * 1e3,
                         "note": "KV pages resident in HBM; query, block tables, lengths H2D and outputs D2H per step"},
        "gpu_launches": args.steps * L * 2,
        "clocks": clocks,
        "tokens_per_s": world * B / (ms_per_step * 1e-3),
    }

    if rank == 0 and world == 1 and not args.skip_cpu:
        line["cpu_baseline"], line["parity"] = cpu_baseline_and_parity(
            torch, tq, args, pools, tables, q_dev, out_dev, lay)
    if not args.skip_secondary:
        sec = {}
        # ---- the same B sequences dealt over the ranks (strong scaling, no collective) ----------
        if B % world == 0:
            b_loc = B // world
            # fewer sequences are split more ways: the split partials need their own, larger workspace
            ws_loc = torch.empty(max(tq.decode_workspace_bytes(b_loc, HQ, N, cfg), 16), dtype=torch.uint8, device=dev)

            def step_strong():
                for l in range(L):
                    tq.decode_paged("turbo_prod", q_dev[l][:b_loc], pools[l], tables[l][:b_loc], lens[:b_loc],
                                    lay, cfg, output=out_dev[l][:b_loc], max_kv_tokens=N, workspace=ws_loc,
                                    stream=stream)
            for _ in range(args.warmup):
                step_strong()
            sync_all()
            e0.record()
            for _ in range(args.steps):
                step_strong()
            e1.record()
            sync_all()
            ms_strong = max_over_ranks(e0.elapsed_time(e1)) / args.steps
            sec["decode_strong"] = {
                "value": bytes_per_step / (ms_strong * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": ms_strong,
                "scaling": "strong", "sequences_total": B, "sequences_per_rank": b_loc,
                "note": "config 3 with its 32 sequences in total: 32/N per rank, no collective"}
        pools = staging = host_pool = tables_in = None  # free 10+ GB before the other workloads
        torch.cuda.empty_cache()
        if rank == 0:
            sec.update(store_numbers(torch, tq, dev, gen, peak, cpu=(world == 1 and not args.skip_cpu)))
        sec["store_sharded"] = store_sharded(torch, dist, tq, dev, rank, world, peak)
        torch.cuda.empty_cache()
        lc = longctx_measure(torch, dist, tq, dev, rank, world, 8, 131072, 28, 28, 4, ("peer", "nccl"),
                             steps=max(2, min(args.steps, 5)), warmup=3)
        sec["longctx_kvsplit"] = lc.get("peer") if world > 1 else next(iter(lc.values()))
        if world > 1:
            sec["longctx_kvsplit_nccl"] = lc.get("nccl")
        torch.cuda.empty_cache()
        if rank == 0 and world == 1:
            sec["decode_turbo_mse"] = decode_mse_numbers(torch, tq, dev, gen, B, N, HQ, H, peak)
            torch.cuda.empty_cache()
            sec["prefill_turbo_mse"] = prefill_numbers(torch, tq, dev, gen)
            if not args.skip_cpu:
                sec["cpu_attention_ref_single_head"] = cpu_attention_ref_numbers()
        line["secondary"] = sec
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def decode_mse_numbers(torch, tq, dev, gen, B, N, HQ, H, peak, layers=4, steps=5):
    """The headline decode shape over turbo_mse pages (4-bit K and V, 132 bytes per token-head): `layers`
    pools of B sequences x N tokens packed on the device, pages permuted, every launch reads another pool
    (inputs larger than L2)."""
    cfg = tq.default_config()
    cfg.num_kv_heads = H
    lay = tq.make_mse_layout_for(cfg)
    pages_per_seq = N // 16
    pages = B * pages_per_seq
    pools = torch.zeros(layers, pages * lay.page_size_bytes, dtype=torch.uint8, device=dev)
    tables = torch.empty(layers, B, pages_per_seq, dtype=torch.int32, device=dev)
    tpos = torch.arange(N, device=dev)
    for l in range(layers):
        tables[l] = torch.randperm(pages, device=dev, generator=gen).to(torch.int32).view(B, pages_per_seq)
        for b in range(B):
            k, v = synth_kv(torch, N, H, dev, gen)
            slots = (tables[l, b][tpos // 16].to(torch.int64) * 16 + tpos % 16).to(torch.int32)
            tq.mse_pack(k, v, slots, pools[l], lay, cfg)
    lens = torch.full((B,), N, dtype=torch.int32, device=dev)
    q = torch.randn(layers, B, HQ, 128, device=dev, generator=gen).to(torch.float16)
    out = torch.zeros(layers, B, HQ, 128, dtype=torch.float16, device=dev)
    ws = torch.empty(max(tq.decode_workspace_bytes(B, HQ, N, cfg), 16), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    def step():
        for l in range(layers):
            tq.decode_paged("turbo_mse", q[l], pools[l], tables[l], lens, lay, cfg, output=out[l],
                            max_kv_tokens=N, workspace=ws, stream=stream)
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (steps * layers)
    nbytes = B * (N * H * 132 + pages_per_seq * 4)
    gbs = nbytes / (us * 1e-6) / 1e9
    return {"value": gbs, "unit": UNIT, "us_per_layer": us, "frac_of_hbm_peak": gbs / peak,
            "bytes_per_launch": nbytes, "shape": f"b{B}_kv{N}_q{HQ}kv{H}"}


def prefill_numbers(torch, tq, dev, gen, batch=8, nq=256, n=32768, hq=16, h=2, iters=5):
    """Chunked query prefill (turbo_mse prefix + causal fp16 chunk): 256 query tokens attend to a
    32768-token compressed prefix, batch 8, 16 q / 2 kv heads.  TFLOP/s over 4*B*Hq*Nq*Nkv*D
    (prefix) + 2*B*Hq*Nq^2*D (causal chunk) flops, against the measured bf16 tensor peak."""
    cfg = tq.default_config()
    cfg.num_kv_heads = h
    lay = tq.make_mse_layout_for(cfg)
    pages = batch * n // 16
    pool = torch.zeros(pages * lay.page_size_bytes, dtype=torch.uint8, device=dev)
    tables = torch.randperm(pages, device=dev, generator=gen).to(torch.int32).view(batch, n // 16).contiguous()
    t = torch.arange(n, device=dev)
    for b in range(batch):
        k, v = synth_kv(torch, n, h, dev, gen)
        tq.mse_pack(k, v, (tables[b][t // 16].to(torch.int64) * 16 + t % 16).to(torch.int32), pool, lay, cfg)
    q = torch.randn(batch, nq, hq, 128, device=dev, generator=gen).to(torch.float16)
    ck, cv = synth_kv(torch, batch * nq, h, dev, gen)
    ck, cv = ck.view(batch, nq, h, 128), cv.view(batch, nq, h, 128)
    lens = torch.full((batch,), n, dtype=torch.int32, device=dev)
    out = torch.empty_like(q)
    for _ in range(3):
        tq.mse_prefill_paged(q, pool, tables, lens, ck, cv, out, lay, cfg)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        tq.mse_prefill_paged(q, pool, tables, lens, ck, cv, out, lay, cfg)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    flops = 4.0 * batch * hq * nq * n * 128 + 2.0 * batch * hq * nq * nq * 128
    tensor_peak = 1655.3
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        tensor_peak = float(json.loads(pk.read_text())["bf16_tflops"])
    return {"value": flops / ms / 1e9, "unit": "TFLOP/s", "ms": ms, "frac_of_tensor_peak": flops / ms / 1e9 / tensor_peak,
            "shape": f"b{batch}_q{nq}_kv{n}_q{hq}kv{h}", "note": "tcgen05 + TMEM tensor tiles"}


def side_workload(args):
    """--workload store | prefill: the secondary kernels alone (used for ncu captures)."""
    import torch

    import turborag_b200
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    tq = turborag_b200.TurboQuantWrapper()
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    peak, _ = peaks()
    if args.workload == "store":
        res = store_numbers(torch, tq, dev, gen, peak)
        print(json.dumps({"metric": "quantize-pack GB/s", "value": res["pack_turbo_prod"]["value"], "unit": "GB/s",
                          "n_gpus": 1, "config": {"workload": "store_16docs_x8192_L1_kv2_d128"}, "secondary": res}))
    elif args.workload == "load":
        res = load_numbers(torch, dev, gen, tokens=args.kv_tokens or 8192, layers=args.layers or 36)
        print(json.dumps({"metric": "document load ms (disk -> [1,H,N,D] fp16 cache, all layers)",
                          "value": res["ours_ms"], "unit": "ms", "n_gpus": 1, "higher_is_better": False,
                          "config": {"workload": res["shape"]}, "secondary": res}))
    elif args.workload == "ttft":
        res = ttft_numbers(torch, dev, gen, tokens=args.kv_tokens or 8192, layers=args.layers or 36)
        print(json.dumps({"metric": "stored document -> attention outputs of the question chunk, all layers (ms)",
                          "value": res["compressed_pages_ms"], "unit": "ms", "n_gpus": 1, "higher_is_better": False,
                          "config": {"workload": res["shape"]}, "secondary": res}))
    else:
        res = prefill_numbers(torch, tq, dev, gen, batch=args.batch or 8, iters=max(1, args.steps))
        print(json.dumps({"metric": "chunk prefill TFLOP/s", "value": res["value"], "unit": "TFLOP/s", "n_gpus": 1,
                          "config": {"workload": "prefill_turbo_mse_" + res["shape"]}, "secondary": res}))


def ttft_numbers(torch, dev, gen, tokens, layers, question=64):
    """The attention part of answering a question over a stored document (no model weights): from
    the files on disk to the attention outputs of a `question`-token chunk in every layer.
      dequantised_cache_ms : the reference's flow on this library's kernels -- load + dequantise every
                             layer into fp16 [1, H, N, D] (what build_dynamic_cache does), then fp16
                             attention of the chunk over [document ; chunk] per layer (torch SDPA);
      compressed_pages_ms  : load the compressed pools only and let tq_mse_prefill_paged read them.
    Files in the page cache, wall clock, best of 5; both produce the chunk's attention output per layer."""
    import tempfile
    import time

    import torch.nn.functional as F

    from turborag_b200.store import CAGStore
    H, D, HQ = 2, 128, 16
    with tempfile.TemporaryDirectory() as tmp:
        st = CAGStore(tmp)
        for l in range(layers):
            k, v = synth_kv(torch, tokens, H, dev, gen)
            st.pack_document("doc", l, k, v, "turbo_mse")
        st.export_container("doc", layers, "turbo_mse", (H, D))
        cfg = st._make_cfg_from_shape((H, D))
        lay = st.tq.make_mse_layout_for(cfg)
        q = torch.randn(1, question, HQ, D, device=dev, generator=gen).to(torch.float16)
        ck, cv = synth_kv(torch, question, H, dev, gen)
        ck, cv = ck.view(1, question, H, D), cv.view(1, question, H, D)
        pages = (tokens + 15) // 16
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, -1)
        lens = torch.tensor([tokens], dtype=torch.int32, device=dev)
        causal = torch.ones(question, tokens + question, dtype=torch.bool, device=dev)
        causal[:, tokens:] = torch.tril(torch.ones(question, question, dtype=torch.bool, device=dev))

        def dequantised():
            outs = []
            loaded, _ = st.load_container_hnd("doc", "turbo_mse", (H, D))
            for _, k4, v4 in loaded:
                kk = torch.cat([k4, ck.permute(0, 2, 1, 3)], dim=2)
                vv = torch.cat([v4, cv.permute(0, 2, 1, 3)], dim=2)
                outs.append(F.scaled_dot_product_attention(q.permute(0, 2, 1, 3), kk, vv, attn_mask=causal,
                                                           enable_gqa=True))
            torch.cuda.synchronize()
            return outs

        def compressed():
            outs = []
            loaded, _ = st.load_container_pools("doc", "turbo_mse", (H, D))
            for _, pool in loaded:
                out = torch.empty_like(q)
                st.tq.mse_prefill_paged(q, pool, table, lens, ck, cv, out, lay, cfg)
                outs.append(out)
            torch.cuda.synchronize()
            return outs

        a, b = dequantised(), compressed()
        err = max(float(((x.permute(0, 2, 1, 3).float() - y.float()).abs().amax(-1) /
                         x.float().abs().amax(-1).permute(0, 2, 1).clamp_min(1e-6)).max()) for x, y in zip(a, b))
        times = {}
        for name, fn in (("compressed_pages_ms", compressed), ("dequantised_cache_ms", dequantised)):
            best = 1e9
            for _ in range(5):
                t0 = time.perf_counter()
                fn()
                best = min(best, (time.perf_counter() - t0) * 1e3)
            times[name] = best
    return {"shape": f"ttft_turbo_mse_{tokens}tok_L{layers}_q{question}_hq{HQ}kv{H}", **times,
            "max_rel_diff_between_the_two": err,
            "device_bytes_for_the_document": {"compressed_pages": layers * st.vram_bytes("turbo_mse", tokens, (H, D)),
                                              "dequantised_cache": layers * 2 * tokens * H * D * 2},
            "note": "wall clock, best of 5, files in the page cache"}


def load_numbers(torch, dev, gen, tokens, layers):
    """Time from files on disk to the dequantised [1, H, N, D] fp16 tensors of every layer of one
    stored document: the store's overlapped path (pinned readinto, side-stream copy,
    [H, N, D]-writing dequant) against the reference's sequence of host copies (read_bytes ->
    bytearray -> frombuffer -> clone -> .to(cuda), dequant to [N, H, D], permute().contiguous()),
    both on this library's kernels and on the same files (page cache warm)."""
    import tempfile
    import time

    from turborag_b200.store import CAGStore
    H, D = 2, 128
    with tempfile.TemporaryDirectory() as tmp:
        st = CAGStore(tmp)
        for l in range(layers):
            k, v = synth_kv(torch, tokens, H, dev, gen)
            st.pack_document("doc", l, k, v, "turbo_prod")
        cfg = st._make_cfg_from_shape((H, D))
        lay = st.tq.make_layout_for(cfg)

        def ours():
            out, n = st.load_layers_hnd("doc", layers, "turbo_prod", (H, D))
            torch.cuda.synchronize()
            return out

        def reference_style():
            out = []
            for l in range(layers):
                raw = st._pool_path("doc", l, "turbo_prod").read_bytes()
                meta = torch.load(st._meta_path("doc", l, "turbo_prod"), weights_only=False)
                pool = torch.frombuffer(bytearray(raw), dtype=torch.uint8).clone().to(dev, non_blocking=True)
                slots = meta["slots"].to(dev)
                k = torch.zeros(tokens, H, D, device=dev, dtype=torch.float16)
                v = torch.zeros_like(k)
                st.tq.dequant(pool, slots, k, v, lay, cfg)
                out.append((l, k.permute(1, 0, 2).unsqueeze(0).contiguous(), v.permute(1, 0, 2).unsqueeze(0).contiguous()))
            torch.cuda.synchronize()
            return out

        st.export_container("doc", layers, "turbo_prod", (H, D))

        def container():
            out, n = st.load_container_hnd("doc", "turbo_prod", (H, D))
            torch.cuda.synchronize()
            return out

        a, b, c = ours(), reference_style(), container()
        same = all(torch.equal(x[1], y[1]) and torch.equal(x[2], y[2]) and torch.equal(x[1], z[1]) and
                   torch.equal(x[2], z[2]) for x, y, z in zip(a, b, c))
        times = {}
        for name, fn in (("ours_ms", ours), ("container_ms", container), ("reference_style_ms", reference_style)):
            best = 1e9
            for _ in range(5):
                t0 = time.perf_counter()
                fn()
                best = min(best, (time.perf_counter() - t0) * 1e3)
            times[name] = best
        pool_bytes = layers * st.vram_bytes("turbo_prod", tokens, (H, D))
    return {"shape": f"load_turbo_prod_{tokens}tok_L{layers}_kv{H}_d{D}", **times, "identical_output": bool(same),
            "pool_bytes": pool_bytes, "note": "wall clock, best of 5, files in the page cache"}


def store_sharded(torch, dist, tq, dev, rank, world, peak, layers=36, docs=64, tokens=8192, H=2, passes=3):
    """Offline store build at its stated size: 36 layers x 64 documents x 8192 tokens, 2 kv heads.
    The 2304 (layer, document) units are dealt to the ranks by parallel.shard_range (contiguous,
    layer-major, no communication); a rank packs (turbo_prod and turbo_mse) and dequantises (both,
    into fp16 [layer, head, token, dim]) the documents of a layer that fell to it with one launch per
    kernel -- their pages are contiguous in the layer's pool, so a document's slice of it is byte
    for byte the pool a per-document call writes.  GB/s of algorithmic bytes over the max-over-ranks
    time of a pass.  Inputs: one set of 64 synthetic documents reused for every layer (268 MB per
    tensor, larger than L2); outputs and pools are distinct memory for every unit."""
    from turborag_b200.parallel import shard_range
    cfg = tq.default_config()
    cfg.num_kv_heads = H
    gen = torch.Generator(device=dev)
    gen.manual_seed(4242)
    k_all, v_all = synth_kv(torch, docs * tokens, H, dev, gen)
    slots = torch.arange(docs * tokens, dtype=torch.int32, device=dev)
    units = shard_range(layers * docs, rank, world)
    runs = []  # (layer, first document, one past the last document) of this rank
    for u in units:
        l, d = divmod(u, docs)
        if runs and runs[-1][0] == l and runs[-1][2] == d:
            runs[-1][2] = d + 1
        else:
            runs.append([l, d, d + 1])
    lays = {s: tq.layout_for_scheme(s, cfg) for s in ("turbo_prod", "turbo_mse")}
    pools = {s: [torch.zeros((hi - lo) * (tokens // 16) * lays[s].page_size_bytes, dtype=torch.uint8, device=dev)
                 for _, lo, hi in runs] for s in lays}
    outs = [(torch.empty(H, (hi - lo) * tokens, 128, dtype=torch.float16, device=dev),
             torch.empty(H, (hi - lo) * tokens, 128, dtype=torch.float16, device=dev)) for _, lo, hi in runs]
    stream = torch.cuda.current_stream().cuda_stream

    def one_pass():
        for i, (_, lo, hi) in enumerate(runs):
            n = (hi - lo) * tokens
            k, v = k_all[lo * tokens:hi * tokens], v_all[lo * tokens:hi * tokens]
            tq.pack(k, v, slots[:n], pools["turbo_prod"][i], lays["turbo_prod"], cfg, stream=stream)
            tq.mse_pack(k, v, slots[:n], pools["turbo_mse"][i], lays["turbo_mse"], cfg, stream=stream)
            for s in ("turbo_prod", "turbo_mse"):
                tq.dequant_hnd(s, pools[s][i], slots[:n], outs[i][0], outs[i][1], lays[s], cfg, stream=stream)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    one_pass()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(passes):
        one_pass()
    e1.record()
    sync_all()
    t = torch.tensor([e0.elapsed_time(e1) / passes], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    per_token = sum(2 * (2 * H * 128 * 2 + 4 + H * w) for w in (134, 132))  # pack + dequant, both schemes
    total = layers * docs * tokens * per_token
    gbs = total / (ms * 1e-3) / 1e9
    return {"value": gbs, "unit": "GB/s", "ms_per_pass": ms, "scaling": "strong", "units": layers * docs,
            "units_per_rank": len(units), "launches_per_rank_per_pass": 4 * len(runs),
            "frac_of_hbm_peak_per_gpu": gbs / world / peak,
            "shape": f"L{layers}_docs{docs}_x{tokens}_kv{H}", "ops": "pack turbo_prod + pack turbo_mse + dequant both into [head, token, dim]"}


def cpu_pack_numbers(tokens=8192, H=2):
    """The CPU oracle's quantiser (the port of the reference's pack kernels) on one store unit of
    8192 tokens, on one thread and on all host cores (OpenMP over token-heads)."""
    from oracle import oracle as O
    rng = np.random.default_rng(0)
    k = rng.standard_normal((tokens, H, 128)).astype(np.float32)
    k[:, :, list(OUTLIERS)] *= 8
    k = k.astype(np.float16)
    v = rng.standard_normal((tokens, H, 128)).astype(np.float16)
    slots = np.arange(tokens, dtype=np.int32)
    cfg = O.make_config(H)
    cores = host_threads()
    res = {}
    for scheme, w in (("turbo_prod", 134), ("turbo_mse", 132)):
        nbytes = tokens * (2 * H * 128 * 2 + 4 + H * w)
        for label, threads in (("all_cores", cores), ("one_thread", 1)):
            O.set_threads(threads)
            O.pack(scheme, k, v, slots, cfg)
            reps, t0 = 0, time.perf_counter()
            while reps < 3 or time.perf_counter() - t0 < 1.0:
                O.pack(scheme, k, v, slots, cfg)
                reps += 1
            dt = (time.perf_counter() - t0) / reps
            res[f"{scheme}_{label}"] = {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": threads}
    O.set_threads(cores)
    res["kind"] = "port"
    res["sample"] = f"one (layer, document) unit: {tokens} tokens x {H} kv heads"
    return res


def cpu_attention_ref_numbers(n=32768, d=128, pairs=32):
    """attention_ref_single_head (the reference's one CPU routine on this path: fp32 dense attention
    of one query over one head's fp16 K/V), its own compiled code when oracle/_ref holds it (else the
    oracle's restatement): one call on one thread, and `pairs` (sequence, head) calls spread over the
    host cores by a thread pool.  Bytes = the fp16 K and V it reads (4 x 128 B per token)."""
    from concurrent.futures import ThreadPoolExecutor

    from oracle import oracle as O
    rng = np.random.default_rng(1)
    q = rng.standard_normal(d).astype(np.float16)
    k = rng.standard_normal((n, d)).astype(np.float16)
    v = rng.standard_normal((n, d)).astype(np.float16)
    own = O.ref_host() is not None
    fn = O.ref_attention_single_head if own else O.attention_ref_single_head
    fn(q, k, v)
    t0 = time.perf_counter()
    fn(q, k, v)
    one = time.perf_counter() - t0
    cores = host_threads()
    with ThreadPoolExecutor(max_workers=cores) as ex:
        t0 = time.perf_counter()
        list(ex.map(lambda _: fn(q, k, v), range(pairs)))
        many = time.perf_counter() - t0
    nbytes = n * d * 2 * 2
    return {"one_thread": {"value": nbytes / one / 1e9, "unit": "GB/s of fp16 K/V", "cores": 1, "ms_per_head": one * 1e3},
            "all_cores": {"value": pairs * nbytes / many / 1e9, "unit": "GB/s of fp16 K/V", "cores": min(cores, pairs)},
            "kind": "reference" if own else "port",
            "sample": f"{pairs} (sequence, head) pairs x {n} tokens x {d} dims, one query row each"}


def store_numbers(torch, tq, dev, gen, peak, cpu=False):
    """quantize-pack and dequant GB/s on the offline-store shape: 16 documents x 8192 tokens of
    one layer (2 kv heads), permuted pages; inputs 2 x 67 MB, larger than L2."""
    H, n = 2, 16 * 8192
    cfg = tq.default_config()
    cfg.num_kv_heads = H
    k, v = synth_kv(torch, n, H, dev, gen)
    perm = torch.randperm(n // 16, device=dev, generator=gen)
    t = torch.arange(n, device=dev)
    slots = (perm[t // 16] * 16 + t % 16).to(torch.int32)
    ok, ov = torch.empty_like(k), torch.empty_like(v)
    res = {}
    for scheme, w in (("turbo_prod", 134), ("turbo_mse", 132)):
        lay = tq.layout_for_scheme(scheme, cfg)
        pool = torch.zeros((n // 16) * lay.page_size_bytes, dtype=torch.uint8, device=dev)
        pack = tq.pack if scheme == "turbo_prod" else tq.mse_pack
        deq = tq.dequant if scheme == "turbo_prod" else tq.mse_dequant
        by = n * (2 * H * 128 * 2 + 4 + H * w)
        for name, fn in (("pack", lambda: pack(k, v, slots, pool, lay, cfg)),
                         ("dequant", lambda: deq(pool, slots, ok, ov, lay, cfg))):
            for _ in range(3):
                fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(10):
                fn()
            e1.record()
            torch.cuda.synchronize()
            gbs = by / (e0.elapsed_time(e1) / 10 * 1e-3) / 1e9
            res[f"{name}_{scheme}"] = {"value": gbs, "unit": "GB/s", "frac_of_hbm_peak": gbs / peak,
                                       "bytes_per_token": by // n}
    if cpu:
        res["cpu_baseline_pack"] = cpu_pack_numbers()
    return res


def cpu_baseline_and_parity(torch, tq, args, pools, tables, q_dev, out_dev, lay):
    """Oracle decode on host cores over a bounded sample of layer 0 (same pages, same queries),
    timed, and compared with what the GPU produced for those sequences."""
    from oracle import oracle as O
    B, N, HQ, H = args.batch, args.kv_tokens, args.q_heads, args.kv_heads
    cfg = O.make_config(H)
    pool = pools[0].cpu().numpy()
    tab = tables[0].cpu().numpy()
    q = q_dev[0].cpu().numpy()
    got = out_dev[0].cpu().numpy().astype(np.float32)
    cores = host_threads()
    # calibrate on one sequence, then size the sample for roughly 10-20 s of CPU work
    t0 = time.perf_counter()
    O.decode_paged("turbo_prod", q[:1], pool, tab[:1], [N], cfg)
    t1 = time.perf_counter() - t0
    # one sequence keeps at most HQ threads busy; more sequences fill the remaining cores
    est_per_seq = t1 if cores <= HQ else t1 * HQ / cores
    s = int(max(1, min(B, round(15.0 / max(est_per_seq, 1e-3)))))
    t0 = time.perf_counter()
    ref = O.decode_paged("turbo_prod", q[:s], pool, tab[:s], [N] * s, cfg).astype(np.float32)
    dt = time.perf_counter() - t0
    nbytes = s * (N * H * 134 + (N // 16) * 4)
    err = float((np.abs(got[:s] - ref).max(-1) / np.abs(ref).max(-1)).max())
    sample = f"{s} of {B} sequences x {N} tokens, layer 0 of {args.layers}, OpenMP over (sequence, query head)"
    return ({"value": nbytes / dt / 1e9, "unit": UNIT, "cores": min(cores, s * HQ), "kind": "port",
             "sample": sample, "seconds": dt},
            {"decode_rel_err_vs_oracle": err, "sequences_checked": s, "tolerance": 2e-3})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "longctx", "store", "prefill", "load", "ttft"])
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--kv-tokens", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--q-heads", type=int, default=None)
    ap.add_argument("--kv-heads", type=int, default=None)
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="longctx on several GPUs: how the split-KV partials travel")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-secondary", action="store_true")
    args = ap.parse_args()
    if args.workload in ("store", "prefill", "load", "ttft"):
        side_workload(args)
        return
    shape = {"decode": (32, 32768, 36, 16, 2), "longctx": (8, 131072, 28, 28, 4)}[args.workload]
    for name, val in zip(("batch", "kv_tokens", "layers", "q_heads", "kv_heads"), shape):
        if getattr(args, name) is None:
            setattr(args, name, val)
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        reference_arm(args)
    elif args.workload == "longctx":
        longctx(args)
    else:
        ours(args)


if __name__ == "__main__":
    main()
