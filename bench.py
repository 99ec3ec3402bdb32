#!/usr/bin/env python
"""Benchmark of the LiteDSA sparse-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c1] [--impl ours|reference]

One "step" is one pass of the hot path (union_qm + masked_mla_fp8) over one chunk of
query tokens of the configuration the headline metric is quoted on (config 1: 8192 query
tokens at the tail of a 32K FP8 KV cache, 64 heads, top-k 2048, 75 % overlap inside a
tile).  Synthetic, seeded data (litetopk_b200.synth); the KV cache is drawn in the
"ref-compatible" mode (per-128 scales all equal one power of two, q and rope on the e4m3
grid) so the identical operands are consumable by the all-e4m3 reference-format kernel.

N > 1 (launched under torchrun, one rank per GPU): every rank owns an independent chunk
of the same shape (weak scaling: tile-aligned query blocks, KV cache replicated) and the
bf16 outputs are all-gathered with NCCL, chunk by chunk on a side stream while the next
chunk computes.  Prints ONE JSON line on rank 0.

--impl reference times the CPU restatement of the reference path (oracle/) on the host
cores on a bounded sample of the same workload; the reference has no CPU implementation
of its own and its GPU module is a checker here, not a product path.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from litetopk_b200 import synth  # noqa: E402

METRIC = "sparse_mla_prefill_query_tokens_per_s"
# DRAM bytes per launch of masked_mla_fp8_kernel on the benchmark workload, from the ncu
# capture summarised in profiles/masked_mla_fp8_kernel_c1_2048tok.md (scaled to 8192 tokens)
ATTN_DRAM_TRAFFIC_BYTES = 700_000_000  # 189.3 MB captured on 2048 tokens, q/out/index part scaled x4


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self._stop = threading.Event()
        self._t = None

    def _run(self):
        try:
            p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                  "-i", str(self.gpu), "-lms", "100"], stdout=subprocess.PIPE, text=True)
        except OSError:
            return
        while not self._stop.is_set():
            line = p.stdout.readline()
            if not line:
                break
            self.rows.append([x.strip() for x in line.split(",")])
        p.terminate()

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        time.sleep(0.15)
        self._stop.set()
        self._t.join(timeout=2)

    def summary(self):
        mhz, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                mhz.append(float(r[1])); mx = float(r[2])
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(mhz)}


def cpu_reference_sample(w: synth.Workload, tiles: int, seed: int):
    """One pass of the CPU restatement (union + reference-numerics attention) over `tiles` tiles."""
    import numpy as np
    from oracle import attention_oracle as ao
    from oracle import union_oracle as uo
    idx = synth.make_topk(w, seed=seed, num_tiles=tiles)
    kv = synth.make_kv_cache(w.s_kv, seed=seed, mode="refcompat")
    q = synth.make_q(tiles * w.group, w.heads, seed=seed, mode="refcompat")
    q8, kv8, qs, ks = synth.refcompat_operands(q, kv)
    q8f = q8.view(torch.float8_e4m3fn).float().view(tiles, 128, 576)
    kv8f = kv8.view(torch.float8_e4m3fn).float()

    def step():
        u, c, m = uo.union_qm_oracle(idx.numpy(), w.group, w.s_kv)
        return ao.masked_mla_refnum(q8f, kv8f, torch.from_numpy(u), torch.from_numpy(c),
                                    torch.from_numpy(m.astype(np.int64)), synth.SM_SCALE * qs * ks,
                                    ks, w.heads, tile_chunk=8)
    return step, tiles * w.group


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tiles = args.cpu_tiles
    step, tokens = cpu_reference_sample(w, tiles, seed=1)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = tokens / dt
    cores = torch.get_num_threads()
    sample = f"{tiles} tiles ({tokens} query tokens) of {w.name} per step, PyTorch eager CPU oracle"
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "e4m3",
            "data": "synthetic", "config": config_dict(w, args),
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port",
                             "sample": sample},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def config_dict(w, args):
    return {"workload": f"{w.name}: {w.tokens} query tokens at the tail of a {w.s_kv}-token FP8 KV cache, "
                        f"{w.heads} q heads (d_qk 576, d_v 512), top-k {w.topk}, "
                        f"{int(w.overlap[0] * 100)}-{int(w.overlap[1] * 100)}% in-tile overlap, per GPU",
            "kv_format": "e4m3 codes + one power-of-two scale per 128 dims (all equal; ref-compatible), "
                         "bf16 rope on the e4m3 grid",
            "tokens_per_gpu": w.tokens, "tokens_per_tile": w.group, "seed": 1,
            "l2_policy": "inputs+outputs per step (~0.9 GB) exceed the 126 MB L2; the 19 MB KV cache stays "
                         "resident by design",
            "parallelism": f"dp{args.gpus} (query-token blocks; KV replicated; all-gather of out)"}


def run_dsv4(args, w):
    """Config 3 (DSv4 packed BF16 two-range attention), single GPU: a secondary bench line."""
    from litetopk_b200 import api
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    q, kc, kr = synth.make_dsv4(w, seed=1, device=dev)
    pos0 = w.pos0
    step = lambda: api.dsv4_c128a_bf16(q, kc, kr, pos0, synth.SM_SCALE, window=w.window, ratio=w.ratio)
    api.dsv4_status(reset=True)
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    with ClockSampler(0) as clk:
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    if api.dsv4_status()[0] != 0:
        raise SystemExit("device-side wait expired")
    pairs = synth.attended_pairs(w)
    flop = pairs * synth.FLOP_PER_PAIR
    peaks = load_peaks()
    ach = flop / (ms * 1e-3) / 1e12
    # bytes a tile reads: its compressed prefix and window rows once (bf16, 576 dims)
    G = w.group
    p_last = torch.arange(w.pos0 + G - 1, w.pos0 + w.tokens, G, dtype=torch.int64)
    rows = int((torch.clamp(p_last // w.ratio, max=w.n_compressed) + w.window + G - 1).sum())
    line = {"metric": METRIC, "value": w.tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{w.name}: DSv4 packed BF16 attention, {w.tokens} query tokens at the tail of a "
                                   f"{w.s_kv}-token context, {w.heads} heads, compressed prefix (<= {w.n_compressed} "
                                   f"entries, ratio {w.ratio}) + window {w.window}", "seed": 1},
            "effective_tflops": ach,
            "roofline": {"kernel": "dsv4_kernel", "bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops"], "traffic": None,
                         "peak_source": f"bf16 dense of {peaks['source']}",
                         "kv_bytes_per_step": rows * 1152, "kv_gbs": rows * 1152 / (ms * 1e-3) / 1e9},
            "gpu_launches": args.steps, "clocks": clk.summary(), "cpu_baseline": None, "e2e": None}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="c1")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-tiles", type=int, default=32)
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--e2e-q", choices=("e4m3", "bf16"), default="e4m3",
                    help="dtype of the host-resident queries of the end-to-end leg")
    ap.add_argument("--gather", choices=("auto", "fused", "ce", "nccl"), default="auto",
                    help="N > 1: how the ranks' outputs are gathered (auto: the fastest measured "
                         "form for this N: epilogue peer stores up to 4 GPUs, NCCL beyond)")
    ap.add_argument("--scaling", choices=("weak", "strong"), default="weak",
                    help="N > 1: the configuration per GPU (weak) or split across the GPUs (strong)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tokens", type=int, default=0,
                    help="shrink the workload to this many query tokens per GPU (profiling aid; "
                         "the default, the full configuration, is the only benchmark number)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    w = synth.CONFIGS[args.config]
    if args.tokens:
        w = synth.scaled(w, tokens=args.tokens)
    if w.kind == "dsv4":
        return run_dsv4(args, w)
    if args.impl == "reference":
        return run_reference(args, w)

    from litetopk_b200 import api
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if args.gather == "auto":
        args.gather = "fused" if world <= 4 else "nccl"
    if args.scaling == "strong" and world > 1:
        if w.tokens % (world * w.group):
            raise SystemExit("strong scaling needs tokens divisible by gpus x tokens-per-tile")
        w = synth.scaled(w, tokens=w.tokens // world)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_
        dist = dist_
        dist.init_process_group("nccl", device_id=dev)

    # ---- resident operands of this rank's chunk (seed differs per rank: independent chunks)
    seed = 1 + rank
    idx = synth.make_topk(w, seed=seed, device=dev)
    kv656 = synth.make_kv_cache(w.s_kv, seed=1, device=dev, mode="refcompat")
    q = synth.make_q(w.tokens, w.heads, seed=seed, device=dev, mode="refcompat")
    ks = qs = synth.REFCOMPAT_SCALE
    kv8 = api.repack_kv656(kv656, ks)
    q8 = api.quantize_e4m3(q, qs).view(w.tiles, 128, 576)
    G, ng, cap = w.group, w.tiles, w.cap
    u = torch.empty((ng, cap), dtype=torch.int32, device=dev)
    cnt = torch.empty((ng,), dtype=torch.int32, device=dev)
    msk = torch.empty((ng, G, cap // 32), dtype=torch.int32, device=dev)
    out = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=dev) if world == 1 else None
    lse = torch.empty((ng, 128), dtype=torch.float32, device=dev)
    sm = synth.SM_SCALE * qs * ks
    n_chunks = 4 if world > 1 else 1
    gatherer = None
    peer_out = None
    gather_kind = "none"
    if world > 1:
        from litetopk_b200 import dist as ldist
        if args.gather in ("fused", "ce"):
            try:   # the kernel's epilogue writes every rank's copy through peer-mapped memory
                peer_out = ldist.PeerGatheredOutput(ng, (128, 512), torch.bfloat16, dev)
                gather_kind = ("fused: TMA tile stores of the attention epilogue into every rank's buffer (symmetric memory) + barrier"
                               if args.gather == "fused" else
                               "ce: chunked copy-engine pushes into every rank's buffer (symmetric memory) on side streams + barrier")
            except Exception as e:     # symmetric memory not available on this box
                gather_kind = f"nccl (symmetric memory unavailable: {type(e).__name__})"
        flags = torch.tensor([1 if peer_out is not None else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        if int(flags.item()) == 0:
            peer_out = None
            if gather_kind.startswith(("fused", "ce")):
                gather_kind = "nccl (symmetric memory unavailable on a peer)"
        if peer_out is None:
            if args.gather == "nccl":
                gather_kind = "nccl: chunked all_gather_into_tensor on a side stream"
            gatherer = ldist.ChunkedAllGather(ng, (128, 512), torch.bfloat16, dev, n_chunks=n_chunks)
    launches = [0]
    attn_events = []
    timed_flag = [False]
    gather_on = [True]

    def attn_chunk(a, b, dst, peers=None):
        if timed_flag[0]:
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
        api.masked_mla_fp8_out(q8[a:b], kv8, u[a:b], sm, ks, cnt[a:b], msk[a:b], w.heads, dst, None,
                               lse[a:b], peer_outs=peers)
        launches[0] += 1
        if timed_flag[0]:
            e1.record(); attn_events.append((e0, e1, b - a))

    def step(timed=False):
        timed_flag[0] = timed
        api.union_qm_out(idx, u, cnt, msk, None, None, 1, w.s_kv)
        launches[0] += 1
        if peer_out is not None and gather_on[0] and args.gather == "ce":
            ldist.copy_engine_sharded_attention(attn_chunk, peer_out, n_chunks)
        elif peer_out is not None and args.gather == "ce":
            cb = ldist.chunk_bounds(ng, n_chunks)
            for i in range(n_chunks):
                attn_chunk(cb[i], cb[i + 1], peer_out.local()[cb[i]:cb[i + 1]])
        elif peer_out is not None and gather_on[0]:
            ldist.fused_sharded_attention(lambda dst, peers: attn_chunk(0, ng, dst, peers), peer_out)
        elif peer_out is not None:
            attn_chunk(0, ng, peer_out.local())
        elif world > 1 and gather_on[0]:
            ldist.sharded_attention(attn_chunk, gatherer)
        elif world > 1:
            for i in range(gatherer.n_chunks):
                attn_chunk(gatherer.bounds[i], gatherer.bounds[i + 1], gatherer.local(i))
        else:
            attn_chunk(0, ng, out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    api.attn_status(reset=True)
    for _ in range(args.warmup):
        step()
    barrier()
    launches[0] = 0
    ev0 = torch.cuda.Event(enable_timing=True); ev1 = torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        barrier()
        ev0.record()
        for _ in range(args.steps):
            step(timed=True)
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1) / args.steps
    st = api.attn_status()
    if st[0] != 0:
        raise SystemExit(f"device-side wait expired: status {st}")
    attn_ms = sum(e0.elapsed_time(e1) for e0, e1, _ in attn_events) / args.steps   # all chunks of a step
    if world > 1:
        t = torch.tensor([ms, attn_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, attn_ms = float(t[0]), float(t[1])
    launches_per_step = launches[0] // args.steps
    ms_compute_only = None
    if world > 1:   # the same steps without the collective: what the all-gather costs
        gather_on[0] = False
        barrier()
        c0 = torch.cuda.Event(enable_timing=True); c1 = torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(args.steps):
            step()
        c1.record()
        barrier()
        t = torch.tensor([c0.elapsed_time(c1) / args.steps], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_compute_only = float(t[0])
        gather_on[0] = True

    # ---- end to end through the public API with host buffers (rank-local), copies inside the timing
    # q travels as e4m3 codes, the input dtype of the reference operator
    # (masked_mla_fp8(q8, ...), kernels/b200/dsa/litedsa.cu:77); --e2e-q bf16 uploads bf16 queries
    # and quantises them on the device inside the timed region instead
    q_src = q if args.e2e_q == "bf16" else q8.view(w.tokens, w.heads, 576)
    q_host = q_src.cpu().pin_memory(); idx_host = idx.cpu().pin_memory()
    out_host = torch.empty((w.tokens, w.heads, 512), dtype=torch.bfloat16).pin_memory()
    lse_host = torch.empty((w.tokens, w.heads), dtype=torch.float32).pin_memory()

    def e2e_step():
        # chunks of 512 tokens: upload, kernels and download of neighbouring chunks overlap
        api.sparse_prefill_host(q_host, kv8, idx_host, synth.SM_SCALE, out_host=out_host,
                                lse_host=lse_host, kv_scale=ks, q_scale=qs, seq_space=w.s_kv)

    for _ in range(min(2, args.e2e_steps)):
        e2e_step()
    barrier()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / args.e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t[0])
    h2d = q_host.numel() * q_host.element_size() + idx_host.numel() * 4
    d2h = out_host.numel() * 2 + lse_host.numel() * 4

    # ---- work model: 2176 FLOP per attended (query-head, key) pair; gather bytes per union row
    pairs = int((idx >= 0).sum().item()) * w.heads
    union_rows = int(cnt.sum().item())
    flop = pairs * synth.FLOP_PER_PAIR
    peaks = load_peaks()
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    achieved = flop / (attn_ms * 1e-3) / 1e12

    line = {
        "metric": METRIC, "value": world * w.tokens / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "e4m3",
        "data": "synthetic", "config": config_dict(w, args),
        "effective_tflops": world * flop / (ms * 1e-3) / 1e12,
        "compute_only": None if ms_compute_only is None else {
            "ms_per_step": ms_compute_only, "value": world * w.tokens / (ms_compute_only * 1e-3),
            "note": "same steps with the all-gather of the outputs switched off"},
        "gather": gather_kind,
        "all_gather_bytes_per_rank_per_step": (world - 1) * ng * 128 * 512 * 2,
        "roofline": {"kernel": "masked_mla_fp8_kernel", "bound": "tensor", "achieved": achieved,
                     "peak": fp8_peak, "unit": "TFLOP/s", "frac": achieved / fp8_peak,
                     "traffic": ATTN_DRAM_TRAFFIC_BYTES if (w.name == "c1" and not args.tokens) else None,
                     "peak_source": f"2 x bf16 dense {peaks['bf16_tflops']} TFLOP/s of {peaks['source']} "
                                    "(FP8 dense is not in MEASURED_PEAKS.json); nominal FP8 dense 4500",
                     "kernel_ms_per_launch": attn_ms / (1 if (peer_out is not None and args.gather == "fused") else n_chunks),
                     "algorithmic_flop_per_step": flop,
                     "executed_flop_per_step": union_rows * 128 * synth.FLOP_PER_PAIR,
                     "gather_bytes_per_step": union_rows * 576,
                     "gather_gbs": union_rows * 576 / (attn_ms * 1e-3) / 1e9},
        "e2e": {"value": world * w.tokens / (e2e_ms * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                "host_q_dtype": args.e2e_q},
        "gpu_launches": launches_per_step * args.steps,
        "gpu_launches_per_step": launches_per_step,
        "clocks": None, "cpu_baseline": None,
    }
    if rank == 0:
        line["clocks"] = clk.summary()
        if world == 1 and not args.no_cpu_baseline:
            stp, tokens = cpu_reference_sample(w, args.cpu_tiles, seed=1)
            stp()
            t0 = time.perf_counter()
            reps = 3
            for _ in range(reps):
                stp()
            dt = (time.perf_counter() - t0) / reps
            line["cpu_baseline"] = {
                "value": tokens / dt, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                "sample": f"{args.cpu_tiles} tiles ({tokens} query tokens) of {w.name}, union + "
                          "reference-numerics attention in PyTorch eager on the host cores"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
