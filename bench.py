#!/usr/bin/env python
"""Benchmark of the LiteDSA sparse-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c1] [--impl ours|reference]

One "step" is one pass of the hot path (union_qm + masked_mla_fp8) over one chunk of
query tokens of the configuration the headline metric is quoted on (config 1: 8192 query
tokens at the tail of a 32K FP8 KV cache, 64 heads, top-k 2048, 75 % overlap inside a
tile).  Synthetic, seeded data (litetopk_b200.synth); the KV cache of the headline is drawn
in the "ref-compatible" mode (per-128 scales all equal one power of two, q and rope on the
e4m3 grid) so that the identical operands are consumable by the reference's own sm_100a
module, which is timed beside ours.

The ONE JSON line rank 0 prints carries, beside the headline contract keys:
  roofline        masked_mla_fp8_kernel against the FP8 dense rate measured here by the
                  library's own tcgen05 probe (and 2 x the measured bf16 figure beside it)
  ref_module      the reference's sm_100a module on the same operands, timed in a child
                  process (the product process never maps the checker)
  configs         secondary records for configs 2, 3 and 4 (N = 1 only)
  native          config 1 on a cache whose per-128 scales differ, bf16 q (the bf16 route)
  indexer         the step before: FP8 index logits + exact top-k selection on the config-1 shape
  merge_kv_splits the lse merge of KV-split outputs (HBM-bound)
  stock_sparse_mla the stock per-token sparse MLA prefill (FlashMLA, library code) on configs 1, 2, 4
  c4_strong       config 4 split over the N ranks (strong scaling) with its all-gather
  e2e             through api.sparse_prefill_host with pinned host buffers and bf16 queries:
                  median step of a window, the better of two windows (both arms alike; the
                  --impl reference arm uploads the same bf16 queries and quantises with torch ops)
  gather_verified N > 1: every rank's gathered buffer equals what the owners computed

N > 1 (launched under torchrun, one rank per GPU): every rank owns an independent chunk
of the same shape (weak scaling: tile-aligned query blocks, KV cache replicated) and the
bf16 outputs are all-gathered.

--impl reference times the reference's own sm_100a module (oracle/_ref, compiled from the
reference checkout by oracle/build_ref.sh) on the same operands on ONE GPU; when the module
is absent it falls back to the CPU restatement of the path (oracle/) and says so.
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
# DRAM bytes per launch of masked_mla_fp8_kernel on the benchmark workload: ncu capture of the
# kernel on 2048 tokens of config 1 (197.8 MB read + written), q / out / index part scaled x 4
# ((197.8 - 18.9 MB of KV cache) x 4 + 18.9)
ATTN_DRAM_TRAFFIC_BYTES = 735_000_000
REF_SO = os.path.join(ROOT, "oracle", "_ref", "litedsa_ref.so")
REF_DSV4_SO = os.path.join(ROOT, "oracle", "_ref", "litedsa_dsv4_ref.so")


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


def cuda_time(fn, steps, warmup=3):
    """Average milliseconds per call of fn over `steps` calls (CUDA events on the current stream)."""
    for _ in range(warmup):
        fn()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def cuda_time_steps(fn, steps, warmup=3):
    """Milliseconds of each of `steps` consecutive calls of fn (CUDA events between the calls, no
    synchronisation inside the loop)."""
    for _ in range(warmup):
        fn()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    torch.cuda.synchronize()
    ev[0].record()
    for i in range(steps):
        fn()
        ev[i + 1].record()
    torch.cuda.synchronize()
    return [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]


def median(xs):
    ys = sorted(xs)
    n = len(ys)
    return ys[n // 2] if n % 2 else 0.5 * (ys[n // 2 - 1] + ys[n // 2])


E2E_METHOD = ("median over the timed steps of a window, the better of two windows taken at different "
              "times of the run (the host's PCIe path is shared with other tenants: a window can run "
              "at half the copy rate); the same method in both arms")


# ------------------------------------------------------------------------------------ CPU restatement
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


def cpu_baseline_record(w, tiles, reps=3):
    stp, tokens = cpu_reference_sample(w, tiles, seed=1)
    stp()
    t0 = time.perf_counter()
    for _ in range(reps):
        stp()
    dt = (time.perf_counter() - t0) / reps
    return {"value": tokens / dt, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{tiles} tiles ({tokens} query tokens) of {w.name}, union + reference-numerics "
                      "attention in PyTorch eager on the host cores"}


# ------------------------------------------------------------------------------------ the reference's sm_100a module
def _refcompat_gpu_operands(w, seed, dev):
    """Ref-compatible operands of a workload built with torch ops only (no product library)."""
    idx = synth.make_topk(w, seed=seed, device=dev)
    kv = synth.make_kv_cache(w.s_kv, seed=1, device=dev, mode="refcompat")
    q = synth.make_q(w.tokens, w.heads, seed=seed, device=dev, mode="refcompat")
    q8, kv8, qs, ks = synth.refcompat_operands(q, kv)
    return idx, q8.view(w.tiles, 128, 576), kv8, qs, ks


def ref_module_measure(w, steps, dev, e2e_steps=0):
    """Times the reference's own module (union_qm + masked_mla_fp8, or its DSv4 operator) on the
    workload's seeded operands.  Returns a dict, or {'unavailable': why}."""
    try:
        import tvm_ffi
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"tvm_ffi not importable ({type(e).__name__})"}
    if w.kind == "dsv4":
        if not os.path.exists(REF_DSV4_SO):
            return {"unavailable": "oracle/_ref/litedsa_dsv4_ref.so not built"}
        mod = tvm_ffi.load_module(REF_DSV4_SO)
        q, kc, kr = synth.make_dsv4(w, seed=1, device=dev)
        ops = synth.dsv4_rank_space_operands(q[..., :512].contiguous(), kc[:, :512].contiguous(),
                                             kr[:, :512].contiguous(), w.pos0, w.heads, w.window, w.ratio)
        del q, kr
        ng = w.tiles
        out = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=dev)
        lse = torch.empty((ng, 128), dtype=torch.float32, device=dev)
        sink = torch.full((128,), -float("inf"), dtype=torch.float32, device=dev)
        ms = cuda_time(lambda: mod.dsv4_masked_mla_bf16(ops[0], ops[1], ops[2], ops[3], ops[4], ops[5], ops[6],
                                                         float(synth.SM_SCALE), w.heads, out, lse, sink), steps)
        return {"attn_ms": ms, "union_us": None, "ms_per_step": ms, "value": w.tokens / (ms * 1e-3),
                "note": "the reference kernel covers d = 512 only: rope dims dropped (6 % fewer FLOP), "
                        "union list + rank ranges prebuilt outside the timing"}
    if not os.path.exists(REF_SO):
        return {"unavailable": "oracle/_ref/litedsa_ref.so not built"}
    mod = tvm_ffi.load_module(REF_SO)
    idx, q8, kv8, qs, ks = _refcompat_gpu_operands(w, 1, dev)
    ng, G, cap = w.tiles, w.group, w.cap
    u = torch.empty((ng, cap), dtype=torch.int32, device=dev)
    cnt = torch.empty((ng,), dtype=torch.int32, device=dev)
    msk = torch.empty((ng, G, cap // 32), dtype=torch.int32, device=dev)
    req = torch.zeros((ng,), dtype=torch.int32, device=dev)
    tab = torch.arange(w.s_kv, dtype=torch.int32, device=dev)[None, :].contiguous()
    out = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=dev)
    lse = torch.empty((ng, 128), dtype=torch.float32, device=dev)
    ml = torch.empty_like(lse)
    sm = float(synth.SM_SCALE * qs * ks)
    kv3 = kv8.view(w.s_kv, 1, 576)

    def union():
        mod.union_qm(idx, u, cnt, msk, req, tab, 1, w.s_kv)

    def attn():
        mod.masked_mla_fp8(q8, kv3, u.view(ng, 1, cap), sm, float(ks), cnt, msk, w.heads, out, ml, lse)

    union()
    union_ms = cuda_time(union, steps)
    attn_ms = cuda_time(attn, steps)
    step_ms = cuda_time(lambda: (union(), attn()), steps)
    rec = {"union_us": union_ms * 1e3, "attn_ms": attn_ms, "ms_per_step": step_ms,
           "value": w.tokens / (step_ms * 1e-3)}
    if e2e_steps:
        # The module through host buffers the plain way (it has no host-side pipeline), one stream.
        # Headline form, like the other arm's: the configuration's bf16 queries are uploaded and
        # brought to the operator's e4m3 input with plain torch ops on the device (the reference
        # ships no quantiser), then both operators, then out + lse are downloaded.  Beside it the
        # form whose host queries are e4m3 codes already.
        q_bf16 = (q8.view(torch.float8_e4m3fn).float() * qs).to(torch.bfloat16)     # exact: q is on the e4m3 grid
        hosts = {"bf16": q_bf16.cpu().pin_memory(), "e4m3": q8.cpu().pin_memory()}
        idx_host = idx.cpu().pin_memory()
        out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        lse_host = torch.empty(lse.shape, dtype=lse.dtype).pin_memory()
        inv = 1.0 / float(qs)

        def e2e_bf16():
            q_bf16.copy_(hosts["bf16"], non_blocking=True); idx.copy_(idx_host, non_blocking=True)
            q8.copy_((q_bf16 * inv).to(torch.float8_e4m3fn).view(torch.uint8))
            union(); attn()
            out_host.copy_(out, non_blocking=True); lse_host.copy_(lse, non_blocking=True)

        def e2e_e4m3():
            q8.copy_(hosts["e4m3"], non_blocking=True); idx.copy_(idx_host, non_blocking=True)
            union(); attn()
            out_host.copy_(out, non_blocking=True); lse_host.copy_(lse, non_blocking=True)
        wins = {"bf16": [], "e4m3": []}
        for _ in range(2):
            wins["bf16"].append(median(cuda_time_steps(e2e_bf16, e2e_steps)))
            wins["e4m3"].append(median(cuda_time_steps(e2e_e4m3, e2e_steps)))
            cuda_time(lambda: (union(), attn()), steps)          # a little distance between the windows
        recs = {}
        for name in ("bf16", "e4m3"):
            ms = min(wins[name])
            recs[name] = {"value": w.tokens / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
                          "windows_ms": wins[name],
                          "h2d_bytes_per_step": hosts[name].numel() * hosts[name].element_size() + idx_host.numel() * 4,
                          "d2h_bytes_per_step": out_host.numel() * 2 + lse_host.numel() * 4,
                          "host_q_dtype": name}
        rec["e2e"] = dict(recs["bf16"])
        rec["e2e"]["e4m3_q"] = recs["e4m3"]
        rec["e2e"]["method"] = E2E_METHOD
        rec["e2e"]["note"] = ("upload, (bf16 form: e4m3 quantisation with torch ops,) union_qm, masked_mla_fp8, "
                              "download in sequence")
    return rec


def ref_module_worker(args, w):
    """Child-process entry: time the reference module and print one JSON line."""
    torch.cuda.set_device(0)
    print(json.dumps(ref_module_measure(w, args.steps, torch.device("cuda", 0))), flush=True)


def ref_module_leg(cfg_name, tokens, steps):
    """Run the reference-module timing in a child process so this process never maps it."""
    cmd = [sys.executable, os.path.abspath(__file__), "--ref-module-worker", "--config", cfg_name,
           "--steps", str(steps)]
    if tokens:
        cmd += ["--tokens", str(tokens)]
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    env["CUDA_VISIBLE_DEVICES"] = os.environ.get("LOCAL_RANK", "0") if "CUDA_VISIBLE_DEVICES" not in os.environ \
        else os.environ["CUDA_VISIBLE_DEVICES"].split(",")[int(os.environ.get("LOCAL_RANK", "0"))]
    try:
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=420)
    except subprocess.TimeoutExpired:
        return {"unavailable": "reference-module child timed out"}
    for line in reversed(r.stdout.strip().splitlines()):
        if line.startswith("{"):
            try:
                return json.loads(line)
            except ValueError:
                break
    return {"unavailable": f"reference-module child failed (exit {r.returncode}): {r.stderr.strip()[-200:]}"}


def run_reference(args, w):
    """--impl reference: the reference's own module on one GPU (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = torch.get_num_threads()
    rec = None
    if torch.cuda.is_available():
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        rec = ref_module_measure(w, max(args.steps, 3), torch.device("cuda", torch.cuda.current_device()),
                                 e2e_steps=args.e2e_steps)
    line = {"impl": "reference", "metric": METRIC, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "data": "synthetic", "config": config_dict(w, args)}
    if rec is not None and "unavailable" not in rec:
        e2e = rec.pop("e2e", None) or {"value": rec["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                                       "d2h_bytes_per_step": 0}
        line.update({"value": rec["value"], "ms_per_step": rec["ms_per_step"], "dtype": "e4m3" if w.kind == "fp8" else "bf16",
                     "reference_class": "gpu_module",
                     "reference_note": "the reference's own sm_100a module (union_qm + masked_mla_fp8) on ONE GPU, "
                                       "operands resident; it has no multi-GPU path, so the figure does not grow with N",
                     "ref_module": rec, "e2e": e2e,
                     "cpu_baseline": {"value": rec["value"], "unit": "tokens/s", "cores": 0, "kind": "reference",
                                      "sample": f"the whole of {w.name} per step on one B200 (the reference has no "
                                                "CPU implementation; its GPU module is the reference arm)"}})
        print(json.dumps(line), flush=True)
        return
    # fallback: the CPU restatement (the module is not built here)
    tiles = args.cpu_tiles
    step, tokens = cpu_reference_sample(w, tiles, seed=1)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = tokens / dt
    sample = f"{tiles} tiles ({tokens} query tokens) of {w.name} per step, PyTorch eager CPU oracle"
    line.update({"value": val, "ms_per_step": dt * 1e3, "dtype": "e4m3", "reference_class": "cpu_port",
                 "reference_note": "reference module unavailable: " + (rec or {}).get("unavailable", "no CUDA device"),
                 "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
                 "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    print(json.dumps(line), flush=True)


def config_dict(w, args):
    if w.kind == "dsv4":
        return {"workload": f"{w.name}: DSv4 packed BF16 attention, {w.tokens} query tokens at the tail of a "
                            f"{w.s_kv}-token context, {w.heads} heads, compressed prefix (<= {w.n_compressed} "
                            f"entries, ratio {w.ratio}) + window {w.window}", "seed": 1}
    return {"workload": f"{w.name}: {w.tokens} query tokens at the tail of a {w.s_kv}-token FP8 KV cache, "
                        f"{w.heads} q heads (d_qk 576, d_v 512), top-k {w.topk}, "
                        f"{int(w.overlap[0] * 100)}-{int(w.overlap[1] * 100)}% in-tile overlap, per GPU",
            "kv_format": "e4m3 codes + one power-of-two scale per 128 dims (all equal; ref-compatible), "
                         "bf16 rope on the e4m3 grid",
            "tokens_per_gpu": w.tokens, "tokens_per_tile": w.group, "seed": 1,
            "l2_policy": "inputs+outputs per step (~0.9 GB) exceed the 126 MB L2; the 19 MB KV cache stays "
                         "resident by design",
            "parallelism": f"dp{args.gpus} (query-token blocks; KV replicated; all-gather of out)"}


# ------------------------------------------------------------------------------------ single-GPU records
def fp8_peaks(api):
    """FP8 / bf16 dense rates measured by the library's own tcgen05 probe on this GPU."""
    rec = {}
    for kind in ("fp8", "bf16"):
        for m in (256, 128):
            try:
                rec[f"{kind}_m{m}"] = api.probe_mma_tflops(kind, m_pair=m, iters=16384)
            except Exception as e:  # noqa: BLE001
                rec[f"{kind}_m{m}"] = None
                rec["error"] = f"{type(e).__name__}: {e}"
    return rec


def fp8_config_record(api, w, dev, steps, fp8_peak, with_ref, label=None):
    """Device-resident union + FP8 attention on a whole configuration (ref-compatible data)."""
    idx = synth.make_topk(w, seed=1, device=dev)
    kv656 = synth.make_kv_cache(w.s_kv, seed=1, device=dev, mode="refcompat")
    q = synth.make_q(w.tokens, w.heads, seed=1, device=dev, mode="refcompat")
    ks = qs = synth.REFCOMPAT_SCALE
    kv8 = api.repack_kv656(kv656, ks)
    q8 = api.quantize_e4m3(q, qs).view(w.tiles, 128, 576)
    del q, kv656
    G, ng, cap = w.group, w.tiles, w.cap
    u = torch.empty((ng, cap), dtype=torch.int32, device=dev)
    cnt = torch.empty((ng,), dtype=torch.int32, device=dev)
    msk = torch.empty((ng, G, cap // 32), dtype=torch.int32, device=dev)
    out = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=dev)
    lse = torch.empty((ng, 128), dtype=torch.float32, device=dev)
    sm = synth.SM_SCALE * qs * ks
    union = lambda: api.union_qm_out(idx, u, cnt, msk, None, None, 1, w.s_kv)  # noqa: E731
    attn = lambda: api.masked_mla_fp8_out(q8, kv8, u, sm, ks, cnt, msk, w.heads, out, None, lse)  # noqa: E731
    api.attn_status(reset=True)
    union()
    union_ms = cuda_time(union, steps)
    attn_ms = cuda_time(attn, steps)
    step_ms = cuda_time(lambda: (union(), attn()), steps)
    if api.attn_status()[0] != 0:
        raise SystemExit("device-side wait expired")
    pairs = int((idx >= 0).sum().item()) * w.heads
    rows = int(cnt.sum().item())
    flop = pairs * synth.FLOP_PER_PAIR
    ach = flop / (attn_ms * 1e-3) / 1e12
    union_bytes = idx.numel() * 4 + rows * 4 + ng * 4 + int(((cnt + 31) // 32).sum().item()) * G * 4
    rec = {"workload": label or w.name, "tokens": w.tokens, "ms_per_step": step_ms,
           "value": w.tokens / (step_ms * 1e-3), "unit": "tokens/s",
           "kernel_ms_per_launch": attn_ms, "union_us": union_ms * 1e3,
           "effective_tflops": ach, "executed_tflops": rows * 128 * synth.FLOP_PER_PAIR / (attn_ms * 1e-3) / 1e12,
           "frac": ach / fp8_peak, "union_gbs": union_bytes / (union_ms * 1e-3) / 1e9,
           "gather_gbs": rows * 576 / (attn_ms * 1e-3) / 1e9}
    del idx, q8, kv8, u, cnt, msk, out, lse
    torch.cuda.empty_cache()
    if with_ref:
        ref = ref_module_leg(w.name, 0, steps)
        if "unavailable" not in ref:
            ref["ratio_attn"] = ref["attn_ms"] / attn_ms
            ref["ratio_union"] = ref["union_us"] / (union_ms * 1e3)
            ref["ratio_path"] = ref["ms_per_step"] / step_ms
        rec["ref_module"] = ref
    return rec


def dsv4_config_record(api, w, dev, steps, bf16_peak, with_ref):
    q, kc, kr = synth.make_dsv4(w, seed=1, device=dev)
    pos0 = w.pos0
    step = lambda: api.dsv4_c128a_bf16(q, kc, kr, pos0, synth.SM_SCALE, window=w.window, ratio=w.ratio)  # noqa: E731
    api.dsv4_status(reset=True)
    ms = cuda_time(step, steps)
    if api.dsv4_status()[0] != 0:
        raise SystemExit("device-side wait expired")
    pairs = synth.attended_pairs(w)
    flop = pairs * synth.FLOP_PER_PAIR
    ach = flop / (ms * 1e-3) / 1e12
    G = w.group
    p_last = torch.arange(w.pos0 + G - 1, w.pos0 + w.tokens, G, dtype=torch.int64)
    rows = int((torch.clamp(p_last // w.ratio, max=w.n_compressed) + w.window + G - 1).sum())
    rec = {"workload": w.name, "tokens": w.tokens, "ms_per_step": ms, "value": w.tokens / (ms * 1e-3),
           "unit": "tokens/s", "kernel_ms_per_launch": ms, "effective_tflops": ach, "frac": ach / bf16_peak,
           "peak": bf16_peak, "dtype": "bf16", "kv_bytes_per_step": rows * 1152,
           "kv_gbs": rows * 1152 / (ms * 1e-3) / 1e9}
    # the same problem through the entry point with the reference's argument list (gathered
    # index list + rank ranges, 576 dims)
    ops = synth.dsv4_rank_space_operands(q, kc, kr, pos0, w.heads, w.window, w.ratio)
    ng = w.tiles
    out = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=dev)
    lse = torch.empty((ng, 128), dtype=torch.float32, device=dev)
    api.bf16_status(reset=True)
    api.dsv4_status(reset=True)
    call = lambda detect: api.dsv4_masked_mla_bf16_out(ops[0], ops[1], ops[2], ops[3], ops[4], ops[5], ops[6],  # noqa: E731
                                                       synth.SM_SCALE, w.heads, out, lse, None, detect_runs=detect)
    ms_g = cuda_time(lambda: call(True), steps)       # lists classified on the device: the range kernel runs
    ms_gg = cuda_time(lambda: call(False), steps)     # the gather kernel, whatever the lists look like
    if api.bf16_status()[0] != 0 or api.dsv4_status()[0] != 0:
        raise SystemExit("device-side wait expired")
    rec["gathered_list_form"] = {"ms_per_step": ms_g, "value": w.tokens / (ms_g * 1e-3),
                                 "frac": flop / (ms_g * 1e-3) / 1e12 / bf16_peak,
                                 "entry": "dsv4_masked_mla_bf16 (reference argument list), 576 dims; the index "
                                          "lists are classified on the device (two contiguous runs each) and "
                                          "the range kernel reads K / V with tiled TMA loads",
                                 "gather_kernel_ms": ms_gg}
    del q, kc, kr, ops, out, lse
    torch.cuda.empty_cache()
    if with_ref:
        ref = ref_module_leg(w.name, 0, steps)
        if "unavailable" not in ref:
            ref["ratio_attn"] = ref["attn_ms"] / ms
            ref["ratio_same_signature"] = ref["attn_ms"] / ms_g     # both through the reference's argument list
        rec["ref_module"] = ref
    return rec


def native_record(api, w, dev, steps, bf16_peak):
    """Config shape on a cache whose per-128 scales differ, bf16 N(0,1) q: the bf16 route."""
    idx = synth.make_topk(w, seed=1, device=dev)
    kv656 = synth.make_kv_cache(w.s_kv, seed=1, device=dev, mode="native")
    q = synth.make_q(w.tokens, w.heads, seed=1, device=dev, mode="native")
    G, ng, cap = w.group, w.tiles, w.cap
    u = torch.empty((ng, cap), dtype=torch.int32, device=dev)
    cnt = torch.empty((ng,), dtype=torch.int32, device=dev)
    msk = torch.empty((ng, G, cap // 32), dtype=torch.int32, device=dev)
    out = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=dev)
    lse = torch.empty((ng, 128), dtype=torch.float32, device=dev)
    ws = torch.empty((w.s_kv, 576), dtype=torch.bfloat16, device=dev)
    qt = q.view(ng, 128, 576)
    deq = lambda: api.dequant_kv656(kv656, ws)  # noqa: E731
    union = lambda: api.union_qm_out(idx, u, cnt, msk, None, None, 1, w.s_kv)  # noqa: E731
    attn = lambda: api.masked_mla_bf16_out(qt, ws, u, synth.SM_SCALE, cnt, msk, w.heads, out, None, lse)  # noqa: E731
    api.bf16_status(reset=True)
    deq(); union()
    deq_ms = cuda_time(deq, steps)
    attn_ms = cuda_time(attn, steps)
    step_ms = cuda_time(lambda: (deq(), union(), attn()), steps)
    if api.bf16_status()[0] != 0:
        raise SystemExit("device-side wait expired")
    pairs = int((idx >= 0).sum().item()) * w.heads
    flop = pairs * synth.FLOP_PER_PAIR
    ach = flop / (attn_ms * 1e-3) / 1e12
    rec = {"workload": f"{w.name}, native cache (per-128 fp32 scales amax/448, bf16 rope), bf16 N(0,1) q",
           "route": "dequant_kv656 -> union_qm -> masked_mla_bf16 (bf16 tcgen05 MMAs)",
           "ms_per_step": step_ms, "value": w.tokens / (step_ms * 1e-3), "unit": "tokens/s",
           "kernel_ms_per_launch": attn_ms, "dequant_us": deq_ms * 1e3, "effective_tflops": ach,
           "frac": ach / bf16_peak, "peak": bf16_peak, "dtype": "bf16"}
    del idx, kv656, q, u, cnt, msk, out, lse, ws
    torch.cuda.empty_cache()
    return rec


def indexer_record(api, w, dev, steps, fp8_peak, hbm_gbs, index_heads=64):
    """The step before the union on the headline's shape: FP8 index logits of the config's query
    tokens against its whole KV length, then the exact top-k selection that yields topk_idx."""
    T, S, k = w.tokens, w.s_kv, w.topk
    pos0 = S - T
    q8, k8, wts, ks = synth.make_indexer_operands(T, S, index_heads, seed=1, device=dev)
    logits = torch.empty((T, S), dtype=torch.float32, device=dev)
    sel = torch.empty((T, k), dtype=torch.int32, device=dev)
    f_log = lambda: api.index_logits_fp8(q8, k8, wts, ks, pos0, out=logits)  # noqa: E731
    f_sel = lambda: api.topk_select(logits, k, q_pos0=pos0, out=sel)  # noqa: E731
    api.index_status(reset=True)
    f_log(); f_sel()
    log_ms = cuda_time(f_log, steps)
    sel_ms = cuda_time(f_sel, steps)
    step_ms = cuda_time(lambda: (f_log(), f_sel()), steps)
    if api.index_status()[0] != 0:
        raise SystemExit("device-side wait expired")
    # causal (token, key) pairs; every pair costs Hi x 128 multiply-adds
    pairs = T * pos0 + T * (T + 1) // 2
    flop = 2.0 * pairs * index_heads * 128
    ach = flop / (log_ms * 1e-3) / 1e12
    sel_gbs = (pairs * 4 + T * k * 4) / (sel_ms * 1e-3) / 1e9
    # spot check of the selection on a few rows: count, range and threshold property on the kernel's logits
    rows = [0, T // 2, T - 1]
    lg = logits[rows].cpu()
    sl = sel[rows].cpu()
    ok = True
    for i, r in enumerate(rows):
        n = pos0 + r + 1
        live = sl[i][sl[i] >= 0].long()
        ok &= int(live.numel()) == min(k, n) and int(live.unique().numel()) == int(live.numel())
        if n > k and live.numel():
            rest = torch.ones(n, dtype=torch.bool)
            rest[live] = False
            ok &= bool(lg[i, :n][rest].max() <= lg[i, live].min())
    rec = {"workload": f"{w.name} shape: {T} query tokens x {S} keys, {index_heads} index heads of dim 128 (e4m3), "
                       f"top-k {k}", "route": "index_logits_fp8 -> topk_select -> topk_idx",
           "ms_per_step": step_ms, "value": T / (step_ms * 1e-3), "unit": "tokens/s",
           "logits_ms": log_ms, "logits_tflops": ach, "logits_frac": ach / fp8_peak, "logits_peak": fp8_peak,
           "select_ms": sel_ms, "select_gbs": sel_gbs, "select_frac": sel_gbs / hbm_gbs, "select_peak_gbs": hbm_gbs,
           "selection_checked": bool(ok), "dtype": "e4m3"}
    del q8, k8, wts, ks, logits, sel
    torch.cuda.empty_cache()
    return rec


def deepgemm_index_logits(w, dev, steps, index_heads=64):
    """DeepGEMM's FP8 MQA-logits kernel (the production kernel of the same operator, as shipped
    inside the vLLM package of this image; library code, JIT-compiled on first use) on the
    indexer record's operands: its time, and its agreement with the library's kernel."""
    try:
        import vllm.third_party.deep_gemm as dg
        fn = dg.fp8_fp4_mqa_logits
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"DeepGEMM not importable ({type(e).__name__})"}
    from litetopk_b200 import api
    T, S = w.tokens, w.s_kv
    pos0 = S - T
    q8, k8, wts, ks = synth.make_indexer_operands(T, S, index_heads, seed=1, device=dev)
    start = torch.zeros((T,), dtype=torch.int32, device=dev)
    end = (pos0 + torch.arange(T, device=dev) + 1).to(torch.int32)
    qf, kf = q8.view(torch.float8_e4m3fn), k8.view(torch.float8_e4m3fn)
    call = lambda: fn((qf, None), (kf, ks), wts, start, end, clean_logits=True)  # noqa: E731
    try:
        ref = call()
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"DeepGEMM kernel could not be built or run ({type(e).__name__})"}
    ms = cuda_time(call, steps)
    mine = api.index_logits_fp8(q8, k8, wts, ks, pos0)
    fin = torch.isfinite(mine)
    same_mask = bool(torch.equal(fin, torch.isfinite(ref[:, :S])))
    diff = float((mine[fin] - ref[:, :S][fin]).abs().max()) if same_mask else None
    rec = {"kernel": "DeepGEMM fp8_fp4_mqa_logits (vllm.third_party.deep_gemm)", "ms": ms,
           "same_mask": same_mask, "max_abs_diff": diff, "max_abs_logit": float(mine[fin].abs().max())}
    del q8, k8, wts, ks, ref, mine
    torch.cuda.empty_cache()
    return rec


def vllm_topk_per_row(w, dev, steps, index_heads=64):
    """vLLM's top_k_per_row_prefill (the selection its DeepSeek-V3.2 indexer uses; library code,
    precompiled in the package of this image) on the indexer record's logits: its time and its
    agreement with the library's topk_select."""
    try:
        from vllm import _custom_ops as ops
        fn = ops.top_k_per_row_prefill
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"vLLM custom ops not importable ({type(e).__name__})"}
    from litetopk_b200 import api
    T, S, k = w.tokens, w.s_kv, w.topk
    pos0 = S - T
    q8, k8, wts, ks = synth.make_indexer_operands(T, S, index_heads, seed=1, device=dev)
    logits = api.index_logits_fp8(q8, k8, wts, ks, pos0)
    del q8, k8, wts, ks
    start = torch.zeros((T,), dtype=torch.int32, device=dev)
    end = (pos0 + torch.arange(T, device=dev) + 1).to(torch.int32)
    ref = torch.full((T, k), -1, dtype=torch.int32, device=dev)
    call = lambda: fn(logits, start, end, ref, T, logits.stride(0), logits.stride(1), k)  # noqa: E731
    try:
        call()
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"vLLM top_k_per_row_prefill could not run ({type(e).__name__})"}
    ms = cuda_time(call, steps)
    mine = api.topk_select(logits, k, q_pos0=pos0)
    vg = torch.sort(torch.gather(logits, 1, mine.clamp_min(0).long()), dim=1).values
    vr = torch.sort(torch.gather(logits, 1, ref.clamp_min(0).long()), dim=1).values
    rows_diff = int((torch.sort(mine, dim=1).values != torch.sort(ref, dim=1).values).any(dim=1).sum())
    rec = {"kernel": "vLLM top_k_per_row_prefill", "ms": ms, "same_selected_values": bool(torch.equal(vg, vr)),
           "rows_with_other_positions": rows_diff,
           "note": "rows differ only where the k-th value is tied (the values selected are the same)"}
    del logits, ref, mine, vg, vr
    torch.cuda.empty_cache()
    return rec


def stock_sparse_mla(w, dev, steps):
    """The stock per-token sparse MLA prefill (FlashMLA's sparse_prefill_fwd as shipped inside the
    vLLM package of this image; library code, bf16, no union / grouping) on a configuration's
    operands: the attention the reference's method replaces.  It takes 64 or 128 query heads, so
    configurations with fewer heads are padded with zero heads the way a tensor-parallel caller
    of the stock kernel pads them.  Also compares its output with the library's path."""
    try:
        from vllm.third_party.flashmla.flash_mla_interface import flash_mla_sparse_fwd
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"FlashMLA not importable ({type(e).__name__})"}
    from litetopk_b200 import api
    idx = synth.make_topk(w, seed=1, device=dev)
    kv = synth.make_kv_cache(w.s_kv, seed=1, device=dev, mode="refcompat")
    q = synth.make_q(w.tokens, w.heads, seed=1, device=dev, mode="refcompat")
    q8, kv8, qs, ks = synth.refcompat_operands(q, kv)
    del q, kv
    kv_bf16 = (kv8.view(torch.float8_e4m3fn).float() * ks).to(torch.bfloat16).view(w.s_kv, 1, 576)
    heads_run = max(64, w.heads)
    q_bf16 = torch.zeros((w.tokens, heads_run, 576), dtype=torch.bfloat16, device=dev)
    q_bf16[:, :w.heads] = (q8.view(torch.float8_e4m3fn).float() * qs).to(torch.bfloat16).view(w.tokens, w.heads, 576)
    ind = idx.view(w.tokens, 1, w.topk).contiguous()
    call = lambda: flash_mla_sparse_fwd(q_bf16, kv_bf16, ind, float(synth.SM_SCALE))  # noqa: E731
    try:
        o_ref, _, lse_ref = call()
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"FlashMLA sparse prefill could not run ({type(e).__name__}: {str(e)[:80]})"}
    ms = cuda_time(call, steps)
    q8v = q8.view(w.tokens, w.heads, 576)
    ours = lambda: api.sparse_prefill(q8v, kv8, idx, synth.SM_SCALE, kv_scale=ks, q_scale=qs, seq_space=w.s_kv)  # noqa: E731
    out, lse = ours()
    ours_ms = cuda_time(ours, steps)
    a, b = out.float().flatten(), o_ref[:, :w.heads].float().flatten()
    rec = {"kernel": "FlashMLA sparse_prefill_fwd (vllm.third_party.flashmla), bf16, per-token lists",
           "heads_run": heads_run, "ms": ms, "ours_ms": ours_ms, "ratio": ms / ours_ms,
           "out_cosine": float(torch.nn.functional.cosine_similarity(a, b, dim=0)),
           "out_max_abs_diff": float((a - b).abs().max()),
           "lse_max_abs_diff": float((lse - lse_ref[:, :w.heads]).abs().max()),
           "note": "ours = union_qm + masked_mla_fp8 (e4m3 P): cosine ~0.9998 against a bf16 kernel is its quantisation"}
    del idx, q8, kv8, kv_bf16, q_bf16, ind, o_ref, lse_ref, out, lse
    torch.cuda.empty_cache()
    return rec


def merge_record(api, dev, steps, hbm_gbs, part_tiles=8192, div=2):
    """The lse merge of KV-split outputs (HBM-bound): `part_tiles` slices of 128 rows merged `div` to one."""
    o = torch.randn((part_tiles, 128, 512), device=dev).to(torch.bfloat16)
    lsep = torch.randn((part_tiles, 128), device=dev)
    out = torch.empty((part_tiles // div, 128, 512), dtype=torch.bfloat16, device=dev)
    lse = torch.empty((part_tiles // div, 128), dtype=torch.float32, device=dev)
    ms = cuda_time(lambda: api.merge_kv_splits(o, lsep, div, out=out, lse=lse), steps)
    nbytes = o.numel() * 2 + lsep.numel() * 4 + out.numel() * 2 + lse.numel() * 4
    gbs = nbytes / (ms * 1e-3) / 1e9
    del o, lsep, out, lse
    return {"workload": f"{part_tiles} part tiles, q_group_div {div}", "ms": ms, "gbs": gbs,
            "frac": gbs / hbm_gbs, "peak_gbs": hbm_gbs, "bytes": nbytes}


def host_copy_bandwidth(dev, mb=256):
    """Plain pinned-memory copy rates of this rank (GB/s): the bound of the end-to-end leg."""
    n = mb << 20
    h = torch.empty((n,), dtype=torch.uint8).pin_memory()
    d = torch.empty((n,), dtype=torch.uint8, device=dev)
    h2d = cuda_time(lambda: d.copy_(h, non_blocking=True), 4, warmup=1)
    d2h = cuda_time(lambda: h.copy_(d, non_blocking=True), 4, warmup=1)
    return {"h2d_gbs": n / (h2d * 1e-3) / 1e9, "d2h_gbs": n / (d2h * 1e-3) / 1e9, "mbytes": mb}


# ------------------------------------------------------------------------------------ sharded runs
def slot_checksums(t: torch.Tensor) -> torch.Tensor:
    """Two position-sensitive 64-bit checksums of a bf16 tensor's bits."""
    v = t.reshape(-1).view(torch.int16)
    s0 = torch.zeros((), dtype=torch.int64, device=t.device)
    s1 = torch.zeros((), dtype=torch.int64, device=t.device)
    step = 1 << 26
    for a in range(0, v.numel(), step):
        c = v[a:a + step].to(torch.int64)
        pos = (torch.arange(a, a + c.numel(), device=t.device, dtype=torch.int64) % 65521) + 1
        s0 += c.sum()
        s1 += (c * pos).sum()
    return torch.stack([s0, s1])


class ShardedRun:
    """One rank's share of a workload: union + attention with the outputs all-gathered."""

    def __init__(self, api, dist, w, world, rank, dev, gather, n_chunks=4):
        from litetopk_b200 import dist as ldist
        self.api, self.dist, self.ldist, self.w, self.world, self.rank, self.dev = api, dist, ldist, w, world, rank, dev
        seed = 1 + rank
        self.idx = synth.make_topk(w, seed=seed, device=dev)
        kv656 = synth.make_kv_cache(w.s_kv, seed=1, device=dev, mode="refcompat")
        q = synth.make_q(w.tokens, w.heads, seed=seed, device=dev, mode="refcompat")
        self.ks = self.qs = synth.REFCOMPAT_SCALE
        self.kv8 = api.repack_kv656(kv656, self.ks)
        self.q8 = api.quantize_e4m3(q, self.qs).view(w.tiles, 128, 576)
        self.q_bf16 = q
        G, ng, cap = w.group, w.tiles, w.cap
        self.u = torch.empty((ng, cap), dtype=torch.int32, device=dev)
        self.cnt = torch.empty((ng,), dtype=torch.int32, device=dev)
        self.msk = torch.empty((ng, G, cap // 32), dtype=torch.int32, device=dev)
        self.out = torch.empty((ng, 128, 512), dtype=torch.bfloat16, device=dev) if world == 1 else None
        self.lse = torch.empty((ng, 128), dtype=torch.float32, device=dev)
        self.sm = synth.SM_SCALE * self.qs * self.ks
        self.n_chunks = n_chunks if world > 1 else 1
        self.gather = gather
        self.gatherer = None
        self.peer_out = None
        self.kind = "none"
        if world > 1:
            if gather in ("fused", "ce"):
                try:   # the kernel's epilogue writes every rank's copy through peer-mapped memory
                    self.peer_out = ldist.PeerGatheredOutput(ng, (128, 512), torch.bfloat16, dev)
                    self.kind = ("fused: TMA tile stores of the attention epilogue into every rank's buffer "
                                 "(symmetric memory) + barrier" if gather == "fused" else
                                 "ce: chunked copy-engine pushes into every rank's buffer (symmetric memory) "
                                 "on side streams + barrier")
                except Exception as e:  # noqa: BLE001  symmetric memory not available on this box
                    self.kind = f"nccl (symmetric memory unavailable: {type(e).__name__})"
            flags = torch.tensor([1 if self.peer_out is not None else 0], dtype=torch.int32, device=dev)
            dist.all_reduce(flags, op=dist.ReduceOp.MIN)
            if int(flags.item()) == 0:
                self.peer_out = None
                if self.kind.startswith(("fused", "ce")):
                    self.kind = "nccl (symmetric memory unavailable on a peer)"
            if self.peer_out is None:
                if gather == "nccl":
                    self.kind = "nccl: chunked all_gather_into_tensor on a side stream"
                self.gatherer = ldist.ChunkedAllGather(ng, (128, 512), torch.bfloat16, dev, n_chunks=self.n_chunks)
        self.launches = 0
        self.attn_events = []
        self.timed = False
        self.gather_on = True

    def attn_chunk(self, a, b, dst, peers=None):
        if self.timed:
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
        self.api.masked_mla_fp8_out(self.q8[a:b], self.kv8, self.u[a:b], self.sm, self.ks, self.cnt[a:b],
                                    self.msk[a:b], self.w.heads, dst, None, self.lse[a:b], peer_outs=peers)
        self.launches += 1
        if self.timed:
            e1.record(); self.attn_events.append((e0, e1))

    def step(self, timed=False):
        self.timed = timed
        ld, ng = self.ldist, self.w.tiles
        self.api.union_qm_out(self.idx, self.u, self.cnt, self.msk, None, None, 1, self.w.s_kv)
        self.launches += 1
        po = self.peer_out
        if po is not None and self.gather_on and self.gather == "ce":
            ld.copy_engine_sharded_attention(self.attn_chunk, po, self.n_chunks)
        elif po is not None and self.gather == "ce":
            cb = ld.chunk_bounds(ng, self.n_chunks)
            for i in range(self.n_chunks):
                self.attn_chunk(cb[i], cb[i + 1], po.local()[cb[i]:cb[i + 1]])
        elif po is not None and self.gather_on:
            ld.fused_sharded_attention(lambda dst, peers: self.attn_chunk(0, ng, dst, peers), po)
        elif po is not None:
            self.attn_chunk(0, ng, po.local())
        elif self.world > 1 and self.gather_on:
            ld.sharded_attention(self.attn_chunk, self.gatherer)
        elif self.world > 1:
            for i in range(self.gatherer.n_chunks):
                self.attn_chunk(self.gatherer.bounds[i], self.gatherer.bounds[i + 1], self.gatherer.local(i))
        else:
            self.attn_chunk(0, ng, self.out)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def measure(self, steps, warmup, clock_gpu=None):
        api, dist, world, dev = self.api, self.dist, self.world, self.dev
        api.attn_status(reset=True)
        for _ in range(warmup):
            self.step()
        self.barrier()
        self.launches = 0
        ev0 = torch.cuda.Event(enable_timing=True); ev1 = torch.cuda.Event(enable_timing=True)
        clk = ClockSampler(clock_gpu) if clock_gpu is not None else None
        if clk:
            clk.__enter__()
        self.barrier()
        ev0.record()
        for _ in range(steps):
            self.step(timed=True)
        ev1.record()
        self.barrier()
        if clk:
            clk.__exit__()
        ms = ev0.elapsed_time(ev1) / steps
        st = api.attn_status()
        if st[0] != 0:
            raise SystemExit(f"device-side wait expired: status {st}")
        attn_ms = sum(e0.elapsed_time(e1) for e0, e1 in self.attn_events) / steps   # all chunks of a step
        self.attn_events = []
        if world > 1:
            t = torch.tensor([ms, attn_ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms, attn_ms = float(t[0]), float(t[1])
        res = {"ms": ms, "attn_ms": attn_ms, "launches_per_step": self.launches // steps,
               "clocks": clk.summary() if clk else None, "compute_only_ms": None, "gather_verified": None}
        fused = self.peer_out is not None and self.gather == "fused"
        res["kernel_ms_per_launch"] = attn_ms / (1 if fused else self.n_chunks)
        if world > 1:
            res["gather_verified"] = self.verify_gather()
            # the same steps without the collective: what the all-gather costs
            self.gather_on = False
            self.barrier()
            c0 = torch.cuda.Event(enable_timing=True); c1 = torch.cuda.Event(enable_timing=True)
            c0.record()
            for _ in range(steps):
                self.step()
            c1.record()
            self.barrier()
            t = torch.tensor([c0.elapsed_time(c1) / steps], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res["compute_only_ms"] = float(t[0])
            self.gather_on = True
        return res

    def slot(self, r):
        """Rank r's rows as held in THIS rank's gathered buffers (list of tensors, chunk order)."""
        if self.peer_out is not None:
            return [self.peer_out.gathered()[r]]
        return [b[r] for b in self.gatherer.bufs]

    def verify_gather(self) -> bool:
        """After a gathered step: every rank's copy of every slot carries the checksums the
        owning rank computed over what its own kernel wrote."""
        dist, world, dev = self.dist, self.world, self.dev
        self.barrier()
        mine = torch.stack([slot_checksums(t) for t in self.slot(self.rank)]).sum(dim=0)
        allc = torch.empty((world, 2), dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(allc, mine.view(1, 2))
        ok = True
        for r in range(world):
            got = torch.stack([slot_checksums(t) for t in self.slot(r)]).sum(dim=0)
            ok = ok and bool(torch.equal(got, allc[r]))
        nonzero = bool((allc != 0).any(dim=1).all())          # nobody gathered an untouched buffer
        flag = torch.tensor([1 if (ok and nonzero) else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return bool(int(flag.item()))

    def free(self):
        for k in ("idx", "kv8", "q8", "q_bf16", "u", "cnt", "msk", "out", "lse", "gatherer", "peer_out"):
            setattr(self, k, None)
        torch.cuda.empty_cache()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="c1")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-tiles", type=int, default=32)
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--gather", choices=("auto", "fused", "ce", "nccl"), default="auto",
                    help="N > 1: how the ranks' outputs are gathered (auto: the fastest measured "
                         "form: the attention epilogue's peer stores at every N up to 8)")
    ap.add_argument("--scaling", choices=("weak", "strong"), default="weak",
                    help="N > 1: the configuration per GPU (weak) or split across the GPUs (strong)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="headline only: skip the secondary records (configs, native, c4_strong, ref_module)")
    ap.add_argument("--tokens", type=int, default=0,
                    help="shrink the workload to this many query tokens per GPU (profiling aid; "
                         "the default, the full configuration, is the only benchmark number)")
    ap.add_argument("--only-indexer", action="store_true",
                    help="run only the indexer + top-k leg on the chosen config's shape (profiling aid)")
    ap.add_argument("--only-native", action="store_true",
                    help="run only the native-cache (bf16 route) record of the workload and print it "
                         "(profiling aid for masked_mla_bf16_kernel)")
    ap.add_argument("--measure-fp8-peak", action="store_true",
                    help="print the tcgen05 dense rates measured by the library's probe and exit")
    ap.add_argument("--ref-module-worker", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    w = synth.CONFIGS[args.config]
    if args.tokens:
        w = synth.scaled(w, tokens=args.tokens)
    if args.ref_module_worker:
        return ref_module_worker(args, w)
    if args.impl == "reference":
        return run_reference(args, w)

    from litetopk_b200 import api
    if args.measure_fp8_peak:
        torch.cuda.set_device(0)
        print(json.dumps({"tcgen05_dense_tflops": fp8_peaks(api), "bf16_cublas": load_peaks()}), flush=True)
        return
    if args.only_native:
        torch.cuda.set_device(0)
        print(json.dumps(native_record(api, w, torch.device("cuda", 0), args.steps, load_peaks()["bf16_tflops"])),
              flush=True)
        return
    if args.only_indexer:
        torch.cuda.set_device(0)
        pk = load_peaks()
        print(json.dumps(indexer_record(api, w, torch.device("cuda", 0), args.steps, 2 * pk["bf16_tflops"],
                                        pk["hbm_gbs"])), flush=True)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    peaks = load_peaks()

    if w.kind == "dsv4":        # --config c3: the DSv4 kernel as the headline of its own line
        probe = fp8_peaks(api)
        rec = dsv4_config_record(api, w, dev, args.steps, peaks["bf16_tflops"], with_ref=not args.no_extras)
        line = {"metric": METRIC, "value": rec["value"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": rec["ms_per_step"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": config_dict(w, args), "effective_tflops": rec["effective_tflops"],
                "roofline": {"kernel": "dsv4_kernel", "bound": "tensor", "achieved": rec["effective_tflops"],
                             "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": rec["frac"], "traffic": None,
                             "peak_source": f"bf16 dense (cuBLAS) of {peaks['source']}", "tcgen05_probe": probe},
                "record": rec, "gpu_launches": args.steps, "cpu_baseline": None, "e2e": None}
        print(json.dumps(line), flush=True)
        return

    if args.gather == "auto":
        args.gather = "fused" if world <= 8 else "nccl"
    if args.scaling == "strong" and world > 1:
        if w.tokens % (world * w.group):
            raise SystemExit("strong scaling needs tokens divisible by gpus x tokens-per-tile")
        w = synth.scaled(w, tokens=w.tokens // world)
    dist = None
    if world > 1:
        import torch.distributed as dist_
        dist = dist_
        dist.init_process_group("nccl", device_id=dev)

    # ---- tensor-core rates of this GPU, measured by the library's own probe
    probe = fp8_peaks(api)
    fp8_measured = probe.get("fp8_m256")
    fp8_2x = 2.0 * peaks["bf16_tflops"]
    fp8_peak = fp8_measured if fp8_measured else fp8_2x

    # ---- headline: this rank's chunk, union + attention (+ the all-gather at N > 1)
    run = ShardedRun(api, dist, w, world, rank, dev, args.gather)
    res = run.measure(args.steps, args.warmup, clock_gpu=local)
    ms, attn_ms = res["ms"], res["attn_ms"]

    # ---- end to end through the public API with host buffers (rank-local), copies inside the timing
    # headline form: bf16 queries uploaded and quantised on the device inside the timed region;
    # beside it the reference operator's own input dtype (e4m3 codes prepared by the caller)
    ks, qs = run.ks, run.qs
    kv8_e2e = run.kv8
    idx_host = run.idx.cpu().pin_memory()
    out_host = torch.empty((w.tokens, w.heads, 512), dtype=torch.bfloat16).pin_memory()
    lse_host = torch.empty((w.tokens, w.heads), dtype=torch.float32).pin_memory()
    q_hosts = {"bf16": run.q_bf16.cpu().pin_memory(),
               "e4m3": run.q8.view(w.tokens, w.heads, 576).cpu().pin_memory()}
    e2e_windows = {"bf16": [], "e4m3": []}

    def e2e_window():
        """One window: the median step time of each form (max over ranks)."""
        for name in ("bf16", "e4m3"):
            q_host = q_hosts[name]

            def e2e_step():
                # chunks of 512 tokens: upload, kernels and download of neighbouring chunks overlap
                api.sparse_prefill_host(q_host, kv8_e2e, idx_host, synth.SM_SCALE, out_host=out_host,
                                        lse_host=lse_host, kv_scale=ks, q_scale=qs, seq_space=w.s_kv)
            if world > 1:
                dist.barrier()
            e2e_ms = median(cuda_time_steps(e2e_step, args.e2e_steps))
            if world > 1:
                t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                e2e_ms = float(t[0])
            e2e_windows[name].append(e2e_ms)

    e2e_window()
    copy_bw = host_copy_bandwidth(dev)
    if world > 1:
        t = torch.tensor([copy_bw["h2d_gbs"], copy_bw["d2h_gbs"]], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        copy_bw = {"h2d_gbs": float(t[0]), "d2h_gbs": float(t[1]), "mbytes": copy_bw["mbytes"],
                   "note": "slowest rank, copies of all ranks not concurrent"}
        e2e_window()          # N > 1: the second window follows at once (every rank takes part)

    def e2e_record():
        recs = {}
        for name in ("bf16", "e4m3"):
            ms_e = min(e2e_windows[name])
            q_host = q_hosts[name]
            recs[name] = {"value": world * w.tokens / (ms_e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e,
                          "windows_ms": list(e2e_windows[name]),
                          "h2d_bytes_per_step": q_host.numel() * q_host.element_size() + idx_host.numel() * 4,
                          "d2h_bytes_per_step": out_host.numel() * 2 + lse_host.numel() * 4, "host_q_dtype": name}
        head = dict(recs["bf16"])
        head["e4m3_q"] = recs["e4m3"]
        head["host_copy_bandwidth"] = copy_bw
        head["method"] = E2E_METHOD
        return head

    # ---- work model: 2176 FLOP per attended (query-head, key) pair; gather bytes per union row
    pairs = int((run.idx >= 0).sum().item()) * w.heads
    union_rows = int(run.cnt.sum().item())
    flop = pairs * synth.FLOP_PER_PAIR
    achieved = flop / (attn_ms * 1e-3) / 1e12
    ng = w.tiles
    gather_bytes = (world - 1) * ng * 128 * 512 * 2
    gather_kind = run.kind
    run.free()

    line = {
        "metric": METRIC, "value": world * w.tokens / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "e4m3",
        "data": "synthetic", "config": config_dict(w, args),
        "effective_tflops": world * flop / (ms * 1e-3) / 1e12,
        "compute_only": None if res["compute_only_ms"] is None else {
            "ms_per_step": res["compute_only_ms"], "value": world * w.tokens / (res["compute_only_ms"] * 1e-3),
            "note": "same steps with the all-gather of the outputs switched off"},
        "gather": gather_kind, "gather_verified": res["gather_verified"],
        "all_gather_bytes_per_rank_per_step": gather_bytes,
        "all_gather_ingress_gbs_per_rank": None if world == 1 else gather_bytes / (ms * 1e-3) / 1e9,
        "roofline": {"kernel": "masked_mla_fp8_kernel", "bound": "tensor", "achieved": achieved,
                     "peak": fp8_peak, "unit": "TFLOP/s", "frac": achieved / fp8_peak,
                     "traffic": ATTN_DRAM_TRAFFIC_BYTES if (w.name == "c1" and not args.tokens) else None,
                     "peak_source": ("FP8 dense rate measured on this GPU by the library's tcgen05 probe "
                                     "(kind::f8f6f4, cta_group::2, M 256 x N 256, operands in shared memory)"
                                     if fp8_measured else
                                     f"2 x bf16 dense {peaks['bf16_tflops']} TFLOP/s of {peaks['source']} (probe failed)"),
                     "peak_fp8_measured": fp8_measured, "peak_2x_bf16_cublas": fp8_2x, "peak_nominal": 4500.0,
                     "frac_of_2x_bf16": achieved / fp8_2x, "tcgen05_probe": probe,
                     "kernel_ms_per_launch": res["kernel_ms_per_launch"],
                     "algorithmic_flop_per_step": flop,
                     "executed_flop_per_step": union_rows * 128 * synth.FLOP_PER_PAIR,
                     "gather_bytes_per_step": union_rows * 576,
                     "gather_gbs": union_rows * 576 / (attn_ms * 1e-3) / 1e9},
        "e2e": None,
        "gpu_launches": res["launches_per_step"] * args.steps,
        "gpu_launches_per_step": res["launches_per_step"],
        "clocks": res["clocks"], "cpu_baseline": None,
    }

    extras = not args.no_extras and not args.tokens and args.config == "c1" and args.scaling == "weak"
    sec_steps = max(3, min(args.steps, 10))
    if extras and world == 1:
        # the reference's module on the headline's operands, then the other configurations
        ref = ref_module_leg(w.name, 0, args.steps)
        if "unavailable" not in ref:
            union_us = (ms - attn_ms) * 1e3
            ref["ratio_attn"] = ref["attn_ms"] / attn_ms
            ref["ratio_union"] = ref["union_us"] / union_us if union_us > 0 else None
            ref["ratio_path"] = ref["ms_per_step"] / ms
        line["ref_module"] = ref
        cfgs = {}
        cfgs["c2"] = fp8_config_record(api, synth.CONFIGS["c2"], dev, sec_steps, fp8_peak, True)
        cfgs["c3"] = dsv4_config_record(api, synth.CONFIGS["c3"], dev, sec_steps, peaks["bf16_tflops"], True)
        cfgs["c4"] = fp8_config_record(api, synth.CONFIGS["c4"], dev, sec_steps, fp8_peak, True)
        line["configs"] = cfgs
        line["c4_strong"] = {"n_gpus": 1, "ms_per_step": cfgs["c4"]["ms_per_step"], "value": cfgs["c4"]["value"],
                             "compute_only_ms": cfgs["c4"]["ms_per_step"], "gather": "none",
                             "note": "config 4 on one GPU: the base of the strong-scaling curve"}
        line["native"] = native_record(api, synth.CONFIGS["c1"], dev, sec_steps, peaks["bf16_tflops"])
        line["indexer"] = indexer_record(api, synth.CONFIGS["c1"], dev, sec_steps, fp8_peak, peaks["hbm_gbs"])
        line["merge_kv_splits"] = merge_record(api, dev, sec_steps, peaks["hbm_gbs"])
    elif extras:
        # config 4 split over the ranks (strong scaling) with the all-gather of its outputs
        w4 = synth.CONFIGS["c4"]
        if w4.tokens % (world * w4.group) == 0:
            w4r = synth.scaled(w4, tokens=w4.tokens // world)
            run4 = ShardedRun(api, dist, w4r, world, rank, dev, args.gather)
            r4 = run4.measure(sec_steps, 3)
            gb = (world - 1) * w4r.tiles * 128 * 512 * 2
            line["c4_strong"] = {"n_gpus": world, "tokens_total": w4.tokens, "ms_per_step": r4["ms"],
                                 "value": w4.tokens / (r4["ms"] * 1e-3), "compute_only_ms": r4["compute_only_ms"],
                                 "gather": run4.kind, "gather_verified": r4["gather_verified"],
                                 "all_gather_bytes_per_rank_per_step": gb,
                                 "all_gather_ingress_gbs_per_rank": gb / (r4["ms"] * 1e-3) / 1e9,
                                 "note": "speed-up = the N = 1 line's c4_strong.ms_per_step / this one"}
            run4.free()
    if world == 1:
        e2e_window()          # the second window, after everything else this run measures
        if "indexer" in line:
            # last, so that importing the other package cannot disturb any figure above
            dgr = deepgemm_index_logits(synth.CONFIGS["c1"], dev, sec_steps)
            if "ms" in dgr:
                dgr["ratio"] = dgr["ms"] / line["indexer"]["logits_ms"]
            line["indexer"]["deepgemm"] = dgr
            vtr = vllm_topk_per_row(synth.CONFIGS["c1"], dev, sec_steps)
            if "ms" in vtr:
                vtr["ratio"] = vtr["ms"] / line["indexer"]["select_ms"]
            line["indexer"]["vllm_topk"] = vtr
        if extras:
            line["stock_sparse_mla"] = {c: stock_sparse_mla(synth.CONFIGS[c], dev, sec_steps) for c in ("c1", "c2", "c4")}
    line["e2e"] = e2e_record()
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_record(w, args.cpu_tiles)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
