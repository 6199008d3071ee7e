#!/usr/bin/env python
"""Benchmark of the TriAttention runtime KV-compression hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c1|c0|...]

A step = one score -> select -> compact pass over the whole synthetic paged cache of the chosen
configuration (default: the Qwen3-8B-shaped cache, 36 layers, 8 requests x 32768 tokens, budget 2048,
window 128).  Prints ONE JSON line (rank 0).  Under torchrun each rank owns Hkv/N KV heads of N times
as many requests (tensor-parallel sharding by KV head, no collective, per-GPU work fixed).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))
sys.path.insert(1, str(REPO / "tests"))  # synth.py: the seeded workload generator shared with the tests

CONFIGS = {
    # name: layers, q heads, kv heads, head_dim, theta, batch, tokens, budget, window
    "c0": dict(L=1, Hq=32, Hkv=8, D=128, theta=1e6, B=1, T=4096, budget=2048, window=128),
    "c1": dict(L=36, Hq=32, Hkv=8, D=128, theta=1e6, B=8, T=32768, budget=2048, window=128),
    "c2": dict(L=64, Hq=64, Hkv=8, D=128, theta=1e6, B=16, T=32768, budget=2048, window=128),
    "c3s": dict(L=32, Hq=32, Hkv=8, D=128, theta=5e5, B=64, T=2176, budget=2048, window=128,
                llama3=dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                            original_max_position_embeddings=8192)),
}
BLOCK_SIZE = 16
METRIC = "cached keys scored+pruned/sec per GPU & KV HBM GB/s vs peak, at 1/2/4/8 B200"
UNIT = "keys/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c1", choices=sorted(CONFIGS))
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (smaller captures)")
    ap.add_argument("--batch", type=int, default=0, help="override the request count")
    ap.add_argument("--tokens", type=int, default=0, help="override the cached length")
    ap.add_argument("--budget", type=int, default=0, help="override the KV budget")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--aggregation", choices=("mean", "max"), default="mean",
                    help="aggregation over the future-offset set (the reference's default is mean)")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="on ONE GPU, run the shard one rank owns under tensor parallelism of this degree "
                         "(the path has no collective, so this is that rank's whole job)")
    return ap.parse_args()


def measured_peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# DRAM traffic of the score kernel per key from the ncu capture summarised in
# profiles/score_paged_mma_kernel_c1_2layers.md (dram__bytes_read + dram__bytes_write = 1.0743 GB + 64.5 MB for
# 4 194 304 keys); traffic grows in proportion to the keys scored, so a full launch is this figure x its keys.
SCORE_DRAM_BYTES_PER_KEY_NCU = (1.074343e9 + 64.52e6) / 4194304.0


def algorithmic_bytes_per_key(T: int, k: int) -> float:
    """K read once (256 B) + K and V of the kept tokens read and written (4 x 256 B x k/T)."""
    return 256.0 + 1024.0 * k / T


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def resolve_config(args, world: int):
    c = dict(CONFIGS[args.config])
    if args.layers:
        c["L"] = args.layers
    if args.batch:
        c["B"] = args.batch
    if args.tokens:
        c["T"] = args.tokens
    if getattr(args, "budget", 0):
        c["budget"] = args.budget
    if c["Hkv"] % world:
        raise SystemExit(f"--gpus {world} does not divide {c['Hkv']} KV heads")
    c["g"] = c["Hq"] // c["Hkv"]
    c["Hkv_local"] = c["Hkv"] // world
    c["B_local"] = c["B"] * world  # per-GPU key count stays fixed: weak scaling by KV-head sharding
    c["k"] = min(c["budget"], c["T"])
    return c


# ----------------------------------------------------------------------------- synthetic workload (device)
def build_device_workload(c: dict, rank: int, device: torch.device, config_idx: int):
    """Paged bf16 K/V for every layer, a random block permutation per request and synthetic statistics.

    Same distributions as triattention_b200.synth (pre-RoPE N(0,1) x per-channel log-uniform scale in
    [0.1, 10], rotated at positions 0..T-1; V ~ N(0,1)); drawn with a seeded device generator so that the
    38 GB of the full configuration are produced in seconds.
    """
    from triattention_b200 import ops
    import synth

    seed = synth.seed_for(config_idx, 0, rank)
    gen = torch.Generator(device=device).manual_seed(seed)
    cgen = torch.Generator().manual_seed(seed)
    L, B, T, H, D = c["L"], c["B_local"], c["T"], c["Hkv_local"], c["D"]
    F = D // 2
    nblk = (T + BLOCK_SIZE - 1) // BLOCK_SIZE
    nb_total = B * nblk + 16
    inv_freq = synth.rope_inv_freq(D, c["theta"], c.get("llama3"))
    full_stats = synth.make_stats(L, c["Hq"], D, inv_freq, cgen)
    # rank r owns KV heads [r*Hkv_local, ...) and the matching query-head statistics rows
    h0 = rank * c["Hkv_local"] * c["g"]
    h1 = h0 + c["Hkv_local"] * c["g"]
    offsets = torch.tensor([float(2 ** i) for i in range(17)])
    stats = ops.DeviceStats(
        full_stats.q_mean_real[:, h0:h1].contiguous().to(device), full_stats.q_mean_imag[:, h0:h1].contiguous().to(device),
        full_stats.q_abs_mean[:, h0:h1].contiguous().to(device), torch.ones((L, h1 - h0, F), device=device),
        inv_freq.to(device), offsets.to(device))
    perm = torch.randperm(nb_total - 1, generator=cgen)[: B * nblk] + 1
    block_ids = [perm[b * nblk : (b + 1) * nblk].tolist() for b in range(B)]
    perm_dev = perm.to(device)
    pos = torch.arange(nblk * BLOCK_SIZE, device=device, dtype=torch.float32)
    ang = pos.view(-1, 1) * inv_freq.to(device).view(1, F)
    cos, sin = torch.cos(ang).view(nblk, BLOCK_SIZE, 1, F), torch.sin(ang).view(nblk, BLOCK_SIZE, 1, F)
    lo, hi = torch.log(torch.tensor(0.1)).item(), torch.log(torch.tensor(10.0)).item()
    caches = []
    for _l in range(L):
        cache = torch.empty((2, nb_total, BLOCK_SIZE, H, D), dtype=torch.bfloat16, device=device)
        scale = torch.exp(lo + (hi - lo) * torch.rand((H, D), generator=gen, device=device))
        for b in range(B):
            pre = torch.randn((nblk, BLOCK_SIZE, H, D), generator=gen, device=device) * scale
            pr, pi = pre[..., :F], pre[..., F:]
            rot = torch.cat([pr * cos - pi * sin, pr * sin + pi * cos], dim=-1).to(torch.bfloat16)
            idx = perm_dev[b * nblk : (b + 1) * nblk]
            cache[0].index_copy_(0, idx, rot)
            cache[1].index_copy_(0, idx, torch.randn((nblk, BLOCK_SIZE, H, D), generator=gen, device=device).to(torch.bfloat16))
            del pre, rot
        cache[:, 0].zero_()
        caches.append(cache)
    return caches, block_ids, stats


class PrefixSaver:
    """Keeps a pristine copy of the slots compaction overwrites and puts them back between timed steps."""

    def __init__(self, caches, block_ids, k: int):
        nreq = (k + BLOCK_SIZE - 1) // BLOCK_SIZE
        ids = [i for ids in block_ids for i in ids[:nreq]]
        self.idx = torch.as_tensor(ids, dtype=torch.long, device=caches[0].device)
        self.saved = [c.index_select(1, self.idx) for c in caches]
        self.caches = caches

    def restore(self):
        for c, s in zip(self.caches, self.saved):
            c.index_copy_(1, self.idx, s)


def dist_setup(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and args.impl == "ours":
        # the reference arm runs on rank 0's host cores only: it needs no process group
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def max_over_ranks(x: float, world: int, device) -> float:
    if world <= 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ----------------------------------------------------------------------------- CPU baseline (checker port)
def cpu_baseline_run(c: dict, sample_layers: int, sample_tokens: int, repeats: int = 1):
    """Times the CPU restatement of the reference path (oracle/) on a bounded slice of the workload.

    One request, ``sample_layers`` layers, all KV heads, ``sample_tokens`` tokens: selection (score, z-norm,
    guards, group max, layer mean, top-k) plus per-head compaction of every sampled layer.
    Returns (keys_per_second, seconds, description).
    """
    import oracle
    import synth

    gen = torch.Generator().manual_seed(synth.seed_for(1, 9, 0))
    D, H, g = c["D"], c["Hkv"], c["g"]
    T = min(sample_tokens, c["T"])
    inv_freq = synth.rope_inv_freq(D, c["theta"], c.get("llama3"))
    stats = synth.make_stats(sample_layers, c["Hq"], D, inv_freq, gen)
    nblk = (T + BLOCK_SIZE - 1) // BLOCK_SIZE
    block_ids = synth.random_block_ids(nblk, nblk + 4, gen)
    caches = []
    for _l in range(sample_layers):
        cache = synth.make_paged_layer(nblk + 4, BLOCK_SIZE, H, D, kv_axis=0)
        k = synth.make_rotated_keys(H, T, D, inv_freq, gen)
        v = synth.make_values(H, T, D, gen)
        synth.write_tokens_to_paged(cache, 0, block_ids, BLOCK_SIZE, k, v)
        caches.append(cache)
    sl = {l: {"q_mean_real": stats.q_mean_real[l], "q_mean_imag": stats.q_mean_imag[l],
              "q_abs_mean": stats.q_abs_mean[l], "freq_scale_sq": torch.ones_like(stats.q_abs_mean[l])}
          for l in range(sample_layers)}
    offsets = oracle.geometric_offsets()
    kk = min(c["budget"], T)
    best = None
    for _ in range(repeats):
        work = [x.clone() for x in caches]
        layers = [(l, x, block_ids, BLOCK_SIZE) for l, x in enumerate(work)]
        t0 = time.perf_counter()
        keep = oracle.select_group_per_head(layers, sl, inv_freq, offsets, T, T, kk, window_size=c["window"], kv_axis=0)
        for x in work:
            oracle.compact_per_head(x, block_ids, BLOCK_SIZE, keep, T, preserve_dropped_tokens=True, kv_axis=0)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    keys = sample_layers * H * T
    desc = f"1 request x {sample_layers} layers x {H} KV heads x {T} tokens (g={g}), budget {kk}"
    return keys / best, best, desc


def run_reference(args, world, rank):
    """Reference arm: the CPU path of the reference (its restatement in oracle/, all host threads)."""
    if rank != 0:
        return
    c = resolve_config(args, 1)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample_layers, sample_tokens = min(2, c["L"]), min(c["T"], 32768)
    for _ in range(args.warmup):
        cpu_baseline_run(c, 1, min(2048, c["T"]))
    times, kps = [], []
    desc = ""
    for _ in range(args.steps):
        v, dt, desc = cpu_baseline_run(c, sample_layers, sample_tokens)
        times.append(dt)
        kps.append(v)
    value = statistics.mean(kps)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args, c), "sample": desc},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(args, c):
    return (f"{args.config}: {c['L']} layers, {c['Hq']}q/{c['Hkv']}kv heads, head_dim {c['D']}, "
            f"{c['B']} requests x {c['T']} tokens, paged bf16 block {BLOCK_SIZE}, budget {c['budget']}, window {c['window']}"
            + (", max over offsets" if getattr(args, "aggregation", "mean") == "max" else ""))


# ----------------------------------------------------------------------------- our arm
def run_ours(args, world, rank, local):
    from triattention_b200 import _native, engine, ops

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    _native.load()
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    shard_of = args.shard_of if (args.shard_of and world == 1) else 0
    c = resolve_config(args, shard_of or world)
    config_idx = sorted(CONFIGS).index(args.config)
    caches, block_ids, stats = build_device_workload(c, rank, device, config_idx)
    view = ops.PagedCacheView.from_layers(caches, kv_axis=0)
    B, T, k, L, H = c["B_local"], c["T"], c["k"], c["L"], c["Hkv_local"]
    saver = PrefixSaver(caches, block_ids, k)
    comp = engine.PagedCompressor(stats, window=c["window"],
                                  offset_agg=(_native.OFFSETS_MAX if args.aggregation == "max" else _native.OFFSETS_MEAN),
                                  use_cuda_graph=os.environ.get("TRIATTN_BENCH_CUDA_GRAPH") == "1")
    seq_lens, round_starts, budgets = [T] * B, [T] * B, [k] * B
    keys_per_gpu = L * B * H * T

    # device-resident metadata for the kernel-only measurement
    nblk = (T + BLOCK_SIZE - 1) // BLOCK_SIZE
    bt = torch.tensor([ids[:nblk] for ids in block_ids], dtype=torch.int32, device=device)
    d_seq = torch.tensor(seq_lens, dtype=torch.int32, device=device)
    d_rs = torch.tensor(round_starts, dtype=torch.int32, device=device)
    d_kc = torch.tensor(budgets, dtype=torch.int32, device=device)
    d_status = torch.zeros(1, dtype=torch.int32, device=device)
    layout = view.layout(B, c["g"], nblk)
    agg = _native.OFFSETS_MAX if args.aggregation == "max" else _native.OFFSETS_MEAN
    ws = torch.empty(ops.compress_workspace_bytes(layout, 17, agg, k), dtype=torch.uint8, device=device)
    keep_out = torch.empty((B, H, k), dtype=torch.int32, device=device)

    def device_step():
        ops.compress_paged(view, layout, stats, bt, d_seq, d_rs, None, d_kc, k, c["window"], offset_agg=agg,
                           workspace=ws, keep_out=keep_out, status=d_status)

    def timed(fn, steps):
        """Per-step CUDA-event time on the launching stream; the cache prefix is restored (untimed) between steps."""
        ms = []
        for _ in range(steps):
            saver.restore()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ms.append(e0.elapsed_time(e1))
        return ms

    timed(device_step, max(args.warmup, 3))
    sampler = ClockSampler(local)
    barrier(world)
    torch.cuda.synchronize()
    sampler.start()
    t_sampler = time.perf_counter()
    ms = timed(device_step, args.steps)
    torch.cuda.synchronize()
    # nvidia-smi needs a few hundred ms to deliver samples: keep the same load running (untimed) until it has
    while time.perf_counter() - t_sampler < 0.6:
        timed(device_step, 1)
    barrier(world)
    clocks = sampler.stop()
    step_ms = max_over_ranks(statistics.mean(ms), world, device)
    status_bits = int(d_status.item())

    # end to end through the public batched API: host lists -> pinned -> H2D, kernels, D2H of the status word
    import numpy as np
    host_block_ids = [np.asarray(ids, dtype=np.int32) for ids in block_ids]  # host-side block tables, as an engine keeps them

    def e2e_once():
        saver.restore()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        res = comp.compress(view, host_block_ids, seq_lens, round_starts, budgets)
        torch.cuda.synchronize()
        return time.perf_counter() - t0, res

    for _ in range(max(args.warmup, 3)):
        e2e_once()
    barrier(world)
    e2e_t, res = [], None
    for _ in range(args.steps):
        dt, res = e2e_once()
        e2e_t.append(dt)
    e2e_s = max_over_ranks(statistics.mean(e2e_t), world, device)
    barrier(world)

    # per-stage device times (same inputs) for the roofline of the dominant kernel
    stage_ms = {n: [] for n in ("prep", "score", "finalize", "select", "compact")}
    for _ in range(max(3, args.steps)):
        saver.restore()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
        torch.cuda.synchronize()
        ev[0].record()
        w = ops.prep_weights_fused(stats, d_rs, agg)
        ev[1].record()
        raw, mom = ops.score_paged(view, layout, bt, d_seq, w, agg, 17, status=d_status)
        ev[2].record()
        fin = ops.finalize_scores(layout, raw, mom, d_seq, None, c["window"])
        ev[3].record()
        keep = ops.select_topk(fin.view(-1, fin.shape[-1]), d_seq, d_kc, B, H, k, d_status)
        ev[4].record()
        ops.compact_paged(view, layout, bt, d_seq, keep, (0, H * k, k), d_kc, d_status)
        ev[5].record()
        torch.cuda.synchronize()
        for i, n in enumerate(stage_ms):
            stage_ms[n].append(ev[i].elapsed_time(ev[i + 1]))
        del w, raw, mom, fin, keep
    stage = {n: statistics.median(v) for n, v in stage_ms.items()}

    if rank != 0:
        return
    peak, peak_kind = measured_peaks()
    value = keys_per_gpu * world / (step_ms * 1e-3)
    bytes_step = keys_per_gpu * algorithmic_bytes_per_key(T, k)
    score_bytes = keys_per_gpu * 256.0
    achieved = score_bytes / (stage["score"] * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload_name(args, c), "per_gpu": f"{H} KV heads x {B} requests",
                   "sharding": (f"shard 0 of tp{shard_of} run alone on one GPU (no collective in the path)" if shard_of
                                else f"tp{world} by KV head, no collective"), "l2": "inputs larger than L2 (K alone is "
                   f"{score_bytes / 1e9:.1f} GB per step); compacted prefix restored untimed between steps"},
        "keys_per_s_per_gpu": value / world,
        "step_hbm_gbs": bytes_step / (step_ms * 1e-3) / 1e9, "step_hbm_frac": bytes_step / (step_ms * 1e-3) / 1e9 / peak,
        "stage_ms": stage,
        "roofline": {"kernel": ("score_paged_mma_max_kernel" if args.aggregation == "max" else "score_paged_mma_kernel"),
                     "bound": "hbm", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                     "traffic": (keys_per_gpu * SCORE_DRAM_BYTES_PER_KEY_NCU
                                 if (c["D"], c["g"], c["Hkv_local"]) == (128, 4, 8) else None),
                     "traffic_note": "bytes per launch, scaled by keys from a 2-layer ncu capture of the same shape"},
        "e2e": {"value": keys_per_gpu * world / e2e_s, "unit": UNIT, "h2d_bytes_per_step": res.h2d_bytes,
                "d2h_bytes_per_step": res.d2h_bytes, "ms_per_step": e2e_s * 1e3},
        "gpu_launches": 5 * args.steps,
        "clocks": clocks, "device_status": status_bits | res.device_status,
    }
    if not args.no_cpu_baseline and world == 1:
        torch.set_num_threads(os.cpu_count() or 1)
        cpu_baseline_run(c, 1, min(2048, c["T"]))
        v, dt, desc = cpu_baseline_run(c, min(2, c["L"]), min(c["T"], 32768))
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                                "sample": desc, "seconds": dt}
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    world, rank, local = dist_setup(args)
    if args.gpus != world and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    try:
        if args.impl == "reference":
            run_reference(args, world, rank)
        else:
            run_ours(args, world, rank, local)
    finally:
        if world > 1 and args.impl == "ours":
            import torch.distributed as dist
            if dist.is_initialized():
                dist.destroy_process_group()


if __name__ == "__main__":
    main()
