#!/usr/bin/env python
"""Benchmark of the TriAttention runtime KV-compression hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c1|c0|c2|c3s|c3]

A step = one score -> select -> compact pass over the whole synthetic paged cache of the chosen
configuration (default: the Qwen3-8B-shaped cache, 36 layers, 8 requests x 32768 tokens, budget 2048,
window 128).  Prints ONE JSON line (rank 0).  Under torchrun each rank owns Hkv/N KV heads of N times
as many requests (tensor-parallel sharding by KV head, no collective, per-GPU work fixed); with two or
more ranks the line also carries the Qwen3-32B-shaped shard in both selection modes (``extra.c2``).

``--config c3`` runs the decode-interleaved driver instead (64 ragged requests, one token per step,
compression whenever a request reaches budget + 128), once through the per-request hook and once through
the batched engine.  ``--sweep`` runs the length / batch / budget sweep and prints one line per point.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
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
CONFIGS["c3"] = dict(CONFIGS["c3s"])
BLOCK_SIZE = 16
METRIC = "cached keys scored+pruned/sec per GPU & KV HBM GB/s vs peak, at 1/2/4/8 B200"
UNIT = "keys/s"
SCORE_TOL = 1e-3  # |delta| / max(|ref|, sigma_row) of scores; also the tie window (in sigma_row) of keep sets


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_gpu"],
                    help="reference: the reference's CPU path on the host cores; reference_gpu (informational): the "
                         "reference's own Triton scorer and torch glue on this GPU, through its unmodified selector")
    ap.add_argument("--config", default="c1", choices=sorted(CONFIGS))
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (smaller captures)")
    ap.add_argument("--batch", type=int, default=0, help="override the request count")
    ap.add_argument("--tokens", type=int, default=0, help="override the cached length")
    ap.add_argument("--budget", type=int, default=0, help="override the KV budget")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the correctness gate against the CPU checker")
    ap.add_argument("--no-c2", action="store_true", help="with 2+ ranks: skip the Qwen3-32B-shaped legs (extra.c2)")
    ap.add_argument("--c2-layers", type=int, default=0, help="layer count of the extra.c2 legs (default: all 64)")
    ap.add_argument("--aggregation", choices=("mean", "max"), default="mean",
                    help="aggregation over the future-offset set (the reference's default is mean)")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="on ONE GPU, run the shard one rank owns under tensor parallelism of this degree "
                         "(the path has no collective, so this is that rank's whole job)")
    ap.add_argument("--workspace-mb", type=int, default=0,
                    help="cap the step's scratch (MB): the step is cut into chunks of as many layers as fit")
    ap.add_argument("--decode-steps", type=int, default=4096, help="--config c3: decode steps per request")
    ap.add_argument("--cuda-graph", action="store_true",
                    help="replay the step from a CUDA graph once a geometry repeats (engine option use_cuda_graph)")
    ap.add_argument("--sweep", action="store_true", help="length / batch / budget sweep on the Qwen3-8B shape")
    ap.add_argument("--sweep-points", default="", help="comma list of T:B:budget points (default: the built-in grid)")
    return ap.parse_args()


def measured_peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# DRAM traffic of the score kernel per key (dram__bytes_read + dram__bytes_write) from the ncu captures summarised
# under profiles/ (score_paged_mma_kernel_c1_2layers.md, score_paged_mma_kernel_c2_tp8_4layers.md,
# score_paged_umma_max_kernel_c1_2layers.md); K is read once and the raw scores are written once, so traffic grows
# in proportion to the keys scored and a full launch is this figure x its keys.
SCORE_DRAM_BYTES_PER_KEY_NCU = {
    ("mean", 4): (1.074308e9 + 65.17e6) / 4194304.0,     # 271.7 B: 256 B of K + 16 B of raw scores
    ("mean", 8): (4.299350e9 + 529.34e6) / 16777216.0,   # 287.8 B: 256 B of K + 32 B of raw scores
    ("max", 4): (1.079208e9 + 66.39e6) / 4194304.0,      # 273.1 B
}


def score_kernel_name(c: dict, aggregation: str) -> str:
    """The kernel triattn_score_paged dispatches to for this shape (csrc/api.cu score_paged_impl)."""
    if aggregation == "max":
        tcgen05 = c["D"] == 128 and BLOCK_SIZE % 16 == 0 and c["L"] <= 128
        return "score_paged_umma_max_kernel" if tcgen05 else "score_paged_mma_max_kernel"
    return "score_paged_mma_kernel"


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


def resolve_config(args, world: int, name: str | None = None):
    name = name or args.config
    c = dict(CONFIGS[name])
    if name == args.config:
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

    Same distributions as the seeded CPU generator of the tests (pre-RoPE N(0,1) x per-channel log-uniform scale
    in [0.1, 10], rotated at positions 0..T-1; V ~ N(0,1)); drawn with a seeded device generator so that the
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
        # the reference arms run on rank 0 only: they need no process group
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


# ----------------------------------------------------------------------------- CPU baseline
def _cpu_slice_inputs(c: dict, sample_layers: int, T: int):
    import synth

    gen = torch.Generator().manual_seed(synth.seed_for(1, 9, 0))
    D, H = c["D"], c["Hkv"]
    inv_freq = synth.rope_inv_freq(D, c["theta"], c.get("llama3"))
    stats = synth.make_stats(sample_layers, c["Hq"], D, inv_freq, gen)
    nblk = (T + BLOCK_SIZE - 1) // BLOCK_SIZE
    block_ids = synth.random_block_ids(nblk, nblk + 4, gen)
    caches = []
    for _l in range(sample_layers):
        cache = synth.make_paged_layer(nblk + 4, BLOCK_SIZE, H, D, kv_axis=0)
        synth.write_tokens_to_paged(cache, 0, block_ids, BLOCK_SIZE, synth.make_rotated_keys(H, T, D, inv_freq, gen),
                                    synth.make_values(H, T, D, gen))
        caches.append(cache)
    return stats, caches, block_ids, inv_freq


def cpu_baseline_run(c: dict, sample_layers: int, sample_tokens: int, repeats: int = 1):
    """Times the reference's CPU path on a bounded slice of the workload: one request, ``sample_layers`` layers,
    all KV heads, ``sample_tokens`` tokens - group selection (score, z-norm, guards, group max, layer mean, top-k)
    plus per-head compaction of every sampled layer.

    Runs the reference's own code from oracle/_ref when that copy is present (``kind: "reference"``), otherwise
    the restatement in oracle/ (``kind: "port"``).  Returns (keys_per_second, seconds, description, kind).
    """
    import oracle
    import synth
    from oracle import ref_runner

    T = min(sample_tokens, c["T"])
    H, g = c["Hkv"], c["g"]
    stats, caches, block_ids, inv_freq = _cpu_slice_inputs(c, sample_layers, T)
    kk = min(c["budget"], T)
    use_ref = ref_runner.available()
    best = None
    with tempfile.TemporaryDirectory() as td:
        if use_ref:
            sel = ref_runner.make_group_selector(ref_runner.stats_file(td, synth.save_stats_pt, stats), c["budget"], c["window"])
        else:
            sl = {l: {"q_mean_real": stats.q_mean_real[l], "q_mean_imag": stats.q_mean_imag[l],
                      "q_abs_mean": stats.q_abs_mean[l], "freq_scale_sq": torch.ones_like(stats.q_abs_mean[l])}
                  for l in range(sample_layers)}
            offsets = oracle.geometric_offsets()
        for _ in range(repeats):
            work = [x.clone() for x in caches]
            if use_ref:
                _, dt = ref_runner.select_and_compact(sel, work, block_ids, BLOCK_SIZE, T, T, kk)
            else:
                layers = [(l, x, block_ids, BLOCK_SIZE) for l, x in enumerate(work)]
                t0 = time.perf_counter()
                keep = oracle.select_group_per_head(layers, sl, inv_freq, offsets, T, T, kk, window_size=c["window"], kv_axis=0)
                for x in work:
                    oracle.compact_per_head(x, block_ids, BLOCK_SIZE, keep, T, preserve_dropped_tokens=True, kv_axis=0)
                dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
    keys = sample_layers * H * T
    desc = f"1 request x {sample_layers} layers x {H} KV heads x {T} tokens (g={g}), budget {kk}"
    return keys / best, best, desc, ("reference" if use_ref else "port")


def run_reference(args, world, rank):
    """Reference arm: the reference's CPU path on all host threads (its own code from oracle/_ref when present)."""
    if rank != 0:
        return
    name = "c3s" if args.config == "c3" else args.config
    c = resolve_config(args, 1, name)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample_layers, sample_tokens = min(2, c["L"]), min(c["T"], 32768)
    for _ in range(args.warmup):
        cpu_baseline_run(c, 1, min(2048, c["T"]))
    times, kps, desc, kind = [], [], "", "port"
    for _ in range(args.steps):
        v, dt, desc, kind = cpu_baseline_run(c, sample_layers, sample_tokens)
        times.append(dt)
        kps.append(v)
    value = statistics.mean(kps)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args, c), "sample": desc},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind, "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_reference_gpu(args, rank):
    """Informational: the reference's own GPU path (Triton scorer + torch selection and compaction, from
    oracle/_ref, unmodified) on this GPU, on the slice the CPU baseline uses: one request x two layers."""
    if rank != 0:
        return
    import synth
    from oracle import ref_runner

    if not ref_runner.available() or not torch.cuda.is_available():
        print(json.dumps({"impl": "reference_gpu", "unavailable": "needs oracle/_ref and a CUDA device"}), flush=True)
        return
    c = resolve_config(args, 1, "c3s" if args.config == "c3" else args.config)
    L2, T = min(2, c["L"]), min(c["T"], 32768)
    stats, caches, block_ids, _ = _cpu_slice_inputs(c, L2, T)
    kk = min(c["budget"], T)
    times = []
    try:
        with tempfile.TemporaryDirectory() as td:
            sel = ref_runner.make_group_selector(ref_runner.stats_file(td, synth.save_stats_pt, stats), c["budget"], c["window"], gpu=True)
            for it in range(args.warmup + args.steps):
                work = [x.cuda() for x in caches]
                _, dt = ref_runner.select_and_compact(sel, work, block_ids, BLOCK_SIZE, T, T, kk)
                if it >= args.warmup:
                    times.append(dt)
    except Exception as exc:
        print(json.dumps({"impl": "reference_gpu", "unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}), flush=True)
        return
    keys = L2 * c["Hkv"] * T
    dt = statistics.mean(times)
    print(json.dumps({"impl": "reference_gpu", "metric": METRIC, "value": keys / dt, "unit": UNIT, "n_gpus": 1,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
                      "data": "synthetic", "config": {"workload": workload_name(args, c),
                      "sample": f"1 request x {L2} layers x {c['Hkv']} KV heads x {T} tokens, budget {kk}",
                      "path": "reference Triton scorer + torch top-k + torch compaction, wall clock, device synchronised"}}),
          flush=True)


def workload_name(args, c):
    return (f"{args.config}: {c['L']} layers, {c['Hq']}q/{c['Hkv']}kv heads, head_dim {c['D']}, "
            f"{c['B']} requests x {c['T']} tokens, paged bf16 block {BLOCK_SIZE}, budget {c['budget']}, window {c['window']}"
            + (", max over offsets" if getattr(args, "aggregation", "mean") == "max" else ""))


# ----------------------------------------------------------------------------- correctness gate
def _score_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max |got - ref| / max(|ref|, sigma_row) over finite entries (rows along the last axis)."""
    finite = torch.isfinite(ref)
    if not torch.equal(torch.isfinite(got), finite):
        return float("inf")
    g, r = torch.where(finite, got, 0.0), torch.where(finite, ref, 0.0)
    n = finite.sum(dim=-1, keepdim=True).clamp_min(2)
    mean = r.sum(dim=-1, keepdim=True) / n
    sigma = torch.sqrt((torch.where(finite, (r - mean) ** 2, 0.0)).sum(dim=-1, keepdim=True) / (n - 1))
    return float(((g - r).abs() / torch.maximum(r.abs(), sigma).clamp_min(1e-6)).max())


def _keep_diffs(keep: torch.Tensor, ref_keep: torch.Tensor, ref_scores: torch.Tensor):
    """(all differing indices are near-ties, number of differing indices): a differing index must have a reference
    score within SCORE_TOL * sigma_row of the cut-off."""
    ok, n = True, 0
    for r in range(keep.shape[0]):
        a, b = set(keep[r].tolist()), set(ref_keep[r].tolist())
        if a == b:
            continue
        row = ref_scores[r]
        fin = row[torch.isfinite(row)]
        sigma = float(fin.std()) if fin.numel() > 1 else 1.0
        cut = float(row[ref_keep[r]].min())
        for i in a ^ b:
            n += 1
            if abs(float(row[i]) - cut) > SCORE_TOL * max(sigma, 1e-6):
                ok = False
    return ok, n


def parity_gate(c, caches, block_ids, stats, window, agg, saver):
    """The timed data against the CPU checker: request 0, the first two layers, on the SAME device tensors the
    timed steps ran on.  Scores within SCORE_TOL, keep sets equal except near-ties, compacted prefix bit-exact."""
    import oracle
    from triattention_b200 import _native, engine, ops

    saver.restore()
    T, k, H, g = c["T"], c["k"], c["Hkv_local"], c["g"]
    L2 = min(2, len(caches))
    nblk = (T + BLOCK_SIZE - 1) // BLOCK_SIZE
    ids0 = block_ids[0][:nblk]
    dev = caches[0].device
    idx = torch.as_tensor(ids0, dtype=torch.long, device=dev)
    host = [caches[l].index_select(1, idx).cpu() for l in range(L2)]     # request 0's blocks, in logical order
    host_ids = list(range(nblk))
    st2 = stats.select_layers(range(L2))
    sl = {l: {"q_mean_real": st2.q_mean_real[l].cpu(), "q_mean_imag": st2.q_mean_imag[l].cpu(),
              "q_abs_mean": st2.q_abs_mean[l].cpu(), "freq_scale_sq": st2.freq_scale_sq[l].cpu()} for l in range(L2)}
    t0 = time.perf_counter()
    layers = [(l, h, host_ids, BLOCK_SIZE) for l, h in enumerate(host)]
    ref_final = oracle.final_scores_group_per_head(layers, sl, st2.omega.cpu(), st2.offsets.cpu(), T, T, window_size=window,
                                                   aggregation="max" if agg == _native.OFFSETS_MAX else "mean", kv_axis=0)
    ref_keep = oracle.topk_lowest_index(ref_final, k)
    cpu_s = time.perf_counter() - t0
    # device: staged scores, then the fused step, on the benchmark's own cache tensors
    view = ops.PagedCacheView.from_layers([caches[l] for l in range(L2)], kv_axis=0)
    bt = torch.tensor([ids0], dtype=torch.int32, device=dev)
    layout = view.layout(1, g, nblk)
    meta = torch.tensor([T, T, k, 0], dtype=torch.int32, device=dev)
    w = ops.prep_weights_fused(st2, meta[1:2], agg)
    raw, mom = ops.score_paged(view, layout, bt, meta[0:1], w, agg, int(st2.offsets.numel()), status=meta[3:4])
    fin = ops.finalize_scores(layout, raw, mom, meta[0:1], None, window)
    err = _score_err(fin[0, 0, :, :T].cpu(), ref_final)
    comp = engine.PagedCompressor(st2, window=window, offset_agg=agg)
    res = comp.compress(view, [ids0], [T], [T], [k])
    keep = res.keep[0].cpu().long()
    ties_ok, ndiff = _keep_diffs(keep, ref_keep, ref_final)
    prefix_ok = True
    nkeep_blk = (k + BLOCK_SIZE - 1) // BLOCK_SIZE
    for l in range(L2):
        exp = host[l].clone()
        oracle.compact_per_head(exp, host_ids, BLOCK_SIZE, keep, T, preserve_dropped_tokens=False, kv_axis=0)
        got = caches[l].index_select(1, idx[:nkeep_blk]).cpu()
        prefix_ok = prefix_ok and torch.equal(got.view(torch.int16), exp[:, :nkeep_blk].view(torch.int16))
    status = int(meta[3].item()) | res.device_status
    saver.restore()
    ok = bool(err <= SCORE_TOL and ties_ok and prefix_ok and status == 0)
    return {"checked": True, "ok": ok, "max_score_err": err, "near_tie_diffs": ndiff, "keep_sets_ok": ties_ok,
            "compacted_prefix_bit_exact": prefix_ok, "device_status": status, "tolerance": SCORE_TOL,
            "slice": f"request 0, layers 0-{L2 - 1}, {H} KV heads x {T} tokens of the timed device data",
            "checker_seconds": cpu_s}


# ----------------------------------------------------------------------------- Qwen3-32B-shaped legs (2+ ranks)
def run_c2_legs(args, world, rank, local):
    """BASELINE config 2 under tensor parallelism: 64 layers, 64 query / 8 KV heads, 16 requests x 32768 tokens,
    sharded by KV head over the ranks (total work fixed).  Per-KV-head selection (no collective) and layer-shared
    selection (one NCCL all-reduce(MAX) of the fp32 score rows between finalize and select)."""
    import torch.distributed as dist
    from triattention_b200 import engine, ops, tp

    device = torch.device("cuda", local)
    c = dict(CONFIGS["c2"])
    if args.c2_layers:
        c["L"] = args.c2_layers
    c["g"] = c["Hq"] // c["Hkv"]
    c["Hkv_local"] = c["Hkv"] // world
    c["B_local"] = c["B"]             # strong scaling: every rank holds all requests, 8/N of the heads
    c["k"] = c["budget"]
    caches, block_ids, stats = build_device_workload(c, rank, device, sorted(CONFIGS).index("c2"))
    view = ops.PagedCacheView.from_layers(caches, kv_axis=0)
    B, T, k, L, H = c["B_local"], c["T"], c["k"], c["L"], c["Hkv_local"]
    saver = PrefixSaver(caches, block_ids, k)
    keys_per_gpu = L * B * H * T
    seq, rs, bud = [T] * B, [T] * B, [k] * B
    out = {"workload": f"c2: {L} layers, 64q/8kv heads, head_dim 128, {B} requests x {T} tokens, budget {k}; "
                       f"tp{world} by KV head ({H} local), strong scaling", "keys_per_gpu": keys_per_gpu}
    peak, _ = measured_peaks()
    steps = max(2, min(args.steps, 3))

    # ---- per-KV-head selection: no collective.  Device time of the fused call with resident metadata (as the
    # headline `value`), and the same step end to end through the batched engine (host block tables -> H2D -> ...).
    import numpy as np
    host_ids = [np.asarray(ids, dtype=np.int32) for ids in block_ids]
    nblk = (T + BLOCK_SIZE - 1) // BLOCK_SIZE
    bt = torch.tensor([ids[:nblk] for ids in block_ids], dtype=torch.int32, device=device)
    meta = torch.tensor([seq, rs, bud], dtype=torch.int32, device=device)
    st = torch.zeros(1, dtype=torch.int32, device=device)
    layout = view.layout(B, c["g"], nblk)
    ws = torch.empty(ops.compress_workspace_bytes(layout, 17, 0, k), dtype=torch.uint8, device=device)
    keep_out = torch.empty((B, H, k), dtype=torch.int32, device=device)

    def device_once():
        saver.restore()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        ops.compress_paged(view, layout, stats, bt, meta[0], meta[1], None, meta[2], k, c["window"], workspace=ws,
                           keep_out=keep_out, status=st)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    for _ in range(2):
        device_once()
    barrier(world)
    ph_ms = max_over_ranks(statistics.mean(device_once() for _ in range(steps)), world, device)
    del ws, keep_out
    comp = engine.PagedCompressor(stats, window=c["window"])

    def per_head_once():
        saver.restore()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        res = comp.compress(view, host_ids, seq, rs, bud)
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3, res

    for _ in range(2):
        per_head_once()
    barrier(world)
    ph_e2e_ms = max_over_ranks(statistics.mean(per_head_once()[0] for _ in range(steps)), world, device)
    # scorer alone, for its roofline fraction
    w = ops.prep_weights_fused(stats, meta[1])
    sc = []
    raw = mom = None
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        raw, mom = ops.score_paged(view, layout, bt, meta[0], w, status=st, raw=raw, moments=mom)
        e1.record()
        torch.cuda.synchronize()
        sc.append(e0.elapsed_time(e1))
    del raw, mom, w
    score_ms = statistics.median(sc)
    out["per_head"] = {"ms_per_step": ph_ms, "keys_per_s_per_gpu": keys_per_gpu / (ph_ms * 1e-3),
                       "keys_per_s_total": keys_per_gpu * world / (ph_ms * 1e-3), "collective": "none",
                       "e2e_ms_per_step": ph_e2e_ms, "device_status": int(st.item()),
                       "score_ms": score_ms, "score_hbm_frac": keys_per_gpu * 256.0 / (score_ms * 1e-3) / 1e9 / peak,
                       "step_hbm_frac": keys_per_gpu * algorithmic_bytes_per_key(T, k) / (ph_ms * 1e-3) / 1e9 / peak}
    del comp
    torch.cuda.empty_cache()

    # ---- layer-shared selection: the [L, B, t_pad] fp32 rows cross the ranks (peer stores, else NCCL)
    def shared_once():
        saver.restore()
        timings = {}
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        res = engine.compress_layer_shared(view, stats, host_ids, seq, rs, bud, window=c["window"], timings=timings)
        e1.record()
        torch.cuda.synchronize()
        return (e0.elapsed_time(e1), timings["allreduce_ms"](), timings["allreduce_bytes"], res, timings["exchange"],
                timings.get("multicast_bound"))

    for _ in range(2):
        shared_once()
    barrier(world)
    # median of 5: a single collective now and then takes a millisecond longer (seen with NCCL alone as well)
    runs = [shared_once() for _ in range(5)]
    sh_ms = max_over_ranks(statistics.median(r[0] for r in runs), world, device)
    ar_ms = max_over_ranks(statistics.median(r[1] for r in runs), world, device)
    keep = runs[-1][3].keep.contiguous()
    # every rank must hold the same keep sets (deterministic top-k on identical reduced rows)
    lo_t, hi_t = keep.clone(), keep.clone()
    dist.all_reduce(lo_t, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi_t, op=dist.ReduceOp.MAX)
    same = bool(torch.equal(lo_t, hi_t))
    out["layer_shared"] = {"ms_per_step": sh_ms, "keys_per_s_per_gpu": keys_per_gpu / (sh_ms * 1e-3),
                           "keys_per_s_total": keys_per_gpu * world / (sh_ms * 1e-3),
                           "collective": runs[-1][4] if runs[-1][4].startswith("peer stores") else "NCCL " + runs[-1][4],
                           "allreduce_ms": ar_ms, "allreduce_share": ar_ms / sh_ms, "allreduce_bytes": runs[-1][2],
                           "multicast_bound": runs[-1][5], "runs_ms": [round(r[0], 3) for r in runs], "runs_exchange_ms": [round(r[1], 3) for r in runs],
                           "rank_keep_sets_identical": same, "device_status": runs[-1][3].device_status}
    del caches, saver, view, runs, keep, lo_t, hi_t
    torch.cuda.empty_cache()

    # ---- small shape: the sharded runs against a single-GPU run with all heads (both modes)
    import synth
    gen = torch.Generator().manual_seed(synth.seed_for(2, 7, 0))
    Ls, Hq, Hkv, D = 2, 64, 8, 128
    lens, buds = [900, 1500], [256, 512]
    inv = synth.rope_inv_freq(D, 1e6)
    sst = synth.make_stats(Ls, Hq, D, inv, gen)
    nb = [(t + BLOCK_SIZE - 1) // BLOCK_SIZE for t in lens]
    perm = synth.random_block_ids(sum(nb), sum(nb) + 5, gen)
    ids = [perm[: nb[0]], perm[nb[0]:]]
    cpu = []
    for _ in range(Ls):
        cc = synth.make_paged_layer(sum(nb) + 5, BLOCK_SIZE, Hkv, D, kv_axis=0)
        for b, t in enumerate(lens):
            synth.write_tokens_to_paged(cc, 0, ids[b], BLOCK_SIZE, synth.make_rotated_keys(Hkv, t, D, inv, gen),
                                        synth.make_values(Hkv, t, D, gen))
        cpu.append(cc)
    off = torch.tensor([float(2 ** i) for i in range(17)])
    full = ops.DeviceStats(sst.q_mean_real.to(device), sst.q_mean_imag.to(device), sst.q_abs_mean.to(device),
                           torch.ones_like(sst.q_abs_mean).to(device), inv.to(device), off.to(device))
    lo, hi = tp.head_range(Hkv, rank, world)
    shard = tp.shard_stats(full, rank, world)
    mine = [x[:, :, :, lo:hi].contiguous().to(device) for x in cpu]
    r1 = engine.PagedCompressor(shard, window=32).compress(ops.PagedCacheView.from_layers(mine, kv_axis=0), ids, lens, lens, buds)
    mine2 = [x[:, :, :, lo:hi].contiguous().to(device) for x in cpu]
    r2 = engine.compress_layer_shared(ops.PagedCacheView.from_layers(mine2, kv_axis=0), shard, ids, lens, lens, buds, window=32)
    one = [x.to(device) for x in cpu]
    s1 = engine.PagedCompressor(full, window=32).compress(ops.PagedCacheView.from_layers(one, kv_axis=0), ids, lens, lens, buds)
    one2 = [x.to(device) for x in cpu]
    s2 = engine.compress_layer_shared(ops.PagedCacheView.from_layers(one2, kv_axis=0), full, ids, lens, lens, buds, window=32,
                                      process_group=False)
    ok = (torch.equal(r1.keep, s1.keep[:, lo:hi]) and torch.equal(r2.keep, s2.keep)
          and all(torch.equal(a, b[:, :, :, lo:hi]) for a, b in zip(mine, one))
          and all(torch.equal(a, b[:, :, :, lo:hi]) for a, b in zip(mine2, one2)))
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    out["parity"] = {"sharded_equals_single_gpu": bool(flag.item()), "rank_keep_sets_identical": same,
                     "shape": "2 layers, 64q/8kv heads, requests of 900 and 1500 tokens, both modes, keep sets and caches"}
    return out


# ----------------------------------------------------------------------------- our arm
def measure(args, c, world, rank, local, config_idx):
    """Builds the workload of configuration ``c`` on this rank and times it: the fused device step, the end-to-end
    call through the batched engine, and every stage on its own.  Returns a dictionary of measurements plus the
    live workload (for the correctness gate)."""
    from triattention_b200 import _native, engine, ops

    device = torch.device("cuda", local)
    caches, block_ids, stats = build_device_workload(c, rank, device, config_idx)
    view = ops.PagedCacheView.from_layers(caches, kv_axis=0)
    B, T, k, L, H = c["B_local"], c["T"], c["k"], c["L"], c["Hkv_local"]
    saver = PrefixSaver(caches, block_ids, k)
    agg = _native.OFFSETS_MAX if args.aggregation == "max" else _native.OFFSETS_MEAN
    comp = engine.PagedCompressor(stats, window=c["window"], offset_agg=agg,
                                  use_cuda_graph=bool(args.cuda_graph),
                                  max_workspace_bytes=(args.workspace_mb << 20) if args.workspace_mb else None)
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
    ws_full = ops.compress_workspace_bytes(layout, 17, agg, k)
    ws_min = ops.compress_workspace_bytes_min(layout, 17, agg, k)
    ws_bytes = ws_full if not args.workspace_mb else min(ws_full, max(ws_min, args.workspace_mb << 20))
    per_layer = (ws_full - ws_min) // (L - 1) if L > 1 else 0
    chunk_layers = L if per_layer == 0 else min(L, 1 + (ws_bytes - ws_min) // per_layer)
    n_chunks = (L + chunk_layers - 1) // chunk_layers
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
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
    del ws, keep_out, bt, comp
    return dict(step_ms=step_ms, e2e_s=e2e_s, stage=stage, clocks=clocks, keys_per_gpu=keys_per_gpu, ws_bytes=ws_bytes,
                n_chunks=n_chunks, device_status=status_bits | res.device_status, h2d=res.h2d_bytes, d2h=res.d2h_bytes,
                agg=agg, caches=caches, block_ids=block_ids, stats=stats, saver=saver)


def run_ours(args, world, rank, local):
    from triattention_b200 import _native

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    _native.load()
    torch.cuda.set_device(torch.device("cuda", local))
    shard_of = args.shard_of if (args.shard_of and world == 1) else 0
    c = resolve_config(args, shard_of or world)
    m = measure(args, c, world, rank, local, sorted(CONFIGS).index(args.config))
    B, T, k, L, H = c["B_local"], c["T"], c["k"], c["L"], c["Hkv_local"]
    step_ms, e2e_s, stage, keys_per_gpu = m["step_ms"], m["e2e_s"], m["stage"], m["keys_per_gpu"]

    parity = None
    if not args.no_parity and rank == 0:
        parity = parity_gate(c, m["caches"], m["block_ids"], m["stats"], c["window"], m["agg"], m["saver"])
    for key in ("caches", "block_ids", "stats", "saver"):
        m.pop(key)

    extra = {}
    if world >= 2 and not args.no_c2 and args.config == "c1":
        torch.cuda.empty_cache()
        barrier(world)
        extra["c2"] = run_c2_legs(args, world, rank, local)

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
                   f"{score_bytes / 1e9:.1f} GB per step); compacted prefix restored untimed between steps",
                   "workspace_bytes": m["ws_bytes"], "layer_chunks": m["n_chunks"]},
        "keys_per_s_per_gpu": value / world,
        "step_hbm_gbs": bytes_step / (step_ms * 1e-3) / 1e9, "step_hbm_frac": bytes_step / (step_ms * 1e-3) / 1e9 / peak,
        "stage_ms": stage,
        "roofline": {"kernel": score_kernel_name(c, args.aggregation),
                     "bound": "hbm", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                     "traffic": (keys_per_gpu * SCORE_DRAM_BYTES_PER_KEY_NCU[(args.aggregation, c["g"])]
                                 if c["D"] == 128 and (args.aggregation, c["g"]) in SCORE_DRAM_BYTES_PER_KEY_NCU else None),
                     "traffic_note": "bytes per launch, scaled by keys from a small ncu capture of the same kernel "
                                     "and group size (profiles/)"},
        "e2e": {"value": keys_per_gpu * world / e2e_s, "unit": UNIT, "h2d_bytes_per_step": m["h2d"],
                "d2h_bytes_per_step": m["d2h"], "ms_per_step": e2e_s * 1e3,
                "api": "engine.PagedCompressor.compress (host block tables -> pinned -> H2D, kernels, D2H status)"},
        # prep, top-k, compaction + per chunk of layers: score, finalize (+ the tensor-map stamp of the tcgen05 scorer)
        "gpu_launches": (3 + (3 if score_kernel_name(c, args.aggregation) == "score_paged_umma_max_kernel" else 2)
                         * m["n_chunks"]) * args.steps,
        "clocks": m["clocks"], "device_status": m["device_status"],
    }
    if parity is not None:
        line["parity"] = parity
    if extra:
        line["extra"] = extra
    if not args.no_cpu_baseline and world == 1:
        torch.set_num_threads(os.cpu_count() or 1)
        cpu_baseline_run(c, 1, min(2048, c["T"]))
        v, dt, desc, kind = cpu_baseline_run(c, min(2, c["L"]), min(c["T"], 32768))
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
                                "sample": desc, "seconds": dt}
    print(json.dumps(line), flush=True)
    if m["device_status"] != 0:
        raise SystemExit(f"device status {m['device_status']:#x}: a kernel flagged bad metadata or a wait that ran out")
    if parity is not None and not parity["ok"]:
        raise SystemExit("parity gate failed: " + json.dumps(parity))
    if extra.get("c2", {}).get("parity") and not all(extra["c2"]["parity"][x] for x in
                                                        ("sharded_equals_single_gpu", "rank_keep_sets_identical")):
        raise SystemExit("config-2 parity failed: " + json.dumps(extra["c2"]["parity"]))


def main():
    args = parse_args()
    world, rank, local = dist_setup(args)
    if args.gpus != world and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    try:
        if args.impl == "reference":
            run_reference(args, world, rank)
        elif args.impl == "reference_gpu":
            run_reference_gpu(args, rank)
        elif args.config == "c3":
            from bench_decode import run_decode_interleaved
            run_decode_interleaved(args, world, rank, local)
        elif args.sweep:
            from bench_decode import run_sweep
            run_sweep(args, world, rank, local)
        else:
            run_ours(args, world, rank, local)
    finally:
        if world > 1 and args.impl == "ours":
            import torch.distributed as dist
            if dist.is_initialized():
                dist.destroy_process_group()


if __name__ == "__main__":
    main()
