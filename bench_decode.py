"""Two further drivers of bench.py: the decode-interleaved workload (``--config c3``) and the
length / batch / budget sweep (``--sweep``).

Decode-interleaved compression (Llama-3.1-8B shapes: 32 layers, 32 query / 8 KV heads, head_dim 128, llama3-scaled
RoPE).  64 requests with prompt lengths drawn uniformly from 4096..32768 arrive in waves of 8; every request then
decodes one token per step and is compressed to the budget (2048) whenever its cache reaches budget + 128 tokens, so
it sees one large compression followed by one of 2176 -> 2048 tokens every 128 steps.  ``round_start`` is the absolute
number of tokens the request has computed (triattention/vllm/runtime/hook_group_pipeline.py:78).  The same seeded
simulation runs twice: (a) one request at a time through the hook installed by ``install_runner_compression_hook``,
as the reference's worker loop does (runtime/runner_compression_actions.py:11-237), and (b) with all requests that
triggered in a step in one ``PagedCompressor.compress`` call.  Both must leave bit-identical caches.
"""
from __future__ import annotations

import json
import os
import statistics
import time
import types

import torch

import bench as B


class _Pool:
    """Free list of cache blocks (block 0 stays unused, like a null block)."""

    def __init__(self, n: int):
        self.free = list(range(n - 1, 0, -1))

    def take(self, n: int):
        if n > len(self.free):
            raise RuntimeError("block pool exhausted")
        out = self.free[-n:][::-1]
        del self.free[-n:]
        return out

    def give(self, ids):
        self.free.extend(reversed([int(i) for i in ids]))


def _percentiles(xs):
    if not xs:
        return {}
    s = sorted(xs)
    pick = lambda q: s[min(len(s) - 1, int(q * len(s)))]
    return {"n": len(s), "p50_ms": pick(0.50), "p90_ms": pick(0.90), "p99_ms": pick(0.99), "mean_ms": statistics.mean(s)}


def _simulate(path: str, c, R: int, decode_steps: int, wave: int, gap: int, device, rank: int, world: int,
              cuda_graph: bool = False):
    """One full run of the decode-interleaved workload through ``path`` ('hook' or 'engine').

    Returns (records, cache hash): one record per trigger (or per engine call) with its cached length and wall time.
    """
    import synth
    from triattention_b200 import engine, hook as hook_mod, ops
    from triattention_b200.config import TriAttentionRuntimeConfig
    from triattention_b200.signals import CompressionSignal

    L, H, D, bs = c["L"], c["Hkv"] // world, c["D"], B.BLOCK_SIZE
    F = D // 2
    budget, slack, window = c["budget"], 128, c["window"]
    seed = synth.seed_for(3, 1, rank)
    gen = torch.Generator(device=device).manual_seed(seed)
    cgen = torch.Generator().manual_seed(seed)
    inv = synth.rope_inv_freq(D, c["theta"], c.get("llama3"))
    inv_d = inv.to(device)
    full = synth.make_stats(L, c["Hq"], D, inv, cgen)
    g = c["Hq"] // c["Hkv"]
    h0, h1 = rank * H * g, (rank + 1) * H * g
    off = torch.tensor([float(2 ** i) for i in range(17)])
    stats = ops.DeviceStats(full.q_mean_real[:, h0:h1].contiguous().to(device), full.q_mean_imag[:, h0:h1].contiguous().to(device),
                            full.q_abs_mean[:, h0:h1].contiguous().to(device), torch.ones((L, h1 - h0, F), device=device),
                            inv_d, off.to(device))
    # prompt lengths: multiples of the block size in [4096, 32768]
    T0 = (torch.randint(4096 // bs, 32768 // bs + 1, (R,), generator=cgen) * bs).tolist()
    per_req_steady = (budget + slack) // bs + 1
    n_blocks = wave * (32768 // bs + slack // bs + 1) + R * per_req_steady + 64
    pool = _Pool(n_blocks)
    caches = [torch.zeros((2, n_blocks, bs, H, D), dtype=torch.bfloat16, device=device) for _ in range(L)]
    lo, hi = torch.log(torch.tensor(0.1)).item(), torch.log(torch.tensor(10.0)).item()
    scale = torch.exp(lo + (hi - lo) * torch.rand((L, 1, 1, H, D), generator=gen, device=device))
    view = ops.PagedCacheView.from_layers(caches, kv_axis=0)

    def write_tokens(reqs, start_slots, positions0, count):
        """K/V of ``count`` consecutive tokens for each listed request, all layers at once: K ~ N(0,1) x per-channel
        scale rotated at the tokens' ABSOLUTE positions, V ~ N(0,1); slots are block-aligned."""
        n = len(reqs)
        nb = count // bs
        blk = torch.tensor([ids[r][start_slots[i] // bs: start_slots[i] // bs + nb] for i, r in enumerate(reqs)],
                           dtype=torch.long, device=device).reshape(-1)
        pos = (torch.tensor(positions0, dtype=torch.float32, device=device).view(n, 1)
               + torch.arange(count, dtype=torch.float32, device=device).view(1, count))
        ang = pos.view(n, nb, bs, 1, 1) * inv_d.view(1, 1, 1, 1, F)
        cos, sin = torch.cos(ang), torch.sin(ang)
        for l in range(L):
            pre = torch.randn((n, nb, bs, H, D), generator=gen, device=device) * scale[l]
            pr, pi = pre[..., :F], pre[..., F:]
            rot = torch.cat([pr * cos - pi * sin, pr * sin + pi * cos], dim=-1).to(torch.bfloat16)
            caches[l][0].index_copy_(0, blk, rot.view(n * nb, bs, H, D))
            caches[l][1].index_copy_(0, blk, torch.randn((n * nb, bs, H, D), generator=gen, device=device).to(torch.bfloat16))

    ids = [[] for _ in range(R)]          # block table per request
    cur = [0] * R                          # tokens currently cached
    seen = [0] * R                         # absolute tokens computed (round_start)
    left = [0] * R                         # decode steps still to do
    active = [False] * R
    records = []

    # ---- compression paths
    if path in ("hook", "hook_batch"):
        # the hook loads its statistics from a file, as in serving: this rank's rows in the calibration format
        import tempfile
        tmp = tempfile.TemporaryDirectory()
        sp = os.path.join(tmp.name, "stats.pt")
        synth.save_stats_pt(synth.SyntheticStats(full.q_mean_real[:, h0:h1].contiguous(), full.q_mean_imag[:, h0:h1].contiguous(),
                                                 full.q_abs_mean[:, h0:h1].contiguous(), inv, D, "half"), sp)
        cfg = TriAttentionRuntimeConfig(kv_budget=budget, divide_length=slack, window_size=window, sparse_stats_path=sp,
                                        use_cuda_graph=cuda_graph)
        runner = types.SimpleNamespace(requests={}, kv_caches=caches, cache_config=types.SimpleNamespace(block_size=bs))
        hook_mod.install_runner_compression_hook(runner, cfg)
        hook = runner.triattention_apply_compression
        hook_batch = runner.triattention_apply_compression_batch
    else:
        comp = engine.PagedCompressor(stats, window=window, use_cuda_graph=cuda_graph)

    def compress(trig, step):
        if path == "hook":
            for r in trig:
                req = f"r{r}"
                runner.requests[req] = types.SimpleNamespace(block_ids=(list(ids[r]),), num_computed_tokens=seen[r])
                sig = CompressionSignal(req, True, "length_threshold", cur[r] + 1, step, None, False, 0, 1)
                so = types.SimpleNamespace(num_scheduled_tokens={req: 1})
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                out = hook(req_id=req, signal=sig, scheduler_output=so)
                torch.cuda.synchronize()
                dt = time.perf_counter() - t0
                if not out.get("applied"):
                    raise RuntimeError(f"hook did not compress request {r}: {out}")
                records.append({"T": cur[r], "n": 1, "ms": dt * 1e3})
                kept = list(runner.requests[req].block_ids[0])
                pool.give(ids[r][len(kept):])
                ids[r] = kept
                cur[r] = int(out["cache_len_after"])
        elif path == "hook_batch":
            # the step's triggered requests through the batched hook: the per-request contract, one native call
            reqs = []
            for r in trig:
                req = f"r{r}"
                runner.requests[req] = types.SimpleNamespace(block_ids=(list(ids[r]),), num_computed_tokens=seen[r])
                reqs.append((req, CompressionSignal(req, True, "length_threshold", cur[r] + 1, step, None, False, 0, 1)))
            so = types.SimpleNamespace(num_scheduled_tokens={req: 1 for req, _ in reqs})
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            outs = hook_batch(reqs, so)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            records.append({"T": [cur[r] for r in trig], "n": len(trig), "ms": dt * 1e3})
            for r in trig:
                out = outs[f"r{r}"]
                if not out.get("applied"):
                    raise RuntimeError(f"batched hook did not compress request {r}: {out}")
                kept = list(runner.requests[f"r{r}"].block_ids[0])
                pool.give(ids[r][len(kept):])
                ids[r] = kept
                cur[r] = int(out["cache_len_after"])
        else:
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            res = comp.compress(view, [ids[r] for r in trig], [cur[r] for r in trig], [seen[r] for r in trig],
                                [budget] * len(trig))
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            if res.device_status:
                raise RuntimeError(f"device status {res.device_status}")
            records.append({"T": [cur[r] for r in trig], "n": len(trig), "ms": dt * 1e3})
            for j, r in enumerate(trig):
                pool.give(res.removed_block_ids[j])
                ids[r] = list(res.kept_block_ids[j])
                cur[r] = res.keep_counts[j]

    n_waves = (R + wave - 1) // wave
    total_steps = (n_waves - 1) * gap + decode_steps + 1
    for step in range(total_steps):
        # arrivals: prefill the prompt and the first `slack` decode tokens
        if step % gap == 0 and step // gap < n_waves:
            new = list(range((step // gap) * wave, min(R, (step // gap + 1) * wave)))
            for r in new:
                ids[r] = pool.take(T0[r] // bs + slack // bs)
                cur[r] = seen[r] = T0[r]
                left[r] = decode_steps
                active[r] = True
            # prompts differ in length: write them request by request in chunks of 2048 tokens
            for r in new:
                for s0 in range(0, T0[r] + slack, 2048):
                    n_tok = min(2048, T0[r] + slack - s0)
                    write_tokens([r], [s0], [s0], n_tok)
        # one decode step for every active request (its token was written ahead)
        trig = []
        for r in range(R):
            if active[r] and left[r] > 0:
                cur[r] += 1
                seen[r] += 1
                left[r] -= 1
                if left[r] == 0:
                    active[r] = False
                if cur[r] >= budget + slack:
                    trig.append(r)
        if trig:
            compress(trig, step)
            # the next `slack` tokens of the compressed requests go behind their kept prefix
            todo = [r for r in trig if active[r]]
            for r in todo:
                need = (cur[r] + slack + bs - 1) // bs - len(ids[r])
                if need > 0:
                    ids[r] = ids[r] + pool.take(need)
            if todo:
                write_tokens(todo, [cur[r] for r in todo], [seen[r] for r in todo], slack)
    torch.cuda.synchronize()
    # hash of every request's live tokens, in logical order
    import hashlib
    h = hashlib.sha256()
    for r in range(R):
        nb = (cur[r] + bs - 1) // bs
        idx = torch.tensor(ids[r][:nb], dtype=torch.long, device=device)
        for l in (0, L // 2, L - 1):
            h.update(caches[l].index_select(1, idx).cpu().view(torch.int16).numpy().tobytes())
    return records, h.hexdigest(), T0


def run_decode_interleaved(args, world, rank, local):
    from triattention_b200 import _native

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    _native.load()
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    c = dict(B.CONFIGS["c3"])
    if args.layers:
        c["L"] = args.layers
    R = args.batch or 64
    S = args.decode_steps
    wave, gap = 8, 4
    L, H = c["L"], c["Hkv"] // world
    peak, peak_kind = B.measured_peaks()
    out = {}
    hashes = {}
    for path in ("hook", "hook_batch", "engine"):
        B.barrier(world)
        t0 = time.perf_counter()
        rec, digest, T0 = _simulate(path, c, R, S, wave, gap, device, rank, world, bool(getattr(args, "cuda_graph", False)))
        wall = time.perf_counter() - t0
        hashes[path] = digest
        k = c["budget"]
        first = [r for r in rec if (r["T"] if path == "hook" else max(r["T"])) > k + 128]
        steady = [r for r in rec if r not in first]

        def summarise(rs):
            if not rs:
                return {}
            keys = sum(L * H * (r["T"] if path == "hook" else sum(r["T"])) for r in rs)
            kept = sum(L * H * k * r["n"] for r in rs)
            secs = sum(r["ms"] for r in rs) * 1e-3
            trig = sum(r["n"] for r in rs)
            d = {"triggers": trig, "calls": len(rs), "keys_per_s": keys / secs,
                 "hbm_frac": (keys * 256.0 + kept * 1024.0) / secs / 1e9 / peak,
                 "ms_per_trigger": secs * 1e3 / trig, "call_latency": _percentiles([r["ms"] for r in rs])}
            return d

        out[path] = {"first_compression": summarise(first), "steady_state": summarise(steady),
                     "all": summarise(rec), "simulation_wall_s": wall}
        torch.cuda.empty_cache()
    if rank != 0:
        return
    # the reference's CPU path on one steady-state trigger (all KV heads), timed beside it
    cpu = None
    if not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        cs = B.resolve_config(args, 1, "c3s")
        B.cpu_baseline_run(cs, 1, 2176)
        v, dt, desc, kind = B.cpu_baseline_run(cs, min(cs["L"], 4), 2176)
        cpu = {"value": v, "unit": B.UNIT, "cores": torch.get_num_threads(), "kind": kind, "sample": desc, "seconds": dt,
               "ms_per_trigger_extrapolated": dt * 1e3 * c["L"] / min(cs["L"], 4)}
    eng_all, hook_all = out["engine"]["all"], out["hook"]["all"]
    line = {
        "metric": B.METRIC, "value": eng_all["keys_per_s"] * world, "unit": B.UNIT, "n_gpus": world,
        "steps": S, "warmup": 0, "ms_per_step": eng_all["ms_per_trigger"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"c3: decode-interleaved, {L} layers, 32q/8kv heads, head_dim 128, llama3 RoPE, {R} requests "
                               f"with prompts U{{4096..32768}}, {S} decode steps each, budget {c['budget']} + 128 slack",
                   "arrivals": f"waves of {wave} requests every {gap} steps", "timing": "wall clock around each call, "
                   "device synchronised on both sides (host metadata, H2D, kernels, D2H status inside)",
                   "l2": "every trigger reads its request's whole cache; caches of different requests evict each other"},
        "e2e": {"value": hook_all["keys_per_s"] * world, "unit": B.UNIT, "api": "per-request hook "
                "(install_runner_compression_hook contract)", "ms_per_trigger": hook_all["ms_per_trigger"],
                "h2d_bytes_per_step": None, "d2h_bytes_per_step": 4},
        "paths": out, "paths_leave_identical_caches": hashes["hook"] == hashes["engine"] == hashes["hook_batch"],
        "roofline": {"bound": "hbm", "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                     "frac": out["engine"]["steady_state"].get("hbm_frac"),
                     "note": "steady-state triggers through the batched engine: (256 B per key + 1024 B per kept token) / time"},
        "gpu_launches": 5 * out["engine"]["all"]["calls"],
    }
    if cpu:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)
    if not (hashes["hook"] == hashes["engine"] == hashes["hook_batch"]):
        raise SystemExit("the hook, batched-hook and engine paths left different caches")


# ----------------------------------------------------------------------------- sweep (BASELINE config 4)
DEFAULT_SWEEP = [
    # (tokens, batch, budget, layers): the per-layer work is unchanged when layers are cut to fit one GPU
    (8192, 32, 2048, 36), (16384, 16, 2048, 36), (32768, 8, 2048, 36), (65536, 4, 2048, 36), (131072, 2, 2048, 36),
    (32768, 1, 2048, 36), (32768, 32, 2048, 9), (32768, 128, 2048, 2),
    (32768, 8, 1024, 36), (32768, 8, 4096, 36), (32768, 8, 12000, 36),
]


def run_sweep(args, world, rank, local):
    """Cached length x batch x budget on the Qwen3-8B shape; one JSON line per point (rank 0), per-GPU keys fixed
    across ranks (each rank owns 8/N KV heads of N times the requests).  The CPU column is the reference's CPU
    path on a one-request, two-layer slice of the same length and budget (rank 0, single-GPU runs only)."""
    from triattention_b200 import _native

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    _native.load()
    torch.cuda.set_device(torch.device("cuda", local))
    points = DEFAULT_SWEEP
    if args.sweep_points:
        points = []
        for p in args.sweep_points.split(","):
            t, b, k, *rest = (int(x) for x in p.split(":"))
            points.append((t, b, k, rest[0] if rest else 36))
    peak, _ = B.measured_peaks()
    cpu_cache = {}
    for (T, Bn, k, L) in points:
        c = dict(B.CONFIGS["c1"])
        c.update(L=L, B=Bn, T=T, budget=k)
        c["g"] = c["Hq"] // c["Hkv"]
        c["Hkv_local"] = c["Hkv"] // world
        c["B_local"] = Bn * world
        c["k"] = min(k, T)
        m = B.measure(args, c, world, rank, local, 4)
        for key in ("caches", "block_ids", "stats", "saver"):
            m.pop(key)
        torch.cuda.empty_cache()
        if rank != 0:
            continue
        keys = m["keys_per_gpu"]
        row = {"sweep": {"tokens": T, "batch": Bn, "budget": k, "layers": L}, "n_gpus": world,
               "ms_per_step": m["step_ms"], "keys_per_s_per_gpu": keys / (m["step_ms"] * 1e-3),
               "keys_per_s_total": keys * world / (m["step_ms"] * 1e-3),
               "step_hbm_frac": keys * B.algorithmic_bytes_per_key(T, c["k"]) / (m["step_ms"] * 1e-3) / 1e9 / peak,
               "score_hbm_frac": keys * 256.0 / (m["stage"]["score"] * 1e-3) / 1e9 / peak, "stage_ms": m["stage"],
               "e2e_ms": m["e2e_s"] * 1e3, "clocks": m["clocks"], "device_status": m["device_status"]}
        if not args.no_cpu_baseline and world == 1:
            ck = (min(T, 32768), k)
            if ck not in cpu_cache:
                torch.set_num_threads(os.cpu_count() or 1)
                v, dt, desc, kind = B.cpu_baseline_run(c, 2, ck[0])
                cpu_cache[ck] = {"keys_per_s": v, "kind": kind, "cores": torch.get_num_threads(), "sample": desc}
            row["cpu"] = cpu_cache[ck]
        print(json.dumps(row), flush=True)
        if m["device_status"] != 0:
            raise SystemExit(f"device status {m['device_status']:#x} at sweep point {row['sweep']}")
