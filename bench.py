#!/usr/bin/env python
"""Benchmark of the KV-cache hot path: per-step K/V append + GQA decode attention.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): the decode phase of a Llama-3.1-8B-shaped model - 32 layers,
32 query / 8 KV heads, head_dim 128, bf16 - batch 32, 512-token prompts already in
the cache, one token appended per sequence per step.  One "step" is one pass of the
hot path over the batch: for each of the 32 layers, append the new K/V rows and
attend over the whole cache.  The projections / MLP around it are not part of the
path and are not run.  K/V/Q are seeded N(0,1) synthetic tensors.

Prints ONE JSON line (rank 0).  `value` is decode tokens/s with inputs resident in
HBM (CUDA-graph replay of the step); `e2e` is the same through host buffers (pinned
H2D of the step's K/V/Q, D2H of the attention outputs, inside the timed region);
`roofline` is the decode-attention kernel against the measured HBM copy bandwidth;
`cpu_baseline` is the CPU restatement of the reference's path on this host's cores.
With N > 1 every rank runs the same per-GPU workload on its own sequences (requests
are sharded, no collective on the path): weak scaling.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "amd-pace_b200"))

import torch  # noqa: E402

CFG = dict(n_layers=32, batch=32, hq=32, hkv=8, d=128, prompt=512, max_new=256)
WORKLOAD = "llama31_8b_shape_decode_b32_prompt512_kv_append+gqa_attention_32layers"
FALLBACK_HBM_GBS = 6650.0


def measured_hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def workload_config(n_gpus: int) -> dict:
    """The workload both arms are timed on: identical keys and values in the GPU line and in the
    reference arm's line."""
    return {"workload": WORKLOAD, "batch_per_gpu": CFG["batch"], "global_batch": CFG["batch"] * n_gpus,
            "layers": CFG["n_layers"], "q_heads": CFG["hq"], "kv_heads": CFG["hkv"], "head_dim": CFG["d"],
            "prompt_tokens": CFG["prompt"], "new_tokens": CFG["max_new"],
            "parallelism": f"dp{n_gpus} (sequences sharded, no collective)"}


CPU_SAMPLE_LAYERS, CPU_SAMPLE_WARMUP = 4, 2


def cpu_reference_line(steps: int):
    """The reference's CPU path on this host's cores, on a bounded sample of the workload: the same
    batch, shapes and cache length as the GPU arm, over 4 of the 32 layers (every layer costs the same:
    an append and an attention pass over its own cache), scaled to 32.  The reference's own classes when
    its package has been staged under oracle/_ref/, else the restatement.  Always 2 warm-up steps; the step
    time is the median over the timed steps, so both callers (the `cpu_baseline` leg of the GPU line and
    the reference arm) report the same quantity whatever their step count."""
    from oracle.cpu_path import time_decode_tokens_per_s
    # every host core this process may run on (a launcher such as torchrun sets OMP_NUM_THREADS=1)
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    torch.set_num_threads(max(1, cores))
    cores = torch.get_num_threads()
    tps, step_s, kind = time_decode_tokens_per_s(CFG["n_layers"], CPU_SAMPLE_LAYERS, CFG["batch"], CFG["hq"],
                                                 CFG["hkv"], CFG["d"], CFG["prompt"], CFG["prompt"] + CFG["max_new"],
                                                 steps, CPU_SAMPLE_WARMUP)
    what = ("the reference's own BMCKVCache.update_cache + repeat_kv + MultiHeadAttention(NATIVE)" if kind == "reference"
            else "restatement of the reference layout: BMC append + repeat_kv + torch CPU SDPA with additive mask")
    sample = (f"median of {steps} decode steps over {CPU_SAMPLE_LAYERS} of {CFG['n_layers']} layers ({what}), "
              f"scaled to {CFG['n_layers']} layers")
    return tps, step_s, cores, kind, sample


def run_reference(args, rank):
    if rank != 0:
        return
    steps = max(3, min(args.steps, 200))
    tps, step_s, cores, kind, sample = cpu_reference_line(steps)
    line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": tps, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args.gpus),
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def gpu_local_cores(local_rank: int):
    """Cores NVML reports as local to this rank's GPU (its NUMA node), or None when NVML cannot say.
    Reading only: nothing on the GPU is set."""
    try:
        import pynvml
        pynvml.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        index = local_rank
        if visible:
            ids = [v.strip() for v in visible.split(",") if v.strip()]
            if local_rank < len(ids) and ids[local_rank].isdigit():
                index = int(ids[local_rank])
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cores = [w * 64 + b for w, m in enumerate(mask) for b in range(64) if (int(m) >> b) & 1]
        return cores or None
    except Exception:
        return None


def pin_rank_to_cores(local_rank: int, world: int):
    """Each rank keeps its own slice of the cores this process may run on - set before the CUDA context
    and the pinned buffers exist, so that the rank's copies are driven from, and its pinned memory is
    allocated near, cores no other rank uses (the reference's workers pin themselves the same way,
    pace/utils/worker.py:49-62).  Where NVML names the cores local to the rank's GPU the slice is cut from
    those (the GPUs of one NUMA node share them in rank order): pinned buffers first touched on the far
    socket make every copy cross the inter-socket link.  Returns the slice."""
    try:
        allowed = sorted(os.sched_getaffinity(0))
    except AttributeError:
        return None
    if world <= 1 or len(allowed) < world:
        return allowed
    per = len(allowed) // world
    mine = allowed[local_rank * per:(local_rank + 1) * per]
    try:
        local = gpu_local_cores(local_rank)
        if local:
            near = [c for c in allowed if c in set(local)]
            # ranks whose GPUs report the same core set share it in rank order
            same = [r for r in range(world) if (gpu_local_cores(r) or []) == local]
            if len(near) >= len(same) >= 1 and local_rank in same:
                share = len(near) // len(same)
                k = same.index(local_rank)
                if share >= 1:
                    mine = near[k * share:(k + 1) * share]
    except Exception:
        pass
    try:
        os.sched_setaffinity(0, mine)
    except OSError:
        return allowed
    return mine


RANK_CORES = None


def run_ours(args, rank, world, local_rank):
    cores = RANK_CORES
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU implementation")
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.llm.graph import StepGraph
    from pace_b200.ops import MultiHeadAttention
    from pace_b200.ops.backends.b200 import workspace
    from pace_b200 import _C
    import ctypes as C

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    L, B, Hq, Hkv, D, P0 = (CFG[k] for k in ("n_layers", "batch", "hq", "hkv", "d", "prompt"))
    e2e_steps = min(args.steps, 32)
    roof_reps = 5
    n_blocks = 5
    needed = 2 + args.warmup + args.steps + 1 + 1 + 3 + e2e_steps + 2
    max_new = max(CFG["max_new"], needed) + 8

    class Cfg:
        num_hidden_layers = L

    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    mgr = KVCacheManager(Cfg(), P0 + max_new, KVCacheType.BMC)
    # prompt K/V: appended in 128-token pieces so the staging tensors stay small
    for _ in range(P0 // 128):
        for l in range(L):
            k = torch.randn(B, Hkv, 128, D, device=dev, generator=g, dtype=torch.float32).bfloat16()
            v = torch.randn(B, Hkv, 128, D, device=dev, generator=g, dtype=torch.float32).bfloat16()
            mgr[l].update_cache(k, v, concat_dim=2)
    # the step's inputs, resident on the device: per layer K/V of the new token and the query
    kvq = torch.randn(L, B, Hkv + Hkv + Hq, D, device=dev, generator=g, dtype=torch.float32).bfloat16()
    # Deferred appends: the step's new rows stay where they arrive (kvq is the staging buffer), every
    # layer's decode launch takes its row from there as the newest key, and one kernel at the end of
    # the step stores all 32 layers' rows in the pool.
    k_all, v_all = kvq[:, :, :Hkv].unsqueeze(3), kvq[:, :, Hkv:2 * Hkv].unsqueeze(3)
    mgr.defer_appends = True
    mgr.adopt_staging(k_all, v_all)
    k_new = [k_all[l] for l in range(L)]
    v_new = [v_all[l] for l in range(L)]
    q_new = [kvq[l, :, 2 * Hkv:].unsqueeze(2) for l in range(L)]
    out_all = torch.empty(L, B, 1, Hq, D, device=dev, dtype=torch.bfloat16)
    out_views = [out_all[l].transpose(1, 2) for l in range(L)]   # [B, Hq, 1, D] views the kernel writes through
    mha = MultiHeadAttention()

    def step_fn():
        for l in range(L):
            K, V = mgr[l].update_cache(k_new[l], v_new[l], concat_dim=2)
            mha(q_new[l], K, V, out=out_views[l])
        return out_all

    graph = StepGraph(mgr, step_fn, n_new=1, warmup=2)     # (ends every step with mgr.commit())
    own_launches_per_step = L + 1   # + the page reservation kernel in the steps that reach a new page

    def barrier():
        if world > 1:
            torch.distributed.barrier()

    for _ in range(args.warmup):
        graph.replay()
    torch.cuda.synchronize()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.25)
    torch.cuda.synchronize()
    # The timed region is `--steps` graph replays, bracketed by a barrier and a synchronisation on both
    # sides.  It is taken n_blocks times over the SAME lengths - between blocks the cache is rolled back
    # by `--steps` tokens (remove_cache: lengths only, the pages stay) - and the median block is reported,
    # with the spread of the blocks beside it.
    def timed_block(n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        barrier()
        before = graph.replays_with_reserve
        e0.record()
        for _ in range(n):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        barrier()
        return e0.elapsed_time(e1), graph.replays_with_reserve - before

    block_ms, timed_reserves = [], 0
    for blk in range(n_blocks):
        t_ms, timed_reserves = timed_block(args.steps)
        block_ms.append(t_ms)
        if blk + 1 < n_blocks:
            mgr.remove_cache(args.steps)
    ms = statistics.median(block_ms)
    time.sleep(0.15)
    clocks = sampler.stop()
    mgr.pool.check_status()
    len_after_timed = mgr[0].seq_len

    # ---- end to end: host buffers in, host buffers out, copies inside the timed region ----
    # One step = the host->device copy of every layer's new K/V/Q rows from pinned memory, the 32
    # [append, attention] pairs, and the device->host copy of every layer's attention output; the
    # caller synchronises after every step.  The copies are cut into chunks of layers and recorded in
    # the same CUDA graph on two side streams, so that inside a step a chunk's copies overlap the
    # other chunks' kernels (layer l only needs layer l's rows).  Steps do not overlap one another.
    host_in = torch.empty(kvq.shape, dtype=kvq.dtype).pin_memory()
    host_in.copy_(kvq.cpu())
    host_out = torch.empty(out_all.shape, dtype=out_all.dtype).pin_memory()
    n_chunks = 8 if L % 8 == 0 else 1   # (copies in growing chunks - 1, 2, 4, 8, 17 layers - measured slower: 1.17 ms per step)
    per = L // n_chunks
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    # how fast the copies in are next to the compute they feed, with every rank copying at once
    barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(5):
        with torch.cuda.stream(copy_in):
            for c in range(n_chunks):
                kvq[c * per:(c + 1) * per].copy_(host_in[c * per:(c + 1) * per], non_blocking=True)
        copy_in.synchronize()
    h2d_probe_ms = (time.perf_counter() - t0) * 1e3 / 5
    barrier()
    sparse_joins = h2d_probe_ms < 0.7 * (ms / args.steps)

    def step_e2e():
        main = torch.cuda.current_stream()
        copy_in.wait_stream(main)
        copy_out.wait_stream(main)
        arrived = []
        with torch.cuda.stream(copy_in):
            for c in range(n_chunks):
                kvq[c * per:(c + 1) * per].copy_(host_in[c * per:(c + 1) * per], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_in)
                arrived.append(ev)
        # The link brings rows about twice as fast as the layers consume them, so the copies in run ahead after
        # the first chunk; a cross-stream join in front of a kernel costs about 7 us whether or not it has to
        # wait, so the kernels join the copy stream only in front of chunks 0, 1, 2 and 4 (for the copies of
        # chunks 0 | 1 | 2-3 | 4-7) instead of in front of every chunk (0.677 -> 0.656 ms per step; splitting
        # the first chunk so that layer 0 waits for one layer's rows only gained nothing measurable).
        # Where the link is not that much faster (several ranks sharing the host's memory system), every chunk
        # joins for its own copy: a late join for four chunks' copies would hold the kernels back.
        join_for = ({c: min(n_chunks, 2 * c if c else 1) - 1 for c in range(n_chunks) if c & (c - 1) == 0}
                    if sparse_joins else {c: c for c in range(n_chunks)})
        for c in range(n_chunks):
            if c in join_for:
                main.wait_event(arrived[join_for[c]])
            for l in range(c * per, (c + 1) * per):
                K, V = mgr[l].update_cache(k_new[l], v_new[l], concat_dim=2)
                mha(q_new[l], K, V, out=out_views[l])
            done = torch.cuda.Event()
            done.record(main)
            copy_out.wait_event(done)
            with torch.cuda.stream(copy_out):
                host_out[c * per:(c + 1) * per].copy_(out_all[c * per:(c + 1) * per], non_blocking=True)
        main.wait_stream(copy_in)
        main.wait_stream(copy_out)
        return out_all

    graph_e2e = StepGraph(mgr, step_e2e, n_new=1, warmup=1)
    for _ in range(3):
        graph_e2e.replay()
    torch.cuda.synchronize()
    barrier()
    # Three blocks of e2e_steps steps over the same lengths (rolled back in between), the median block is
    # reported: one step is 0.7 ms with a host round trip in it, and a single block of twenty-odd ms has
    # read anything from 0.67 to 0.99 ms per step on one box depending on what the host did just before.
    e2e_blocks = []
    for blk in range(3):
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        barrier()
        t0 = time.perf_counter()
        f0.record()
        for _ in range(e2e_steps):
            graph_e2e.replay()
            torch.cuda.current_stream().synchronize()      # the caller has the step's result in host memory
        f1.record()
        torch.cuda.synchronize()
        e2e_wall = time.perf_counter() - t0
        e2e_blocks.append(max(f0.elapsed_time(f1), e2e_wall * 1e3))
        if blk < 2:
            mgr.remove_cache(e2e_steps)
    e2e_ms = statistics.median(e2e_blocks)
    mgr.pool.check_status()
    if not torch.equal(host_out, out_all.cpu()):
        raise SystemExit("bench.py: the end-to-end step's host result differs from the device result")
    barrier()

    # the step's copies alone, one direction at a time (same chunks, same pinned buffers, all ranks at
    # once): which direction gives way when several ranks share the host's memory system
    def copies_only(direction):
        def fn():
            for c in range(n_chunks):
                if direction == "h2d":
                    kvq[c * per:(c + 1) * per].copy_(host_in[c * per:(c + 1) * per], non_blocking=True)
                else:
                    host_out[c * per:(c + 1) * per].copy_(out_all[c * per:(c + 1) * per], non_blocking=True)
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            fn()
            torch.cuda.current_stream().synchronize()
        dt = time.perf_counter() - t0
        barrier()
        return dt * 1e3 / e2e_steps
    h2d_ms, d2h_ms = copies_only("h2d"), copies_only("d2h")

    # ---- the decode-attention kernel alone: 32 back-to-back launches, one per layer.  With no append
    # between them consecutive launches are ordered one after the other (a programmatic dependent waits
    # for the launch in front), so this is the duration of an isolated launch; inside the step the
    # next layer's launch starts while this one drains, and the roofline below takes the step's time. ----
    lens_now = mgr[0].seq_len
    K_handles = [(mgr[l].key, mgr[l].value) for l in range(L)]
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    rg = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        for l in range(L):
            mha(q_new[l], *K_handles[l])
    s.synchronize()
    with torch.cuda.graph(rg, stream=s):
        for l in range(L):
            mha(q_new[l], *K_handles[l])
    for _ in range(3):
        rg.replay()
    torch.cuda.synchronize()
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    r0.record()
    for _ in range(roof_reps):
        rg.replay()
    r1.record()
    torch.cuda.synchronize()
    alone_us = r0.elapsed_time(r1) * 1e3 / (roof_reps * L)
    del rg

    # ---- the same step at other cache lengths of the configuration's range (512 .. 768 tokens): the cache
    # is rolled back or grown (untimed replays) to the wanted length, then a block of steps is timed ----
    def alg_bytes_at(kv_len):
        return B * (2 * Hkv * D * 2 * kv_len) + 2 * B * Hq * D * 2
    peak, peak_kind = measured_hbm_peak()
    sweep_steps = max(4, min(args.steps, 16))
    by_len = {}
    for target in (() if args.no_sweep else (512, 640, CFG["prompt"] + CFG["max_new"] - sweep_steps)):
        cur = mgr[0].seq_len
        if cur > target:
            mgr.remove_cache(cur - target)
        for _ in range(max(0, target - cur)):
            graph.replay()
        t_ms, _ = timed_block(sweep_steps)
        mean_len = target + (sweep_steps + 1) / 2.0
        us = t_ms * 1e3 / (sweep_steps * L)
        by_len[str(target)] = {"kv_len_mean": mean_len, "us_per_launch": us,
                               "frac": alg_bytes_at(mean_len) / (us * 1e-6) / 1e9 / peak}
    mgr.pool.check_status()
    # Roofline over the timed region: the step is L x [append, attention] with the one-token appends
    # running beside the attention launches, so a launch's share of the step is step time / L (the
    # appends' time counts against the kernel).  Algorithmic bytes of one launch: K and V rows of every
    # cached token once, q in, o out (bf16, GQA), at the mean length of the timed steps.
    attn_us = ms * 1e3 / (args.steps * L)
    len_mean = len_after_timed - (args.steps + 1) / 2.0 + 1
    alg_bytes = alg_bytes_at(len_mean)
    achieved = alg_bytes / (attn_us * 1e-6) / 1e9

    # ---- reduce over ranks: slowest rank sets the time ----
    if world > 1:
        t = torch.tensor([ms, e2e_ms, alone_us, h2d_ms, d2h_ms, max(block_ms), min(block_ms)], device=dev,
                         dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms, e2e_ms, alone_us, h2d_ms, d2h_ms, blk_max, blk_min = (float(x) for x in t.tolist())
        block_ms = [blk_min, ms, blk_max]
        attn_us = ms * 1e3 / (args.steps * L)
        achieved = alg_bytes / (attn_us * 1e-6) / 1e9
    tokens = B * args.steps * world
    value = tokens / (ms * 1e-3)
    e2e_value = B * e2e_steps * world / (e2e_ms * 1e-3)
    if rank != 0:
        return
    line = {
        "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(world),
        "timed_region": {"kv_len_start": len_after_timed - args.steps, "kv_len_end": len_after_timed,
                         "page_tokens": mgr.pool.page_tokens,
                         "l2": "inputs_larger_than_l2 (%.1f GB of K/V per step)" % (L * alg_bytes / 1e9),
                         "launch": "one CUDA graph per step: 32 decode launches that take the step's new K/V row "
                                   "from the staging buffer, then one commit of all layers",
                         "blocks": n_blocks, "block_ms": block_ms,
                         "block_spread": (max(block_ms) - min(block_ms)) / ms,
                         "note": f"median of {n_blocks} blocks of --steps replays over the same lengths (the cache "
                                 "is rolled back by --steps tokens between blocks)",
                         "cores_of_this_rank": len(cores) if cores else None},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": host_in.numel() * 2,
                "d2h_bytes_per_step": host_out.numel() * 2, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                "h2d_only_ms_per_step": h2d_ms, "d2h_only_ms_per_step": d2h_ms,
                "block_ms_per_step": [b / e2e_steps for b in e2e_blocks],
                "overlap": f"within a step only: copies in {n_chunks} chunks of {per} layers on side streams of the "
                           "step's CUDA graph (the kernels join the copies in in front of "
                           + ("chunks 0, 1, 2 and 4" if sparse_joins else "every chunk") + "); the host synchronises after every step"},
        "gpu_launches": (own_launches_per_step * args.steps + timed_reserves) * world,
        "gpu_launches_note": (f"{own_launches_per_step} own kernels per step: {L} decode attention launches and the commit "
                              f"of the step's rows, plus the page reservation kernel in the {timed_reserves} of "
                              f"{args.steps} steps in which a sequence reached a new page"),
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "attn_mma_kernel<128,1,4> (GQA decode, 4 query heads packed per MMA tile, two CTAs per SM)",
                     "achieved": achieved, "peak": peak,
                     "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                     "frac_of_nominal_8TBs": achieved / 8000.0, "us_per_launch": attn_us,
                     "us_per_launch_note": "timed step / 32: the commit of the step's rows counts against the launches",
                     "by_kv_len": by_len,
                     "us_per_launch_alone": alone_us, "kv_len": len_mean,
                     "frac_alone": (B * (2 * Hkv * D * 2 * lens_now) + 2 * B * Hq * D * 2) / (alone_us * 1e-6) / 1e9 / peak,
                     "alg_bytes_per_launch": alg_bytes, "traffic": None},
    }
    if world == 1 and not args.no_aux:
        # side numbers of the multi-token kernels on the same record: PARD verify (16 x 9 tokens over 1033
        # cached) and a 512-token prefill chunk over 4096 cached, 4 layers each
        mgr.release()
        del mgr, graph, graph_e2e
        torch.cuda.empty_cache()
        aux = {}
        for wl in ("verify", "prefill"):
            a = aux_measure(wl, layers=4, head_dim=D, past=3584, steps=32)
            aux[wl] = {"us_per_launch": a["us_per_launch"], "hbm_frac_of_measured": a["hbm"]["frac_of_measured"],
                       "us_best_single_launch": a["us_best_single_launch"],
                       "tflops": a["tensor"]["achieved_tflops"],
                       "tensor_frac_of_measured_burst": a["tensor"]["frac_of_measured_burst"],
                       "tensor_frac_of_measured_sustained": a["tensor"]["frac_of_measured_sustained"],
                       "tflops_best_single_launch": a["tensor"]["achieved_tflops_best_single_launch"],
                       "best_single_launch_frac_of_measured_burst": a["tensor"]["best_single_launch_frac_of_measured_burst"],
                       "shape": f"B={a['batch']} q_len={a['q_len']} kv_len={a['kv_len']}"}
        lin = linear_measure()["shapes"]
        aux["linear_skinny"] = {k: {"us": v["us_skinny"], "us_library_gemm": v["us_library"], "hbm_frac_of_measured": v["frac_skinny"],
                                    "library_gemm_hbm_frac_of_measured": v["frac_library"]} for k, v in lin.items()}
        line["aux"] = {"verify_us": aux["verify"]["us_per_launch"], "prefill_tflops": aux["prefill"]["tflops"],
                       "linear_skinny": aux["linear_skinny"],
                       "prefill_tflops_best_single_launch": aux["prefill"]["tflops_best_single_launch"],
                       "verify": aux["verify"], "prefill": aux["prefill"]}
    if world == 1 and not args.no_cpu_baseline:
        tps, _, cpu_cores, kind, sample = cpu_reference_line(steps=8)
        line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": cpu_cores, "kind": kind, "sample": sample}
    traffic_file = os.path.join(ROOT, "profiles", "attn_decode_traffic.json")
    if os.path.exists(traffic_file):
        try:
            t = json.load(open(traffic_file))
            # DRAM bytes of the captured launch scale with the rows a launch streams: whole pages, the
            # partly filled last page in boxes of 16 rows
            rows_now = B * ((int(len_mean) + 15) // 16) * 16
            line["roofline"]["traffic"] = t["dram_bytes_per_launch"] * rows_now / t["rows_per_launch"]
        except Exception:
            pass
    print(json.dumps(line), flush=True)


def run_aux(args):
    print(json.dumps(aux_measure(args.workload, min(args.layers, 8), args.head_dim, args.past, args.steps)), flush=True)


def aux_measure(workload, layers, head_dim, past, steps):
    """Side measurements of the multi-token attention kernels: PARD verify (config 4: batch 16, 9 query
    tokens over 1033 cached) and a 512-token prefill chunk (config 3: batch 8, 512 queries over a cache
    of `past` + 512).  Times the attention kernel alone over `layers` layers visited round-robin (cold
    L2) and returns the figures as a dict."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    dev = torch.device("cuda", torch.cuda.current_device())
    L = layers
    Hq, Hkv, D = CFG["hq"], CFG["hkv"], head_dim
    if workload == "verify":
        B, S, kv_len = 16, 9, 1024 + 9
    else:
        B, S, kv_len = 8, 512, past + 512

    class Cfg:
        num_hidden_layers = L

    g = torch.Generator(device=dev).manual_seed(7)
    mgr = KVCacheManager(Cfg(), kv_len + 64, KVCacheType.BMC)
    for l in range(L):
        done = 0
        while done < kv_len:
            n = min(512, kv_len - done)
            k = torch.randn(B, Hkv, n, D, device=dev, generator=g, dtype=torch.float32).bfloat16()
            mgr[l].update_cache(k, k.flip(2), concat_dim=2)
            done += n
    q = torch.randn(B, S, Hq, D, device=dev, generator=g, dtype=torch.float32).bfloat16().transpose(1, 2)
    mha = MultiHeadAttention()
    hs = [(mgr[l].key, mgr[l].value) for l in range(L)]
    out = torch.empty(B, S, Hq, D, dtype=torch.bfloat16, device=dev).transpose(1, 2)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for l in range(L):
            mha(q, *hs[l], out=out)
    side.synchronize()
    graph = torch.cuda.CUDAGraph()          # back-to-back launches without host gaps
    with torch.cuda.graph(graph, stream=side):
        for l in range(L):
            mha(q, *hs[l], out=out)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(1, steps // 8)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (reps * L)
    # The loop above runs for tens of milliseconds at full load: the SM clock settles where the power cap
    # puts it, which is what MEASURED_PEAKS calls "sustained".  Its "burst" figure is the best of ten single
    # GEMMs; the like-for-like number here is the best of ten single launches (cold L2: a different layer
    # each time), each timed on its own.
    singles = []
    with torch.cuda.stream(side):
        for n in range(10):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            mha(q, *hs[n % L], out=out)
            b.record()
            b.synchronize()
            singles.append(a.elapsed_time(b) * 1e3)
    us_best = min(singles)
    mgr.pool.check_status()
    alg_bytes = B * (2 * Hkv * D * 2 * kv_len) + 2 * B * Hq * D * 2 * S
    # causal: query s sees past + s + 1 keys; 4 flops per (query head, key, dim)
    flops = sum(4 * Hq * D * (kv_len - S + s + 1) for s in range(S)) * B
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(
        os.path.join(ROOT, "MEASURED_PEAKS.json")) else {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": 1590.0}
    line = {"workload": workload, "batch": B, "q_len": S, "kv_len": kv_len, "head_dim": D,
            "page_tokens": mgr.pool.page_tokens, "us_per_launch": us,
            "hbm": {"alg_bytes": alg_bytes, "achieved_gbs": alg_bytes / us / 1e3,
                    "frac_of_measured": alg_bytes / us / 1e3 / peaks["hbm_gbs"]},
            "us_best_single_launch": us_best,
            "tensor": {"flops": flops, "achieved_tflops": flops / us / 1e6,
                       "frac_of_measured_burst": flops / us / 1e6 / peaks["bf16_tflops"],
                       "frac_of_measured_sustained": flops / us / 1e6 / peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]),
                       "achieved_tflops_best_single_launch": flops / us_best / 1e6,
                       "best_single_launch_frac_of_measured_burst": flops / us_best / 1e6 / peaks["bf16_tflops"],
                       "note": "achieved_tflops: back-to-back launches for tens of ms (clock under the power cap, compare "
                               "with the sustained GEMM figure); best_single_launch: best of 10 launches timed one by one "
                               "(compare with the burst GEMM figure, itself a best of 10)"}}
    mgr.release()
    return line


def run_rope(args):
    """Side measurement of the fused RoPE + append kernel against the unfused sequence it replaces
    (table lookup + elementwise rotation as torch ops, then the plain append), on the decode shape
    (batch 32, 1 token: launch-bound) and on 2048 new tokens per sequence (batch 8: long enough for the
    GPU, not the host, to set the pace), 32/8 heads of 128.  Layers are visited round-robin.  Prints
    one JSON line."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import RotaryEmbedding
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    L = min(args.layers, 8)
    Hq, Hkv, D = CFG["hq"], CFG["hkv"], args.head_dim
    rope = RotaryEmbedding({"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192}, D, 131072, 500000.0).to(dev)

    class Cfg:
        num_hidden_layers = L

    out = {"workload": "rope_append", "head_dim": D, "layers": L}
    g = torch.Generator(device=dev).manual_seed(11)
    for tag, B, n, past in (("decode_b32_n1", 32, 1, 512), ("prefill_b8_n2048", 8, 2048, 0)):
        reps = 10
        qkv = torch.randn(B, n, (Hq + 2 * Hkv) * D, device=dev, generator=g, dtype=torch.float32).bfloat16()
        q = qkv[..., : Hq * D].view(B, n, Hq, D)
        k = qkv[..., Hq * D: (Hq + Hkv) * D].view(B, n, Hkv, D)
        v = qkv[..., (Hq + Hkv) * D:].view(B, n, Hkv, D)
        pos = (torch.arange(n, device=dev) + past).expand(B, n)
        rows = rope.table_rows(pos)
        q_out = torch.empty(B, n, Hq, D, dtype=torch.bfloat16, device=dev)
        times = {}
        for mode in ("fused", "unfused"):
            mgr = KVCacheManager(Cfg(), past + n * (reps + 4) + 64, KVCacheType.BMC)
            if past:
                old = torch.zeros(B, Hkv, past, D, dtype=torch.bfloat16, device=dev)
                for l in range(L):
                    mgr[l].update_cache(old, old, concat_dim=2)

            def step():
                for l in range(L):
                    if mode == "fused":
                        mgr[l].update_cache_rope(q, k, v, rows, rope, query_out=q_out)
                    else:
                        qr, kr = rope(q, pos)(query=q.transpose(1, 2), key=k.transpose(1, 2))
                        mgr[l].update_cache(kr, v.transpose(1, 2), concat_dim=2)
            for _ in range(3):
                step()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                step()
            e1.record()
            torch.cuda.synchronize()
            mgr.pool.check_status()
            times[mode] = e0.elapsed_time(e1) * 1e3 / (reps * L)
            mgr.release()
        alg = B * n * (Hq + 2 * Hkv) * D * 2 * 2 + B * n * rope.rotary_dim * 4
        out[tag] = {"us_fused": times["fused"], "us_unfused_torch_rope_plus_append": times["unfused"],
                    "alg_bytes": alg, "fused_gbs": alg / times["fused"] / 1e3,
                    "note": "host-launched, one call per layer (launch overhead included on both sides)"}
    print(json.dumps(out), flush=True)


def run_device_loop(args):
    """Side measurement of the whole decode step of a Llama-3.1-8B-shaped model (random weights,
    `--layers` of its 32 layers; projections/MLP/LM head are cuBLAS through torch, the KV path is this
    library): tokens/s of the host-driven loop (one Python step per token, a host synchronisation for
    the argmax) against the device-resident loop (one CUDA graph per token).  Batch 32, 512-token
    prompt, 64 new tokens.  Prints one JSON line."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.llm.device_loop import GreedyDeviceLoop
    from pace_b200.llm.models.llama import LlamaForCausalLM
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)

    class Cfg:
        hidden_size, intermediate_size, num_hidden_layers = 4096, 14336, min(args.layers, 32)
        num_attention_heads, num_key_value_heads, vocab_size = 32, 8, 128256
        max_position_embeddings, rope_theta, rms_norm_eps, pad_token_id = 8192, 500000.0, 1e-5, 0
        rope_scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                        "original_max_position_embeddings": 8192}

    cfg = Cfg()
    with torch.device(dev):
        model = LlamaForCausalLM(cfg).to(torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(5)
    with torch.no_grad():
        for p_ in model.parameters():
            if p_.dim() >= 2:
                p_.normal_(0.0, 0.02, generator=g)
    model.eval()
    B, P0, N = CFG["batch"], CFG["prompt"], 64
    prompts = torch.randint(1, cfg.vocab_size, (B, P0), device=dev, generator=g)
    res = {}
    for mode in ("host_loop", "device_loop"):
        mgr = KVCacheManager(cfg, P0 + N + 8, KVCacheType.BMC)
        with torch.inference_mode():
            done = 0
            while done < P0:                       # chunked prefill keeps the activations small
                n = min(128, P0 - done)
                pos = (torch.arange(n, device=dev) + done).expand(B, n)
                hidden = model.model.forward_tokens(prompts[:, done: done + n], mgr, pos)
                done += n
            nxt = model.lm_head(hidden[:, -1:]).float().argmax(dim=-1).reshape(B)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            if mode == "host_loop":
                pos = torch.full((B, 1), P0, device=dev)
                for _ in range(N):
                    hidden = model.model.forward_tokens(nxt.reshape(B, 1), mgr, pos)
                    nxt = model.lm_head(hidden)[:, -1].float().argmax(dim=-1)
                    _ = nxt.tolist()               # the reference's loop hands the tokens to Python every step
                    pos = pos + 1
            else:
                loop = GreedyDeviceLoop(model, mgr, nxt, torch.full((B,), P0, device=dev), max_new_tokens=N)
                t0 = time.perf_counter()           # graph capture is set-up, not decoding
                loop.run(poll_every=32)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
        mgr.pool.check_status()
        steps = N if mode == "host_loop" else N - 1
        res[mode] = {"ms_per_token_step": dt * 1e3 / steps, "tokens_per_s": B * steps / dt}
        mgr.release()
    res.update({"workload": "device_loop", "model": f"llama-3.1-8b shape, {cfg.num_hidden_layers} layers, random weights",
                "batch": B, "prompt": P0, "new_tokens": N})
    print(json.dumps(res), flush=True)


def run_serving(args):
    """Side measurement of the two serving loops over one paged pool on a Llama-3.1-8B-shaped model
    (`--layers` of its layers, default 8 here; random weights): 48 requests with prompt lengths drawn
    log-uniformly from 64..4096 tokens (seeded), 32 new tokens each, 16 cache slots, a pool of 24576
    tokens.  Wave admission (a wave is admitted, runs to the end, is released) against continuous
    batching (a finished request's slot and pages go to the next one at once).  Prints one JSON line."""
    import math
    from pace_b200.llm.models.llama import LlamaForCausalLM
    from pace_b200.llm.serving import ContinuousBatcher, WaveServer
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)

    class Cfg:
        hidden_size, intermediate_size, num_hidden_layers = 4096, 14336, min(args.layers, 8)
        num_attention_heads, num_key_value_heads, vocab_size = 32, 8, 128256
        max_position_embeddings, rope_theta, rms_norm_eps, pad_token_id = 8192, 500000.0, 1e-5, 0
        rope_scaling = None

    cfg = Cfg()
    with torch.device(dev):
        model = LlamaForCausalLM(cfg).to(torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(6)
    with torch.no_grad():
        for p_ in model.parameters():
            if p_.dim() >= 2:
                p_.normal_(0.0, 0.02, generator=g)
    model.eval()
    gc = torch.Generator().manual_seed(7)
    lens = [int(math.exp(math.log(64) + float(torch.rand(1, generator=gc)) * math.log(4096 / 64))) for _ in range(48)]
    prompts = [torch.randint(1, cfg.vocab_size, (n,), generator=gc) for n in lens]
    new = 32
    res = {"workload": "serving", "model": f"llama-3.1-8b shape, {cfg.num_hidden_layers} layers, random weights",
           "requests": len(prompts), "prompt_tokens": sum(lens), "new_tokens_each": new, "slots": 16,
           "pool_tokens": 24576}
    for name, cls in (("wave", WaveServer), ("continuous", ContinuousBatcher)):
        srv = cls(model, pool_tokens=24576, max_batch=16, max_seq_len=4096 + new + 64, prefill_chunk=512)
        srv.run(prompts[:4], 4)                      # warm-up (allocator, cuBLAS handles)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs, st = srv.run(prompts, new)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        assert all(len(o) == new for o in outs)
        res[name] = {"seconds": dt, "total_tokens_per_s": (sum(lens) + new * len(prompts)) / dt,
                     "output_tokens_per_s": new * len(prompts) / dt,
                     "steps_or_waves": getattr(st, "steps", None) or getattr(st, "waves", None)}
    print(json.dumps(res), flush=True)


def linear_measure():
    """Side measurement of the weight-streaming linear kernel on the four layer shapes of a
    Llama-3.1-8B-shaped decode step (batch 32): fused QKV 4096 -> 6144, o_proj 4096 -> 4096, gate+up
    4096 -> 28672, down 14336 -> 4096.  Several weight matrices per shape are visited round-robin inside
    one CUDA graph (more bytes than L2 holds, every launch streams from DRAM; consecutive launches overlap
    the way they do inside a decoder layer); the same chain through the library GEMM beside it."""
    from pace_b200.ops.linear import linear_skinny as linear
    dev = torch.device("cuda", torch.cuda.current_device())
    peak, _ = measured_hbm_peak()
    g = torch.Generator(device=dev).manual_seed(3)
    out = {"workload": "linear", "tokens": 32, "peak_gbs": peak, "shapes": {}}
    for name, n, k in (("qkv", 6144, 4096), ("o_proj", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)):
        copies = max(2, int(400e6 // (n * k * 2)) + 1)
        ws = [(torch.randn(n, k, device=dev, generator=g, dtype=torch.float32) * 0.02).bfloat16() for _ in range(copies)]
        x = torch.randn(32, k, device=dev, generator=g, dtype=torch.float32).bfloat16()
        res = {}
        for impl, fn in (("skinny", linear), ("library", torch.nn.functional.linear)):
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for w in ws:
                    fn(x, w)
            side.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=side):
                for w in ws:
                    fn(x, w)
            for _ in range(3):
                gr.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 10
            e0.record()
            for _ in range(reps):
                gr.replay()
            e1.record()
            torch.cuda.synchronize()
            res[impl] = e0.elapsed_time(e1) * 1e3 / (reps * copies)
            del gr
        nbytes = n * k * 2 + 32 * (n + k) * 2
        out["shapes"][name] = {"n": n, "k": k, "us_skinny": res["skinny"], "us_library": res["library"],
                               "gbs_skinny": nbytes / res["skinny"] / 1e3, "frac_skinny": nbytes / res["skinny"] / 1e3 / peak,
                               "frac_library": nbytes / res["library"] / 1e3 / peak}
        del ws
        torch.cuda.empty_cache()
    return out


def run_linear(args):
    print(json.dumps(linear_measure()), flush=True)


def main():
    # stdout carries the JSON line and nothing else: whatever native libraries print to file descriptor 1
    # (NCCL's version banner on some ranks) goes to stderr, Python's own prints keep the real stdout
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(real_stdout, "w", buffering=1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-aux", action="store_true", help="skip the verify / prefill side numbers of the bench line")
    ap.add_argument("--no-sweep", action="store_true", help="profiling aid: skip the timed blocks at other cache lengths")
    ap.add_argument("--layers", type=int, default=CFG["n_layers"],
                    help="profiling aid: fewer layers = less device memory; the bench line is only valid at 32")
    ap.add_argument("--workload", default="decode", choices=["decode", "verify", "prefill", "rope_append", "device_loop", "serving", "linear"],
                    help="decode = the bench line; verify / prefill = side measurements of the multi-token kernels")
    ap.add_argument("--past", type=int, default=3584, help="prefill side measurement: tokens cached before the chunk")
    ap.add_argument("--head-dim", type=int, default=128, choices=[64, 128])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    CFG["n_layers"] = args.layers
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    global RANK_CORES
    RANK_CORES = pin_rank_to_cores(local_rank, world)
    if args.workload in ("rope_append", "device_loop", "serving", "linear"):
        if rank == 0:
            {"rope_append": run_rope, "device_loop": run_device_loop, "serving": run_serving,
             "linear": run_linear}[args.workload](args)
        return
    if args.workload != "decode":
        if rank == 0:
            run_aux(args)
        return
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
