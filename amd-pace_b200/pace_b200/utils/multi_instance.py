"""Multi-instance data-parallel serving: one model instance per GPU, requests sharded by sequence.

    python -m pace_b200.utils.multi_instance --gpus 8 --requests-per-gpu 256 --min-len 256 --max-len 32768

The shape of the reference's examples/multi_instance_pace.py:139-274: N worker processes, each with
its own model and KV pool on its own device, serve their share of the requests; only request
indices go in and (tokens, seconds) come out; whole-box throughput = all tokens over the slowest
instance's time.  Prompts are seeded random token ids with log-uniform lengths, weights are random
N(0, 0.02) of the given shape: there is no dataset or checkpoint behind it.
"""
import argparse
import json
import math
import multiprocessing as mp
import os
import time

from pace_b200.utils.worker import (Dispatcher, MultipleProcesses, Worker, box_throughput, serve_items,
                                    shard_requests)


class _Cfg:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def make_prompt_lengths(n: int, lo: int, hi: int, seed: int):
    import torch
    g = torch.Generator().manual_seed(seed)
    u = torch.rand(n, generator=g)
    return [int(round(math.exp(math.log(lo) + float(x) * (math.log(hi) - math.log(lo))))) for x in u]


def _init_instance(rank, args):
    import torch
    from pace_b200.llm.models.llama import LlamaForCausalLM, random_init_
    from pace_b200.llm.serving import ContinuousBatcher, WaveServer
    cfg = _Cfg(hidden_size=args.hidden, intermediate_size=args.ffn, num_hidden_layers=args.layers,
               num_attention_heads=args.heads, num_key_value_heads=args.kv_heads, vocab_size=args.vocab,
               max_position_embeddings=args.max_len + args.new_tokens + 64, rope_theta=500000.0, rms_norm_eps=1e-5,
               pad_token_id=0)
    dev = torch.device("cuda", torch.cuda.current_device())
    model = random_init_(LlamaForCausalLM(cfg).to(torch.bfloat16), seed=1).to(dev).eval()
    cls = ContinuousBatcher if args.scheduler == "continuous" else WaveServer
    server = cls(model, pool_tokens=args.pool_tokens, max_batch=args.max_batch,
                 max_seq_len=args.max_len + args.new_tokens, prefill_chunk=512)
    return {"rank": rank, "server": server, "cfg": cfg}


def _serve(state, args, world, in_queue, out_queue):
    """Takes request shards from the queue until the stop marker: normally its own one, and those of
    instances that died when the dispatcher hands them out again."""
    import torch
    rank = state["rank"]
    lengths = make_prompt_lengths(args.requests_per_gpu * world, args.min_len, args.max_len, seed=7)

    def one_shard(shard):
        mine = shard_requests(len(lengths), world, shard)
        g = torch.Generator().manual_seed(100 + shard)
        prompts = [torch.randint(1, args.vocab, (lengths[i],), generator=g) for i in mine]
        t0 = time.perf_counter()
        _, stats = state["server"].run(prompts, args.new_tokens)
        dt = time.perf_counter() - t0
        # (wave admission separates prefill from decode time; continuous batching interleaves them)
        return (rank, stats.output_tokens, stats.prompt_tokens, dt, getattr(stats, "decode_s", dt),
                getattr(stats, "waves", None) or stats.steps, getattr(stats, "kv_bytes_read", 0),
                getattr(stats, "admissions", None) or getattr(stats, "waves", 0))
    serve_items(rank, in_queue, out_queue, one_shard)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--requests-per-gpu", type=int, default=256)
    ap.add_argument("--min-len", type=int, default=256)
    ap.add_argument("--max-len", type=int, default=32768)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--pool-tokens", type=int, default=1 << 20)
    ap.add_argument("--max-batch", type=int, default=256)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--scheduler", choices=["continuous", "wave"], default="continuous")
    ap.add_argument("--timeout-s", type=float, default=3600.0, help="give up when the shards are not served by then")
    args = ap.parse_args()
    ctx = mp.get_context("spawn")
    inq, out = ctx.Queue(), ctx.Queue()
    # every instance keeps its own slice of the host cores (the reference gives each instance
    # physical_cores // instances, examples/multi_instance_pace.py:201-238)
    try:
        allowed = sorted(os.sched_getaffinity(0))
    except AttributeError:
        allowed = []
    per = len(allowed) // args.gpus if args.gpus else 0
    cores = [allowed[r * per:(r + 1) * per] if per else None for r in range(args.gpus)]
    workers = [Worker(r, cores[r], _init_instance, (r, args), _serve, (args, args.gpus, inq, out), device_index=r, ctx=ctx)
               for r in range(args.gpus)]
    pool = MultipleProcesses(workers)
    pool.run()
    # one work item per instance: its shard of the requests; a dead instance's shard goes to a survivor
    disp = Dispatcher(pool, inq, out, list(range(args.gpus)), poll_s=1.0)
    by_shard = disp.run(timeout_s=args.timeout_s)
    pool.join(60)
    # per instance: tokens and seconds summed over the shards it served
    per_rank = {}
    for r in by_shard.values():
        acc = per_rank.setdefault(r[0], [r[0], 0, 0, 0.0, 0.0, 0, 0, 0])
        for i in range(1, 8):
            acc[i] += r[i]
    results = [tuple(v) for v in per_rank.values()]
    agg, ref_style = box_throughput([(r[1], r[3]) for r in results], args.gpus)
    decode_tps = sum(r[1] for r in results) / max(r[4] for r in results)
    print(json.dumps({"n_gpus": args.gpus, "requests": args.requests_per_gpu * args.gpus,
                      "output_tokens": sum(r[1] for r in results), "prompt_tokens": sum(r[2] for r in results),
                      "box_output_tokens_per_s": agg, "reference_style_tokens_per_s": ref_style,
                      "box_decode_tokens_per_s": decode_tps, "scheduler": args.scheduler,
                      "box_total_tokens_per_s": sum(r[1] + r[2] for r in results) / max(r[3] for r in results),
                      "steps_or_waves_per_gpu": [r[5] for r in sorted(results)],
                      "admission_steps_per_gpu": [r[7] for r in sorted(results)],
                      "seconds_per_gpu": [round(r[3], 2) for r in sorted(results)],
                      "kv_read_gb_per_s_per_gpu": [round(r[6] / r[3] / 1e9, 1) for r in sorted(results)],
                      "layers": args.layers,
                      "failed_workers": pool.failed(), "requeued_shards": disp.requeued}))


if __name__ == "__main__":
    main()
