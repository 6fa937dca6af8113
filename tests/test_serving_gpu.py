"""Wave admission on a shared long-lived pool: ragged chunked prefill, decode, page recycling."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class Cfg:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def _model():
    from pace_b200.llm.models.llama import LlamaForCausalLM, random_init_
    cfg = Cfg(hidden_size=256, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=1, vocab_size=97, max_position_embeddings=1024, rope_theta=500000.0,
              rms_norm_eps=1e-5, pad_token_id=0)
    return random_init_(LlamaForCausalLM(cfg).to(torch.bfloat16), 3).to(DEV).eval()


def test_waves_recycle_pages_and_match_single_request_runs():
    from pace_b200.llm.serving import WaveServer
    model = _model()
    g = torch.Generator().manual_seed(8)
    lens = [300, 37, 129, 64, 511, 5, 200]
    prompts = [torch.randint(1, 97, (n,), generator=g) for n in lens]
    new = 6
    small = WaveServer(model, pool_tokens=64 * 14, max_batch=4, max_seq_len=600, prefill_chunk=128)
    free0 = small.pool.query()[1]
    outs, stats = small.run(prompts, new)
    assert stats.waves >= 3 and sum(stats.wave_sizes) == len(prompts)       # the pool forced several waves
    assert stats.prompt_tokens == sum(lens) and stats.output_tokens == new * len(prompts)
    assert all(len(o) == new for o in outs)
    bits, free1 = small.pool.query()
    assert bits == 0 and free1 == free0 and small.pool.host_free_pages == free0   # every page came back
    # one request at a time on a roomy pool: same first token (later ones may flip on bf16 ties)
    big = WaveServer(model, pool_tokens=64 * 64, max_batch=1, max_seq_len=600, prefill_chunk=512)
    agree = 0
    for i, p in enumerate(prompts):
        o, _ = big.run([p], new)
        agree += int(o[0][0] == outs[i][0])
    assert agree >= len(prompts) - 1


def test_request_larger_than_the_pool_is_refused():
    from pace_b200.llm.serving import WaveServer
    server = WaveServer(_model(), pool_tokens=64 * 3, max_batch=2, max_seq_len=600)
    with pytest.raises(RuntimeError, match="does not fit the KV pool"):
        server.run([torch.randint(1, 97, (400,))], 4)


def test_continuous_batching_serves_every_request_and_returns_every_page():
    """Requests join and leave a fixed set of slots step by step; what each one generates starts with
    the token a run of that request alone produces, and the pool ends as full as it began."""
    from pace_b200.llm.serving import ContinuousBatcher, WaveServer
    model = _model()
    g = torch.Generator().manual_seed(9)
    lens = [300, 37, 129, 64, 511, 5, 200, 90, 33]
    prompts = [torch.randint(1, 97, (n,), generator=g) for n in lens]
    new = 7
    cb = ContinuousBatcher(model, pool_tokens=64 * 16, max_batch=4, max_seq_len=600, prefill_chunk=128)
    free0 = cb.pool.query()[1]
    outs, stats = cb.run(prompts, new)
    assert all(o is not None and len(o) == new for o in outs)
    assert stats.prompt_tokens == sum(lens) and stats.output_tokens == new * len(prompts)
    assert 2 <= stats.max_running <= 4
    bits, free1 = cb.pool.query()
    assert bits == 0 and free1 == free0 and cb.pool.host_free_pages == free0 and cb.reserved_pages == 0
    assert all(n == 0 for n in cb.manager[0].seq_lens)
    big = WaveServer(model, pool_tokens=64 * 64, max_batch=1, max_seq_len=600, prefill_chunk=512)
    agree = sum(int(big.run([p], new)[0][0][0] == outs[i][0]) for i, p in enumerate(prompts))
    assert agree >= len(prompts) - 1
    # a second run on the same batcher reuses the recycled slots and pages
    outs2, _ = cb.run(prompts[:3], new)
    assert [o[0] for o in outs2] == [o[0] for o in outs[:3]]
    with pytest.raises(RuntimeError, match="does not fit the KV pool"):
        cb.run([torch.randint(1, 97, (590,))], 600)


def test_router_in_front_of_the_continuous_batcher():
    """Requests arrive concurrently at the batch-window router (the reference's router logic without its HTTP
    hops, pace/server/router.py:112-225) and are served by the continuous batcher on the paged pool: every
    request gets its own number of tokens, and the same tokens as when the batcher is called directly."""
    import asyncio
    from pace_b200.llm.router import BatchWindowRouter, CompletionRequest, batcher_backend
    from pace_b200.llm.serving import ContinuousBatcher
    model = _model()
    g = torch.Generator().manual_seed(10)
    lens, new = [120, 9, 260, 64, 33, 75], [5, 3, 7, 1, 4, 6]
    prompts = [torch.randint(1, 97, (n,), generator=g) for n in lens]
    cb = ContinuousBatcher(model, pool_tokens=64 * 16, max_batch=4, max_seq_len=400, prefill_chunk=128)
    direct, _ = cb.run(prompts, max(new))

    async def main():
        r = BatchWindowRouter(batcher_backend(cb), ["llama"], max_batch_size=4, batch_timeout=0.2)
        await r.start()
        outs = await asyncio.gather(*(r.complete(CompletionRequest("llama", p.tolist(), max_tokens=n))
                                      for p, n in zip(prompts, new)))
        await r.stop()
        return r.batches, outs
    batches, outs = asyncio.run(main())
    assert batches == [4, 2]
    for i, o in enumerate(outs):
        ids = o["choices"][0]["token_ids"]
        assert len(ids) == new[i] and o["usage"]["prompt_tokens"] == lens[i], o["choices"][0]["text"]
        assert ids[0] == direct[i][0]                         # the first token never depends on batch mates
    assert cb.pool.query()[0] == 0 and cb.reserved_pages == 0
