"""The batch-window router against the reference router's rules (pace/server/router.py:112-225): the window,
the batch-size limit, the mixed-model refusal, the OpenAI-style record.  No GPU: the batch is "served" by a
function that echoes each prompt reversed."""
import asyncio

import pytest

from pace_b200.llm.router import MIXED_MODELS, BatchWindowRouter, CompletionRequest


def _echo(prompts, max_new):
    return [list(reversed(p))[:n] for p, n in zip(prompts, max_new)]


def _run(coro):
    return asyncio.run(coro)


def test_requests_inside_the_window_share_a_batch_and_the_size_is_capped():
    async def main():
        r = BatchWindowRouter(_echo, ["m"], max_batch_size=4, batch_timeout=0.3)
        await r.start()
        reqs = [CompletionRequest("m", [i, i + 1, i + 2], max_tokens=2) for i in range(6)]
        outs = await asyncio.gather(*(r.complete(q) for q in reqs))
        await r.stop()
        return r.batches, outs
    batches, outs = _run(main())
    assert batches == [4, 2]                                   # six requests at once: a full batch, then the rest
    for i, o in enumerate(outs):
        assert o["object"] == "text_completion" and o["model"] == "m" and o["id"].startswith("cmpl-")
        assert o["choices"][0]["token_ids"] == [i + 2, i + 1]  # each request's own max_tokens
        assert o["choices"][0]["finish_reason"] == "length"
        assert o["usage"] == {"prompt_tokens": 3, "completion_tokens": 2, "total_tokens": 5}


def test_a_late_request_opens_a_new_window():
    async def main():
        r = BatchWindowRouter(_echo, ["m"], max_batch_size=8, batch_timeout=0.1)
        await r.start()
        a = asyncio.ensure_future(r.complete(CompletionRequest("m", [1, 2])))
        await asyncio.sleep(0.4)                               # the first window has closed and been served
        b = await r.complete(CompletionRequest("m", [3, 4]))
        a = await a
        await r.stop()
        return r.batches, a, b
    batches, a, b = _run(main())
    assert batches == [1, 1]
    assert a["choices"][0]["token_ids"] == [2, 1] and b["choices"][0]["token_ids"] == [4, 3]
    assert a["choices"][0]["finish_reason"] == "stop"          # fewer tokens than max_tokens


def test_mixed_models_unknown_models_sampling_and_a_failing_backend():
    def broken(prompts, max_new):
        raise RuntimeError("pool exhausted")

    async def main():
        r = BatchWindowRouter(_echo, ["m", "n"], max_batch_size=4, batch_timeout=0.2)
        await r.start()
        first, second = await asyncio.gather(r.complete(CompletionRequest("m", [1])), r.complete(CompletionRequest("n", [2])))
        unknown = await r.complete(CompletionRequest("x", [1]))
        sampled = await r.complete(CompletionRequest("m", [1], temperature=0.7))
        await r.stop()
        idle = await r.complete(CompletionRequest("m", [1]))
        rb = BatchWindowRouter(broken, ["m"], max_batch_size=2, batch_timeout=0.05)
        await rb.start()
        failed = await rb.complete(CompletionRequest("m", [1]))
        await rb.stop()
        return first, second, unknown, sampled, idle, failed
    first, second, unknown, sampled, idle, failed = _run(main())
    assert first["choices"][0]["token_ids"] == [1]
    assert second["choices"][0]["text"] == MIXED_MODELS and second["choices"][0]["finish_reason"] == "error"
    assert unknown == {"error": "Requested model 'x' is not available."}
    assert "greedy" in sampled["error"]
    assert idle == {"error": "Inference server not ready. Please try again later."}
    assert failed["choices"][0]["text"] == "Error: pool exhausted"


def test_constructor_checks():
    with pytest.raises(ValueError):
        BatchWindowRouter(_echo, ["m"], max_batch_size=0)
