"""Batch-window router in front of a serving loop, without a transport.

The reference's router (pace/server/router.py:112-191) is an HTTP front end: requests in the OpenAI
``/v1/completions`` shape wait in an asyncio queue; a worker takes the first one, keeps collecting for
``batch_timeout`` seconds or until ``max_batch_size`` requests are there, refuses requests whose model
differs from the batch's, sends the batch to the inference server and resolves each request's future
with its output; the endpoint wraps that output in a ``text_completion`` record (router.py:200-225).

This module keeps that logic - the queue, the batch window, the mixed-model refusal, the record - and
replaces the two HTTP hops by calls: ``complete()`` is what the endpoint would await, ``serve_batch`` is
whatever runs a batch (``ContinuousBatcher.run`` / ``WaveServer.run`` of pace_b200.llm.serving behind a
small adapter, see ``batcher_backend``).  Tokenisation is not part of the KV-cache path, so prompts and
outputs are token ids (``prompt`` is a list of ids, ``choices[0].token_ids`` the completion); sampling
parameters are carried in the request as in the reference but only greedy decoding is served
(``temperature`` 0).  Each request gets its own ``max_tokens`` (the reference applies the first request's
generation arguments to the whole batch, router.py:153-168; with equal arguments the two agree).
"""
import asyncio
import time
import uuid
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Union

MIXED_MODELS = "Error: Mixed models in batch."


@dataclass
class CompletionRequest:
    """Fields and defaults of the reference's request model (router.py:46-54); ``prompt`` holds token ids."""
    model: str
    prompt: List[int]
    max_tokens: int = 100
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 50
    seed: Optional[int] = None
    stop: Optional[Union[str, List[str]]] = None


@dataclass
class _Queued:
    req: CompletionRequest
    future: "asyncio.Future" = field(default=None)


class BatchWindowRouter:
    """``serve_batch(prompts, max_new_per_request) -> outputs`` runs one batch (token id lists in, token id
    lists out, same order); it is called in a worker thread so that requests keep arriving meanwhile."""

    def __init__(self, serve_batch: Callable[[List[List[int]], List[int]], List[List[int]]], models: Sequence[str],
                 max_batch_size: int = 4, batch_timeout: float = 0.5):
        if max_batch_size < 1 or batch_timeout < 0:
            raise ValueError("max_batch_size must be positive and batch_timeout non-negative")
        self.serve_batch = serve_batch
        self.models = set(models)
        self.max_batch_size = max_batch_size
        self.batch_timeout = batch_timeout
        self.queue: "asyncio.Queue[_Queued]" = None
        self.batches: List[int] = []          # sizes of the batches sent so far
        self._worker: Optional["asyncio.Task"] = None

    async def start(self):
        self.queue = asyncio.Queue()
        self._worker = asyncio.get_running_loop().create_task(self._batch_worker())

    async def stop(self):
        if self._worker is not None:
            self._worker.cancel()
            try:
                await self._worker
            except asyncio.CancelledError:
                pass
            self._worker = None

    async def complete(self, req: CompletionRequest) -> dict:
        """What the reference's ``/v1/completions`` handler does with one request (router.py:200-225)."""
        if self._worker is None:
            return {"error": "Inference server not ready. Please try again later."}
        if req.model not in self.models:
            return {"error": f"Requested model '{req.model}' is not available."}
        if req.temperature > 0:
            return {"error": "Only greedy decoding (temperature 0) is served."}
        item = _Queued(req, asyncio.get_running_loop().create_future())
        await self.queue.put(item)
        out = await item.future
        if isinstance(out, str):              # the batch worker's error text, as in the reference
            text, ids, finish = out, [], "error"
        else:
            text, ids, finish = None, list(out), "length" if len(out) >= req.max_tokens else "stop"
        return {"id": f"cmpl-{uuid.uuid4().hex[:24]}", "object": "text_completion", "created": int(time.time()),
                "model": req.model,
                "choices": [{"index": 0, "text": text, "token_ids": ids, "logprobs": None, "finish_reason": finish}],
                "usage": {"prompt_tokens": len(req.prompt), "completion_tokens": len(ids),
                          "total_tokens": len(req.prompt) + len(ids)}}

    async def _batch_worker(self):
        loop = asyncio.get_running_loop()
        while True:
            first = await self.queue.get()    # wait for at least one request, then open the batch window
            batch = [first]
            start = time.monotonic()
            while len(batch) < self.max_batch_size:
                remaining = self.batch_timeout - (time.monotonic() - start)
                if remaining <= 0:
                    break
                try:
                    batch.append(await asyncio.wait_for(self.queue.get(), timeout=remaining))
                except asyncio.TimeoutError:
                    break
            model = batch[0].req.model        # every request of a batch must name the same model
            run = []
            for item in batch:
                if item.req.model != model:
                    item.future.set_result(MIXED_MODELS)
                else:
                    run.append(item)
            self.batches.append(len(run))
            try:
                outputs = await loop.run_in_executor(None, self.serve_batch, [list(i.req.prompt) for i in run],
                                                     [i.req.max_tokens for i in run])
            except Exception as e:            # the reference answers empty strings when the server call fails
                outputs = [f"Error: {e}"] * len(run)
            for item, out in zip(run, outputs):
                if not item.future.done():
                    item.future.set_result(out)


def batcher_backend(batcher):
    """Adapter from a serving loop of pace_b200.llm.serving (``run(prompts, max_new)``, prompts as 1-D host
    tensors of token ids) to ``serve_batch``: the batch runs for the largest ``max_tokens`` asked and every
    request keeps its own count."""
    import torch

    def serve_batch(prompts: List[List[int]], max_new: List[int]) -> List[List[int]]:
        outputs, _ = batcher.run([torch.tensor(p, dtype=torch.long) for p in prompts], max(max_new))
        return [list(o)[:n] for o, n in zip(outputs, max_new)]
    return serve_batch
