"""CUDA-graph replay of a fixed-shape decode step.

The reference pays Python and operator-dispatch overhead on every layer of every
generated token (pace/llm/generator.py:715-818 drives pace/llm/models/llama.py:155-165).
On a GPU that overhead exceeds the kernels' run time, so the launch sequence of one
step - per layer: K/V append, attention - is recorded once and replayed.  This works
because block tables and lengths are device-resident: the same recorded launches see
the lengths grow from replay to replay, and the page reservation kernel of the first
layer runs every step.
"""
from typing import Callable, Sequence

import torch

from pace_b200.llm.cache import KVCacheManager


class StepGraph:
    """Records ``step_fn()`` (which appends ``n_new`` tokens per sequence to every layer of
    ``manager`` and attends) and replays it.

    ``step_fn`` must use fixed tensors for its inputs and outputs; refill them between
    replays.  Two eager warm-up steps run first (they append real tokens).  With deferred
    appends (``manager.defer_appends``) the step ends with ``manager.commit()``: the recorded
    sequence is then the layers' attention launches back to back and one batched append.
    """

    def __init__(self, manager: KVCacheManager, step_fn: Callable[[], object], n_new: int = 1, warmup: int = 2):
        self.manager = manager
        self.n_new = n_new
        self.stream = torch.cuda.Stream()
        self.replays_with_reserve = 0    # replays that needed the page reservation kernel
        self.graph = torch.cuda.CUDAGraph()
        inner = step_fn

        def step_fn():
            out = inner()
            manager.commit()
            return out
        manager.static_launch = True
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            for _ in range(warmup):
                step_fn()
        self.stream.synchronize()
        manager.capturing = True
        try:
            with torch.cuda.graph(self.graph, stream=self.stream):
                self.result = step_fn()
            # The same step without the page reservation kernel, for the replays (63 of 64 with 64-token
            # pages) in which the host mirror shows that no sequence reaches a new page and no page is
            # shared after a beam gather: the reservation is a one-block kernel outside the chain of
            # programmatic dependent launches, and the whole step waits for it.
            self.graph_no_reserve = torch.cuda.CUDAGraph()
            manager.skip_reserve = True
            with torch.cuda.graph(self.graph_no_reserve, stream=self.stream, pool=self.graph.pool()):
                second = step_fn()
            if isinstance(self.result, torch.Tensor) and isinstance(second, torch.Tensor) \
                    and second.data_ptr() != self.result.data_ptr():
                raise ValueError("StepGraph: step_fn must write its result into a fixed tensor (pass out= to the "
                                 "attention op); it returned a different buffer on the second recording")
        finally:
            manager.capturing = False
            manager.skip_reserve = False

    def replay(self):
        """One more step.  The host mirror of lengths / pages advances as the kernels will."""
        grow = self.manager.advance_host_mirror(self.n_new)
        if grow or self.manager.pool.shared_pages:
            self.replays_with_reserve += 1
            self.graph.replay()
        else:
            self.graph_no_reserve.replay()
        return self.result
