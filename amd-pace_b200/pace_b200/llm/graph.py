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
    replays.  Two eager warm-up steps run first (they append real tokens).
    """

    def __init__(self, manager: KVCacheManager, step_fn: Callable[[], object], n_new: int = 1, warmup: int = 2):
        self.manager = manager
        self.n_new = n_new
        self.stream = torch.cuda.Stream()
        self.graph = torch.cuda.CUDAGraph()
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
        finally:
            manager.capturing = False

    def replay(self):
        """One more step.  The host mirror of lengths / pages advances as the kernels will."""
        counts = [self.n_new] * len(self.manager.slots)
        for c in self.manager.cache_objects:
            c._host_account(counts)
        self.graph.replay()
        return self.result
