"""One model instance per GPU, requests sharded by sequence, no collective on the hot path.

The reference's only parallelism is multi-instance data parallelism: N worker processes, each with
a full model and pinned to its own CPU cores, pull batch indices from a shared queue and report
(tokens, seconds) (pace/utils/worker.py:11-100, examples/multi_instance_pace.py:201-274).  The same
shape here, with a GPU per worker: ``Worker`` binds its process to one CUDA device (and, optionally,
a CPU core list) before ``init_func`` builds the model and its KV pool there, waits for ``start()``,
then runs ``target_func``.  No tensor crosses a process boundary - only request indices in and
(tokens, seconds) tuples out - so nothing crosses NVLink either.
"""
import multiprocessing as mp
import os
from typing import Callable, List, Optional, Sequence, Tuple


def bind_device_and_cores(device_index: Optional[int], cores: Optional[Sequence[int]]) -> None:
    """What the reference's ``thread_bind`` (csrc/core/threading.cpp:17-31) does for CPU cores, plus
    the choice of GPU: must run in the worker process before CUDA is initialised there."""
    if cores:
        try:
            os.sched_setaffinity(0, set(int(c) for c in cores))
        except (AttributeError, OSError):
            pass
    if device_index is not None:
        import torch
        if torch.cuda.is_available():
            torch.cuda.set_device(device_index)


class Worker:
    def __init__(self, worker_id: int, cores_list, init_func: Callable, init_args: tuple, target_func: Callable,
                 target_args: tuple, device_index: Optional[int] = None, ctx=None):
        self.worker_id = worker_id
        self.cores_list = cores_list
        self.device_index = device_index
        ctx = ctx or mp.get_context("spawn")       # CUDA does not survive fork
        self.condition = ctx.Condition()
        self.flag = ctx.Value("i", 0)
        self.init_func, self.init_args = init_func, init_args
        self.target_func, self.target_args = target_func, target_args
        self.process = ctx.Process(target=_worker_main, args=(self,))
        self.process.start()

    def start(self) -> None:
        with self.condition:
            self.flag.value = 1
            self.condition.notify()

    def join(self, timeout: Optional[float] = None) -> None:
        self.process.join(timeout)

    @property
    def exitcode(self):
        return self.process.exitcode


def _worker_main(w: Worker) -> None:
    bind_device_and_cores(w.device_index, w.cores_list)
    state = w.init_func(*w.init_args)
    with w.condition:
        while w.flag.value == 0:
            w.condition.wait()
    if state is not None:
        w.target_func(state, *w.target_args)
    else:
        w.target_func(*w.target_args)


class MultipleProcesses:
    def __init__(self, workers: List[Worker]):
        self.workers = workers

    def run(self) -> None:
        for w in self.workers:
            w.start()

    def join(self, timeout: Optional[float] = None) -> None:
        for w in self.workers:
            w.join(timeout)

    def failed(self) -> List[int]:
        """Workers that exited abnormally (``Dispatcher`` hands out again what they held)."""
        return [w.worker_id for w in self.workers if w.exitcode not in (0, None)]

    def alive(self) -> List[int]:
        return [w.worker_id for w in self.workers if w.exitcode is None]


def serve_items(worker_id: int, ip_queue, op_queue, fn: Callable) -> None:
    """A worker's loop under a ``Dispatcher``: take an item, say so, work on it, report the result."""
    while True:
        item = ip_queue.get()
        if item is None:
            return
        op_queue.put(("take", worker_id, item, None))
        op_queue.put(("done", worker_id, item, fn(item)))


class Dispatcher:
    """Hands work items (request shards, batch indices) to the workers through a queue and collects
    one result per item.  The reference fills a queue and joins it
    (examples/multi_instance_pace.py:204-238), which waits for ever when a worker dies with an item in
    hand; here every wait has a time limit, dead workers are noticed between polls, and the items a
    dead worker had taken are handed out again to the survivors.  An item lost between the queue and
    its worker's announcement is found when the survivors fall idle.  Results are kept once per item
    (the first to arrive), so handing an item out twice is harmless."""

    def __init__(self, pool: MultipleProcesses, ip_queue, op_queue, items: Sequence, poll_s: float = 0.5):
        self.pool, self.ip, self.op = pool, ip_queue, op_queue
        self.items = list(items)
        self.poll_s = poll_s
        self.requeued: List = []

    def run(self, timeout_s: Optional[float] = None) -> dict:
        import queue as _queue
        import time as _time
        for it in self.items:
            self.ip.put(it)
        results: dict = {}
        holding = {w.worker_id: set() for w in self.pool.workers}
        buried = set()
        deadline = None if timeout_s is None else _time.monotonic() + timeout_s
        idle_polls = 0
        while len(results) < len(self.items):
            try:
                kind, wid, item, res = self.op.get(timeout=self.poll_s)
                idle_polls = 0
                if kind == "take":
                    holding[wid].add(item)
                else:
                    holding[wid].discard(item)
                    results.setdefault(item, res)
                continue
            except _queue.Empty:
                idle_polls += 1
            for wid in self.pool.failed():
                if wid in buried:
                    continue
                buried.add(wid)
                for item in sorted(holding[wid]):
                    if item not in results:
                        self.requeued.append(item)
                        self.ip.put(item)
                holding[wid].clear()
            alive = self.pool.alive()
            if not alive:
                raise RuntimeError(f"every worker has exited with {len(self.items) - len(results)} items undone")
            # survivors idle, nothing announced, items still undone: one was lost on its way to a worker that died
            if buried and idle_polls >= 4 and not any(holding[w] for w in alive):
                for item in self.items:
                    if item not in results and item not in self.requeued:
                        self.requeued.append(item)
                        self.ip.put(item)
                idle_polls = 0
            if deadline is not None and _time.monotonic() > deadline:
                raise TimeoutError(f"{len(self.items) - len(results)} items undone after {timeout_s} s")
        for _ in self.pool.alive():
            self.ip.put(None)
        return results


# ---- request sharding and throughput accounting -----------------------------------------------

def shard_requests(n_requests: int, world: int, rank: int) -> range:
    """Contiguous, balanced shard of request indices for one rank (sizes differ by at most one)."""
    base, extra = divmod(n_requests, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def fill_queue(queue, n_batches: int, n_workers: int) -> None:
    """Batch indices followed by one stop marker per worker (examples/multi_instance_pace.py:204-214)."""
    for i in range(n_batches):
        queue.put(i)
    for _ in range(n_workers):
        queue.put(None)


def box_throughput(results: Sequence[Tuple[int, float]], instances: int) -> Tuple[float, float]:
    """(sum of tokens / slowest instance's time, the reference's sum(tokens)/sum(time) x instances)
    (examples/multi_instance_pace.py:260-274)."""
    tokens = sum(t for t, _ in results)
    slowest = max(s for _, s in results)
    total_s = sum(s for _, s in results)
    return tokens / slowest, tokens / total_s * instances


def reduce_step_time(ms: float, group=None) -> float:
    """Max over ranks of a per-rank time, on whatever backend the process group uses."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return ms
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
