"""Host side of the multi-GPU shape (one instance per GPU, sharded requests) on CPU: 2 gloo ranks,
2 worker processes, a worker that dies.  No GPU, no collective on any data path."""
import multiprocessing as mp
import os
import time

import pytest
import torch

from pace_b200.utils.worker import (Dispatcher, MultipleProcesses, Worker, box_throughput, fill_queue,
                                    reduce_step_time, serve_items, shard_requests)


def test_shards_cover_every_request_once():
    for n in (0, 1, 7, 256, 1000):
        for world in (1, 2, 4, 8):
            got = [i for r in range(world) for i in shard_requests(n, world, r)]
            assert got == list(range(n))
            sizes = [len(shard_requests(n, world, r)) for r in range(world)]
            assert max(sizes) - min(sizes) <= 1


def test_box_throughput_definitions():
    agg, ref_style = box_throughput([(1000, 2.0), (1000, 4.0)], instances=2)
    assert agg == 2000 / 4.0 and abs(ref_style - 2000 / 6.0 * 2) < 1e-9


def _rank_main(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mine = list(shard_requests(11, world, rank))
    slow = reduce_step_time(10.0 * (rank + 1))           # the slowest rank sets the time
    n = torch.tensor([len(mine)])
    dist.all_reduce(n)
    out.put((rank, mine, slow, int(n.item())))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_reduce():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(out.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert res[0][1] + res[1][1] == list(range(11))
    assert res[0][2] == res[1][2] == 20.0
    assert res[0][3] == res[1][3] == 11


def _init(worker_id):
    return {"id": worker_id}


def _serve(state, ip_queue, op_queue, die_on):
    while True:
        item = ip_queue.get()
        if item is None:
            ip_queue.task_done()
            return
        if item == die_on and state["id"] == 0:
            os._exit(17)                                   # a worker process lost between steps
        op_queue.put((state["id"], item, 100, 0.01))
        ip_queue.task_done()


@pytest.mark.timeout(300)
def test_workers_pull_batches_and_a_dead_worker_is_noticed():
    ctx = mp.get_context("spawn")
    ip, op = ctx.JoinableQueue(), ctx.Queue()
    workers = [Worker(i, None, _init, (i,), _serve, (ip, op, 3), device_index=None, ctx=ctx) for i in range(2)]
    fill_queue(ip, 8, 2)
    pool = MultipleProcesses(workers)
    pool.run()
    pool.join(60)
    got = []
    while not op.empty():
        got.append(op.get())
    done = sorted(b for _, b, _, _ in got)
    failed = pool.failed()
    if failed:                                             # worker 0 met batch 3 and died
        assert failed == [0] and 3 not in done
        missing = sorted(set(range(8)) - set(done))
        assert 3 in missing                                # what the dispatcher has to re-queue
    else:                                                  # worker 1 happened to take batch 3
        assert done == list(range(8))
    agg, _ = box_throughput([(t, s) for _, _, t, s in got], instances=2)
    assert agg > 0


def _serve_dispatched(state, ip_queue, op_queue, second_item_taken):
    seen = []

    def work(item):
        seen.append(item)
        if state["id"] == 0 and len(seen) == 2:
            second_item_taken.set()
            time.sleep(0.3)                                # (its announcement of the item has left the process by now)
            os._exit(17)                                   # worker 0 is lost with its second item in hand
        if state["id"] == 1 and len(seen) == 1:
            second_item_taken.wait(60)                     # the survivor does not empty the queue before that happens
        time.sleep(0.05)
        return (state["id"], item * item)
    serve_items(state["id"], ip_queue, op_queue, work)


@pytest.mark.timeout(300)
def test_dispatcher_hands_a_dead_workers_item_out_again():
    """A worker process dies on the host between two items (exit, no GPU involved): the dispatcher
    notices, hands the item it held to the survivor, and every item gets its one result; no wait is
    without a time limit."""
    ctx = mp.get_context("spawn")
    ip, op, taken = ctx.Queue(), ctx.Queue(), ctx.Event()
    workers = [Worker(i, None, _init, (i,), _serve_dispatched, (ip, op, taken), device_index=None, ctx=ctx) for i in range(2)]
    pool = MultipleProcesses(workers)
    pool.run()
    disp = Dispatcher(pool, ip, op, list(range(8)), poll_s=0.2)
    t0 = time.monotonic()
    results = disp.run(timeout_s=120)
    assert time.monotonic() - t0 < 60
    pool.join(30)
    assert sorted(results) == list(range(8))
    assert all(results[i][1] == i * i for i in range(8))
    assert pool.failed() == [0]
    assert len(disp.requeued) >= 1                          # what worker 0 held when it died
    assert all(results[i][0] == 1 for i in disp.requeued)   # ... was served by the survivor


def _serve_nothing(state, ip_queue, op_queue):
    os._exit(3)


@pytest.mark.timeout(300)
def test_dispatcher_gives_up_when_every_worker_is_gone():
    ctx = mp.get_context("spawn")
    ip, op = ctx.Queue(), ctx.Queue()
    workers = [Worker(i, None, _init, (i,), _serve_nothing, (ip, op), device_index=None, ctx=ctx) for i in range(2)]
    pool = MultipleProcesses(workers)
    pool.run()
    with pytest.raises(RuntimeError, match="every worker has exited"):
        Dispatcher(pool, ip, op, [0, 1, 2], poll_s=0.2).run(timeout_s=60)
    pool.join(30)
