"""Data-parallel host logic on CPU ranks (gloo, world size 2): sharding, the flat int32 gradient
bucket, its all-reduce and replica consistency, with the oracle standing in for the kernels."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from niti_b200.dp import GradBucket, shard_range
from oracle import niti_oracle as O
from tests.golden.make_golden import synth_images, xavier_exp

CFG = [16, "M", 32, "M", 512, "M"]
GLOBAL_BATCH = 6
SEED = 99


def _setup():
    rng = np.random.default_rng(SEED)
    shapes, cin = [], 3
    for c in CFG:
        if c != "M":
            shapes.append((c, 3, 3, cin))
            cin = c
    shapes.append((10, 8192))
    weights = [rng.integers(-127, 128, size=s).astype(np.int8) for s in shapes]
    x = synth_images(rng, GLOBAL_BATCH)
    tgt = rng.integers(0, 10, size=GLOBAL_BATCH)
    return shapes, weights, [xavier_exp(s) for s in shapes], x, tgt


def _shard_grads(shapes, weights, wexps, x, tgt, lo, hi):
    net = O.Net(CFG, weights, wexps, dropout=True, mu=5, seed=SEED)
    x8, xe = O.float_to_int8(x[lo:hi])
    net.forward(np.ascontiguousarray(x8.transpose(0, 2, 3, 1)), xe, step=0, sample_offset=lo)
    return net, net.backward(tgt[lo:hi], step=0, sample_offset=lo, update=False)


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shapes, weights, wexps, x, tgt = _setup()
        lo, hi = shard_range(GLOBAL_BATCH, rank, world)
        net, grads = _shard_grads(shapes, weights, wexps, x, tgt, lo, hi)
        bucket = GradBucket(shapes, "cpu")
        for i, v in enumerate(bucket.views):
            v.copy_(torch.from_numpy(grads[i].astype(np.int32)))
        bucket.allreduce_()
        summed = {i: v.numpy().astype(np.int64) for i, v in enumerate(bucket.views)}
        net.apply_grads(summed, step=0)
        q.put((rank, bucket.checksum(), [w.tobytes() for w in net.w]))
    finally:
        dist.destroy_process_group()


def test_shard_range_covers_batch():
    for gb in (1, 5, 128, 257):
        for world in (1, 2, 3, 8):
            spans = [shard_range(gb, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == gb
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1


def test_bucket_views_are_aligned_and_disjoint():
    b = GradBucket([(3, 3), (10, 7), (2,)], "cpu")
    assert all(o % 4 == 0 for o in b.offsets)
    for i, v in enumerate(b.views):
        v.fill_(i + 1)
    assert [int(v.sum()) for v in b.views] == [9, 140, 6]


def test_two_rank_step_matches_replica_sum():
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=240) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # replicas agree with each other ...
    assert results[0][1] == results[1][1] and results[0][2] == results[1][2]
    # ... and with "independent replicas on the shards + int64 sum + one update"
    shapes, weights, wexps, x, tgt = _setup()
    total = None
    for r in range(world):
        lo, hi = shard_range(GLOBAL_BATCH, r, world)
        net, g = _shard_grads(shapes, weights, wexps, x, tgt, lo, hi)
        total = g if total is None else {i: total[i] + g[i] for i in g}
    net.apply_grads(total, step=0)
    assert [w.tobytes() for w in net.w] == results[0][2]


def test_comm_groups_cover_bucket_in_backward_order():
    shapes = [(128, 3, 3, 3), (128, 3, 3, 128), (256, 3, 3, 128), (256, 3, 3, 256), (512, 3, 3, 256), (512, 3, 3, 512), (10, 8192)]
    b = GradBucket(shapes, "cpu")
    groups = b.comm_groups(min_bytes=4 << 20)
    # last layers first, contiguous, disjoint, covering the whole flat buffer, no small message except possibly the last
    assert groups[0][1] == len(shapes) - 1 and groups[-1][0] == 0
    assert all(g[0] <= g[1] for g in groups)
    assert all(a[0] == b_[1] + 1 for a, b_ in zip(groups, groups[1:]))
    assert groups[0][3] == b.flat.numel() and groups[-1][2] == 0
    assert all(a[2] == b_[3] for a, b_ in zip(groups, groups[1:]))
    assert all((g[3] - g[2]) * 4 >= 4 << 20 for g in groups[:-1])
    assert GradBucket([(4, 4)], "cpu").comm_groups() == [(0, 0, 0, 16)]


def test_bucket_adopts_external_memory():
    """The peer-memory exchange keeps the bucket inside an arena the other ranks can address."""
    shapes = [(128, 3, 3, 3), (10, 8192), (5, 7)]
    n = GradBucket.numel_for(shapes)
    arena = torch.zeros(n + 8, dtype=torch.int32)
    b = GradBucket(shapes, "cpu", flat=arena[4:4 + n])
    assert b.flat.data_ptr() == arena.data_ptr() + 16 and b.flat.numel() == n
    b.views[2].fill_(3)
    assert int(arena.sum()) == 3 * 35 and all(o % 4 == 0 for o in b.offsets)
