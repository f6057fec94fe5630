"""Data-parallel training on a GPU with two processes, each with half of a batch.  Default mode: the ranks equal two
independent oracle replicas on the shards whose int32 gradients are summed before ONE update.  Global-exact mode: they
equal one oracle on the whole batch, bit for bit.  Both ranks share cuda:0 and talk over gloo (host-side collectives
only; no kernel of one rank waits for a kernel of the other)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from oracle import dp_oracle, niti_oracle as O
from tests.golden.make_golden import synth_images, xavier_exp

pytestmark = pytest.mark.gpu

CFG = [128, "M", 128, "M", 512, "M"]
GLOBAL_BATCH, STEPS, SEED = 8, 2, 31


def _data():
    rng = np.random.default_rng(SEED)
    shapes, cin = [], 3
    for c in CFG:
        if c != "M":
            shapes.append((c, 3, 3, cin))
            cin = c
    shapes.append((10, 8192))
    weights = [rng.integers(-127, 128, size=s).astype(np.int8) for s in shapes]
    batches = [(synth_images(rng, GLOBAL_BATCH), rng.integers(0, 10, size=GLOBAL_BATCH)) for _ in range(STEPS)]
    return shapes, weights, [xavier_exp(s) for s in shapes], batches


def _worker(rank, world, port, q, exact):
    import torch.distributed as dist
    from niti_b200 import ti_torch, ti_vgg
    from niti_b200.dp import shard_range
    from niti_b200.trainer import Trainer
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shapes, weights, wexps, batches = _data()
        ti_torch.GRAD_BITWIDTH, ti_torch.TRAINING = 5, True
        model = ti_vgg.TiVGG_cifar(list(CFG), dropout=True, fuse_relu=True)
        for l, w, e in zip(model.weighted_layers(), weights, wexps):
            l.weight = torch.from_numpy(w).to("cuda:0")
            l.weight_exp = ti_torch.exp_tensor(e, "cuda:0")
        lo, hi = shard_range(GLOBAL_BATCH, rank, world)
        tr = Trainer(model, hi - lo, "cuda:0", rank=rank, world=world, use_graph=not exact, seed=SEED, global_exact=exact,
                     warmup_steps=1, sample_offset=lo)
        logits = []
        for x, t in batches:
            out, exp = tr.step(torch.from_numpy(x[lo:hi].copy()).pin_memory(), torch.from_numpy(t[lo:hi].copy()).pin_memory())
            tr.sync()
            logits.append((out.numpy().copy(), int(exp)))
        q.put((rank, lo, hi, logits, [l.weight.cpu().numpy().tobytes() for l in model.weighted_layers()]))
    finally:
        ti_torch.GLOBAL_MAX_GROUP = None
        dist.destroy_process_group()


def _run_ranks(exact):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, exact)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return results


def test_two_ranks_equal_one_process_on_the_whole_batch():
    results = _run_ranks(True)
    shapes, weights, wexps, batches = _data()
    net = O.Net(CFG, weights, wexps, dropout=True, mu=5, seed=SEED)
    want = []
    for step, (x, t) in enumerate(batches):
        x8, xe = O.float_to_int8(x)
        out, e = net.forward(np.ascontiguousarray(x8.transpose(0, 2, 3, 1)), xe, step=step)
        net.backward(t, step=step)
        want.append((out, e))
    for rank, lo, hi, logits, wbytes in results:
        for step in range(STEPS):
            assert np.array_equal(logits[step][0], want[step][0][lo:hi]), f"rank {rank} step {step}: logits"
            assert logits[step][1] == want[step][1]
        for i, b in enumerate(wbytes):
            assert b == net.w[i].tobytes(), f"rank {rank}: weights of layer {i}"


def test_two_ranks_equal_independent_replicas_with_summed_gradients():
    """The default data-parallel step (graph replay included): rank-local shifts, one exact int32 sum, one update."""
    results = _run_ranks(False)
    shapes, weights, wexps, batches = _data()
    spans = sorted((lo, hi) for _, lo, hi, _, _ in results)
    want, want_w = dp_oracle.expected(CFG, weights, wexps, batches, spans, SEED)
    for rank, lo, hi, logits, wbytes in results:
        for step in range(STEPS):
            assert np.array_equal(logits[step][0], want[(step, lo)][0]), f"rank {rank} step {step}: logits"
            assert logits[step][1] == want[(step, lo)][1]
        for i, b in enumerate(wbytes):
            assert b == want_w[i].tobytes(), f"rank {rank}: weights of layer {i}"
