"""The data-parallel update over peer memory (niti_dp_update_i8) on two GPUs: two processes, one GPU each, NCCL for
the rendezvous only.  The ranks must equal two independent oracle replicas on the shards whose int32 gradients are
summed before ONE update, exactly like the all-reduce route.  Needs two GPUs with peer access: skipped otherwise."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from oracle import dp_oracle
from tests.test_gpu_dp_exact import CFG, GLOBAL_BATCH, SEED, STEPS, _data

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    import torch.distributed as dist
    from niti_b200 import ops, ti_torch, ti_vgg
    from niti_b200.dp import shard_range
    from niti_b200.trainer import Trainer
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    tr = None
    try:
        shapes, weights, wexps, batches = _data()
        ti_torch.GRAD_BITWIDTH, ti_torch.TRAINING = 5, True
        model = ti_vgg.TiVGG_cifar(list(CFG), dropout=True, fuse_relu=True)
        for l, w, e in zip(model.weighted_layers(), weights, wexps):
            l.weight = torch.from_numpy(w).to(dev)
            l.weight_exp = ti_torch.exp_tensor(e, dev)
        lo, hi = shard_range(GLOBAL_BATCH, rank, world)
        tr = Trainer(model, hi - lo, dev, rank=rank, world=world, use_graph=True, seed=SEED, warmup_steps=1, peer_update=True,
                     sample_offset=lo)
        assert tr.peer is not None
        logits = []
        for x, t in batches:
            out, exp = tr.step(torch.from_numpy(x[lo:hi].copy()).pin_memory(), torch.from_numpy(t[lo:hi].copy()).pin_memory())
            tr.sync()
            logits.append((out.numpy().copy(), int(exp)))
        bucket_clear = int(tr.bucket.flat.abs().max().item()) == 0
        q.put((rank, lo, hi, logits, [l.weight.cpu().numpy().tobytes() for l in model.weighted_layers()], bucket_clear))
    finally:
        if tr is not None:
            tr.close()
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_memory_update_equals_summed_gradient_update():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    shapes, weights, wexps, batches = _data()
    spans = sorted((lo, hi) for _, lo, hi, _, _, _ in results)
    want, want_w = dp_oracle.expected(CFG, weights, wexps, batches, spans, SEED)
    for rank, lo, hi, logits, wbytes, bucket_clear in results:
        assert bucket_clear, f"rank {rank}: the gradient bucket is not zero after the update"
        for step in range(STEPS):
            assert np.array_equal(logits[step][0], want[(step, lo)][0]), f"rank {rank} step {step}: logits"
            assert logits[step][1] == want[(step, lo)][1]
        for i, b in enumerate(wbytes):
            assert b == want_w[i].tobytes(), f"rank {rank}: weights of layer {i}"
