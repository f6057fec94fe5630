"""The data-parallel update over peer memory (niti_dp_update_i8) on two GPUs: two processes, one GPU each, NCCL for
the rendezvous only.  The ranks must equal two independent oracle replicas on the shards whose int32 gradients are
summed before ONE update, exactly like the all-reduce route.  Needs two GPUs with peer access: skipped otherwise."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from oracle import dp_oracle, niti_oracle as O
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
        ti_torch.WGRAD_GROUP = 2  # this net has two layers with side-stream gradients: a full group, so their slices are PUSHED
        model = ti_vgg.TiVGG_cifar(list(CFG), dropout=True, fuse_relu=True)
        for l, w, e in zip(model.weighted_layers(), weights, wexps):
            l.weight = torch.from_numpy(w).to(dev)
            l.weight_exp = ti_torch.exp_tensor(e, dev)
        lo, hi = shard_range(GLOBAL_BATCH, rank, world)
        tr = Trainer(model, hi - lo, dev, rank=rank, world=world, use_graph=True, seed=SEED, warmup_steps=1, peer_update=True,
                     sample_offset=lo, push_gradients=True)
        assert tr.peer is not None
        pushed_seen = []
        logits = []
        for x, t in batches:
            out, exp = tr.step(torch.from_numpy(x[lo:hi].copy()).pin_memory(), torch.from_numpy(t[lo:hi].copy()).pin_memory())
            tr.sync()
            logits.append((out.numpy().copy(), int(exp)))
            pushed_seen.append(sorted(tr._pushed or []))
        assert pushed_seen[0] == [1, 2, 3], pushed_seen  # both later conv layers and the classifier went by copy engine
        bucket_clear = int(tr.bucket.flat.abs().max().item()) == 0
        final_w = [l.weight.cpu().numpy().tobytes() for l in model.weighted_layers()]
        # a checkpoint loaded AFTER graph capture and after the weights moved into the peer-visible arena: the values
        # are copied into that memory, so the next step trains on them on every rank
        sd, wi = {}, 0
        for idx, l in enumerate(model.forward_layers):
            if hasattr(l, "weight"):
                sd[f"layers.{idx}.weight"] = torch.from_numpy(weights[wi])
                sd[f"layers.{idx}.weight_exp"] = torch.tensor(float(wexps[wi]))  # the reference's checkpoints hold floats
                wi += 1
        model.load_state_dict(sd)
        tr.resync()
        x, t = batches[0]
        out, exp = tr.step(torch.from_numpy(x[lo:hi].copy()).pin_memory(), torch.from_numpy(t[lo:hi].copy()).pin_memory())
        tr.sync()
        reloaded = (out.numpy().copy(), int(exp), [l.weight.cpu().numpy().tobytes() for l in model.weighted_layers()])
        q.put((rank, lo, hi, logits, final_w, bucket_clear, reloaded))
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
    spans = sorted((lo, hi) for _, lo, hi, _, _, _, _ in results)
    want, want_w = dp_oracle.expected(CFG, weights, wexps, batches, spans, SEED)
    # the step after the reload: the initial weights again, batch 0, but the random bits of step STEPS
    nets = [O.Net(CFG, weights, wexps, dropout=True, mu=5, seed=SEED) for _ in spans]
    grads, again = [], {}
    for net, (lo, hi) in zip(nets, spans):
        x8, xe = O.float_to_int8(batches[0][0][lo:hi])
        again[lo] = net.forward(np.ascontiguousarray(x8.transpose(0, 2, 3, 1)), xe, step=STEPS, sample_offset=lo)
        grads.append(net.backward(batches[0][1][lo:hi], step=STEPS, sample_offset=lo, update=False))
    summed = {i: sum(np.asarray(g[i], dtype=np.int64) for g in grads) for i in range(len(shapes))}
    nets[0].apply_grads(summed, step=STEPS)
    for rank, lo, hi, logits, wbytes, bucket_clear, reloaded in results:
        assert np.array_equal(reloaded[0], again[lo][0]) and reloaded[1] == again[lo][1], f"rank {rank}: logits after the reload"
        for i, b in enumerate(reloaded[2]):
            assert b == nets[0].w[i].tobytes(), f"rank {rank}: weights of layer {i} after the reload"
        assert bucket_clear, f"rank {rank}: the gradient bucket is not zero after the update"
        for step in range(STEPS):
            assert np.array_equal(logits[step][0], want[(step, lo)][0]), f"rank {rank} step {step}: logits"
            assert logits[step][1] == want[(step, lo)][1]
        for i, b in enumerate(wbytes):
            assert b == want_w[i].tobytes(), f"rank {rank}: weights of layer {i}"
