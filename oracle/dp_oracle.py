"""What a data-parallel run must produce, from independent oracle replicas (TEST INFRASTRUCTURE).

The reference trains on one GPU; data parallelism is defined here from its single-process step
(ti_net.py:17-32): every rank runs the reference's forward / backward on its contiguous shard of the batch
with its own activation / error exponents, the int32 weight-gradient accumulators of all ranks are summed
(exactly, as int64), and ONE ``weight_update`` (ti_torch.py:16-21) is applied to every replica.  Used by the
multi-GPU tests and by the benchmark's parity check of the exchange route it is about to time.
"""
import numpy as np

from . import niti_oracle as O


def expected(cfg, weights, wexps, batches, spans, seed, mu=5, dropout=True):
    """``batches``: [(float32 images [B,3,32,32], labels [B])] of the GLOBAL batch per step; ``spans``: the ranks'
    [lo, hi) shards.  Returns ({(step, lo): (int8 logits, exponent)}, final weights per layer)."""
    nets = [O.Net(cfg, weights, wexps, dropout=dropout, mu=mu, seed=seed) for _ in spans]
    want = {}
    for step, (x, t) in enumerate(batches):
        grads = []
        for net, (lo, hi) in zip(nets, spans):
            x8, xe = O.float_to_int8(x[lo:hi])
            out, e = net.forward(np.ascontiguousarray(x8.transpose(0, 2, 3, 1)), xe, step=step, sample_offset=lo)
            want[(step, lo)] = (out, e)
            grads.append(net.backward(t[lo:hi], step=step, sample_offset=lo, update=False))
        summed = {i: sum(np.asarray(g[i], dtype=np.int64) for g in grads) for i in range(len(weights))}
        for net in nets:
            net.apply_grads(summed, step=step)
    return want, [np.array(w) for w in nets[0].w]
