"""Training-step driver: host buffers in, one integer training step on the GPU, logits out.

``Trainer.step`` is the public call a user makes per batch: it copies the float images and
labels from pinned host memory, runs TiNet.forward + TiNet.backward (loss, error
back-propagation, weight gradients, integer update) and copies the int8 logits and their
exponent back.  After two eager steps the device work is captured in CUDA graphs and replayed,
because a step is ~100 short kernels and would otherwise be bound by launch overhead.
With a process group of more than one rank the batch is sharded (one process per GPU).  Ranks on
different GPUs of one node exchange through one kernel over peer memory that sums the gradients
slice by slice, updates and stores the new weights into every replica (all in the same graph);
otherwise the int32 gradient bucket is all-reduced by NCCL between the backward graph and the
update graph, and every rank applies the same update.
"""
import warnings

import torch
import torch.distributed as dist

from . import ops, ti_torch
from .dp import GradBucket
from .peer import PeerArena, peers_on_one_node


class StepResult:
    """What ``Trainer.step`` returns: unpacks as ``(logits, exponent)`` (pinned host tensors) and carries the
    event after which they are valid, so a caller can read step i's logits while step i+1 is already running.
    ``wait`` also looks at the kernels' status word as it stood after this step and raises if one of their bounded
    waits had run out (the trainer then refuses further steps, see ``Trainer.reset_exchange``)."""

    def __init__(self, out, exp, done, status=None, owner=None):
        self.out, self.exp, self.done, self.status, self.owner = out, exp, done, status, owner

    def __iter__(self):
        return iter((self.out, self.exp))

    def wait(self):
        self.done.synchronize()
        if self.status is not None and int(self.status[0]) != 0:
            msg = ops.status_message(self.status.tolist())
            if self.owner is not None:
                self.owner._failed = msg
            raise RuntimeError(msg)
        return self.out, self.exp


class Trainer:
    """One integer training step per ``step`` call; see the module docstring.

    Data parallel over peer memory: the ranks' update kernels wait for one another, with a limit of 4 s per
    barrier.  Ranks must therefore enter their steps within 4 s of each other: after anything that may hold one
    rank back longer (evaluation, a checkpoint, a long host pause) call ``resync()`` on every rank before the
    next step.  A wait that does run out is reported by ``StepResult.wait`` / ``sync``; from then on ``step``
    raises, because the replicas may no longer agree: restore the weights on every rank (``load_state_dict``)
    and call ``reset_exchange()`` (collective) to continue.

    ``sample_offset``: global index of this rank's first sample (``dp.shard_range(global_batch, rank, world)[0]``);
    default ``rank * local_batch``, which is right for equal shards.  It keys the per-sample random bits.
    """

    def __init__(self, model, local_batch, device, group=None, rank=0, world=1, use_graph=True, seed=0,
                 in_shape=(3, 32, 32), warmup_steps=2, keep_gradients=False, wgrad_side_stream=True,
                 global_exact=False, peer_update="auto", sample_offset=None, push_gradients="auto"):
        self.model, self.device, self.group = model, torch.device(device), group
        self.rank, self.world, self.use_graph = rank, world, use_graph
        self.local_batch = local_batch
        self.keep_gradients = keep_gradients
        # global-exact mode: every activation / error maximum is MAX-reduced over the ranks, so the ranks together
        # compute bit for bit what one process computes on the whole batch (eager execution, two-pass requantisation)
        self.global_exact = bool(global_exact) and world > 1
        ti_torch.GLOBAL_MAX_GROUP = (group if group is not None else True) if self.global_exact else None
        if self.global_exact:
            self.use_graph = use_graph = False
        # weight-gradient kernels run beside the error-backward kernels on a second stream (joined before the update)
        self.side = torch.cuda.Stream(device=self.device) if (wgrad_side_stream and not keep_gradients) else None
        self.layers = model.weighted_layers()
        # With more than one rank the exchange is either ONE kernel per rank over peer memory (reduce-scatter of the
        # gradients, update of the own slice, new weights stored into every replica: ops.dp_update) when the ranks sit
        # on different GPUs of one node, or an NCCL all-reduce of the bucket followed by the update launch.
        self.peer = None
        # peer-memory route: a group of weight gradients that is complete long before the backward pass ends (and the
        # classifier's) is PUSHED to the slices' owners by copy-engine transfers under the rest of the backward pass; the
        # update kernel then sums local memory for those layers and reads the peers' buckets only for the late ones
        # ("auto": two ranks only.  Measured on B200s, VGG-small-7, 128 images per GPU: 0.4766 -> 0.460-0.468 ms per step on
        # two GPUs; on four the update kernel gets 20 us shorter (reduce phase 25 -> 6.6 us) but the step does not, 0.4927 ->
        # 0.4948 ms: fifteen copies per rank instead of five, and they end later than the backward pass they hide under.)
        self.push_gradients = (world == 2) if push_gradients == "auto" else bool(push_gradients)
        self.push_stream = None
        self._pushed = None   # indices (into self.layers) pushed in the step being enqueued
        shapes = [l.weight.shape for l in self.layers]
        if self._peer_update_possible(peer_update):
            self._setup_peer(shapes)
        if self.peer is None:
            self.bucket = GradBucket(shapes, self.device)
        for l, v in zip(self.layers, self.bucket.views):
            l.grad_buffer = v
            l.defer_update = True  # one launch updates every layer at the end of the step (after the all-reduce, if any)
            # ... and zeroes the bucket, so that the weight-gradient kernels add into it with no clearing pass;
            # keep_gradients leaves each step's int32 gradients readable in the bucket instead (one memset per layer)
            l.grad_accumulate = not keep_gradients
            l.wgrad_stream = self.side
        # The all-reduce is NOT overlapped with the backward pass: starting each bucket segment's all-reduce as soon as its
        # gradients were enqueued was built and measured 9 % slower on 2 B200s (NCCL's kernels take SMs away from the
        # one-CTA-per-SM contraction kernels and delay the cooperative ones, which need every SM free).
        self.x = torch.zeros((local_batch,) + tuple(in_shape), dtype=torch.float32, device=self.device)
        self.t = torch.zeros((local_batch,), dtype=torch.int64, device=self.device)
        # two result slots, used alternately: step i's logits stay readable while step i+1 writes the other slot
        self._out_hosts = [torch.zeros((local_batch, self.layers[-1].weight.shape[0]), dtype=torch.int8).pin_memory() for _ in range(2)]
        self._exp_hosts = [torch.zeros((), dtype=torch.int32).pin_memory() for _ in range(2)]
        self._done = [torch.cuda.Event() for _ in range(2)]
        self._res_slot = 0
        self.out_host, self.exp_host = self._out_hosts[0], self._exp_hosts[0]
        self.h2d_bytes = self.x.numel() * 4 + self.t.numel() * 8
        self.d2h_bytes = self.out_host.numel() + 4
        ti_torch.set_seed(seed, self.device)
        self.sample_offset = rank * local_batch if sample_offset is None else int(sample_offset)
        ti_torch.SAMPLE_OFFSET = self.sample_offset
        self._status_hosts = [torch.zeros(4, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._failed = None  # message of a kernel wait that ran out: no further steps until reset_exchange()
        # input prefetch: two staging slots filled from pinned host memory on a copy stream while the previous step computes
        self.copy_stream = torch.cuda.Stream(device=self.device)
        self._stage_x = [torch.zeros_like(self.x) for _ in range(2)]
        self._stage_t = [torch.zeros_like(self.t) for _ in range(2)]
        self._slot_ready = [torch.cuda.Event() for _ in range(2)]
        self._slot_free = [torch.cuda.Event() for _ in range(2)]
        for e in self._slot_free:
            e.record(torch.cuda.current_stream(self.device))
        self._pf_slot, self._pf_key = 0, None
        self._graphs = None
        self._eager_steps = 0
        self._warmup_steps = warmup_steps
        self.kernels_per_step = None

    # ------------------------------------------------------------------ peer-memory update
    def _peer_update_possible(self, wanted):
        if not wanted or self.world < 2 or self.world > 8 or self.keep_gradients or self.global_exact:
            return False
        if self.device.type != "cuda" or len(self.layers) > 16 or any(l.weight.numel() % 4 for l in self.layers):
            return False
        if dist.get_backend(self.group) != "nccl" or not peers_on_one_node(self.device, self.group):
            if wanted is True:
                raise RuntimeError("peer_update needs an NCCL group whose ranks sit on different GPUs of one node")
            return False
        return True

    def _setup_peer(self, shapes):
        w_offs, off = [], 0
        for l in self.layers:
            w_offs.append(off)
            off += (l.weight.numel() + 255) // 256 * 256
        g_off, g_numel = off, GradBucket.numel_for(shapes)
        x_off = (g_off + 4 * g_numel + 255) // 256 * 256
        # staging: for every layer, room for each rank's contribution to the own slice (slices differ by at most one group)
        s_off, self._stage = (x_off + ops.dp_exchange_bytes() + 255) // 256 * 256, []
        end = s_off
        for l in self.layers:
            groups = l.weight.numel() // 4
            cap = ((groups + self.world - 1) // self.world * 16 + 255) // 256 * 256
            self._stage.append((end, cap))
            end += cap * self.world
        arena = PeerArena(end, self.device, self.group)
        if not arena.ok:
            warnings.warn(f"peer mapping failed ({arena.error or 'on another rank'}): falling back to the NCCL all-reduce")
            return
        for l, o in zip(self.layers, w_offs):  # the weights move into the arena, where the peers' kernels store updates
            v = arena.view(o, l.weight.numel(), torch.int8, l.weight.shape)
            v.copy_(l.weight)
            l.weight = v
        self.bucket = GradBucket(shapes, self.device, flat=arena.view(g_off, 4 * g_numel, torch.int32))
        self._dp_items = [(w_offs[i], self.bucket.offsets[i], l.weight.numel(), 16 * l.layer_id + 2)
                          for i, l in enumerate(self.layers)]
        self._dp_ptrs = (list(arena.ptrs), [p + g_off for p in arena.ptrs], [p + x_off for p in arena.ptrs])
        self.peer = arena
        if self.push_gradients and self.side is not None:
            # one stream per destination: copies to different peers run on different copy engines side by side
            self.push_stream = [torch.cuda.Stream(device=self.device) for _ in range(self.world - 1)]
            ti_torch.WGRAD_FLUSH_HOOK = self._push_hook
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def resync(self):
        """Collective: brings the ranks back in step on the host (call on every rank after a pause that may have
        held one of them back for more than a second or so, before the next ``step``)."""
        if self.world > 1:
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
            torch.cuda.synchronize(self.device)

    def reset_exchange(self):
        """Collective: after a reported wait expiry, clear the exchange area, the gradient bucket and the status word on
        every rank so that steps may resume.  The weights are NOT repaired: a step that gave up may have updated some
        slices and not others, so load the same checkpoint on every rank first."""
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(self.group)
        if self.peer is not None:
            x_off = self._dp_ptrs[2][self.rank] - self.peer.ptrs[self.rank]
            self.peer.view(x_off, ops.dp_exchange_bytes(), torch.uint8).zero_()
        self.bucket.flat.zero_()
        ops.status_word(self.device).zero_()
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(self.group)
        self._failed = None

    def close(self):
        """Collective: unmaps the peers' memory (call on every rank before the process group goes away)."""
        if self.peer is not None:
            torch.cuda.synchronize(self.device)
            for l in self.layers:  # the arena is about to be freed: the model keeps its weights in memory of its own
                l.weight = l.weight.clone()
                l.grad_buffer = None
            self.peer.close()
            self.peer = None
            self._graphs = None
            if ti_torch.WGRAD_FLUSH_HOOK == self._push_hook:
                ti_torch.WGRAD_FLUSH_HOOK = None

    # ------------------------------------------------------------------ pieces of one step
    def _slice(self, i, r):
        """Word groups [lo, hi) of layer i that rank r owns in the update kernel."""
        groups = self.layers[i].weight.numel() // 4
        return groups * r // self.world, groups * (r + 1) // self.world

    def _push_hook(self, stream, group):
        """Called by ti_torch right after a full group of weight gradients went out on `stream`: behind that launch
        these layers' gradients (and the classifier's, which came with the head kernel) are final.  Every slice goes to
        its owner's staging memory now, by device-to-device copies on a stream of its own: the copy engines move it over
        NVLink while the SMs run the rest of the backward pass."""
        if self.peer is None or self._pushed is None:
            return
        index = {id(l): i for i, l in enumerate(self.layers)}
        take = [index[id(l)] for l in group if id(l) in index and index[id(l)] not in self._pushed]
        head = len(self.layers) - 1
        if not self._pushed and not hasattr(self.layers[head], "padding"):
            take.append(head)
        if not take:
            return
        bucket = self._dp_ptrs[1][self.rank]
        peers = [(self.rank + 1 + k) % self.world for k in range(self.world - 1)]  # every rank starts with its right neighbour
        for ps, r in zip(self.push_stream, peers):
            ps.wait_stream(stream)
            with torch.cuda.stream(ps):
                for i in sorted(take, key=lambda i: -self._dp_items[i][2]):  # the large layers first
                    g_off = self._dp_items[i][1]
                    base, cap = self._stage[i]
                    lo, hi = self._slice(i, r)
                    if hi > lo:
                        ops.peer_copy(self.peer.ptrs[r] + base + self.rank * cap, bucket + 4 * (g_off + 4 * lo), 16 * (hi - lo))
        self._pushed.extend(take)

    def _forward_backward(self):
        self._pushed = [] if self.push_stream is not None else None
        self.model.train_step(self.x, self.t)
        if self.side is not None:
            ti_torch.flush_wgrad()  # a group of weight gradients that never filled up
            torch.cuda.current_stream(self.device).wait_stream(self.side)
        if self.push_stream is not None:
            for ps in self.push_stream:
                torch.cuda.current_stream(self.device).wait_stream(ps)

    def _update(self):
        if self.peer is not None:
            items = []
            for i, it in enumerate(self._dp_items):
                staged = None
                if self._pushed and i in self._pushed:
                    # rank r's contribution to the own slice lies at base + r * cap of the OWN arena; the kernel indexes
                    # by word group of the whole layer, hence the slice's first group is taken off
                    lo, _ = self._slice(i, self.rank)
                    base, cap = self._stage[i]
                    staged = [self.peer.ptrs[self.rank] + base + r * cap - 16 * lo for r in range(self.world)] + [0] * (8 - self.world)
                items.append(tuple(it) + (staged,))
            ops.dp_update(items, self.rank, self.world, *self._dp_ptrs, ti_torch.GRAD_BITWIDTH,
                          ti_torch._mode(ti_torch.GRAD_ROUND_METHOD), ti_torch.RNG_SEED(self.device), self.device)
        else:
            ti_torch.weight_update_all(self.layers, clear=not self.keep_gradients)
        ti_torch.advance_seed(self.device)

    def _run_eager(self):
        self._forward_backward()
        if self.world > 1 and self.peer is None:
            self.bucket.allreduce_(self.group)
        self._update()

    def _capture(self):
        torch.cuda.synchronize(self.device)
        if self.peer is not None:
            dist.barrier(self.group)  # capture takes each rank a different time: start the replays together
        g1 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g1):
            self._forward_backward()
            if self.world == 1 or self.peer is not None:
                self._update()
        g2 = None
        if self.world > 1 and self.peer is None:
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2, pool=g1.pool()):
                self._update()
        self._graphs = (g1, g2)
        if self.peer is not None:
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)

    def run_device_step(self):
        """The device part of a step on inputs already resident in self.x / self.t."""
        if self.use_graph and self._graphs is None and self._eager_steps >= self._warmup_steps:
            self._capture()
        if self._graphs is not None:
            g1, g2 = self._graphs
            g1.replay()
            if g2 is not None:
                self.bucket.allreduce_(self.group)
                g2.replay()
        else:
            self._run_eager()
            self._eager_steps += 1

    # ------------------------------------------------------------------ public call
    def prefetch(self, x_host, target_host):
        """Start the host-to-device copy of a LATER batch now (on a copy stream, into a staging slot), so that it
        overlaps the step in flight; ``step`` recognises the batch by its host buffers and takes it from the slot."""
        slot = self._pf_slot = 1 - self._pf_slot
        self.copy_stream.wait_event(self._slot_free[slot])  # the step that used this slot has copied it out
        with torch.cuda.stream(self.copy_stream):
            self._stage_x[slot].copy_(x_host, non_blocking=True)
            self._stage_t[slot].copy_(target_host, non_blocking=True)
            self._slot_ready[slot].record(self.copy_stream)
        self._pf_key = (x_host.data_ptr(), target_host.data_ptr(), slot)

    def step(self, x_host, target_host, prefetch_next=None):
        """x_host float32 [B,3,32,32] and target_host int64 [B] in (pinned) host memory.
        Returns (pinned int8 logits [B, classes], pinned int32 exponent); valid after the
        stream is synchronised (``Trainer.sync``).  ``prefetch_next=(x, t)``: the next batch, whose copy
        then runs beside this step's kernels."""
        if self._failed is not None:
            raise RuntimeError(f"{self._failed}; the trainer takes no further steps until reset_exchange()")
        main = torch.cuda.current_stream(self.device)
        if self._pf_key is not None and self._pf_key[:2] == (x_host.data_ptr(), target_host.data_ptr()):
            slot = self._pf_key[2]
            self._pf_key = None
            main.wait_event(self._slot_ready[slot])
            self.x.copy_(self._stage_x[slot], non_blocking=True)
            self.t.copy_(self._stage_t[slot], non_blocking=True)
            self._slot_free[slot].record(main)
        else:
            self.x.copy_(x_host, non_blocking=True)
            self.t.copy_(target_host, non_blocking=True)
        if prefetch_next is not None:
            self.prefetch(*prefetch_next)
        self.run_device_step()
        k = self._res_slot = 1 - self._res_slot
        self.out_host, self.exp_host = self._out_hosts[k], self._exp_hosts[k]
        self.out_host.copy_(self.model.out, non_blocking=True)
        self.exp_host.copy_(self.model.out_exp, non_blocking=True)
        self._status_hosts[k].copy_(ops.status_word(self.device), non_blocking=True)
        self._done[k].record(main)
        return StepResult(self.out_host, self.exp_host, self._done[k], self._status_hosts[k], self)

    def sync(self):
        torch.cuda.synchronize(self.device)
        try:
            ops.check_status(self.device)
        except RuntimeError as e:
            self._failed = str(e)
            raise

    def replica_checksum(self):
        """Digest of all weights; equal on every rank of a healthy data-parallel run."""
        tot = 0
        for l in self.layers:
            w = l.weight.to(torch.int64).flatten()
            tot = (tot * 1000003 + int((w * (torch.arange(w.numel(), device=w.device) % 65521 + 1)).sum().item())) % (1 << 61)
        return tot
