"""Gradient reduction overlapped with the backward pass of data-parallel training.

The reference gets this from DistributedDataParallel's bucketed all-reduces (keras/src/backend/torch/trainer.py:83-92).
Here the gradients already live in one flat arena in the order in which backward produces them, so a bucket is a
contiguous range of it.  The schedule is learned, not hooked into autograd's internals: during one ordinary step every
"a gradient contribution to parameter i has been issued" event is counted; from then on a bucket is reduced (by this
package's peer-memory all-reduce, on a second stream) as soon as every parameter in it has received its expected number
of contributions, while the backward pass carries on.  Buckets are reduced in arena order on every rank, so ranks never
disagree about which launch they are in.  The step ends with the main stream waiting for the reduction stream; inside a
recorded step the fork and join become edges of the graph.

Events come from two places: ``shadow.grad_slot`` (a kernel is about to add a weight gradient into the arena itself) and
``register_post_accumulate_grad_hook`` (autograd accumulated into the arena view).  A slot event precedes its kernel's
launch, so a bucket that an event completes is reduced when the next event arrives (or when backward has returned).
"""

import os

import torch


def enabled():
    return os.environ.get("KERAS_B200_DP_OVERLAP", "1") != "0"


def plan_buckets(offsets, total, target_bytes, max_buckets):
    """Cut a flat fp32 arena of ``total`` elements into contiguous buckets at variable boundaries.

    ``offsets``: variable index -> first element of that variable in the arena.  Returns ``(buckets, bucket_of)``: the
    ``(offset, numel)`` ranges in arena order (which is the order in which backward completes them) and, per variable, the
    index of its bucket.  About ``target_bytes`` each, at most ``max_buckets``; a variable is never split."""
    order = sorted(offsets, key=lambda i: offsets[i])
    n = max(1, min(max_buckets, (total * 4 + target_bytes - 1) // target_bytes))
    per = (total + n - 1) // n
    buckets, bucket_of = [], {}
    start = 0
    for pos, i in enumerate(order):
        end = offsets[order[pos + 1]] if pos + 1 < len(order) else total
        bucket_of[i] = len(buckets)
        if end - start >= per or pos + 1 == len(order):
            buckets.append((start, end - start))
            start = end
    return buckets, [bucket_of[i] for i in range(len(order))]


class GradientOverlap:
    def __init__(self, arena, reducer, world, target_bytes=None, max_buckets=8):
        if target_bytes is None:
            # launch latency, not link count, sizes a bucket on NVSwitch: a few tens of megabytes each, at most eight launches
            target_bytes = int(os.environ.get("KERAS_B200_DP_BUCKET_BYTES", str(32 << 20)))
        self.arena, self.reducer, self.scale = arena, reducer, 1.0 / world
        params = [v._value for v in arena.variables]
        self.index_of = {id(p): i for i, p in enumerate(params)}
        self._params = params  # keeps the ids valid
        self.stream = torch.cuda.Stream(device=arena.flat.device)
        self.buckets, self.bucket_of = self._make_buckets(target_bytes, max_buckets)
        self.expected = None
        self.counts = [0] * len(params)
        self.mode = None
        self.launched = 0
        self.remaining = []
        self.failed = None
        self._hooks = [p.register_post_accumulate_grad_hook(self._accumulated) for p in params if p.requires_grad]

    def close(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []

    def _make_buckets(self, target_bytes, max_buckets):
        return plan_buckets(self.arena.offsets, self.arena.total, target_bytes, max_buckets)

    # -- events ---------------------------------------------------------------------------------------------------------
    def _accumulated(self, param):
        self.note(param)

    def note(self, param):
        if self.mode is None:
            return
        i = self.index_of.get(id(param))
        if i is None:
            return
        if self.mode == "run":
            self._flush()
            if self.bucket_of[i] < self.launched:
                # cannot be repaired for this step: the bucket has been reduced without this contribution
                self.failed = self.arena.variables[i].path
                return
            self.remaining[self.bucket_of[i]] -= 1
        self.counts[i] += 1

    # -- one step -------------------------------------------------------------------------------------------------------
    def begin(self):
        """Call before backward.  The first call learns the schedule (the caller reduces the whole arena afterwards)."""
        self.counts = [0] * len(self.counts)
        self.failed = None
        if self.expected is None:
            self.mode = "learn"
            return
        self.mode = "run"
        self.launched = 0
        self.remaining = [0] * len(self.buckets)
        for i, n in enumerate(self.expected):
            self.remaining[self.bucket_of[i]] += n

    def finish(self):
        """Call after backward.  Returns True when the arena has been reduced (bucket by bucket), False when the caller still
        has to reduce it (the learning step)."""
        mode, self.mode = self.mode, None
        if mode == "learn":
            self.expected = list(self.counts)
            return False
        if self.failed is not None:
            raise RuntimeError(f"The gradient of '{self.failed}' received a contribution after its bucket had been reduced: the backward pass of this "
                               "model does not repeat from step to step. Set KERAS_B200_DP_OVERLAP=0 to reduce gradients after the backward pass.")
        while self.launched < len(self.buckets):
            self._launch()
        done = torch.cuda.Event()
        done.record(self.stream)
        torch.cuda.current_stream().wait_event(done)
        return True

    def _flush(self):
        while self.launched < len(self.buckets) and self.remaining[self.launched] <= 0:
            self._launch()

    def _launch(self):
        offset, numel = self.buckets[self.launched]
        self.launched += 1
        ready = torch.cuda.Event()
        ready.record()  # everything issued so far on the compute stream: all contributions to this bucket
        self.stream.wait_event(ready)
        with torch.cuda.stream(self.stream):
            self.reducer.all_reduce(offset, numel, scale=self.scale)
