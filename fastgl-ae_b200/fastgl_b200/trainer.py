"""Data-parallel mini-batch training loop: the hot loop of the reference's ``run()`` (train_fastgl.py:310-405)
rebuilt around windowed fused sampling.

One process per GPU.  Every rank holds the whole by-destination CSR and the feature table in its HBM
(train_fastgl.py:219-244 keeps the CSR on the GPU too; the feature table replaces the CPU tensor plus the
MatchServer cache), takes its own share of the shuffled training seeds (the ``use_ddp`` split of
train_fastgl.py:252), samples a window of mini-batches per kernel launch, optionally Match-Reorders the
window, and trains batch by batch.  The only collective is one all-reduce of the flat gradient buffer per step.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn.functional as F

import fastgl

from .sampler import FusedMapSampler
from .scheduler import MatchReorder


def shard_seeds(train_nids: torch.Tensor, rank: int, world: int, epoch_seed: int) -> torch.Tensor:
    """Shuffle with a generator every rank seeds alike, then take a contiguous, equally sized share
    (padding by wrap-around like DistributedSampler, which DGL's ``use_ddp`` uses)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(epoch_seed)
    perm = torch.randperm(train_nids.numel(), generator=gen).to(train_nids.device)
    per = math.ceil(train_nids.numel() / world)
    if per * world > perm.numel():
        perm = torch.cat([perm, perm[: per * world - perm.numel()]])
    return train_nids[perm[rank * per: (rank + 1) * per]].to(torch.int32)


class FlatGrads:
    """All parameter gradients as views of one buffer, so that the data-parallel step is one all-reduce."""

    def __init__(self, params):
        self.params = [p for p in params if p.requires_grad]
        total = sum(p.numel() for p in self.params)
        self.buffer = torch.zeros(total, dtype=self.params[0].dtype, device=self.params[0].device)
        off = 0
        for p in self.params:
            p.grad = self.buffer[off: off + p.numel()].view_as(p)
            off += p.numel()

    def zero(self):
        self.buffer.zero_()

    def all_reduce(self, world: int):
        if world > 1:
            dist.all_reduce(self.buffer)
            self.buffer.div_(world)


class Trainer:
    def __init__(self, indptr, indices, feat, labels, train_nids, model, fanouts, batch_size=1024, window=8,
                 lr=0.01, weight_decay=5e-4, reorder=False, rank=0, world=1, rng_seed=12345, n_teams=0,
                 window_layer0=True):
        self.dev = feat.device
        self.feat, self.labels = feat, labels
        self.model = model
        self.fanouts = list(fanouts)
        self.batch_size, self.window = int(batch_size), int(window)
        self.rank, self.world = rank, world
        self.n_teams = n_teams
        self.n_nodes = indptr.numel() - 1
        self.sampler = FusedMapSampler(self.fanouts, replace=False, rng_seed=rng_seed + 7919 * rank)
        self.sampler.edge_src, self.sampler.edge_ptr, self.sampler.nodes_num = indices, indptr, self.n_nodes
        self.matcher = MatchReorder(self.n_nodes) if reorder else None
        self.grads = FlatGrads(model.parameters())
        self.opt = torch.optim.Adam(model.parameters(), lr=lr, weight_decay=weight_decay, fused=True)
        self.train_nids = train_nids
        self.epoch = 0
        self._set_epoch_seeds()
        self.sampled_edges = 0
        self.last_loss = None
        self.layer0_events = []   # (start, end, block | window) of the first-layer aggregation, when timed
        self.sample_events = []   # (start, end, n_batches) of the fused sampling launches, when timed
        self.time_layer0 = False
        # The first layer's [self | neighbour-mean] rows do not depend on the weights, so they are produced for
        # the whole window by one launch straight from the feature table.
        self.window_layer0 = bool(window_layer0) and hasattr(model, "layers") and hasattr(model.layers[0], "input_dim")
        self._layer0_buf = None

    def _set_epoch_seeds(self):
        self.my_seeds = shard_seeds(self.train_nids, self.rank, self.world, 12345 + self.epoch)
        self.cursor = 0

    def steps_per_epoch(self) -> int:
        return math.ceil(self.my_seeds.numel() / self.batch_size)

    def _next_window_seeds(self, n_batches: int):
        """int32[n_batches, batch_size] seeds (wrapping into the next epoch's shuffle) and their counts."""
        rows, counts = [], []
        for _ in range(n_batches):
            if self.cursor >= self.my_seeds.numel():
                self.epoch += 1
                self._set_epoch_seeds()
            chunk = self.my_seeds[self.cursor: self.cursor + self.batch_size]
            self.cursor += self.batch_size
            counts.append(chunk.numel())
            if chunk.numel() < self.batch_size:
                chunk = torch.cat([chunk, chunk.new_zeros(self.batch_size - chunk.numel())])
            rows.append(chunk)
        return torch.stack(rows).contiguous(), torch.tensor(counts, dtype=torch.int32)

    def aggregate_window_layer0(self, fb):
        """[self | mean of neighbours] rows of the input layer for every batch of the window: (buffer, row_off)."""
        hop = len(self.fanouts) - 1
        D = self.feat.size(1)
        total = int(fb.counts_host()[:, hop].sum())
        if self._layer0_buf is None or self._layer0_buf.size(0) < total:
            self._layer0_buf = torch.empty((int(total * 1.25) + 1, 2 * D), dtype=torch.float32, device=self.dev)
        buf = self._layer0_buf
        if self.time_layer0:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        row_off = fastgl.aggregate_window(fastgl.AGG_MEAN, fb, hop, self.feat, buf[:, D:], self_out=buf[:, :D])
        if self.time_layer0:
            end.record()
            self.layer0_events.append((start, end, fb))
        return buf, row_off

    def train_batch(self, fb, b: int, labels_of=None, layer0=None):
        input_nodes, blocks = self.sampler.window_blocks(fb, b)
        seeds = input_nodes[: blocks[-1].n_dst]
        y = self.labels[seeds.long()] if labels_of is None else labels_of
        if layer0 is not None:
            buf, row_off = layer0
            logits = self.model(blocks, None, layer0=buf[row_off[b]: row_off[b + 1]])
        else:
            self.model.layer0_timer = self.layer0_events if self.time_layer0 else None
            logits = self.model(blocks, self.feat, input_nodes=input_nodes)
        loss = F.cross_entropy(logits, y)
        self.grads.zero()
        loss.backward()
        self.grads.all_reduce(self.world)
        self.opt.step()
        self.sampled_edges += sum(blk.num_edges() for blk in blocks)
        self.last_loss = loss
        return loss

    def run_steps(self, n_steps: int, host_seeds=None, read_loss_each_step: bool = False):
        """Train ``n_steps`` mini-batches.  ``host_seeds`` (pinned int32[n_steps, batch_size] + counts) makes every
        window copy its seeds from the host inside the loop; ``read_loss_each_step`` reads the loss back per step."""
        done = 0
        losses = []
        while done < n_steps:
            nb = min(self.window, n_steps - done)
            if host_seeds is not None:
                seeds_h, counts_h = host_seeds
                seeds = seeds_h[done: done + nb].to(self.dev, non_blocking=True)
                counts = counts_h[done: done + nb].to(self.dev, non_blocking=True)
            else:
                seeds, counts = self._next_window_seeds(nb)
                counts = counts.to(self.dev, non_blocking=True)
            if self.time_layer0:
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
            fb = self.sampler.sample_window(seeds, counts, n_teams=self.n_teams)
            if self.time_layer0:
                end.record()
                self.sample_events.append((start, end, nb))
            layer0 = self.aggregate_window_layer0(fb) if self.window_layer0 else None
            order = list(range(nb))
            if self.matcher is not None:
                order = self.matcher.reorder([fb.input_nodes(b) for b in range(nb)])
            for b in order:
                loss = self.train_batch(fb, b, layer0=layer0)
                if read_loss_each_step:
                    losses.append(float(loss.item()))
            done += nb
        return losses
