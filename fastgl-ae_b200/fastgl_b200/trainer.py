"""Data-parallel mini-batch training loop: the hot loop of the reference's ``run()`` (train_fastgl.py:310-405)
rebuilt around windowed fused sampling.

One process per GPU.  Every rank holds the whole by-destination CSR and the feature table in its HBM
(train_fastgl.py:219-244 keeps the CSR on the GPU too; the feature table replaces the CPU tensor plus the
MatchServer cache), takes its own share of the shuffled training seeds (the ``use_ddp`` split of
train_fastgl.py:252), samples a window of mini-batches per kernel launch, optionally Match-Reorders the
window, and trains batch by batch.  The only collective is one all-reduce of the flat gradient buffer per step.
"""
from __future__ import annotations

import gc
import math
from concurrent.futures import ThreadPoolExecutor

import torch
import torch.distributed as dist
import torch.nn.functional as F

import fastgl

from .block import Block
from .layers import GCN
from .sage_step import SageStepProgram
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
        total = (total + 3) // 4 * 4      # whole 128-bit vectors: the padding stays zero
        self.buffer = torch.zeros(total, dtype=self.params[0].dtype, device=self.params[0].device)
        off = 0
        for p in self.params:
            p.grad = self.buffer[off: off + p.numel()].view_as(p)
            off += p.numel()

    def zero(self):
        self.buffer.zero_()

    def all_reduce(self, world: int):
        if world > 1:
            if dist.get_backend() == "nccl":
                dist.all_reduce(self.buffer, op=dist.ReduceOp.AVG)   # one kernel: sum and scale
            else:
                dist.all_reduce(self.buffer)
                self.buffer.div_(world)


class FlatAdam:
    """Adam (torch.optim.Adam's arithmetic, L2 weight decay) as one launch over all parameters: the parameters are
    moved into one flat buffer (each ``p.data`` becomes a view of it, in the order of ``FlatGrads``) next to flat
    first- and second-moment buffers.  The step count lives on the device and the launch advances it, so the launch
    can be captured in a CUDA graph.  With ``peers`` (a ``fastgl.PeerSync``) the same launch first averages the
    gradient over the data-parallel ranks through peer-mapped buffers: no separate collective."""

    def __init__(self, grads: FlatGrads, lr, weight_decay, betas=(0.9, 0.999), eps=1e-8, peers=None):
        self.grads = grads
        self.peers = peers
        self.lr, self.weight_decay, self.betas, self.eps = lr, weight_decay, betas, eps
        self.flat = torch.zeros_like(grads.buffer)
        off = 0
        with torch.no_grad():
            for p in grads.params:
                view = self.flat[off: off + p.numel()].view_as(p)
                view.copy_(p.data)
                p.data = view
                off += p.numel()
        self.exp_avg = torch.zeros_like(self.flat)
        self.exp_avg_sq = torch.zeros_like(self.flat)
        self.step_dev = torch.zeros(3, dtype=torch.int32, device=self.flat.device)

    def step(self):
        if self.peers is not None:
            fastgl.allreduce_adam_(self.peers, self.flat, self.grads.buffer, self.exp_avg, self.exp_avg_sq, self.step_dev,
                                   lr=self.lr, betas=self.betas, eps=self.eps, weight_decay=self.weight_decay)
        else:
            fastgl.adam_step_(self.flat, self.grads.buffer, self.exp_avg, self.exp_avg_sq, self.step_dev, lr=self.lr,
                              betas=self.betas, eps=self.eps, weight_decay=self.weight_decay)

    def zero_state(self):
        self.exp_avg.zero_()
        self.exp_avg_sq.zero_()
        self.step_dev[:2].zero_()     # the exchange counter [2] keeps counting: the peers' flags are monotonic


class GraphedStep:
    """The per-mini-batch part of a training step -- inner layers forward, loss, backward and (single GPU) the
    optimizer step -- captured once as a CUDA graph over buffers of fixed, padded shape and replayed for every
    mini-batch.  A staging kernel copies the batch's first-layer rows and inner blocks into those buffers and
    writes the real row counts, which the aggregation kernels read on the device.  The captured work is the
    hand-written launch sequence of ``sage_step.SageStepProgram`` (about 25 launches).  This removes the host launches
    that otherwise bound the step time (the reference even blocks on an event three times per step,
    train_fastgl.py:348,362,373)."""

    def __init__(self, trainer, pad_dst):
        self.tr = trainer
        tr = trainer
        dev, D = tr.dev, tr.feat.size(1)
        L = len(tr.fanouts)
        self.L = L
        self.pad_dst = list(pad_dst)            # padded destination count of block i (input layer first)
        assert len(self.pad_dst) == L and self.pad_dst[-1] == tr.batch_size
        self.x0 = torch.zeros((self.pad_dst[0], 2 * D), dtype=torch.float32, device=dev)
        self.sizes = torch.zeros(8, dtype=torch.int32, device=dev)   # [0, L): real row counts; [L]: step index
        self.seeds = torch.zeros(tr.batch_size, dtype=torch.int32, device=dev)
        self.steps_staged = 0
        self.blocks = [None]
        for i in range(1, L):
            ptr = torch.zeros(self.pad_dst[i] + 1, dtype=torch.int32, device=dev)
            src = torch.zeros(self.pad_dst[i] * tr.fanouts[i], dtype=torch.int32, device=dev)
            self.blocks.append(Block(ptr, src, self.pad_dst[i - 1], self.pad_dst[i], n_dst_dev=self.sizes[i: i + 1]))
        self.graph = None
        self.loss = None
        # With the library collective, data-parallel runs keep the gradient all-reduce between two graphs
        # (forward/backward, optimizer step): every rank then issues the collective the same way whether or not its
        # batch fitted the padded shapes.  With the one-launch exchange the optimizer launch averages the gradients
        # itself, so the whole step is one graph.
        self.step_in_graph = tr.world == 1 or tr.oneshot
        self.opt_graph = None
        self.program = SageStepProgram(tr.model, tr.grads, tr.labels, self.x0, self.seeds, self.sizes, self.blocks,
                                       self.pad_dst, self.sizes[L: L + 1], rng_seed=tr.sampler.rng_seed, matmul=tr.matmul)
        self.program.x0_presplit = self.program.split

    def fits(self, counts_row) -> bool:
        L = self.L
        return all(int(counts_row[L - 1 - i]) <= self.pad_dst[i] for i in range(L))

    def stage(self, fb, b, counts_row, layer0):
        """Copy mini-batch ``b`` of the window into the static buffers (one kernel launch; addresses are computed
        here so that no tensor views are created per step)."""
        L = self.L
        buf, row_off = layer0
        n_dst = [int(counts_row[L - 1 - i]) for i in range(L)]
        row_bytes = buf.stride(0) * 4
        # only the batch's own seeds: the rows after a short batch keep earlier (valid) node ids
        segs = [(self.seeds.data_ptr(), fb.nodes.data_ptr() + b * fb.nodes.stride(0) * 4, n_dst[L - 1] * 4)]
        prog = self.program
        if prog.split:
            # the input layer's rows go straight from the window buffer into the operand form of the error-compensated
            # products, [hi | lo | hi]; the plain copy in x0 is not needed
            x3, c = prog.x3[0], buf.size(1)
            base, ld3 = x3.data_ptr(), x3.stride(0)
            fastgl.split_tf32_raw(buf.data_ptr() + row_off[b] * row_bytes, n_dst[0], c, buf.stride(0),
                                  [(base, ld3, 0), (base + 4 * c, ld3, 1), (base + 8 * c, ld3, 0)], self.tr.dev)
        else:
            segs.append((self.x0.data_ptr(), buf.data_ptr() + row_off[b] * row_bytes, n_dst[0] * row_bytes))
        for i in range(1, L):
            h = L - 1 - i
            ptr, src = fb.block_indptr[h], fb.block_src[h]
            segs.append((self.blocks[i].indptr.data_ptr(), ptr.data_ptr() + b * ptr.stride(0) * 4, (n_dst[i] + 1) * 4))
            segs.append((self.blocks[i].src.data_ptr(), src.data_ptr() + b * src.stride(0) * 4, int(counts_row[8 + h]) * 4))
        self.steps_staged += 1
        fastgl.stage_segments_raw(segs, self.sizes.data_ptr(), n_dst + [self.steps_staged & 0x7fffffff], self.tr.dev)

    def _forward_backward(self):
        with torch.no_grad():
            return self.program.forward_backward()

    def capture(self):
        """Warm up on a side stream (restoring model and optimizer afterwards) and capture the step."""
        tr = self.tr
        model_state = {k: v.clone() for k, v in tr.model.state_dict().items()}
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                self._forward_backward()
                tr.opt.step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        # undo the warm-up steps in place: the graphs must capture the very tensors the optimizer will keep using
        tr.model.load_state_dict(model_state)
        tr.zero_optimizer_state()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.loss = self._forward_backward()
            if self.step_in_graph:
                tr.opt.step()
        if not self.step_in_graph:
            self.opt_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.opt_graph):
                tr.opt.step()

    def replay(self):
        self.graph.replay()
        if not self.step_in_graph:
            self.tr.grads.all_reduce(self.tr.world)
            self.opt_graph.replay()
        return self.loss


class Trainer:
    def __init__(self, indptr, indices, feat, labels, train_nids, model, fanouts, batch_size=1024, window=8,
                 lr=0.01, weight_decay=5e-4, reorder=False, rank=0, world=1, rng_seed=12345, n_teams=0,
                 window_layer0=True, cuda_graph=False, table_direct=True, table_slots=None, grad_sync="auto",
                 matmul="fp32"):
        self.dev = feat.device
        self.feat, self.labels = feat, labels
        self.model = model
        self.fanouts = list(fanouts)
        self.batch_size, self.window = int(batch_size), int(window)
        self.rank, self.world = rank, world
        self.n_teams = n_teams
        # dense products of the hand-written step: "fp32" (cuBLAS SIMT kernels) or "3xtf32" (error-compensated TF32 on
        # the tensor cores, float32-level error); the autograd fallback always follows torch's global setting
        self.matmul = matmul
        self.table_direct = bool(table_direct)   # GCN: first layer reads the feature table through the block's ids
        # cap of the sampler's per-team hashtable: None = learn it from the first window, 0 = worst-case size
        self._auto_table = table_slots is None
        self.table_slots = 0 if table_slots is None else int(table_slots)
        self.table_overflows = 0
        self.n_nodes = indptr.numel() - 1
        self.sampler = FusedMapSampler(self.fanouts, replace=False, rng_seed=rng_seed + 7919 * rank)
        self.sampler.edge_src, self.sampler.edge_ptr, self.sampler.nodes_num = indices, indptr, self.n_nodes
        self.matcher = MatchReorder(self.n_nodes) if reorder else None
        self.grads = FlatGrads(model.parameters())
        self.lr, self.weight_decay = lr, weight_decay
        # GraphSAGE (layers with a self term and a stacked weight) has the hand-written step and the flat optimizer
        self.sage = hasattr(model, "layers") and hasattr(model.layers[0], "input_dim")
        self.use_graph = bool(cuda_graph) and self.sage
        self.graphed = None
        self.graph_fallbacks = 0
        # gradient averaging across ranks: "nccl" = one all-reduce call per step between forward/backward and the
        # optimizer; "oneshot" = the optimizer launch exchanges the gradients itself through peer-mapped buffers
        # (GraphSAGE's flat optimizer on CUDA ranks of one box); "auto" picks the latter where it applies
        if grad_sync not in ("auto", "nccl", "oneshot"):
            raise ValueError("grad_sync must be auto, nccl or oneshot")
        can_oneshot = world > 1 and self.sage and self.dev.type == "cuda" and world <= 8
        if grad_sync == "oneshot" and not can_oneshot:
            raise ValueError("grad_sync='oneshot' needs 2..8 CUDA ranks and the GraphSAGE model")
        self.oneshot = can_oneshot and grad_sync != "nccl"
        self._peers = None
        self.reset_optimizer()
        self.train_nids = train_nids
        self._train_nids_host = train_nids.cpu()
        self._shuffler = ThreadPoolExecutor(max_workers=1)
        self._next_seeds = None
        self.epoch = 0
        self._set_epoch_seeds()
        self.sampled_edges = 0
        self.last_loss = None
        self.last_order = None    # order in which the last window's mini-batches were trained
        self.layer0_events = []   # (start, end, block | window) of the first-layer aggregation, when timed
        self._loss_host = None
        self.sample_events = []   # (start, end, n_batches) of the fused sampling launches, when timed
        self.time_layer0 = False
        # The first layer's [self | neighbour-mean] rows do not depend on the weights, so they are produced for
        # the whole window by one launch straight from the feature table.
        self.window_layer0 = bool(window_layer0) and self.sage
        self._layer0_buf = None

    def grad_sync_kind(self) -> str:
        if self.world == 1:
            return "none (one rank)"
        return "one-launch peer-store exchange fused with Adam" if self.oneshot else "NCCL all-reduce between two graphs"

    def _peer_sync(self):
        """Collective over the default group: allocate this rank's receive buffer and flags, map the peers'."""
        if self._peers is None:
            from .sharding import open_peer_tensors
            n = self.grads.buffer.numel()
            n_recv, n_flags = fastgl.PeerSync.sizes(n, self.world)
            recv = torch.zeros(n_recv, dtype=torch.float32, device=self.dev)
            flags = torch.zeros(n_flags, dtype=torch.int32, device=self.dev)
            torch.cuda.synchronize(self.dev)
            self._peers = fastgl.PeerSync(self.rank, self.world, open_peer_tensors(recv), open_peer_tensors(flags), n)
        return self._peers

    def release_peers(self):
        """Drop the mappings of the peers' buffers (before any rank frees its own)."""
        if isinstance(getattr(self, "opt", None), FlatAdam):
            self.opt.peers = None
        self._peers = None
        self.graphed = None

    def _sync_and_step(self):
        if not self.oneshot:
            self.grads.all_reduce(self.world)
        self.opt.step()

    def reset_optimizer(self):
        if self.sage:
            self.opt = FlatAdam(self.grads, self.lr, self.weight_decay, peers=self._peer_sync() if self.oneshot else None)
        else:
            self.opt = torch.optim.Adam(self.model.parameters(), lr=self.lr, weight_decay=self.weight_decay, fused=True)

    def zero_optimizer_state(self):
        if isinstance(self.opt, FlatAdam):
            self.opt.zero_state()
            return
        for state in self.opt.state.values():
            for v in state.values():
                if torch.is_tensor(v):
                    v.zero_()

    def _sampler_teams(self) -> int:
        """Teams of the fused sampler: as many mini-batches in flight as the window has (up to 16) once the tables
        are small enough for all of them to stay in L2 together, else the library's default."""
        if self.n_teams > 0 or self.table_slots == 0:
            return self.n_teams
        teams = min(self.window, 16)
        return teams if teams * self.table_slots * 8 <= (64 << 20) else 0

    def _ensure_graph(self, fb, b, layer0):
        """Build and capture the step program on the shapes of window ``fb`` (staged with its batch ``b``)."""
        if self.graphed is not None:
            return
        L = len(self.fanouts)
        pad = []
        for i in range(L):
            n = int(fb.counts_host()[:, L - 1 - i].max())
            pad.append(self.batch_size if i == L - 1 else ((int(n * 1.12) + 255) // 256) * 256)
        self.graphed = GraphedStep(self, pad)
        self.graphed.stage(fb, b, fb.counts_list()[b], layer0)
        self.graphed.capture()

    def _graph_step(self, fb, b, layer0):
        """Replay the captured step for batch ``b``; returns None when the batch does not fit the padded shapes."""
        counts_row = fb.counts_list()[b]
        self._ensure_graph(fb, b, layer0)
        if not self.graphed.fits(counts_row):
            self.graph_fallbacks += 1
            return None
        self.graphed.stage(fb, b, counts_row, layer0)
        return self.graphed.replay()

    def prime(self):
        """One-time set-up that would otherwise happen inside the first windows of training: sample one full window
        of this rank's seeds (without consuming them or their random-number counters), size the sampler's tables and
        workspace from it, and capture the step program on its shapes.  Parameters and optimizer state are left as
        they were."""
        if not self.my_seeds.numel():
            return
        nb = self.window
        need = nb * self.batch_size
        reps = -(-need // self.my_seeds.numel())
        seeds = self.my_seeds.repeat(reps)[:need].view(nb, self.batch_size).contiguous()
        counts = torch.full((nb,), self.batch_size, dtype=torch.int32, device=self.dev)
        counter = self.sampler.batch_counter
        fb = self.sampler.sample_window(seeds, counts, n_teams=self._sampler_teams(), slot=0, table_slots=self.table_slots)
        fb.start_readback()
        fb.counts_host()
        if fb.device_status != 0:
            fastgl.check_status(self.dev)
        if self._auto_table and self.table_slots == 0:
            most = int(fb.counts_host()[:, len(self.fanouts)].max())
            self.table_slots = 1 << max(12, math.ceil(math.log2(max(1.0, 2.5 * most))))
            self.sampler.sample_window(seeds, torch.zeros_like(counts), n_teams=self._sampler_teams(), slot=1,
                                       table_slots=self.table_slots)
        if self.use_graph and self.window_layer0:
            layer0 = self.aggregate_window_layer0(fb)
            self._ensure_graph(fb, 0, layer0)
        self.sampler.batch_counter = counter
        torch.cuda.synchronize(self.dev)
        # Everything built so far (graph, tables, the captured step and its buffers) lives as long as the trainer:
        # moving it out of the garbage collector's generations keeps the collections that the training loop's own
        # short-lived objects trigger from walking it again and again (3 % of the step time, measured).
        gc.collect()
        gc.freeze()

    def _shuffled_share(self, epoch: int) -> torch.Tensor:
        return shard_seeds(self._train_nids_host, self.rank, self.world, 12345 + epoch)   # host only: no CUDA call

    def _set_epoch_seeds(self):
        """This epoch's share of the shuffled seeds.  The shuffle is a host permutation (the same on every rank
        and on any device); the next epoch's is drawn on a worker thread while this epoch trains."""
        share = self._next_seeds.result() if self._next_seeds is not None else self._shuffled_share(self.epoch)
        self.my_seeds = share.to(self.dev)
        self._next_seeds = self._shuffler.submit(self._shuffled_share, self.epoch + 1)
        self.cursor = 0

    def steps_per_epoch(self) -> int:
        return math.ceil(self.my_seeds.numel() / self.batch_size)

    def _next_window_seeds(self, n_batches: int):
        """int32[n_batches, batch_size] seeds (wrapping into the next epoch's shuffle) and their counts."""
        span = n_batches * self.batch_size
        if 0 < span <= self.my_seeds.numel() - self.cursor:
            # the whole window lies inside this epoch's shuffle: a view, no kernels
            seeds = self.my_seeds[self.cursor: self.cursor + span].view(n_batches, self.batch_size)
            self.cursor += span
            return seeds, torch.full((n_batches,), self.batch_size, dtype=torch.int32)
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
        timing = None
        if self.time_layer0:    # the events go directly around the launch: no host-side preparation in the interval
            timing = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        row_off = fastgl.aggregate_window(fastgl.AGG_MEAN, fb, hop, self.feat, buf[:, D:], self_out=buf[:, :D], timing=timing)
        if timing is not None:
            self.layer0_events.append((timing[0], timing[1], fb))
        return buf, row_off

    def train_batch(self, fb, b: int, labels_of=None, layer0=None):
        if self.use_graph and layer0 is not None and labels_of is None:
            loss = self._graph_step(fb, b, layer0)
            if loss is not None:
                c = fb.counts_list()[b]
                self.sampled_edges += sum(c[8: 8 + len(self.fanouts)])
                self.last_loss = loss
                return loss
        input_nodes, blocks = self.sampler.window_blocks(fb, b)
        seeds = input_nodes[: blocks[-1].n_dst]
        y = self.labels[seeds.long()] if labels_of is None else labels_of
        if layer0 is not None:
            buf, row_off = layer0
            logits = self.model(blocks, None, layer0=buf[row_off[b]: row_off[b + 1]])
        elif self.sage:
            self.model.layer0_timer = self.layer0_events if self.time_layer0 else None
            logits = self.model(blocks, self.feat, input_nodes=input_nodes)
        elif isinstance(self.model, GCN) and self.table_direct:
            # GCN's first layer aggregates straight from the feature table: no gathered copy of the input rows
            logits = self.model(blocks, self.feat, neighbor_list=self.fanouts, input_nodes=input_nodes)
        else:
            # the reference's models (GCN / GIN) take the gathered input rows (train_fastgl.py:357,365)
            batch_inputs = fastgl.gather_rows(self.feat, input_nodes)
            logits = self.model(blocks, batch_inputs, neighbor_list=self.fanouts)
        loss = F.cross_entropy(logits, y)
        self.grads.zero()
        loss.backward()
        self._sync_and_step()
        self.sampled_edges += sum(blk.num_edges() for blk in blocks)
        self.last_loss = loss
        return loss

    def run_steps(self, n_steps: int, host_seeds=None, read_loss_each_step: bool = False):
        """Train ``n_steps`` mini-batches.  ``host_seeds`` (pinned int32[n_steps, batch_size] + counts) makes every
        window copy its seeds from the host inside the loop; ``read_loss_each_step`` reads the loss back per step."""
        done = 0
        losses = []
        # the loss of every step goes to pinned host memory with an asynchronous copy; it is read one step later,
        # after the next step has been enqueued, so the read-back does not drain the GPU
        pending = None
        if read_loss_each_step and self._loss_host is None:
            self._loss_host = torch.zeros(2, dtype=torch.float32).pin_memory()
        # The next window is sampled two steps before the current one ends, and only its counts are waited for:
        # the host then prepares that window while the GPU still has steps to run, so the GPU never waits for it.
        windows_sampled = 0

        def launch_sampler(seeds, counts, slot):
            nb = seeds.size(0)
            timing = None
            if self.time_layer0:
                timing = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            fb = self.sampler.sample_window(seeds, counts, n_teams=self._sampler_teams(), slot=slot,
                                            table_slots=self.table_slots, timing=timing)
            if timing is not None:
                self.sample_events.append((timing[0], timing[1], nb))
            if self.matcher is not None:
                # Match-Reorder's overlap matrix is computed on the device right behind the sampler and rides along
                # with the counts read-back, so ordering the window costs the host no extra synchronisation
                self.matcher.enqueue(fb.nodes, fb.counts[:, len(self.fanouts)], key=slot)
            fb.start_readback()
            return fb

        def sample_next(first_step):
            nonlocal windows_sampled
            nb = min(self.window, n_steps - first_step)
            if host_seeds is not None:
                seeds_h, counts_h = host_seeds
                seeds = seeds_h[first_step: first_step + nb].to(self.dev, non_blocking=True)
                counts = counts_h[first_step: first_step + nb].to(self.dev, non_blocking=True)
            else:
                seeds, counts = self._next_window_seeds(nb)
                counts = counts.to(self.dev, non_blocking=True)
            slot = windows_sampled & 1
            windows_sampled += 1
            return launch_sampler(seeds, counts, slot), nb, seeds, counts, slot

        nxt = sample_next(0) if n_steps > 0 else None
        while done < n_steps:
            fb, nb, seeds, counts, slot = nxt
            nxt = None
            fb.counts_host()
            if fb.device_status != 0:
                code = fb.device_status
                if code not in (fastgl.ERR_PROBE, fastgl.ERR_CAPACITY) or self.table_slots == 0:
                    # Not a table that was capped too small: a node id or a label out of range, a bounded wait that
                    # gave up ... -- recorded by this window's sampler or by the training steps enqueued before it.
                    # Clear the status and stop: the rows concerned contributed nothing.
                    fastgl.check_status(self.dev)
                    raise RuntimeError(f"device status: {fastgl.status_str(code)}")
                # The capped hashtable was too small for this window: clear the status, drop the cap and sample the
                # same window again -- same seeds, same Philox counters.
                try:
                    fastgl.check_status(self.dev)
                except RuntimeError:
                    pass
                self.table_slots, self._auto_table = 0, False
                self.table_overflows += 1
                self.sampler.batch_counter -= nb
                fb = launch_sampler(seeds, counts, slot)
                fb.counts_host()
                if fb.device_status != 0:
                    fastgl.check_status(self.dev)
            elif self._auto_table and self.table_slots == 0:
                # size the table from what a window really holds: 2.5 slots per node of the largest batch seen,
                # which keeps it L2-resident (the worst-case size is 16 MB per team at the benchmark shapes)
                most = int(fb.counts_host()[:, len(self.fanouts)].max())
                self.table_slots = 1 << max(12, math.ceil(math.log2(max(1.0, 2.5 * most))))
                # let the library size its workspace for the new team count now (an empty window through the
                # other set of buffers), not in front of the next window's launch
                self.sampler.sample_window(seeds, torch.zeros_like(counts), n_teams=self._sampler_teams(), slot=slot ^ 1,
                                           table_slots=self.table_slots)
                self.sampler.batch_counter -= nb
            layer0 = self.aggregate_window_layer0(fb) if self.window_layer0 else None
            order = list(range(nb))
            if self.matcher is not None:
                order = self.matcher.order(fb.counts_host()[:, len(self.fanouts)].tolist(), key=slot)
            self.last_order = order
            for i, b in enumerate(order):
                if i == max(0, nb - 2) and done + nb < n_steps:
                    nxt = sample_next(done + nb)
                loss = self.train_batch(fb, b, layer0=layer0)
                if read_loss_each_step:
                    loss_slot = len(losses) & 1 if pending is None else 1 - pending[1]
                    self._loss_host[loss_slot: loss_slot + 1].copy_(loss.detach().reshape(1), non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record()
                    if pending is not None:
                        pending[0].synchronize()
                        losses.append(float(self._loss_host[pending[1]]))
                    pending = (ev, loss_slot)
            done += nb
        if pending is not None:
            pending[0].synchronize()
            losses.append(float(self._loss_host[pending[1]]))
        return losses
