"""The Fused-Map sampler on top of the ``fastgl`` ops.

``FusedMapSampler.sample_blocks`` keeps the reference's per-hop loop and return value
(FusedMapSampler.py:63-109): walk ``reversed(fanouts)``, ``fastgl.sample_node`` then
``fastgl.transfer_edge_id``, the unique nodes of one hop are the seeds of the next, blocks come back
input-layer first.  ``sample_window`` is the B200 path: every hop of a whole window of mini-batches (the
batches Match-Reorder looks at together, utilis.py:35-39) in one persistent kernel launch, with a single
read-back of the per-batch counts.
"""
from __future__ import annotations

import torch

import fastgl

from .block import Block


class FusedMapSampler:
    def __init__(self, fanouts, replace: bool = False, rng_seed: int = 12345):
        self.fanouts = list(fanouts)
        self.replace = bool(replace)
        self.rng_seed = int(rng_seed)
        self.batch_counter = 0
        # set by the trainer, as train_fastgl.py:240-244 does
        self.edge_src = None   # int32 sources sorted by destination
        self.edge_dst = None   # unused by the kernels; kept for interface parity
        self.edge_ptr = None   # int32 or int64 offsets, n_nodes + 1
        self.nodes_num = 0
        self._window_out = {}

    # --- reference-shaped path: one mini-batch, one op call per hop ---------------------------------
    def sample_blocks(self, g, seed_nodes, exclude_eids=None):
        """Returns ``(input_nodes, output_nodes, blocks)`` like FusedMapSampler.py:109."""
        output_nodes = seed_nodes.int().contiguous()
        cur = output_nodes
        blocks = []
        ctr = self.batch_counter * 8
        self.batch_counter += 1
        for hop, fanout in enumerate(reversed(self.fanouts)):
            src_g, dst_g, ptr, n_edges = fastgl.sample_node_csr(self.edge_src, self.edge_ptr, cur, fanout,
                                                                replace=self.replace, rng_seed=self.rng_seed,
                                                                rng_ctr=ctr + hop)
            n_dst = cur.numel()
            max_src_num = min(self.nodes_num, fanout * n_dst)  # FusedMapSampler.py:95
            src_l, dst_l, uniq = fastgl.transfer_edge_id(src_g, dst_g, cur, n_dst, n_dst + n_edges, max_src_num, n_edges)
            blocks.insert(0, Block(ptr, src_l, uniq.numel(), n_dst, dst_l))
            cur = uniq
        return cur, output_nodes, blocks

    # --- B200 path: a window of mini-batches per launch -----------------------------------------------
    def sample_window(self, seeds: torch.Tensor, seed_counts: torch.Tensor, n_teams: int = 0, reuse: bool = True,
                      slot: int = 0, table_slots: int = 0, timing=None):
        """``seeds`` int32[n_batches, batch_size] on the GPU, ``seed_counts`` int32[n_batches].

        Returns the device-resident ``fastgl.FusedBatch``; batch ``b`` draws with the same Philox counters
        ``sample_blocks`` would use for the ``b``-th call, so both paths give identical blocks.  With ``reuse`` the
        result lives in buffers kept per geometry and ``slot``: a caller that samples the next window while the
        previous one is still being consumed alternates the slot.  ``table_slots`` caps the per-team hashtable
        (0 = sized for the worst case); a table that turns out too small is reported through the status word."""
        key = (seeds.size(0), seeds.size(1), seeds.device, slot)
        out = self._window_out.get(key) if reuse else None
        ctr = self.batch_counter * 8
        self.batch_counter += seeds.size(0)
        fb = fastgl.sample_map_fused(self.edge_ptr, self.edge_src, seeds, seed_counts, list(reversed(self.fanouts)),
                                     replace=self.replace, rng_seed=self.rng_seed, rng_ctr=ctr, n_teams=n_teams, out=out,
                                     table_slots=table_slots, timing=timing)
        if reuse:
            self._window_out[key] = fb
        return fb

    @staticmethod
    def window_blocks(fb, b: int):
        """``(input_nodes, blocks)`` of mini-batch ``b`` of a window (reads the counts back once per window)."""
        blocks = [Block(ptr, src, n_src, n_dst) for ptr, src, n_src, n_dst in fb.blocks(b)]
        return fb.input_nodes(b), blocks
