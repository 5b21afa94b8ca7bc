"""Host-side companions of the ``fastgl`` ops: synthetic graphs, the Fused-Map sampler, the GNN layers,
the Match-Reorder scheduler and the data-parallel trainer (mirrors of the reference's FusedMapSampler.py,
GraphConv.py, utilis.py / MatchReorderServer.py and the hot loop of train_fastgl.py)."""
