"""Regenerates tests/golden/hotpath_small.npz from the numpy oracle (oracle/oracle_np.py).

The reference ships no golden vectors, tests or CPU code path, so these fixtures pin the oracle against
itself over time (and the C restatement and the CUDA kernels against it); they are NOT outputs of the
reference.  Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from conftest import make_graph  # noqa: E402
from oracle import oracle_np as on  # noqa: E402


def main():
    indptr, indices = make_graph(300, 8, seed=3, hub=60)
    rng = np.random.default_rng(11)
    seeds = rng.choice(300, size=24, replace=False).astype(np.int32)
    seeds[0] = 0  # the hub
    out = dict(indptr=indptr, indices=indices, seeds=seeds)
    for name, replace in (("norep", False), ("rep", True)):
        ptr, src, dst = on.sample(indptr, indices, seeds, 5, replace=replace, rng_seed=12345, rng_ctr=3)
        sl, dl, uniq = on.map_edges(src, dst, seeds)
        out.update({f"{name}_ptr": ptr, f"{name}_src": src, f"{name}_dst": dst, f"{name}_src_local": sl,
                    f"{name}_dst_local": dl, f"{name}_unique": uniq})
    inputs, _, blocks = on.sample_blocks(indptr, indices, seeds, [4, 3], rng_seed=99, rng_ctr=16)
    out["mh_inputs"] = inputs
    for i, blk in enumerate(blocks):
        out[f"mh_ptr{i}"] = blk["indptr"]
        out[f"mh_src{i}"] = blk["src_local"]
    blk = blocks[0]
    x = rng.standard_normal((blk["n_src"], 6)).astype(np.float32)
    dy = rng.standard_normal((blk["n_dst"], 6)).astype(np.float32)
    src_deg = np.maximum(on.cal_deg(blk["src_local"], blk["n_src"]), 1)
    dst_deg = np.maximum(np.diff(blk["indptr"]), 1).astype(np.int32)
    out.update(x=x, dy=dy, src_deg=src_deg, dst_deg=dst_deg)
    for mode, tag in ((on.MODE_SUM, "sum"), (on.MODE_MEAN, "mean"), (on.MODE_SYMNORM, "sym")):
        out[f"fwd_{tag}"] = on.aggregate_fwd(mode, blk["indptr"], blk["src_local"], x, blk["n_dst"], src_deg, dst_deg)
        out[f"bwd_{tag}"] = on.aggregate_bwd(mode, blk["indptr"], blk["src_local"], dy, blk["n_src"], src_deg, dst_deg)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "hotpath_small.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
