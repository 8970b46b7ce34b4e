"""Generates tests/golden/*.npz by running the REFERENCE's own CPU code (oracle/_ref/gege_ref.so, built by
`make -C oracle` from the reference checkout) on the seeded cases of tests/workloads.py.

Run from the repository root where the reference checkout is available:  python tests/golden/make_golden.py
The fixtures hold inputs and the reference's outputs, so the tests need neither the checkout nor this script.
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "oracle" / "_ref"))
sys.path.insert(0, str(ROOT / "tests"))
import gege_ref  # noqa: E402
import workloads  # noqa: E402


def t(a):
    return None if a is None else torch.from_numpy(a)


def main():
    torch.set_num_threads(1)
    out_dir = Path(__file__).resolve().parent
    for name in workloads.GOLDEN_CASES:
        c = workloads.golden_case(name)
        B, C, N, D, R, U = c.dims
        has_rel = c.rel is not None
        model = gege_ref.RefModel(c.kind, max(R, 1), D, c.inv_rel is not None, c.lr, c.lr)
        if has_rel:
            model.set_relations(t(c.rel), t(c.inv_rel) if c.inv_rel is not None else torch.Tensor())
        ref_filter = gege_ref.deg_negative_local_filter(t(c.deg_rows), t(c.edges)).numpy() if c.deg_rows is not None else np.empty((0, 2), np.int64)
        assert np.array_equal(ref_filter, c.filt), "workloads.deg_filter disagrees with the reference filter"
        out = model.train_batch(t(c.edges), t(c.emb), t(c.state), t(c.dst_negs), t(c.src_negs), t(c.filt),
                                t(c.filt) if c.src_negs is not None else None, True, True)
        rels = model.get_relations() if has_rel else []
        save = dict(edges=c.edges, emb=c.emb, state=c.state, dst_negs=c.dst_negs, filt=c.filt, lr=np.float32(c.lr),
                    kind=np.array(c.kind))
        for k, v in (("rel", c.rel), ("inv_rel", c.inv_rel), ("src_negs", c.src_negs), ("deg_rows", c.deg_rows)):
            if v is not None:
                save[k] = v
        for k, v in out.items():
            save["ref_" + k] = v.numpy()
        if has_rel:
            save["ref_rel_after"], save["ref_rel_state_after"] = rels[0].numpy(), rels[1].numpy()
            if c.inv_rel is not None:
                save["ref_inv_rel_after"], save["ref_inv_rel_state_after"] = rels[2].numpy(), rels[3].numpy()
        np.savez_compressed(out_dir / f"{name}.npz", **save)
        print(name, "loss", float(out["loss"]), {k: tuple(v.shape) for k, v in out.items()})


if __name__ == "__main__":
    main()
