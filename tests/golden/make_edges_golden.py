#!/usr/bin/env python3
"""Records outputs of the reference's own native module (torchbiggraph/util.cpp, compiled by
oracle/build_ref.py) for the deterministic edge utilities: reverse_permutation, shuffle, sub_bucket.

    python oracle/build_ref.py --reference /path/to/PyTorch-BigGraph
    python tests/golden/make_edges_golden.py

Writes tests/golden/edges_<case>.npz: seeded inputs and what the reference returned for them.  The CPU
oracle (oracle/pbg_edges.py) and the CUDA entry points are both held to these bit for bit."""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle.build_ref import load_built  # noqa: E402

CASES = {
    # name: edges, relations, lhs / rhs entity counts per relation, sub-parts, dynamic, host threads of the reference run
    "one_relation_2x2": dict(E=5000, counts_l=[1000], counts_r=[1000], n_l=2, n_r=2, dyn=False, threads=3, shared=True),
    "halves_of_the_rhs": dict(E=4000, counts_l=[777], counts_r=[1501], n_l=1, n_r=2, dyn=False, threads=4, shared=False),
    "three_relations_two_types": dict(E=6000, counts_l=[500, 500, 901], counts_r=[500, 901, 500], n_l=4, n_r=3, dyn=False,
                                      threads=5, shared=False),
    "dynamic_relations_8x8": dict(E=20000, counts_l=[4099], counts_r=[4099], n_l=8, n_r=8, dyn=True, threads=7, shared=True,
                                  num_dyn=37),
    "empty_bucket": dict(E=0, counts_l=[10], counts_r=[10], n_l=2, n_r=2, dyn=False, threads=2, shared=True),
    "uneven_sub_partitions": dict(E=3000, counts_l=[10], counts_r=[7], n_l=4, n_r=3, dyn=False, threads=1, shared=False),
}


def main():
    C = load_built()
    if C is None:
        raise SystemExit("oracle/_ref/_C.so is missing: run oracle/build_ref.py first")
    for name, c in CASES.items():
        rng = np.random.default_rng(abs(hash(name)) % 2**31 if False else sum(map(ord, name)))
        R = len(c["counts_l"])
        # one permutation per entity count (relations over the same type share it, as train_gpu.py:499-509 does)
        perms = {}
        for cnt in set(c["counts_l"]) | set(c["counts_r"]):
            perms[cnt] = rng.permutation(cnt).astype(np.int64)
        lperms = [perms[x] for x in c["counts_l"]]
        rperms = [perms[x] if c["shared"] or x not in c["counts_l"] else rng.permutation(x).astype(np.int64) for x in c["counts_r"]]
        E = c["E"]
        rel_types = rng.integers(0, R, E)
        rel = rng.integers(0, c.get("num_dyn", R), E) if c["dyn"] else rel_types
        pick = np.zeros(E, np.int64) if c["dyn"] else rel_types
        lhs = (rng.random(E) * np.asarray(c["counts_l"])[pick]).astype(np.int64)
        rhs = (rng.random(E) * np.asarray(c["counts_r"])[pick]).astype(np.int64)
        t = lambda a: torch.tensor(np.asarray(a, np.int64))
        lo, ro, relo = torch.empty(E, dtype=torch.long), torch.empty(E, dtype=torch.long), torch.empty(E, dtype=torch.long)
        res = C.sub_bucket(t(lhs), t(rhs), t(rel), list(c["counts_l"]), [t(p) for p in lperms], list(c["counts_r"]),
                           [t(p) for p in rperms], lo, ro, relo, c["n_l"], c["n_r"], c["threads"], c["dyn"])
        counts = np.array([len(res[i, j][0]) for i in range(c["n_l"]) for j in range(c["n_r"])], np.int64)
        # shuffle / reverse_permutation on the same case: a row permutation of an [E, 3] int64 edge table and of a float table
        perm = rng.permutation(max(E, 1)).astype(np.int64)[:E] if E else np.zeros(0, np.int64)
        if E:
            perm = rng.permutation(E).astype(np.int64)
        table = rng.standard_normal((E, 5)).astype(np.float32)
        ids = rng.integers(0, 10**12, E)
        tt, ti = torch.tensor(table.copy()), torch.tensor(ids.copy())
        if E:
            C.shuffle(tt, t(perm), 3)
            C.shuffle(ti, t(perm), 2)
            rev = C.reverse_permutation(t(perm), 3).numpy()
        else:
            rev = np.zeros(0, np.int64)
        out = dict(lhs=lhs, rhs=rhs, rel=rel, n_l=c["n_l"], n_r=c["n_r"], dyn=c["dyn"], counts_l=np.array(c["counts_l"]),
                   counts_r=np.array(c["counts_r"]), lhs_out=lo.numpy(), rhs_out=ro.numpy(), rel_out=relo.numpy(),
                   sub_counts=counts, perm=perm, table=table, ids=ids, table_shuffled=tt.numpy(), ids_shuffled=ti.numpy(),
                   perm_reversed=rev)
        for i, p in enumerate(lperms):
            out[f"lperm_{i}"] = p
        for i, p in enumerate(rperms):
            out[f"rperm_{i}"] = p
        np.savez_compressed(os.path.join(HERE, f"edges_{name}.npz"), **out)
        print(name, "edges", E, "sub-bucket sizes", counts.tolist())


if __name__ == "__main__":
    main()
