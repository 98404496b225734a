"""CPU restatement (NumPy) of the reference's native edge utilities -- test infrastructure, never
imported by the product.  Each function follows torchbiggraph/util.cpp:

  reverse_permutation  util.cpp:103-125   res[perm[i]] = i
  shuffle              util.cpp:127-220   in place, row i moves to row perm[i]
  sub_bucket           util.cpp:260-423   stable split of a bucket's edges into N x M sub-buckets
  randperm             util.cpp:14-101    a seeded uniformly random permutation

The first three are deterministic and pinned bit for bit against the compiled reference module
(tests/golden/edges_*.npz, recorded by tests/golden/make_edges_golden.py).  randperm in the reference
is a Mersenne-Twister stream per host thread, so its output depends on the thread count; what callers
rely on is the contract (a permutation, fixed by the seed, uniformly distributed), and that contract is
what `check_permutation` states."""
import numpy as np


def reverse_permutation(perm):
    perm = np.asarray(perm, np.int64)
    out = np.empty_like(perm)
    out[perm] = np.arange(len(perm), dtype=np.int64)
    return out


def shuffle(rows, perm):
    """Returns the shuffled copy: out[perm[i]] = rows[i] (the reference does it in place by following
    the permutation's cycles, util.cpp:187-207)."""
    rows, perm = np.asarray(rows), np.asarray(perm, np.int64)
    if rows.shape[0] != perm.shape[0]:
        raise ValueError("Tensor and permutation must have the same number of elements on the first dimension")
    if len(perm) and (perm.min() < 0 or perm.max() >= len(perm)):
        raise ValueError("Permutation has out-of-bound values")
    out = np.empty_like(rows)
    out[perm] = rows
    return out


def sub_bucket(lhs, rhs, rel, lhs_counts, lhs_perms, rhs_counts, rhs_perms, n_lhs, n_rhs, dynamic_relations):
    """{(i, j): (lhs, rhs, rel)} plus the concatenated outputs.  An entity's offset goes through its
    type's permutation; the permuted offset // ceil(count / parts) is its sub-partition and the
    remainder its offset inside it (util.cpp:300-317, 374-390).  Edges keep their input order inside a
    sub-bucket (the per-thread offsets of util.cpp:344-362 are laid out in thread order, and every
    thread walks a contiguous range), sub-buckets follow each other in (i, j) row-major order."""
    lhs, rhs, rel = (np.asarray(a, np.int64) for a in (lhs, rhs, rel))
    relid = np.zeros_like(rel) if dynamic_relations else rel
    if len(rel) and relid.max() >= len(lhs_perms):
        raise ValueError("rel > numRelations")
    lsz = np.array([-(-c // n_lhs) for c in lhs_counts], np.int64)
    rsz = np.array([-(-c // n_rhs) for c in rhs_counts], np.int64)
    lo = np.empty_like(lhs)
    ro = np.empty_like(rhs)
    for r in np.unique(relid):
        m = relid == r
        lo[m] = np.asarray(lhs_perms[r], np.int64)[lhs[m]]
        ro[m] = np.asarray(rhs_perms[r], np.int64)[rhs[m]]
    lpart, rpart = lo // lsz[relid], ro // rsz[relid]
    key = lpart * n_rhs + rpart
    order = np.argsort(key, kind="stable")
    lhs_out, rhs_out, rel_out = (lo % lsz[relid])[order], (ro % rsz[relid])[order], rel[order]
    counts = np.bincount(key, minlength=n_lhs * n_rhs).astype(np.int64)
    ends = np.cumsum(counts)
    res = {}
    for i in range(n_lhs):
        for j in range(n_rhs):
            b = i * n_rhs + j
            s = slice(int(ends[b] - counts[b]), int(ends[b]))
            res[i, j] = (lhs_out[s], rhs_out[s], rel_out[s])
    return res, (lhs_out, rhs_out, rel_out), counts


def check_permutation(perm, n):
    """The contract of randperm: every value of range(n) exactly once."""
    perm = np.asarray(perm, np.int64)
    return perm.shape == (n,) and np.array_equal(np.sort(perm), np.arange(n, dtype=np.int64))
