"""The CPU restatement of the reference's native edge utilities (oracle/pbg_edges.py) against outputs of the
reference module itself (torchbiggraph/util.cpp compiled by oracle/build_ref.py, recorded in
tests/golden/edges_*.npz by tests/golden/make_edges_golden.py): bit for bit."""
import glob
import os

import numpy as np
import pytest

from golden_util import GOLDEN
from oracle import pbg_edges as E


def edge_cases():
    return sorted(os.path.basename(p)[len("edges_"):-len(".npz")] for p in glob.glob(os.path.join(GOLDEN, "edges_*.npz")))


def load_edges(name):
    z = np.load(os.path.join(GOLDEN, f"edges_{name}.npz"))
    R = len(z["counts_l"])
    return z, [z[f"lperm_{i}"] for i in range(R)], [z[f"rperm_{i}"] for i in range(R)]


def test_golden_cases_exist():
    assert len(edge_cases()) >= 6


@pytest.mark.parametrize("name", edge_cases())
def test_sub_bucket_matches_the_reference_module(name):
    z, lp, rp = load_edges(name)
    res, (lo, ro, relo), counts = E.sub_bucket(z["lhs"], z["rhs"], z["rel"], z["counts_l"].tolist(), lp, z["counts_r"].tolist(), rp,
                                               int(z["n_l"]), int(z["n_r"]), bool(z["dyn"]))
    assert np.array_equal(counts, z["sub_counts"])
    assert np.array_equal(lo, z["lhs_out"]) and np.array_equal(ro, z["rhs_out"]) and np.array_equal(relo, z["rel_out"])
    assert sum(len(v[0]) for v in res.values()) == len(z["lhs"])


@pytest.mark.parametrize("name", edge_cases())
def test_shuffle_and_reverse_permutation_match_the_reference_module(name):
    z, _, _ = load_edges(name)
    assert np.array_equal(E.shuffle(z["table"], z["perm"]), z["table_shuffled"])
    assert np.array_equal(E.shuffle(z["ids"], z["perm"]), z["ids_shuffled"])
    rev = E.reverse_permutation(z["perm"])
    assert np.array_equal(rev, z["perm_reversed"])
    # shuffling by the reverse permutation undoes the shuffle (train_gpu.py:505, 630-632)
    assert np.array_equal(E.shuffle(z["table_shuffled"], rev), z["table"])


def test_shuffle_refuses_out_of_range_permutations():
    with pytest.raises(ValueError):
        E.shuffle(np.zeros((3, 2)), np.array([0, 1, 3]))
    with pytest.raises(ValueError):
        E.shuffle(np.zeros((3, 2)), np.array([0, 1]))
