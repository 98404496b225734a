"""The device edge-list utilities (torchbiggraph_b200._C over pbg_reverse_permutation / pbg_shuffle_rows /
pbg_randperm / pbg_sub_bucket) against outputs of the reference's native module recorded in
tests/golden/edges_*.npz and against the CPU oracle: bit for bit (integer and byte work)."""
import numpy as np
import pytest
import torch

from oracle import pbg_edges as E
from test_oracle_edges import edge_cases, load_edges

pytestmark = pytest.mark.gpu


def _t(a):
    return torch.tensor(np.asarray(a)).cuda()


@pytest.mark.parametrize("name", edge_cases())
def test_sub_bucket_matches_the_reference_module(name):
    from torchbiggraph_b200 import _C
    z, lp, rp = load_edges(name)
    n = len(z["lhs"])
    lo, ro, relo = (torch.full((n,), -1, dtype=torch.long, device="cuda") for _ in range(3))
    res = _C.sub_bucket(_t(z["lhs"]), _t(z["rhs"]), _t(z["rel"]), z["counts_l"].tolist(), [_t(p) for p in lp],
                        z["counts_r"].tolist(), [_t(p) for p in rp], lo, ro, relo, int(z["n_l"]), int(z["n_r"]), 8, bool(z["dyn"]))
    assert np.array_equal(lo.cpu().numpy(), z["lhs_out"])
    assert np.array_equal(ro.cpu().numpy(), z["rhs_out"])
    assert np.array_equal(relo.cpu().numpy(), z["rel_out"])
    counts = [len(res[i, j][0]) for i in range(int(z["n_l"])) for j in range(int(z["n_r"]))]
    assert counts == z["sub_counts"].tolist()
    start = 0
    for (i, j), (l, r, rl) in sorted(res.items()):             # the values are views of the output tensors
        assert l.data_ptr() == lo.data_ptr() + 8 * start and len(l) == len(r) == len(rl)
        start += len(l)


@pytest.mark.parametrize("name", edge_cases())
def test_shuffle_and_reverse_permutation_match_the_reference_module(name):
    from torchbiggraph_b200 import _C
    z, _, _ = load_edges(name)
    table, ids, perm = _t(z["table"]), _t(z["ids"]), _t(z["perm"])
    _C.shuffle(table, perm, 4)
    _C.shuffle(ids, perm, 4)
    assert np.array_equal(table.cpu().numpy(), z["table_shuffled"])
    assert np.array_equal(ids.cpu().numpy(), z["ids_shuffled"])
    rev = _C.reverse_permutation(perm, 4)
    assert np.array_equal(rev.cpu().numpy(), z["perm_reversed"])
    _C.shuffle(table, rev, 4)                                  # train_gpu.py:505, 630-632: back to the original order
    assert np.array_equal(table.cpu().numpy(), z["table"])


@pytest.mark.parametrize("row_bytes_case", ["embedding_rows_1024", "three_bytes", "int64_scalar", "odd_float_rows"])
def test_shuffle_row_widths(row_bytes_case):
    from torchbiggraph_b200 import _C
    rng = np.random.default_rng(3)
    n = 3001
    data = {"embedding_rows_1024": rng.standard_normal((n, 1024)).astype(np.float32),
            "three_bytes": rng.integers(0, 255, (n, 3)).astype(np.uint8),
            "int64_scalar": rng.integers(0, 10**15, n),
            "odd_float_rows": rng.standard_normal((n, 7, 3)).astype(np.float32)}[row_bytes_case]
    perm = rng.permutation(n)
    t = _t(data)
    _C.shuffle(t, _t(perm), 1)
    assert np.array_equal(t.cpu().numpy(), E.shuffle(data, perm))


def test_shuffle_errors_keep_the_reference_types():
    from torchbiggraph_b200 import _C
    t = torch.zeros(4, 2, device="cuda")
    with pytest.raises(ValueError, match="out-of-bound"):
        _C.shuffle(t, torch.tensor([0, 1, 2, 4], device="cuda"), 1)
    with pytest.raises(ValueError, match="same number"):
        _C.shuffle(t, torch.tensor([0, 1, 2], device="cuda"), 1)
    with pytest.raises(ValueError, match="int64"):
        _C.shuffle(t, torch.tensor([0, 1, 2, 3], device="cuda", dtype=torch.int32), 1)
    _C.shuffle(t, torch.tensor([1, 0, 3, 2], device="cuda"), 1)    # the context is still usable


def test_sub_bucket_reports_a_relation_outside_its_range():
    from torchbiggraph_b200 import _C
    perm = torch.arange(10, device="cuda")
    lhs = torch.tensor([1, 2, 3], device="cuda"); rel = torch.tensor([0, 5, 0], device="cuda")
    out = [torch.empty(3, dtype=torch.long, device="cuda") for _ in range(3)]
    with pytest.raises(RuntimeError, match="numRelations"):
        _C.sub_bucket(lhs, lhs.clone(), rel, [10], [perm], [10], [perm], *out, 2, 2, 1, False)
    with pytest.raises(RuntimeError, match="Inconsistent"):
        _C.sub_bucket(lhs, lhs.clone(), rel, [10, 10], [perm], [10], [perm], *out, 2, 2, 1, False)


@pytest.mark.parametrize("n", [1, 2, 1000, 269507, 3_000_001])
def test_randperm_is_a_seeded_uniform_permutation(n):
    from torchbiggraph_b200 import _C
    a = _C.randperm(n, 8, seed=5).cpu().numpy()
    assert E.check_permutation(a, n)
    assert np.array_equal(a, _C.randperm(n, 1, seed=5).cpu().numpy())          # fixed by the seed, not by num_threads
    if n >= 1000:
        b = _C.randperm(n, 8, seed=6).cpu().numpy()
        assert E.check_permutation(b, n) and not np.array_equal(a, b)
        # uniformity: the mean displacement of a uniform permutation is n / 3, and positions are uncorrelated with values
        disp = np.abs(a - np.arange(n)).mean()
        assert abs(disp - n / 3) < 0.05 * n
        assert abs(np.corrcoef(a, np.arange(n))[0, 1]) < 0.1


def test_full_size_bucket_split_in_halves_is_a_stable_partition():
    """A bucket of the benchmark's size (269,507 edges over two 302,974-row partitions) split into the two row
    halves of its rhs partition: sizes add up, every output offset lies inside its half, and an edge's position
    inside its half follows input order (checked against the oracle's stable argsort)."""
    from torchbiggraph_b200 import _C
    rng = np.random.default_rng(9)
    rows, n = 302_974, 269_507
    lhs, rhs = rng.integers(0, rows, n), rng.integers(0, rows, n)
    ident = torch.arange(rows, device="cuda")
    out = [torch.empty(n, dtype=torch.long, device="cuda") for _ in range(3)]
    res = _C.sub_bucket(_t(lhs), _t(rhs), torch.zeros(n, dtype=torch.long, device="cuda"), [rows], [ident], [rows], [ident],
                        *out, 1, 2, 1, False)
    _, (lo, ro, relo), counts = E.sub_bucket(lhs, rhs, np.zeros(n, np.int64), [rows], [np.arange(rows)], [rows], [np.arange(rows)], 1, 2, False)
    assert [len(res[0, 0][0]), len(res[0, 1][0])] == counts.tolist() and counts.sum() == n
    assert np.array_equal(out[0].cpu().numpy(), lo) and np.array_equal(out[1].cpu().numpy(), ro)
    half = -(-rows // 2)
    assert int(out[1].max()) < half
