"""The allocation-free RowAdagrad entry point (pbg_row_adagrad_static) against the context-based
one (pbg_row_adagrad).  It exists for callers that cannot allocate device memory -- all of HBM
already belongs to partitions, or another allocator owns the device -- so it works out of a fixed
scratch array inside the library.  Collected last on purpose: if it fails, a run that stops at the
first failure has already been through every other test.  Calls go through the C ABI."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL = 1e-4     # the tolerance of the other GPU parity tests


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def test_static_entry_point_matches_context_entry_point_twice_in_a_row():
    from b200_util import Rig
    from torchbiggraph_b200 import _lib
    L = _lib.lib()
    rng = np.random.default_rng(7)
    N, D = 3000, 200
    c = dict(D=D, N=N, N2=N, dyn=False, R=1, separate=False, id_range=None, steps=1, w_scale=0.1,
             disable_lhs=False, disable_rhs=False, n_rel_std=1, rel_idx=0, rel_weight=1.0, margin=0.1,
             lr=0.1, relation_lr=None, op="none", comp="dot", loss="softmax", B=1000, nb=50, nu=50, name="na")
    W0 = rng.standard_normal((N, D)).astype(np.float32)
    G0 = rng.random(N).astype(np.float32)
    rig = Rig(c, W0, G0, k=5)                              # owns a context (sort capacity 20000 rows)
    nat = rig.trainer._context(rig.model, 1000)
    Wa, Ga = rig.W_lhs, rig.opt_l.sum_for(rig.W_lhs)       # updated through the context
    Wb, Gb = Wa.clone(), Ga.clone()                        # updated through the static entry point
    for call, n in enumerate((5000, 16384)):               # second call: the stated maximum
        rows = torch.tensor(rng.integers(0, 400, n)).cuda()          # many duplicate rows
        grads = torch.tensor(rng.standard_normal((n, D)).astype(np.float32)).cuda()
        _lib.check(L.pbg_row_adagrad(nat.ctx, _ptr(Wa), _ptr(Ga), N, _ptr(rows), _ptr(grads), n, 0.05), nat.ctx)
        st = L.pbg_row_adagrad_static(_ptr(Wb), _ptr(Gb), N, D, _ptr(rows), _ptr(grads), n, 0.05, None)
        assert st == 0, L.pbg_status_string(st)
        torch.cuda.synchronize()
        np.testing.assert_allclose(Wb.cpu().numpy(), Wa.cpu().numpy(), rtol=RTOL, atol=1e-6, err_msg=f"call {call}")
        np.testing.assert_allclose(Gb.cpu().numpy(), Ga.cpu().numpy(), rtol=RTOL, atol=1e-7, err_msg=f"call {call}")
    assert not np.array_equal(Wb.cpu().numpy(), W0)        # the calls did change the table


def test_static_entry_point_rejects_sizes_beyond_its_scratch():
    from torchbiggraph_b200 import _lib
    L = _lib.lib()
    D, n = 64, 16385
    W = torch.zeros(10, D, device="cuda"); G = torch.zeros(10, device="cuda")
    rows = torch.zeros(n, dtype=torch.long, device="cuda"); grads = torch.ones(n, D, device="cuda")
    st = L.pbg_row_adagrad_static(_ptr(W), _ptr(G), 10, D, _ptr(rows), _ptr(grads), n, 0.1, None)
    assert st == _lib.PBG_ERR_TOO_LARGE
    assert b"maximum" in L.pbg_status_string(st)
    torch.cuda.synchronize()
    assert float(W.abs().sum()) == 0.0                     # nothing was touched
    st = L.pbg_row_adagrad_static(_ptr(W), _ptr(G), 10, 30, _ptr(rows), _ptr(grads), 4, 0.1, None)
    assert st == _lib.PBG_ERR_UNSUPPORTED                  # dim must be a multiple of 4


def _numpy_row_adagrad(W, G, rows, grads, lr):
    """RowAdagrad.step on a sparse gradient in float64 (torchbiggraph/row_adagrad.py:80-96): duplicates are
    summed, G += mean(g^2), w -= lr g / (sqrt(G) + 1e-10).  Rows outside the table are left out."""
    W, G = W.astype(np.float64), G.astype(np.float64)
    order = np.argsort(rows, kind="stable")
    r, g = rows[order], grads.astype(np.float64)[order]
    ok = (r >= 0) & (r < W.shape[0])
    r, g = r[ok], g[ok]
    uniq, start = np.unique(r, return_index=True)
    total = np.add.reduceat(g, start, axis=0)
    G[uniq] += (total * total).mean(axis=1)
    W[uniq] -= lr * total / (np.sqrt(G[uniq]) + 1e-10)[:, None]
    return W, G


def test_static_entry_point_matches_numpy_at_its_maximum_and_reports_bad_rows():
    """The entry point alone (no context anywhere in this test) against a float64 NumPy step at the
    stated maximum of 16384 gradient rows; then a call with one row id past the table and one negative
    id, which must come back as PBG_ERR_INDEX_RANGE with those two gradient rows left out and every
    other row stepped; then a clean call, which must return PBG_OK again -- the error word lives in the
    array every call shares, so this shows that a call starts from a cleared one."""
    from torchbiggraph_b200 import _lib
    L = _lib.lib()
    rng = np.random.default_rng(11)
    N, D, n = 5000, 128, 16384
    W = rng.standard_normal((N, D)).astype(np.float32)
    G = rng.random(N).astype(np.float32)
    Wd, Gd = torch.tensor(W).cuda(), torch.tensor(G).cuda()
    Wn, Gn = W, G
    for call, bad in enumerate((False, True, False)):
        rows = rng.integers(0, 700, n)
        if bad:
            rows[123], rows[4567] = N, -3
        grads = rng.standard_normal((n, D)).astype(np.float32)
        rd, gd = torch.tensor(rows).cuda(), torch.tensor(grads).cuda()
        st = L.pbg_row_adagrad_static(_ptr(Wd), _ptr(Gd), N, D, _ptr(rd), _ptr(gd), n, 0.05, None)
        assert st == (_lib.PBG_ERR_INDEX_RANGE if bad else 0), (call, L.pbg_status_string(st))
        Wn, Gn = _numpy_row_adagrad(Wn, Gn, rows, grads, 0.05)
        torch.cuda.synchronize()
        np.testing.assert_allclose(Wd.cpu().numpy(), Wn, rtol=RTOL, atol=1e-6, err_msg=f"call {call}")
        np.testing.assert_allclose(Gd.cpu().numpy(), Gn, rtol=RTOL, atol=1e-7, err_msg=f"call {call}")
        Wn, Gn = Wd.cpu().numpy(), Gd.cpu().numpy()        # the next call starts from the device's fp32 values
