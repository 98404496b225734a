"""The arithmetic of the bf16x6 precision tier, restated in NumPy (no GPU): an fp32 value as three
bf16 planes, and a dot product from the six plane products of order <= 2 accumulated in fp32.
Pins the two facts the tier rests on: the planes hold the value exactly, and dropping the three
products of order >= 3 costs less than fp32 accumulation itself."""
import numpy as np


def bf16_round(x):
    """fp32 -> nearest bf16 (ties to even), returned as fp32."""
    u = np.asarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def planes(x):
    x = np.asarray(x, np.float32)
    b0 = bf16_round(x)
    r1 = (x - b0).astype(np.float32)          # exact in fp32
    b1 = bf16_round(r1)
    r2 = (r1 - b1).astype(np.float32)         # exact in fp32
    b2 = bf16_round(r2)
    return b0, b1, b2


def test_three_planes_hold_an_fp32_value_exactly():
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(200000).astype(np.float32) * 10.0 ** rng.integers(-6, 6, 200000),
                        np.array([0.0, 1.0, -1.0, 3.1415927, 1e-20, -65504.0, 1.0000001], np.float32)]).astype(np.float32)
    b0, b1, b2 = planes(x)
    for b in (b0, b1, b2):                    # every plane is a bf16 value
        assert np.array_equal(b.view(np.uint32) & 0xFFFF, np.zeros(b.shape, np.uint32))
    s = b0.astype(np.float64) + b1.astype(np.float64) + b2.astype(np.float64)
    assert np.array_equal(s, x.astype(np.float64))


def test_six_plane_products_match_fp64_to_fp32_accumulation_level():
    rng = np.random.default_rng(1)
    K = 1024
    a = rng.standard_normal((64, K)).astype(np.float32)
    b = rng.standard_normal((48, K)).astype(np.float32)
    pa, pb = planes(a), planes(b)
    acc = np.zeros((64, 48), np.float32)
    # the order the kernel issues them in: smallest contributions first
    for i, j in ((2, 0), (0, 2), (1, 1), (1, 0), (0, 1), (0, 0)):
        acc = (acc + (pa[i].astype(np.float64) @ pb[j].astype(np.float64).T).astype(np.float32)).astype(np.float32)
    want = a.astype(np.float64) @ b.astype(np.float64).T
    scale = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64).T          # sum |a_k b_k|
    err = np.abs(acc - want) / scale
    assert err.max() < 2e-6
    # the products left out (order >= 3) are below 2^-23 of sum |a b|
    left = sum(np.abs(pa[i]).astype(np.float64) @ np.abs(pb[j]).astype(np.float64).T for i, j in ((1, 2), (2, 1), (2, 2)))
    assert (left / scale).max() < 2.0 ** -23


def test_three_products_on_two_planes_carry_sixteen_bits():
    """The bf16x3 tier: x ~ b0 + b1 (what two planes leave out is below 2^-16 of |x|) and a dot product
    from b1.b0 + b0.b1 + b0.b0.  What is left out -- b1.b1 and the third plane's products -- is below
    2^-15 of sum |a b| in the worst case; over K random-sign terms the error of the sum is far smaller
    than that bound, a few 1e-6 of the sum's own scale."""
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(200000) * 10.0 ** rng.integers(-6, 6, 200000)).astype(np.float32)
    b0, b1, _ = planes(x)
    two = b0.astype(np.float64) + b1.astype(np.float64)
    nz = x != 0
    assert (np.abs(two - x.astype(np.float64))[nz] / np.abs(x.astype(np.float64))[nz]).max() <= 2.0 ** -16
    K = 1024
    a = rng.standard_normal((64, K)).astype(np.float32)
    b = rng.standard_normal((48, K)).astype(np.float32)
    pa, pb = planes(a), planes(b)
    acc = np.zeros((64, 48), np.float32)
    for i, j in ((1, 0), (0, 1), (0, 0)):
        acc = (acc + (pa[i].astype(np.float64) @ pb[j].astype(np.float64).T).astype(np.float32)).astype(np.float32)
    want = a.astype(np.float64) @ b.astype(np.float64).T
    scale = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64).T
    err = np.abs(acc - want) / scale
    assert err.max() < 2.0 ** -15                       # the worst-case bound
    assert err.max() < 3e-6                             # measured over random-sign sums of 1024 terms
    rel = np.abs(acc - want) / np.sqrt((a.astype(np.float64) ** 2) @ (b.astype(np.float64) ** 2).T)   # against the sum's own scale
    assert np.sqrt((rel ** 2).mean()) < 1e-5
