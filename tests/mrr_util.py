"""Planted-structure graphs and a plain NumPy MRR evaluator shared by the script that records the
reference's MRR (tests/golden/make_mrr_golden.py) and by the GPU end-to-end test."""
import numpy as np

CASES = {
    # name: entities, relations, edges, noise, dim, operator, dynamic, epochs (+ overrides of COMMON)
    "std_translation": dict(N=3000, R=1, E=40000, noise=0.2, D=32, op="translation", dyn=False, epochs=6),
    "dyn_complex_diagonal": dict(N=3000, R=8, E=40000, noise=0.2, D=32, op="complex_diagonal", dyn=True, epochs=6),
    # the 15k-entity multi-relation configuration at its full size: 1345 relations with Zipf(1.0) frequencies,
    # 483,142 edges, dim 400, complex_diagonal / dot / softmax with dynamic relations, batches of 5000 cut into
    # chunks of 1000 batch negatives, no uniform negatives (97 batches per epoch: 14 batches in flight are a
    # seventh of an epoch, as in the benchmark run)
    "kg15k_shape": dict(N=14951, R=1345, E=483142, noise=0.2, D=400, op="complex_diagonal", dyn=True, epochs=3,
                        batch=5000, nb=1000, nu=0, rel_zipf=1.0, held_out=2000),
    # power-law endpoints (Zipf 1.1 over permuted ids: the top row collects about a tenth of all endpoints, so a
    # wave of batches in flight reads hub rows that many of its own batches update), dim 256, 100 + 100 negatives
    "powerlaw_hubs": dict(N=20000, R=1, E=200000, noise=0.2, D=256, op="translation", dyn=False, epochs=8,
                          batch=1000, nb=100, nu=100, endpoint_zipf=1.1, held_out=5000),
}
COMMON = dict(comp="dot", loss="softmax", lr=0.1, batch=500, nb=50, nu=50, init_scale=1e-3, held_out=1500)


def setting(case, key):
    """A training setting of the case: its own value if it has one, else the common one."""
    return CASES[case].get(key, COMMON[key])


def planted_graph(case, seed=0):
    """Each relation is a random permutation map u -> pi_r(u); a `noise` fraction of edges gets a
    uniformly random destination.  Returns (train lhs, rhs, rel), (test lhs, rhs, rel), initial W."""
    c = CASES[case]
    rng = np.random.default_rng(seed)
    perms = [rng.permutation(c["N"]) for _ in range(c["R"])]
    if "rel_zipf" in c:
        pr = np.arange(1, c["R"] + 1, dtype=np.float64) ** -c["rel_zipf"]
        rel = rng.choice(c["R"], c["E"], p=pr / pr.sum())
    else:
        rel = rng.integers(0, c["R"], c["E"])
    if "endpoint_zipf" in c:
        pe = np.arange(1, c["N"] + 1, dtype=np.float64) ** -c["endpoint_zipf"]
        lhs = rng.permutation(c["N"])[rng.choice(c["N"], c["E"], p=pe / pe.sum())]
    else:
        lhs = rng.integers(0, c["N"], c["E"])
    rhs = np.array([perms[r][u] for r, u in zip(rel, lhs)])
    noisy = rng.random(c["E"]) < c["noise"]
    rhs[noisy] = rng.integers(0, c["N"], int(noisy.sum()))
    h = c.get("held_out", COMMON["held_out"])
    clean = np.flatnonzero(~noisy)
    test_idx = clean[:h]
    mask = np.ones(c["E"], bool)
    mask[test_idx] = False
    W0 = (rng.standard_normal((c["N"], c["D"])) * COMMON["init_scale"]).astype(np.float32)
    tr = (lhs[mask], rhs[mask], rel[mask])
    te = (lhs[test_idx], rhs[test_idx], rel[test_idx])
    return tr, te, W0


def epoch_order(n, epoch, seed=0):
    return np.random.default_rng(1000 * seed + epoch).permutation(n)


def mrr_rhs(case, W, theta_lhs_or_rhs, test):
    """Rank of the true destination among ALL entities (ties count against the model).
    standard relations: score(u, v') = <u, op_rhs(v')>; dynamic: <op_lhs[r](u), v'> (model.py:705-758)."""
    c = CASES[case]
    lhs, rhs, rel = test
    W = W.astype(np.float64)
    th = None if theta_lhs_or_rhs is None else theta_lhs_or_rhs.astype(np.float64)

    def op(x, p):
        if c["op"] == "translation":
            return x + p
        h = c["D"] // 2
        a, b, pr, pi = x[..., :h], x[..., h:], p[..., :h], p[..., h:]
        return np.concatenate([a * pr - b * pi, a * pi + b * pr], -1)

    rr = []
    if not c["dyn"]:
        cand = op(W, th[0][None, :])
        for u, v in zip(lhs, rhs):
            s = cand @ W[u]
            rr.append(1.0 / (1 + int((s > s[v]).sum())))
    else:
        for u, v, r in zip(lhs, rhs, rel):
            q = op(W[u][None, :], th[r][None, :])[0]
            s = W @ q
            rr.append(1.0 / (1 + int((s > s[v]).sum())))
    return float(np.mean(rr))
