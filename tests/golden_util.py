"""Helpers shared by the golden-fixture tests: load a step fixture into oracle/CUDA inputs."""
import glob
import json
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def step_fixture_names():
    return sorted(os.path.basename(p)[len("step_"):-len(".npz")] for p in glob.glob(os.path.join(GOLDEN, "step_*.npz")))


def load_step(name):
    z = np.load(os.path.join(GOLDEN, f"step_{name}.npz"))
    cfg = json.loads(str(z["config"]))
    return cfg, z


def oracle_config(c):
    from oracle.pbg_step import StepConfig
    weights = [1.0]
    if not c["dyn"]:
        weights = [c["rel_weight"] if i == c["rel_idx"] else 1.0 for i in range(c["n_rel_std"])]
    return StepConfig(dim=c["D"], operator=c["op"], comparator=c["comp"], loss=c["loss"], margin=c["margin"],
                      lr=c["lr"], relation_lr=c["relation_lr"], num_batch_negs=c["nb"], num_uniform_negs=c["nu"],
                      dynamic=c["dyn"], num_rels=(c["R"] if c["dyn"] else c["n_rel_std"]),
                      disable_lhs_negs=c["disable_lhs"], disable_rhs_negs=c["disable_rhs"],
                      relation_weights=weights, regularization_coef=c.get("reg_coef", 0.0), max_norm=c.get("max_norm"))


def oracle_state(c, z, dtype=np.float64):
    from oracle.pbg_step import BucketState
    W = z["W_lhs0"].astype(dtype)
    G = z["G_lhs0"].astype(dtype)
    if c["separate"]:
        W2, G2 = z["W_rhs0"].astype(dtype), z["G_rhs0"].astype(dtype)
    else:
        W2, G2 = W, G
    st = BucketState(W, G, W2, G2)
    if "theta_rhs0" in z:
        st.theta_rhs = z["theta_rhs0"].astype(dtype)
        st.acc_rhs = np.zeros_like(st.theta_rhs)
    if "theta_lhs0" in z and c["dyn"]:
        st.theta_lhs = z["theta_lhs0"].astype(dtype)
        st.acc_lhs = np.zeros_like(st.theta_lhs)
    if "glob_e0" in z.files:                       # global embeddings: lhs is entity type e, rhs is e or f
        st.glob_lhs = z["glob_e0"].astype(dtype)
        st.gacc_lhs = np.zeros_like(st.glob_lhs)
        if c["separate"]:
            st.glob_rhs = z["glob_f0"].astype(dtype)
            st.gacc_rhs = np.zeros_like(st.glob_rhs)
        else:
            st.glob_rhs, st.gacc_rhs = st.glob_lhs, st.gacc_lhs
    return st


def weight_of(c, z, step):
    """Per-edge weights of the step (EdgeList.weight), or None."""
    key = f"weight_{step}"
    return z[key] if key in z.files else None


def batch_of(c, z, step):
    rel = z[f"rel_{step}"]
    rel = rel if c["dyn"] else int(rel)
    ul = None if c["disable_lhs"] else z[f"ul_{step}"]
    ur = None if c["disable_rhs"] else z[f"ur_{step}"]
    return z[f"lhs_{step}"], z[f"rhs_{step}"], rel, ul, ur
