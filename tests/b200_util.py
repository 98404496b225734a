"""Builds a torchbiggraph_b200 model + trainer from a golden step fixture / oracle state."""
import numpy as np
import torch

import torchbiggraph_b200 as T


def make_config(c, precision="fp32", k=1):
    ents = {"e": T.EntitySchema(num_partitions=1)}
    rhs_ent = "e"
    if c["separate"]:
        ents["f"] = T.EntitySchema(num_partitions=1)
        rhs_ent = "f"
    nrel = 1 if c["dyn"] else c["n_rel_std"]
    rels = [T.RelationSchema(name=f"r{i}", lhs="e", rhs=rhs_ent, operator=c["op"],
                             weight=(c["rel_weight"] if i == c["rel_idx"] else 1.0)) for i in range(nrel)]
    B, nb = c["B"], c["nb"]
    cfg_batch = max(B, 1) if nb == 0 else ((B - 1) // nb + 1) * nb
    return T.ConfigSchema(entities=ents, relations=rels, dimension=c["D"], comparator=c["comp"], loss_fn=c["loss"],
                          margin=c["margin"], lr=c["lr"], relation_lr=c["relation_lr"], batch_size=cfg_batch,
                          num_batch_negs=nb, num_uniform_negs=c["nu"], disable_lhs_negs=c["disable_lhs"],
                          disable_rhs_negs=c["disable_rhs"], dynamic_relations=c["dyn"],
                          num_dynamic_rels=(c["R"] if c["dyn"] else 0), precision=precision, batches_in_flight=k,
                          global_emb=bool(c.get("global_emb", False)), regularization_coef=c.get("reg_coef", 0.0), max_norm=c.get("max_norm")), rhs_ent


class Rig:
    """Model, trainer and tensors for one bucket, initialised from numpy arrays."""

    def __init__(self, c, W_lhs, G_lhs, W_rhs=None, G_rhs=None, theta_rhs=None, theta_lhs=None,
                 acc_rhs=None, acc_lhs=None, precision="fp32", k=1, device="cuda", glob=None):
        self.c = c
        cfg, rhs_ent = make_config(c, precision, k)
        self.cfg = cfg
        self.model = T.make_model(cfg, device)
        f32 = lambda a: torch.tensor(np.asarray(a, np.float32), device=device).contiguous()
        if theta_rhs is not None and self.model.rhs_op_table is not None:
            self.model.rhs_op_table.copy_(f32(theta_rhs))
        if theta_lhs is not None and self.model.lhs_op_table is not None:
            self.model.lhs_op_table.copy_(f32(theta_lhs))
        for ent, g in (glob or {}).items():                  # global embeddings {entity type: vector}
            self.model.global_embs["emb_" + ent].copy_(f32(g))
        self.trainer = T.B200Trainer(T.make_optimizer(cfg, self.model.parameters(), False),
                                     T.LOSS_FUNCTIONS.get_class(c["loss"])(margin=c["margin"]),
                                     [r.weight for r in cfg.relations])
        if acc_rhs is not None and self.model.rhs_op_table is not None:
            self.trainer.model_optimizer.sum_for(self.model.rhs_op_table).copy_(f32(acc_rhs))
        if acc_lhs is not None and self.model.lhs_op_table is not None:
            self.trainer.model_optimizer.sum_for(self.model.lhs_op_table).copy_(f32(acc_lhs))
        self.W_lhs = f32(W_lhs)
        self.model.set_embeddings("e", T.Side.LHS, self.W_lhs)
        self.opt_l = T.make_optimizer(cfg, [self.W_lhs], True)
        self.opt_l.sum_for(self.W_lhs).copy_(f32(G_lhs))
        self.trainer.partitioned_optimizers["e", 0] = self.opt_l
        if W_rhs is not None:
            self.W_rhs = f32(W_rhs)
            self.opt_r = T.make_optimizer(cfg, [self.W_rhs], True)
            self.opt_r.sum_for(self.W_rhs).copy_(f32(G_rhs))
            self.trainer.partitioned_optimizers[rhs_ent, 0] = self.opt_r
        else:
            self.W_rhs, self.opt_r = self.W_lhs, self.opt_l
        self.model.set_embeddings(rhs_ent, T.Side.RHS, self.W_rhs)

    @classmethod
    def from_fixture(cls, c, z, **kw):
        sep = c["separate"]
        return cls(c, z["W_lhs0"], z["G_lhs0"], z["W_rhs0"] if sep else None, z["G_rhs0"] if sep else None,
                   z["theta_rhs0"] if "theta_rhs0" in z else None,
                   z["theta_lhs0"] if ("theta_lhs0" in z and c["dyn"]) else None,
                   glob={e: z[f"glob_{e}0"] for e in ("e", "f") if f"glob_{e}0" in z.files} or None, **kw)

    @classmethod
    def from_oracle_state(cls, c, st, **kw):
        sep = not st.shared
        glob = gacc = None
        if st.glob_lhs is not None:
            glob, gacc = {"e": st.glob_lhs}, {"e": st.gacc_lhs}
            if st.glob_rhs is not st.glob_lhs:
                glob["f"], gacc["f"] = st.glob_rhs, st.gacc_rhs
        rig = cls(c, st.W_lhs, st.G_lhs, st.W_rhs if sep else None, st.G_rhs if sep else None,
                  st.theta_rhs, st.theta_lhs, st.acc_rhs, st.acc_lhs, glob=glob, **kw)
        for ent, a in (gacc or {}).items():
            rig.trainer.model_optimizer.sum_for(rig.model.global_embs["emb_" + ent]).copy_(
                torch.tensor(np.asarray(a, np.float32), device=rig.W_lhs.device))
        return rig

    def edges(self, lhs, rhs, rel, weight=None):
        t = lambda a: torch.tensor(np.asarray(a, np.int64))
        w = None if weight is None else torch.tensor(np.asarray(weight, np.float32))
        return T.EdgeList(T.EntityList.from_tensor(t(lhs)), T.EntityList.from_tensor(t(rhs)), t(rel), w)

    def glob(self, ent="e"):
        return self.model.global_embs["emb_" + ent].cpu().numpy()

    def gacc(self, ent="e"):
        return self.trainer.model_optimizer.sum_for(self.model.global_embs["emb_" + ent]).cpu().numpy()

    def G(self, side="lhs"):
        opt, w = (self.opt_l, self.W_lhs) if side == "lhs" else (self.opt_r, self.W_rhs)
        return opt.sum_for(w).cpu().numpy()

    def acc(self, side="rhs"):
        tab = self.model.rhs_op_table if side == "rhs" else self.model.lhs_op_table
        return None if tab is None else self.trainer.model_optimizer.sum_for(tab).cpu().numpy()

    def theta(self, side="rhs"):
        tab = self.model.rhs_op_table if side == "rhs" else self.model.lhs_op_table
        return None if tab is None else tab.cpu().numpy()
