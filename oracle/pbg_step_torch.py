"""fp32 PyTorch-on-CPU port of PyTorch-BigGraph's training step (TEST / BASELINE INFRASTRUCTURE ONLY).

Purpose: the timed CPU baseline of bench.py.  It issues the same ATen calls as the reference's
own CPU trainer -- F.embedding(sparse=True), torch.bmm / baddbmm, the torch.nn.functional loss
kernels, autograd, sparse-gradient coalesce + index_add_ -- so that its speed on the host cores
stands for the reference's (torchbiggraph/train_cpu.py:86-112 driven HOGWILD-style from
train_cpu.py:849-884).  The product never imports it.

Parity status: PINNED (tests/test_oracle_golden.py::test_torch_port_matches_reference runs it on
the reference-generated step fixtures).

Restates: model.py:57-75 (embedding, sampling), :159-303 (comparators), :478-856 (forward),
operators.py:49-157 & 197-338, losses.py:53-161, batching.py:139-150, row_adagrad.py:48-109,
async_adagrad.py:19-87.
"""
from typing import Optional

import torch
import torch.nn.functional as F


class StepModel:
    """Embedding tables + operator tables of one bucket, trained in place on the CPU."""

    def __init__(self, dim, operator="none", comparator="dot", loss="ranking", margin=0.1, lr=0.1,
                 relation_lr=None, num_batch_negs=50, num_uniform_negs=50, dynamic=False, num_rels=1,
                 relation_weights=(1.0,)):
        self.dim, self.op, self.cmp, self.loss, self.margin = dim, operator, comparator, loss, margin
        self.lr, self.rel_lr = lr, (lr if relation_lr is None else relation_lr)
        self.nb, self.nu, self.dynamic, self.num_rels = num_batch_negs, num_uniform_negs, dynamic, num_rels
        self.relation_weights = list(relation_weights)
        self.theta = {}     # side -> Parameter [R, dim]
        self.acc = {}
        if operator != "none":
            for side in (("rhs", "lhs") if dynamic else ("rhs",)):
                t = torch.zeros(num_rels, dim)
                if operator == "diagonal":
                    t.fill_(1.0)
                elif operator == "complex_diagonal":
                    t[:, : dim // 2] = 1.0
                self.theta[side] = torch.nn.Parameter(t)
                self.acc[side] = torch.zeros_like(t)

    def attach(self, W_lhs: torch.Tensor, G_lhs: torch.Tensor, W_rhs: torch.Tensor, G_rhs: torch.Tensor):
        """Tables may live in shared memory (HOGWILD workers update them without locks)."""
        self.W = {"lhs": W_lhs.requires_grad_(True), "rhs": W_rhs if W_rhs is W_lhs else W_rhs.requires_grad_(True)}
        self.G = {"lhs": G_lhs, "rhs": G_rhs}

    # ---- pieces of the forward pass ------------------------------------------------------------
    def _operator(self, x, side, rel):
        if self.op == "none":
            return x
        t = self.theta[side]
        p = t[rel] if torch.is_tensor(rel) else t[rel].unsqueeze(0)
        if p.dim() < x.dim():
            p = p.unsqueeze(-2)
        if self.op == "translation":
            return x + p
        if self.op == "diagonal":
            return x * p
        h = self.dim // 2
        a, b, pr, pi = x[..., :h], x[..., h:], p[..., :h], p[..., h:]
        return torch.cat([a * pr - b * pi, a * pi + b * pr], -1)

    def _prepare(self, x):
        if self.cmp != "cos":
            return x
        return x * x.norm(2, dim=-1).reciprocal().unsqueeze(-1)

    def _pos(self, a, b):
        if self.cmp in ("dot", "cos"):
            return (a * b).sum(-1)
        q = (a - b).pow(2).sum(-1)
        return -q if self.cmp == "squared_l2" else q.clamp_min(1e-30).sqrt().neg()

    def _neg(self, a, n):
        if self.cmp in ("dot", "cos"):
            return torch.bmm(a, n.transpose(-1, -2))
        asq, nsq = a.norm(dim=-1).pow(2), n.norm(dim=-1).pow(2)
        q = torch.baddbmm(nsq.unsqueeze(-2), a, n.transpose(-2, -1), alpha=-2).add(asq.unsqueeze(-1))
        return q.neg() if self.cmp == "squared_l2" else q.clamp_min(1e-30).sqrt().neg()

    def _loss(self, pos, neg):
        n, m = neg.shape
        if self.loss == "logistic":
            w = 1.0 / m if m > 0 else 0.0
            return (F.binary_cross_entropy_with_logits(pos, torch.ones_like(pos), reduction="sum")
                    + w * F.binary_cross_entropy_with_logits(neg, torch.zeros_like(neg), reduction="sum"))
        if n == 0 or m == 0:
            return torch.zeros((), requires_grad=True)
        if self.loss == "ranking":
            return F.margin_ranking_loss(neg, pos.unsqueeze(1), target=pos.new_full((1, 1), -1.0),
                                         margin=self.margin, reduction="sum")
        scores = torch.cat([pos.unsqueeze(1), neg.logsumexp(dim=1, keepdim=True)], dim=1)
        return F.cross_entropy(scores, pos.new_zeros((n,), dtype=torch.long), reduction="sum")

    def _direction(self, src_side, dst_side, src_ids, dst_ids, rel, usrc, udst, both_sides):
        """One pass: negatives on the src side (and on the dst side too when both_sides)."""
        B = src_ids.shape[0]
        P = min(self.nb, B) if self.nb > 0 else min(self.nu, B)
        C = (B - 1) // P + 1
        D = self.dim
        xs = self._prepare(F.embedding(src_ids, self.W[src_side], sparse=True))
        xd = self._prepare(self._operator(F.embedding(dst_ids, self.W[dst_side], sparse=True), dst_side, rel))
        pad = C * P - B
        if pad:
            xs = torch.cat([xs, xs.new_zeros((pad, D))])
            xd = torch.cat([xd, xd.new_zeros((pad, D))])
        xs, xd = xs.view(C, P, D), xd.view(C, P, D)
        last = B - (C - 1) * P
        ar = torch.arange(P)

        def negatives(pos, ids, side, apply_op):
            if ids is None:
                return None
            parts = [pos] if self.nb > 0 else []
            if ids.shape[1] > 0:
                u = F.embedding(ids, self.W[side], sparse=True)
                if apply_op:
                    u = self._operator(u, side, rel if not torch.is_tensor(rel) else rel)
                parts.append(self._prepare(u))
            return torch.cat(parts, dim=1) if parts else pos.new_zeros((C, 0, D))

        def mask(S):
            if self.nb > 0:
                S[:, ar, ar] = -1e9
                S[-1, :last, last:P] = -1e9
            return S.flatten(0, 1)[:B]

        pos = self._pos(xs, xd).flatten(0, 1)[:B]
        nsrc = negatives(xs, usrc, src_side, False)
        out_src = mask(self._neg(xd, nsrc)) if nsrc is not None else pos.new_zeros((B, 0))
        out_dst = None
        if both_sides:
            ndst = negatives(xd, udst, dst_side, True)
            out_dst = mask(self._neg(xs, ndst)) if ndst is not None else pos.new_zeros((B, 0))
        return pos, out_src, out_dst

    # ---- one training step -----------------------------------------------------------------------
    def train_batch(self, lhs, rhs, rel, ul=None, ur=None, draw=True):
        """lhs, rhs: LongTensor [B]; rel: int or LongTensor [B]; ul / ur: [C, U] ids, or drawn here
        with torch.randint in the reference's order (lhs side first) when None and draw."""
        for p in list(self.theta.values()) + list({id(v): v for v in self.W.values()}.values()):
            p.grad = None
        B = lhs.shape[0]
        P = min(self.nb, B) if self.nb > 0 else min(self.nu, B)
        C = (B - 1) // P + 1
        if draw and ul is None:
            ul = torch.randint(0, self.W["lhs"].shape[0], (C, self.nu))
        if draw and ur is None:
            ur = torch.randint(0, self.W["rhs"].shape[0], (C, self.nu))
        if not self.dynamic:
            pos, sl, sr = self._direction("lhs", "rhs", lhs, rhs, int(rel), ul, ur, True)
            lp = rp = pos
            w = self.relation_weights[int(rel)]
        else:
            lp, sl, _ = self._direction("lhs", "rhs", lhs, rhs, rel, ul, None, False)
            rp, sr, _ = self._direction("rhs", "lhs", rhs, lhs, rel, ur, None, False)
            w = self.relation_weights[0]
        loss = w * (self._loss(lp, sl) + self._loss(rp, sr))
        stats = {"loss": float(loss.detach()), "violators_lhs": int((sl > lp.unsqueeze(1)).sum()),
                 "violators_rhs": int((sr > rp.unsqueeze(1)).sum()), "count": B}
        loss.backward()
        with torch.no_grad():
            for side, t in self.theta.items():          # AsyncAdagrad, dense
                if t.grad is None:
                    continue
                g = t.grad
                self.acc[side].add_(g * g)
                t.addcdiv_(g, self.acc[side].sqrt().add_(1e-10), value=-self.rel_lr)
            for side in (("lhs",) if self.W["lhs"] is self.W["rhs"] else ("lhs", "rhs")):   # RowAdagrad, sparse
                Wt = self.W[side]
                if Wt.grad is None:
                    continue
                g = Wt.grad.coalesce()
                idx, val = g._indices()[0], g._values()
                if idx.numel() == 0:
                    continue
                local = self.G[side][idx]
                delta = (val * val).mean(1)
                self.G[side].index_add_(0, idx, delta)
                local += delta
                std = local.sqrt_().add_(1e-10).unsqueeze(1)
                Wt.data.index_add_(0, idx, -self.lr * val / std)
        return stats
