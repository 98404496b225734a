"""The reference's native module `torchbiggraph._C` (torchbiggraph/util.cpp:425-460) with the same four
functions and argument lists, on CUDA tensors: `randperm`, `reverse_permutation`, `shuffle`, `sub_bucket`.

The reference runs them on host threads over CPU tensors; here the tensors live on the device and the
`num_threads` arguments are accepted and ignored.  Everything is computed by libpbg_b200.so (pbg_edges.cu);
PyTorch only owns the memory.  Errors keep the reference's types: what util.cpp throws as
std::invalid_argument arrives as ValueError, std::runtime_error as RuntimeError."""
import ctypes as C
from typing import Dict, List, Sequence, Tuple

import torch

from . import _lib

_contexts: Dict[int, C.c_void_p] = {}


def _ctx(device: torch.device) -> C.c_void_p:
    """A small library context per device: the utilities only use its stream, error word and sort scratch."""
    if device.type != "cuda":
        raise RuntimeError("torchbiggraph_b200._C works on CUDA tensors only (no CPU fallback)")
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _contexts:
        L = _lib.lib()
        cfg = _lib.PbgConfig(dim=4, op=0, comparator=0, loss=1, dynamic_relations=0, num_rels=1, num_batch_negs=1,
                             num_uniform_negs=1, precision=0, max_batch_size=1, batches_in_flight=1, lr=0.1, relation_lr=0.1)
        ctx = C.c_void_p()
        st = L.pbg_create(C.byref(cfg), idx, None, C.byref(ctx))
        if st != 0:
            msg = L.pbg_last_error(ctx).decode() if ctx else ""
            L.pbg_destroy(ctx)
            raise _lib.PbgError(st, msg)
        _contexts[idx] = ctx
    return _contexts[idx]


def _p(t: torch.Tensor):
    return C.c_void_p(t.data_ptr())


def _sync_torch(device):
    # the library works on the legacy default stream of its context; order it after PyTorch's current stream
    torch.cuda.current_stream(device).synchronize()


def randperm(num_items: int, num_threads: int = 1, seed: int = -1, device="cuda") -> torch.Tensor:
    """util.cpp:14-101: a random permutation of range(num_items) as an int64 tensor.  seed < 0 draws one from
    PyTorch's generator (the reference then uses its default seed)."""
    device = torch.device(device)
    if seed < 0:
        seed = int(torch.randint(0, 2**62, (1,)).item())
    out = torch.empty(num_items, dtype=torch.long, device=device)
    ctx = _ctx(out.device)
    _sync_torch(out.device)
    _lib.check(_lib.lib().pbg_randperm(ctx, num_items, seed, _p(out)), ctx)
    return out


def reverse_permutation(perm: torch.Tensor, num_threads: int = 1) -> torch.Tensor:
    """util.cpp:103-125: res[perm[i]] = i."""
    if perm.dtype != torch.long or perm.dim() != 1:
        raise ValueError("Permutation must be a 1-dimensional int64 tensor")
    perm = perm.contiguous()
    out = torch.empty_like(perm)
    ctx = _ctx(perm.device)
    _sync_torch(perm.device)
    _check_value(_lib.lib().pbg_reverse_permutation(ctx, _p(perm), perm.shape[0], _p(out)), ctx)
    return out


def _check_value(status, ctx):
    if status == _lib.PBG_ERR_INDEX_RANGE:
        raise ValueError(_lib.lib().pbg_last_error(ctx).decode())
    _lib.check(status, ctx)


def shuffle(tensor: torch.Tensor, permutation: torch.Tensor, num_threads: int = 1) -> None:
    """util.cpp:127-220: in place, row i of `tensor` moves to row permutation[i]."""
    if permutation.dtype != torch.long:
        raise ValueError("Permutation must have int64 dtype")
    if permutation.dim() != 1:
        raise ValueError("Permutation must have exactly one dimension")
    if tensor.dim() < 1:
        raise ValueError("Tensor must have at least one dimension")
    rows = tensor.shape[0]
    if rows != permutation.shape[0]:
        raise ValueError("Tensor and permutation must have the same number of elements on the first dimension")
    if rows == 0 or tensor[0].numel() == 0:
        return
    if not tensor.is_contiguous():
        raise ValueError("Each sub-tensor of tensor (along the first dimension) must be contiguous")
    if tensor.device != permutation.device:
        raise ValueError("Tensor and permutation must be on the same device")
    out = torch.empty_like(tensor)
    ctx = _ctx(tensor.device)
    _sync_torch(tensor.device)
    row_bytes = tensor[0].numel() * tensor.element_size()
    _check_value(_lib.lib().pbg_shuffle_rows(ctx, _p(tensor), _p(out), rows, row_bytes, _p(permutation.contiguous())), ctx)
    tensor.copy_(out)


def sub_bucket(lhs_in: torch.Tensor, rhs_in: torch.Tensor, rel_in: torch.Tensor, lhs_entity_counts: Sequence[int],
               lhs_perms: Sequence[torch.Tensor], rhs_entity_count: Sequence[int], rhs_perms: Sequence[torch.Tensor],
               lhs_out: torch.Tensor, rhs_out: torch.Tensor, rel_out: torch.Tensor, num_lhs_sub_parts: int,
               num_rhs_sub_parts: int, num_threads: int = 1, dynamic_relations: bool = False
               ) -> Dict[Tuple[int, int], Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]:
    """util.cpp:260-423: {(i, j): (lhs, rhs, rel)} as views of the three output tensors."""
    R = len(lhs_perms)
    if len(rhs_perms) != R or len(lhs_entity_counts) != R or len(rhs_entity_count) != R:
        raise RuntimeError("Inconsistent num_relations")
    n = rel_in.shape[0]
    for t in (lhs_in, rhs_in, rel_in, lhs_out, rhs_out, rel_out):
        if t.dtype != torch.long or t.dim() != 1 or t.shape[0] != n or not t.is_contiguous():
            raise ValueError("edge tensors must be contiguous 1-dimensional int64 tensors of one length")
    ctx = _ctx(lhs_in.device)
    lperms = [p.contiguous() for p in lhs_perms]
    rperms = [p.contiguous() for p in rhs_perms]
    lc = (C.c_int64 * R)(*[int(x) for x in lhs_entity_counts])
    rc = (C.c_int64 * R)(*[int(x) for x in rhs_entity_count])
    lp = (C.c_void_p * R)(*[p.data_ptr() for p in lperms])
    rp = (C.c_void_p * R)(*[p.data_ptr() for p in rperms])
    nb = num_lhs_sub_parts * num_rhs_sub_parts
    counts = (C.c_int64 * nb)()
    _sync_torch(lhs_in.device)
    st = _lib.lib().pbg_sub_bucket(ctx, _p(lhs_in), _p(rhs_in), _p(rel_in), n, R, lc, lp, rc, rp, _p(lhs_out), _p(rhs_out),
                                   _p(rel_out), num_lhs_sub_parts, num_rhs_sub_parts, int(bool(dynamic_relations)), counts)
    if st == _lib.PBG_ERR_INDEX_RANGE:
        raise RuntimeError(_lib.lib().pbg_last_error(ctx).decode())
    _lib.check(st, ctx)
    res, start = {}, 0
    for i in range(num_lhs_sub_parts):
        for j in range(num_rhs_sub_parts):
            stop = start + counts[i * num_rhs_sub_parts + j]
            res[i, j] = (lhs_out[start:stop], rhs_out[start:stop], rel_out[start:stop])
            start = stop
    return res
