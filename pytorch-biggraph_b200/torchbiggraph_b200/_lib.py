"""ctypes binding of libpbg_b200.so (include/pbg_b200.h).

The library is the only compute path of this package: when it is missing the import of
`torchbiggraph_b200._lib.lib()` raises, there is no PyTorch or CPU fallback.  It stands where the
reference loads its native module (torchbiggraph/train_gpu.py:41-46)."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpbg_b200.so")

OPERATOR_CODES = {"none": 0, "diagonal": 1, "translation": 2, "complex_diagonal": 3, "linear": 4, "affine": 5}
COMPARATOR_CODES = {"dot": 0, "cos": 1, "l2": 2, "squared_l2": 3}
LOSS_CODES = {"logistic": 0, "ranking": 1, "softmax": 2}
PRECISION_CODES = {"fp32": 0, "tf32x3": 1, "tf32": 2, "bf16x6": 3, "bf16x3": 4}

PBG_OK, PBG_ERR_BAD_ARGUMENT, PBG_ERR_UNSUPPORTED, PBG_ERR_INDEX_RANGE = 0, 1, 2, 3
PBG_ERR_TIMEOUT, PBG_ERR_CUDA, PBG_ERR_NO_DEVICE, PBG_ERR_TOO_LARGE = 4, 5, 6, 7


class PbgConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "dim", "op", "comparator", "loss", "dynamic_relations", "num_rels", "num_batch_negs",
        "num_uniform_negs", "disable_lhs_negs", "disable_rhs_negs", "precision", "max_batch_size",
        "batches_in_flight")] + [("margin", C.c_float), ("lr", C.c_float), ("relation_lr", C.c_float),
                                    ("regularization_coef", C.c_float), ("max_norm", C.c_float)]


class PbgBucket(C.Structure):
    _fields_ = [("lhs_emb", C.c_void_p), ("lhs_state", C.c_void_p), ("lhs_rows", C.c_int64),
                ("rhs_emb", C.c_void_p), ("rhs_state", C.c_void_p), ("rhs_rows", C.c_int64),
                ("rhs_op", C.c_void_p), ("rhs_op_state", C.c_void_p),
                ("lhs_op", C.c_void_p), ("lhs_op_state", C.c_void_p),
                ("relation_weights", C.POINTER(C.c_float)),
                ("lhs_global", C.c_void_p), ("lhs_global_state", C.c_void_p),
                ("rhs_global", C.c_void_p), ("rhs_global_state", C.c_void_p)]


class PbgBatch(C.Structure):
    _fields_ = [("offset", C.c_int64), ("count", C.c_int32), ("rel", C.c_int32)]


class PbgBatchStats(C.Structure):
    _fields_ = [("loss", C.c_float), ("reg", C.c_float), ("violators_lhs", C.c_int64),
                ("violators_rhs", C.c_int64), ("count", C.c_int64)]


class PbgEvalStats(C.Structure):
    _fields_ = [("loss", C.c_float)] + [(n, C.c_double) for n in ("pos_rank", "mrr", "r1", "r10", "r50", "auc")] + [("count", C.c_int64)]


# every symbol include/pbg_b200.h declares: (name, restype, argtypes)
_P = C.c_void_p
SYMBOLS = [
    ("pbg_version", C.c_char_p, []),
    ("pbg_status_string", C.c_char_p, [C.c_int]),
    ("pbg_create", C.c_int, [C.POINTER(PbgConfig), C.c_int, _P, C.POINTER(_P)]),
    ("pbg_destroy", C.c_int, [_P]),
    ("pbg_last_error", C.c_char_p, [_P]),
    ("pbg_workspace_bytes", C.c_int64, [_P]),
    ("pbg_set_hyperparameters", C.c_int, [_P, C.c_float, C.c_float, C.c_float]),
    ("pbg_train_batches", C.c_int, [_P, C.POINTER(PbgBucket), _P, _P, _P, C.c_int64, C.POINTER(PbgBatch),
                                    C.c_int32, _P, _P, C.c_uint64, C.POINTER(PbgBatchStats)]),
    ("pbg_train_batches_host", C.c_int, [_P, C.POINTER(PbgBucket), _P, _P, _P, C.c_int64, C.POINTER(PbgBatch),
                                         C.c_int32, _P, _P, C.c_uint64, C.POINTER(PbgBatchStats)]),
    ("pbg_read_stats", C.c_int, [_P, C.POINTER(PbgBatchStats)]),
    ("pbg_score_batch", C.c_int, [_P, C.POINTER(PbgBucket), _P, _P, _P, C.c_int32, C.c_int32, _P, _P,
                                  C.c_uint64, _P, _P, _P, _P]),
    ("pbg_eval_batch", C.c_int, [_P, C.POINTER(PbgBucket), _P, _P, _P, C.c_int32, C.c_int32, _P, _P,
                                 C.c_uint64, C.POINTER(PbgEvalStats)]),
    ("pbg_eval_batch_all_negs", C.c_int, [_P, C.POINTER(PbgBucket), _P, _P, _P, C.c_int32, C.c_int32,
                                          C.c_uint64, C.POINTER(PbgEvalStats)]),
    ("pbg_neg_columns", C.c_int, [_P, C.c_int32] + [C.POINTER(C.c_int32)] * 4),
    ("pbg_row_adagrad", C.c_int, [_P, _P, _P, C.c_int64, _P, _P, C.c_int32, C.c_float]),
    ("pbg_row_adagrad_static", C.c_int, [_P, _P, C.c_int64, C.c_int32, _P, _P, C.c_int32, C.c_float, _P]),
    ("pbg_reverse_permutation", C.c_int, [_P, _P, C.c_int64, _P]),
    ("pbg_shuffle_rows", C.c_int, [_P, _P, _P, C.c_int64, C.c_int64, _P]),
    ("pbg_randperm", C.c_int, [_P, C.c_int64, C.c_uint64, _P]),
    ("pbg_sub_bucket", C.c_int, [_P, _P, _P, _P, C.c_int64, C.c_int32, C.POINTER(C.c_int64), C.POINTER(_P),
                                 C.POINTER(C.c_int64), C.POINTER(_P), _P, _P, _P, C.c_int32, C.c_int32, C.c_int32,
                                 C.POINTER(C.c_int64)]),
    ("pbg_launch_count", C.c_int64, [_P]),
    ("pbg_set_edge_weights", C.c_int, [_P, C.c_void_p]),
    ("pbg_set_profiling", C.c_int, [_P, C.c_int]),
    ("pbg_kernel_times", C.c_int, [_P, C.POINTER(C.c_double), C.POINTER(C.c_int64)]),
]
KERNEL_CLASSES = ("sort", "gather", "score", "loss", "grad", "update", "stats")

_lib = None


class PbgError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"pbg_b200 status {status}: {message}")
        self.status = status


def lib():
    """Loads the native library once.  Raises if it has not been built (no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python pytorch-biggraph_b200/build.py`. "
                "This package has no CPU or PyTorch fallback for the training step.")
        handle = C.CDLL(LIB_PATH)
        for name, res, args in SYMBOLS:
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status, ctx=None):
    if status != PBG_OK:
        L = lib()
        msg = L.pbg_last_error(ctx).decode() if ctx else ""
        raise PbgError(status, f"{L.pbg_status_string(status).decode()}: {msg}")
