"""ctypes binding of libchurten_b200.so (the C ABI declared in include/churten_b200.h).

The library is the product: there is no CPU or PyTorch fallback.  If it has not
been built, importing this module raises with the command that builds it.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_double, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

_PKG = Path(__file__).resolve().parent
# CHURTEN_B200_LIB points at another build of the library (e.g. an experimental variant)
LIB_PATH = Path(os.environ.get("CHURTEN_B200_LIB") or _PKG / "libchurten_b200.so")

F32, F64, F16, BF16 = 0, 1, 2, 3  # enum cb200_dtype

STEPS_ALREADY_BUMPED, WORKSPACE_PREPARED = 1, 2  # enum cb200_call_flags

OK = 0
ERR_INVALID_ARGUMENT = 1
ERR_WORKSPACE = 2
ERR_CUDA = 3
ERR_UNSUPPORTED = 4

# name -> (restype, argtypes); mirrors include/churten_b200.h line for line.
_P = c_void_p
SIGNATURES = {
    "cb200_version": (c_int, []),
    "cb200_last_error": (c_char_p, []),
    "cb200_workspace_bytes": (c_size_t, [c_int64]),
    "cb200_workspace_prepare": (c_int, [_P, c_size_t, c_int64, _P]),
    "cb200_adam_step": (
        c_int,
        # dtype params grads exp_avgs exp_avg_sqs max_exp_avg_sqs state_steps
        [c_int, _P, _P, _P, _P, _P, _P,
         # lr beta1 beta2 eps weight_decay active_mask
         _P, _P, _P, _P, _P, _P,
         # n_rows row_len strides amsgrad maximize decoupled steps_already_bumped active_rows_hint
         c_int64, c_int64, _P, c_int, c_int, c_int, c_int, c_int64,
         # workspace workspace_bytes stream
         _P, c_size_t, _P],
    ),
    "cb200_sgd_step": (
        c_int,
        # dtype params grads momentum_buffers state_steps lr momentum dampening weight_decay
        [c_int, _P, _P, _P, _P, _P, _P, _P, _P,
         # active_mask nesterov_rows n_rows row_len strides nesterov maximize
         _P, _P, c_int64, c_int64, _P, c_int, c_int,
         # steps_already_bumped active_rows_hint workspace workspace_bytes stream
         c_int, c_int64, _P, c_size_t, _P],
    ),
    "cb200_adagrad_step": (
        c_int,
        # dtype params grads state_sums state_steps lr lr_decay weight_decay eps active_mask
        [c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P,
         # n_rows row_len strides maximize steps_already_bumped active_rows_hint
         c_int64, c_int64, _P, c_int, c_int, c_int64,
         # workspace workspace_bytes stream
         _P, c_size_t, _P],
    ),
    "cb200_adam_step_from_parts": (
        c_int,
        # the arguments of cb200_adam_step with `grads` replaced by a cb200_grad_parts*
        [c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
         c_int64, c_int64, _P, c_int, c_int, c_int, c_int, c_int64, _P, c_size_t, _P],
    ),
    "cb200_sgd_step_from_parts": (
        c_int,
        [c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_int64, c_int64, _P, c_int, c_int,
         c_int, c_int64, _P, c_size_t, _P],
    ),
    "cb200_adagrad_step_from_parts": (
        c_int,
        [c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_int64, c_int64, _P, c_int, c_int, c_int64,
         _P, c_size_t, _P],
    ),
    "cb200_adam_step_mixed": (
        c_int,
        # moment_dtype params grads exp_avgs exp_avg_sqs max_exp_avg_sqs state_steps lr beta1 beta2 eps wd mask
        [c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
         # n_rows row_len amsgrad maximize decoupled steps_already_bumped active_rows_hint ws ws_bytes stream
         c_int64, c_int64, c_int, c_int, c_int, c_int, c_int64, _P, c_size_t, _P],
    ),
    "cb200_adam_step_mixed_from_parts": (
        c_int,
        # the arguments of cb200_adam_step_mixed with `grads` replaced by a cb200_grad_parts*
        [c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
         c_int64, c_int64, c_int, c_int, c_int, c_int, c_int64, _P, c_size_t, _P],
    ),
    "cb200_sgd_step_mixed": (
        c_int,
        # buffer_dtype params grads momentum_buffers state_steps lr momentum dampening wd mask nesterov_rows
        [c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
         # n_rows row_len nesterov maximize steps_already_bumped active_rows_hint ws ws_bytes stream
         c_int64, c_int64, c_int, c_int, c_int, c_int64, _P, c_size_t, _P],
    ),
    "cb200_sgd_step_mixed_from_parts": (
        c_int,
        # the arguments of cb200_sgd_step_mixed with `grads` replaced by a cb200_grad_parts*
        [c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
         c_int64, c_int64, c_int, c_int, c_int, c_int64, _P, c_size_t, _P],
    ),
    "cb200_scatter_rows": (
        c_int,
        # dst dst_row_stride dst_row_len n_rows n_parts parts offsets numels row_strides stream
        [_P, c_int64, c_int64, c_int64, c_int, _P, _P, _P, _P, _P],
    ),
    "cb200_copy_rows_masked": (
        c_int,
        # n_leaves dst src row_bytes dst_strides src_strides row_mask invert_mask n_rows stream
        [c_int, _P, _P, _P, _P, _P, _P, c_int, c_int64, _P],
    ),
    "cb200_lr_schedule": (
        c_int,
        # policy base_lrs clock lr active_mask lower upper best num_bad cooldown_counter score n stream
        [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_int64, _P],
    ),
    "cb200_early_stopping_tick": (
        c_int,
        # score active_mask misses threshold best_epoch improved all_stopped counters n_rows
        [_P, _P, _P, _P, _P, _P, _P, _P, c_int64,
         # epoch patience threshold_value threshold_relative lower_is_better stream
         c_int, c_int, c_double, c_int, c_int, _P],
    ),
    "cb200_adam_step_static_scratch": (
        c_int,
        # the arguments of cb200_adam_step without workspace and workspace_bytes
        [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
         c_int64, c_int64, _P, c_int, c_int, c_int, c_int64, _P],
    ),
    # n_read n_write buffers state_steps active_mask n_rows row_len workspace workspace_bytes stream
    "cb200_stream_ceiling": (c_int, [c_int, c_int, _P, _P, _P, c_int64, c_int64, _P, c_size_t, _P]),
    "cb200_set_launch_geometry": (c_int, [c_int, c_int, c_int]),
    "cb200_launch_count": (c_int64, []),
}

# enum cb200_lr_kind
LR_STEP, LR_MULTISTEP, LR_EXPONENTIAL, LR_COSINE, LR_WARM_RESTART, LR_PLATEAU = range(6)
LR_MAX_MILESTONES = 32


MAX_GRAD_PARTS = 96


class GradPartsTable(ctypes.Structure):
    """struct cb200_grad_parts."""

    _fields_ = [
        ("n_parts", c_int),
        ("ptr", c_void_p * MAX_GRAD_PARTS),
        ("row_stride", c_int64 * MAX_GRAD_PARTS),
        ("offset", c_int64 * MAX_GRAD_PARTS),
        ("numel", c_int64 * MAX_GRAD_PARTS),
    ]


class LrPolicy(ctypes.Structure):
    """struct cb200_lr_policy."""

    _fields_ = [
        ("kind", c_int), ("gamma", c_double), ("step_size", c_double), ("t_max", c_double),
        ("eta_min", c_double), ("base_period", c_double), ("period_mult", c_double),
        ("max_restarts", c_int), ("n_milestones", c_int),
        ("milestones", c_double * LR_MAX_MILESTONES),
        ("mode_max", c_int), ("threshold_rel", c_int), ("threshold", c_double),
        ("factor", c_double), ("patience", c_double), ("cooldown", c_double),
    ]


class LibraryMissing(ImportError):
    pass


def _open(path: Path, signatures: dict) -> ctypes.CDLL:
    if not path.exists():
        raise LibraryMissing(
            f"{path.name} has not been built (looked in {path.parent}). Build it with "
            "`python -m churten_b200.csrc.build`; there is no fallback implementation."
        )
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in signatures.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is missing
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


_lib: ctypes.CDLL | None = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = _open(LIB_PATH, SIGNATURES)
    return _lib


def last_error() -> str:
    return lib().cb200_last_error().decode("utf-8", "replace")


def check(status: int, op: str) -> None:
    """Turn a non-zero status into the RuntimeError the reference's TORCH_CHECKs raise."""
    if status != OK:
        raise RuntimeError(f"{op}: {last_error()} (cb200 status {status})")
