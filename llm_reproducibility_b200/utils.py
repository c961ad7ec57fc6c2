"""Environment switches of the invariant modes (reference: src/utils.py:4-61).

Each switch is an integer environment variable; anything that does not parse as an integer
counts as off.
"""
import os


def _int_flag(name: str) -> bool:
    try:
        return int(os.getenv(name, "0")) != 0
    except ValueError:
        return False


def batch_invariant_is_enabled() -> bool:
    return _int_flag("VLLM_BATCH_INVARIANT")


def tp_invariant_is_enabled() -> bool:
    on = _int_flag("VLLM_TP_INVARIANT")
    if on:
        assert batch_invariant_is_enabled(), "Batch invariance must be enabled when TP invariance is enabled"
    return on


def check_invariant_compat() -> bool:
    return _int_flag("VLLM_TP_INVARIANT") and _int_flag("VLLM_BATCH_INVARIANT")


def compatible_mode_is_enabled() -> bool:
    return _int_flag("ALIGN_TRAIN_INFERENCE")


def tp_invariant_matmul_is_enabled() -> bool:
    """$TP_INVARIANT_MATMUL: selects the tree matmul in the stand-alone demo (simple_matmul.py:8)."""
    return _int_flag("TP_INVARIANT_MATMUL")
