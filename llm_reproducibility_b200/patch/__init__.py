"""`apply_patches()`: install the invariant ops into vLLM according to the environment
(reference: src/patch/__init__.py:7-37).

Only the TP-invariant row-split patch belongs to this package.  The batch-invariant aten
overrides and the attention-alignment patch of the reference are other subsystems; when
their switches are set, `apply_patches` says so instead of importing them eagerly (the
reference's eager import is what makes `import src.patch` fail on newer vLLM).
"""
import os

from .patch_tp_invariant import patch_tp_invariant

__all__ = ["apply_patches", "patch_tp_invariant"]


def apply_patches():
    from ..utils import batch_invariant_is_enabled, compatible_mode_is_enabled, tp_invariant_is_enabled

    if not batch_invariant_is_enabled() and not tp_invariant_is_enabled() and not compatible_mode_is_enabled():
        print("No patches applied to vLLM.\n")
        return
    if batch_invariant_is_enabled():
        print("VLLM_BATCH_INVARIANT is set: batch-invariant aten overrides are not part of this package")
    if tp_invariant_is_enabled():
        # $TBIK_MAX_TP: the largest TP degree whose bits must equal those of all smaller ones (default 8)
        patch_tp_invariant(max_tp=int(os.environ.get("TBIK_MAX_TP", "8")))
    if compatible_mode_is_enabled():
        print("ALIGN_TRAIN_INFERENCE is set: attention alignment is not part of this package")
    print("Successfully applied patches\n")
