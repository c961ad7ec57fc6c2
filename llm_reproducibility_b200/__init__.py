"""B200-native implementation of the TP-invariant row-split path (tree matmul + tree all-reduce).

Sub-packages mirror the reference project's importable surface:
  tbik.tree_based_matmul       matmul_tp_persistent
  tbik.tree_based_all_reduce   tree_all_reduce_sum, tree_all_reduce_sum_native
  mini_allreduce               CustomAllreduce, CustomTreeAllreduce, custom_all_reduce_ops
  patch                        apply_patches, patch_tp_invariant
  utils                        environment switches
`install_aliases()` additionally registers them under the reference's own module names
(`src`, `tbik`, `mini_allreduce`, `tbik_kernel`) so existing callers keep their imports.
"""
__version__ = "0.1.0"


def install_aliases() -> None:
    """Register this package's modules under the reference project's import names
    (`src`, `src.tbik`, `tbik`, `src.patch`, `src.utils`, `mini_allreduce`, `tbik_kernel`)."""
    import importlib
    import sys

    pkg = sys.modules[__name__]
    names = {
        "src": pkg,
        "src.utils": importlib.import_module(__name__ + ".utils"),
        "src.tbik": importlib.import_module(__name__ + ".tbik"),
        "src.tbik.tree_based_matmul": importlib.import_module(__name__ + ".tbik.tree_based_matmul"),
        "src.tbik.tree_based_all_reduce": importlib.import_module(__name__ + ".tbik.tree_based_all_reduce"),
        "src.patch": importlib.import_module(__name__ + ".patch"),
        "mini_allreduce": importlib.import_module(__name__ + ".mini_allreduce"),
        "mini_allreduce.custom_all_reduce_ops": importlib.import_module(__name__ + ".mini_allreduce.custom_all_reduce_ops"),
        "tbik_kernel": importlib.import_module(__name__ + ".tbik_kernel"),
        "tbik_kernel.allreduce": importlib.import_module(__name__ + ".tbik_kernel.allreduce"),
    }
    names["tbik"] = names["src.tbik"]
    names["tbik.tree_based_matmul"] = names["src.tbik.tree_based_matmul"]
    names["tbik.tree_based_all_reduce"] = names["src.tbik.tree_based_all_reduce"]
    for alias, mod in names.items():
        sys.modules.setdefault(alias, mod)
