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
