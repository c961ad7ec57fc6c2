"""Tree-based invariant kernels: the two ops of the row-split path."""
