"""tensorplay_b200 -- sm_100a reduction and top-k operators behind TensorPlay's operator surface.

The package holds the CUDA kernels and their C ABI (csrc/, include/tpb200.h), the host-side
mirror of the reference's reduction methods (ops), and the one-process-per-GPU sharding layer
(sharded).  Importing it never touches the GPU; the first operator call loads libtpb200.so and
raises if it is missing (there is no CPU or PyTorch fallback).
"""
from .ops import (all, any, argmax, argmin, contiguous, copy_, log_softmax, max, max_with_indices, mean, median, min,
                  min_with_indices, norm, prod, softmax, std, sum, topk, var)
from .sharded import ShardedReducer, flat_partition, row_block

__all__ = ["sum", "mean", "var", "std", "max", "min", "argmax", "argmin", "prod", "norm", "all", "any", "topk",
           "softmax", "log_softmax", "median", "copy_", "contiguous", "max_with_indices",
           "min_with_indices", "ShardedReducer", "row_block", "flat_partition"]
