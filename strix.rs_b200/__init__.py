"""strix.rs_b200 -- B200 (sm_100a) weight accelerator for strix.rs's quantized-matmul path.

The product is the C-ABI library ``lib/libstrix_cuda.so`` (see ``include/strix_cuda.h``).
This package holds its sources (``csrc/``), the build recipe (``build.py``), a
Python mirror of the reference's ``WeightAccel`` trait over that ABI (``accel.py``)
and the seeded synthetic-tensor generators used by the tests and the bench
(``synth.py``).

The directory name contains a dot, so it is loaded by path (see
``__graft_entry__.load_package``) under the module name ``strix_rs_b200``.
"""
from .accel import (ACT_F32, ACT_Q8DOT, PRE_GEGLU, PRE_NONE, PRE_RMSNORM, PRE_SWIGLU, CudaWeightAccel,
                    StrixCudaError, fold_argmax_shards, library_path, load_library, shard_begin)

__all__ = ["CudaWeightAccel", "StrixCudaError", "load_library", "library_path", "shard_begin", "fold_argmax_shards", "ACT_F32",
           "ACT_Q8DOT", "PRE_NONE", "PRE_RMSNORM", "PRE_SWIGLU", "PRE_GEGLU"]
