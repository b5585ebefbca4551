"""B200-native (sm_100a) implementation of Litespark-Inference's ternary-matmul hot path.

The directory name carries a hyphen, so it cannot be imported by name; load it with
``__graft_entry__.load_package()`` (repo root), which registers it as
``litespark_inference_b200``.  The sub-package ``torchless`` mirrors the reference's
``litespark_inference.torchless`` interface (kernel wrappers, runtime, model containers).

No torch import anywhere in this package; CUDA is reached through ``_lspk_sm100.so`` via ctypes.
"""
__version__ = "0.1.0"
