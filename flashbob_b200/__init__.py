"""Second-order scaled-dot-product attention for NVIDIA B200 (sm_100a).

`sdpa_bob` is the one public operator: attention whose first gradients (taken with
`create_graph=True`) can be differentiated again.  Forward, first backward and second backward
run as hand-written CUDA kernels in libbob_sm100.so (C ABI in include/bob_sm100.h).
"""

from .interface import sdpa_bob

__all__ = ["sdpa_bob"]
