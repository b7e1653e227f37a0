"""quantibbler_b200: the quantibbler-kernels hot path for NVIDIA B200 (sm_100a).

The product is ``libqk_kernels.so`` (CUDA + C ABI, ``include/qk_kernels.h``).  This
package holds its sources (``csrc/``), its in-tree build (``_build``) and a thin host
layer that mirrors the reference's Python and Rust interfaces for the path
(``kernels``, ``gpu``).
"""

from ._lib import DeviceError, KernelError  # noqa: F401

__version__ = "0.1.0"
