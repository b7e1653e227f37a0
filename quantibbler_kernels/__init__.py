"""Drop-in for the reference's ``quantibbler_kernels`` extension module.

``src/quantibbler/kernels/__init__.py:39-45`` of the reference does
``import quantibbler_kernels as _kernels`` and treats a successful import as the
``"rust"`` backend; with this package on ``sys.path`` that import resolves here and the
products run on the B200 through libqk_kernels.so.
"""

from quantibbler_b200.kernels import *  # noqa: F401,F403
from quantibbler_b200.kernels import __all__  # noqa: F401
