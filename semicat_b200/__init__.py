"""semicat_b200 - B200 (sm_100a) flash-attention JVP kernels behind the reference's ``sdpa_jvp`` API.

Public surface: :func:`sdpa_jvp`, :func:`safe_sdpa_jvp` (``semicat_b200.functional``), the raw
tensor-level launchers in ``semicat_b200.ops`` and the hook that installs them into the reference
package (``semicat_b200.hooks``).  The CUDA code lives in ``semicat_b200/csrc`` and is reached
only through the C ABI of ``include/jvpattn.h``.
"""
from .functional import safe_sdpa_jvp, sdpa_jvp, set_kernel_family  # noqa: F401

__version__ = "0.1.0"
