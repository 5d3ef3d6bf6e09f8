"""linquant_b200: sm_100a CUDA implementation of LinQuant's INT8 chunkwise linear-recurrence prefill.

``linquant_b200.kernels`` keeps the call surface of the reference's ``linquant.kernels`` package; the device
code lives in ``csrc/`` behind the C ABI of ``include/linquant_b200.h``."""

__version__ = "0.1.0"


def check_status(device=None):
    """Raises if a kernel of this package gave up on a bounded device-side wait on ``device`` (default: the current
    CUDA device) since the last check; see ``linquant_b200._cabi.check_status``. The ops return without synchronising
    and never read the word themselves, so a caller that wants the guarantee calls this after its forward pass."""
    from . import _cabi

    _cabi.check_status(device)
