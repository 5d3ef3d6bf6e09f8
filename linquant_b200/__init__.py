"""linquant_b200: sm_100a CUDA implementation of LinQuant's INT8 chunkwise linear-recurrence prefill.

``linquant_b200.kernels`` keeps the call surface of the reference's ``linquant.kernels`` package; the device
code lives in ``csrc/`` behind the C ABI of ``include/linquant_b200.h``."""

__version__ = "0.1.0"
