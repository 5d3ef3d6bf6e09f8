"""INT8 chunk kernels of the zoo lineage (same names as ``linquant/kernels/zoo/__init__.py``)."""

from .simple_gla import chunk_simple_gla_int8  # noqa: F401
