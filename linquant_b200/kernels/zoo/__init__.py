"""INT8 chunk kernels of the zoo lineage (same names as ``linquant/kernels/zoo/__init__.py``)."""

from .gated_delta_rule import chunk_delta_int8  # noqa: F401
from .gla import chunk_gla_int8  # noqa: F401
from .kda import chunk_kda_int8  # noqa: F401
from .simple_gla import chunk_simple_gla_int8  # noqa: F401
