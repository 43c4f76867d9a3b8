"""tilefusion_b200 -- B200-native fused attention behind TileFusion's operator API.

``import tilefusion_b200 as tilefusion`` gives the same surface as TileFusion's
Python package for this path (``python/__init__.py:19-40`` there loads
``libtilefusion.so`` with ctypes at import, which registers
``torch.ops.tilefusion.*``):

* ``tilefusion_b200.ops.flash_attention(query, key, value, tile_length_q,
  tile_length_kv, tile_hidden_qk, tile_hidden_v, softmax_scale, causal)``
* ``tilefusion_b200.ops.flash_decoding(query, key, value, ...)`` (added)

There is no CPU or eager fallback: if the native library cannot be loaded the
import of the operator layer raises.
"""

from . import _cabi  # noqa: F401  (loads libtilefusion_b200.so)
from . import ops  # noqa: F401
from .host_pipeline import HostPipeline  # noqa: F401

__all__ = ["ops", "load_torch_ops", "HostPipeline"]


def load_torch_ops() -> None:
    """Load the operator layer so that ``torch.ops.tilefusion.*`` exists."""
    from ._torch_ops import ensure_loaded

    ensure_loaded()
