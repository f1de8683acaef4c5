"""B200-native MoE expert-parallel dispatch/combine behind Mooncake EP's `Buffer` API.

`mooncake_b200.mooncake_ep_buffer.Buffer` is the drop-in for
`mooncake.mooncake_ep_buffer.Buffer`, `mooncake_b200.mooncake_elastic_buffer.ElasticBuffer`
for `mooncake.mooncake_elastic_buffer.ElasticBuffer` (one NVLink domain); `mooncake_b200.ep` is the native module
(`mooncake.ep`). Importing the package loads `libmcep.so` (building it with nvcc
when absent) - there is no pure-Python or CPU path.
"""
from . import ep  # noqa: F401  (loads the shared library; fails loudly without it)
from .mooncake_ep_buffer import Buffer, EventOverlap  # noqa: F401
from .mooncake_elastic_buffer import ElasticBuffer, EPHandle  # noqa: F401

__all__ = ["Buffer", "EventOverlap", "ElasticBuffer", "EPHandle", "ep"]
