"""torq_b200: host side of the B200 execution backend for the quantized layer ops the
Torq compiler emits. The compute lives in libtorq_b200.so (hand-written sm_100a
CUDA behind the C ABI of include/torq_b200.h); this package builds op-list
executables and drives that library. There is no CPU fallback."""
from .oplist import Graph, TensorRef  # noqa: F401
from .quant import quantize_multiplier  # noqa: F401
