"""Device-resident counterpart of ``litespark_inference.torchless``: same module layout
(kernel, runtime, model, pack, quantize, ops), CUDA underneath."""
from . import kernel, model, ops, pack, quantize, synthetic  # noqa: F401
from .model import (BitNetConfig, FalconTernaryConfig, PackedBitNetModel, PackedFalconModel,  # noqa: F401
                    PackedLayer, PackedProjection)
