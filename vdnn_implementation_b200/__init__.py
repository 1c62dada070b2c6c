"""B200-native vDNN training path: Python host side over the C ABI of libvdnn_b200.so.

The package mirrors the reference's driver vocabulary (Network, Layer types, vdnn policies,
algorithm modes).  All arithmetic runs in the CUDA library; there is no CPU or PyTorch fallback:
importing `lib()` without the built shared object raises.
"""
from .abi import (  # noqa: F401
    ALEXNET, ALEXNET_LRN, BASELINE, CONV, CUSTOM_CNN, FC_CONV, FC_GEMM, GOOGLENET, LRN, OVERFEAT, POOL,
    RELU, SOFTMAX, VDNN_ALL, VDNN_CONV, VDNN_DYNAMIC_ALGO, VDNN_MEMORY_OPT_ALGO, VDNN_NONE,
    VDNN_PERF_OPT_ALGO, VGG16_64, VGG16_128, VGG16_256, ENGINE_AUTO, ENGINE_FFMA, ENGINE_TCGEN05,
    ConvDesc, LayerSpec, VdnnError, lib, lib_path,
)
from .network import Network  # noqa: F401
from . import ops  # noqa: F401
