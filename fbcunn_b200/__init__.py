"""B200-native FFT spatial convolution behind the nn.SpatialConvolutionFBFFT interface.

    capi        ctypes binding of the C ABI (include/fbfftconv.h)
    module      SpatialConvolutionFBFFT (and its Gemm-variant name), FFTWrapper, CuBLASWrapper:
                host-side mirrors of the reference's Lua modules
    tiled       SpatialConvolutionFFTTiled: the same convolution on tiles of the image
    tuned       SpatialConvolution: times the candidates on first use and keeps the fastest
    lua/        the LuaJIT FFI file a Torch7 installation would load
    csrc/       CUDA kernels (sm_100a) and the C ABI
"""
from . import capi  # noqa: F401
from .module import CuBLASWrapper, FFTWrapper, SpatialConvolutionFBFFT, SpatialConvolutionFBFFTGemm  # noqa: F401
from .tiled import SpatialConvolutionFFTTiled  # noqa: F401
from .tuned import SpatialConvolution  # noqa: F401
