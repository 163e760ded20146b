"""B200-native FFT spatial convolution behind the nn.SpatialConvolutionFBFFT interface.

    capi        ctypes binding of the C ABI (include/fbfftconv.h)
    module      SpatialConvolutionFBFFT: host-side mirror of the reference's Lua module
    lua/        the LuaJIT FFI file a Torch7 installation would load
    csrc/       CUDA kernels (sm_100a) and the C ABI
"""
from . import capi  # noqa: F401
from .module import FFTWrapper, SpatialConvolutionFBFFT  # noqa: F401
