"""CPU oracle for the FFT spatial-convolution path -- TEST INFRASTRUCTURE ONLY.

Holds the fp64 restatement of the reference's algorithm (``refconv.c`` for the
spatial definition, ``spectral.py`` for the frequency-domain one) and, when it was
compiled, the reference's own CPU convolution (``_ref/libfbcunn_ref.so``).  Only the
tests, the smoke check and the benchmark's CPU-baseline leg may import this
package; the product path never does.
"""
from .refconv import (  # noqa: F401
    Shape,
    acc_grad_bias,
    acc_grad_weight,
    acc_grad_weight_planes,
    build,
    reference_available,
    reference_acc_grad_weight,
    reference_update_grad_input,
    reference_update_output,
    update_grad_input,
    update_grad_input_planes,
    update_output,
    update_output_planes,
)
