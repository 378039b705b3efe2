"""mlx_b200 - B200-native (sm_100a) affine quantized matmul operators.

Drop-in for the reference's ``quantize`` / ``dequantize`` / ``quantized_matmul`` /
``gather_qmm`` operators; see ``mlx_b200.ops`` for the operator front-end and
``include/b200q.h`` for the C ABI of the CUDA library underneath.
"""
__all__ = ["quantize", "dequantize", "quantized_matmul", "gather_qmm", "gather_qmm_chain", "gather_qmm_swiglu",
           "quantized_embedding",
           "qmm_kernel_name", "set_weights_constant"]


def __getattr__(name):
    if name in __all__:
        from . import ops

        return getattr(ops, name)
    raise AttributeError(name)
