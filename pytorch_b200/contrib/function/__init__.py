from .quantized_mlp import w8a8_swiglu_mlp  # noqa: F401
