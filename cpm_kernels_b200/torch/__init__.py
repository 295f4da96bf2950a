"""torch.Tensor-level interface of the path (cpm_kernels/torch/__init__.py:3 exports ``bmm``)."""
from .gemm import bmm, bmm_gelu, layernorm_quantize, bmm_quantized_b, GEMMInt8, GEMMFloat, quantize, calc_scale, round_i8, gemm_and_scale  # noqa: F401
from .gelu import gelu, gelu_inplace, OpGeLU  # noqa: F401
from .transpose import transpose, transposeTH, OpTranspose  # noqa: F401
