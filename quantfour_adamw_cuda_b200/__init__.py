"""quantfour_adamw_cuda_b200: AdamW with 4-bit optimizer states for NVIDIA B200 (sm_100a).

The package mirrors the public surface of the reference project's ``optim`` directory for its one
hot path, the fused optimizer step:

  FourBitAdamW (aliases AdamWFused_QuantFour, AdamW_Fused_QuantFour, AdamW_QuantFour)
      the optimizer class (optim/fused_quantfour.py:25, optim/adamw_fourbit_triton.py:137)
  fused_4bit, fused_single_tensor
      the extension module's two functions (optim/cuda_fused_interface.cc:66-69)
  quantize_m / dequantize_m / quantize_v / dequantize_v (+ *_v_block)
      the stand-alone quantize / dequantize pieces
  ShardedFourBitAdamW (quantfour_adamw_cuda_b200.zero1)
      optimizer state sharded across ranks with an all-gather of the updated parameters

All compute goes through libquantfour_b200.so (C ABI in include/quantfour_b200.h); importing the
package does not load it, the first call does, and a missing library raises.
"""
from .functional import (dequantize_m, dequantize_v, dequantize_v_block, fused_4bit, fused_single_tensor, quantize_m,
                         quantize_v, quantize_v_block)
from .optimizer import (AdamW_Fused_QuantFour, AdamW_QuantFour, AdamWFused_QuantFour, FourBitAdamW,
                        enable_param_quantization, make_hyper)

__all__ = [
    "FourBitAdamW", "AdamWFused_QuantFour", "AdamW_Fused_QuantFour", "AdamW_QuantFour",
    "fused_4bit", "fused_single_tensor", "quantize_m", "dequantize_m", "quantize_v", "dequantize_v",
    "quantize_v_block", "dequantize_v_block", "enable_param_quantization", "make_hyper",
]
