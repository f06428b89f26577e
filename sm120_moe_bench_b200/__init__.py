"""B200 (sm_100a) fused NVFP4 MoE expert layer: PyTorch host side over a C-ABI CUDA library.

Public surface:
  * ``ops``          -- thin torch wrappers of the C entry points (routing, permutation tables,
                        activation quantiser, decoder, the fused layer);
  * ``verdict_moe``  -- ``VerdictMoEExperts`` / ``VerdictMoEMonolithic``, the operator classes with the
                        reference's method set and argument meaning;
  * ``synth``        -- seeded synthetic NVFP4 layers in the reference's tensor layout.
"""
from . import _lib  # noqa: F401  (fails loudly when the CUDA library is absent)
from .ops import (MoEShape, MoEWeights, Workspace, build_tables, dequantize, fused_moe,  # noqa: F401
                  quantize, route)
