"""B200-native pair-stack operators behind the reference's operator API.

The CUDA library (``lib/liblocalfold_pairstack.so``, C ABI in
``include/localfold_pairstack.h``) does all the arithmetic; there is no CPU or
eager fallback - a missing library raises on first use.
"""
from .operators import (  # noqa: F401
    Af3GridSelfAttentionGpu, Af3MsaAttentionGpu, Af3SingleAttentionGpu, Af3TransitionGpu, AttentionGpu, Device,
    EncodedTensor, GlobalColumnAttentionGpu, OuterProductMeanGpu, PreparedWeights, RangeError, TransitionGpu,
    TriangleMultiplicationIncomingGpu, TriangleMultiplicationOutgoingGpu,
    af3_triangle_multiplication, create_device, distogram_logits, error_metrics, int5_decode, validate_triangle_input,
)
from .pipeline import PairStackPipeline  # noqa: F401
from .stack import Af3MsaBlockGpu, Af3MsaStackGpu, Af3PairformerStackGpu, EvoformerBlockGpu, EvoformerStackGpu, ExtraMsaBlockGpu, ExtraMsaStackGpu, PairStackGpu, PreparedMsaBlock, PreparedPairBlock  # noqa: F401
