from .moe_block import QuantFusedDeepseekV2MoEBlock, QuantFusedMixtralMoEBlock
from .packed_linear import PackedLinear, is_packed_linear
