from .moe_block import QuantFusedDeepseekV2MoEBlock, QuantFusedMixtralMoEBlock
from .packed_linear import PackedLinear, is_packed_linear
from .quant_linear import QuantLinear
from .patch import create_gemlite_from_hqq, prepare_for_inference, replace_linear_recursive, replace_moe_blocks
from .kv_cache import StaticCache, StaticLayer
from .decoder import MixtralDecoder, decode_n_tokens, decode_one_token, generate, prefill
