"""Load-time tools around the packed format: emit it from a quantiser's output, read it from an
HQQ-format checkpoint layer, and check a packing against the weights it came from."""
from .emit import (check_packing, dequantize_torch, emit_packed_linear, pack_kernel_form_torch, quantise_codes,
                   unpack_kernel_form_torch)
from .hqq_format import hqq_pack, hqq_unpack, packed_linear_from_hqq
