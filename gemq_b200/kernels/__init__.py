"""B200 replacements of gemq/triton_kernels: same function names and signatures."""
from .utils import (dequantize, pack_kernel_form, pack_weights_over_cols, pack_weights_over_cols_triton,
                    unpack_over_cols, unpack_over_cols_triton)
from .dequant_gemv import (dequant_gemv_rows, dequant_sel_splitk_gemv, dequant_sel_splitk_gemv_triton,
                           dequant_splitk_gemv, dequant_splitk_gemv_triton)
from .fused_dequant_bmm import (fused_dequant_down_proj, fused_dequant_down_proj_triton, fused_dequant_up_proj,
                                fused_dequant_up_proj_triton)
from .dequant_gemm import dequant_gemm, dequant_gemm_triton
from .dequant_group_gemm import dequant_group_gemm, dequant_group_gemm_triton
