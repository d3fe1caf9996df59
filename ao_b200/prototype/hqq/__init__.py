from .hqq_tinygemm_linear import hqq_quants_to_torch_quants, hqq_to_tinygemm_weight
from .mixed_mm import mixed_mm, pack_2xint4, pack_hqq_from_rowmajor, triton_mixed_mm

__all__ = ["hqq_quants_to_torch_quants", "hqq_to_tinygemm_weight", "mixed_mm", "pack_2xint4", "pack_hqq_from_rowmajor",
           "triton_mixed_mm"]
