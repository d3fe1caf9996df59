from .mixed_mm import mixed_mm, pack_2xint4, pack_hqq_from_rowmajor, triton_mixed_mm

__all__ = ["mixed_mm", "pack_2xint4", "pack_hqq_from_rowmajor", "triton_mixed_mm"]
