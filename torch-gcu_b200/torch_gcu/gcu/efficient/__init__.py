from .op import gcu_index, rms_norm_residual, rope, rope_tables, sdpa_flash, swiglu, swiglu_packed  # noqa: F401
