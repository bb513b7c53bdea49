from .op import gcu_index, linear_rope, linear_swiglu, rms_norm_residual, rope, rope_kv_append, rope_tables, sdpa_flash, swiglu, swiglu_packed  # noqa: F401
