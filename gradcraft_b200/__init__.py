"""gradcraft_b200: sm_100a backend for GradCraft's training hot path (C ABI in include/gradc_b200.h)."""
from . import capi  # noqa: F401
