"""Architectures expressed as plans of parts."""
from .plan import LayerCall, ModelPlan

__all__ = ["LayerCall", "ModelPlan"]
