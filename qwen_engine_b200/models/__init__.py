from .decoder import DecoderModel, LayerSpec, ModelLayout, PlanEntry
from .qwen3 import qwen3_layout

__all__ = ["DecoderModel", "LayerSpec", "ModelLayout", "PlanEntry", "qwen3_layout"]
