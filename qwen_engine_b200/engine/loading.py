"""From a model folder to a loaded model with its cache and step function."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..cache.manager import CacheManager
from ..config import ModelConfig
from ..models.decoder import DecoderModel
from ..registry import build_model, config_from_folder
from ..weights import RandomSource, SafetensorsSource
from .runner import ModelRunner


@dataclass
class LoadedModel:
    config: ModelConfig
    model: DecoderModel
    cache: CacheManager
    runner: ModelRunner


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError(f"qwen_engine_b200 runs on a CUDA device only, not on {device}")
    if not torch.cuda.is_available():
        raise RuntimeError("qwen_engine_b200 needs a CUDA device and torch sees none; there is no CPU path")
    return device


def load_model(model_dir: Optional[str], dtype: torch.dtype, device, page_size: int, num_pages: int,
               num_state_slots: int, enable_prefix_cache: bool = True, config: Optional[ModelConfig] = None,
               random_seed: Optional[int] = None, random_std: float = 0.02, random_norm_std: float = 0.1,
               poison_cache=False, check_device: bool = True,
               use_cuda_graphs: bool = True) -> LoadedModel:
    """Read ``config.json``, pick the model class by its ``architectures`` entry, load
    ``model.safetensors`` by tensor name (or draw seeded random weights when ``model_dir``
    is None and a configuration is given), and set up the cache and the step function."""
    if check_device:
        device = require_cuda(device)
        torch.cuda.set_device(device)
    if model_dir is not None:
        config = config_from_folder(model_dir)
        source, where = SafetensorsSource(model_dir), f"model folder {model_dir!r}"
    else:
        if config is None or random_seed is None:
            raise ValueError("without a model folder, a configuration and a seed are needed")
        source = None
        where = "random weights"
    model = build_model(config)
    if source is None:
        source = RandomSource(model.weight_manifest(), random_seed, random_std, random_norm_std)
    model.load_weights(source, dtype, device, where)
    cache = CacheManager(model.cache_specs(), page_size, num_pages, num_state_slots, dtype, device,
                         enable_prefix_cache=enable_prefix_cache, poison=poison_cache)
    runner = ModelRunner(model, cache, device, dtype, use_cuda_graphs=use_cuda_graphs)
    return LoadedModel(config, model, cache, runner)
