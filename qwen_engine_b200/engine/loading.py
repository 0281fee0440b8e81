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


def pages_for_memory_fraction(model: DecoderModel, page_size: int, dtype: torch.dtype, device, fraction: float,
                              reserve_bytes: int = 1 << 30) -> int:
    """How many pages per cache group fit when the process may use ``fraction`` of the device's memory: what is
    left of that share after the weights (everything the process holds now) and a reserve for the steps'
    scratch memory, divided by the bytes one page takes in every group together."""
    free, total = torch.cuda.mem_get_info(torch.device(device))
    budget = int(total * fraction) - (total - free) - reserve_bytes
    specs = [s for s in model.cache_specs() if s is not None and hasattr(s, "num_kv_heads")]
    per_page = sum(2 * s.num_kv_heads * page_size * s.head_dim * dtype.itemsize for s in specs)
    if per_page == 0:
        return 1
    pages = budget // per_page
    if pages < 1:
        raise RuntimeError(f"gpu_memory_fraction = {fraction} leaves no room for the cache: {budget / 2**30:.2f} GiB "
                           f"after the weights, a page of all layers takes {per_page} bytes")
    return int(pages)


def load_model(model_dir: Optional[str], dtype: torch.dtype, device, page_size: int, num_pages: Optional[int],
               num_state_slots: int, enable_prefix_cache: bool = True, config: Optional[ModelConfig] = None,
               random_seed: Optional[int] = None, random_std: float = 0.02, random_norm_std: float = 0.1,
               poison_cache=False, check_device: bool = True,
               use_cuda_graphs: bool = True, gpu_memory_fraction: Optional[float] = None) -> LoadedModel:
    """Read ``config.json``, pick the model class by its ``architectures`` entry, load
    ``model.safetensors`` by tensor name (or draw seeded random weights when ``model_dir``
    is None and a configuration is given), and set up the cache and the step function.
    ``num_pages`` None: the cache is sized from ``gpu_memory_fraction`` once the weights are on the device."""
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
    if num_pages is None:
        if gpu_memory_fraction is None:
            raise ValueError("the number of pages, or the share of the device's memory to size the cache from, is needed")
        num_pages = pages_for_memory_fraction(model, page_size, dtype, device, gpu_memory_fraction)
    cache = CacheManager(model.cache_specs(), page_size, num_pages, num_state_slots, dtype, device,
                         enable_prefix_cache=enable_prefix_cache, poison=poison_cache)
    runner = ModelRunner(model, cache, device, dtype, use_cuda_graphs=use_cuda_graphs)
    return LoadedModel(config, model, cache, runner)
