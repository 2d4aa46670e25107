"""Engine and sampling options.  Names and meanings follow the reference's
``EngineConfig`` and ``SamplingParams`` (sid/config.py:60-107) where it has
them; the determinism modes, DVR windows and split-KV policy knobs of the
reference are not part of this engine.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

_DTYPES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}


@dataclass
class EngineConfig:
    # A folder with config.json and *.safetensors.  None: ``model_config`` (a typed
    # configuration, e.g. ``preset("qwen3_0_6b")``) with random weights drawn on
    # the device from ``random_seed``.
    model_path: Optional[str] = None
    model_config: Any = None
    random_seed: Optional[int] = None

    dtype: str = "bfloat16"              # "bfloat16" | "float32" (the true 32-bit path)

    # cache (sid/config.py:66-70)
    kv_pool_tokens: int = 256 * 1024     # tokens the page pool of each layer group holds
    # If set (0 < f <= 1): the pools are sized instead from the device memory that is free
    # once the weights are loaded: f of it pays for pages, shared between the groups by
    # their bytes per page (a window group gets no more than its requests can ever hold).
    gpu_memory_fraction: Optional[float] = None
    page_size: int = 16                  # tokens per page
    max_reqs: int = 256                  # per-request state slots (block-table rows)
    max_seq_len: int = 32768             # block-table width in tokens
    max_prompt_len: Optional[int] = None  # longer prompts are rejected; None: max_seq_len

    # scheduling (sid/config.py:73-74)
    max_prefill_tokens: int = 8192       # token budget of one step; prompts are cut to fit
    max_decode_batch: int = 256          # sequences running at a time

    # bfloat16 matrix products of more than 64 rows go to the library (cuBLAS), as all of
    # the reference's do.  False: every product runs on the package's own kernel, whose
    # order of summation depends on the weight's shape alone; a token's bfloat16 bits are
    # then the same whatever its step holds (prompt portions are slower).  The switch is
    # one per process: the engine built last sets it.
    library_products: bool = True
    # Which kernel takes the products of more than 64 rows while ``library_products`` is on:
    # "library", "own" (the package's tcgen05 kernel for many rows) or "auto" (the package's
    # kernel where it fuses the feed-forward's gate, the library elsewhere); None: the
    # environment's DIB200_LARGE_PRODUCTS, else "auto".  One per process, like the switch above.
    large_products: Optional[str] = None

    # Debug checks on the host, every step: the step's packed metadata is validated before
    # it reaches the device (every index a kernel follows lies inside what it indexes) and the
    # cache manager's books are checked (no page lost, held twice or freed twice).  The
    # counterpart of the reference's SID_DEBUG_ALLOC (sid/engine/kv_cache.py:50-52).  Default:
    # the environment's DIB200_DEBUG=1.
    debug_checks: Optional[bool] = None

    cuda_graphs: bool = True             # replay pure-decode steps as CUDA graphs
    async_scheduling: bool = True        # sampled tokens stay on the device for the next step;
                                         # the host reads them one step late
    device: str = "cuda"

    def __post_init__(self):
        if self.dtype not in _DTYPES:
            raise ValueError(f"dtype must be one of {sorted(set(_DTYPES))}, got {self.dtype!r}")
        self.dtype = _DTYPES[self.dtype]
        if self.model_path is None and self.model_config is None:
            raise ValueError("EngineConfig needs model_path (a folder) or model_config")
        if self.model_path is None and self.random_seed is None:
            raise ValueError("model_config without model_path needs random_seed")
        if self.page_size < 1 or self.kv_pool_tokens < self.page_size:
            raise ValueError("page_size must be positive and kv_pool_tokens at least one page")
        for name in ("max_reqs", "max_seq_len", "max_prefill_tokens", "max_decode_batch"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be positive")
        if self.large_products not in (None, "library", "own", "auto"):
            raise ValueError("large_products must be 'library', 'own' or 'auto'")
        if self.gpu_memory_fraction is not None and not 0.0 < self.gpu_memory_fraction <= 1.0:
            raise ValueError("gpu_memory_fraction must be in (0, 1]")
        if self.debug_checks is None:
            import os
            self.debug_checks = os.environ.get("DIB200_DEBUG", "0") == "1"
        if self.max_prompt_len is None:
            self.max_prompt_len = self.max_seq_len

    @property
    def num_pages(self) -> int:
        return self.kv_pool_tokens // self.page_size


@dataclass
class SamplingParams:
    """sid/config.py:90-107 without ``is_deterministic`` (a DVR option)."""

    temperature: float = 0.0        # 0 => greedy argmax
    top_k: int = -1                 # -1 => disabled
    top_p: float = 1.0
    max_new_tokens: int = 128
    seed: int = 42
    stop_token_ids: Optional[list] = None
    ignore_eos: bool = False

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
