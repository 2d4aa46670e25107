"""The step function and what it owns: the model, its weights and the cache.

``ModelRunner.step(entries)`` runs exactly the tokens it is given, as one batch,
from the cache that earlier steps left, and returns float32 logits at the wanted
places.  The reference's counterpart is ``ModelRunner.forward`` over a
``ForwardBatch`` built for one mode (sid/engine/model_runner.py:36-96); its
numerics pinning (TF32 and reduced-precision reductions off, :28-33) is kept for
the library matrix products.
"""

from __future__ import annotations

import time

import torch

from ..cache.manager import CacheManager, pages_for_budget
from ..config.engine_config import EngineConfig
from ..models.registry import build_model, config_from_dir
from ..weights.loader import load_weights
from ..weights.random_init import random_tensors_on_device
from .batch import SequenceInput, StepBatch, build_step_batch, check_packed

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def pin_numerics() -> None:
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False


class ModelRunner:
    def __init__(self, cfg: EngineConfig):
        pin_numerics()
        self.cfg = cfg
        self.device = torch.device(cfg.device)
        self.dtype = _TORCH_DTYPES[cfg.dtype]
        # every kernel wrapper refuses tensors that are not on a CUDA device, so a
        # CPU device fails at the first operation with that message
        self.model_config = (config_from_dir(cfg.model_path) if cfg.model_path is not None
                             else cfg.model_config)
        self.model = build_model(self.model_config, self.dtype, self.device)
        specs = self.model.tensor_specs()
        with torch.inference_mode():
            if cfg.model_path is not None:
                tensors = load_weights(cfg.model_path, specs, self.model.plan, self.dtype, self.device)
            else:
                tensors = random_tensors_on_device(specs, cfg.random_seed, self.dtype, self.device)
            self.model.load(tensors)
        self.max_positions = self.model.plan.max_positions
        if self.dtype == torch.bfloat16 and self.device.type == "cuda":
            from ..kernels import gemm_bf16
            gemm_bf16.set_library_products(cfg.library_products)
            if cfg.large_products is not None:
                gemm_bf16.set_large_products(cfg.large_products)
        num_pages = cfg.num_pages + 1
        if cfg.gpu_memory_fraction is not None and self.device.type == "cuda":
            free, _ = torch.cuda.mem_get_info(self.device)
            num_pages = pages_for_budget(self.model.cache_specs(), int(free * cfg.gpu_memory_fraction),
                                         cfg.page_size, self.dtype, cfg.max_reqs + 1,
                                         cfg.max_prefill_tokens)
        self.cache = CacheManager(self.model.cache_specs(), num_pages=num_pages,
                                  page_size=cfg.page_size, max_reqs=cfg.max_reqs + 1,
                                  max_seq_len=min(cfg.max_seq_len, self.max_positions),
                                  dtype=self.dtype, device=self.device)
        self.steps_run = 0
        self.tokens_run = 0
        # pure-decode steps, and steps of any other shape that come again, are replayed as
        # CUDA graphs
        self.step_graphs = self.decode_graphs = None
        if cfg.cuda_graphs and self.device.type == "cuda":
            from .graphs import DecodeGraphs, StepGraphs
            self.step_graphs = StepGraphs(self.model, self.cache, self.device)
            self.decode_graphs = DecodeGraphs(self.model, self.cache, self.device)
        self._checked_kernels = False
        self._check = None
        if cfg.debug_checks:
            groups = list(self.cache.page_groups.values())
            vocab = self.model.plan.vocab_size
            self._check = lambda host, lay, prev=0: check_packed(
                host, lay, self.cache, groups, vocab, self.max_positions, prev)
            for g in (self.step_graphs, self.decode_graphs):
                if g is not None:
                    g.check = self._check

    @torch.inference_mode()
    def step(self, entries: list[SequenceInput], prev_tokens=None):
        """Returns (logits float32 [R, V], the StepBatch).  Row order: the wanted
        places of the batch's sequences in batch order; ``batch.logit_rows[i]``
        are the rows of the caller's i-th entry.  ``prev_tokens`` (int32, on the
        device): the tokens the previous step sampled, for entries whose last token
        is still there (``pending_row``)."""
        for e in entries:
            self.cache.allocate(e.slot, e.num_computed + len(e.tokens))
        self.cache.reset_fresh_state()
        replayed = None
        if self.decode_graphs is not None and self.decode_graphs.usable(entries):
            replayed = self.decode_graphs.run(entries, prev_tokens)
        elif self.step_graphs is not None:
            replayed = self.step_graphs.run(entries, prev_tokens)
        if replayed is not None:
            logits, batch = replayed
        else:
            check = None
            if self._check is not None:
                n_prev = 0 if prev_tokens is None else int(prev_tokens.shape[0])
                check = lambda host, lay: self._check(host, lay, n_prev)
            # with graphs on, a launched step runs with the rows its bucket's graph will have
            pad_to = None
            if self.step_graphs is not None and not self.cache.state_groups \
                    and any(len(e.tokens) > 1 for e in entries):
                pad_to = self.step_graphs.padded_tokens
            timed = self.step_graphs is not None and self.step_graphs._launching is not None
            if timed:
                t0 = time.perf_counter()
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record()
            batch = build_step_batch(entries, self.cache, self.device, check=check, pad_to=pad_to)
            if batch.num_patches:
                from ..kernels import ops
                ops.patch_token_ids(batch.input_ids, batch.patch_dst, batch.patch_src, prev_tokens)
            logits = self.model.forward(batch, self.cache)
            if timed:
                # what the step graphs decide by: did the host keep the GPU waiting?
                ev1.record()
                self.step_graphs.launched(time.perf_counter() - t0, ev0, ev1)
            if not self._checked_kernels and self.device.type == "cuda":
                # the first launched step loads the kernel libraries: read their error
                # words once here (a synchronisation), later ones at the engine's checks
                from ..kernels import ops
                ops.check_kernel_status()
                self._checked_kernels = True
        for e in entries:
            self.cache.release_passed(e.slot, e.num_computed + len(e.tokens))
        if self._check is not None:
            self.cache.check_invariants()
        self.steps_run += 1
        self.tokens_run += sum(len(e.tokens) for e in entries)
        return logits, batch
