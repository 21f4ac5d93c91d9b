"""The engine: a model, its cache and the step function behind one object.

    eng = Engine.from_folder("model_dir", dtype="bfloat16")
    out = eng.generate([[1, 2, 3]], max_new_tokens=16)          # list of token-id lists

``dtype="bfloat16"`` runs the serving kernels; ``dtype="float32"`` runs the whole
model in true 32-bit arithmetic.  The engine needs a CUDA device and the kernel
library; there is no CPU path.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..config.registry import resolve
from ..config.schema import load_json
from ..parts.base import Runtime
from ..parts.build import build_model
from ..weights import loader as wl
from ..weights.random_init import random_tensors
from .batch import StepEntry
from .step import GraphedDecode, step as _step

DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
}


def _dtype(d) -> torch.dtype:
    if isinstance(d, torch.dtype):
        if d not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {d}: the engine runs in bfloat16 or float32")
        return d
    try:
        return DTYPES[str(d).lower()]
    except KeyError:
        raise ValueError(f"dtype {d!r}: expected bfloat16 or float32") from None


class Engine:
    def __init__(self, config, spec, model, *, page_size=64, n_pages=None, max_tokens=None, max_slots=64,
                 max_positions=None, cuda_graphs=True):
        """Use :meth:`from_folder` or :meth:`from_random`.  The cache pool holds
        ``n_pages`` pages per group, or enough for ``max_tokens`` positions."""
        self.config = config
        self.spec = spec
        self.model = model
        self.rt: Runtime = model.rt
        self.page_size = page_size
        max_positions = max_positions or spec.max_positions
        if n_pages is None:
            if max_tokens is None:
                max_tokens = min(max_positions * 4, 65536)
            n_pages = (max_tokens + page_size - 1) // page_size
        self.cache = CacheManager(
            model.cache_specs(), page_size=page_size, n_pages=n_pages, max_slots=max_slots,
            max_positions=max_positions, device=self.rt.device, dtype=self.rt.dtype,
        )
        # decode steps replay CUDA graphs when every part of the model can be captured (and no kernel trace is on:
        # a replayed graph's kernels cannot be timed one by one)
        from ..kernels import ops

        traced = ops.trace_enabled()
        self.graphs = GraphedDecode(model, self.cache) if cuda_graphs and not traced and model.graph_safe() else None

    # ---- construction ---------------------------------------------------------
    @classmethod
    def from_folder(cls, folder: str, dtype="bfloat16", device="cuda:0", **cache_opts) -> "Engine":
        _require_cuda(device)
        config, spec = resolve(load_json(folder))
        model = build_model(spec)
        rt = Runtime(torch.device(device), _dtype(dtype))
        src, files = wl.open_folder(folder, model.tensor_decls(), rt.device, rt.dtype)
        try:
            model.load(src, rt)
        finally:
            files.close()
        return cls(config, spec, model, **cache_opts)

    @classmethod
    def from_random(cls, config, seed=0, dtype="bfloat16", device="cuda:0", std=0.02, norm_init="ones",
                    on_device=False, **cache_opts) -> "Engine":
        """Random weights without a folder, by the rule of ``weights.random_init`` (the same values as
        ``write_random_model`` writes for this configuration and seed).  ``on_device=True`` draws them on the device
        (fast for large models); the values are the same bit for bit."""
        _require_cuda(device)
        obj = load_json(config) if isinstance(config, str) else config
        config, spec = resolve(obj)
        model = build_model(spec)
        rt = Runtime(torch.device(device), _dtype(dtype))
        decls = {d.name: d for d in model.tensor_decls()}
        from ..weights.random_init import random_tensor

        gen_device = rt.device if on_device else "cpu"
        src = wl.WeightSource(
            lambda n: random_tensor(decls[n], seed, torch.bfloat16, std, norm_init, gen_device),
            decls.keys(), rt.device, rt.dtype, stored_dtype=lambda n: torch.bfloat16,
        )
        model.load(src, rt)
        return cls(config, spec, model, **cache_opts)

    # ---- the step function ------------------------------------------------------
    def open_request(self) -> Optional[int]:
        return self.cache.open_request()

    def close_request(self, slot: int) -> None:
        self.cache.close_request(slot)

    def step(self, entries: Sequence[StepEntry], check: bool = True) -> torch.Tensor:
        """Run the entries' tokens as one batch; [wanted, vocab] float32 logits."""
        return _step(self.model, self.cache, entries, check=check, graphs=self.graphs)

    def decode_ahead(self, slots, tokens, sampling=None):
        """Decoding of these requests issued one step ahead of the host (see
        :class:`~ferrox_b200.engine.step.DecodeAhead`), or None while no graph of this batch size exists.  Greedy, or
        with ``sampling`` (per request its SamplingParams and generator) sampled inside the graph."""
        from .step import DecodeAhead

        if not DecodeAhead.ready(self.graphs, len(slots)):
            return None
        return DecodeAhead(self.model, self.cache, self.graphs, slots, tokens, sampling)

    # ---- tracing ------------------------------------------------------------------
    @staticmethod
    def trace_start() -> None:
        """Device time per class of kernel from now on (see ``kernels.ops``): call before the engine is made, so
        that it leaves CUDA graphs off; :meth:`trace_stop` returns the sums."""
        from ..kernels import ops

        ops.trace_start()

    @staticmethod
    def trace_stop() -> dict:
        from ..kernels import ops

        return ops.trace_stop()

    # ---- generation -------------------------------------------------------------
    def generate(self, prompts, max_new_tokens=128, temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.0,
                 seed=0, ignore_eos=False, eos_token_id=None, max_batch_tokens=2048, return_stats=False):
        """Greedy (temperature 0) or sampled continuation of each prompt.  ``prompts``
        is a list of token-id lists (a single list of ints is one prompt; strings are
        encoded byte by byte).  Returns the generated ids of each prompt, in order."""
        from ..sampling.sampler import SamplingParams
        from .scheduler import Scheduler, encode_prompt

        single = bool(prompts) and isinstance(prompts[0], int)
        plist = [prompts] if single else list(prompts)
        plist = [encode_prompt(p, self.spec.vocab_size) for p in plist]
        eos = self.spec.eos_token_ids if eos_token_id is None else (
            tuple(eos_token_id) if isinstance(eos_token_id, (list, tuple)) else (eos_token_id,))
        sched = Scheduler(self, max_batch_tokens=max_batch_tokens)
        ids = []
        for i, p in enumerate(plist):
            params = SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p,
                                    repetition_penalty=repetition_penalty, seed=seed + i)
            ids.append(sched.add_request(p, max_new_tokens, params, eos_ids=() if ignore_eos else eos))
        sched.run()
        outs = [sched.result(i) for i in ids]
        outs = outs[0] if single else outs
        if return_stats:
            c = sched.counters
            n = max(1, c.decode_steps)
            return outs, {
                "steps": c.steps, "prefill_tokens": c.prefill_tokens, "decode_tokens": c.decode_step_tokens,
                "decode_steps": c.decode_steps, "decode_seconds": c.decode_seconds, "preemptions": c.preemptions,
                "ahead_steps": c.ahead_steps,
                "h2d_bytes_per_decode_step": c.decode_h2d_bytes / n, "d2h_bytes_per_decode_step": c.decode_d2h_bytes / n,
            }
        return outs


def _require_cuda(device) -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("ferrox_b200 needs a CUDA device (sm_100a); there is no CPU path")
    if torch.device(device).type != "cuda":
        raise RuntimeError(f"device {device!r}: the engine runs on CUDA devices only")
