#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--shape a2.7b|a14b] [--repeats 3]

Default workload: the layer sizes of the Qwen1.5-MoE-A2.7B shape (24 layers, hidden
2048, 16 heads of 128, 60 experts top-4 of width 1408, shared expert 5632, vocab
151936) with random bfloat16 weights, 8 requests whose prompts of 2,048 random
tokens are prefilled first and which then decode inside a 4,096-token context.  A
"step" is one decode step of the whole batch.  ``value`` is decoded tokens per
second timed on the device with CUDA events: the region of K steps is timed
``--repeats`` times (the requests go on decoding) and the median region counts, with
the spread of the regions beside it; ``e2e`` is the same through ``Engine.generate``
with host token lists in and out.  Every point (the headline batch, batch 1 and 64,
the prompt) carries its time, its bytes or flops and its fraction of the measured
peak.  One JSON line is printed.
The weights (tens of GB) and the cache are far larger than L2, so no flush between
steps is needed.  ``--gpus N`` with N > 1 is not built: one line says so, exit 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

A27B = dict(
    architectures=["Qwen2MoeForCausalLM"], num_hidden_layers=24, hidden_size=2048, num_attention_heads=16,
    num_key_value_heads=16, head_dim=128, num_experts=60, num_experts_per_tok=4, moe_intermediate_size=1408,
    shared_expert_intermediate_size=5632, intermediate_size=5632, decoder_sparse_step=1, mlp_only_layers=[],
    norm_topk_prob=False, qkv_bias=True, vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6,
    use_sliding_window=False, tie_word_embeddings=False, max_position_embeddings=4096,
)
# The larger shape, on request (--shape a14b): Qwen2-57B-A14B, 114 GB of bfloat16 weights.
A14B = dict(
    A27B, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, num_experts=64,
    num_experts_per_tok=8, moe_intermediate_size=2560, shared_expert_intermediate_size=20480, intermediate_size=20480,
)
SHAPES = {"a2.7b": ("Qwen1.5-MoE-A2.7B shape", A27B), "a14b": ("Qwen2-57B-A14B shape", A14B)}
CONTEXT = 4096
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out, src = dict(FALLBACK_PEAKS), "fallback"
    if os.path.exists(path):
        try:
            with open(path) as f:
                m = json.load(f)
            for k in out:
                if isinstance(m.get(k), (int, float)) and m[k] > 0:
                    out[k] = float(m[k])
            src = "measured"
        except (OSError, ValueError):
            pass
    out["source"] = src
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [c.strip() for c in line.split(",")]))

    def stop(self, begin=None, end=None):
        """The samples taken between ``begin`` and ``end`` (time.monotonic() of the host; all samples if none fell there)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [r for t, r in self.rows if begin is not None and begin <= t <= end]
        for r in inside or [r for _, r in self.rows]:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm():
    # The reference is a Rust workspace; pip cannot build it and no Rust toolchain is installed.
    print(json.dumps({"impl": "reference",
                      "unavailable": "antonellof/ferrox is a Rust workspace: no cargo/rustc in this image and no "
                                     "Python package to pip-install; its CUDA path also needs GGUF quantized weights"}))
    return 0


def decode_bytes(model, eng, batch, ctx_len, n_layers):
    """Bytes one decode step has to read: every weight it uses once (for experts: the
    expected number of distinct experts per layer under uniform routing) and the
    cached keys and values of the live requests."""
    cfg = eng.config
    es = 2  # bfloat16
    H, d = cfg.hidden_size, cfg.head_dim
    attn = ((cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * d * H + H * cfg.num_attention_heads * d) * es
    router = cfg.num_experts * H * es
    expert = 3 * cfg.moe_intermediate_size * H * es
    shared = 3 * cfg.shared_expert_intermediate_size * H * es + H * es
    E, K = cfg.num_experts, cfg.num_experts_per_tok
    distinct = E * (1.0 - (1.0 - K / E) ** batch)
    per_layer = attn + router + distinct * expert + shared
    head = cfg.vocab_size * H * es
    embed_rows = batch * H * es
    kv = batch * ctx_len * 2 * cfg.num_key_value_heads * d * es * n_layers
    return per_layer * n_layers + head + embed_rows + kv


def prefill_flops(cfg, T, n_layers):
    H, d, nh, nkv = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    per_tok = 2 * H * (nh + 2 * nkv) * d + 2 * nh * d * H  # qkv, o
    per_tok += 2 * H * cfg.num_experts  # router
    per_tok += cfg.num_experts_per_tok * 3 * 2 * H * cfg.moe_intermediate_size
    per_tok += 3 * 2 * H * cfg.shared_expert_intermediate_size + 2 * H
    attn = 2 * 2 * nh * d * (T * (T + 1) / 2)  # QK^T and PV over the causal triangle
    return n_layers * (per_tok * T + attn) + 2 * H * cfg.vocab_size  # head at the last position


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", default="a2.7b", choices=sorted(SHAPES), help="layer sizes (default: the headline shape)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers of the same sizes (named in config); 0 = all")
    ap.add_argument("--points", default="1,64", help="further decode batch sizes for 'points' ('' = none)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--repeats", type=int, default=3, help="timed regions of --steps steps each; the median counts")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not built")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch

    from ferrox_b200 import Engine, StepEntry
    from ferrox_b200.kernels import ops

    torch.manual_seed(0)
    shape_name, shape = SHAPES[args.shape]
    full_layers = shape["num_hidden_layers"]
    args.layers = args.layers or full_layers
    cfg = dict(shape, num_hidden_layers=args.layers)
    point_batches = [int(b) for b in args.points.split(",") if b.strip()]
    max_batch = max([args.batch] + point_batches)
    args.repeats = max(1, args.repeats)
    total_new = args.warmup + args.repeats * args.steps + 2
    ps = args.page_size
    pages_per_req = (PREFILL_TOKENS + 2 * total_new + 8 + ps - 1) // ps + 1
    t_load = time.time()
    eng = Engine.from_random(cfg, seed=0, dtype="bfloat16", on_device=True, page_size=ps,
                             n_pages=pages_per_req * max_batch + (PREFILL_TOKENS // ps + 2), max_slots=max_batch + 1,
                             max_positions=CONTEXT)
    torch.cuda.synchronize()
    load_s = time.time() - t_load
    pk = peaks()
    V = eng.spec.vocab_size
    gen = torch.Generator().manual_seed(1)

    def random_prompt(n):
        return torch.randint(0, V, (n,), generator=gen).tolist()

    def timed(fn):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    # ---- prefill of 2,048 tokens (one request, logits at the last position) -------
    def prefill_once():
        slot = eng.open_request()
        eng.step([StepEntry(slot, random_prompt(PREFILL_TOKENS), want=[PREFILL_TOKENS - 1])], check=False)
        return slot

    for _ in range(2):
        eng.close_request(prefill_once())
    holder = {}
    pre_runs = []
    for _ in range(3):
        pre_runs.append(timed(lambda: holder.__setitem__("s", prefill_once())))
        eng.close_request(holder["s"])
    pre_ms = statistics.median(pre_runs)
    pre_flops = prefill_flops(eng.config, PREFILL_TOKENS, args.layers)
    prefill = {"value": PREFILL_TOKENS / (pre_ms / 1e3), "tokens": PREFILL_TOKENS, "ms": pre_ms,
               "frac": pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12),
               # a prompt of some 10 ms is neither a burst nor a seconds-long loop: the fraction is of the burst
               # figure (the larger denominator); the one of the sustained figure stands beside it
               "of": pk["source"] + " burst", "peak_tflops": pk["bf16_tflops"],
               "frac_of_sustained": pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12),
               "flops": pre_flops, "runs_ms": pre_runs,
               "spread_pct": 100.0 * (max(pre_runs) - min(pre_runs)) / pre_ms}

    # ---- the same prompt in portions of 256 tokens (a small token budget: every portion but the first sits behind
    # a cached prefix, which the prompt attention cuts into runs of key blocks) ------------------------------------
    def portions_once(portion=256):
        slot = eng.open_request()
        toks = random_prompt(PREFILL_TOKENS)
        for i in range(0, PREFILL_TOKENS, portion):
            last = i + portion >= PREFILL_TOKENS
            eng.step([StepEntry(slot, toks[i:i + portion], want=[len(toks[i:i + portion]) - 1] if last else [])], check=False)
        return slot

    eng.close_request(portions_once())
    por_runs = []
    for _ in range(3):
        por_runs.append(timed(lambda: holder.__setitem__("s", portions_once())))
        eng.close_request(holder["s"])
    por_ms = statistics.median(por_runs)
    prefill["portions_of_256"] = {"value": PREFILL_TOKENS / (por_ms / 1e3), "ms": por_ms, "steps": PREFILL_TOKENS // 256,
                                  "runs_ms": por_runs}

    # ---- decode ------------------------------------------------------------------
    def decode_run(batch, steps, warmup, repeats, sample_clocks=False):
        """``repeats`` timed regions of ``steps`` decode steps each, back to back on the same requests.  Returns the
        regions' (ms per step, context length in the middle of the region), the kernels launched in one region and
        the clock record over all regions."""
        slots = []
        for _ in range(batch):
            slot = eng.open_request()
            eng.step([StepEntry(slot, random_prompt(PREFILL_TOKENS), want=[])], check=False)
            slots.append(slot)
        ids = torch.randint(0, V, (batch,), generator=gen).tolist()
        out = torch.empty(batch, dtype=torch.int32, device="cuda")

        def one_step():
            nonlocal ids
            logits = eng.step([StepEntry(s, [t], want=[0]) for s, t in zip(slots, ids)], check=False)
            ids = ops.argmax(logits, out).tolist()

        run_ids = [ids]

        def k_steps():
            # the engine's own way of decoding greedily: steps replayed from the CUDA graph of this batch size, issued
            # one ahead of the host, every step's tokens read back (one step late) from pinned memory
            run = eng.decode_ahead(slots, run_ids[0])
            if run is None:
                for _ in range(steps):
                    one_step()
                run_ids[0] = ids
                return
            last = run_ids[0]
            for _ in range(steps):
                run.issue()
                if run.issued - run.collected == 2:
                    last = run.collect()
            while run.collected < run.issued:
                last = run.collect()
            run.close()
            run_ids[0] = last

        # (the sampler runs from before the warm-up, so that it is up when the timed regions begin; only samples
        # taken during them count)
        clocks = ClockSampler()
        if sample_clocks:
            clocks.start()
        for _ in range(warmup):
            one_step()
        run_ids[0] = ids
        regions, launches = [], 0
        torch.cuda.synchronize()
        t_begin = time.monotonic()
        for r in range(repeats):
            before = ops.launch_count()
            ms = timed(k_steps)
            launches = ops.launch_count() - before
            ids = run_ids[0]
            regions.append((ms / steps, PREFILL_TOKENS + warmup + r * steps + steps // 2))
        clk = clocks.stop(t_begin, time.monotonic()) if sample_clocks else None
        for s in slots:
            eng.close_request(s)
        return regions, launches, clk

    def point(batch, regions):
        """The median region of a decode point with its bytes, its fraction of the HBM peak and the regions' spread."""
        order = sorted(regions)
        ms, ctx = order[len(order) // 2]
        need = decode_bytes(eng.model, eng, batch, ctx, args.layers)
        achieved = need / (ms / 1e3) / 1e9
        return {"value": batch / (ms / 1e3), "ms_per_step": ms, "context_at_timing": ctx, "bytes_per_step": need,
                "achieved_gbs": achieved, "frac": achieved / pk["hbm_gbs"], "of": pk["source"], "repeats": len(regions),
                "ms_per_step_all": [r[0] for r in regions],
                "spread_pct": 100.0 * (order[-1][0] - order[0][0]) / ms}

    regions, launches, clk = decode_run(args.batch, args.steps, args.warmup, args.repeats, sample_clocks=True)
    head = point(args.batch, regions)
    ms_step, value, ctx_mid, need, achieved = (head["ms_per_step"], head["value"], head["context_at_timing"],
                                               head["bytes_per_step"], head["achieved_gbs"])
    points, points_detail = {}, {}
    for b in point_batches:
        pr, _, _ = decode_run(b, args.steps, 3, args.repeats)
        points_detail[f"decode_b{b}"] = point(b, pr)
        points[f"decode_b{b}"] = points_detail[f"decode_b{b}"]["value"]

    # ---- end to end through Engine.generate ------------------------------------------
    e2e = None
    if not args.no_e2e:
        prompts = [random_prompt(PREFILL_TOKENS) for _ in range(args.batch)]
        # warm-up through the same entry point (a batch size is run eagerly when it is first seen and captured as a CUDA
        # graph the second time), then the timed call.  The token budget of a step admits all prompts at once, so that
        # the requests decode together from the first step to the last: the metric is decoding at this batch size.
        budget = PREFILL_TOKENS * args.batch + args.batch
        eng.generate(prompts, max_new_tokens=max(3, args.warmup), temperature=0.0, ignore_eos=True, max_batch_tokens=budget)
        n_new = args.steps + 1
        outs, stats = eng.generate(prompts, max_new_tokens=n_new, temperature=0.0, ignore_eos=True,
                                   max_batch_tokens=budget, return_stats=True)
        assert all(len(o) == n_new for o in outs)
        e2e = {"value": stats["decode_tokens"] / stats["decode_seconds"] if stats["decode_seconds"] > 0 else None,
               "unit": "tokens/s", "h2d_bytes_per_step": stats["h2d_bytes_per_decode_step"],
               "d2h_bytes_per_step": stats["d2h_bytes_per_decode_step"], "decode_steps": stats["decode_steps"],
               "steps_issued_ahead": stats["ahead_steps"]}

    line = {
        "metric": "decode tokens/s at batch %d (%s, context %d)" % (args.batch, shape_name, CONTEXT),
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random N(0,0.02) weights drawn on the device, uniform random token ids",
        "config": {
            "model": shape_name, "layers": args.layers, "layers_full": full_layers, "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "experts": cfg["num_experts"], "top_k": cfg["num_experts_per_tok"],
            "moe_intermediate": cfg["moe_intermediate_size"],
            "shared_intermediate": cfg["shared_expert_intermediate_size"], "vocab": cfg["vocab_size"],
            "global_batch": args.batch, "seq_len": CONTEXT,
            "prompt_tokens": PREFILL_TOKENS, "context_at_timing": ctx_mid, "page_size": ps, "parallelism": "single GPU",
            "l2": "weights and cache exceed L2, no flush", "load_s": round(load_s, 1),
        },
        "repeats": args.repeats, "ms_per_step_all": head["ms_per_step_all"], "spread_pct": head["spread_pct"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "of": pk["source"], "bytes_per_step": need},
        "points": points, "points_detail": points_detail, "e2e": e2e, "gpu_launches": launches, "clocks": clk,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
