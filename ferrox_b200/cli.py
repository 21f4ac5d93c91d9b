"""Command line in the reference's llama.cpp manner:

    ferrox -m MODEL_DIR -p "prompt" -n 64 --temp 0.8

Options keep the reference's names, defaults and meanings where it has them
(crates/ferrox-cli/src/run.rs:20-125): ``-m/--model``, ``-p/--prompt``, ``-f/--file``,
``-n/--n-predict`` (128; -1 fills the context), ``-c/--ctx-size`` (0 = the model's),
``--temp`` (0.8; 0 = greedy), ``--top-k`` (40; 0 = off), ``--top-p`` (0.95),
``--repeat-penalty`` (1.1; 1 = off), ``-s/--seed`` (-1 = from the clock),
``-e/--escape``, ``--ignore-eos``, ``--verbose-prompt``.  A leading ``run`` is
accepted and optional, as the reference inserts it itself (main.rs:254-296).
``-m`` names a model folder (config.json + safetensors) instead of a GGUF file.
Options without a counterpart here (threads, devices, GPU layers, KV dtype) are
not offered: there is one backend.  Added: ``--tokens`` (prompt as token ids),
``--dtype``, ``--page-size``, ``--num-pages``, ``--max-batch-tokens``, ``--random``.

Text prompts use the byte-level tokenizer (tokenizer.rs:40-56); the generated text
goes to stdout and, as in the reference (run.rs:680-695), one line to stderr:
``ferrox: prompt N tokens, X t/s; predict M tokens, Y t/s``.
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="ferrox", description="generation on one B200 with the model that config.json names")
    ap.add_argument("-m", "--model", help="model folder (config.json + model.safetensors)")
    ap.add_argument("--random", metavar="CONFIG_JSON", help="random weights for this config.json instead of -m")
    ap.add_argument("--weights-seed", type=int, default=0, help="seed of --random")
    ap.add_argument("-p", "--prompt", default="", help="prompt text (byte-level tokens)")
    ap.add_argument("-f", "--file", help="read the prompt from a file")
    ap.add_argument("--tokens", help="prompt as comma-separated token ids")
    ap.add_argument("-n", "--n-predict", type=int, default=128, help="tokens to predict (-1 = fill the context)")
    ap.add_argument("-c", "--ctx-size", type=int, default=0, help="context size (0 = the model's)")
    ap.add_argument("--temp", type=float, default=0.8, dest="temperature", help="temperature (0 = greedy)")
    ap.add_argument("--top-k", type=int, default=40, help="top-k (0 = off)")
    ap.add_argument("--top-p", type=float, default=0.95, help="nucleus threshold")
    ap.add_argument("--repeat-penalty", type=float, default=1.1, help="repetition penalty (1.0 = off)")
    ap.add_argument("-s", "--seed", type=int, default=-1, help="sampling seed (-1 = from the clock)")
    ap.add_argument("-e", "--escape", action="store_true", help="process \\n \\t \\r \\\\ in -p")
    ap.add_argument("--ignore-eos", action="store_true", help="do not stop at the end-of-sequence token")
    ap.add_argument("--verbose-prompt", action="store_true", help="print the prompt's token ids first")
    ap.add_argument("--trace-kernels", action="store_true",
                    help="sum the device time of every class of kernel and print the table to stderr at the end "
                         "(launches then run one by one, without CUDA graphs: for looking, not for speed)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--num-pages", type=int, default=0, help="cache pages per layer group (0 = one context's worth)")
    ap.add_argument("--max-batch-tokens", type=int, default=2048, help="token budget of one step")
    ap.add_argument("--print-ids", action="store_true", help="print generated token ids instead of text")
    return ap


def _unescape(s: str) -> str:
    return s.replace("\\n", "\n").replace("\\t", "\t").replace("\\r", "\r").replace("\\\\", "\\")


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "run":
        argv = argv[1:]
    args = build_parser().parse_args(argv)
    if not args.model and not args.random:
        print("ferrox: -m MODEL_DIR (or --random CONFIG_JSON) is required", file=sys.stderr)
        return 2

    from .engine.engine import Engine
    from .engine.scheduler import Scheduler, encode_prompt
    from .sampling.sampler import SamplingParams

    if args.trace_kernels:
        Engine.trace_start()   # before the engine is made: it then leaves CUDA graphs off
    t0 = time.time()
    cache = dict(page_size=args.page_size, max_slots=4)
    if args.ctx_size:
        cache["max_positions"] = args.ctx_size
    if args.random:
        with open(args.random) as f:
            cfg = json.load(f)
        if args.num_pages:
            cache["n_pages"] = args.num_pages
        else:
            cache["max_tokens"] = args.ctx_size or cfg["max_position_embeddings"]
        eng = Engine.from_random(cfg, seed=args.weights_seed, dtype=args.dtype, **cache)
    else:
        from .config.schema import load_json

        if args.num_pages:
            cache["n_pages"] = args.num_pages
        else:
            cache["max_tokens"] = args.ctx_size or load_json(args.model)["max_position_embeddings"]
        eng = Engine.from_folder(args.model, dtype=args.dtype, **cache)
    print(f"ferrox: loaded in {time.time() - t0:.2f}s", file=sys.stderr)

    as_ids = args.print_ids
    if args.tokens:
        prompt = encode_prompt([int(t) for t in args.tokens.split(",") if t.strip()], eng.spec.vocab_size)
        as_ids = True
    else:
        text = args.prompt
        if args.file:
            with open(args.file, "r", encoding="utf-8") as f:
                text = f.read()
        if args.escape:
            text = _unescape(text)
        prompt = encode_prompt(text, eng.spec.vocab_size)
    if not prompt:
        prompt = [0]  # the reference runs token 0 at position 0 for an empty prompt (run.rs:651-654)
    ctx = eng.cache.max_positions
    if len(prompt) >= ctx:
        print(f"ferrox: prompt length {len(prompt)} >= context size {ctx}; raise -c or shorten prompt", file=sys.stderr)
        return 1
    if args.verbose_prompt:
        print(f"ferrox: prompt tokens: {prompt}", file=sys.stderr)
    seed = args.seed if args.seed >= 0 else int(time.time_ns() & 0x7FFFFFFFFFFFFFFF)
    params = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                            repetition_penalty=args.repeat_penalty, seed=seed)
    sched = Scheduler(eng, max_batch_tokens=args.max_batch_tokens)
    rid = sched.add_request(prompt, args.n_predict, params, eos_ids=() if args.ignore_eos else eng.spec.eos_token_ids)
    req = sched.requests[rid]

    import torch

    out = sys.stdout
    printed = 0
    t_prefill = time.time()
    prefill_secs = None
    while not sched.idle:
        sched.step()
        if prefill_secs is None and req.generated:
            torch.cuda.synchronize()
            prefill_secs = time.time() - t_prefill
            t_decode = time.time()
        new = req.generated[printed:]
        printed = len(req.generated)
        if new:
            if as_ids:
                out.write("".join(f"{t} " for t in new))
            else:
                out.buffer.write(bytes(t for t in new if t < 256))
            out.flush()
    torch.cuda.synchronize()
    if prefill_secs is None:
        prefill_secs, decode_secs = time.time() - t_prefill, 0.0
    else:
        decode_secs = time.time() - t_decode
    out.write("\n")
    out.flush()
    n_gen = len(req.generated)
    ptps = len(prompt) / prefill_secs if prefill_secs > 0 else 0.0
    dtps = max(0, n_gen - 1) / decode_secs if decode_secs > 0 else 0.0
    print(f"ferrox: prompt {len(prompt)} tokens, {ptps:.2f} t/s; predict {n_gen} tokens, {dtps:.2f} t/s", file=sys.stderr)
    if args.trace_kernels:
        times = Engine.trace_stop()
        total = sum(ms for _, ms in times.values()) or 1.0
        print("ferrox: device time by part and entry point (launches one by one, no graphs):", file=sys.stderr)
        for key, (n, ms) in sorted(times.items(), key=lambda kv: -kv[1][1]):
            print(f"ferrox:   {key:40s} {n:7d} launches {ms:10.3f} ms {100.0 * ms / total:5.1f} %", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
