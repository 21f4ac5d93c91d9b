"""Trace replay: feed given token ids through a model step by step and write logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N
    trace_run --random CONFIG.json --seed S --dtype ... --out DIR --max-tokens N

Steps arrive on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

Every entry of a step joins one batch of the engine's own step function (the one
generation uses: same model, cache manager and kernels); nothing is sampled.  For
a step in which logits are wanted, ``<out>/<step>.f32`` receives them as
little-endian float32 [wanted, vocab], in the order of the entries and of ``want``.
After each step ``done <step>`` is printed and flushed.  Requests named in ``end``
give their pages and slot back after the step.  The cache pool is sized for
``--max-tokens`` positions (each live request's length rounded up to a page), so
pages are used again as requests end.

The reference's nearest tool prints one decode step's logits for cross-checks
(``run-real --token --pos``, crates/ferrox-cli/src/main.rs:87-101).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    src = ap.add_mutually_exclusive_group(required=True)
    src.add_argument("--model", help="folder with config.json and model.safetensors")
    src.add_argument("--random", metavar="CONFIG", help="a config.json (or a folder holding one): random weights drawn "
                     "on the device by the rule of the random-weights mode, the values a folder written by it holds")
    ap.add_argument("--seed", type=int, default=0, help="seed of --random (default 0)")
    ap.add_argument("--std", type=float, default=0.02, help="standard deviation of --random (default 0.02)")
    ap.add_argument("--norm-init", default="ones", choices=["ones", "around_one", "normal"],
                    help="norm weights of --random (default ones)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most positions live requests hold at any time (each rounded up to a page)")
    ap.add_argument("--page-size", type=int, default=64, help="positions per cache page (default 64)")
    ap.add_argument("--max-requests", type=int, default=8, help="most requests live at a time")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    from .batch import StepEntry
    from .engine import Engine

    os.makedirs(args.out, exist_ok=True)
    ps = args.page_size
    n_pages = max(1, (args.max_tokens + ps - 1) // ps)
    opts = dict(dtype=args.dtype, device=args.device, page_size=ps, n_pages=n_pages, max_slots=args.max_requests)
    if args.model is not None:
        eng = Engine.from_folder(args.model, **opts)
    else:
        eng = Engine.from_random(args.random, seed=args.seed, std=args.std, norm_init=args.norm_init, on_device=True,
                                 **opts)
    slots = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        obj = json.loads(line)
        entries = []
        for e in obj.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slot = eng.open_request()
                if slot is None:
                    raise RuntimeError(f"step {obj.get('step')}: more than {args.max_requests} live requests")
                slots[rid] = slot
            entries.append(StepEntry(slot=slots[rid], tokens=[int(t) for t in e["tokens"]],
                                     want=[int(i) for i in e.get("want", [])]))
        logits = eng.step(entries)
        if logits.shape[0] > 0:
            arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            arr.tofile(os.path.join(args.out, f"{obj['step']}.f32"))
        for rid in obj.get("end", []):
            if rid in slots:
                eng.close_request(slots.pop(rid))
        print(f"done {obj['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
