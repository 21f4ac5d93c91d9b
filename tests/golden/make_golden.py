#!/usr/bin/env python3
"""Anchors the plain implementation (tests/plain_qwen2moe.py) on the reference's own
golden logits.

The reference (antonellof/ferrox) cannot be compiled here (Rust, no toolchain), but it
ships three tiny GGUF models with the logits its decoder must produce for token 3 at
position 0 (crates/ferrox-models/tests/gguf_roundtrip.rs:17-22, 94-99, 150-172;
fixtures under crates/ferrox-models/tests/fixtures; hyper-parameters
crates/ferrox-models/src/config.rs:558-680).  This script reads those files with a
small GGUF reader (F32 and Q8_0 tensors), renames the tensors to the checkpoint
names the plain implementation uses, runs it, and writes its logits beside the
reference's constants into ``ferrox_fixture_logits.json``.  ``tests/test_golden.py``
checks the committed numbers (and recomputes them when the reference tree is there).

    python tests/golden/make_golden.py /path/to/reference

What this anchors: tensor orientation ([out, in]), RMSNorm, the head-to-kv-head map,
softmax-then-top-k routing with renormalisation, an ungated shared expert, SwiGLU, a
leading dense layer, the final norm and an untied head.  One token at position 0 does
not exercise rotary angles, multi-key softmax, q/k/v bias, the sigmoid gate, windows
or tying; those rest on the formulas cited in the plain implementation.
"""
import json
import os
import re
import struct
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import plain_qwen2moe as plain  # noqa: E402

FIXTURES = {
    "dense": ("ferrox_real_test.gguf", "GOLDEN_LOGITS"),
    "moe": ("ferrox_real_moe_test.gguf", "GOLDEN_MOE_LOGITS"),
    "mixed": ("ferrox_real_mixed_test.gguf", "GOLDEN_MIXED_LOGITS"),
}


def read_gguf(path):
    raw = open(path, "rb").read()
    pos = 0

    def take(fmt):
        nonlocal pos
        v = struct.unpack_from("<" + fmt, raw, pos)
        pos += struct.calcsize("<" + fmt)
        return v[0] if len(v) == 1 else v

    def string():
        nonlocal pos
        n = take("Q")
        s = raw[pos:pos + n].decode("utf-8")
        pos += n
        return s

    scalar = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 7: "?", 10: "Q", 11: "q", 12: "d"}

    def value(t):
        if t in scalar:
            return take(scalar[t])
        if t == 8:
            return string()
        if t == 9:
            et, n = take("I"), take("Q")
            return [value(et) for _ in range(n)]
        raise ValueError(f"GGUF value type {t}")

    assert raw[:4] == b"GGUF"
    pos = 4
    take("I")  # version
    n_tensors, n_kv = take("Q"), take("Q")
    meta = {}
    for _ in range(n_kv):
        k = string()
        meta[k] = value(take("I"))
    infos = []
    for _ in range(n_tensors):
        name = string()
        nd = take("I")
        dims = [take("Q") for _ in range(nd)]
        infos.append((name, dims, take("I"), take("Q")))
    align = meta.get("general.alignment", 32)
    start = (pos + align - 1) // align * align
    tensors = {}
    for name, dims, ty, off in infos:
        n = int(np.prod(dims))
        if ty == 0:  # F32
            a = np.frombuffer(raw, dtype="<f4", count=n, offset=start + off).astype(np.float32)
        elif ty == 8:  # Q8_0: blocks of (f16 scale, 32 x int8)
            blocks = np.frombuffer(raw, dtype=np.dtype([("d", "<f2"), ("q", "i1", 32)]), count=n // 32, offset=start + off)
            a = (blocks["d"].astype(np.float32)[:, None] * blocks["q"].astype(np.float32)).reshape(-1)
        else:
            raise ValueError(f"{name}: ggml type {ty} not handled")
        tensors[name] = torch.from_numpy(a.reshape(list(reversed(dims))).copy())  # ne[0] is the innermost extent
    return meta, tensors


def to_checkpoint_names(meta, t):
    arch = meta["general.architecture"]
    L = meta[f"{arch}.block_count"]
    w = {"model.embed_tokens.weight": t["token_embd.weight"], "model.norm.weight": t["output_norm.weight"]}
    if "output.weight" in t:
        w["lm_head.weight"] = t["output.weight"]
    moe_layers = []
    for l in range(L):
        g, p = f"blk.{l}.", f"model.layers.{l}."
        w[p + "input_layernorm.weight"] = t[g + "attn_norm.weight"]
        w[p + "post_attention_layernorm.weight"] = t[g + "ffn_norm.weight"]
        for a, b in (("attn_q", "q_proj"), ("attn_k", "k_proj"), ("attn_v", "v_proj"), ("attn_output", "o_proj")):
            w[p + f"self_attn.{b}.weight"] = t[g + a + ".weight"]
            if g + a + ".bias" in t:
                w[p + f"self_attn.{b}.bias"] = t[g + a + ".bias"]
        if g + "ffn_gate_inp.weight" in t:
            moe_layers.append(l)
            w[p + "mlp.gate.weight"] = t[g + "ffn_gate_inp.weight"]
            for e in range(t[g + "ffn_gate_exps.weight"].shape[0]):
                for a, b in (("gate", "gate_proj"), ("up", "up_proj"), ("down", "down_proj")):
                    w[p + f"mlp.experts.{e}.{b}.weight"] = t[g + f"ffn_{a}_exps.weight"][e]
            if g + "ffn_gate_shexp.weight" in t:
                for a, b in (("gate", "gate_proj"), ("up", "up_proj"), ("down", "down_proj")):
                    w[p + f"mlp.shared_expert.{b}.weight"] = t[g + f"ffn_{a}_shexp.weight"]
        else:
            for a, b in (("gate", "gate_proj"), ("up", "up_proj"), ("down", "down_proj")):
                w[p + f"mlp.{b}.weight"] = t[g + f"ffn_{a}.weight"]
    H = t["token_embd.weight"].shape[1]
    nh = meta[f"{arch}.attention.head_count"]
    cfg = dict(
        num_hidden_layers=L, hidden_size=H, num_attention_heads=nh,
        num_key_value_heads=meta.get(f"{arch}.attention.head_count_kv", nh),
        head_dim=t["blk.0.attn_q.weight"].shape[0] // nh,
        rope_theta=meta.get(f"{arch}.rope.freq_base", 10000.0),
        rms_norm_eps=meta.get(f"{arch}.attention.layer_norm_rms_epsilon", 1e-5),
        num_experts=meta.get(f"{arch}.expert_count", 0) if moe_layers else 0,
        num_experts_per_tok=meta.get(f"{arch}.expert_used_count", 1),
        mlp_only_layers=[l for l in range(L) if l not in moe_layers], decoder_sparse_step=1,
        norm_topk_prob=True,  # the fixtures' hand-written presets say so (config.rs:558-680)
    )
    return cfg, w


def reference_constants(ref_root):
    src = open(os.path.join(ref_root, "crates/ferrox-models/tests/gguf_roundtrip.rs")).read()
    out = {}
    for name in ("GOLDEN_LOGITS", "GOLDEN_MOE_LOGITS", "GOLDEN_MIXED_LOGITS"):
        m = re.search(r"const " + name + r": \[f32; (\d+)\] = \[(.*?)\];", src, re.S)
        out[name] = [float(x) for x in m.group(2).replace("\n", " ").split(",") if x.strip()]
        assert len(out[name]) == int(m.group(1))
    return out


def compute(ref_root):
    consts = reference_constants(ref_root)
    result = {}
    for key, (fname, cname) in FIXTURES.items():
        meta, tensors = read_gguf(os.path.join(ref_root, "crates/ferrox-models/tests/fixtures", fname))
        cfg, w = to_checkpoint_names(meta, tensors)
        logits = plain.forward(cfg, w, [3])[0]
        result[key] = {"fixture": fname, "config": cfg, "plain_logits": [float(x) for x in logits],
                       "reference_constant": cname, "reference_logits": consts[cname]}
    return result


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <checkout of the reference>")
    root = sys.argv[1]
    res = compute(root)
    for k, v in res.items():
        err = max(abs(a - b) for a, b in zip(v["plain_logits"], v["reference_logits"]))
        print(f"{k}: max |plain - reference| = {err:.2e}")
    with open(os.path.join(HERE, "ferrox_fixture_logits.json"), "w") as f:
        json.dump(res, f, indent=1)
