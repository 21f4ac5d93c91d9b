"""A plain, slow implementation of Qwen2-MoE: whole sequences, no cache, one
function per part.  It is the yardstick the engine is measured against and shares
no code with the product path (it even reads safetensors by itself).

Provenance: the reference (antonellof/ferrox) is a Rust workspace and no Rust
toolchain exists on the machines this was written on, so its model code could not
be compiled or imported; this file rests on the reference's formulas, cited per
function as ``path:line`` inside the reference tree.  ``tests/golden`` anchors it
on the reference's own golden logits where its fixture files are at hand.

Everything runs in the dtype given (float32 by default; float64 to arbitrate when
two 32-bit results differ by rounding).  Run on the CPU.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, Optional

import numpy as np
import torch


# --------------------------------------------------------------------------- files
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """8-byte little-endian header length, JSON header, data
    (crates/ferrox-safetensors/src/lib.rs:154-277)."""
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n].decode("utf-8"))
    data = raw[8 + n:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        shape = info["shape"]
        if info["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(data[b:e], dtype="<f4").copy())
        elif info["dtype"] == "BF16":
            # bf16 -> f32: the 16 bits are the high half (crates/ferrox-quant/src/lib.rs:193-201)
            u = np.frombuffer(data[b:e], dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).copy())
        elif info["dtype"] == "F16":
            t = torch.from_numpy(np.frombuffer(data[b:e], dtype="<f2").astype(np.float32))
        else:
            raise ValueError(f"{name}: dtype {info['dtype']} not handled by the plain reader")
        out[name] = t.reshape(shape)
    return out


def load_model(folder: str, dtype=torch.float32):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w = {k: v.to(dtype) for k, v in read_safetensors(os.path.join(folder, "model.safetensors")).items()}
    return cfg, w


# --------------------------------------------------------------------------- config questions
def head_dim(cfg) -> int:
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def layer_is_moe(cfg, l: int) -> bool:
    """Dense where mlp_only_layers lists the layer, where there are no experts, or
    where decoder_sparse_step skips it (the reference only knows leading dense
    layers, crates/ferrox-models/src/config.rs:247-249)."""
    if cfg.get("num_experts", 0) == 0 or l in cfg.get("mlp_only_layers", []):
        return False
    return (l + 1) % cfg.get("decoder_sparse_step", 1) == 0


def layer_window(cfg, l: int) -> Optional[int]:
    if cfg.get("use_sliding_window", False) and cfg.get("sliding_window") and l >= cfg.get(
        "max_window_layers", cfg["num_hidden_layers"]
    ):
        return cfg["sliding_window"]
    return None


# --------------------------------------------------------------------------- parts
def rms_norm(x, w, eps):
    """x * (1/sqrt(mean(x^2)+eps)) * w (crates/ferrox-core/src/matmul.rs:62-69)."""
    scale = 1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x * scale * w


def rope_neox(x, positions, theta):
    """x: [T, heads, d].  Pairs (i, i+d/2) rotated by pos * theta^(-2i/d)
    (crates/ferrox-core/src/attention.rs:20-32)."""
    d = x.shape[-1]
    half = d // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = 1.0 / torch.pow(torch.tensor(theta, dtype=x.dtype), (2 * i) / d)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]  # [T, half]
    sin, cos = torch.sin(angle)[:, None, :], torch.cos(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)


def attention(q, k, v, window: Optional[int]):
    """q: [T, nh, d], k, v: [T, nkv, d]; query t sees keys max(0, t-W+1)..t; head h
    uses kv head h // (nh/nkv); scale 1/sqrt(d); softmax over the visible keys
    (crates/ferrox-core/src/attention.rs:402-452 causal, :484-524 window)."""
    T, nh, d = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = 1.0 / math.sqrt(d)
    out = torch.zeros_like(q)
    t = torch.arange(T)
    visible = t[None, :] <= t[:, None]
    if window is not None:
        visible &= t[None, :] > t[:, None] - window
    for h in range(nh):
        kv = h // group
        s = (q[:, h, :] @ k[:, kv, :].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, kv, :]
    return out


def attention_block(x, w, cfg, l, positions):
    """q/k/v projections with bias, rotary on q and k, attention, output projection
    (crates/ferrox-models/src/decoder.rs:2075-2157)."""
    p = f"model.layers.{l}.self_attn."
    nh, nkv, d = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"]), head_dim(cfg)
    T = x.shape[0]

    def proj(name, heads):
        y = x @ w[p + name + ".weight"].T
        if p + name + ".bias" in w:
            y = y + w[p + name + ".bias"]
        return y.reshape(T, heads, d)

    q, k, v = proj("q_proj", nh), proj("k_proj", nkv), proj("v_proj", nkv)
    theta = cfg.get("rope_theta", 10000.0)
    q, k = rope_neox(q, positions, theta), rope_neox(k, positions, theta)
    o = attention(q, k, v, layer_window(cfg, l))
    return o.reshape(T, nh * d) @ w[p + "o_proj.weight"].T


def silu(x):
    """x / (1 + exp(-x)) (crates/ferrox-core/src/matmul.rs:268-272)."""
    return x / (1.0 + torch.exp(-x))


def swiglu_mlp(x, gate, up, down):
    """down( silu(gate x) * (up x) ) (crates/ferrox-moe/src/lib.rs:655-658)."""
    return (silu(x @ gate.T) * (x @ up.T)) @ down.T


def route(logits, k, renorm, chosen=None):
    """Softmax over all experts, the k largest in descending order (lowest index
    first among equals), weights = those probabilities, divided by their sum when
    renorm (crates/ferrox-moe/src/lib.rs:333-355).  ``chosen``: this set of experts
    instead of the k largest (what a router with slightly rounded logits may decide)."""
    p = torch.softmax(logits, dim=-1)
    order = sorted(range(p.numel()) if chosen is None else chosen, key=lambda e: (-float(p[e]), e))[:k]
    wts = p[order]
    if renorm:
        wts = wts / wts.sum()
    return order, wts


def router_margins(x, w, cfg, l):
    """For each token, how clearly the router separates the last expert it takes from
    the first it leaves out: the gap between their logits, relative to the largest
    |logit| of the token.  A reduced-precision engine cannot be expected to make the
    same choice where this gap is a few roundings of a logit."""
    lg = x @ w[f"model.layers.{l}.mlp.gate.weight"].T
    k = cfg["num_experts_per_tok"]
    if lg.shape[-1] <= k:
        return torch.full((x.shape[0],), float("inf"))
    top = torch.topk(lg, k + 1, dim=-1).values
    return ((top[:, k - 1] - top[:, k]) / lg.abs().max(dim=-1).values).to(torch.float32)


def moe_block(x, w, cfg, l, chosen=None):
    """Router, routed experts summed in rank order, shared expert scaled by
    sigmoid(w_sg . x) (crates/ferrox-moe/src/lib.rs:735-752;
    crates/ferrox-models/src/decoder.rs:2660-2681).  The tokens that chose an expert go
    through it together (the reference buckets tokens by expert the same way,
    decoder.rs:2792-2890); every token's outputs are then added in the order of its ranks."""
    p = f"model.layers.{l}.mlp."
    T = x.shape[0]
    k, renorm = cfg["num_experts_per_tok"], cfg.get("norm_topk_prob", False)
    router_logits = x @ w[p + "gate.weight"].T
    picks = [route(router_logits[t], k, renorm, chosen) for t in range(T)]
    by_expert = {}
    for t, (experts, _) in enumerate(picks):
        for e in experts:
            by_expert.setdefault(e, []).append(t)
    expert_out = {}
    for e, rows in by_expert.items():
        y = swiglu_mlp(x[rows], w[p + f"experts.{e}.gate_proj.weight"], w[p + f"experts.{e}.up_proj.weight"],
                       w[p + f"experts.{e}.down_proj.weight"])
        for i, t in enumerate(rows):
            expert_out[(t, e)] = y[i]
    out = torch.zeros_like(x)
    for t, (experts, wts) in enumerate(picks):
        y = torch.zeros_like(x[t])
        for e, wt in zip(experts, wts):
            y = y + wt * expert_out[(t, e)]
        out[t] = y
    if p + "shared_expert.gate_proj.weight" in w:
        s = swiglu_mlp(x, w[p + "shared_expert.gate_proj.weight"], w[p + "shared_expert.up_proj.weight"],
                       w[p + "shared_expert.down_proj.weight"])
        if p + "shared_expert_gate.weight" in w:
            g = torch.sigmoid(x @ w[p + "shared_expert_gate.weight"].reshape(-1))
            s = s * g[:, None]
        out = out + s
    return out


def moe_block_token_by_token(x, w, cfg, l):
    """The same block one token at a time, as the reference's single-token path runs it
    (crates/ferrox-moe/src/lib.rs:735-752); kept to check the bucketed form above."""
    p = f"model.layers.{l}.mlp."
    out = torch.zeros_like(x)
    k, renorm = cfg["num_experts_per_tok"], cfg.get("norm_topk_prob", False)
    router_logits = x @ w[p + "gate.weight"].T
    for t in range(x.shape[0]):
        experts, wts = route(router_logits[t], k, renorm)
        y = torch.zeros_like(x[t])
        for e, wt in zip(experts, wts):
            y = y + wt * swiglu_mlp(
                x[t], w[p + f"experts.{e}.gate_proj.weight"], w[p + f"experts.{e}.up_proj.weight"],
                w[p + f"experts.{e}.down_proj.weight"],
            )
        out[t] = y
    if p + "shared_expert.gate_proj.weight" in w:
        s = swiglu_mlp(x, w[p + "shared_expert.gate_proj.weight"], w[p + "shared_expert.up_proj.weight"],
                       w[p + "shared_expert.down_proj.weight"])
        if p + "shared_expert_gate.weight" in w:
            g = torch.sigmoid(x @ w[p + "shared_expert_gate.weight"].reshape(-1))
            s = s * g[:, None]
        out = out + s
    return out


def dense_block(x, w, l):
    p = f"model.layers.{l}.mlp."
    return swiglu_mlp(x, w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"])


# --------------------------------------------------------------------------- whole model
def close_choices(logits, k, rel):
    """The sets of k experts that differ from the k largest in one expert, where the one
    left and the one taken both lie within rel * max|logit| of the border between taken
    and left out: the choices a router may make whose logits are off by that much."""
    order = sorted(range(logits.numel()), key=lambda e: (-float(logits[e]), e))
    if len(order) <= k:
        return []
    band = rel * float(logits.abs().max())
    lo, hi = float(logits[order[k]]), float(logits[order[k - 1]])
    out = [e for e in order[:k] if float(logits[e]) <= lo + band]
    into = [e for e in order[k:] if float(logits[e]) >= hi - band]
    return [[e for e in order[:k] if e != a] + [b] for a in out for b in into]


def one_layer_position(cfg, w, h_t, n_t, chosen):
    """Logits of one position of a model of ONE layer from its residual stream after attention
    (h_t), the normed input of the feed-forward (n_t) and the experts its router is to take."""
    assert cfg["num_hidden_layers"] == 1
    h = h_t[None] + moe_block(n_t[None], w, cfg, 0, chosen)
    hn = rms_norm(h, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-6))
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return (hn @ head.T)[0]


def forward(cfg, w, tokens, return_hidden=False, return_margins=False, return_ffn_inputs=False):
    """Logits [T, vocab] for one whole sequence starting at position 0
    (crates/ferrox-models/src/decoder.rs:3014-3677 and :2952-2973).  ``return_ffn_inputs``:
    also, for the last layer, the residual stream after attention and the normed input of
    the feed-forward."""
    dtype = w["model.embed_tokens.weight"].dtype
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    eps = cfg.get("rms_norm_eps", 1e-6)
    h = w["model.embed_tokens.weight"][tokens].clone()
    margins = torch.full((tokens.numel(),), float("inf"))
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        h = h + attention_block(rms_norm(h, w[p + "input_layernorm.weight"], eps), w, cfg, l, positions)
        n = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        if layer_is_moe(cfg, l) and return_margins:
            margins = torch.minimum(margins, router_margins(n, w, cfg, l))
        ffn_inputs = (h, n)
        h = h + (moe_block(n, w, cfg, l) if layer_is_moe(cfg, l) else dense_block(n, w, l))
    hn = rms_norm(h, w["model.norm.weight"], eps)
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    logits = hn @ head.T
    assert logits.dtype == dtype
    if return_ffn_inputs:
        return logits, margins, ffn_inputs
    if return_margins:
        return logits, margins
    return (logits, h) if return_hidden else logits


def greedy(cfg, w, prompt, n_new):
    """Greedy continuation by recomputing the whole sequence for every token."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(cfg, w, seq)[-1]))
        out.append(nxt)
        seq.append(nxt)
    return out
