"""Each part alone against the plain implementation's function for it, and the
framework's openness: a toy mixer with per-request state, a toy architecture and a
schedule that runs a layer twice are defined HERE, registered, built, loaded from a
random model folder and stepped, with no change to the framework's files."""
import math
from dataclasses import dataclass

import pytest
import torch

import plain_qwen2moe as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = {"float32": (torch.float32, 3e-5), "bfloat16": (torch.bfloat16, 2e-2)}


def rel(got, want):
    return float((got.float().cpu() - want.float().cpu()).abs().max() / want.float().abs().max().clamp_min(1e-30))


def load_part(spec, tensors, dtype):
    from ferrox_b200.parts.base import Runtime, build_part
    from ferrox_b200.parts import build  # noqa: F401  (registers the built-in parts)
    from ferrox_b200.weights import loader as wl

    part = build_part(spec)
    rt = Runtime(torch.device(DEV), dtype)
    part.load(wl.from_dict(tensors, part.tensor_decls(), DEV, dtype), rt)
    return part, rt


def random_tensors(part_spec, seed=0, std=0.1):
    from ferrox_b200.parts.base import build_part
    from ferrox_b200.parts import build  # noqa: F401
    from ferrox_b200.weights.random_init import random_tensors as rt

    return dict(rt(build_part(part_spec).tensor_decls(), seed, torch.bfloat16, std, "around_one"))


# ------------------------------------------------------------------ parts alone
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_norm_alone(dtype):
    from ferrox_b200.parts.specs import NormSpec

    dt, tol = DTYPES[dtype]
    spec = NormSpec(size=80, eps=3e-6, prefix="n.")
    w = random_tensors(spec)
    part, rt = load_part(spec, w, dt)
    h = torch.randn(7, 80, generator=torch.Generator().manual_seed(0)) * 4
    got = part.forward(h.to(DEV))
    assert got.dtype == dt and rel(got, plain.rms_norm(h, w["n.weight"].float(), 3e-6)) < tol
    rows = torch.tensor([6, 1], dtype=torch.int32, device=DEV)
    assert torch.equal(part.forward(h.to(DEV), rows=rows), got[[6, 1]])


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_mlp_alone(dtype):
    from ferrox_b200.parts.specs import DenseMlpSpec

    dt, tol = DTYPES[dtype]
    spec = DenseMlpSpec(hidden=96, intermediate=160, prefix="m.")
    w = random_tensors(spec)
    part, rt = load_part(spec, w, dt)
    for T in (3, 70):  # the decode-sized and the prompt-sized kernels
        x = torch.randn(T, 96, generator=torch.Generator().manual_seed(T))
        h = torch.randn(T, 96, generator=torch.Generator().manual_seed(T + 1))
        xd = x.to(dt)
        want = h + plain.swiglu_mlp(xd.float(), w["m.gate_proj.weight"].float(), w["m.up_proj.weight"].float(),
                                    w["m.down_proj.weight"].float())
        hd = h.to(DEV)
        part.forward_add(xd.to(DEV), hd, _FakeBatch())
        assert rel(hd, want) < tol


class _FakeBatch:
    def __init__(self):
        from ferrox_b200.kernels import ops

        self.stream = ops.stream_ptr()
        self.status = torch.zeros(1, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("renorm,gate,shared", [(False, True, 64), (True, False, 64), (True, True, 0)])
def test_moe_alone(dtype, renorm, gate, shared):
    from ferrox_b200.parts.specs import MoeSpec

    dt, tol = DTYPES[dtype]
    spec = MoeSpec(hidden=64, n_experts=6, top_k=2, expert_intermediate=32, shared_intermediate=shared,
                   norm_topk_prob=renorm, shared_gate=gate, prefix="model.layers.0.mlp.")
    w = random_tensors(spec, std=0.3)
    if not gate:
        w = {k: v for k, v in w.items() if "shared_expert_gate" not in k}
    part, rt = load_part(spec, w, dt)
    cfg = dict(num_experts_per_tok=2, norm_topk_prob=renorm)
    wf = {k: v.float() for k, v in w.items()}
    for T in (5, 90):
        x = (torch.randn(T, 64, generator=torch.Generator().manual_seed(T))).to(dt)
        # keep tokens whose routing is decided beyond rounding
        lg = x.float() @ wf["model.layers.0.mlp.gate.weight"].T
        top = torch.topk(lg, 3, dim=-1).values
        keep = (top[:, 1] - top[:, 2]) > 0.05 * lg.abs().max()
        h = torch.randn(T, 64, generator=torch.Generator().manual_seed(T + 1))
        want = h + plain.moe_block(x.float(), wf, cfg, 0)
        hd = h.to(DEV)
        part.forward_add(x.to(DEV), hd, _FakeBatch())
        assert int(keep.sum()) > T // 2
        assert rel(hd.cpu()[keep], want[keep]) < tol


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("window,bias", [(None, True), (9, False)])
def test_attention_alone_in_two_steps(dtype, window, bias):
    """A prompt portion, then a second portion and a decoded token of another request in one batch."""
    from ferrox_b200.parts.specs import AttentionSpec, PositionSpec

    dt, tol = DTYPES[dtype]
    nh, nkv, d, H = 6, 2, 32, 80
    spec = AttentionSpec(hidden=H, n_heads=nh, n_kv_heads=nkv, head_dim=d, qkv_bias=bias,
                         position=PositionSpec(rotary_dim=d, theta=50000.0), window=window,
                         prefix="model.layers.0.self_attn.")
    w = random_tensors(spec, std=0.2)
    part, rt = load_part(spec, w, dt)
    from ferrox_b200.cache.manager import CacheManager
    from ferrox_b200.engine.batch import StepEntry, flatten
    from ferrox_b200.kernels import ops

    cm = CacheManager([part.cache_spec()], page_size=4, n_pages=64, max_slots=4, max_positions=256, device=DEV, dtype=dt)
    cfg = dict(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=d, hidden_size=H, rope_theta=50000.0,
               use_sliding_window=window is not None, sliding_window=window, max_window_layers=0, num_hidden_layers=1)
    wf = {k: v.float() for k, v in w.items()}
    g = torch.Generator().manual_seed(3)
    xa = torch.randn(30, H, generator=g).to(dt)
    xb = torch.randn(21, H, generator=g).to(dt)
    want_a = plain.attention_block(xa.float(), wf, cfg, 0, torch.arange(30))
    want_b = plain.attention_block(xb.float(), wf, cfg, 0, torch.arange(21))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    sa, sb = cm.open_request(), cm.open_request()

    def run(portions):
        entries = []
        for slot, x0, x1 in portions:
            e = StepEntry(slot, list(range(x1 - x0)))
            e.start = cm.seq_len[slot]
            assert cm.reserve(slot, e.start + x1 - x0)
            entries.append(e)
        cm.sync_tables()
        batch = flatten(entries, DEV, status, ops.stream_ptr())
        xs = torch.cat([(xa if slot == sa else xb)[x0:x1] for slot, x0, x1 in portions]).to(DEV)
        h = torch.zeros(xs.shape[0], H, dtype=torch.float32, device=DEV)
        part.forward_add(xs, h, batch, cm.layer_cache(0))
        for e in entries:
            cm.commit(e.slot, e.start + len(e.tokens))
        return h.cpu()

    h1 = run([(sa, 0, 17), (sb, 0, 20)])
    h2 = run([(sa, 17, 30), (sb, 20, 21)])
    assert int(status) == 0
    assert rel(h1[:17], want_a[:17]) < tol and rel(h1[17:], want_b[:20]) < tol
    assert rel(h2[:13], want_a[17:]) < tol and rel(h2[13:], want_b[20:]) < tol


# ------------------------------------------------------------------ toy parts and a toy architecture
@dataclass(frozen=True)
class RunningMeanSpec:
    hidden: int
    prefix: str
    kind: str = "toy_running_mean"


def _toy_classes():
    from ferrox_b200.cache.specs import CacheSpec, StateSpec
    from ferrox_b200.parts.base import Mixer
    from ferrox_b200.weights.loader import TensorDecl

    class RunningMean(Mixer):
        """h += W . mean(x of this request so far).  Its state per request is the running
        sum and the count, kept in the cache manager's slot for the request."""

        def cache_spec(self):
            return CacheSpec(state=StateSpec((self.spec.hidden + 1,), torch.float32))

        def tensor_decls(self):
            return [TensorDecl(self.spec.prefix + "mix.weight", (self.spec.hidden, self.spec.hidden))]

        def load(self, src, rt):
            super().load(src, rt)
            self.w = src.get(self.spec.prefix + "mix.weight").float()

        def forward_add(self, x, h, batch, cache):
            t = 0
            for e in batch.entries:
                n = len(e.tokens)
                st = cache.state[e.slot]
                xs = x[t:t + n].float()
                sums = st[:-1] + torch.cumsum(xs, dim=0)
                counts = st[-1] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
                h[t:t + n] += (sums / counts[:, None]) @ self.w.T
                st[:-1] = sums[-1]
                st[-1] = counts[-1]
                t += n

    return RunningMean


TOY_ARCH = "ToyMixForCausalLM"


def _register_toy():
    from ferrox_b200 import register_architecture, register_part
    from ferrox_b200.parts.specs import (AttentionSpec, BlockSpec, DenseMlpSpec, ModelSpec, NormSpec, PositionSpec,
                                         ScheduleEntry)

    register_part("toy_running_mean", _toy_classes(), replace=True)

    def config_from_json(obj):
        return dict(obj)

    def model_spec(c):
        H = c["hidden_size"]

        def block(l, mixer):
            p = f"model.layers.{l}."
            return BlockSpec(norm1=NormSpec(H, 1e-5, p + "input_layernorm."), mixer=mixer,
                             norm2=NormSpec(H, 1e-5, p + "post_attention_layernorm."),
                             ffn=DenseMlpSpec(H, c["intermediate_size"], p + "mlp."))

        attn = AttentionSpec(hidden=H, n_heads=2, n_kv_heads=1, head_dim=16, qkv_bias=False,
                             position=PositionSpec(16, 10000.0), window=None, prefix="model.layers.1.self_attn.")
        layers = (block(0, RunningMeanSpec(H, "model.layers.0.toy.")), block(1, attn))
        # layer 0 (state), layer 1 (keys and values), then layer 1 AGAIN on a cache of its own
        schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(1, 2))
        return ModelSpec(architecture=TOY_ARCH, vocab_size=c["vocab_size"], hidden=H, max_positions=64, layers=layers,
                         schedule=schedule, final_norm=NormSpec(H, 1e-5, "model.norm."), head_name="lm_head.weight")

    register_architecture(TOY_ARCH, config_from_json, model_spec, replace=True)


def _toy_plain(cfg, w, tokens):
    """The toy model, whole sequence, in plain torch."""
    H = cfg["hidden_size"]
    x = w["model.embed_tokens.weight"][torch.as_tensor(tokens)].clone()
    pos = torch.arange(len(tokens))
    acfg = dict(num_attention_heads=2, num_key_value_heads=1, head_dim=16, hidden_size=H, rope_theta=10000.0,
                num_hidden_layers=2)

    def mlp(h, l):
        n = plain.rms_norm(h, w[f"model.layers.{l}.post_attention_layernorm.weight"], 1e-5)
        return h + plain.dense_block(n, w, l)

    n = plain.rms_norm(x, w["model.layers.0.input_layernorm.weight"], 1e-5)
    mean = torch.cumsum(n, 0) / torch.arange(1, len(tokens) + 1)[:, None]
    x = mlp(x + mean @ w["model.layers.0.toy.mix.weight"].T, 0)
    for _ in range(2):
        n = plain.rms_norm(x, w["model.layers.1.input_layernorm.weight"], 1e-5)
        x = mlp(x + plain.attention_block(n, w, acfg, 1, pos), 1)
    return plain.rms_norm(x, w["model.norm.weight"], 1e-5) @ w["lm_head.weight"].T


def test_toy_mixer_with_state_and_a_layer_run_twice(tmp_path):
    import ferrox_b200
    from ferrox_b200 import Engine, StepEntry

    _register_toy()
    cfg = dict(architectures=[TOY_ARCH], hidden_size=48, intermediate_size=64, vocab_size=97)
    folder = ferrox_b200.write_random_model(str(tmp_path / "toy"), cfg, seed=4, std=0.2, norm_init="around_one")
    w = {k: v.float() for k, v in plain.read_safetensors(folder + "/model.safetensors").items()}
    eng = Engine.from_folder(folder, dtype="float32", page_size=4, n_pages=24, max_slots=3)
    assert eng.graphs is None  # a part written in Python is not captured in a CUDA graph
    assert set(eng.cache.groups) == {None} and eng.cache.groups[None].caches == [1, 2]
    assert eng.cache.layer_cache(0).k is None and eng.cache.layer_cache(0).state.shape == (3, 49)
    g = torch.Generator().manual_seed(0)
    seqs = {s: torch.randint(0, 97, (n,), generator=g).tolist() for s, n in (("a", 23), ("b", 9), ("c", 14))}
    want = {s: _toy_plain(cfg, w, t) for s, t in seqs.items()}

    def feed(slot, toks):
        return StepEntry(slot, toks, want=list(range(len(toks))))

    # a and b in mixed portions; then b ends and c takes over its slot (state zeroed, pages reused)
    sa, sb = eng.open_request(), eng.open_request()
    o1 = eng.step([feed(sa, seqs["a"][:10]), feed(sb, seqs["b"][:2])]).cpu()
    o2 = eng.step([feed(sa, seqs["a"][10:11]), feed(sb, seqs["b"][2:])]).cpu()
    eng.close_request(sb)
    sc = eng.open_request()
    assert sc == sb
    o3 = eng.step([feed(sc, seqs["c"]), feed(sa, seqs["a"][11:])]).cpu()
    got_a = torch.cat([o1[:10], o2[:1], o3[14:]])
    got_b = torch.cat([o1[10:], o2[1:]])
    got_c = o3[:14]
    for got, s in ((got_a, "a"), (got_b, "b"), (got_c, "c")):
        assert rel(got, want[s]) < 3e-5, s
    eng.close_request(sa)
    eng.close_request(sc)
    eng.cache.check_invariants()
    # generation works through the public entry point as well
    out = eng.generate([seqs["b"]], max_new_tokens=4)[0]
    assert out[0] == int(want["b"][-1].argmax())


# ------------------------------------------------------------------ more toy parts: a routed feed-forward, another position encoding
@dataclass(frozen=True)
class HashRoutedSpec:
    hidden: int
    n_branches: int
    prefix: str
    kind: str = "toy_hash_routed_ffn"


@dataclass(frozen=True)
class UnrotatedSpec:
    """A position part of another kind than the rotary one: it leaves queries and keys as projected
    (order then comes from the causal mask and the window alone)."""
    kind: str = "toy_unrotated_position"


def _register_more_toys():
    from ferrox_b200 import register_part
    from ferrox_b200.kernels import ops
    from ferrox_b200.parts.base import FeedForward
    from ferrox_b200.parts.position import PositionEncoding
    from ferrox_b200.weights.loader import TensorDecl

    class HashRouted(FeedForward):
        """Routing without a router matrix: token t of the step goes to branch (position mod n); each
        branch is a single matrix.  Shows a feed-forward that needs the batch's positions."""

        def tensor_decls(self):
            s = self.spec
            return [TensorDecl(s.prefix + f"branch.{b}.weight", (s.hidden, s.hidden)) for b in range(s.n_branches)]

        def load(self, src, rt):
            super().load(src, rt)
            self.w = torch.stack([src.get(self.spec.prefix + f"branch.{b}.weight").float()
                                  for b in range(self.spec.n_branches)])

        def forward_add(self, x, h, batch):
            branch = (batch.positions.long() % self.spec.n_branches)
            h += torch.einsum("th,toh->to", x.float(), self.w[branch])

    class Unrotated(PositionEncoding):
        def rotate_and_store(self, qkv, batch, cache, n_heads, n_kv_heads, head_dim):
            # nothing to encode: keys and values go to their pages as projected
            ops.rope_kv_write(qkv, batch.positions, batch.token_seq, batch.seq_slot, None, 0, cache.k, cache.v,
                              cache.block_table, cache.page_size, n_heads, n_kv_heads, head_dim,
                              write_cache=cache.writes, status=batch.status, stream=batch.stream)

    register_part("toy_hash_routed_ffn", HashRouted, replace=True)
    register_part("toy_unrotated_position", Unrotated, replace=True)


def test_toy_routed_feed_forward_and_unrotated_attention(tmp_path):
    """A block made of the framework's attention with a position part that does not rotate, and a toy
    feed-forward routed by position; built from specs, loaded from a random folder, stepped in two cuts."""
    import ferrox_b200
    from ferrox_b200 import Engine, StepEntry, register_architecture
    from ferrox_b200.parts.specs import AttentionSpec, BlockSpec, ModelSpec, NormSpec, ScheduleEntry

    _register_more_toys()
    H = 32

    def model_spec(c):
        p = "model.layers.0."
        attn = AttentionSpec(hidden=H, n_heads=2, n_kv_heads=2, head_dim=16, qkv_bias=True,
                             position=UnrotatedSpec(), window=5, prefix=p + "self_attn.")
        blk = BlockSpec(NormSpec(H, 1e-6, p + "input_layernorm."), attn, NormSpec(H, 1e-6, p + "post_attention_layernorm."),
                        HashRoutedSpec(H, 3, p + "mlp."))
        return ModelSpec(architecture="ToyRoutedForCausalLM", vocab_size=50, hidden=H, max_positions=64, layers=(blk,),
                         schedule=(ScheduleEntry(0, 0),), final_norm=NormSpec(H, 1e-6, "model.norm."), head_name=None)

    register_architecture("ToyRoutedForCausalLM", dict, model_spec, replace=True)
    cfg = dict(architectures=["ToyRoutedForCausalLM"])
    folder = ferrox_b200.write_random_model(str(tmp_path / "toy2"), cfg, seed=2, std=0.3, norm_init="around_one")
    w = {k: v.float() for k, v in plain.read_safetensors(folder + "/model.safetensors").items()}
    toks = [3, 9, 44, 1, 0, 17, 8, 8, 30, 2, 5]

    # plain statement, without rotation
    x = w["model.embed_tokens.weight"][torch.tensor(toks)]
    n = plain.rms_norm(x, w["model.layers.0.input_layernorm.weight"], 1e-6)
    T = len(toks)

    def proj(name, heads):
        return (n @ w[f"model.layers.0.self_attn.{name}.weight"].T + w[f"model.layers.0.self_attn.{name}.bias"]).reshape(T, heads, 16)

    o = plain.attention(proj("q_proj", 2), proj("k_proj", 2), proj("v_proj", 2), 5)
    x = x + o.reshape(T, 32) @ w["model.layers.0.self_attn.o_proj.weight"].T
    n = plain.rms_norm(x, w["model.layers.0.post_attention_layernorm.weight"], 1e-6)
    x = x + torch.stack([n[t] @ w[f"model.layers.0.mlp.branch.{t % 3}.weight"].T for t in range(T)])
    want = plain.rms_norm(x, w["model.norm.weight"], 1e-6) @ w["model.embed_tokens.weight"].T

    eng = Engine.from_folder(folder, dtype="float32", page_size=4, n_pages=8, max_slots=2)
    s = eng.open_request()
    a = eng.step([StepEntry(s, toks[:7], want=list(range(7)))]).cpu()
    b = eng.step([StepEntry(s, toks[7:], want=list(range(4)))]).cpu()
    assert rel(torch.cat([a, b]), want) < 3e-5


# ------------------------------------------------------------------ a rotary encoding of another kind, defined here
@dataclass(frozen=True)
class AdjacentRopeSpec:
    """Adjacent pairs (2i, 2i+1) with each band's frequency divided by a factor
    (the reference: crates/ferrox-core/src/attention.rs:340-352 and :319-337)."""
    rotary_dim: int
    theta: float
    factors: tuple
    kind: str = "toy_rope_adjacent"


def _register_adjacent_rope():
    from ferrox_b200 import register_part
    from ferrox_b200.kernels import ops
    from ferrox_b200.parts.position import RotaryEncoding

    class AdjacentRope(RotaryEncoding):
        pairing = ops.PAIR_ADJACENT

        def frequencies(self):
            return super().frequencies() / torch.tensor(self.spec.factors, dtype=torch.float32)

    register_part("toy_rope_adjacent", AdjacentRope, replace=True)


def _rope_adjacent_plain(x, positions, theta, factors, rotary_dim):
    """x: [T, heads, d]; attention.rs:340-352 with the per-band division of :319-337, over the first rotary_dim."""
    out = x.clone()
    half = rotary_dim // 2
    for t, pos in enumerate(positions):
        for i in range(half):
            freq = 1.0 / theta ** ((2 * i) / rotary_dim)
            angle = pos * freq / factors[i]
            s, c = math.sin(angle), math.cos(angle)
            a, b = x[t, :, 2 * i], x[t, :, 2 * i + 1]
            out[t, :, 2 * i] = a * c - b * s
            out[t, :, 2 * i + 1] = a * s + b * c
    return out


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("rotary", [16, 12])
def test_toy_rotary_encoding_with_adjacent_pairs_and_band_factors(tmp_path, dtype, rotary):
    """Another position encoding is another part: adjacent pairs, per-band frequency factors and a rotary width below
    the head size, registered here, built by the framework's attention from its spec, run in two cuts and a decode
    step, against a plain statement of the reference's interleaved formula."""
    import ferrox_b200
    from ferrox_b200 import Engine, StepEntry, register_architecture
    from ferrox_b200.parts.specs import AttentionSpec, BlockSpec, DenseMlpSpec, ModelSpec, NormSpec, ScheduleEntry

    _register_adjacent_rope()
    H, nh, nkv, d, theta = 48, 3, 1, 16, 500.0
    factors = tuple(1.0 + 0.5 * i for i in range(rotary // 2))

    def model_spec(c):
        p = "model.layers.0."
        attn = AttentionSpec(hidden=H, n_heads=nh, n_kv_heads=nkv, head_dim=d, qkv_bias=True,
                             position=AdjacentRopeSpec(rotary, theta, factors), window=None, prefix=p + "self_attn.")
        blk = BlockSpec(NormSpec(H, 1e-6, p + "input_layernorm."), attn, NormSpec(H, 1e-6, p + "post_attention_layernorm."),
                        DenseMlpSpec(H, 64, p + "mlp."))
        return ModelSpec(architecture="ToyAdjacentRopeForCausalLM", vocab_size=61, hidden=H, max_positions=64, layers=(blk,),
                         schedule=(ScheduleEntry(0, 0),), final_norm=NormSpec(H, 1e-6, "model.norm."), head_name=None)

    register_architecture("ToyAdjacentRopeForCausalLM", dict, model_spec, replace=True)
    folder = ferrox_b200.write_random_model(str(tmp_path / "toy3"), dict(architectures=["ToyAdjacentRopeForCausalLM"]),
                                            seed=6, std=0.3, norm_init="around_one")
    w = {k: v.float() for k, v in plain.read_safetensors(folder + "/model.safetensors").items()}
    toks = [(7 * i + 3) % 61 for i in range(29)]
    T = len(toks)
    x = w["model.embed_tokens.weight"][torch.tensor(toks)]
    n = plain.rms_norm(x, w["model.layers.0.input_layernorm.weight"], 1e-6)

    def proj(name, heads):
        return (n @ w[f"model.layers.0.self_attn.{name}.weight"].T + w[f"model.layers.0.self_attn.{name}.bias"]).reshape(T, heads, d)

    q = _rope_adjacent_plain(proj("q_proj", nh), range(T), theta, factors, rotary)
    k = _rope_adjacent_plain(proj("k_proj", nkv), range(T), theta, factors, rotary)
    x = x + plain.attention(q, k, proj("v_proj", nkv), None).reshape(T, nh * d) @ w["model.layers.0.self_attn.o_proj.weight"].T
    n = plain.rms_norm(x, w["model.layers.0.post_attention_layernorm.weight"], 1e-6)
    x = x + plain.dense_block(n, w, 0)
    want = plain.rms_norm(x, w["model.norm.weight"], 1e-6) @ w["model.embed_tokens.weight"].T

    dt, tol = DTYPES[dtype]
    eng = Engine.from_folder(folder, dtype=dtype, page_size=4, n_pages=8, max_slots=2)
    assert eng.graphs is not None   # the part only enqueues kernels: decode steps are captured
    s = eng.open_request()
    outs = [eng.step([StepEntry(s, toks[:11], want=list(range(11)))]).cpu(),
            eng.step([StepEntry(s, toks[11:26], want=list(range(15)))]).cpu()]
    for t in range(26, T):   # decode steps: eager, captured, replayed
        outs.append(eng.step([StepEntry(s, toks[t:t + 1], want=[0])]).cpu().clone())
    assert rel(torch.cat(outs), want) < tol
    # and the pairing matters: the split-half rule on the same weights gives other logits
    assert rel(torch.cat(outs), _with_halves(w, toks, theta, factors, rotary, H, nh, nkv, d)) > 10 * tol


def _with_halves(w, toks, theta, factors, rotary, H, nh, nkv, d):
    T = len(toks)
    x = w["model.embed_tokens.weight"][torch.tensor(toks)]
    n = plain.rms_norm(x, w["model.layers.0.input_layernorm.weight"], 1e-6)

    def proj(name, heads):
        return (n @ w[f"model.layers.0.self_attn.{name}.weight"].T + w[f"model.layers.0.self_attn.{name}.bias"]).reshape(T, heads, d)

    def rot(v):
        out = v.clone()
        out[..., :rotary] = plain.rope_neox(v[..., :rotary], torch.arange(T), theta)
        return out

    x = x + plain.attention(rot(proj("q_proj", nh)), rot(proj("k_proj", nkv)), proj("v_proj", nkv), None).reshape(
        T, nh * d) @ w["model.layers.0.self_attn.o_proj.weight"].T
    n = plain.rms_norm(x, w["model.layers.0.post_attention_layernorm.weight"], 1e-6)
    x = x + plain.dense_block(n, w, 0)
    return plain.rms_norm(x, w["model.norm.weight"], 1e-6) @ w["model.embed_tokens.weight"].T


# ------------------------------------------------------------------ a mixer whose pages hold one vector per position
@dataclass(frozen=True)
class LatentAttentionSpec:
    hidden: int
    latent: int
    window: object
    prefix: str
    kind: str = "toy_latent_attention"


def _register_latent_mixer():
    from ferrox_b200 import register_part
    from ferrox_b200.cache.specs import CacheSpec, PagedSpec, PagedTensorSpec
    from ferrox_b200.parts.base import Mixer
    from ferrox_b200.weights.loader import TensorDecl

    class LatentAttention(Mixer):
        """c_t = Wc x_t is all a position stores (one vector, no separate keys and values); the output at t is
        Wo . softmax_s(c_t . c_s / sqrt(latent)) c_s over the visible positions s of its request."""

        def cache_spec(self):
            s = self.spec
            return CacheSpec(paged=PagedSpec((PagedTensorSpec("latent", (s.latent,), dtype=torch.float32),), s.window))

        def tensor_decls(self):
            s = self.spec
            return [TensorDecl(s.prefix + "down.weight", (s.latent, s.hidden)),
                    TensorDecl(s.prefix + "up.weight", (s.hidden, s.latent))]

        def load(self, src, rt):
            super().load(src, rt)
            self.w_c = src.get(self.spec.prefix + "down.weight").float()
            self.w_o = src.get(self.spec.prefix + "up.weight").float()

        def forward_add(self, x, h, batch, cache):
            pages, ps, W = cache.pages["latent"], cache.page_size, self.spec.window
            t = 0
            for e in batch.entries:
                n = len(e.tokens)
                c = x[t:t + n].float() @ self.w_c.T
                row = cache.block_table[e.slot].long()
                new = torch.arange(e.start, e.start + n, device=x.device)
                assert int(row[new // ps].min()) >= 0
                pages[row[new // ps], new % ps] = c
                lo = 0 if W is None else max(0, e.start - W + 1)
                old = torch.arange(lo, e.start + n, device=x.device)
                assert int(row[old // ps].min()) >= 0, "a position inside the window has lost its page"
                ctx = pages[row[old // ps], old % ps]                     # [keys, latent], read back from the pages
                sc = (c @ ctx.T) / math.sqrt(self.spec.latent)
                vis = old[None, :] <= new[:, None]
                if W is not None:
                    vis &= old[None, :] > new[:, None] - W
                p = torch.softmax(sc.masked_fill(~vis, float("-inf")), dim=-1)
                h[t:t + n] += (p @ ctx) @ self.w_o.T
                t += n

    register_part("toy_latent_attention", LatentAttention, replace=True)


@pytest.mark.parametrize("window", [None, 6])
def test_toy_mixer_with_one_vector_per_position_in_pages(tmp_path, window):
    """A mixer declares its own paged payload (one 24-wide vector per position, 32-bit, no keys and values); the
    manager gives it pages and a block table like any other layer, in a group of its own when its window differs,
    gives pages back past the window and at the end, and another request uses them again."""
    import ferrox_b200
    import replay_util as ru
    from ferrox_b200 import Engine, register_architecture
    from ferrox_b200.parts.specs import AttentionSpec, BlockSpec, DenseMlpSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry

    _register_latent_mixer()
    H, L = 40, 24

    def model_spec(c):
        def block(l, mixer):
            p = f"model.layers.{l}."
            return BlockSpec(NormSpec(H, 1e-6, p + "input_layernorm."), mixer, NormSpec(H, 1e-6, p + "post_attention_layernorm."),
                             DenseMlpSpec(H, 56, p + "mlp."))

        attn = AttentionSpec(hidden=H, n_heads=2, n_kv_heads=2, head_dim=16, qkv_bias=False,
                             position=PositionSpec(16, 10000.0), window=None, prefix="model.layers.1.self_attn.")
        layers = (block(0, LatentAttentionSpec(H, L, window, "model.layers.0.mix.")), block(1, attn))
        return ModelSpec(architecture="ToyLatentForCausalLM", vocab_size=83, hidden=H, max_positions=64, layers=layers,
                         schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1)),
                         final_norm=NormSpec(H, 1e-6, "model.norm."), head_name="lm_head.weight")

    register_architecture("ToyLatentForCausalLM", dict, model_spec, replace=True)
    folder = ferrox_b200.write_random_model(str(tmp_path / "toy4"), dict(architectures=["ToyLatentForCausalLM"]),
                                            seed=8, std=0.3, norm_init="around_one")
    w = {k: v.float() for k, v in plain.read_safetensors(folder + "/model.safetensors").items()}
    acfg = dict(num_attention_heads=2, num_key_value_heads=2, head_dim=16, hidden_size=H, rope_theta=10000.0,
                num_hidden_layers=2)

    def whole(toks):
        T = len(toks)
        x = w["model.embed_tokens.weight"][torch.tensor(toks)]
        n = plain.rms_norm(x, w["model.layers.0.input_layernorm.weight"], 1e-6)
        c = n @ w["model.layers.0.mix.down.weight"].T
        t = torch.arange(T)
        vis = t[None, :] <= t[:, None]
        if window is not None:
            vis &= t[None, :] > t[:, None] - window
        p = torch.softmax(((c @ c.T) / math.sqrt(L)).masked_fill(~vis, float("-inf")), dim=-1)
        x = x + (p @ c) @ w["model.layers.0.mix.up.weight"].T
        x = x + plain.dense_block(plain.rms_norm(x, w["model.layers.0.post_attention_layernorm.weight"], 1e-6), w, 0)
        n = plain.rms_norm(x, w["model.layers.1.input_layernorm.weight"], 1e-6)
        x = x + plain.attention_block(n, w, acfg, 1, t)
        x = x + plain.dense_block(plain.rms_norm(x, w["model.layers.1.post_attention_layernorm.weight"], 1e-6), w, 1)
        return plain.rms_norm(x, w["model.norm.weight"], 1e-6) @ w["lm_head.weight"].T

    g = torch.Generator().manual_seed(1)
    prompts = {f"r{i}": torch.randint(0, 83, (n,), generator=g).tolist() for i, n in enumerate((31, 9, 22, 40, 17))}
    want = {r: whole(t) for r, t in prompts.items()}
    # so few pages that they are used again: 3 live requests of up to 40 positions, pages of 4
    eng = Engine.from_folder(folder, dtype="float32", page_size=4, n_pages=3 * 10, max_slots=3)
    assert set(eng.cache.groups) == ({None} if window is None else {None, window})
    lat = eng.cache.layer_cache(0)
    assert lat.k is None and lat.pages["latent"].shape == (30, 4, L) and lat.pages["latent"].dtype == torch.float32
    got = ru.run_mixed(eng, prompts, seed=3, max_live=3, max_portion=7)
    for r in prompts:
        assert rel(got[r], want[r]) < 3e-5, r
    assert all(n == eng.cache.groups[k].pool.n_pages for k, n in eng.cache.free_pages().items())
    if window is not None:
        assert eng.cache.peak_pages[window] < eng.cache.peak_pages[None]   # the windowed group gave pages back early
