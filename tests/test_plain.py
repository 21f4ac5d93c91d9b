"""The plain implementation checked against the reference's own numbers and
identities (values copied from the reference's unit tests, cited per test)."""
import math

import torch

import plain_qwen2moe as plain
from ferrox_b200.sampling.sampler import XorShift64


def test_router_goldens():
    # crates/ferrox-moe/src/lib.rs:864-893: logits 1..8, k=3
    logits = torch.arange(1.0, 9.0)
    ids, w = plain.route(logits, 3, False)
    assert ids == [7, 6, 5]
    # the reference's own tolerance for these constants is 1e-4
    assert torch.allclose(w, torch.tensor([0.6323223, 0.2326232, 0.0855683]), atol=1e-4, rtol=0)
    assert abs(float(w.sum()) - 0.9505138) < 1e-4
    _, wn = plain.route(logits, 3, True)
    assert abs(float(wn.sum()) - 1.0) < 1e-6 and torch.allclose(wn, w / w.sum())
    ids, _ = plain.route(torch.tensor([0.5, 2.0, 2.0, 0.1]), 2, False)
    assert ids == [1, 2]  # equal probabilities: the lower index first


def test_rms_norm_and_silu():
    x = torch.tensor([[3.0, 4.0]])
    got = plain.rms_norm(x, torch.tensor([1.0, 2.0]), 0.0)
    s = 1.0 / math.sqrt(12.5)
    assert torch.allclose(got, torch.tensor([[3 * s, 8 * s]]))
    assert abs(float(plain.silu(torch.tensor(0.0)))) == 0.0
    assert abs(float(plain.silu(torch.tensor(1.0))) - 1 / (1 + math.exp(-1))) < 1e-7


def test_rope_pairs_split_halves_and_keeps_norm():
    x = torch.randn(5, 2, 8)
    pos = torch.tensor([0, 1, 2, 7, 100])
    y = plain.rope_neox(x, pos, 10000.0)
    assert torch.equal(y[0], x[0])  # position 0: no rotation
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    # pair (0, 4) at position 1 turns by 1 radian (frequency of i=0 is 1)
    a, b = x[1, 0, 0], x[1, 0, 4]
    assert torch.allclose(y[1, 0, 0], a * math.cos(1) - b * math.sin(1), atol=1e-6)
    assert torch.allclose(y[1, 0, 4], a * math.sin(1) + b * math.cos(1), atol=1e-6)


def test_window_identities():
    torch.manual_seed(0)
    q, k, v = torch.randn(12, 4, 8), torch.randn(12, 2, 8), torch.randn(12, 2, 8)
    full = plain.attention(q, k, v, None)
    assert torch.allclose(plain.attention(q, k, v, 12), full)  # window >= history == full (attention.rs:1043)
    w3 = plain.attention(q, k, v, 3)
    assert torch.allclose(w3[:3], full[:3]) and not torch.allclose(w3[5], full[5])
    # window ignores old keys (attention.rs:1076): changing key 0 does not move query 5 under W=3
    k2 = k.clone()
    k2[0] += 5.0
    assert torch.allclose(plain.attention(q, k2, v, 3)[5], w3[5])
    # a single key: the output is that key's value (softmax of one score)
    assert torch.allclose(full[0, 1], v[0, 0]) and torch.allclose(full[0, 2], v[0, 1])


def test_reference_generator():
    # crates/ferrox-models/src/sampling.rs:67-84
    g = XorShift64(0)
    assert g.state == 0x9E3779B97F4A7C15
    s = 42
    s ^= (s << 13) & (2**64 - 1)
    s ^= s >> 7
    s ^= (s << 17) & (2**64 - 1)
    h = XorShift64(42)
    assert h.next_u64() == s
    draws = [XorShift64(5).next_f32() for _ in range(3)]
    assert draws[0] == draws[1] and all(0.0 <= d < 1.0 for d in draws)


def test_experts_in_buckets_equal_experts_token_by_token(tmp_path):
    """The feed-forward with the tokens of an expert taken together against the same block one token at a time
    (the reference runs both forms: crates/ferrox-moe/src/lib.rs:735-752 and decoder.rs:2792-2890)."""
    from ferrox_b200 import write_random_model
    from tiny_configs import TINY_B

    folder = write_random_model(str(tmp_path / "b"), TINY_B, seed=1, std=0.3, norm_init="around_one")
    cfg, w = plain.load_model(folder, torch.float64)
    x = torch.randn(23, TINY_B["hidden_size"], dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    a, b = plain.moe_block(x, w, cfg, 1), plain.moe_block_token_by_token(x, w, cfg, 1)
    assert float((a - b).abs().max()) < 1e-12 * float(b.abs().max())
