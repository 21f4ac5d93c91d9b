"""The entry point that allocates nothing, called through its exported C symbol.

Some users of the kernel library run where device memory cannot be allocated (inside
a stream callback, a fixed-budget real-time loop, a process that gave all device
memory to another pool).  For them ``fx_decode_attention_noalloc`` keeps its scratch
in a fixed array inside the library.  This test calls that symbol directly with
ctypes, twice in a row with different inputs (the array keeps the first call's
contents), and checks both results against the ordinary entry point, which takes
caller-provided scratch.  It also checks that a request beyond the fixed size is
refused.  The file's name makes pytest collect it last.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _symbol():
    from ferrox_b200.kernels import lib

    fn = lib.load().fx_decode_attention_noalloc
    P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float
    fn.argtypes = [P, L, P, P, I, P, I, I, P, P, P, P, L, I, I, I, I, I, F, I, I, P]
    fn.restype = I
    return fn


def _case(seed, dtype, n_tokens, nh, nkv, d, ps, length):
    g = torch.Generator().manual_seed(seed)
    n_pages = n_tokens * (-(-length // ps)) + 2
    kp = torch.randn(n_pages, nkv, ps, d, generator=g).to(dtype).to(DEV)
    vp = torch.randn(n_pages, nkv, ps, d, generator=g).to(dtype).to(DEV)
    width = -(-length // ps)
    perm = torch.randperm(n_pages, generator=g)[: n_tokens * width].reshape(n_tokens, width)
    table = perm.to(torch.int32).to(DEV)
    q = torch.randn(n_tokens, nh * d, generator=g).to(dtype).to(DEV)
    positions = torch.randint(0, length, (n_tokens,), generator=g).to(torch.int32).to(DEV)
    positions[0] = length - 1
    token_seq = torch.arange(n_tokens, dtype=torch.int32, device=DEV)
    seq_slot = torch.arange(n_tokens, dtype=torch.int32, device=DEV)
    return q, kp, vp, table, positions, token_seq, seq_slot


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_no_alloc_entry_matches_the_ordinary_one_twice(dtype):
    from ferrox_b200.kernels import ops

    fn = _symbol()
    nh, nkv, d, ps, length, window = 8, 2, 64, 16, 300, 0
    split_len, n_splits = 64, 5
    code = ops.BF16 if dtype == torch.bfloat16 else ops.F32
    stream = torch.cuda.current_stream().cuda_stream
    for call, (seed, n_tokens, win) in enumerate([(1, 6, 0), (2, 3, 100)]):
        q, kp, vp, table, positions, token_seq, seq_slot = _case(seed, dtype, n_tokens, nh, nkv, d, ps, length)
        scale = 1.0 / math.sqrt(d)
        want = torch.empty(n_tokens, nh * d, dtype=dtype, device=DEV)
        pa = torch.empty(n_tokens, nh, n_splits, d, device=DEV)
        pm = torch.empty(n_tokens, nh, n_splits, 2, device=DEV)
        ops.decode_attention(q, kp, vp, table, ps, positions, token_seq, seq_slot, want, nh, nkv, d, win, scale,
                             split_len, n_splits, pa, pm)
        got = torch.full_like(want, float("nan"))
        before = torch.cuda.memory_allocated()
        rc = fn(q.data_ptr(), q.stride(0), kp.data_ptr(), vp.data_ptr(), code, table.data_ptr(), table.shape[1], ps,
                positions.data_ptr(), token_seq.data_ptr(), seq_slot.data_ptr(), got.data_ptr(), got.stride(0),
                n_tokens, nh, nkv, d, win, scale, split_len, n_splits, stream)
        assert rc == 0, f"call {call}: status {rc}"
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.isfinite(got.float()).all()
        # same kernels, same order of sums: the tolerance of the kernel tests is far from needed
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err < (2e-6 if dtype == torch.float32 else 1e-2), (call, err)


def test_no_alloc_entry_refuses_more_than_its_array_holds():
    fn = _symbol()
    q = torch.zeros(1, 16, device=DEV)
    # 4096 tokens x 64 heads x 16 splits x (128 + 2) floats is far beyond 2 Mi floats
    rc = fn(q.data_ptr(), 16, q.data_ptr(), q.data_ptr(), 0, q.data_ptr(), 1, 16, q.data_ptr(), q.data_ptr(),
            q.data_ptr(), q.data_ptr(), 16, 4096, 64, 64, 128, 0, 1.0, 64, 16, None)
    assert rc == -5
