"""The entry point that allocates nothing, called through its exported C symbol.

Some users of the kernel library run where device memory cannot be allocated (inside
a stream callback, a fixed-budget real-time loop, a process that gave all device
memory to another pool).  For them ``fx_decode_attention_noalloc`` keeps its scratch
in a fixed array inside the library.  This test calls that symbol directly with
ctypes, twice in a row with different inputs (the array keeps the first call's
contents), and checks both results against a plain 32-bit statement of attention
and against the ordinary entry point, which takes caller-provided scratch.  The
second call has a window that leaves the first key ranges without visible keys.  It
also checks the fixed size from both sides: the largest request that fits is
served, the next larger one is refused.  The file's name makes pytest collect it last.
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


def _plain(q, kp, vp, table, positions, nh, nkv, d, ps, window, scale):
    """softmax(q . k * scale) v per token and head over positions max(0, p - W + 1) .. p, in 32 bits on the CPU."""
    q, kp, vp, table = q.float().cpu(), kp.float().cpu(), vp.float().cpu(), table.cpu().long()
    out = torch.zeros(q.shape[0], nh, d)
    for t, pos in enumerate(positions.cpu().tolist()):
        lo = max(0, pos - window + 1) if window else 0
        idx = torch.arange(lo, pos + 1)
        k = kp[table[t, idx // ps], :, idx % ps]          # [keys, nkv, d]
        v = vp[table[t, idx // ps], :, idx % ps]
        for h in range(nh):
            kv = h // (nh // nkv)
            p = torch.softmax((k[:, kv] @ q[t, h * d:(h + 1) * d]) * scale, 0)
            out[t, h] = p @ v[:, kv]
    return out.reshape(q.shape[0], nh * d)


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
        tol = 2e-6 if dtype == torch.float32 else 1e-2
        # first against the plain statement of attention (an error common to both entry points would pass the
        # second comparison) ...
        ref = _plain(q, kp, vp, table, positions, nh, nkv, d, ps, win, scale)
        err = float((got.float().cpu() - ref).abs().max() / ref.abs().max())
        assert err < tol, (call, err)
        if win:   # the window leaves the first key ranges of the longest request empty
            assert int(positions[0]) - win + 1 >= 2 * split_len
        # ... then against the ordinary entry point
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err < tol, (call, err)


def test_no_alloc_entry_serves_the_largest_request_that_fits_and_refuses_the_next():
    """25 tokens x 31 heads x 41 key ranges x (64 + 2) floats = 2,097,150 of the array's 2,097,152 floats (head
    sizes are multiples of 4, so no request lands on the limit itself): served and right.  One key range more is
    over the limit: refused with -5 before anything is launched."""
    from ferrox_b200.kernels import ops

    fn = _symbol()
    n_tokens, nh, nkv, d, ps, length, n_splits = 25, 31, 1, 64, 16, 700, 41
    assert n_tokens * nh * n_splits * (d + 2) == 2 * 1024 * 1024 - 2
    q, kp, vp, table, positions, token_seq, seq_slot = _case(5, torch.float32, n_tokens, nh, nkv, d, ps, length)
    scale = 1.0 / math.sqrt(d)
    got = torch.full((n_tokens, nh * d), float("nan"), device=DEV)
    stream = torch.cuda.current_stream().cuda_stream

    def call(splits):
        return fn(q.data_ptr(), q.stride(0), kp.data_ptr(), vp.data_ptr(), ops.F32, table.data_ptr(), table.shape[1],
                  ps, positions.data_ptr(), token_seq.data_ptr(), seq_slot.data_ptr(), got.data_ptr(), got.stride(0),
                  n_tokens, nh, nkv, d, 0, scale, 0, splits, stream)

    assert call(n_splits) == 0
    torch.cuda.synchronize()
    ref = _plain(q, kp, vp, table, positions, nh, nkv, d, ps, 0, scale)
    assert float((got.cpu() - ref).abs().max() / ref.abs().max()) < 2e-6
    got.fill_(float("nan"))
    assert call(n_splits + 1) == -5
    torch.cuda.synchronize()
    assert torch.isnan(got).all()   # nothing ran


def test_no_alloc_entry_refuses_more_than_its_array_holds():
    fn = _symbol()
    q = torch.zeros(1, 16, device=DEV)
    # 4096 tokens x 64 heads x 16 splits x (128 + 2) floats is far beyond 2 Mi floats
    rc = fn(q.data_ptr(), 16, q.data_ptr(), q.data_ptr(), 0, q.data_ptr(), 1, 16, q.data_ptr(), q.data_ptr(),
            q.data_ptr(), q.data_ptr(), 16, 4096, 64, 64, 128, 0, 1.0, 64, 16, None)
    assert rc == -5
