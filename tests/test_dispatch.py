"""The host-side choices between kernels and launch shapes (pure functions of sizes; no GPU)."""
from ferrox_b200.kernels import ops
from ferrox_b200.parts.moe import expert_tile_tokens


def test_decode_split_plan_depends_on_sizes_only_and_stays_in_bounds():
    for tokens in (1, 2, 3, 8, 16, 33, 64, 200):
        for kv_blocks in (1, 4, 16, 28):
            for ctx in (64, 500, 4096, 32768):
                split_len, n = ops.decode_split_plan(tokens, kv_blocks, ctx)
                assert split_len == 0 and 1 <= n <= ops.DECODE_MAX_SPLITS
                assert n <= max(1, -(-ctx // 64))          # no run shorter than one tile of keys
                assert (split_len, n) == ops.decode_split_plan(tokens, kv_blocks, ctx)
    # 8 tokens x 16 kv heads: two runs fill one wave (256 of 444 blocks); a third adds no bandwidth
    assert ops.decode_split_plan(8, 16, 4096) == (0, 2)
    # the kernel that holds two blocks an SM and writes a single run's result itself
    assert ops.decode_split_plan(8, 16, 4096, 2, single_is_final=True) == (0, 2)
    assert ops.decode_split_plan(16, 16, 4096, 2, single_is_final=True) == (0, 1)
    assert ops.decode_split_plan(64, 16, 4096, 2, single_is_final=True) == (0, 1)
    # a single request: many runs, but no more than fill the machine
    assert 8 <= ops.decode_split_plan(1, 16, 4096)[1] <= ops.DECODE_MAX_SPLITS
    assert 8 <= ops.decode_split_plan(1, 16, 4096, 2, single_is_final=True)[1] <= ops.DECODE_MAX_SPLITS
    # many requests already fill the machine
    assert ops.decode_split_plan(200, 16, 4096)[1] <= 2


def test_which_product_kernel_takes_which_sizes():
    # few tokens against a big matrix: swapped roles only where measured faster
    assert not ops.swap_better(8, 6144, 2048) and ops.swap_better(40, 6144, 2048)
    assert ops.swap_better(8, 151936, 2048) and not ops.swap_better(4, 151936, 2048)
    assert not ops.swap_better(64, 2048, 5632)              # few rows of W: too few tiles
    # plain dense products of few tokens: runs of K so that 150 to 300 CTAs stream the matrix
    assert ops.swap_k_splits(64, 2048, 2048) == 8 and ops.swap_k_splits(64, 2048, 5632) == 8
    assert ops.swap_k_splits(64, 6144, 2048) == 4 and ops.swap_k_splits(8, 2048, 2048) == 0
    assert ops.swap_k_splits(32, 2048, 5632) > 0 and ops.swap_k_splits(32, 2048, 2048) == 0
    assert ops.swap_k_splits(64, 2048, 256) == 1      # never more runs than K allows
    # pairs of SMs need two rounds of 256 x 256 tiles for 74 pairs
    assert ops.pairs_better(2048, 6144) and not ops.pairs_better(2048, 2048) and not ops.pairs_better(512, 6144)
    assert ops.pairs_better(2048, 5632, gated=True)


def test_expert_tile_tokens_by_rows_per_expert():
    assert expert_tile_tokens(8, 4, 60) == (32, 32)
    assert expert_tile_tokens(64, 4, 60) == (32, 32)
    assert expert_tile_tokens(200, 4, 60) == (64, 64)
    assert expert_tile_tokens(2048, 4, 60) is None
    assert expert_tile_tokens(16, 8, 10) == (64, 64)       # few experts: more rows each


def test_decode_attention_by_tma_where_pages_and_heads_fit_its_boxes():
    import torch

    bf, f32 = torch.bfloat16, torch.float32
    # head sizes in steps of 64 on pages of a multiple of 64 positions, bfloat16 only
    assert ops.decode_tma_blocks_per_sm(bf, 128, 64) == 2 and ops.decode_tma_blocks_per_sm(bf, 64, 128) == 2
    assert ops.decode_tma_blocks_per_sm(bf, 256, 64) == 1 and ops.decode_tma_blocks_per_sm(bf, 192, 64) == 1
    for dtype, d, ps in ((f32, 128, 64), (bf, 96, 64), (bf, 128, 16), (bf, 128, 96), (bf, 320, 64), (bf, 0, 64)):
        assert ops.decode_tma_blocks_per_sm(dtype, d, ps) == 0


def test_routing_in_one_block_only_for_small_steps():
    assert ops.ROUTE_SMALL_MAX_TOKENS <= 64      # the one-block kernel takes a token per warp and round
    assert 32 * ops.ROUTE_SMALL_MAX_EXPERTS * 4 + (2 * ops.ROUTE_SMALL_MAX_EXPERTS + 1) * 4 <= 48 * 1024   # its shared memory


def test_prompt_attention_items_cover_every_key_block_once():
    """The planner of the tcgen05 prompt attention: every tile's key blocks are covered exactly once by its items, in
    order; a tile that was cut has consecutive parts and one merge row; heavy items come first; the cut depends on the
    step's sizes alone."""
    import random

    rng = random.Random(0)
    for trial in range(60):
        entries = [(rng.randint(1, 3000), rng.choice([0, 0, 5, 127, 128, 1000, 4097])) for _ in range(rng.randint(1, 4))]
        window = rng.choice([0, 0, 1, 100, 2048])
        heads = rng.choice([1, 16, 28])
        run_blocks = rng.choice([-1, -1, 0, 1, 2, 5])
        items, merges, parts = ops.prefill_tc_plan(entries, window, heads, run_blocks=run_blocks)
        again = ops.prefill_tc_plan(entries, window, heads, run_blocks=run_blocks)
        assert (items == again[0]).all() and (merges == again[1]).all() and parts == again[2]
        lengths = [int(it[5] - it[4]) for it in items]
        assert lengths == sorted(lengths, reverse=True) and min(lengths) >= 1
        by_tile = {}
        for tok0, rows, b, pos0, kb, ke, part, _ in items.tolist():
            by_tile.setdefault((tok0, rows, b, pos0), []).append((kb, ke, part))
        flat, n_tiles = 0, 0
        for b, (n, start) in enumerate(entries):
            for i in range(0, n, 256):
                rows, pos0 = min(256, n - i), start + i
                runs = sorted(by_tile[(flat + i, rows, b, pos0)])
                first = (max(0, pos0 - window + 1) if window else 0) // 128
                end = (pos0 + rows - 1) // 128 + 1
                assert runs[0][0] == first and runs[-1][1] == end
                assert all(a[1] == c[0] for a, c in zip(runs, runs[1:]))            # no gap, no overlap
                if len(runs) == 1:
                    assert runs[0][2] == -1
                else:
                    ps = [r[2] for r in runs]
                    assert ps == list(range(ps[0], ps[0] + len(runs))) and len(runs) <= ops.PREFILL_MAX_RUNS
                    assert [flat + i, rows, ps[0], len(runs)] in merges.tolist()
                n_tiles += 1
            flat += n
        assert len(by_tile) == n_tiles and parts == sum(m[3] for m in merges.tolist())
    # a prompt of 2,048 tokens on 16 heads: 128 whole tiles fit the 148 SMs at once; cutting would cost more than it saves
    items, merges, parts = ops.prefill_tc_plan([(2048, 0)], None, 16, sms=148)
    assert len(items) == 8 and parts == 0 and len(merges) == 0
    # a portion of 256 tokens behind 6,000 cached positions: one tile with 49 key blocks, cut so that all SMs work
    items, merges, parts = ops.prefill_tc_plan([(256, 6000)], None, 16, sms=148)
    assert parts == len(items) >= 6 and merges.tolist() == [[0, 256, 0, parts]]
    assert max(int(it[5] - it[4]) for it in items) <= 8
    # forced runs of four key blocks
    items, merges, parts = ops.prefill_tc_plan([(2048, 0)], None, 16, sms=148, run_blocks=4)
    assert len(items) == 20 and max(int(it[5] - it[4]) for it in items) == 4 and len(merges) == 6
