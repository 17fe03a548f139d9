"""The plans that split a matrix product over K, and the decode attention's choice of its
block shape (host arithmetic only)."""
import random

from yalm_b200.parts import decode_plan
from yalm_b200.parts.linear import _valid_splits, plan_splits, plan_splits_many


def test_few_tokens_fill_the_block_slots():
    # 7B sizes at batch 8: q/k/v 48 tiles -> 6 slices, o-proj 32 -> 8, down 32 -> 9
    assert plan_splits(8, 6144, 4096) == 6
    assert plan_splits(8, 4096, 4096) == 8
    assert plan_splits(8, 4096, 14336) == 9
    for M, N, K in ((1, 4096, 4096), (8, 2048, 8192), (64, 4096, 14336), (16, 640, 448)):
        S = plan_splits(M, N, K)
        assert S >= 1 and _valid_splits(-(-K // 64), S)


def test_many_tokens_split_only_where_tiles_leave_pairs_idle():
    # 512 tokens x 4,096 features are 32 tiles of 256 tokens on 74 pairs: two slices fill them
    assert plan_splits_many(512, 4096, 4096) == 2
    assert plan_splits_many(512, 4096, 14336) == 2
    # from 2,048 tokens on the tiles fill the pairs by themselves
    for M in (2048, 4096, 8192):
        assert plan_splits_many(M, 4096, 4096) == 1
        assert plan_splits_many(M, 4096, 14336) == 1
        assert plan_splits_many(M, 28672, 4096) == 1
    for M in range(257, 3000, 97):
        for N, K in ((4096, 4096), (4096, 14336), (2048, 2048), (2048, 8192), (640, 448), (6144, 4096)):
            S = plan_splits_many(M, N, K)
            nkb = -(-K // 64)
            assert S == 1 or (_valid_splits(nkb, S) and nkb // S >= 16)
            # the partial sums, written and read once, stay within twice the weights' bytes
            assert S == 1 or 2 * S * M * N * 4 <= 2 * (2 * N * K)


def test_grid_time_of_the_decode_attention_estimate():
    one = decode_plan.grid_time([32768.0], 148, 4 * decode_plan.WARP_RATE)
    assert abs(one - (decode_plan.START_US + 0.5 + decode_plan.END_US)) < 1e-9
    # 149 equal blocks on 148 slots take two rounds; on 296 slots at half the rate each, one
    blocks = [32 * 32768.0] * 149
    two_rounds = decode_plan.grid_time(blocks, 148, 4 * decode_plan.WARP_RATE)
    one_round = decode_plan.grid_time(blocks, 296, 2 * decode_plan.WARP_RATE)
    assert two_rounds > 1.9 * decode_plan.grid_time(blocks[:148], 148, 4 * decode_plan.WARP_RATE) - 8
    assert one_round < two_rounds
    # many blocks: the memory's rate bounds the grid from below
    blocks = [16 * 32768.0] * 2000
    assert decode_plan.grid_time(blocks, 296, 2 * decode_plan.WARP_RATE) >= sum(blocks) / decode_plan.MEMORY_RATE


def test_decode_attention_block_shape_follows_the_measurements():
    """Cases whose faster shape was measured on a B200 at 7B sizes (8 kv heads of 128) and at
    Llama-3.2-1B sizes (8 kv heads of 64); sequences longest first, as the engine orders them."""
    pick = lambda chunks, hd=128: decode_plan.decode_warps(decode_plan.rounded(chunks), 8, hd, 148)
    assert pick([32] * 18) == 4                   # every block has an SM
    assert pick([33] * 20) == 2                   # 160 long blocks: one round of two-warp blocks
    assert pick([17] * 24) == 2
    assert pick([33] * 40) == 4                   # three rounds of four against two of two warps at half rate
    assert pick([17] * 48) == 4
    rng = random.Random(5)
    ragged = lambda n, lo, hi: sorted((-(-rng.randint(lo, hi) // 64) for _ in range(n)), reverse=True)
    for n in (20, 24, 32, 40):
        assert pick(ragged(n, 64, 2048)) == 4     # short blocks fill in behind long four-warp blocks
    for n in (64, 96, 128):
        assert pick(ragged(n, 64, 2048)) == 2     # many rounds: starts and ends under other blocks' copies
        assert pick(ragged(n, 64, 512)) == 2
    assert pick(ragged(32, 16, 1024), 64) == 4    # head size 64: two four-warp blocks share an SM anyway
    assert pick(ragged(128, 16, 1024), 64) == 2
    assert decode_plan.rounded((3, 16, 17, 33, 61)) == (3, 16, 18, 36, 64)
