"""The plans that split a matrix product over K (host arithmetic only)."""
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
