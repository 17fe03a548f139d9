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


class _Lengths:
    def __init__(self, past, bound):
        self.past, self.ctx_bound, self.n_seqs = list(past), bound, len(past)


def _attention(window=None):
    from yalm_b200.config import config_from_dict
    from yalm_b200.parts import Model, Runtime
    cfg = {"architectures": ["MistralForCausalLM"], "model_type": "mistral", "hidden_size": 4096,
           "intermediate_size": 14336, "num_hidden_layers": 1, "num_attention_heads": 32,
           "num_key_value_heads": 8, "vocab_size": 32000, "rms_norm_eps": 1e-5, "rope_theta": 1e6,
           "max_position_embeddings": 32768, "sliding_window": window, "hidden_act": "silu",
           "tie_word_embeddings": False}
    model = Model(config_from_dict(cfg).to_spec(), Runtime.shapes_only())
    return next(iter(model.layers[0].mixers().values()))


def test_chunks_per_block_of_the_decode_attention():
    att = _attention()
    plan = lambda past, bound: att.decode_chunks_per_block(_Lengths(past, bound), bound)
    # one long sequence: about six parts, not the sixteen that would give every block an SM
    assert plan([959], 1024) == 3 and plan([1899], 2048) == 6 and plan([3899], 4096) == 11
    # up to eight chunks at the step's bound: one part
    assert plan([299], 512) == 8 and plan([299] * 8, 512) == 8
    # many sequences: whole sequences, nothing to merge
    assert plan([700] * 20, 1024) == 16 and plan([100, 2000] * 32, 2048) == 32
    # counted at the lengths the sequences have when the longest reaches the bound: sixteen of
    # 700 keys fit 148 SMs in runs of 11 chunks today and of 16 (whole) at 1,024
    assert plan([699] * 16, 1024) == 16
    # eight ragged sequences at batch 8: every block resident at the bound, and no sequence
    # in more than six parts
    past = [1032, 955, 930, 798, 737, 634, 503, 207]
    cpc = plan(past, 1536)
    at_bound = [-(-(p + 1 + 1536 - 1033) // 64) for p in past]
    assert 8 * sum(-(-c // cpc) for c in at_bound) <= 148 < 8 * sum(-(-c // (cpc - 1)) for c in at_bound)
    assert max(-(-c // cpc) for c in at_bound) <= 6
    # a window bounds what a query sees, and so the chunks
    win = _attention(window=256)
    assert win.decode_chunks_per_block(_Lengths([5000], 5120), 256) == 4
    # the block shape: four warps while every block has an SM, two where many whole sequences
    # come in waves; forced figures pass through
    assert att.decode_warps(_Lengths([700] * 16, 1024), 1024, 16) == 4
    assert att.decode_warps(_Lengths([2040] * 20, 2048), 2048, 32) == 2
    assert att.decode_warps(_Lengths([700] * 16, 1024), 1024, 8) == 4       # blocks are parts: four warps
    att.rt.decode_attention_warps, att.rt.decode_attention_chunks = 2, 5
    assert att.decode_warps(_Lengths([700] * 16, 1024), 1024, 16) == 2
    assert plan([959], 1024) == 5
