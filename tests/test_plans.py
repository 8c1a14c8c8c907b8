"""The host-side plans of the kernels, without a GPU: how decode attention
shares a sequence's pages among CTAs."""
import pytest

from foundry_b200.kernels import ops


@pytest.fixture(autouse=True)
def b200(monkeypatch):
    monkeypatch.setattr(ops, "sm_count", lambda: 148)


def test_decode_attention_plan():
    plan = ops.decode_plan
    # 8 sequences x 8 kv heads of 128: two CTAs fit an SM, so four ranges keep all resident
    assert plan(64, 48, 128) == (4, 3)
    # from 16 sequences on, whole sequences already ask for what memory delivers
    assert plan(128, 48, 128) == (1, 3)
    # ... unless their lengths are unequal: the longest sequence's CTA is what the batch waits for
    assert plan(128, 128, 128, unequal=True) == (2, 3)
    # four CTAs of head size 64 fit an SM
    assert plan(64, 48, 64) == (8, 3)
    assert plan(256, 64, 64, unequal=True) == (2, 3)
    assert plan(256, 41, 64) == (1, 3)
    # one sequence: a cluster of eight; a very long one: several clusters of eight
    assert plan(8, 48, 128) == (8, 3)
    splits, _ = plan(8, 1024, 128)
    assert splits >= 16 and splits % 8 == 0 and 8 * splits <= 2 * 148
    # never more ranges than pages, never a cluster of 3, 5, 6 or 7
    for pairs in (1, 3, 8, 24, 40, 56, 96, 200, 600):
        for pages in (1, 2, 3, 5, 7, 20, 100):
            for dim in (16, 32, 64, 128):
                for unequal in (False, True):
                    splits, stages = plan(pairs, pages, dim, unequal)
                    assert 1 <= splits <= max(1, pages) and stages == 3
                    assert splits & (splits - 1) == 0


def test_products_of_many_rows_pick_their_form():
    """More than 128 token rows: two SMs per 256-row tile, the widest tile among
    those with the fewest rounds over the 74 pairs; up to 768 rows the one-tile
    form instead while one round of its tiles covers the product unsplit."""
    assert ops.prompt_plan(2048, 16384) == (256, 2)
    assert ops.prompt_plan(2048, 3072) == (256, 2)
    bn, form = ops.prompt_plan(600, 9 * 144)  # 3 row blocks x 9 tiles of 144 = 27 tiles: one round
    assert form == 2 and bn == 256
    splits, fits = ops._one_tile_plan(512, 3072, 3072)  # 4 x 24 tiles on 148 SMs, unsplit
    assert (splits, fits) == (1, True)
    splits, fits = ops._one_tile_plan(512, 5120, 3072)  # 160 tiles: more than a round
    assert not fits
    splits, fits = ops._one_tile_plan(64, 3072, 8192)   # 24 tiles: K shared six ways
    assert splits == 6 and fits


def test_which_fused_projection_takes_a_step():
    """The q/k/v projection with rotation and cache write in its epilogue: the
    weight-streaming product up to 16 rows, the few-rows tcgen05 product up to
    64, the token-major products beyond, each only for what its epilogue can do."""
    import torch
    w = torch.zeros((24 + 16) * 128, 3072, dtype=torch.bfloat16)
    few, some, many = (torch.zeros(n, 3072, dtype=torch.bfloat16) for n in (8, 48, 2048))
    assert ops.qkv_rope_fusable(few, w, 128, 128, None)
    assert not ops.qkv_rope_fusable(some, w, 128, 128, None)
    assert ops.qkv_rows_rope_fusable(some, w, 128, 128, None, "interleaved")
    assert not ops.qkv_rows_rope_fusable(some, w, 128, 128, None, "half")
    assert ops.qkv_tc_rope_fusable(many, w, 128, 128, None, "interleaved")
    assert not ops.qkv_tc_rope_fusable(many, w, 128, 128, None, "half")
    w48 = torch.zeros((4 + 4) * 48, 3072, dtype=torch.bfloat16)
    assert not ops.qkv_tc_rope_fusable(many, w48, 48, 48, None, "interleaved")  # 32 features straddle heads
    assert not ops.qkv_tc_rope_fusable(many.float(), w.float(), 128, 128, None, "interleaved")
    # 300 rows of this width run split along K (float32 planes): the rotary kernel stays
    narrow = torch.zeros(8 * 128, 3072, dtype=torch.bfloat16)
    assert not ops.qkv_tc_rope_fusable(torch.zeros(300, 3072, dtype=torch.bfloat16), narrow, 128,
                                       128, None, "interleaved")
