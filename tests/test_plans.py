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
