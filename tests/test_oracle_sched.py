"""Scheduler oracle: the invariants the reference checks in tests/test_scheduler.py, over the
same shape grid, plus a hand-checked known answer."""
import pytest

from helpers import orc

CASES = [(1, 512, 4), (1, 512, 8), (1, 1024, 8), (1, 2048, 16), (4, 512, 8), (4, 1024, 16), (8, 512, 8),
         (8, 1024, 32), (8, 2048, 32), (16, 512, 32), (32, 512, 64), (1, 2048, 32), (16, 512, 4),
         (64, 2048, 74), (64, 2048, 64), (128, 2048, 74), (2, 2048, 1)]


@pytest.mark.parametrize("b,topk,parts", CASES)
def test_uniform(b, topk, parts):
    meta, ns = orc.sched_meta_ref(b, topk, 0, parts, 5)
    orc.verify_schedule(meta, ns, orc.expected_blocks(b, topk, 0, None, None), b)
    assert ns[b] >= b


@pytest.mark.parametrize("tl,topk,parts", [([256, 512, 128, 512], 512, 8), ([64] * 8, 512, 8),
                                          ([1024, 64, 64, 64], 1024, 8), ([0, 512], 512, 4),
                                          ([100, 200, 300], 512, 4)])
def test_topk_length(tl, topk, parts):
    b = len(tl)
    meta, ns = orc.sched_meta_ref(b, topk, 0, parts, 5, topk_length=tl)
    orc.verify_schedule(meta, ns, orc.expected_blocks(b, topk, 0, tl, None), b)


def test_extra_topk():
    tl, etl = [256, 512, 128, 512], [128, 64, 256, 0]
    meta, ns = orc.sched_meta_ref(4, 512, 256, 8, 5, topk_length=tl, extra_topk_length=etl)
    orc.verify_schedule(meta, ns, orc.expected_blocks(4, 512, 256, tl, etl), 4)


def test_known_answer_one_request_per_partition():
    # b == parts with equal lengths: each partition gets exactly one whole request
    meta, ns = orc.sched_meta_ref(4, 2048, 0, 4, 5)
    assert ns == [0, 1, 2, 3, 4]
    for i, m in enumerate(meta):
        assert m[:7] == [i, i, 0, 32, 0, 0, 0]


def test_known_answer_single_request_split():
    # 32 blocks + 5 overhead over 4 partitions: budget ceil(37/4)+5 = 15 -> 10 blocks each
    meta, ns = orc.sched_meta_ref(1, 2048, 0, 4, 5)
    assert [m[2:4] for m in meta] == [[0, 10], [10, 20], [20, 30], [30, 32]]
    assert ns == [0, 4]
    assert all(m[5] == 1 and m[6] == 1 for m in meta[:3])
