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


@pytest.mark.parametrize("b,topk,k", [(1, 2048, 8), (4, 2048, 8), (8, 2048, 4), (12, 2048, 4), (16, 1024, 4), (32, 2048, 2),
                                      (37, 2048, 2), (3, 1000, 2), (5, 512, 2)])
def test_equal_partitions_are_what_the_scheduler_lays_out(b, topk, k):
    """The schedule that the attention kernel derives itself for equally long requests (pair p: partition p % k of
    request p // k, blocks [(p % k) n/k, +n/k), every part a split) is what the scheduler gives for k * b partitions and
    a fixed overhead of 0; the kernel numbers its partial records j * b + r instead of the scheduler's r * k + j."""
    n = -(-topk // 64)
    assert n % k == 0
    meta, ns = orc.sched_meta_ref(b, topk, 0, k * b, 0)
    assert ns == [r * k for r in range(b + 1)]
    for p, m in enumerate(meta):
        r, j = divmod(p, k)
        assert m[:4] == [r, r, j * (n // k), (j + 1) * (n // k)], (p, m)
        assert m[4] == j and (m[5], m[6]) == (1, 1)
    # the policy only proposes such cuts
    from sparse_mla_sm120_b200._runtime import pick_split
    parts, overhead = pick_split(b, 148, n, uniform=True)
    assert overhead != 0 or (parts % b == 0 and n % (parts // b) == 0)
