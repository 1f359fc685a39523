"""Launch plans that are plain functions of sizes (no device needed)."""

from layover_b200 import ops

SMS = 148


def test_decode_plan_for_equal_lengths_keeps_the_measured_choices():
    plan = lambda seqs, ctx: ops.decode_plan(seqs, 32, 8, 128, ctx, SMS)
    assert plan(1, 3072) == (16, 3)            # one sequence: a cluster of 16, every block on an SM of its own
    assert plan(2, 3072) == (8, 3)
    assert plan(8, 3072) == (4, 3)
    assert plan(16, 3072) == (2, 3)
    assert plan(32, 3072) == (1, 3)
    assert plan(64, 3072) == (4, 2)            # more blocks than two an SM hold: three slower ones an SM
    assert plan(1, 32768)[0] > 16              # a long lone sequence: more splits, merged through scratch memory
    assert ops.decode_plan(8, 32, 8, 64, 3072, SMS)[1] == 3      # other head sizes have the three-stage kernel only


def test_decode_plan_cuts_further_when_the_longest_sequence_stands_out():
    plan = lambda seqs, ctx, mean: ops.decode_plan(seqs, 32, 8, 128, ctx, SMS, mean)
    # a mean close to the longest changes nothing
    assert plan(32, 8192, 7000) == ops.decode_plan(32, 32, 8, 128, 8192, SMS)
    assert plan(8, 8192, 4096) == (8, 2)
    assert plan(8, 3072, 1500) == (4, 3)       # at least 12 tiles a block, and two blocks an SM still hold them
    assert plan(16, 3072, 1500) == (4, 2)
    assert plan(16, 8192, 4096) == (8, 2)
    assert plan(32, 8192, 4096) == (4, 2)
    assert plan(32, 3072, 1500) == (4, 2)
    # few blocks (one round anyway) and very many (already cut for three blocks an SM) keep their plans
    assert plan(2, 8192, 3000) == ops.decode_plan(2, 32, 8, 128, 8192, SMS)
    assert plan(128, 8192, 3000) == ops.decode_plan(128, 32, 8, 128, 8192, SMS)
    # groups of more than 8 heads have no two-stage variant
    assert ops.decode_plan(16, 64, 4, 128, 8192, SMS, 3000) == ops.decode_plan(16, 64, 4, 128, 8192, SMS)
    for seqs in range(1, 200, 7):
        for ctx in (130, 1000, 5000, 70000):
            splits, stages = plan(seqs, ctx, ctx // 3)
            assert splits >= 1 and stages in (2, 3)
