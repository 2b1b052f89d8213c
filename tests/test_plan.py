"""The backward's planner (host logic, no GPU)."""

from fold_attention_b200.backward.plan import Plan, plan_dense, plan_varlen, tile_config, work_items


def test_the_dense_plan_follows_the_request_shape():
    # both headline shapes keep a key block's dK / dV inside one CTA
    assert plan_dense(4, 32, 32, 8192, 128, True) == Plan(1, 0)
    assert plan_dense(4, 32, 8, 8192, 128, True) == Plan(4, 0)
    assert plan_dense(2, 32, 8, 8192, 128, True) == Plan(4, 0)
    # too few, too long whole-group items for 148 SMs: cut the group
    assert plan_dense(2, 32, 1, 8192, 128, True) == Plan(4, 0) and Plan(4, 0).folds(32)
    # a whole group may be a larger share of an SM's tiles than a folding subgroup: its dK / dV stay private
    assert plan_dense(1, 32, 8, 8192, 128, True) == Plan(4, 0) and not Plan(4, 0).folds(4)
    assert plan_dense(1, 16, 4, 8192, 128, True) == Plan(1, 0) and Plan(1, 0).folds(4)
    # one long sequence, few heads: even single heads are too long, so the query range is cut too
    assert plan_dense(1, 4, 1, 8192, 128, True) == Plan(1, 28)
    assert plan_dense(1, 8, 2, 8192, 128, True) == Plan(1, 56)
    assert plan_dense(1, 4, 4, 32768, 128, True) == Plan(1, 0)   # 256 key blocks: a single head's items already balance
    # small calls are left whole
    assert plan_dense(2, 8, 2, 1024, 128, True) == Plan(4, 0)
    assert plan_dense(1, 8, 8, 2048, 128, True) == Plan(1, 0)
    # the mma.sync main loop never folds
    assert plan_dense(2, 32, 1, 8192, 64, True, tile_config(64)) == Plan(32, 0)
    assert plan_varlen(32, 1, tile_config(96)) == Plan(32, 0)


def test_the_packed_plan_has_nothing_but_head_counts_to_read():
    assert plan_varlen(32, 8) == Plan(4, 0)
    assert plan_varlen(32, 32) == Plan(1, 0)
    assert plan_varlen(64, 8) == Plan(4, 0)
    assert plan_varlen(48, 4) == Plan(3, 0)   # 12 -> 6 -> 3


def test_work_items():
    assert work_items(4, 32, 32, 8192, Plan(1, 0)) == 4 * 32 * 64
    assert work_items(2, 32, 1, 8192, Plan(4, 0)) == 2 * 8 * 64
    assert work_items(1, 4, 4, 1024, Plan(1, 3)) == 4 * 8 * 3
