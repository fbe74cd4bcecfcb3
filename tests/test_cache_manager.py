"""The cache manager (C++): pages, block tables, windows, state slots (no GPU)."""
import numpy as np
import pytest

from llm_inference_lab_b200.cache import CacheManager, CapacityError, GroupConfig, StateError


def make(pages=8, page_size=4, window=0, max_requests=3, groups=None):
    groups = groups or [GroupConfig(page_size, window, pages)]
    return CacheManager(groups, max_requests)


def test_reserve_commit_close_page_math():
    c = make()
    assert c.open(7) == 0 and c.used_state_slots == 1
    c.reserve(7, 5)                                  # 5 tokens -> 2 pages of 4
    assert c.block_table(7, 0) == [0, 1] and c.free_pages(0) == 6
    assert c.reserved(7) == 5 and c.length(7) == 0   # reserved is not yet final
    c.commit(7, 5)
    c.reserve(7, 3)                                  # fills page 1 exactly: no new page
    assert c.block_table(7, 0) == [0, 1]
    c.commit(7, 3)
    c.reserve(7, 1)
    assert c.block_table(7, 0) == [0, 1, 2] and c.pages_needed(7, 0, 4) == 1
    c.commit(7, 1)
    c.close(7)
    assert c.free_pages(0) == 8 and c.free_state_slots == 3 and not c.has(7)
    c.check_consistency()


def test_freed_pages_are_used_again_first():
    c = make()
    c.open(1), c.open(2)
    c.reserve(1, 8), c.reserve(2, 4)
    assert c.block_table(1, 0) == [0, 1] and c.block_table(2, 0) == [2]
    c.close(1)
    c.open(3)
    c.reserve(3, 12)
    assert c.block_table(3, 0)[:2] == [1, 0], "the pages just given back go out first"
    c.check_consistency()


def test_capacity_errors_leave_state_untouched():
    c = make(pages=3)
    c.open(1)
    c.reserve(1, 8)
    with pytest.raises(CapacityError):
        c.reserve(1, 9)
    assert c.reserved(1) == 8 and c.free_pages(0) == 1
    assert not c.can_reserve([(1, 5)]) and c.can_reserve([(1, 4)])
    c.open(2), c.open(3)
    with pytest.raises(CapacityError, match="state slot"):
        c.open(4)
    assert not c.can_reserve([(1, 4), (2, 1)])
    c.check_consistency()


def test_rollback_returns_only_uncommitted_pages():
    c = make()
    c.open(1)
    c.reserve(1, 6), c.commit(1, 6)
    c.reserve(1, 9)                                  # a step that then fails
    assert c.free_pages(0) == 4
    c.rollback(1)
    assert c.reserved(1) == 6 and c.length(1) == 6 and c.block_table(1, 0) == [0, 1] and c.free_pages(0) == 6
    c.check_consistency()


def test_misuse_is_refused():
    c = make()
    c.open(1)
    with pytest.raises(StateError):
        c.open(1)
    with pytest.raises(StateError):
        c.commit(1, 1)                               # nothing reserved
    with pytest.raises(StateError):
        c.reserve(9, 1)                              # unknown request
    c.close(1)
    with pytest.raises(StateError):
        c.close(1)                                   # freed twice


def test_window_gives_pages_back_when_passed():
    c = make(pages=16, page_size=4, window=6)
    c.open(1)
    c.reserve(1, 10)
    assert c.block_table(1, 0) == [0, 1, 2]
    c.commit(1, 10)              # next query sits at 10 and reads keys 5..10: page 0 (keys 0..3) is out of reach
    assert c.block_table(1, 0) == [-1, 1, 2] and c.free_pages(0) == 14
    for _ in range(30):
        c.reserve(1, 1), c.commit(1, 1)
        assert c.held_pages(1, 0) <= 3
    assert c.length(1) == 40
    c.check_consistency()
    c.close(1)
    assert c.free_pages(0) == 16


def test_groups_have_pages_of_their_own():
    c = make(groups=[GroupConfig(4, 0, 6), GroupConfig(4, 5, 3)], max_requests=2)
    c.open(1)
    c.reserve(1, 12), c.commit(1, 12)
    assert c.used_pages(0) == 3 and c.held_pages(1, 1) <= 2
    with pytest.raises(CapacityError, match="group 1"):
        c.reserve(1, 12)                             # the windowed group lacks pages for so large a portion
    for _ in range(3):
        c.reserve(1, 4), c.commit(1, 4)
    assert c.used_pages(0) == 6 and c.held_pages(1, 1) <= 2
    with pytest.raises(CapacityError, match="group 0"):
        c.reserve(1, 1)
    assert c.pages_at_peak(0, 100, 8) == 25 and c.pages_at_peak(1, 100, 8) == 4 and c.pages_at_peak(1, 3, 8) == 1
    c.close(1)
    c.check_consistency()


def test_pack_writes_positions_slots_and_tables():
    c = make(groups=[GroupConfig(4, 0, 8), GroupConfig(4, 6, 8)], max_requests=4)
    c.open(10), c.open(11)
    c.reserve(10, 9), c.commit(10, 9)
    c.reserve(11, 3)
    c.reserve(10, 1)
    L = c.layout(8, 4, [4, 4])
    buf = np.full(L.total, -99, dtype=np.int32)
    c.pack([(11, 3), (10, 1)], L, buf, pad_tokens=6, pad_requests=4)
    assert buf[L.q_start:L.q_start + 5].tolist() == [0, 3, 4, 5, 6]
    assert buf[L.kv_len:L.kv_len + 4].tolist() == [3, 10, 0, 0]
    assert buf[L.pos0:L.pos0 + 2].tolist() == [0, 9]
    assert buf[L.row_req:L.row_req + 6].tolist() == [0, 0, 0, 1, 2, 3]
    assert buf[L.row_pos:L.row_pos + 6].tolist() == [0, 1, 2, 9, -1, -1]
    table10 = c.block_table(10, 0)
    assert buf[L.row_slot[0] + 3] == table10[2] * 4 + 1
    assert buf[L.row_slot[0] + 4] == -1
    got = buf[L.block_table[1]:L.block_table[1] + 16].reshape(4, 4)
    assert got[1].tolist() == c.block_table(10, 1) + [-1] and got[1][0] == -1, "the window released block 0"
    assert (got[2:] == -1).all()
    with pytest.raises(Exception):
        c.pack([(11, 3)], c.layout(2, 1, [4, 4]), buf)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    """Random opens, steps, failed steps and closes: no page is lost, held twice or freed twice."""
    rng = np.random.default_rng(seed)
    groups = [GroupConfig(4, 0, 40), GroupConfig(4, int(rng.integers(3, 20)), 24)]
    c = CacheManager(groups, 5)
    live = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.2 and c.free_state_slots:
            c.open(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.75 and live:
            rid = int(rng.choice(list(live)))
            n = int(rng.integers(1, 12))
            if c.can_reserve([(rid, n)]):
                c.reserve(rid, n)
                if rng.random() < 0.15:
                    c.rollback(rid)
                else:
                    c.commit(rid, n)
                    live[rid] += n
            else:
                with pytest.raises(CapacityError):
                    c.reserve(rid, n)
        elif live:
            rid = int(rng.choice(list(live)))
            c.close(rid)
            del live[rid]
        c.check_consistency()
        for rid, n in live.items():
            assert c.length(rid) == n and c.held_pages(rid, 0) == -(-n // 4)
            w = groups[1].window
            assert c.held_pages(rid, 1) <= -(-(w + 1) // 4) + 1
    for rid in list(live):
        c.close(rid)
    assert c.free_pages(0) == 40 and c.free_pages(1) == 24 and c.free_state_slots == 5
