"""Host side of the step loop: page pool invariants and the scheduling policy of the reference engine
(engine.py:143-252) on scripted scenarios with made-up sampled tokens.  No GPU, no torch."""
import pytest

from inference_engine_b200.engine import PagePool, Scheduler


def test_page_pool_promises_and_pages():
    pool = PagePool(10, first=2)  # pages 2..9
    assert pool.uncommitted() == 8
    assert pool.commit(5) and not pool.commit(4) and pool.uncommitted() == 3
    got = [pool.take(), pool.take()]
    assert got == [2, 3] and pool.committed == 3 and pool.uncommitted() == 3
    pool.release(got, leftover_promises=3)
    assert pool.committed == 0 and pool.uncommitted() == 8 and sorted(pool.free) == list(range(2, 10))


def make(max_batch=4, max_len=64, page=16, pages=64, budget=24, min_first=8, stop=-1):
    pool = PagePool(pages)
    return Scheduler(max_batch, max_len, page, pool, budget, min_first, stop), pool


def test_policy_decoders_first_then_chunks_then_admissions():
    s, pool = make()
    a = s.submit(list(range(100, 130)), 3)  # 30-token prompt
    b = s.submit(list(range(200, 205)), 2)  # 5-token prompt
    # step 1: budget 24: A's first chunk takes all of it, B is not admitted (no budget left)
    st = s.plan()
    assert [(r.id, len(t)) for r, t in st.entries] == [(0, 24)] and st.num_decoding == 0 and not st.decode_only
    assert len(a.pages) == 2 and a.committed == 0  # lifetime ceil((30 + 3 - 1) / 16) = 2 pages, both in use already
    assert s.commit(st, [7]) == [] and a.cached_len == 24 and a.output == []
    # step 2: A continues with its last 6 tokens, then B is admitted with its whole 5-token prompt
    st = s.plan()
    assert [(r.id, t) for r, t in st.entries] == [(0, list(range(124, 130))), (1, list(range(200, 205)))]
    assert s.commit(st, [11, 22]) == [] and a.output == [11] and b.output == [22] and a.t_first_token is not None
    # step 3: both decode, decoders first in running order, one token each = the last sampled one
    st = s.plan()
    assert st.decode_only and [(r.id, t) for r, t in st.entries] == [(0, [11]), (1, [22])]
    fin = s.commit(st, [12, 23])
    assert [r.id for r in fin] == [1] and b.output == [22, 23] and b.pages == [] and b.t_finish is not None
    # step 4: A's last token; afterwards everything is back in the pool
    st = s.plan()
    assert [(r.id, t) for r, t in st.entries] == [(0, [12])]
    assert [r.id for r in s.commit(st, [13])] == [0] and a.output == [11, 12, 13]
    assert s.idle() and pool.committed == 0 and pool.uncommitted() == 64


def test_lifetime_page_accounting_is_exact():
    s, pool = make()
    a = s.submit(list(range(30)), 3)
    assert s.lifetime_pages(a) == 2  # 30 + 3 - 1 = 32 tokens are ever written
    st = s.plan()
    assert len(a.pages) == 2 and a.committed == 0 and pool.committed == 0
    s.commit(st, [1])


def test_first_chunk_rule_and_fcfs():
    s, _ = make(budget=24, min_first=8)
    a = s.submit(list(range(20)), 2)
    b = s.submit(list(range(30)), 2)
    c = s.submit(list(range(3)), 2)
    st = s.plan()
    # A takes 20 of 24; B's first chunk would be 4 < min(30, 8): not admitted, and C must not overtake B
    assert [(r.id, len(t)) for r, t in st.entries] == [(0, 20)]
    s.commit(st, [5])
    st = s.plan()  # A decodes (1), B gets the remaining 23
    assert [(r.id, len(t)) for r, t in st.entries] == [(0, 1), (1, 23)] and st.num_decoding == 1
    s.commit(st, [6, 0])
    st = s.plan()  # A finished (2 tokens); B continues with its last 7, C admitted with its whole prompt
    assert [(r.id, len(t)) for r, t in st.entries] == [(1, 7), (2, 3)]


def test_admission_waits_for_pages_and_for_a_batch_slot():
    s, pool = make(max_batch=2, pages=5, budget=40, min_first=8, max_len=64)
    a = s.submit(list(range(40)), 9)   # lifetime ceil(48 / 16) = 3 pages
    b = s.submit(list(range(20)), 20)  # lifetime ceil(39 / 16) = 3 pages: does not fit beside A
    st = s.plan()
    assert [(r.id, len(t)) for r, t in st.entries] == [(0, 40)] and pool.uncommitted() == 2 and not b.admitted
    s.commit(st, [1])
    for _ in range(8):
        st = s.plan()
        assert [r.id for r, _ in st.entries] == [0]
        s.commit(st, [1])
    assert a.t_finish is not None and pool.uncommitted() == 5
    st = s.plan()
    assert [(r.id, len(t)) for r, t in st.entries] == [(1, 20)] and b.admitted


def test_stop_token_and_row_end_finish_a_request():
    s, pool = make(stop=99, max_len=20, budget=24)
    a = s.submit(list(range(10)), 10)
    st = s.plan()
    s.commit(st, [5])
    st = s.plan()
    assert [r.id for r in s.commit(st, [99])] == [0] and a.output == [5, 99]
    b = s.submit(list(range(15)), 5)  # 15 + 5 = max_len: the row fills up first
    st = s.plan()
    s.commit(st, [1])
    outs = 1
    while not s.idle():
        st = s.plan()
        s.commit(st, [1])
        outs += 1
    assert len(b.output) == outs and b.cached_len + 1 >= 20 and pool.committed == 0


def test_budget_must_cover_batch_plus_first_chunk():
    with pytest.raises(AssertionError):
        make(max_batch=20, budget=24, min_first=8)


def test_a_request_larger_than_the_pool_is_refused_at_submission():
    """It could never be admitted: planning would stop at it for ever and every later request would starve."""
    s, pool = make(pages=4, max_len=512, budget=64)
    with pytest.raises(ValueError):
        s.submit(list(range(100)), 8)  # 107 cached tokens = 7 pages
    ok = s.submit(list(range(40)), 8)  # 47 tokens = 3 pages
    assert s.plan() is not None and ok.admitted
