"""KV-cache bookkeeping: page allocator, prefix index, contiguous and paged pools, task manager, decode metadata."""

import threading

import pytest
import torch

from astrai_b200.inference.cache import Allocator, PagePool, RadixCache, TaskCacheManager
from astrai_b200.inference.cache.pool import page_hash
from astrai_b200.inference.workspace import InferenceWorkspace


def _pool(page_size=4, n_tokens=64, batch=4, seq=32):
    return PagePool(2, 1, 8, max_batch_size=batch, max_seq_len=seq, device="cpu", dtype=torch.float32, page_size=page_size,
                    n_tokens=n_tokens)


def _ws(batch=4, seq=32):
    return InferenceWorkspace(batch, seq, 2, 8, "cpu", torch.float32, n_kv_heads=1, max_prefill_tokens=batch * seq)


# ------------------------------------------------------------------------------------------------ allocator
def test_allocator_hands_out_lowest_index_first_and_reports_exhaustion():
    a = Allocator(4)
    assert [a.alloc() for _ in range(4)] == [0, 1, 2, 3] and a.alloc() == -1 and a.available() == 0
    a.free(2)
    a.free(0)
    assert a.available() == 2 and a.alloc() == 0 and a.alloc() == 2


def test_allocator_refcounts_shared_pages():
    a = Allocator(2)
    p = a.alloc()
    a.inc_ref(p)
    a.inc_ref(p)
    assert a.ref_count(p) == 3
    a.free(p)
    a.free(p)
    assert a.ref_count(p) == 1 and a.available() == 1
    a.free(p)
    assert a.ref_count(p) == 0 and a.available() == 2


def test_retained_pages_are_recycled_oldest_first_and_reported():
    a = Allocator(3)
    gone = []
    a.on_evict = gone.append
    pages = [a.alloc() for _ in range(3)]
    for p in (pages[1], pages[0], pages[2]):
        a.free(p, keep_cached=True)
    assert a.available() == 3
    assert [a.alloc() for _ in range(3)] == [pages[1], pages[0], pages[2]] and gone == [pages[1], pages[0], pages[2]]


def test_touch_refreshes_a_retained_page():
    a = Allocator(2)
    x, y = a.alloc(), a.alloc()
    a.free(x, keep_cached=True)
    a.free(y, keep_cached=True)
    a.touch(x)  # x is now the most recently used
    assert a.alloc() == y


def test_cache_hit_takes_a_page_off_the_retained_ring():
    a = Allocator(2)
    x, y = a.alloc(), a.alloc()
    a.free(x, keep_cached=True)
    a.inc_ref(x)  # prefix hit
    assert a.available() == 0 and a.alloc() == -1
    a.free(x, keep_cached=True)
    assert a.alloc() == x


def test_unheld_pages_are_preferred_over_retained_ones():
    a = Allocator(3)
    evicted = []
    a.on_evict = evicted.append
    x, y, _ = a.alloc(), a.alloc(), a.alloc()
    a.free(x, keep_cached=True)
    a.free(y)
    assert a.alloc() == y and evicted == []


def test_allocator_is_thread_safe():
    a = Allocator(64)
    got = []
    lock = threading.Lock()

    def worker():
        mine = [a.alloc() for _ in range(16)]
        with lock:
            got.extend(mine)

    threads = [threading.Thread(target=worker) for _ in range(4)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert sorted(got) == list(range(64))


# ------------------------------------------------------------------------------------------------ prefix index
def test_only_full_pages_are_indexed():
    r = RadixCache(4)
    ids = list(range(10))
    for i in range(3):
        r.record(100 + i, ids, i)
    assert r.lookup(ids) == [100, 101] and not r.has_page(102)


def test_lookup_needs_exact_tokens_page_by_page():
    r = RadixCache(2)
    r.record(1, [5, 6, 7, 8], 0)
    r.record(2, [5, 6, 7, 8], 1)
    assert r.lookup([5, 6, 7, 8]) == [1, 2] and r.lookup([5, 6, 7, 9]) == [1] and r.lookup([5, 7, 7, 8]) == []
    assert r.lookup([5]) == [] and r.lookup([]) == []


def test_branches_share_their_common_prefix():
    r = RadixCache(2)
    r.record(1, [1, 2, 3, 4], 0)
    r.record(2, [1, 2, 3, 4], 1)
    r.record(3, [1, 2, 9, 9], 1)
    assert r.lookup([1, 2, 3, 4]) == [1, 2] and r.lookup([1, 2, 9, 9, 0]) == [1, 3]


def test_a_gap_in_the_chain_stops_the_lookup():
    r = RadixCache(2)
    r.record(7, [1, 2, 3, 4, 5, 6], 2)  # only the third page of the sequence is known
    assert r.lookup([1, 2, 3, 4, 5, 6]) == [] and r.has_page(7)


def test_eviction_cuts_everything_behind_the_page():
    r = RadixCache(2)
    ids = [1, 2, 3, 4, 5, 6]
    for i in range(3):
        r.record(10 + i, ids, i)
    r.evict(11)
    assert r.lookup(ids) == [10] and not r.has_page(11) and r.has_page(12)
    r.record(21, ids, 1)  # re-materialised by a later request
    assert r.lookup(ids) == [10, 21]


def test_re_recording_a_page_keeps_what_is_chained_behind_it():
    r = RadixCache(2)
    ids = [1, 2, 3, 4]
    r.record(10, ids, 0)
    r.record(11, ids, 1)
    r.record(10, ids, 0)  # a finishing request records its pages again
    assert r.lookup(ids) == [10, 11]


def test_a_recycled_page_leaves_its_old_place():
    r = RadixCache(2)
    r.record(5, [1, 2], 0)
    r.record(5, [3, 4], 0)  # the allocator reused page 5 for other tokens
    assert r.lookup([1, 2]) == [] and r.lookup([3, 4]) == [5]


def test_two_pages_for_the_same_tokens_last_writer_wins():
    r = RadixCache(2)
    r.record(5, [1, 2], 0)
    r.record(6, [1, 2], 0)
    assert r.lookup([1, 2]) == [6] and not r.has_page(5)


def test_page_hash_chains_over_pages():
    ids = list(range(8))
    h0 = page_hash(ids, 0, 4)
    assert page_hash(ids, 1, 4, h0) != page_hash(ids, 1, 4) and page_hash(ids, 0, 4) == h0


# ------------------------------------------------------------------------------------------------ pools + task manager
def test_contiguous_pool_rows_are_fixed_ranges():
    pool = PagePool(1, 1, 4, max_batch_size=2, max_seq_len=8, device="cpu", dtype=torch.float32)
    assert pool.contiguous and pool.allocator is None and pool.prefix is None
    assert pool.req_pool.host[1].tolist() == list(range(8, 16))


def test_paged_pool_without_prefix_index_at_page_size_one():
    pool = _pool(page_size=1, n_tokens=16)
    assert not pool.contiguous and pool.prefix is None and pool.allocator.n_pages == 16


def test_pool_for_model_defaults_to_paged_with_radix():
    from helpers import tiny_config

    pool = PagePool.for_model(tiny_config(), 2, 40, "cpu", torch.float32)
    assert not pool.contiguous and pool.page_size == 16 and pool.prefix is not None
    assert pool.n_tokens == 2 * 48  # rows rounded up to whole pages
    flat = PagePool.for_model(tiny_config(), 2, 40, "cpu", torch.float32, paged=False)
    assert flat.contiguous


def test_slots_follow_the_pages_in_order():
    pool = _pool(page_size=4, n_tokens=32)
    mgr = TaskCacheManager(pool)
    assert mgr.task_alloc("a", list(range(10)))
    st = mgr.state("a")
    assert len(st.pages) == 3 and st.length == 10
    row = pool.req_pool.host[st.req_idx, :12].tolist()
    assert row == [p * 4 + o for p in st.pages for o in range(4)]


def test_alloc_fails_cleanly_when_pages_run_out():
    pool = _pool(page_size=4, n_tokens=16)
    mgr = TaskCacheManager(pool)
    assert mgr.task_alloc("a", list(range(12)))
    assert not mgr.task_alloc("b", list(range(100, 112)))  # one page left, three needed
    assert mgr.state("b") is None and pool.allocator.available() == 1
    assert mgr.task_alloc("c", [1, 2, 3])


def test_rows_run_out_before_pages():
    pool = _pool(page_size=4, n_tokens=64, batch=2)
    mgr = TaskCacheManager(pool)
    assert mgr.task_alloc("a", [1]) and mgr.task_alloc("b", [2]) and not mgr.task_alloc("c", [3])
    mgr.task_free("a")
    assert mgr.task_alloc("c", [3])


def test_extend_allocates_a_page_only_at_page_boundaries():
    pool = _pool(page_size=4, n_tokens=32)
    mgr = TaskCacheManager(pool)
    mgr.task_alloc("a", list(range(6)))
    before = pool.allocator.available()
    assert mgr.task_extend("a", 6) and mgr.task_extend("a", 7) and pool.allocator.available() == before
    assert mgr.task_extend("a", 8) and pool.allocator.available() == before - 1
    assert mgr.state("a").length == 9
    assert not mgr.task_extend("a", 32)      # beyond max_seq_len
    assert not mgr.task_extend("nope", 0)


def test_prefix_hit_shares_pages_and_counts_cached_tokens():
    pool = _pool(page_size=4, n_tokens=64)
    mgr = TaskCacheManager(pool)
    prompt = list(range(100, 113))  # 13 tokens: three full pages
    mgr.task_alloc("a", prompt)
    mgr.task_record_hashes("a", prompt)
    assert mgr.task_alloc("b", prompt[:9] + [7, 7, 7])
    a, b = mgr.state("a"), mgr.state("b")
    assert mgr.task_cached("b") == 8 and b.pages[:2] == a.pages[:2] and b.pages[2] != a.pages[2]
    assert pool.allocator.ref_count(a.pages[0]) == 2
    mgr.task_free("a")
    assert pool.allocator.ref_count(b.pages[0]) == 1  # still held by b


def test_freed_indexed_pages_stay_reusable_until_evicted():
    pool = _pool(page_size=4, n_tokens=16)
    mgr = TaskCacheManager(pool)
    prompt = list(range(8))
    mgr.task_alloc("a", prompt)
    mgr.task_record_hashes("a", prompt)
    mgr.task_free("a")
    assert pool.allocator.available() == 4 and pool.prefix.lookup(prompt) != []
    mgr.task_alloc("b", prompt + [1])
    assert mgr.task_cached("b") == 8
    mgr.task_free("b")
    assert mgr.task_alloc("big", list(range(50, 66)))  # needs all four pages: the cached ones are evicted
    assert pool.prefix.lookup(prompt) == []


def test_cacheable_ids_exclude_the_last_sampled_token():
    assert TaskCacheManager.task_cacheable_ids("t", [1, 2, 3], [4, 5, 6]) == [1, 2, 3, 4, 5]
    assert TaskCacheManager.task_cacheable_ids("t", [1, 2], []) == [1, 2]


def test_prefill_bind_describes_ragged_queries():
    pool = _pool(page_size=4, n_tokens=64)
    mgr, ws = TaskCacheManager(pool), _ws()
    mgr.task_alloc("a", list(range(9)))
    mgr.task_alloc("b", list(range(20, 25)))
    kv = mgr.bind(["a", "b"], ws, start_positions=[4, 0])
    assert kv.q_lens == [5, 5] and kv.kv_lens == [9, 5] and kv.qo_indptr.tolist() == [0, 5, 10]
    assert kv.kv_indptr.tolist() == [0, 9, 14] and kv.out_cache_loc.numel() == 10
    with pytest.raises(ValueError):
        mgr.bind(["a"], ws, start_pos=9)


def test_chunked_prefill_bind_stops_at_the_chunk_end():
    pool = _pool(page_size=4, n_tokens=64)
    mgr, ws = TaskCacheManager(pool), _ws()
    mgr.task_alloc("a", list(range(20)))
    kv = mgr.bind(["a"], ws, start_positions=[8], end_positions=[16])
    assert kv.q_lens == [8] and kv.kv_lens == [16]


def test_steady_decode_updates_metadata_in_place():
    pool = _pool(page_size=4, n_tokens=64)
    mgr, ws = TaskCacheManager(pool), _ws()
    mgr.task_alloc("a", list(range(5)))
    mgr.task_alloc("b", list(range(3)))
    kv = mgr.bind(["a", "b"], ws)
    assert not mgr.bind_was_steady and kv.seq_lens.tolist() == [5, 3] and kv.kv_indptr.tolist() == [0, 5, 8]
    lens_ptr = kv.seq_lens.data_ptr()
    for step in range(1, 4):
        mgr.task_extend("a", 4 + step)
        mgr.task_extend("b", 2 + step)
        kv = mgr.bind(["a", "b"], ws)
        assert mgr.bind_was_steady and kv.seq_lens.data_ptr() == lens_ptr  # same buffers: a captured graph stays valid
        assert kv.seq_lens.tolist() == [5 + step, 3 + step] and kv.kv_indptr.tolist() == [0, 5 + step, 8 + 2 * step]
    kv = mgr.bind(["b", "a"], ws)  # another order is another batch
    assert not mgr.bind_was_steady and kv.seq_lens.tolist() == [6, 8]


def test_decode_bind_after_alloc_or_free_is_rebuilt():
    pool = _pool(page_size=4, n_tokens=64)
    mgr, ws = TaskCacheManager(pool), _ws()
    mgr.task_alloc("a", [1, 2, 3])
    mgr.bind(["a"], ws)
    mgr.task_alloc("b", [4])
    mgr.task_extend("a", 3)
    mgr.bind(["a"], ws)
    assert not mgr.bind_was_steady  # the batch composition may have changed in between


def test_record_chain_equals_page_by_page_recording():
    """The one-walk form used by the serving loop leaves the index exactly as the page-by-page form does, over random
    sequences with shared prefixes, re-recordings, page reuse under other tokens and evictions in between."""
    import random

    from astrai_b200.inference.cache.strategy import RadixCache

    rng = random.Random(0)
    ps = 4
    a, b = RadixCache(ps), RadixCache(ps)
    prefixes = [[rng.randrange(50) for _ in range(ps * rng.randrange(1, 4))] for _ in range(3)]
    free = list(range(200))
    for step in range(300):
        seq = list(rng.choice(prefixes)) + [rng.randrange(50) for _ in range(rng.randrange(0, 5 * ps))]
        n_pages = -(-len(seq) // ps)
        pages = [free.pop(rng.randrange(len(free))) if (free and rng.random() < 0.7) else rng.randrange(200) for _ in range(n_pages)]
        start = rng.randrange(0, n_pages + 1)
        for i in range(start, min(len(seq) // ps, len(pages))):
            a.record(pages[i], seq, i)
        b.record_chain(pages, seq, start)
        if rng.random() < 0.3:
            victim = rng.randrange(200)
            a.evict(victim)
            b.evict(victim)
            free.append(victim)
        probe = list(rng.choice(prefixes)) + [rng.randrange(50) for _ in range(ps)]
        assert a.lookup(probe) == b.lookup(probe) and a.lookup(seq) == b.lookup(seq), step
        assert a._where == b._where and a._page_of == b._page_of and a._links == b._links, step
