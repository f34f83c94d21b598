"""Radix prefix cache: media-salted block keys, lifetime of block references, snapshot budget, eviction order
(the reference keeps these as tests/test_radix_mm.py and tests/test_radix_lifetime.py)."""
from types import SimpleNamespace

from coffin_b200.cache.paged_cache import BlockPool
from coffin_b200.cache.radix_cache import RadixCache, media_ids_for, media_signature

BS = 4
PAD = 99


def _cache(n_blocks=32, snaps=8):
    pool = BlockPool(n_blocks, BS)
    return pool, RadixCache(pool, max_snapshots=snaps)


def _blocks(pool, n):
    return [pool.alloc() for _ in range(n)]


def _publish(pool, cache, tokens, mm=None, states=None):
    """Insert a computed sequence the way a finished request does, then drop the request's own references."""
    n = len(tokens) // BS
    blocks = _blocks(pool, n)
    cache.insert(tokens, blocks, states=states or {n * BS: f"S{n}"}, mm=mm)
    for b in blocks:
        pool.decref(b)
    return blocks


def _mm(spans, digests):
    return SimpleNamespace(spans=spans, digests=digests)


def test_media_salts_follow_the_images_that_overlap_a_block():
    assert media_ids_for(12, BS, None) == ["", "", ""]
    ids = media_ids_for(12, BS, _mm([(5, 7)], ["A"]))
    assert ids == ["", media_signature(["A"]), ""]
    ids = media_ids_for(12, BS, _mm([(3, 9)], ["A"]))                  # a span crossing two boundaries salts three blocks
    assert ids == [media_signature(["A"])] * 3
    two = media_ids_for(8, BS, _mm([(0, 2), (2, 4)], ["A", "B"]))
    swapped = media_ids_for(8, BS, _mm([(0, 2), (2, 4)], ["B", "A"]))
    assert two[0] != swapped[0] and two[1] == swapped[1] == ""          # order inside a block matters
    assert media_signature(["A"]) == media_signature(["A"]) != media_signature(["B"])


def test_same_tokens_with_another_image_match_nothing_and_with_the_same_image_hit():
    pool, cache = _cache()
    toks = [1, 2, 3, 4, PAD, PAD, PAD, PAD, 5, 6, 7, 8, 9]
    _publish(pool, cache, toks, mm=_mm([(4, 8)], ["A"]), states={4: "s1", 8: "s2", 12: "s3"})
    blocks, n, st = cache.match_prefix(toks, mm=_mm([(4, 8)], ["A"]))
    assert n == 12 and st == "s3"
    for b in blocks:
        pool.decref(b)
    # another picture behind the same placeholder tokens: only the text block before it is shared
    blocks, n, st = cache.match_prefix(toks, mm=_mm([(4, 8)], ["B"]))
    assert n == 4 and st == "s1"
    for b in blocks:
        pool.decref(b)
    # a text request that happens to contain the placeholder ids never matches a salted block
    blocks, n, st = cache.match_prefix(toks, mm=None)
    assert n == 4
    for b in blocks:
        pool.decref(b)
    pool.check()


def test_text_branch_is_shared_up_to_the_image_block():
    pool, cache = _cache()
    text = [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13]
    _publish(pool, cache, text, states={4: "a", 8: "b", 12: "c"})
    img = text[:8] + [PAD] * 4 + [20]
    blocks, n, st = cache.match_prefix(img, mm=_mm([(8, 12)], ["A"]))
    assert n == 8 and st == "b"
    for b in blocks:
        pool.decref(b)
    nodes = cache.n_nodes
    _publish(pool, cache, img, mm=_mm([(8, 12)], ["A"]))
    assert cache.n_nodes == nodes + 1                                     # only the image block is new
    pool.check()


def test_a_match_always_leaves_one_token_to_compute():
    pool, cache = _cache()
    toks = list(range(1, 9))
    _publish(pool, cache, toks, states={4: "a", 8: "b"})
    blocks, n, st = cache.match_prefix(toks)                              # the whole prompt is cached: reuse all but the last block
    assert n == 4 and st == "a"
    for b in blocks:
        pool.decref(b)
    blocks, n, st = cache.match_prefix(toks + [9])
    assert n == 8 and st == "b"
    for b in blocks:
        pool.decref(b)


def test_state_fallback_does_not_pin_the_blocks_it_gave_up():
    pool, cache = _cache()
    toks = list(range(1, 14))
    held = _publish(pool, cache, toks, states={4: "only"})               # deeper nodes carry no snapshot
    blocks, n, st = cache.match_prefix(toks, require_states=True)
    assert n == 4 and st == "only" and blocks == held[:1]
    assert [pool.ref[b] for b in held] == [2, 1, 1]                       # the discarded tail got no reference
    pool.decref(blocks[0])
    blocks, n, st = cache.match_prefix(toks, require_states=False)
    assert n == 12 and st is None
    for b in blocks:
        pool.decref(b)
    pool.check()


def test_last_reader_release_allows_eviction_leaves_first_oldest_first():
    pool, cache = _cache(n_blocks=8)
    a = _publish(pool, cache, [1, 2, 3, 4, 5, 6, 7, 8, 0])
    b = _publish(pool, cache, [1, 2, 3, 4, 9, 9, 9, 9, 0])               # shares the first block with a
    assert cache.n_nodes == 3 and pool.used_blocks == 3                  # b's duplicate of the shared block went back to the pool
    reader, n, _ = cache.match_prefix([1, 2, 3, 4, 5, 6, 7, 8, 0], require_states=False)
    assert n == 8 and cache.evictable() == 1                              # only b's leaf is free to go
    assert cache.evict(5) == 1 and cache.n_nodes == 2
    for blk in reader:
        pool.decref(blk)
    assert cache.evictable() == 2
    assert cache.evict(1) == 1                                            # the leaf before its parent
    assert list(cache.root.children.values())[0].children == {}
    assert cache.evict(4) == 1 and cache.n_nodes == 0
    pool.check()
    assert pool.used_blocks == 0


def test_snapshot_budget_drops_the_least_recently_used_and_reserve_evicts():
    pool, cache = _cache(n_blocks=16, snaps=2)
    for i in range(4):
        _publish(pool, cache, [10 * i + j for j in range(1, 5)] + [0], states={4: f"s{i}"})
    assert cache.stats()["snapshots"] == 2
    hit = [cache.match_prefix([10 * i + j for j in range(1, 5)] + [0])[1] for i in range(4)]
    assert hit == [0, 0, 4, 4]                                            # the two oldest lost their snapshot
    # the matches above hold references; release them and ask for more free blocks than there are
    for n in cache._nodes():
        while pool.ref[n.block] > 1:
            pool.decref(n.block)
    free_before = pool.free_blocks
    assert cache.reserve(free_before + 3) and pool.free_blocks >= free_before + 3
    assert cache.stats()["nodes"] == 1
    cache.clear()
    pool.check()
