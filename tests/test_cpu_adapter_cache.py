"""Adapter cache policies against the reference's own counts (tests/golden/cache_counts.json) and the CPU oracle."""
import json
import os

import numpy as np
import pytest

from katz_b200 import adapter_cache
from katz_b200._lib import KatzError
from oracle import cache_oracle


@pytest.fixture(scope="module")
def golden(golden_dir):
    with open(os.path.join(golden_dir, "cache_counts.json")) as fr:
        return json.load(fr)


def test_oracle_counts_equal_the_reference(golden):
    for policy in ("LRU", "LFU"):
        for field in ("loras", "controlnets"):
            for size, n in golden["loads"][policy][field].items():
                assert cache_oracle.trace_loads(golden["trace"], field, int(size), policy)[0] == n, (policy, field, size)


def test_cache_counts_equal_the_reference(golden):
    for policy in ("LRU", "LFU"):
        for field in ("loras", "controlnets"):
            for size, n in golden["loads"][policy][field].items():
                total, per_req = adapter_cache.trace_loads(golden["trace"], field, int(size), policy)
                assert total == n, (policy, field, size)
                assert per_req == n / len(golden["trace"])


def test_synthetic_trace_is_seeded_and_matches_the_fixture(golden):
    again = adapter_cache.zipf_trace(600, n_loras=24, n_controlnets=6, alpha=1.1, instances=3, seed=7, scene_id="A")
    assert again == golden["trace"]
    assert set(again[0]) == {"timestamp", "ip", "scene_id", "base_model_id", "controlnets", "loras"}


@pytest.mark.parametrize("policy", ["LRU", "LFU"])
def test_cache_against_the_oracle_on_random_sequences(policy):
    rng = np.random.default_rng(3)
    fn = {"LRU": cache_oracle.lru_loads, "LFU": cache_oracle.lfu_loads}[policy]
    for trial in range(40):
        n_ids = int(rng.integers(1, 12))
        ids = [int(v) for v in rng.integers(0, n_ids, size=int(rng.integers(0, 200)))]
        size = int(rng.integers(1, 8))
        assert adapter_cache.replay_loads(ids, size, policy) == fn(ids, size), (trial, size)
    assert adapter_cache.replay_loads([], 3, policy) == 0                      # empty trace
    assert adapter_cache.replay_loads([5] * 50, 1, policy) == 1                # one adapter, smallest cache
    assert adapter_cache.replay_loads(list(range(50)), 50, policy) == 50       # cache as large as the pool: cold misses only


def test_loader_eviction_callback_bytes_and_pinning():
    loaded, evicted = [], []
    c = adapter_cache.AdapterCache(3, "LRU", loader=lambda k: loaded.append(k) or ("adapter", k),
                                   on_evict=lambda k, e: evicted.append((k, e)), capacity_bytes=250, size_of=lambda e: 100)
    assert c.get("a") == (("adapter", "a"), False) and c.get("a")[1] is True
    c.get("b")
    assert c.resident_bytes == 200 and len(c) == 2
    c.get("c")                               # a third entry would make 300 bytes: the least recent one ("a") goes first
    assert evicted == [("a", ("adapter", "a"))] and c.keys() == ["b", "c"]
    c.pinned = {"b"}
    c.get("d")                               # "b" is merged right now and stays; "c" goes
    assert [k for k, _ in evicted] == ["a", "c"] and "b" in c and "d" in c
    s = c.stats()
    assert s["loads"] == 4 and s["hits"] == 1 and s["evictions"] == 2 and s["bytes_loaded"] == 400 and loaded == ["a", "b", "c", "d"]
    c.pinned = {"b", "d"}
    with pytest.raises(KatzError):
        c.get("e")
    with pytest.raises(KatzError):
        adapter_cache.AdapterCache(0)
    with pytest.raises(KatzError):
        adapter_cache.AdapterCache(2, "FIFO")


def test_lfu_keeps_the_popular_adapter():
    c = adapter_cache.AdapterCache(2, "LFU")
    for k in ("hot", "hot", "hot", "x", "y", "z"):
        c.get(k)
    assert "hot" in c and c.keys() == ["hot", "z"]
    lru = adapter_cache.AdapterCache(2, "LRU")
    for k in ("hot", "hot", "hot", "x", "y", "z"):
        lru.get(k)
    assert "hot" not in lru
