"""Device-resident adapter cache and request-trace replay.

The reference studies how often a serving instance must load an adapter under an LRU or an LFU cache of 1..10 adapters
(trace/adapter_loading_analysis.py:48-200, on a production trace that is not distributed with it) and drives its
request loop from a fixed prompt list (sdxl_pipeline.py:141-148). Here the cache is the serving component itself: a
B200 holds 180 GB, one rank-64 SDXL adapter is 340 MB, so hundreds of adapters can stay resident and a switch between
cached adapters is one merge launch. A miss calls the loader (a file reader, the shared-memory client or a pinned
staging buffer: katz_b200.lora_files), registers the tensors with the merger once, and evicts by policy.

  AdapterCache(capacity, policy, loader, on_evict)   ids -> resident entries, hit/miss/eviction counters
  replay_loads(ids, capacity, policy)                the count of loads alone (what the reference's analysis prints)
  trace_loads(requests, field, capacity, policy)     the same over a request trace grouped per serving instance
  zipf_trace(...)                                    a seeded synthetic trace with the fields of the reference's dataset
  CachedLoraStream                                   configuration 5's request stream fed through the cache
"""
from collections import OrderedDict

import numpy as np

from ._lib import KatzError

POLICIES = ("LRU", "LFU")


class AdapterCache:
    """At most `capacity` adapters resident. get(id) returns the entry, loading it through `loader(id)` on a miss.

    LRU evicts the least recently used entry. LFU evicts the entry with the smallest use count and, among equals, the
    one that reached that count first; a newcomer starts at one (the reference's bookkeeping,
    adapter_loading_analysis.py:113-148). `capacity_bytes` bounds the resident bytes as well when `size_of` is given.
    Entries named in `pinned` (the adapter that is merged right now) are never evicted."""

    def __init__(self, capacity, policy="LRU", loader=None, on_evict=None, capacity_bytes=None, size_of=None):
        if policy not in POLICIES:
            raise KatzError("cache policy must be one of %s, not %r" % (POLICIES, policy))
        if capacity < 1:
            raise KatzError("cache capacity must be at least 1")
        self.capacity, self.policy, self.loader, self.on_evict = int(capacity), policy, loader, on_evict
        self.capacity_bytes, self.size_of = capacity_bytes, size_of
        self._entries = OrderedDict()            # LRU: least recent first
        self._count = {}                         # LFU: id -> use count
        self._buckets = {}                       # LFU: use count -> OrderedDict of ids in the order they reached it
        self._bytes = {}
        self.hits = self.loads = self.evictions = 0
        self.bytes_loaded = 0
        self.pinned = set()

    def __contains__(self, key):
        return key in self._entries

    def __len__(self):
        return len(self._entries)

    @property
    def resident_bytes(self):
        return sum(self._bytes.values())

    def keys(self):
        return list(self._entries)

    # ---- policy bookkeeping
    def _touch(self, key):
        if self.policy == "LRU":
            self._entries.move_to_end(key)
            return
        f = self._count[key]
        b = self._buckets[f]
        del b[key]
        if not b:
            del self._buckets[f]
        self._count[key] = f + 1
        self._buckets.setdefault(f + 1, OrderedDict())[key] = None

    def _victim(self):
        if self.policy == "LRU":
            for k in self._entries:
                if k not in self.pinned:
                    return k
            return None
        for f in sorted(self._buckets):
            for k in self._buckets[f]:
                if k not in self.pinned:
                    return k
        return None

    def _drop(self, key):
        entry = self._entries.pop(key)
        self._bytes.pop(key, None)
        if self.policy == "LFU":
            f = self._count.pop(key)
            b = self._buckets[f]
            del b[key]
            if not b:
                del self._buckets[f]
        self.evictions += 1
        if self.on_evict is not None:
            self.on_evict(key, entry)

    def _over(self, extra_bytes):
        if len(self._entries) >= self.capacity:
            return True
        return bool(self.capacity_bytes is not None and self._entries and self.resident_bytes + extra_bytes > self.capacity_bytes)

    # ---- the call
    def get(self, key):
        """The resident entry for `key`; (entry, hit)."""
        if key in self._entries:
            self.hits += 1
            self._touch(key)
            return self._entries[key], True
        entry = self.loader(key) if self.loader is not None else key
        nbytes = int(self.size_of(entry)) if self.size_of is not None else 0
        while self._over(nbytes):
            v = self._victim()
            if v is None:
                raise KatzError("adapter cache: every resident adapter is pinned, nothing can be evicted")
            self._drop(v)
        self._entries[key] = entry
        self._bytes[key] = nbytes
        if self.policy == "LFU":
            self._count[key] = 1
            self._buckets.setdefault(1, OrderedDict())[key] = None
        self.loads += 1
        self.bytes_loaded += nbytes
        return entry, False

    def stats(self):
        n = self.hits + self.loads
        return {"policy": self.policy, "capacity": self.capacity, "lookups": n, "hits": self.hits, "loads": self.loads,
                "evictions": self.evictions, "hit_rate": self.hits / n if n else 0.0, "bytes_loaded": self.bytes_loaded,
                "resident": len(self._entries), "resident_bytes": self.resident_bytes}


def replay_loads(ids, capacity, policy):
    """How many loads the id sequence costs through a cache of `capacity` adapters."""
    c = AdapterCache(capacity, policy)
    for i in ids:
        c.get(i)
    return c.loads


def instance_sequences(requests, field):
    """{serving instance: adapter ids in request order}: requests grouped by `ip`, ordered by `timestamp`; a request
    that names no adapter of the kind contributes nothing (adapter_loading_analysis.py:37-45,62-64)."""
    by_ip = OrderedDict()
    for r in requests:
        by_ip.setdefault(r["ip"], []).append(r)
    out = OrderedDict()
    for ip, reqs in by_ip.items():
        reqs = sorted(reqs, key=lambda r: r["timestamp"])
        out[ip] = [a for r in reqs if r.get(field) for a in r[field]]
    return out


def trace_loads(requests, field, capacity, policy):
    """(total loads over all serving instances, loads per request) for `field` in {"loras", "controlnets"}."""
    total = sum(replay_loads(seq, capacity, policy) for seq in instance_sequences(requests, field).values())
    return total, total / max(len(requests), 1)


def zipf_trace(n_requests, n_loras=64, n_controlnets=8, alpha=1.1, instances=2, max_loras=2, max_controlnets=3, seed=0,
               scene_id="A"):
    """A seeded synthetic request trace with the fields of the reference's dataset (trace/README.md: timestamp, ip,
    scene_id, base_model_id, controlnets, loras). Adapter popularity follows a Zipf law with exponent `alpha`; a request
    names 0..max adapters of each kind. It stands in for the production trace, which is not distributed."""
    rng = np.random.default_rng(seed)

    def zipf_ids(n_items, k):
        if k == 0:
            return []
        p = 1.0 / np.arange(1, n_items + 1) ** alpha
        return [int(v) for v in rng.choice(n_items, size=k, replace=False, p=p / p.sum())]

    reqs = []
    t = 0.0
    for _ in range(n_requests):
        t += float(rng.exponential(1.0))
        reqs.append({"timestamp": t, "ip": "instance-%d" % int(rng.integers(instances)), "scene_id": scene_id,
                     "base_model_id": 0,
                     "controlnets": zipf_ids(n_controlnets, int(rng.integers(0, max_controlnets + 1))),
                     "loras": zipf_ids(n_loras, int(rng.integers(0, max_loras + 1)))})
    return reqs


class CachedLoraStream:
    """Configuration 5's request stream with the adapters behind a cache: a request names adapter ids; a resident
    adapter costs one merge launch, a miss first calls `loader(id)` -> {key: (up, down)} on the device (for instance
    lora_files.to_device_async of a pinned staging buffer) and registers it with the merger.

    denoiser: pipeline.KatzDenoiser; merger: lora.LoraMerger over the denoiser's UNet."""

    def __init__(self, denoiser, merger, loader, capacity, policy="LRU", scale=1.0):
        self.denoiser, self.merger, self.scale = denoiser, merger, scale

        def load(key):
            return merger.register_adapter(loader(key))

        def nbytes(reg):
            return sum(u.numel() * u.element_size() + d.numel() * d.element_size() for u, d in reg.adapter.values())

        self.cache = AdapterCache(capacity, policy, loader=load, size_of=nbytes)
        self.current = None

    def run(self, requests, request_inputs, num_inference_steps=50, seed=0):
        """requests: list of tuples of adapter ids (empty = no adapter). Returns [(final latent, ms)] per request."""
        import torch
        results = []
        self.denoiser.schedule.set_timesteps(num_inference_steps)
        for i, ids in enumerate(requests):
            ids = tuple(ids)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if ids != self.current:
                self.cache.pinned = set(ids)
                regs = [self.cache.get(k)[0] for k in ids]
                if regs:
                    self.merger.merge(regs, [self.scale] * len(regs))
                else:
                    self.merger.restore()
                self.denoiser.unet.invalidate_caches()
                self.current = ids
            lat = self.denoiser.prepare_latents(seed=seed + i)
            lat = self.denoiser.denoise(lat, num_inference_steps=num_inference_steps, **request_inputs(i))
            e1.record()
            results.append((lat.clone(), e0, e1))
        torch.cuda.synchronize()
        self.denoiser.step.check()
        return [(lat, a.elapsed_time(b)) for lat, a, b in results]
