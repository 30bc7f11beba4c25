"""CPU restatement of the reference's adapter-cache accounting. TEST INFRASTRUCTURE ONLY: imported by tests/, never
by the product.

The reference counts how often a serving instance has to load an adapter (a ControlNet or a LoRA) that its cache of
`cache_size` adapters does not hold, for two eviction policies (trace/adapter_loading_analysis.py:48-200):

  LRU  :60-74, :76-88    a hit moves the adapter to the most-recent end; a miss on a full cache drops the least
                         recently used one and counts one load.
  LFU  :113-148, :150-188 every cached adapter carries a use count; a miss on a full cache drops the adapter with the
                         smallest count and, among equals, the one that reached that count first; the newcomer starts
                         at one.

Requests are grouped per serving instance (`ip`) and ordered by timestamp (:37-45); requests that name no adapter of
the kind are skipped; every adapter a request names is looked up in the order given. The restatement below keeps plain
lists and scans them, so each step is visibly the definition; it is quadratic and meant for traces of a few thousand
requests.

Pinned by tests/golden/cache_counts.json, produced by tests/golden/make_golden.py from the reference's own loops.
"""


def lru_loads(ids, cache_size):
    """Number of loads for the id sequence `ids` through an LRU cache of `cache_size` entries."""
    order = []                      # least recently used first
    loads = 0
    for i in ids:
        if i in order:
            order.remove(i)
            order.append(i)
            continue
        if len(order) >= cache_size and order:
            order.pop(0)
        order.append(i)
        loads += 1
    return loads


def lfu_loads(ids, cache_size):
    """Number of loads through an LFU cache: evict the smallest use count, oldest arrival AT that count first."""
    count, since = {}, {}           # id -> use count; id -> the step at which it reached that count
    loads = 0
    for step, i in enumerate(ids):
        if i in count:
            count[i] += 1
            since[i] = step
            continue
        if len(count) >= cache_size:
            victim = min(count, key=lambda k: (count[k], since[k]))
            del count[victim], since[victim]
        count[i], since[i] = 1, step
        loads += 1
    return loads


def per_instance_sequences(requests, field):
    """requests: list of dicts with `ip`, `timestamp` and `field` (a list of ids or None) -> {ip: [ids in order]}."""
    by_ip = {}
    for r in requests:
        by_ip.setdefault(r["ip"], []).append(r)
    out = {}
    for ip, reqs in by_ip.items():
        reqs = sorted(reqs, key=lambda r: r["timestamp"])
        out[ip] = [a for r in reqs if r.get(field) for a in r[field]]
    return out


def trace_loads(requests, field, cache_size, policy):
    """Total loads over all serving instances, and loads per request (the reference's two figures, :92-93)."""
    fn = {"LRU": lru_loads, "LFU": lfu_loads}[policy]
    total = sum(fn(seq, cache_size) for seq in per_instance_sequences(requests, field).values())
    return total, total / max(len(requests), 1)
