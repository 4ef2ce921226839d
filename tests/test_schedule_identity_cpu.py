"""The identity the one-block layer schedule rests on, checked on the CPU against the checker.

The CUDA kernel `layer_schedule_rank_kernel` (nerve_b200/csrc/schedule.cu) builds the compact list of
moe_route_compact, the owned count of moe_route_count and the expert-grouped route lists of both expert
stages from ONE stable ranking of the routes: rank of a route among the listed routes of its expert, found
per warp of 32 routes and summed column-wise over a [warp][bucket] table.  `single_pass_schedule` below is
that algorithm in plain Python, step for step; the expectation is built from the checker's restatement of
the shaders (runtime-rs/shaders/moe_route_compact_batch1.comp.template:26-105,
moe_route_count_batch1.comp.template:21-58) followed by the grouping's definition: the compact entries a
stage visits, stably sorted by expert, without those whose expert is out of range or not resident.
"""
import numpy as np
import pytest

from oracle import moe_oracle as mo

UNBOUND = 0xFFFFFFFF
STATUS_OUT_OF_RANGE, STATUS_NOT_RESIDENT = "route out of range", "expert not resident"


def _local(slots, params, e):
    if slots is None:
        return True
    index = e * params
    return index < slots.size and slots[index] != UNBOUND


def single_pass_schedule(routes, T, K, E, start, count, slots, resident):
    """Plain-Python mirror of the kernel. Returns (compact list as {position: route}, control[2], grouped[2],
    offsets[2], position[2], status set)."""
    n = T * K
    partitioned = count != 0
    B = E + 1  # bucket E: out-of-range ids
    warps = (n + 31) // 32
    table = np.zeros((warps, B + 1), dtype=np.int64)  # last column: owned routes per warp
    bucket = np.full(n, -1, dtype=np.int64)
    before = np.zeros(n, dtype=np.int64)
    owned_before = np.zeros(n, dtype=np.int64)
    totals = [0, 0]
    for w in range(warps):
        seen, owned_seen = {}, 0
        for i in range(32 * w, min(n, 32 * w + 32)):
            e = int(routes[i]) & 0xFFFF
            listed = True
            if partitioned:
                in_range = start <= e < start + count
                listed = in_range and _local(slots[0], 4, e)
                if in_range and _local(slots[1], 2, e):
                    totals[1] += 1
                if listed:
                    owned_before[i] = owned_seen
                    owned_seen += 1
            if listed:
                b = min(e, E)
                bucket[i] = b
                before[i] = seen.get(b, 0)
                seen[b] = before[i] + 1
        for b, c in seen.items():
            table[w, b] = c
        table[w, B] = owned_seen
        totals[0] += owned_seen
    listed_total = totals[0] if partitioned else n
    down_total = totals[1] if partitioned else n
    hist = table.sum(axis=0)
    start_of = np.cumsum(table, axis=0) - table  # exclusive running sums down each column
    status = set()
    if down_total > listed_total:
        status.add(STATUS_OUT_OF_RANGE)
    at = np.full(n, -1, dtype=np.int64)
    rank = np.zeros(n, dtype=np.int64)
    base_all = np.cumsum(hist[:B]) - hist[:B]
    for i in range(n):
        if bucket[i] < 0:
            continue
        w = i // 32
        rank[i] = start_of[w, bucket[i]] + before[i]
        at[i] = start_of[w, B] + owned_before[i] if partitioned else base_all[bucket[i]] + rank[i]
    compact = {int(at[i]): i for i in range(n) if bucket[i] >= 0}
    hist_stage = [hist[:B].copy(), hist[:B].copy()]
    if down_total < listed_total:
        hist_stage[1][:] = 0
        for i in range(n):
            if bucket[i] >= 0 and at[i] < down_total:
                hist_stage[1][bucket[i]] += 1
    grouped, offsets, position = [], [], []
    for stage in range(2):
        kept = np.array([b < E and bool(resident[stage][b]) for b in range(B)])
        counts = np.where(kept, hist_stage[stage], 0)
        base = np.concatenate([np.cumsum(counts) - counts, [counts.sum()]])
        g = np.full(int(counts.sum()), UNBOUND, dtype=np.int64)
        p = np.full(n, UNBOUND, dtype=np.int64)
        for i in range(n):
            if bucket[i] < 0 or (stage == 1 and at[i] >= down_total):
                continue
            if kept[bucket[i]]:
                p[i] = base[bucket[i]] + rank[i]
                g[p[i]] = i
            else:
                status.add(STATUS_OUT_OF_RANGE if bucket[i] == E else STATUS_NOT_RESIDENT)
        grouped.append(g)
        offsets.append(base[: E + 1])
        position.append(p)
    visited = [listed_total, down_total]
    control = [[T, start, count, visited[s], (visited[s] if partitioned else K), T if not partitioned else 1, 1]
               for s in range(2)]
    return compact, control, grouped, offsets, position, status


def by_definition(routes, T, K, E, start, count, slots, resident, I=4):
    """The checker's compact list and counts, then the grouping as defined."""
    n = T * K
    data = K * (I // 2)
    frames = np.full((T, data + K), UNBOUND, dtype=np.uint32)  # schedule words never written stay out of range
    control = [np.array([T, start, count, 0, 0, 0, 0], dtype=np.uint32) for _ in range(2)]
    mo.route_compact(routes, frames, control[0], I, K, 1, slots=slots[0] if count else None, params_per_resource=4)
    mo.route_count(routes, control[1], K, 1, slots=slots[1] if count else None, params_per_resource=2)
    listed = int(control[0][3])
    compact = {c: int(frames[c // K, data + c % K]) for c in range(listed)}
    status = set()
    grouped, offsets, position = [], [], []
    for stage in range(2):
        visited = min(int(control[stage][3]), n)
        per_expert = [[] for _ in range(E)]
        p = np.full(n, UNBOUND, dtype=np.int64)
        for c in range(visited):
            ri = int(frames[c // K, data + c % K])
            if ri >= n:
                status.add(STATUS_OUT_OF_RANGE)
                continue
            e = int(routes[ri]) & 0xFFFF
            if e >= E:
                status.add(STATUS_OUT_OF_RANGE)
            elif not resident[stage][e]:
                status.add(STATUS_NOT_RESIDENT)
            else:
                per_expert[e].append(ri)
        flat = [ri for rows in per_expert for ri in rows]
        for place, ri in enumerate(flat):
            p[ri] = place
        counts = np.array([len(rows) for rows in per_expert], dtype=np.int64)
        grouped.append(np.array(flat, dtype=np.int64))
        offsets.append(np.concatenate([np.cumsum(counts) - counts, [counts.sum()]]))
        position.append(p)
    return compact, [c.tolist() for c in control], grouped, offsets, position, status


def _case(seed, T, K, E, invalid=0.0):
    rng = np.random.default_rng(seed)
    ids = np.stack([np.sort(rng.choice(E, size=K, replace=False)) for _ in range(T)]).astype(np.uint32)
    weights = rng.integers(0, 1 << 16, size=(T, K), dtype=np.uint32)
    routes = ((weights << 16) | ids).reshape(-1)
    if invalid:
        bad = rng.random(T * K) < invalid
        # one out-of-range id: the kernels rank ids past the resource count after all valid ids in source order,
        # the shader by id; with a single such id the two orders coincide
        routes[bad] = (routes[bad] & 0xFFFF0000) | np.uint32(E + 5)
    return rng, routes


def _compare(got, want):
    names = ("compact list", "control words", "grouped routes", "expert offsets", "positions", "status")
    for name, a, b in zip(names, got, want):
        if name in ("grouped routes", "expert offsets", "positions"):
            for stage in range(2):
                np.testing.assert_array_equal(a[stage], b[stage], err_msg=f"{name}, stage {stage}")
        else:
            assert a == b, name


@pytest.mark.parametrize("T,K,E", [(1, 4, 32), (64, 4, 32), (37, 9, 257), (300, 2, 8)])
def test_unpartitioned_schedule_is_one_stable_sort(T, K, E):
    rng, routes = _case(T * 131 + E, T, K, E, invalid=0.05)
    resident = [rng.random(E) < 0.9, rng.random(E) < 0.9]
    args = (routes, T, K, E, 0, 0, [None, None], resident)
    _compare(single_pass_schedule(*args), by_definition(*args))


@pytest.mark.parametrize("T,K,E,start,count", [(64, 4, 32, 8, 8), (50, 1, 16, 0, 16), (90, 3, 40, 35, 5)])
@pytest.mark.parametrize("tables", ["agree", "down owns fewer", "down owns more"])
def test_partitioned_schedule_lists_owned_routes_in_source_order(T, K, E, start, count, tables):
    rng, routes = _case(T * 17 + E + len(tables), T, K, E)
    if K == 1:  # the owner's side of an exchange: unused slots carry an all-ones route word
        routes[rng.random(T) < 0.3] = UNBOUND
    local = rng.random(E) < 0.8
    local_down = local.copy()
    if tables == "down owns fewer":
        local_down &= rng.random(E) < 0.6
    if tables == "down owns more":
        local_down |= rng.random(E) < 0.5
    slots = [np.where(np.repeat(local, 4), 7, UNBOUND).astype(np.uint32),
             np.where(np.repeat(local_down, 2), 7, UNBOUND).astype(np.uint32)]
    resident = [local & (rng.random(E) < 0.95), local_down & (rng.random(E) < 0.95)]
    args = (routes, T, K, E, start, count, slots, resident)
    _compare(single_pass_schedule(*args), by_definition(*args))
