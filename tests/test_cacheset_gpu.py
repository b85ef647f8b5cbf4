"""The reference's cache-set fixtures on the GPU update kernel.

The reference tests its LFU replacement on single cache-set states - five literal ones and
randomised ones - and checks invariants, not bit patterns
(cpp/tests/wholegraph_tensor_ops/cacheset_tests.cu: states :509-720, Random() :81-131, checks
:169-331): the 32 most-counted rows of (cached rows) U (updated rows) end up cached, ties free;
a row that stays cached keeps its line and its modified bit; new lines are clean; the LFU words
hold count >> scale with the smallest scale that fits 14 bits; counters are exact; evicted modified
lines are written back and new lines loaded.

Here each state is written into one set of a cached embedding (tags, LFU words, cache lines, the
per-row counters), one cached gather with adjust_cache = True runs over the update ids (every id
repeated by its increment), and the same invariants are checked on what the kernel left behind -
plus the data: every row reads back with its current value, whichever copy holds it.  This
library counts every row exactly, so the count the reference assigns to a cached row (its scaled
LFU estimate, or counter + increment when it is updated) is what the row's counter is set to.
The literal states come from tests/golden/cacheset_cases.json (made by
tests/golden/make_cacheset_golden.py from the reference's file)."""
import ctypes as C
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
VALID, MODIFIED, MASK14 = 1 << 14, 1 << 15, (1 << 14) - 1
with open(os.path.join(HERE, "golden", "cacheset_cases.json")) as _f:
    CASES = json.load(_f)


@pytest.fixture(scope="module")
def comm(gpu, wgb):
    c = wgb.create_communicator(wgb.UniqueId(), 0, 1)
    yield c
    wgb.destroy_communicator(c)


def random_case(base_scale, coverage, update_count, seed, inc_max):
    """SingleCacheSetTestParam::Random of the reference, restated with a seeded generator."""
    rng = np.random.default_rng(seed)
    lid_perm = rng.permutation(coverage)
    lids, valid, modified, lfu = [-1] * 32, [False] * 32, [False] * 32, [0] * 32
    raw = np.full(coverage, -1, dtype=np.int64)
    for i in range(min(32, coverage)):
        lids[i] = int(lid_perm[i])
        mask = int(rng.integers(0, 4))
        valid[i], modified[i] = bool(mask & 1), bool(mask & 2)
        lfu[i] = int(rng.integers(1, 16384))
        if valid[i]:
            raw[lids[i]] = (lfu[i] << base_scale) + int(rng.integers(0, 1 << base_scale))
    for i in range(coverage):
        if raw[i] == -1:
            raw[i] = int(rng.integers(0, (1 << (14 + base_scale)) + 1))
    upd = rng.permutation(coverage)[:update_count]
    return {"cache_tag_lids": lids, "cache_tag_valid": valid, "cache_tag_modified": modified, "cache_lfu_count": lfu,
            "cache_lfu_count_scale": base_scale, "cache_set_coverage": coverage, "raw_counter": [int(x) for x in raw],
            "start_gid": 0, "to_update_id_count": update_count, "to_update_gids": [int(x) for x in upd],
            "to_update_inc_count": [int(x) for x in rng.integers(1, inc_max + 1, size=update_count)],
            "name": f"random({base_scale},{coverage},{update_count})"}


def run_case(gpu, wgb, comm, case):
    import torch
    MT, ML, AT, DT = (wgb.WholeGraphMemoryType, wgb.WholeGraphMemoryLocation, wgb.WholeGraphAccessType,
                      wgb.WholeGraphDataType)
    cov_case = case["cache_set_coverage"]
    coverage = max(cov_case, 33)                 # a set covers round(32 / ratio) rows and the ratio is below 1
    dim, sets, the_set = 4, 3, 1
    rows = coverage * sets
    policy = wgb.create_cache_policy(comm, MT.MtContinuous, ML.MlDevice, AT.AtReadWrite, 32.0 / coverage)
    emb = wgb.create_embedding(wgb.make_description([rows, dim], DT.DtFloat), comm, MT.MtContinuous, ML.MlDevice,
                               cache_policy=policy)
    try:
        table = wgb.embedding_tensor(emb)
        tags_t, lfu_t, lines_t, got_cov = wgb.embedding_cache_tensors(emb)
        assert got_cov == coverage
        ctr_ptr, ctr_rows = C.c_void_p(), C.c_int64()
        wgb.check(wgb.lib().wholegraph_b200_embedding_get_cache_counters(emb, C.byref(ctr_ptr), C.byref(ctr_rows)),
                  "get_cache_counters")
        assert ctr_rows.value == rows
        counters = gpu.view_device_memory(ctr_ptr.value, [rows], torch.int64)
        row0 = the_set * coverage
        start = case["start_gid"]
        lids, valid = case["cache_tag_lids"], case["cache_tag_valid"]
        modified = [m and v for m, v in zip(case["cache_tag_modified"], valid)]
        scale0 = case["cache_lfu_count_scale"]
        upd = {g - start: inc for g, inc in zip(case["to_update_gids"], case["to_update_inc_count"])}
        cached_before = {lids[i]: i for i in range(32) if valid[i]}
        assert len(cached_before) == sum(valid), "a state with the same row in two lines"

        # table rows and current values: a modified line holds a newer value than the table
        cols = np.arange(dim, dtype=np.float32) / 8
        table_np = (np.arange(rows, dtype=np.float32)[:, None] + cols[None, :]).astype(np.float32)
        value = table_np.copy()
        lines_np = np.zeros((sets * 32, dim), dtype=np.float32)
        tags_np = np.zeros((sets, 32), dtype=np.uint16)
        lfu_np = np.zeros((sets, 32), dtype=np.uint16)
        count = np.zeros(rows, dtype=np.int64)
        count[row0:row0 + cov_case] = case["raw_counter"]
        for i in range(32):
            if not valid[i]:
                continue
            lid = lids[i]
            if modified[i]:
                value[row0 + lid] = table_np[row0 + lid] + 1000
            lines_np[the_set * 32 + i] = value[row0 + lid]
            tags_np[the_set, i] = VALID | (MODIFIED if modified[i] else 0) | lid
            lfu_np[the_set, i] = case["cache_lfu_count"][i] | (((scale0 >> i) & 1) << 14)
            if lid not in upd:      # the reference ranks such a row by its scaled LFU estimate
                count[row0 + lid] = ((case["cache_lfu_count"][i] + 1) << scale0) - 1
        before = count.copy()
        all_rows = torch.arange(rows, device="cuda", dtype=torch.int64)
        gpu.scatter(torch.from_numpy(table_np).cuda(), all_rows, table)
        gpu.scatter(torch.from_numpy(lines_np).cuda(), torch.arange(sets * 32, device="cuda", dtype=torch.int64), lines_t)
        set_ids = torch.arange(sets, device="cuda", dtype=torch.int64)
        gpu.scatter(torch.from_numpy(tags_np.view(np.int16)).cuda(), set_ids, tags_t)
        gpu.scatter(torch.from_numpy(lfu_np.view(np.int16)).cuda(), set_ids, lfu_t)
        counters.copy_(torch.from_numpy(count).cuda())
        torch.cuda.synchronize()

        # one cached gather that counts every update id `increment` times
        ids = torch.repeat_interleave(torch.tensor([row0 + l for l in upd], dtype=torch.int64, device="cuda"),
                                      torch.tensor(list(upd.values()), dtype=torch.int64, device="cuda"))
        ids = ids[torch.randperm(ids.numel(), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))]
        out = torch.zeros((ids.numel(), dim), dtype=torch.float32, device="cuda")
        wi, wo = gpu.wrap_torch_tensor(ids), gpu.wrap_torch_tensor(out)
        wgb.EmbeddingGatherForward(emb, wi, wo, True, wgb.cached_env_fns(), gpu.current_stream_int())
        torch.cuda.synchronize()
        wgb.destroy_wholegraph_tensor(wi)
        wgb.destroy_wholegraph_tensor(wo)
        assert np.array_equal(out.cpu().numpy(), value[ids.cpu().numpy()]), "the cached gather returned stale rows"

        def read(t, n, width, dtype):
            buf = torch.empty((n, width), dtype=dtype, device="cuda")
            gpu.gather(t, torch.arange(n, device="cuda", dtype=torch.int64), buf)
            torch.cuda.synchronize()
            return buf.cpu().numpy()
        tags_after = read(tags_t, sets, 32, torch.int16).view(np.uint16)
        lfu_after = read(lfu_t, sets, 32, torch.int16).view(np.uint16)
        lines_after = read(lines_t, sets * 32, dim, torch.float32)
        table_after = read(table, rows, dim, torch.float32)
        count_after = counters.cpu().numpy()

        # untouched sets stay as they were
        for s in range(sets):
            if s != the_set:
                assert not tags_after[s].any() and np.array_equal(count_after[s * coverage:(s + 1) * coverage],
                                                                  before[s * coverage:(s + 1) * coverage])
        # counters: exact
        want_count = before.copy()
        for lid, inc in upd.items():
            want_count[row0 + lid] += inc
        assert np.array_equal(count_after, want_count)

        # who may and who must be cached
        rank_count = {lid: int(want_count[row0 + lid]) for lid in set(cached_before) | set(upd)}
        ordered = sorted(rank_count.values(), reverse=True)
        if len(ordered) < 32:
            must, maybe, should = set(rank_count), set(), len(ordered)
        else:
            cut = ordered[31]
            must = {l for l, c in rank_count.items() if c > cut}
            maybe = {l for l, c in rank_count.items() if c <= cut}
            should = 32
        tag = tags_after[the_set]
        new_lid = [int(t & MASK14) if t & VALID else -1 for t in tag]
        new_mod = [bool(t & MODIFIED) for t in tag]
        cached_after = {l: i for i, l in enumerate(new_lid) if l >= 0}
        assert len(cached_after) == sum(1 for l in new_lid if l >= 0), "a row sits in two lines"
        assert len(cached_after) == should
        assert must <= set(cached_after) <= must | maybe
        # scale: the smallest shift that brings the largest count below 2^14, spread over bit 14 of the LFU words
        scale = 0
        while (max(ordered) >> scale) >= (1 << 14):
            scale += 1
        got_scale = sum(1 << i for i in range(32) if lfu_after[the_set, i] & (1 << 14))
        assert got_scale == scale
        for i in range(32):
            lid = new_lid[i]
            if lid < 0:
                assert not new_mod[i]
                continue
            assert int(lfu_after[the_set, i] & MASK14) == rank_count[lid] >> scale, (i, lid)
            if lid in cached_before:            # a row that stays keeps its line and its modified bit
                assert cached_before[lid] == i and new_mod[i] == modified[i]
            else:                               # a new row is one of the updated ones and starts clean
                assert lid in upd and not new_mod[i]
            assert np.array_equal(lines_after[the_set * 32 + i], value[row0 + lid]), "a line holds the wrong row"
        # rows without a line: the table holds their current value (evicted modified lines were written back)
        for lid in range(coverage):
            if lid not in cached_after:
                assert np.array_equal(table_after[row0 + lid], value[row0 + lid]), f"row {lid} lost its update"
    finally:
        wgb.destroy_embedding(emb)
        wgb.destroy_cache_policy(policy)


@pytest.mark.parametrize("case", CASES["literal"], ids=[c["name"] for c in CASES["literal"]])
def test_reference_cache_set_states(gpu, wgb, comm, case):
    run_case(gpu, wgb, comm, case)


@pytest.mark.parametrize("triple", CASES["random"], ids=[f"{a}-{b}-{c}" for a, b, c in CASES["random"]])
def test_reference_random_cache_set_states(gpu, wgb, comm, triple):
    base_scale, coverage, update_count = triple
    # increments are drawn from 1..16383 as in the reference unless that would make the id list
    # (every id repeated by its increment) longer than about eight million entries
    inc_max = max(1, min(16383, 16_000_000 // max(update_count, 1)))
    for seed in (1, 2):
        run_case(gpu, wgb, comm, random_case(base_scale, coverage, update_count, seed * 1000 + coverage, inc_max))
