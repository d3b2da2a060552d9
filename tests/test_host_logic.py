"""CPU-only tests: the C-ABI library loads and exports every symbol the header
declares; suffix packing matches the reference's q3_decide_run packing; the
launch schedule covers every key tile of every item exactly once."""
import os
import re

import numpy as np
import pytest

import __graft_entry__ as entry

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def pkg():
    entry.build()
    return entry.load_package()


def test_library_exports_every_declared_symbol(pkg):
    import ctypes
    names = set()
    for h in sorted(os.listdir(os.path.join(ROOT, "include"))):
        hdr = open(os.path.join(ROOT, "include", h)).read()
        hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
        names |= set(re.findall(r"\b(q3_[a-z0-9_]+)\s*\(", hdr))
    assert len(names) > 60 and "q3_cuda_q4k_linear" in names
    L = ctypes.CDLL(pkg.lib_path())
    missing = [n for n in sorted(names) if not hasattr(L, n)]
    assert not missing, missing
    assert b"sm_100a" in pkg.lib().q3_attn_version()


def test_no_gpu_fails_loudly(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(pkg.Q3Error, match="no CUDA device"):
        pkg.Runtime(num_layers=1, n_heads=8, n_kv_heads=1, max_positions=64,
                    max_tokens=16, num_pages=8)


def test_geometry_is_checked_before_any_cuda_call(pkg):
    with pytest.raises(pkg.Q3Error, match="unsupported geometry"):
        pkg.Runtime(num_layers=1, n_heads=12, n_kv_heads=2, max_positions=64,
                    max_tokens=16, num_pages=8)
    with pytest.raises(pkg.Q3Error, match="unsupported geometry"):
        pkg.Runtime(num_layers=1, n_heads=8, n_kv_heads=1, max_positions=64,
                    max_tokens=16, num_pages=8, head_dim=64)


def test_decode_work_rejects_empty_context(pkg):
    work, swb = pkg.decode_work_host(np.asarray([40, 3000], np.uint32))
    assert len(work) == 1 + 3 and swb.tolist() == [0, 1, 4]
    assert work[:, 3].tolist() == [0, 1, 2, 3]          # slot == index of the work item
    with pytest.raises(pkg.Q3Error, match="no context"):
        pkg.decode_work_host(np.asarray([40, 0], np.uint32))


def test_pack_suffix_matches_reference_packing(pkg):
    # ref: src/q3_decide.cu:440-464 - tight packing, positions = P + j
    items = [(5, 3), (2, 1), (7, 4)]
    r = pkg.pack_suffix_host(items, prefix_len=129, max_branches=8, max_suffix=16)
    assert r["tokens"] == 8
    assert r["token_branch"].tolist() == [5, 5, 5, 2, 7, 7, 7, 7]
    assert r["token_local_pos"].tolist() == [0, 1, 2, 0, 0, 1, 2, 3]
    assert r["token_positions"].tolist() == [129, 130, 131, 129, 129, 130, 131, 132]
    assert r["branch_offsets"].tolist() == [0, 3, 4, 8]


@pytest.mark.parametrize("items,msg", [
    ([(0, 0)], "invalid decision item"),           # empty suffix
    ([(0, 17)], "invalid decision item"),          # over max_suffix
    ([(9, 2)], "invalid branch handle"),
    ([(0, 1)] * 9, "bad branch count"),            # more items than branches
])
def test_pack_suffix_rejects(pkg, items, msg):
    with pytest.raises(pkg.Q3Error, match=msg):
        pkg.pack_suffix_host(items, prefix_len=10, max_branches=8, max_suffix=16)


def _check_schedule(pkg, row_tag, row_lp, n_kv, shared_len, ppb, nb, ctas, lockstep=False,
                    balanced=True):
    summ, segs = pkg.schedule_describe(row_tag, row_lp, n_kv, shared_len, ppb, nb, ctas,
                                       lockstep=lockstep)
    assert summ.n_segments == len(segs)
    T = len(row_tag)
    n_tt = (T + 31) // 32
    shared_tiles = ((shared_len + 15) // 16 + 7) // 8
    # expected key tiles per token tile
    exp = []
    for tt in range(n_tt):
        need = {}
        for t in range(tt * 32, min(T, tt * 32 + 32)):
            need[row_tag[t]] = max(need.get(row_tag[t], 0), row_lp[t] // 16 + 1)
        exp.append(shared_tiles + (sum(need.values()) + 7) // 8)
    assert summ.total_key_tiles == n_kv * sum(exp)
    cover = {}
    per_cta = {}
    for s in segs:
        assert s.tile_begin < s.tile_end
        assert s.shared_tiles == shared_tiles
        key = (s.kv_head, s.tok0)
        cover.setdefault(key, []).append((s.tile_begin, s.tile_end, s.partial_slot))
        # cost of a segment as the scheduler charges it: its key tiles + a fixed start-up of 2.5 tiles
        per_cta[s.cta] = per_cta.get(s.cta, 0) + s.tile_end - s.tile_begin + 2.5
    assert len(cover) == n_kv * n_tt
    slots = set()
    n_cut = 0
    for (h, tok0), parts in cover.items():
        parts.sort()
        assert parts[0][0] == 0 and parts[-1][1] == exp[tok0 // 32]
        for a, b in zip(parts, parts[1:]):
            assert a[1] == b[0]                      # contiguous, no overlap
        if len(parts) == 1:
            assert parts[0][2] == -1                 # whole item: direct output
        else:
            n_cut += 1
            for p in parts:
                assert p[2] >= 0 and p[2] not in slots
                slots.add(p[2])
    assert summ.n_cut_items == n_cut and summ.n_slots == len(slots)
    loads = list(per_cta.values())
    assert len(loads) <= summ.grid == min(ctas, summ.total_key_tiles)
    if balanced and len(loads) == summ.grid:
        # cost-balanced stream-K: no CTA is far above the mean
        mean = sum(loads) / len(loads)
        assert max(loads) <= 1.08 * mean + 3.0
    return summ


def test_schedule_prefill(pkg):
    T = 4096
    s = _check_schedule(pkg, np.zeros(T, np.uint32), np.arange(T, dtype=np.uint32),
                        8, 0, 256, 1, 148)
    assert s.grid == 148


def test_schedule_cascade_configs(pkg):
    # 8192-token prefix + 64 branches x 24; 32768 + 128 x 16
    for P, B, n in ((8192, 64, 24), (32768, 128, 16), (129, 32, 13)):
        tag = np.repeat(np.arange(B, dtype=np.uint32), n)
        lp = np.tile(np.arange(n, dtype=np.uint32), B)
        _check_schedule(pkg, tag, lp, 8, P, (n + 15) // 16, B, 148)
        # whole-item waves + stream-K tail: same coverage, same balance (equal items),
        # and no more cut items than CTAs
        s = _check_schedule(pkg, tag, lp, 8, P, (n + 15) // 16, B, 148, lockstep=True)
        assert s.n_cut_items <= 148


def test_schedule_ragged_and_tiny(pkg):
    rng = np.random.default_rng(0)
    lens = rng.integers(1, 70, 11)
    handles = rng.permutation(16)[:11]
    tag = np.concatenate([np.full(n, h, np.uint32) for h, n in zip(handles, lens)])
    lp = np.concatenate([np.arange(n, dtype=np.uint32) for n in lens])
    _check_schedule(pkg, tag, lp, 2, 77, 5, 16, 148)
    _check_schedule(pkg, tag, lp, 1, 0, 5, 16, 7)
    _check_schedule(pkg, tag, lp, 2, 77, 5, 16, 5, lockstep=True, balanced=False)
    _check_schedule(pkg, np.zeros(1, np.uint32), np.zeros(1, np.uint32), 1, 0, 1, 1, 148)


def test_kv_bytes_accounting(pkg):
    # ref: src/q3_decide.cu:54-59 (fp32 K+V); the 129-token prefix of the
    # reference's report is 67,633,152 B
    assert pkg.lib().q3_kv_bytes_for_tokens(129, 64, 8, 128) == 67633152


def test_decode_work_covers_every_page_once(pkg):
    """q3_decode_work_host: every sequence is cut into chunks of at most 64 pages
    that tile its page list exactly; slots are consecutive."""
    ctx = np.asarray([1, 16, 17, 1024, 1025, 16384, 5000], np.uint32)
    work, swb = pkg.decode_work_host(ctx)
    assert swb[0] == 0 and swb[-1] == len(work)
    for s, c in enumerate(ctx):
        chunks = work[swb[s]:swb[s + 1]]
        assert len(chunks) >= 1 and all(ch[0] == s for ch in chunks)
        pages = (int(c) + 15) // 16
        assert chunks[0][1] == 0 and chunks[-1][2] == pages
        for a, b in zip(chunks, chunks[1:]):
            assert a[2] == b[1]
        assert all(0 < ch[2] - ch[1] <= 64 for ch in chunks)
    assert work[:, 3].tolist() == list(range(len(work)))


def test_linear_geometry_and_plan(pkg):
    """Host side of the Q4_K linear: geometry binding as the reference's binder
    does it (ref: src/q3_q4_linear.cu:47-91) and the launch shape."""
    from sera_c_b200 import q4_linear as q4
    g = q4.bind_geometry(5120, 10240)
    assert (g.K, g.N, g.M, g.qtype) == (5120, 10240, 0, 12)
    assert g.weight_bytes == 10240 * 20 * 144
    assert q4.bind_geometry(5120, 1024, qtype=q4.Q6_K).weight_bytes == 1024 * 20 * 210
    for args, msg in (((5000, 128), "multiple of 256"), ((0, 128), "degenerate"),
                      ((256, 0), "degenerate")):
        with pytest.raises(pkg.Q3Error, match=msg):
            q4.bind_geometry(*args)
    with pytest.raises(pkg.Q3Error, match="neither Q4_K nor Q6_K"):
        q4.bind_geometry(256, 128, qtype=2)
    # small batches: one token tile, rounded up to 16
    for m, want in ((1, 16), (16, 16), (17, 32), (100, 112), (256, 256)):
        p = q4.plan(m, 10240)
        assert p.token_tile == want and p.tiles == 80 and p.ctas == 80
    # large batches: a multiple of 16 in [96, 256] that keeps the last wave full
    for m, n in ((2048, 10240), (4096, 10240), (2048, 5120), (300, 256), (100000, 1024)):
        p = q4.plan(m, n)
        assert p.token_tile % 16 == 0 and 96 <= p.token_tile <= 256
        assert p.tiles == -(-m // p.token_tile) * (n // 128)
        assert p.ctas == min(p.tiles, 148)
        # never worse than the plain 256-token tiling under the same cost model
        base = -(-(-(-m // 256) * (n // 128)) // 148) * (256 + 32)
        assert p.tiles_per_cta_max * (p.token_tile + 32) <= base
    assert q4.plan(2048, 5120).token_tile == 192       # 440 tiles = 2.97 waves
    with pytest.raises(pkg.Q3Error, match="invalid argument"):
        q4.plan(16, 100)
