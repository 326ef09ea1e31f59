"""Index arithmetic of the GEMM kernel's stream-K mode, restated on the CPU and checked for the
invariants the cooperative finish relies on (``dynaflow_b200/csrc/mlp.cu``: ``SegmentIter::next``
for the segments, the host's choice of ``sk_per``, the epilogue's slot rule, and the share of a
tile's outputs each contributor sums). Pure Python: no GPU, no library call."""
import pytest


def host_plan(num_tiles: int, num_kb: int, units: int):
    """launch_variant: k-blocks per CTA and grid size when stream-K engages."""
    total = num_tiles * num_kb
    g = min(units, max(1, total // 4))            # at least four k-blocks per CTA
    per = -(-total // g)
    grid = -(-total // per)
    return per, grid


def segments(unit: int, per: int, num_tiles: int, num_kb: int):
    """SegmentIter (stream-K): the unit's range of the tile-major k-block sequence, cut at tile ends."""
    total = num_tiles * num_kb
    cur, end = min(unit * per, total), min((unit + 1) * per, total)
    out = []
    while cur < end:
        tile = cur // num_kb
        kb0 = cur - tile * num_kb
        stop = min((tile + 1) * num_kb, end)
        out.append((tile, kb0, kb0 + stop - cur))
        cur = stop
    return out


@pytest.mark.parametrize("num_tiles,num_kb,units", [(16, 224, 148), (112, 64, 148), (32, 224, 148), (1, 8, 148),
                                                     (3, 9, 5), (7, 64, 16), (14, 28, 140), (2, 1000, 148)])
def test_partial_sums_cover_every_tile_once_and_slots_never_collide(num_tiles, num_kb, units):
    per, grid = host_plan(num_tiles, num_kb, units)
    assert grid <= units and per * grid >= num_tiles * num_kb
    covered = {t: [] for t in range(num_tiles)}
    delivered = {t: 0 for t in range(num_tiles)}
    for unit in range(grid):
        segs = segments(unit, per, num_tiles, num_kb)
        used_slots = set()
        pending = 0
        for tile, kb0, kb1 in segs:
            covered[tile].append((kb0, kb1, unit))
            if kb0 == 0 and kb1 == num_kb:
                continue                                  # whole tile: epilogue straight from tensor memory
            slot = 0 if kb0 > 0 else 1                    # the epilogue's slot rule
            assert slot not in used_slots, "a CTA would overwrite its own partial sums"
            used_slots.add(slot)
            delivered[tile] += 1
            pending += 1
        assert pending <= 2                               # the kernel remembers at most two unfinished tiles
    for t in range(num_tiles):
        ranges = sorted(covered[t])
        assert ranges[0][0] == 0 and ranges[-1][1] == num_kb
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))          # contiguous, no overlap
        # what a contributor computes after the loop: first / last CTA of the tile and their count
        first = (t * num_kb) // per
        last = ((t + 1) * num_kb - 1) // per
        S = last - first + 1
        assert [u for _, _, u in ranges] == list(range(first, last + 1))       # consecutive CTAs, in k order
        if S > 1:
            assert delivered[t] == S                       # the counter value everybody waits for
            # contributor 0 started the tile (slot 1), the others started inside it (slot 0)
            assert ranges[0][0] == 0 and all(r[0] > 0 for r in ranges[1:])
        else:
            assert delivered[t] == 0


@pytest.mark.parametrize("S", [2, 3, 5, 9, 10])
@pytest.mark.parametrize("rows", [1, 16, 100, 128])
def test_operand_swapped_shares_cover_all_outputs(S, rows):
    """Operand-swapped form: contributor s finishes the pairs [s*E/S, (s+1)*E/S) of E = rows*128."""
    E = rows * 128
    seen = []
    for s in range(S):
        lo, hi = s * E // S, (s + 1) * E // S
        seen.extend(range(lo, hi))
    assert seen == list(range(E))


@pytest.mark.parametrize("S", [2, 3, 5, 9, 10])
@pytest.mark.parametrize("groups", [16, 32])
def test_regular_form_column_groups_cover_the_tile(S, groups):
    """Regular form: contributor s finishes the groups [s*G/S, (s+1)*G/S) of eight output columns."""
    seen = []
    for s in range(S):
        seen.extend(range(s * groups // S, (s + 1) * groups // S))
    assert seen == list(range(groups))


def fused_chunks(tiles_m: int, tiles_n: int, tiles_n2: int, g: int = 32, gd: int = 16, max_chunks: int = 64):
    """launch_fused_mlp: the chunk table of the single-launch MLP."""
    while ((tiles_m + g - 1) // g) * (1 + (g + gd - 1) // gd) > max_chunks:
        g *= 2
        gd *= 2
    chunks, start = [], 0

    def add(phase, grp):
        nonlocal start
        group_first = grp * g
        group_gm = min(g, tiles_m - group_first)
        step = gd if phase else g
        for off in range(0, group_gm, step):
            gm = min(step, group_gm - off)
            chunks.append((start, phase, group_first + off, gm))
            start += gm * (tiles_n2 if phase else tiles_n)

    groups = (tiles_m + g - 1) // g
    for grp in range(groups):
        add(0, grp)
        if grp >= 1:
            add(1, grp - 1)
    add(1, groups - 1)
    return chunks, start


@pytest.mark.parametrize("tiles_m", [2, 31, 32, 33, 64, 65, 128, 512, 2000])
def test_single_launch_order_puts_a_panels_gate_up_tiles_before_its_down_tiles(tiles_m):
    tiles_n, tiles_n2 = 112, 16
    chunks, total = fused_chunks(tiles_m, tiles_n, tiles_n2)
    assert len(chunks) <= 64 and total == tiles_m * (tiles_n + tiles_n2)
    last_up_tile = {}
    first_down_tile = {}
    seen = set()
    for start, phase, first_m, gm in chunks:
        n = tiles_n2 if phase else tiles_n
        for within in range(gm * n):
            t = start + within
            m_blk, n_blk = first_m + within % gm, within // gm        # fused_coords
            assert (phase, m_blk, n_blk) not in seen
            seen.add((phase, m_blk, n_blk))
            if phase == 0:
                last_up_tile[m_blk] = max(last_up_tile.get(m_blk, -1), t)
            else:
                first_down_tile[m_blk] = min(first_down_tile.get(m_blk, 1 << 60), t)
    assert len(seen) == total
    for m in range(tiles_m):
        # tiles are handed out in index order: every gate/up tile a down tile waits for is already held by a CTA
        assert last_up_tile[m] < first_down_tile[m]
