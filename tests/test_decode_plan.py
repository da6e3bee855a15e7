"""Host-side checks of the decode work partition (gpu_attn_decode_plan): pure host
code behind the C ABI, no GPU needed when the CTA count is given."""
import numpy as np
import pytest

from llm_simple_b200 import ops


def check_plan(lens, kvh, group, append, n_ctas):
    desc = ops.make_desc(ops.DT_BFLOAT16, len(lens), kvh * group, kvh, 1, 8192)
    plan = ops.DecodePlan(desc, lens, append, n_ctas)
    h = plan.header
    cb, items, groups = plan.tables()
    assert h["magic"] == 0x504c414e and h["n_ctas"] <= n_ctas and h["total_bytes"] == plan.size
    assert cb[0] == 0 and cb[-1] == h["n_items"] and np.all(np.diff(cb) >= 0)
    # every position of every (sequence, KV head) cache is covered exactly once, in order
    pos, n_pieces = {}, {}
    for b_, kvh_, pos0, pos_end, len_old, slot, has_new, _ in items:
        assert len_old == lens[b_] and pos0 % 64 == 0
        assert pos.get((b_, kvh_), 0) == pos0
        pos[(b_, kvh_)] = pos_end
        n_pieces[(b_, kvh_)] = n_pieces.get((b_, kvh_), 0) + 1
        total = len_old + int(append)
        assert pos_end <= total and (pos_end % 64 == 0 or pos_end == total)
        assert has_new == int(bool(append) and pos0 <= len_old < pos_end)
    for b_, L in enumerate(lens):
        for k in range(kvh):
            assert pos[(b_, k)] == L + int(append)
    assert h["total_tiles"] == sum((L + int(append) + 63) // 64 for L in lens) * kvh
    # a cut cache has one scratch slot per piece, consecutive, and one merge group; a whole one none
    cut = {k for k, v in n_pieces.items() if v > 1}
    assert all((r[5] >= 0) == ((r[0], r[1]) in cut) for r in items)
    assert sorted(int(r[5]) for r in items if r[5] >= 0) == list(range(h["n_slots"]))
    assert sorted((g[2], g[3]) for g in groups) == sorted(cut)
    for first, n, b_, kvh_ in groups:
        mine = [int(r[5]) for r in items if (r[0], r[1]) == (b_, kvh_)]
        assert n == len(mine) >= 2 and mine == list(range(first, first + n))
    assert h["max_parts"] == max([g[1] for g in groups], default=0)
    assert plan.workspace_bytes == h["n_slots"] * group * 129 * 4
    return plan, cb, items


@pytest.mark.parametrize("lens,kvh,group,append,n_ctas", [
    ([511], 2, 6, True, 296), ([511], 2, 6, True, 3), ([0], 1, 1, True, 8), ([0, 0], 2, 5, False, 8),
    ([1024, 4096, 1500, 2047, 64, 1, 0, 63, 128], 8, 5, True, 296), ([32768], 8, 5, True, 296),
    ([100] * 300, 8, 5, True, 296), ([2176] * 8, 40, 1, True, 296), ([5, 5, 5], 8, 5, False, 1024),
])
def test_plan_covers_every_position_once(lens, kvh, group, append, n_ctas):
    check_plan(lens, kvh, group, append, n_ctas)


def test_plan_is_balanced_on_ragged_lengths():
    rng = np.random.default_rng(20254)
    lens = [int(x) for x in rng.integers(1024, 4097, size=64)]
    for kvh in (1, 2, 4, 8):
        for n_ctas in (222, 296):
            plan, cb, items = check_plan(lens, kvh, 5, True, n_ctas)
            tiles = np.array([sum((r[3] - r[2] + 63) // 64 for r in items[cb[c]:cb[c + 1]]) for c in range(n_ctas)])
            assert tiles.max() <= tiles.mean() * 1.08 + 2, (kvh, tiles.min(), tiles.mean(), tiles.max())


def test_plan_random_shapes():
    rng = np.random.default_rng(1)
    for _ in range(60):
        batch = int(rng.integers(1, 40))
        lens = [int(x) for x in rng.integers(0, int(rng.choice([4, 70, 700, 5000])), size=batch)]
        check_plan(lens, int(rng.choice([1, 2, 8])), int(rng.choice([1, 5, 16])), bool(rng.integers(0, 2)),
                   int(rng.choice([1, 2, 7, 296, 1024])))


def test_plan_rejects_bad_arguments():
    desc = ops.make_desc(ops.DT_BFLOAT16, 2, 40, 8, 1, 128)
    with pytest.raises(ops.GpuOpsError):
        ops.DecodePlan(desc, [3, -1], True, 8)
    with pytest.raises(ops.GpuOpsError):
        ops.DecodePlan(desc, [3, 4], True, 5000)
    wide = ops.make_desc(ops.DT_BFLOAT16, 1, 34, 2, 1, 128)   # 17 query heads per KV head
    with pytest.raises(ops.GpuOpsError, match="group size"):
        ops.DecodePlan(wide, [3], True, 8)
