"""GPU parity of the planned decode step (gpu_attn_decode_planned_layer: persistent
CTAs on a host-built work partition, K/V tiles by TMA) through the C ABI: against
the oracle run step by step as the reference's layer does it (rope -> append ->
attention, src/llama2_layer_npu.cpp:780-869), bit for bit against the appended
cache rows, and against gpu_attn_decode_layer on the same inputs."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import BF16, D, FP16, assert_parity, dev, host, rnd_bits
from tests.test_decode_gpu import oracle_decode_step, to_layout

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from llm_simple_b200 import ops as o
    o.lib()
    return o


def run_planned(ops, desc, lens, append, n_ctas, out, q_d, k_d, v_d, kc_d, vc_d, tab_d, rope_pos=None, pages=None,
                partial=None):
    plan = ops.DecodePlan(desc, lens, append, n_ctas)
    plan.upload()
    ws = torch.zeros(max(plan.workspace_bytes, 16), dtype=torch.uint8, device="cuda")
    o_p, lse_p = partial if partial is not None else (None, None)
    ops.gpu_attn_decode_planned_layer(desc, pages, plan, out, o_p, lse_p, q_d, k_d, v_d, kc_d, vc_d, tab_d, rope_pos,
                                      ws, plan.workspace_bytes)
    torch.cuda.synchronize()
    assert ops.gpu_ops_kernel_status() == 0
    return plan


@pytest.mark.parametrize("dt,neox,theta", [(BF16, True, 1e6), (FP16, False, 1e4)])
@pytest.mark.parametrize("layout", ["head", "token"])
@pytest.mark.parametrize("H,kvh,lens,n_ctas", [
    (12, 2, [511], 0),                                   # Qwen2.5-1.5B-shaped, one sequence
    (12, 2, [511], 3),                                   # the same on three CTAs: pieces of both heads share a CTA
    (12, 2, [511], 8),                                   # eight CTAs of two tiles: both heads cut in four
    (40, 8, [1024, 4096, 1500, 2047, 64, 1, 0, 63, 128], 0),   # ragged batch, Qwen2.5-14B heads; new token opens a tile
    (40, 8, [1024, 4096, 1500, 2047, 64, 1, 0], 7),      # few CTAs: many pieces per CTA, whole caches inside a share
    (40, 8, [1024, 4096, 1500, 2047, 64, 1, 0], 296),    # every slot of the device
    (40, 8, [4096], 296),                                # one long sequence: every head in many pieces
    (40, 8, [300, 200, 100, 50, 700], 16),
    (40, 40, [2048, 2303, 77], 0),                       # MHA (Llama-2-13B heads)
    (16, 1, [300, 1000], 5),                             # 16 query heads on one KV head: the packing limit
    (16, 1, [300, 1000, 5000], 64),                      # the same, the long cache in 50 pieces: two merge rounds per warp
])
def test_planned_decode_step(ops, dt, neox, theta, layout, H, kvh, lens, n_ctas):
    if dt == FP16 and layout == "token" and kvh == 40:
        pytest.skip("covered by the head-major run")
    batch = len(lens)
    max_pos = max(lens) + 8
    table = orc.init_freq_cis(D, max_pos, theta, dt)
    q = rnd_bits((batch, H * D), dt, 1)
    k_new, v_new = rnd_bits((batch, kvh * D), dt, 2), rnd_bits((batch, kvh * D), dt, 3)
    kc = rnd_bits((batch, max_pos, kvh * D), dt, 4)
    vc = rnd_bits((batch, max_pos, kvh * D), dt, 5)
    # positions that are not cached yet hold NaN: they must never reach a result
    for b, L in enumerate(lens):
        kc[b, L:] = 0x7fc0 if dt == BF16 else 0x7e00
        vc[b, L:] = 0x7fc0 if dt == BF16 else 0x7e00
    desc = ops.make_desc(dt, batch, H, kvh, 1, max_pos, layout=layout, is_neox=neox)
    kc_d = dev(np.stack([to_layout(kc[b], layout, max_pos, kvh) for b in range(batch)]), dt)
    vc_d = dev(np.stack([to_layout(vc[b], layout, max_pos, kvh) for b in range(batch)]), dt)
    out = torch.empty((batch, H * D), dtype=kc_d.dtype, device="cuda")
    run_planned(ops, desc, lens, True, n_ctas, out, dev(q, dt), dev(k_new, dt), dev(v_new, dt), kc_d, vc_d,
                torch.from_numpy(table).cuda())
    got, got_k, got_v = host(out), host(kc_d), host(vc_d)
    for b in range(batch):
        kc_b, vc_b = kc[b].copy(), vc[b].copy()
        gold = oracle_decode_step(q[b], k_new[b], v_new[b], kc_b[:lens[b] + 1], vc_b[:lens[b] + 1], lens[b], table, H,
                                  kvh, neox, dt, orc.MODE_GOLDEN)
        assert_parity(got[b], gold, dt, "seq %d len %d" % (b, lens[b]))
        # the cache now holds the rotated K and the raw V at position lens[b], nothing else changed
        assert np.array_equal(got_k[b].reshape(-1), to_layout(kc_b, layout, max_pos, kvh).reshape(-1))
        assert np.array_equal(got_v[b].reshape(-1), to_layout(vc_b, layout, max_pos, kvh).reshape(-1))


def test_planned_equals_unplanned_entry_point(ops):
    """Same inputs through gpu_attn_decode_layer and the planned path: both within the
    parity bound of the oracle and of each other (the split points differ, so sums are
    ordered differently); the appended rows are the same bits."""
    dt, H, kvh, neox = BF16, 40, 8, True
    rng = np.random.default_rng(5)
    lens = [int(x) for x in rng.integers(1, 3000, size=24)]
    batch, max_pos = len(lens), max(lens) + 8
    table = orc.init_freq_cis(D, max_pos, 1e6, dt)
    tab_d = torch.from_numpy(table).cuda()
    q, k_new, v_new = rnd_bits((batch, H * D), dt, 21), rnd_bits((batch, kvh * D), dt, 22), rnd_bits((batch, kvh * D), dt, 23)
    kc, vc = rnd_bits((batch, kvh, max_pos, D), dt, 24), rnd_bits((batch, kvh, max_pos, D), dt, 25)
    desc = ops.make_desc(dt, batch, H, kvh, 1, max_pos, layout="head", is_neox=neox)
    outs, caches = [], []
    for planned in (False, True):
        kc_d, vc_d = dev(kc, dt), dev(vc, dt)
        out = torch.empty((batch, H * D), dtype=torch.bfloat16, device="cuda")
        if planned:
            run_planned(ops, desc, lens, True, 0, out, dev(q, dt), dev(k_new, dt), dev(v_new, dt), kc_d, vc_d, tab_d)
        else:
            lens_d = torch.tensor(lens, dtype=torch.int32, device="cuda")
            wsb = ops.gpu_attn_decode_workspace_bytes(desc, max(lens) + 1)
            ws = torch.zeros(max(wsb, 16), dtype=torch.uint8, device="cuda")
            ops.gpu_attn_decode_layer(desc, out, None, None, dev(q, dt), dev(k_new, dt), dev(v_new, dt), kc_d, vc_d, tab_d,
                                      lens_d, None, True, max(lens) + 1, ws, wsb)
            torch.cuda.synchronize()
        outs.append(host(out))
        caches.append((host(kc_d), host(vc_d)))
    assert np.array_equal(caches[0][0], caches[1][0]) and np.array_equal(caches[0][1], caches[1][1])
    assert_parity(outs[1], orc.to_f32(outs[0], dt), dt, "planned vs unplanned")


def test_planned_partials_for_a_merge_across_devices(ops):
    """append_new = 0 over position slices with rope_pos: (O, LSE) per slice, an empty slice included,
    merged by gpu_attn_merge_lse_layer, equals attention over the whole cache."""
    dt, H, kvh, neox, total_old, max_pos = BF16, 40, 8, True, 1000, 1024
    table = orc.init_freq_cis(D, max_pos, 1e6, dt)
    tab_d = torch.from_numpy(table).cuda()
    q = rnd_bits((1, H * D), dt, 9)
    kc, vc = rnd_bits((max_pos, kvh * D), dt, 12), rnd_bits((max_pos, kvh * D), dt, 13)
    q_r = orc.rope_single_layer(q, table, total_old, H, neox, dt)
    gold = orc.attn(q_r, kc, vc, 1, total_old, total_old - 1, H // kvh, kvh, D, dt, orc.MODE_GOLDEN, threads=8)[0]
    bounds = [0, 0, 300, 1000]            # the first slice is empty
    parts = len(bounds) - 1
    o_parts = torch.empty((parts, H, D), dtype=torch.float32, device="cuda")
    lse_parts = torch.empty((parts, H), dtype=torch.float32, device="cuda")
    rope_pos = torch.tensor([total_old], dtype=torch.int32, device="cuda")
    for p in range(parts):
        lo, hi = bounds[p], bounds[p + 1]
        cap = max(hi - lo, 1) + 8
        desc = ops.make_desc(dt, 1, H, kvh, 1, cap, layout="head", is_neox=neox)
        ks, vs = np.zeros((cap, kvh * D), np.uint16), np.zeros((cap, kvh * D), np.uint16)
        ks[:hi - lo], vs[:hi - lo] = kc[lo:hi], vc[lo:hi]
        kc_d = dev(to_layout(ks, "head", cap, kvh)[None], dt)
        vc_d = dev(to_layout(vs, "head", cap, kvh)[None], dt)
        run_planned(ops, desc, [hi - lo], False, 4, None, dev(q, dt), None, None, kc_d, vc_d, tab_d, rope_pos=rope_pos,
                    partial=(o_parts[p], lse_parts[p]))
    assert float(lse_parts[0].max()) == float("-inf")
    out = torch.empty((1, H * D), dtype=torch.bfloat16, device="cuda")
    ops.gpu_attn_merge_lse_layer(out, o_parts, lse_parts, parts, H, D, dt)
    torch.cuda.synchronize()
    assert_parity(host(out)[0], gold, dt, "merged slices")


def test_planned_decode_over_a_paged_cache(ops):
    """Pages of 64 and 256 positions handed out in random order, never-written rows NaN: the
    result and the appended rows equal the flat-cache run bit for bit (same plan, same sums)."""
    dt, H, kvh, neox = BF16, 40, 8, True
    lens = [700, 64, 1, 0, 1023, 255]
    batch, cap = len(lens), 1024
    table = orc.init_freq_cis(D, cap + 8, 1e6, dt)
    tab_d = torch.from_numpy(table).cuda()
    q, k_new, v_new = rnd_bits((batch, H * D), dt, 31), rnd_bits((batch, kvh * D), dt, 32), rnd_bits((batch, kvh * D), dt, 33)
    kc, vc = rnd_bits((batch, kvh, cap, D), dt, 34), rnd_bits((batch, kvh, cap, D), dt, 35)
    desc_flat = ops.make_desc(dt, batch, H, kvh, 1, cap, layout="head", is_neox=neox)
    kc_d, vc_d = dev(kc, dt), dev(vc, dt)
    out_flat = torch.empty((batch, H * D), dtype=torch.bfloat16, device="cuda")
    run_planned(ops, desc_flat, lens, True, 0, out_flat, dev(q, dt), dev(k_new, dt), dev(v_new, dt), kc_d, vc_d, tab_d)
    flat_k, flat_v = host(kc_d), host(vc_d)
    for page_size in (64, 256):
        per_seq = cap // page_size
        n_pages = batch * per_seq + 3
        rng = np.random.default_rng(page_size)
        table_np = rng.permutation(n_pages)[:batch * per_seq].astype(np.int32).reshape(batch, per_seq)
        nan = 0x7fc0
        kp = np.full((n_pages, kvh, page_size, D), nan, np.uint16)
        vp = np.full((n_pages, kvh, page_size, D), nan, np.uint16)
        for b, L in enumerate(lens):
            for e in range(per_seq):
                lo, hi = e * page_size, min((e + 1) * page_size, L)
                if hi > lo:
                    kp[table_np[b, e], :, :hi - lo] = kc[b, :, lo:hi]
                    vp[table_np[b, e], :, :hi - lo] = vc[b, :, lo:hi]
        kp_d, vp_d = dev(kp, dt), dev(vp, dt)
        tbl_d = torch.from_numpy(table_np).cuda()
        desc = ops.make_desc(dt, batch, H, kvh, 1, page_size, layout="head", is_neox=neox)
        pages = ops.make_pages(tbl_d, page_size, kvh * page_size * D, n_pages)
        out = torch.empty((batch, H * D), dtype=torch.bfloat16, device="cuda")
        run_planned(ops, desc, lens, True, 0, out, dev(q, dt), dev(k_new, dt), dev(v_new, dt), kp_d, vp_d, tab_d,
                    pages=pages)
        assert np.array_equal(host(out), host(out_flat)), "page size %d" % page_size
        got_k, got_v = host(kp_d), host(vp_d)
        for b, L in enumerate(lens):
            pg, r = table_np[b, L // page_size], L % page_size
            assert np.array_equal(got_k[pg, :, r], flat_k[b, :, L]) and np.array_equal(got_v[pg, :, r], flat_v[b, :, L])


def test_planned_decode_rejects_bad_arguments(ops):
    dt = BF16
    desc = ops.make_desc(dt, 2, 40, 8, 1, 128, layout="head", is_neox=True)
    plan = ops.DecodePlan(desc, [100, 5], True, 0)
    plan.upload()
    t = torch.zeros(2 * 40 * D, dtype=torch.bfloat16, device="cuda")
    other = ops.make_desc(dt, 3, 40, 8, 1, 128, layout="head", is_neox=True)
    with pytest.raises(ops.GpuOpsError, match="plan was built"):
        ops.gpu_attn_decode_planned_layer(other, None, plan, t, None, None, t, t, t, t, t, t, None, None, 0)
    if plan.workspace_bytes:
        with pytest.raises(ops.GpuOpsError, match="workspace"):
            ops.gpu_attn_decode_planned_layer(desc, None, plan, t, None, None, t, t, t, t, t, t, None, None, 0)
    with pytest.raises(ops.GpuOpsError):
        ops.DecodePlan(desc, [100, -1], True, 0)
    # the cache of the descriptor holds 128 positions per sequence: a plan for 128 + the new token does not fit
    long_plan = ops.DecodePlan(desc, [128, 5], True, 0)
    long_plan.upload()
    ws = torch.zeros(max(long_plan.workspace_bytes, 16), dtype=torch.uint8, device="cuda")
    with pytest.raises(ops.GpuOpsError, match="does not fit the cache"):
        ops.gpu_attn_decode_planned_layer(desc, None, long_plan, t, None, None, t, t, t, t, t, t, None, ws,
                                          long_plan.workspace_bytes)
