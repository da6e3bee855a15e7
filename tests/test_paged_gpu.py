"""GPU parity of the paged KV cache: the append and the fused decode step through
a page table against the same operators on a flat cache (bit-identical: the
arithmetic and the split of the cache are the same, only the addresses differ)
and against the oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import BF16, D, FP16, assert_parity, dev, host, rnd_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from llm_simple_b200 import ops as o
    o.lib()
    return o


def _tables(batch, max_pos, page_size, seed):
    """A random, non-contiguous assignment of pool pages to (sequence, page index)."""
    per_seq = (max_pos + page_size - 1) // page_size
    n_pages = batch * per_seq + 3                       # a few pages stay unused
    perm = np.random.default_rng(seed).permutation(n_pages)[:batch * per_seq]
    return perm.reshape(batch, per_seq).astype(np.int32), n_pages


def _gather_flat(pool, table, page_size, layout, kvh, max_pos):
    """Pool -> flat head-major cache [batch][kvh][max_pos][D] as the table maps it."""
    batch, per_seq = table.shape
    out = np.zeros((batch, kvh, per_seq * page_size, D), np.uint16)
    for b in range(batch):
        for i in range(per_seq):
            page = pool[table[b, i]]
            if layout == "token":                       # page [page_size][kvh][D]
                page = page.transpose(1, 0, 2)
            out[b, :, i * page_size:(i + 1) * page_size] = page
    return out[:, :, :max_pos]


@pytest.mark.parametrize("dt,neox,theta", [(FP16, False, 1e4), (BF16, True, 1e6)])
@pytest.mark.parametrize("page_size,layout", [(64, "head"), (256, "head"), (128, "token")])
def test_paged_append_then_decode_matches_flat(ops, dt, neox, theta, page_size, layout):
    batch, H, kvh, max_pos = 5, 10, 2, 1100
    lens = np.array([1000, 64, 63, 511, 0], dtype=np.int32)      # prompt lengths; one empty sequence
    table_np, n_pages = _tables(batch, max_pos, page_size, 3)
    table = torch.from_numpy(table_np).cuda()
    page_shape = (kvh, page_size, D) if layout == "head" else (page_size, kvh, D)
    canary = np.uint16(0x7BCD)
    k_pool = dev(np.full((n_pages,) + page_shape, canary, np.uint16), dt)
    v_pool = dev(np.full((n_pages,) + page_shape, canary, np.uint16), dt)
    k_flat = dev(np.full((batch, kvh, max_pos, D), canary, np.uint16), dt)
    v_flat = dev(np.full((batch, kvh, max_pos, D), canary, np.uint16), dt)
    tab = orc.init_freq_cis(D, max_pos, theta, dt)
    tab_d = torch.from_numpy(tab).cuda()
    pages = ops.make_pages(table, page_size, kvh * page_size * D, n_pages)
    # ---- prompts: every sequence appends m rows at position 0 (rows beyond its length are overwritten later)
    m = int(lens.max())
    q = rnd_bits((batch, m, H * D), dt, 1)
    k, v = rnd_bits((batch, m, kvh * D), dt, 2), rnd_bits((batch, m, kvh * D), dt, 3)
    d_flat = ops.make_desc(dt, batch, H, kvh, m, max_pos, layout="head", is_neox=neox)
    d_page = ops.make_desc(dt, batch, H, kvh, m, page_size, layout=layout, is_neox=neox)
    qo_a = torch.empty((batch, m, H * D), dtype=k_pool.dtype, device="cuda")
    qo_b = torch.empty_like(qo_a)
    ops.gpu_rope_kv_append_layer(d_flat, qo_a, k_flat, v_flat, dev(q, dt), dev(k, dt), dev(v, dt), tab_d, None, 0, m)
    ops.gpu_rope_kv_append_paged_layer(d_page, pages, qo_b, k_pool, v_pool, dev(q, dt), dev(k, dt), dev(v, dt), tab_d,
                                       None, 0, m)
    torch.cuda.synchronize()
    assert torch.equal(qo_a.view(torch.int16), qo_b.view(torch.int16))
    got_k = _gather_flat(host(k_pool), table_np, page_size, layout, kvh, max_pos)
    got_v = _gather_flat(host(v_pool), table_np, page_size, layout, kvh, max_pos)
    assert np.array_equal(got_k, host(k_flat)) and np.array_equal(got_v, host(v_flat))
    # ---- three ragged decode steps on both caches
    lens_d = torch.from_numpy(lens).cuda()
    dd_flat = ops.make_desc(dt, batch, H, kvh, 1, max_pos, layout="head", is_neox=neox)
    dd_page = ops.make_desc(dt, batch, H, kvh, 1, page_size, layout=layout, is_neox=neox)
    ws_bytes = ops.gpu_attn_decode_workspace_bytes(dd_flat, max_pos)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    for step in range(3):
        qn = rnd_bits((batch, H * D), dt, 10 + step)
        kn, vn = rnd_bits((batch, kvh * D), dt, 20 + step), rnd_bits((batch, kvh * D), dt, 30 + step)
        o_a = torch.empty((batch, H * D), dtype=k_pool.dtype, device="cuda")
        o_b = torch.empty_like(o_a)
        mx = int(lens.max()) + step + 1
        ops.gpu_attn_decode_layer(dd_flat, o_a, None, None, dev(qn, dt), dev(kn, dt), dev(vn, dt), k_flat, v_flat,
                                  tab_d, lens_d, None, True, mx, ws, ws_bytes)
        ops.gpu_attn_decode_paged_layer(dd_page, pages, o_b, dev(qn, dt), dev(kn, dt), dev(vn, dt), k_pool, v_pool,
                                        tab_d, lens_d, True, mx, ws, ws_bytes)
        torch.cuda.synchronize()
        assert torch.equal(o_a.view(torch.int16), o_b.view(torch.int16)), "step %d" % step
        if step == 0:
            # against the oracle, sequence 3 (511 cached rows + the new one)
            b, L = 3, int(lens[3])
            kc = host(k_flat)[b].transpose(1, 0, 2).reshape(max_pos, kvh * D).copy()
            vc = host(v_flat)[b].transpose(1, 0, 2).reshape(max_pos, kvh * D).copy()
            q_r = orc.rope_single_layer(qn[b:b + 1], tab, L, H, neox, dt)
            gold = orc.attn(q_r, kc, vc, 1, L + 1, L, H // kvh, kvh, D, dt, orc.MODE_GOLDEN)
            assert_parity(host(o_b)[b], gold[0], dt, "paged decode vs oracle")
        lens_d += 1
    got_k = _gather_flat(host(k_pool), table_np, page_size, layout, kvh, max_pos)
    assert np.array_equal(got_k, host(k_flat))           # the appended rows landed in the right pages


@pytest.mark.parametrize("dt", [FP16, BF16])
@pytest.mark.parametrize("page_size,kernel", [(64, 0), (128, 2), (256, 2), (128, 1), (128, 3), (256, 3)])
def test_paged_chunked_prefill_matches_flat(ops, dt, page_size, kernel):
    """Two prefill chunks (offset 0, then offset m1) over a paged cache whose never-written rows hold
    NaN: the output equals the flat-cache output bit for bit and the NaN rows are never seen.
    kernel 0 = automatic choice (pages of 64 run on the mma.sync kernel), 1 = mma.sync, 2 = tcgen05."""
    batch, H, kvh, m1, m2, max_pos = 2, 8, 2, 200, 130, 512
    nan = np.uint16(0x7E00 if dt == FP16 else 0x7FC0)
    table_np, n_pages = _tables(batch, max_pos, page_size, 5)
    table = torch.from_numpy(table_np).cuda()
    k_pool = dev(np.full((n_pages, kvh, page_size, D), nan, np.uint16), dt)
    v_pool = dev(np.full((n_pages, kvh, page_size, D), nan, np.uint16), dt)
    k_flat = dev(np.full((batch, kvh, max_pos, D), nan, np.uint16), dt)
    v_flat = dev(np.full((batch, kvh, max_pos, D), nan, np.uint16), dt)
    tab = orc.init_freq_cis(D, max_pos, 1e4, dt)
    tab_d = torch.from_numpy(tab).cuda()
    pages = ops.make_pages(table, page_size, kvh * page_size * D, n_pages)
    # the flat reference runs on the kernel the paged call will end up on
    flat_kernel = 1 if (kernel == 1 or page_size < 128) else (kernel or 3)
    try:
        off = 0
        for c, m in enumerate((m1, m2)):
            q = rnd_bits((batch, m, H * D), dt, 100 + c)
            k, v = rnd_bits((batch, m, kvh * D), dt, 110 + c), rnd_bits((batch, m, kvh * D), dt, 120 + c)
            d_flat = ops.make_desc(dt, batch, H, kvh, m, max_pos, layout="head")
            d_page = ops.make_desc(dt, batch, H, kvh, m, page_size, layout="head")
            qe_a = torch.empty((batch, m, H * D), dtype=k_pool.dtype, device="cuda")
            qe_b = torch.empty_like(qe_a)
            o_a, o_b = torch.empty_like(qe_a), torch.empty_like(qe_a)
            ops.gpu_rope_kv_append_layer(d_flat, qe_a, k_flat, v_flat, dev(q, dt), dev(k, dt), dev(v, dt), tab_d, None,
                                         off, m)
            ops.gpu_attn_set_prefill_kernel(flat_kernel)
            ops.gpu_attn_prefill_layer(d_flat, o_a, qe_a, k_flat, v_flat, m, off)
            ops.gpu_attn_set_prefill_kernel(kernel)
            ops.gpu_rope_kv_append_paged_layer(d_page, pages, qe_b, k_pool, v_pool, dev(q, dt), dev(k, dt), dev(v, dt),
                                               tab_d, None, off, m)
            ops.gpu_attn_prefill_paged_layer(d_page, pages, o_b, qe_b, k_pool, v_pool, m, off)
            torch.cuda.synchronize()
            assert ops.gpu_ops_kernel_status() == 0
            assert bool(torch.isfinite(o_b.float()).all()), "chunk %d reads unwritten rows" % c
            assert torch.equal(o_a.view(torch.int16), o_b.view(torch.int16)), "chunk %d" % c
            off += m
        # against the oracle: sequence 1, second chunk
        b, n = 1, m1 + m2
        kc = host(k_flat)[b, :, :n].transpose(1, 0, 2).reshape(n, kvh * D).copy()
        vc = host(v_flat)[b, :, :n].transpose(1, 0, 2).reshape(n, kvh * D).copy()
        gold = orc.attn(host(qe_b)[b], kc, vc, m2, n, m1, H // kvh, kvh, D, dt, orc.MODE_GOLDEN, threads=8)
        assert_parity(host(o_b)[b], gold, dt, "paged prefill vs oracle")
    finally:
        ops.gpu_attn_set_prefill_kernel(0)


def test_paged_rejects_bad_page_description(ops):
    desc = ops.make_desc(FP16, 1, 4, 2, 1, 64)
    t = torch.zeros((1, 4), dtype=torch.int32, device="cuda")
    x = torch.zeros(1024, dtype=torch.float16, device="cuda")
    tab = torch.zeros(64, 64, 2, device="cuda")
    lens = torch.zeros(1, dtype=torch.int32, device="cuda")
    for size in (48, 32, 96):
        with pytest.raises(ops.GpuOpsError):
            ops.gpu_attn_decode_paged_layer(desc, ops.make_pages(t, size, 2 * 64 * 128, 4), x, x, x, x, x, x, tab, lens,
                                            True, 1, None, 0)
    assert "page size" in ops.last_error_string()
