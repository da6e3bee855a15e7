"""GPU parity of the fused decode step (RoPE of the new token's Q/K, KV append,
split-KV grouped-query attention, merge) and of the fused prefill pass, through
the C ABI, against the oracle run as the reference's layer does it step by
step: rope -> append -> attention (src/llama2_layer_npu.cpp:780-869)."""
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


def to_layout(tok_major, layout, max_pos, kvh):
    """[max_pos][kvh*D] token-major -> requested layout."""
    x = tok_major.reshape(max_pos, kvh, D)
    return np.ascontiguousarray(x.transpose(1, 0, 2)) if layout == "head" else x


def oracle_decode_step(q, k_new, v_new, kc_tok, vc_tok, kv_len, table, H, kvh, neox, dt, mode):
    """One sequence: returns (output [H*D], updated token-major caches)."""
    g = H // kvh
    q_r = orc.rope_single_layer(q.reshape(1, -1), table, kv_len, H, neox, dt)
    k_r = orc.rope_single_layer(k_new.reshape(1, -1), table, kv_len, kvh, neox, dt)
    orc.kv_append(kc_tok, vc_tok, k_r, v_new.reshape(1, -1), kv_len, kvh, D)
    return orc.attn(q_r, kc_tok, vc_tok, 1, kv_len + 1, kv_len, g, kvh, D, dt, mode, threads=8)[0]


@pytest.mark.parametrize("dt,neox,theta", [(BF16, True, 1e6), (FP16, False, 1e4)])
@pytest.mark.parametrize("layout", ["head", "token"])
@pytest.mark.parametrize("H,kvh,lens,chunk", [
    (12, 2, [511], 0),                 # Qwen2.5-1.5B-shaped: one sequence, 511 cached tokens
    (12, 2, [511], 64),                # the same, forced into 8 splits
    (40, 8, [1024, 4096, 1500, 2047, 64, 1, 0], 256),   # ragged batch, Qwen2.5-14B heads
    (40, 40, [2048, 2303, 77], 512),   # MHA (Llama-2-13B heads)
    (16, 1, [300, 1000], 128),         # 16 query heads on one KV head: the packing limit
])
def test_fused_decode_step(ops, dt, neox, theta, layout, H, kvh, lens, chunk):
    if dt == FP16 and layout == "token" and kvh == 40:
        pytest.skip("covered by the head-major run")
    batch = len(lens)
    max_pos = max(lens) + 8
    table = orc.init_freq_cis(D, max_pos, theta, dt)
    q = rnd_bits((batch, H * D), dt, 1)
    k_new, v_new = rnd_bits((batch, kvh * D), dt, 2), rnd_bits((batch, kvh * D), dt, 3)
    kc = rnd_bits((batch, max_pos, kvh * D), dt, 4)
    vc = rnd_bits((batch, max_pos, kvh * D), dt, 5)
    desc = ops.make_desc(dt, batch, H, kvh, 1, max_pos, layout=layout, is_neox=neox)
    kc_d = dev(np.stack([to_layout(kc[b], layout, max_pos, kvh) for b in range(batch)]), dt)
    vc_d = dev(np.stack([to_layout(vc[b], layout, max_pos, kvh) for b in range(batch)]), dt)
    out = torch.empty((batch, H * D), dtype=kc_d.dtype, device="cuda")
    lens_d = torch.tensor(lens, dtype=torch.int32, device="cuda")
    ops.gpu_attn_set_decode_chunk(chunk)
    try:
        max_kv = max(lens) + 1
        ws_bytes = ops.gpu_attn_decode_workspace_bytes(desc, max_kv)
        ws = torch.zeros(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
        ops.gpu_attn_decode_layer(desc, out, None, None, dev(q, dt), dev(k_new, dt), dev(v_new, dt), kc_d, vc_d,
                                  torch.from_numpy(table).cuda(), lens_d, None, True, max_kv, ws, ws_bytes)
        torch.cuda.synchronize()
    finally:
        ops.gpu_attn_set_decode_chunk(0)
    got, got_k, got_v = host(out), host(kc_d), host(vc_d)
    for b in range(batch):
        kc_b, vc_b = kc[b].copy(), vc[b].copy()
        gold = oracle_decode_step(q[b], k_new[b], v_new[b], kc_b, vc_b, lens[b], table, H, kvh, neox, dt,
                                  orc.MODE_GOLDEN)
        assert_parity(got[b], gold, dt, "seq %d len %d" % (b, lens[b]))
        # the cache now holds the rotated K and the raw V at position lens[b], nothing else changed
        assert np.array_equal(got_k[b].reshape(-1), to_layout(kc_b, layout, max_pos, kvh).reshape(-1))
        assert np.array_equal(got_v[b].reshape(-1), to_layout(vc_b, layout, max_pos, kvh).reshape(-1))


def test_decode_steps_in_a_row_match_prefill_of_the_whole_sequence(ops):
    """Appending token by token and attending equals one causal pass over all tokens."""
    dt, H, kvh, steps, prompt, neox = BF16, 12, 2, 6, 70, True
    n = prompt + steps
    max_pos = 128
    table = orc.init_freq_cis(D, max_pos, 1e6, dt)
    q, k, v = rnd_bits((n, H * D), dt, 6), rnd_bits((n, kvh * D), dt, 7), rnd_bits((n, kvh * D), dt, 8)
    q_r = orc.rope_single_layer(q, table, 0, H, neox, dt)
    k_r = orc.rope_single_layer(k, table, 0, kvh, neox, dt)
    gold = orc.attn(q_r, k_r, v, n, n, 0, H // kvh, kvh, D, dt, orc.MODE_GOLDEN, threads=8)
    tab_d = torch.from_numpy(table).cuda()
    # fused prefill of the prompt, then fused decode steps, head-major cache
    desc_p = ops.make_desc(dt, 1, H, kvh, prompt, max_pos, layout="head", is_neox=neox)
    kc_d = torch.zeros((1, kvh, max_pos, D), dtype=torch.bfloat16, device="cuda")
    vc_d = torch.zeros_like(kc_d)
    qe_d = torch.empty((prompt, H * D), dtype=torch.bfloat16, device="cuda")
    out_p = torch.empty_like(qe_d)
    ops.gpu_rope_kv_append_layer(desc_p, qe_d, kc_d, vc_d, dev(q[:prompt], dt), dev(k[:prompt], dt),
                                 dev(v[:prompt], dt), tab_d, None, 0, prompt)
    ops.gpu_attn_prefill_layer(desc_p, out_p, qe_d, kc_d, vc_d, prompt, 0)
    torch.cuda.synchronize()
    assert_parity(host(out_p), gold[:prompt], dt, "prefill")
    desc_d = ops.make_desc(dt, 1, H, kvh, 1, max_pos, layout="head", is_neox=neox)
    ws_bytes = ops.gpu_attn_decode_workspace_bytes(desc_d, max_pos)
    ws = torch.zeros(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    out_d = torch.empty((1, H * D), dtype=torch.bfloat16, device="cuda")
    for s in range(steps):
        pos = prompt + s
        lens_d = torch.tensor([pos], dtype=torch.int32, device="cuda")
        ops.gpu_attn_decode_layer(desc_d, out_d, None, None, dev(q[pos:pos + 1], dt), dev(k[pos:pos + 1], dt),
                                  dev(v[pos:pos + 1], dt), kc_d, vc_d, tab_d, lens_d, None, True, max_pos, ws,
                                  ws_bytes)
        torch.cuda.synchronize()
        assert_parity(host(out_d)[0], gold[pos], dt, "decode step %d" % s)


@pytest.mark.parametrize("parts", [2, 4])
def test_partial_outputs_merge_across_slices_like_one_device(ops, parts):
    """Cache cut into contiguous position slices (one per device): per-slice (O, LSE)
    merged by gpu_attn_merge_lse_layer equals attention over the whole cache."""
    dt, H, kvh, neox = BF16, 40, 8, True
    total_old = 1000                      # tokens cached before this step
    max_pos = 1024
    table = orc.init_freq_cis(D, max_pos, 1e6, dt)
    q = rnd_bits((1, H * D), dt, 9)
    k_new, v_new = rnd_bits((1, kvh * D), dt, 10), rnd_bits((1, kvh * D), dt, 11)
    kc, vc = rnd_bits((max_pos, kvh * D), dt, 12), rnd_bits((max_pos, kvh * D), dt, 13)
    kc_b, vc_b = kc.copy(), vc.copy()
    gold = oracle_decode_step(q[0], k_new[0], v_new[0], kc_b, vc_b, total_old, table, H, kvh, neox, dt,
                              orc.MODE_GOLDEN)
    bounds = np.linspace(0, total_old, parts + 1).astype(int)
    tab_d = torch.from_numpy(table).cuda()
    o_parts = torch.empty((parts, H, D), dtype=torch.float32, device="cuda")
    lse_parts = torch.empty((parts, H), dtype=torch.float32, device="cuda")
    rope_pos = torch.tensor([total_old], dtype=torch.int32, device="cuda")
    for p in range(parts):
        lo, hi = int(bounds[p]), int(bounds[p + 1])
        local_max = hi - lo + 8
        desc = ops.make_desc(dt, 1, H, kvh, 1, local_max, layout="head", is_neox=neox)
        kl = np.zeros((local_max, kvh * D), np.uint16)
        vl = np.zeros((local_max, kvh * D), np.uint16)
        kl[:hi - lo], vl[:hi - lo] = kc[lo:hi], vc[lo:hi]
        kl_d = dev(to_layout(kl, "head", local_max, kvh)[None], dt)
        vl_d = dev(to_layout(vl, "head", local_max, kvh)[None], dt)
        last = p == parts - 1          # the owner of the tail appends the new token
        lens_d = torch.tensor([hi - lo], dtype=torch.int32, device="cuda")
        ws_bytes = ops.gpu_attn_decode_workspace_bytes(desc, local_max)
        ws = torch.zeros(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
        ops.gpu_attn_decode_layer(desc, None, o_parts[p], lse_parts[p], dev(q, dt),
                                  dev(k_new, dt) if last else None, dev(v_new, dt) if last else None, kl_d, vl_d,
                                  tab_d, lens_d, rope_pos, last, hi - lo + 1, ws, ws_bytes)
    out = torch.empty((H, D), dtype=torch.bfloat16, device="cuda")
    ops.gpu_attn_merge_lse_layer(out, o_parts, lse_parts, parts, H, D, dt)
    torch.cuda.synchronize()
    assert_parity(host(out).reshape(-1), gold, dt)


def test_empty_slice_gives_minus_inf_lse_and_is_ignored_by_the_merge(ops):
    dt, H, kvh = BF16, 12, 2
    desc = ops.make_desc(dt, 1, H, kvh, 1, 64, layout="head", is_neox=True)
    table = torch.from_numpy(orc.init_freq_cis(D, 64, 1e6, dt)).cuda()
    kc = torch.zeros((1, kvh, 64, D), dtype=torch.bfloat16, device="cuda")
    q = dev(rnd_bits((1, H * D), dt, 14), dt)
    o = torch.full((2, H, D), 7.0, dtype=torch.float32, device="cuda")
    lse = torch.zeros((2, H), dtype=torch.float32, device="cuda")
    zero = torch.zeros(1, dtype=torch.int32, device="cuda")
    ws = torch.zeros(ops.gpu_attn_decode_workspace_bytes(desc, 1), dtype=torch.uint8, device="cuda")
    ops.gpu_attn_decode_layer(desc, None, o[0], lse[0], q, None, None, kc, kc, table, zero, zero, False, 1, ws,
                              ws.numel())
    torch.cuda.synchronize()
    assert torch.all(torch.isneginf(lse[0])) and torch.all(o[0] == 0)
    o[1] = 3.0
    lse[1] = 0.5
    out = torch.empty((H, D), dtype=torch.bfloat16, device="cuda")
    ops.gpu_attn_merge_lse_layer(out, o, lse, 2, H, D, dt)
    torch.cuda.synchronize()
    assert torch.all(out == 3.0)


@pytest.mark.parametrize("layout", ["head", "token"])
def test_batched_chunked_prefill_equals_full(ops, layout):
    """Batch of sequences, prompt fed in two chunks (offset > 0 on the second)."""
    dt, H, kvh, neox, batch, n, cut = FP16, 8, 4, False, 3, 200, 136
    max_pos = 256
    table = orc.init_freq_cis(D, max_pos, 1e4, dt)
    q, k, v = rnd_bits((batch, n, H * D), dt, 15), rnd_bits((batch, n, kvh * D), dt, 16), rnd_bits(
        (batch, n, kvh * D), dt, 17)
    tab_d = torch.from_numpy(table).cuda()
    shape = (batch, kvh, max_pos, D) if layout == "head" else (batch, max_pos, kvh, D)
    kc_d = torch.zeros(shape, dtype=torch.float16, device="cuda")
    vc_d = torch.zeros_like(kc_d)
    outs = []
    for lo, hi in ((0, cut), (cut, n)):
        m = hi - lo
        desc = ops.make_desc(dt, batch, H, kvh, m, max_pos, layout=layout, is_neox=neox)
        qe = torch.empty((batch, m, H * D), dtype=torch.float16, device="cuda")
        out = torch.empty_like(qe)
        ops.gpu_rope_kv_append_layer(desc, qe, kc_d, vc_d, dev(q[:, lo:hi], dt), dev(k[:, lo:hi], dt),
                                     dev(v[:, lo:hi], dt), tab_d, None, lo, m)
        ops.gpu_attn_prefill_layer(desc, out, qe, kc_d, vc_d, m, lo)
        torch.cuda.synchronize()
        outs.append(host(out))
    got = np.concatenate(outs, axis=1)
    for b in range(batch):
        q_r = orc.rope_single_layer(q[b], table, 0, H, neox, dt)
        k_r = orc.rope_single_layer(k[b], table, 0, kvh, neox, dt)
        gold = orc.attn(q_r, k_r, v[b], n, n, 0, H // kvh, kvh, D, dt, orc.MODE_GOLDEN, threads=8)
        assert_parity(got[b], gold, dt, "seq %d" % b)


def test_decode_rejects_missing_workspace_and_bad_arguments(ops):
    dt, H, kvh = BF16, 40, 8
    desc = ops.make_desc(dt, 4, H, kvh, 1, 4096, layout="head")
    x = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    lens = torch.zeros(4, dtype=torch.int32, device="cuda")
    tab = torch.zeros(16, device="cuda")
    with pytest.raises(ops.GpuOpsError) as e:
        ops.gpu_attn_decode_layer(desc, x, None, None, x, x, x, x, x, tab, lens, None, True, 4096, None, 0)
    assert "workspace" in str(e.value)
    with pytest.raises(ops.GpuOpsError):
        ops.gpu_attn_decode_layer(desc, x, None, None, x, None, None, x, x, tab, lens, None, True, 64, None, 0)
    desc.n_heads = 40 * 17
    desc.n_kv_heads = 40
    with pytest.raises(ops.GpuOpsError):
        ops.gpu_attn_decode_layer(desc, x, None, None, x, x, x, x, x, tab, lens, None, True, 64, None, 0)


def test_early_prefetch_gives_the_same_bits(ops):
    """Four layers with caches of their own, three steps: with the early K/V prefetch on, every output
    and every appended row equals the default ordering bit for bit (the usage the option is meant for:
    consecutive launches never read a cache the preceding kernels write)."""
    dt, H, kvh, batch, max_pos, layers = BF16, 10, 2, 6, 700, 4
    lens0 = np.array([600, 1, 64, 255, 0, 333], dtype=np.int32)
    table = torch.from_numpy(orc.init_freq_cis(D, max_pos, 1e6, dt)).cuda()
    desc = ops.make_desc(dt, batch, H, kvh, 1, max_pos, layout="head", is_neox=True)
    ws_bytes = ops.gpu_attn_decode_workspace_bytes(desc, max_pos)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    results = []
    for early in (0, 1):
        ops.gpu_attn_set_decode_early_prefetch(early)
        try:
            kc = [dev(rnd_bits((batch, kvh, max_pos, D), dt, 500 + l), dt) for l in range(layers)]
            vc = [dev(rnd_bits((batch, kvh, max_pos, D), dt, 600 + l), dt) for l in range(layers)]
            lens = torch.from_numpy(lens0.copy()).cuda()
            outs = []
            for step in range(3):
                for l in range(layers):
                    q = dev(rnd_bits((batch, H * D), dt, 1000 + 10 * step + l), dt)
                    k = dev(rnd_bits((batch, kvh * D), dt, 2000 + 10 * step + l), dt)
                    v = dev(rnd_bits((batch, kvh * D), dt, 3000 + 10 * step + l), dt)
                    o = torch.empty((batch, H * D), dtype=torch.bfloat16, device="cuda")
                    ops.gpu_attn_decode_layer(desc, o, None, None, q, k, v, kc[l], vc[l], table, lens, None, True,
                                              int(lens0.max()) + step + 1, ws, ws_bytes)
                    outs.append(o)
                torch.cuda.synchronize()      # the lengths change between steps, not between layers
                lens += 1
            results.append((outs, kc, vc))
        finally:
            ops.gpu_attn_set_decode_early_prefetch(0)
    for a, b in zip(results[0][0], results[1][0]):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    for l in range(layers):
        assert torch.equal(results[0][1][l].view(torch.int16), results[1][1][l].view(torch.int16))
        assert torch.equal(results[0][2][l].view(torch.int16), results[1][2][l].view(torch.int16))


def test_understated_max_kv_len_is_reported_and_reads_nothing_beyond_its_scratch(ops):
    """The caller's bound on the cache lengths (max_kv_len) sizes the grid and the scratch; the kernels take the
    lengths themselves from device memory.  A sequence longer than the bound cannot be served (its last splits are
    never launched), but the call must degrade safely: the status word reports it (code 40), the merge uses only the
    splits that exist (the scratch is followed by NaN here: reading past it would show in the output), and the
    context stays usable."""
    dt, H, kvh, kv_len, chunk, max_pos = BF16, 12, 2, 700, 128, 1024
    table = orc.init_freq_cis(D, max_pos, 1e6, dt)
    q = rnd_bits((1, H * D), dt, 1)
    k_new, v_new = rnd_bits((1, kvh * D), dt, 2), rnd_bits((1, kvh * D), dt, 3)
    kc, vc = rnd_bits((1, kvh, max_pos, D), dt, 4), rnd_bits((1, kvh, max_pos, D), dt, 5)
    desc = ops.make_desc(dt, 1, H, kvh, 1, max_pos, layout="head", is_neox=True)
    out = torch.empty((1, H * D), dtype=torch.bfloat16, device="cuda")
    lens_d = torch.tensor([kv_len], dtype=torch.int32, device="cuda")
    understated = 640                                     # five splits of 128; the sequence needs six
    ops.gpu_attn_set_decode_chunk(chunk)
    try:
        ws_bytes = ops.gpu_attn_decode_workspace_bytes(desc, understated)
        ws = torch.full((ws_bytes // 4 + 4096,), float("nan"), dtype=torch.float32, device="cuda")
        assert ops.gpu_ops_kernel_status() == 0
        ops.gpu_attn_decode_layer(desc, out, None, None, dev(q, dt), dev(k_new, dt), dev(v_new, dt), dev(kc, dt),
                                  dev(vc, dt), torch.from_numpy(table).cuda(), lens_d, None, True, understated, ws,
                                  ws_bytes)
        torch.cuda.synchronize()
        assert ops.gpu_ops_kernel_status() == 40
        assert bool(torch.isfinite(out.float()).all())
        assert bool(torch.isnan(ws[ws_bytes // 4:]).all())    # nothing was written behind the scratch either
    finally:
        ops.gpu_attn_set_decode_chunk(0)
        ops.gpu_ops_clear_kernel_status()
    # the same call with an honest bound works afterwards
    ws_bytes = ops.gpu_attn_decode_workspace_bytes(desc, kv_len + 1)
    ws = torch.zeros(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    kc_d, vc_d = dev(kc, dt), dev(vc, dt)
    ops.gpu_attn_decode_layer(desc, out, None, None, dev(q, dt), dev(k_new, dt), dev(v_new, dt), kc_d, vc_d,
                              torch.from_numpy(table).cuda(), lens_d, None, True, kv_len + 1, ws, ws_bytes)
    torch.cuda.synchronize()
    assert ops.gpu_ops_kernel_status() == 0
    kc_tok = np.ascontiguousarray(kc[0].transpose(1, 0, 2)).reshape(max_pos, kvh * D)
    vc_tok = np.ascontiguousarray(vc[0].transpose(1, 0, 2)).reshape(max_pos, kvh * D)
    gold = oracle_decode_step(q[0], k_new[0], v_new[0], kc_tok, vc_tok, kv_len, table, H, kvh, True, dt, orc.MODE_GOLDEN)
    assert_parity(host(out)[0], gold, dt, "after the reported call")
