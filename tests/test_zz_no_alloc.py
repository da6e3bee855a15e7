"""The decode entry point that allocates nothing (gpu_attn_decode_layer_noalloc).

It exists for hosts that cannot call cudaMalloc when a decode step runs -- a
serving process whose GPU memory is wholly owned by its own pool, a plug-in slot
that must not allocate after start-up, a loop that cannot afford cudaMalloc's
device-wide synchronisation -- and therefore cannot hand gpu_attn_decode_layer a
workspace.  Its split-KV scratch is a fixed 16 MiB array inside the library.

Checked here through the C ABI: two calls in a row (the second with different,
shorter caches, so that anything the first call left in the shared scratch
would show) give the same BITS as the ordinary entry point with a caller
workspace and the same split size -- the two run the same kernels, so a
tolerance would only hide a stale partial that slipped into a merge -- and
agree with the CPU oracle within the tolerance of the other attention tests;
fp16 and a call short enough to need no scratch at all are covered as well; a
call that would need more than the built-in scratch is rejected before anything
is launched.

This file is named so that pytest collects it last: a run that stops at the
first failure has then already run every other test.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import BF16, D, FP16, TORCH_DT, assert_parity, dev, host, rnd_bits

pytestmark = pytest.mark.gpu


def _one_step(ops, lens, seed, use_noalloc, H=40, kvh=8, dt=BF16):
    batch = len(lens)
    max_pos = 4096 + 8
    table = torch.from_numpy(orc.init_freq_cis(D, max_pos, 1e6, dt)).cuda()
    q = dev(rnd_bits((batch, H * D), dt, seed), dt)
    k_new = dev(rnd_bits((batch, kvh * D), dt, seed + 1), dt)
    v_new = dev(rnd_bits((batch, kvh * D), dt, seed + 2), dt)
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    kc = torch.empty((batch, kvh, max_pos, D), dtype=TORCH_DT[dt], device="cuda").normal_(generator=g)
    vc = torch.empty((batch, kvh, max_pos, D), dtype=TORCH_DT[dt], device="cuda").normal_(generator=g)
    kc0, vc0 = host(kc), host(vc)
    desc = ops.make_desc(dt, batch, H, kvh, 1, max_pos, layout="head", is_neox=True)
    lens_d = torch.tensor(lens, dtype=torch.int32, device="cuda")
    out = torch.zeros((batch, H * D), dtype=TORCH_DT[dt], device="cuda")
    max_kv = max(lens) + 1
    if use_noalloc:
        ops.gpu_attn_decode_layer_noalloc(desc, out, q, k_new, v_new, kc, vc, table, lens_d, None, True, max_kv)
    else:
        ops.gpu_attn_set_decode_chunk(512)
        try:
            ws_bytes = ops.gpu_attn_decode_workspace_bytes(desc, max_kv)
            ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
            ops.gpu_attn_decode_layer(desc, out, None, None, q, k_new, v_new, kc, vc, table, lens_d, None, True,
                                      max_kv, ws, ws_bytes)
        finally:
            ops.gpu_attn_set_decode_chunk(0)
    torch.cuda.synchronize()
    inputs = (host(q), host(k_new), host(v_new), kc0, vc0, orc.init_freq_cis(D, max_pos, 1e6, dt))
    return host(out), host(kc), host(vc), inputs


def _oracle_step(inputs, lens, H, kvh, dt):
    """The step on the CPU, sequence by sequence: rope -> append -> attention (fp32 golden)."""
    q, k_new, v_new, kc, vc, table = inputs
    outs = []
    for b, L in enumerate(lens):
        kc_tok = np.ascontiguousarray(kc[b, :, :L + 1].transpose(1, 0, 2)).reshape(L + 1, kvh * D)
        vc_tok = np.ascontiguousarray(vc[b, :, :L + 1].transpose(1, 0, 2)).reshape(L + 1, kvh * D)
        q_r = orc.rope_single_layer(q[b:b + 1], table, L, H, True, dt)
        k_r = orc.rope_single_layer(k_new[b:b + 1], table, L, kvh, True, dt)
        orc.kv_append(kc_tok, vc_tok, k_r, v_new[b:b + 1], L, kvh, D)
        outs.append(orc.attn(q_r, kc_tok, vc_tok, 1, L + 1, L, H // kvh, kvh, D, dt, orc.MODE_GOLDEN, threads=8)[0])
    return np.stack(outs)


@pytest.mark.parametrize("dt", [BF16, FP16])
def test_noalloc_entry_point_matches_the_workspace_entry_point_twice_in_a_row(dt):
    from llm_simple_b200 import ops
    ops.lib()
    ops.gpu_attn_decode_noalloc_prepare()
    H, kvh = 40, 8
    calls = [
        ([4096, 1024, 2500, 3333, 4000, 1500, 2047, 4095], 31),  # up to 9 splits per sequence
        ([700, 64, 1, 0, 1300], 47),                              # shorter: fewer splits than the scratch still holds
        ([511, 300, 17], 53),                                     # one split: the scratch is not used at all
    ]
    for lens, seed in calls:
        ops.gpu_ops_launch_count(True)
        got, got_k, got_v, inputs = _one_step(ops, lens, seed, True, H, kvh, dt)
        assert ops.gpu_ops_launch_count(True) == (2 if max(lens) + 1 > 512 else 1)   # split kernel (+ merge)
        want, want_k, want_v, _ = _one_step(ops, lens, seed, False, H, kvh, dt)
        # same kernels, same split size: the same bits, output and appended K / V rows alike
        assert np.array_equal(got, want)
        assert np.array_equal(got_k, want_k) and np.array_equal(got_v, want_v)
        assert_parity(got, _oracle_step(inputs, lens, H, kvh, dt), dt, "no-alloc decode vs oracle")


def test_noalloc_entry_point_rejects_what_its_scratch_cannot_hold():
    from llm_simple_b200 import ops
    ops.lib()
    dt, H, kvh, batch, max_pos = BF16, 40, 8, 256, 8192
    desc = ops.make_desc(dt, batch, H, kvh, 1, max_pos, layout="head", is_neox=True)
    x = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    lens = torch.zeros(batch, dtype=torch.int32, device="cuda")
    tab = torch.zeros(16, device="cuda")
    # 256 * 40 rows * 16 splits * 516 B = 84.5 MB > 16 MiB: refused on the host, nothing runs
    with pytest.raises(ops.GpuOpsError) as e:
        ops.gpu_attn_decode_layer_noalloc(desc, x, x, x, x, x, x, tab, lens, None, True, max_pos)
    assert "scratch" in str(e.value)
    torch.cuda.synchronize()
