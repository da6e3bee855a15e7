"""The decode entry point that allocates nothing (gpu_attn_decode_layer_noalloc).

It exists for hosts that cannot call cudaMalloc when a decode step runs -- a
serving process whose GPU memory is wholly owned by its own pool, a plug-in slot
that must not allocate after start-up, a loop that cannot afford cudaMalloc's
device-wide synchronisation -- and therefore cannot hand gpu_attn_decode_layer a
workspace.  Its split-KV scratch is a fixed 16 MiB array inside the library.

Checked here through the C ABI: two calls in a row (the second with different,
shorter caches, so that anything the first call left in the shared scratch
would show) give the same result as the ordinary entry point with a caller
workspace, within the tolerance of the other attention tests; a call that would
need more than the built-in scratch is rejected before anything is launched.

This file is named so that pytest collects it last: a run that stops at the
first failure has then already run every other test.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import BF16, D, MAX_ABS, MEAN_ABS, dev, host, rnd_bits

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
    kc = torch.empty((batch, kvh, max_pos, D), dtype=torch.bfloat16, device="cuda").normal_(generator=g)
    vc = torch.empty((batch, kvh, max_pos, D), dtype=torch.bfloat16, device="cuda").normal_(generator=g)
    desc = ops.make_desc(dt, batch, H, kvh, 1, max_pos, layout="head", is_neox=True)
    lens_d = torch.tensor(lens, dtype=torch.int32, device="cuda")
    out = torch.zeros((batch, H * D), dtype=torch.bfloat16, device="cuda")
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
    return orc.to_f32(host(out), dt), host(kc), host(vc)


def test_noalloc_entry_point_matches_the_workspace_entry_point_twice_in_a_row():
    from llm_simple_b200 import ops
    ops.lib()
    calls = [
        ([4096, 1024, 2500, 3333, 4000, 1500, 2047, 4095], 31),  # up to 9 splits per sequence
        ([700, 64, 1, 0, 1300], 47),                              # shorter: fewer splits than the scratch still holds
    ]
    for lens, seed in calls:
        got, got_k, got_v = _one_step(ops, lens, seed, use_noalloc=True)
        want, want_k, want_v = _one_step(ops, lens, seed, use_noalloc=False)
        diff = np.abs(got - want)
        assert np.all(np.isfinite(got))
        assert diff.max() <= MAX_ABS and diff.mean() <= MEAN_ABS, (diff.max(), diff.mean())
        # both entry points appended the same rotated K and raw V
        assert np.array_equal(got_k, want_k) and np.array_equal(got_v, want_v)


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
