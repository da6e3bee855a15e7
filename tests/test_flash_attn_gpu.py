"""GPU parity of the reference-shaped attention operators through the C ABI,
against the oracle in both modes.  Same golden math and shape flags as
tests/flash_attn_test.cpp / tests/flash_attn_main.cpp (m, n, offset, head_num,
head_dim), plus bf16, GQA and decode shapes, with seeded N(0,1) inputs."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import BF16, D, FP16, assert_parity, dev, host, rnd_bits

pytestmark = pytest.mark.gpu

ATTN_FIXTURES = [
    "fa_fp16_m16_n16_o0_h2", "fa_fp16_m7_n300_o293_h3", "fa_fp16_m1_n65_o64_h4", "fa_fp16_m1_n1_o0_h2",
    "fa_fp16_m130_n130_o0_h1", "fa_bf16_gqa_m5_n40_o35_g3_kv2", "fa_bf16_gqa_m1_n129_o128_g6_kv2",
    "fa_bf16_gqa_m33_n97_o64_g5_kv1",
]


@pytest.fixture(scope="module")
def ops():
    from llm_simple_b200 import ops as o
    o.lib()
    return o


@pytest.fixture(params=[1, 2, 3], ids=["mma", "tcgen05", "tcgen05-persistent"])
def prefill_kernel(request, ops):
    ops.gpu_attn_set_prefill_kernel(request.param)
    yield request.param
    ops.gpu_attn_set_prefill_kernel(0)
    # no device-side wait gave up (every wait in the tcgen05 kernel is bounded and reports here)
    assert ops.gpu_ops_kernel_status() == 0


def run_gqa(ops, q, k, v, m, n, offset, g, kvh, dt):
    out = torch.empty((m, g * kvh * D), dtype=dev(q, dt).dtype, device="cuda")
    ops.gpu_flash_attn_gqa_layer(out, dev(q, dt), dev(k, dt), dev(v, dt), m, n, offset, g, kvh, D, dt)
    torch.cuda.synchronize()
    return host(out)


@pytest.mark.parametrize("name", ATTN_FIXTURES)
def test_golden_fixtures(ops, golden, prefill_kernel, name):
    dt, m, n, offset, g, kvh, d = [int(x) for x in golden[name + "/meta"]]
    got = run_gqa(ops, golden[name + "/q"], golden[name + "/k"], golden[name + "/v"], m, n, offset, g, kvh, dt)
    assert_parity(got, golden[name + "/o"], dt, name)


SHAPES = [  # (m, n, offset)
    (256, 256, 0),     # Llama-2-7B-shaped prefill
    (1, 1, 0),
    (1, 512, 511),     # decode
    (7, 300, 293),     # the reference's {1, 7} row counts
    (128, 128, 0),
    (129, 257, 128),
    (64, 64, 0),
    (200, 1000, 800),  # chunk with history, ragged against every tile size
]


@pytest.mark.parametrize("m,n,offset", SHAPES)
@pytest.mark.parametrize("heads", [32, 3])
def test_flash_attn_layer_fp16_mha(ops, prefill_kernel, m, n, offset, heads):
    if heads == 32 and n > 512:
        pytest.skip("kept small for the CPU oracle")
    dt = FP16
    q, k, v = rnd_bits((m, heads * D), dt, 1), rnd_bits((n, heads * D), dt, 2), rnd_bits((n, heads * D), dt, 3)
    out = torch.empty((m, heads * D), dtype=torch.float16, device="cuda")
    ops.gpu_flash_attn_layer(out, dev(q, dt), dev(k, dt), dev(v, dt), m, n, offset, heads, D, dt)
    torch.cuda.synchronize()
    got = host(out)
    gold = orc.attn(q, k, v, m, n, offset, 1, heads, D, dt, orc.MODE_GOLDEN, threads=8)
    strict = orc.attn(q, k, v, m, n, offset, 1, heads, D, dt, orc.MODE_STRICT, threads=8)
    assert_parity(got, gold, dt, "vs fp32 golden")
    assert_parity(got, orc.to_f32(strict, dt), dt, "vs strict layer mode")
    # the reference tests' own verdict at their own tolerance (tests/npu_op_test_util.h:38-39), on the fp32 golden
    assert orc.all_close(orc.to_f32(got, dt), gold, 1e-3, 1e-3)


@pytest.mark.parametrize("m,n,offset", SHAPES)
@pytest.mark.parametrize("g,kvh", [(6, 2), (5, 8), (1, 8)])
@pytest.mark.parametrize("dt", [BF16, FP16])
def test_flash_attn_gqa_layer(ops, prefill_kernel, m, n, offset, g, kvh, dt):
    if dt == FP16 and (g, kvh) != (5, 8):
        pytest.skip("fp16 GQA covered by one group shape")
    q = rnd_bits((m, g * kvh * D), dt, 4)
    k, v = rnd_bits((n, kvh * D), dt, 5), rnd_bits((n, kvh * D), dt, 6)
    got = run_gqa(ops, q, k, v, m, n, offset, g, kvh, dt)
    gold = orc.attn(q, k, v, m, n, offset, g, kvh, D, dt, orc.MODE_GOLDEN, threads=8)
    assert_parity(got, gold, dt)


def test_opt_prefill_layer_is_the_same_operator(ops):
    m, n, offset, heads, dt = 40, 72, 32, 4, FP16
    q, k, v = rnd_bits((m, heads * D), dt, 7), rnd_bits((n, heads * D), dt, 8), rnd_bits((n, heads * D), dt, 9)
    a = torch.empty((m, heads * D), dtype=torch.float16, device="cuda")
    b = torch.empty_like(a)
    ops.gpu_flash_attn_layer(a, dev(q, dt), dev(k, dt), dev(v, dt), m, n, offset, heads, D, dt)
    ops.gpu_flash_attn_opt_prefill_layer(b, dev(q, dt), dev(k, dt), dev(v, dt), m, n, offset, heads, D, dt)
    torch.cuda.synchronize()
    assert torch.equal(a, b)


def test_decode_shape_with_registered_workspace_matches_unsplit(ops):
    """m = 1 over a long cache: split across CTAs when scratch is registered."""
    m, n, g, kvh, dt = 1, 3000, 6, 2, BF16
    q = rnd_bits((m, g * kvh * D), dt, 10)
    k, v = rnd_bits((n, kvh * D), dt, 11), rnd_bits((n, kvh * D), dt, 12)
    unsplit = run_gqa(ops, q, k, v, m, n, n - 1, g, kvh, dt)
    ws = torch.empty(8 << 20, dtype=torch.uint8, device="cuda")
    ops.gpu_ops_set_workspace(ws, ws.numel())
    ops.gpu_attn_set_decode_chunk(256)
    try:
        before = ops.gpu_ops_launch_count(True)
        split = run_gqa(ops, q, k, v, m, n, n - 1, g, kvh, dt)
        assert ops.gpu_ops_launch_count() == 2  # split kernel + merge
    finally:
        ops.gpu_attn_set_decode_chunk(0)
        ops.gpu_ops_set_workspace(None, 0)
    gold = orc.attn(q, k, v, m, n, n - 1, g, kvh, D, dt, orc.MODE_GOLDEN, threads=8)
    assert_parity(unsplit, gold, dt, "unsplit")
    assert_parity(split, gold, dt, "split")


def test_deterministic(ops, prefill_kernel):
    m, n, heads, dt = 300, 300, 4, FP16
    q, k, v = rnd_bits((m, heads * D), dt, 13), rnd_bits((n, heads * D), dt, 14), rnd_bits((n, heads * D), dt, 15)
    outs = []
    for _ in range(2):
        out = torch.empty((m, heads * D), dtype=torch.float16, device="cuda")
        ops.gpu_flash_attn_layer(out, dev(q, dt), dev(k, dt), dev(v, dt), m, n, 0, heads, D, dt)
        torch.cuda.synchronize()
        outs.append(host(out))
    assert np.array_equal(outs[0], outs[1])


def test_output_canary_rows_untouched(ops, prefill_kernel):
    """The op writes exactly m rows of H*D elements."""
    m, n, heads, dt = 70, 70, 2, FP16
    q, k, v = rnd_bits((m, heads * D), dt, 16), rnd_bits((n, heads * D), dt, 17), rnd_bits((n, heads * D), dt, 18)
    buf = torch.full((m + 2, heads * D), 123.0, dtype=torch.float16, device="cuda")
    ops.gpu_flash_attn_layer(buf[1:], dev(q, dt), dev(k, dt), dev(v, dt), m, n, 0, heads, D, dt)
    torch.cuda.synchronize()
    assert torch.all(buf[0] == 123.0) and torch.all(buf[m + 1] == 123.0)


def test_rejects_bad_arguments(ops):
    x = torch.zeros(4, 256, dtype=torch.float16, device="cuda")
    for args in [(0, 4, 0, 2, 128, FP16), (4, 0, 0, 2, 128, FP16), (4, 4, -1, 2, 128, FP16),
                 (4, 4, 0, 2, 64, FP16), (4, 4, 0, 2, 128, 6)]:
        with pytest.raises(ops.GpuOpsError):
            ops.gpu_flash_attn_layer(x, x, x, x, *args)
    with pytest.raises(ops.GpuOpsError):
        ops.gpu_flash_attn_layer(None, x, x, x, 4, 4, 0, 2, 128, FP16)


def test_prefill_over_more_positions_than_a_sequence_caches_is_rejected(ops):
    """Two sequences with caches of 128 positions: a prefill over 120 + 16 positions would read the neighbour's."""
    H, kvh, max_pos, m = 4, 2, 128, 16
    desc = ops.make_desc(FP16, 2, H, kvh, m, max_pos, layout="head")
    q = torch.zeros((2, m, H * 128), dtype=torch.float16, device="cuda")
    cache = torch.zeros((2, kvh, max_pos, 128), dtype=torch.float16, device="cuda")
    ops.gpu_attn_prefill_layer(desc, torch.empty_like(q), q, cache, cache, m, max_pos - m)    # fits exactly
    with pytest.raises(ops.GpuOpsError, match="do not fit the cache"):
        ops.gpu_attn_prefill_layer(desc, torch.empty_like(q), q, cache, cache, m, max_pos - m + 8)
    t = torch.zeros((2, 2), dtype=torch.int32, device="cuda")                                   # 2 pages of 64 per sequence
    pool = torch.zeros((4, kvh, 64, 128), dtype=torch.float16, device="cuda")
    with pytest.raises(ops.GpuOpsError, match="page table rows"):
        ops.gpu_attn_prefill_paged_layer(desc, ops.make_pages(t, 64, kvh * 64 * 128, 4), torch.empty_like(q), q, pool,
                                         pool, m, max_pos - m + 8)
