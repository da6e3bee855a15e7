"""GPU parity of the operators that take a FUSED q|k|v projection row: the plain
split (npu_split_qkv_layer, prebuild/npu_ops.h:27-30) and the pass that splits,
adds the projection bias, rotates and appends in one read of the row.  Bit-exact
against the oracle (split -> bias_add -> rope_single_layer -> kv_append) and
against the unfused operator on pre-split inputs."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import BF16, D, FP16, dev, host, rnd_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from llm_simple_b200 import ops as o
    o.lib()
    return o


@pytest.mark.parametrize("dt", [FP16, BF16])
@pytest.mark.parametrize("rows,H,kvH", [(1, 12, 2), (37, 40, 8), (4096, 40, 8), (0, 4, 4)])
def test_split_qkv_bit_exact(ops, dt, rows, H, kvH):
    qd, kd = H * D, kvH * D
    qkv = rnd_bits((rows, qd + 2 * kd), dt, 11)
    want = orc.split_qkv(qkv, qd, kd, kd)
    qkv_d = dev(qkv, dt) if rows else torch.empty((0, qd + 2 * kd), dtype=torch.float16, device="cuda")
    outs = [torch.full((max(rows, 1), n), 7.0, dtype=qkv_d.dtype, device="cuda") for n in (qd, kd, kd)]
    ops.gpu_split_qkv_layer(outs[0], outs[1], outs[2], qkv_d, rows, qd, kd, kd, dt)
    torch.cuda.synchronize()
    for o, w in zip(outs, want):
        if rows:
            assert np.array_equal(host(o), w)
        else:
            assert float(o.float().min()) == 7.0          # nothing written


@pytest.mark.parametrize("dt", [FP16, BF16])
@pytest.mark.parametrize("rows,width,pad", [(1, 7168, 0), (64, 7168, 0), (5, 256, 128)])
def test_bias_add_bit_exact(ops, dt, rows, width, pad):
    buf = rnd_bits((rows, width + pad), dt, 31)
    bias = rnd_bits((width,), dt, 32)
    want = buf.copy()
    want[:, :width] = orc.bias_add(buf[:, :width], bias, dt)
    x = dev(buf, dt)
    ops.gpu_bias_add_layer(x, x, dev(bias, dt), rows, width, width + pad, dt)   # in place
    torch.cuda.synchronize()
    assert np.array_equal(host(x), want)            # padding columns untouched


def test_split_qkv_rejects_bad_arguments(ops):
    x = torch.zeros(4, 384, dtype=torch.float16, device="cuda")
    o = torch.zeros(4, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(ops.GpuOpsError):
        ops.gpu_split_qkv_layer(o, o, o, x, 4, 100, 128, 156, FP16)       # not multiples of 128
    with pytest.raises(ops.GpuOpsError):
        ops.gpu_split_qkv_layer(o, o, o, x, 4, 128, 128, 128, 6)          # fp32
    with pytest.raises(ops.GpuOpsError):
        ops.gpu_split_qkv_layer(o, o, o, x, -1, 128, 128, 128, FP16)


@pytest.mark.parametrize("dt,neox,theta", [(FP16, False, 1e4), (BF16, True, 1e6)])
@pytest.mark.parametrize("layout", ["token", "head"])
@pytest.mark.parametrize("with_bias", [False, True])
@pytest.mark.parametrize("batch,m,H,kvH,pad", [(1, 256, 32, 32, 0), (3, 5, 12, 2, 64), (8, 1, 40, 8, 0), (5, 1001, 3, 1, 128)])
def test_fused_qkv_rope_kv_append(ops, dt, neox, theta, layout, with_bias, batch, m, H, kvH, pad):
    max_pos = max(320, m + 64)
    qd, kd = H * D, kvH * D
    width = qd + 2 * kd
    row = width + pad                             # a padded row stride must be honoured
    rng = np.random.default_rng(batch * 1000 + m)
    starts = rng.integers(0, max_pos - m + 1, size=batch).astype(np.int32)
    table = orc.init_freq_cis(D, max_pos, theta, dt)
    buf = rnd_bits((batch, m, row), dt, 21)
    qkv = np.ascontiguousarray(buf[..., :width])
    bias = rnd_bits((width,), dt, 22) if with_bias else None
    canary = np.uint16(0x7BCD)
    desc = ops.make_desc(dt, batch, H, kvH, m, max_pos, layout=layout, is_neox=neox)
    shape = (batch, kvH, max_pos, D) if layout == "head" else (batch, max_pos, kvH, D)
    kc_d, vc_d = dev(np.full(shape, canary, np.uint16), dt), dev(np.full(shape, canary, np.uint16), dt)
    buf_d = dev(buf, dt)
    qo_d = torch.empty((batch, m, qd), dtype=buf_d.dtype, device="cuda")
    tab_d = torch.from_numpy(table).cuda()
    starts_d = torch.from_numpy(starts).cuda()
    ops.gpu_qkv_rope_kv_append_layer(desc, qo_d, kc_d, vc_d, buf_d, m * row, row,
                                     dev(bias, dt) if with_bias else None, tab_d, starts_d, 0, m)
    torch.cuda.synchronize()
    got_q, got_k, got_v = host(qo_d), host(kc_d), host(vc_d)
    for b in range(batch):
        s = int(starts[b])
        x = orc.bias_add(qkv[b], bias, dt) if with_bias else qkv[b]
        q, k, v = orc.split_qkv(x, qd, kd, kd)
        wq = orc.rope_single_layer(q, table, s, H, neox, dt)
        wk = orc.rope_single_layer(k, table, s, kvH, neox, dt)
        assert np.array_equal(got_q[b], wq)
        want_k = np.full((max_pos, kd), canary, np.uint16)
        want_v = np.full((max_pos, kd), canary, np.uint16)
        orc.kv_append(want_k, want_v, wk, v, s, kvH, D)
        if layout == "head":
            want_k = want_k.reshape(max_pos, kvH, D).transpose(1, 0, 2)
            want_v = want_v.reshape(max_pos, kvH, D).transpose(1, 0, 2)
        assert np.array_equal(got_k[b].reshape(want_k.shape), want_k)
        assert np.array_equal(got_v[b].reshape(want_v.shape), want_v)
    if not with_bias:
        # the unfused operator on pre-split tensors writes the same bits
        q, k, v = orc.split_qkv(qkv, qd, kd, kd)
        kc2, vc2 = dev(np.full(shape, canary, np.uint16), dt), dev(np.full(shape, canary, np.uint16), dt)
        qo2 = torch.empty_like(qo_d)
        ops.gpu_rope_kv_append_layer(desc, qo2, kc2, vc2, dev(q, dt), dev(k, dt), dev(v, dt), tab_d, starts_d, 0, m)
        torch.cuda.synchronize()
        assert torch.equal(qo2.view(torch.int16), qo_d.view(torch.int16))
        assert torch.equal(kc2.view(torch.int16), kc_d.view(torch.int16))
        assert torch.equal(vc2.view(torch.int16), vc_d.view(torch.int16))


def test_fused_qkv_rejects_bad_strides(ops):
    desc = ops.make_desc(FP16, 1, 4, 2, 2, 16)
    x = torch.zeros(2, 1024, dtype=torch.float16, device="cuda")
    kc = torch.zeros(2, 16, 128, dtype=torch.float16, device="cuda")
    tab = torch.zeros(16, 64, 2, device="cuda")
    with pytest.raises(ops.GpuOpsError):
        ops.gpu_qkv_rope_kv_append_layer(desc, x, kc, kc, x, 2048, 1000, None, tab, None, 0, 2)  # row narrower than q|k|v
    assert "row" in ops.last_error_string()
