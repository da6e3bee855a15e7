"""GPU parity of the attention section of the layer classes (the host layer
that mirrors Llamma2TransformerLayerNPUImpl / Qwen2TransformerLayerNPUImpl,
src/llama2_layer_npu.cpp:283-374 and :780-869) against the oracle run the way
the reference's layer runs: rope -> append -> attention, prefill then decode."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import BF16, D, FP16, assert_parity, dev, host, rnd_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def layer():
    from llm_simple_b200 import layer as lay
    lay.lib()
    return lay


def oracle_layer_steps(q, k, v, H, kvh, prompt, table, neox, dt):
    """Prefill of `prompt` tokens, then one token per step: returns golden [n][H*D]."""
    n = q.shape[0]
    q_r = orc.rope_single_layer(q, table, 0, H, neox, dt)
    k_r = orc.rope_single_layer(k, table, 0, kvh, neox, dt)
    return orc.attn(q_r, k_r, v, n, n, 0, H // kvh, kvh, D, dt, orc.MODE_GOLDEN, threads=8)


@pytest.mark.parametrize("kind,H,kvh,dt,neox,theta", [
    ("llama2", 8, 8, FP16, False, 1e4),      # Llama-2 flavour: MHA, fp16, interleaved pairs
    ("qwen2", 12, 2, BF16, True, 1e6),       # Qwen2.5-1.5B heads
])
@pytest.mark.parametrize("layout", ["token", "head"])
def test_prefill_then_decode_steps(layer, kind, H, kvh, dt, neox, theta, layout):
    prompt, steps, max_seq = 150, 5, 256
    n = prompt + steps
    lay = layer.AttentionLayer(layer.LLAMA2 if kind == "llama2" else layer.QWEN2, H, kvh, max_seq, 1, dt, theta,
                               neox, layer.TOKEN_MAJOR if layout == "token" else layer.HEAD_MAJOR)
    table = orc.init_freq_cis(D, max_seq, theta, dt)
    q, k, v = rnd_bits((n, H * D), dt, 1), rnd_bits((n, kvh * D), dt, 2), rnd_bits((n, kvh * D), dt, 3)
    gold = oracle_layer_steps(q, k, v, H, kvh, prompt, table, neox, dt)
    tdt = dev(q[:1], dt).dtype
    out_p = torch.empty((prompt, H * D), dtype=tdt, device="cuda")
    lay.forward(out_p, dev(q[:prompt], dt), dev(k[:prompt], dt), dev(v[:prompt], dt), 1, prompt, 0)
    torch.cuda.synchronize()
    assert_parity(host(out_p), gold[:prompt], dt, "prefill")
    out_d = torch.empty((1, H * D), dtype=tdt, device="cuda")
    for s in range(steps):
        pos = prompt + s
        lay.forward(out_d, dev(q[pos:pos + 1], dt), dev(k[pos:pos + 1], dt), dev(v[pos:pos + 1], dt), 1, pos + 1,
                    pos)
        torch.cuda.synchronize()
        assert_parity(host(out_d)[0], gold[pos], dt, "decode step %d" % s)
    lay.close()


def test_ragged_batched_decode_and_host_buffers(layer):
    """Qwen2.5-14B heads, ragged lengths; device-pointer and host-buffer entries agree with the oracle."""
    H, kvh, dt, neox, theta = 40, 8, BF16, True, 1e6
    lens = [700, 64, 1300, 5]
    batch, max_seq = len(lens), 1400
    table = orc.init_freq_cis(D, max_seq, theta, dt)
    kc = rnd_bits((batch, max_seq, kvh * D), dt, 4)
    vc = rnd_bits((batch, max_seq, kvh * D), dt, 5)
    q = rnd_bits((batch, H * D), dt, 6)
    k, v = rnd_bits((batch, kvh * D), dt, 7), rnd_bits((batch, kvh * D), dt, 8)

    def head_major(x):
        return np.ascontiguousarray(x.reshape(batch, max_seq, kvh, D).transpose(0, 2, 1, 3))

    gold = []
    for b in range(batch):
        kb, vb = kc[b].copy(), vc[b].copy()
        q_r = orc.rope_single_layer(q[b:b + 1], table, lens[b], H, neox, dt)
        k_r = orc.rope_single_layer(k[b:b + 1], table, lens[b], kvh, neox, dt)
        orc.kv_append(kb, vb, k_r, v[b:b + 1], lens[b], kvh, D)
        gold.append(orc.attn(q_r, kb, vb, 1, lens[b] + 1, lens[b], H // kvh, kvh, D, dt, orc.MODE_GOLDEN,
                             threads=8)[0])
    for entry in ("device", "host"):
        kc_d, vc_d = dev(head_major(kc), dt), dev(head_major(vc), dt)   # caller-owned cache memory, adopted
        lay = layer.AttentionLayer(layer.QWEN2, H, kvh, max_seq, batch, dt, theta, neox, layer.HEAD_MAJOR,
                                   k_cache=kc_d, v_cache=vc_d)
        if entry == "device":
            out = torch.empty((batch, H * D), dtype=torch.bfloat16, device="cuda")
            lay.decode_ragged(out, dev(q, dt), dev(k, dt), dev(v, dt), lens)
            torch.cuda.synchronize()
            got = host(out)
        else:
            qkv = np.concatenate([q, k, v], axis=1)                      # one packed projection row per sequence
            qkv_h = torch.from_numpy(qkv.view(np.int16)).pin_memory()
            out_h = torch.empty((batch, H * D), dtype=torch.int16).pin_memory()
            lay.forward_host(out_h, qkv_h, batch, 1, 0, kv_len=lens)
            torch.cuda.synchronize()
            got = out_h.numpy().view(np.uint16)
        for b in range(batch):
            assert_parity(got[b], gold[b], dt, "%s entry, seq %d" % (entry, b))
        lay.close()


def test_host_buffer_prefill_matches_device_prefill(layer):
    H, kvh, dt, neox, theta, m, max_seq = 8, 4, FP16, False, 1e4, 140, 256
    q, k, v = rnd_bits((m, H * D), dt, 9), rnd_bits((m, kvh * D), dt, 10), rnd_bits((m, kvh * D), dt, 11)
    a = layer.AttentionLayer(layer.QWEN2, H, kvh, max_seq, 1, dt, theta, neox)
    b = layer.AttentionLayer(layer.QWEN2, H, kvh, max_seq, 1, dt, theta, neox)
    out = torch.empty((m, H * D), dtype=torch.float16, device="cuda")
    a.forward(out, dev(q, dt), dev(k, dt), dev(v, dt), 1, m, 0)
    qkv_h = torch.from_numpy(np.concatenate([q, k, v], axis=1).view(np.int16)).pin_memory()
    out_h = torch.empty((m, H * D), dtype=torch.int16).pin_memory()
    b.forward_host(out_h, qkv_h, 1, m, 0)
    torch.cuda.synchronize()
    assert np.array_equal(host(out), out_h.numpy().view(np.uint16))
    a.close()
    b.close()


def test_host_buffer_calls_back_to_back_equal_the_strictly_ordered_ones(layer):
    """A prompt and eight one-token steps through forward_host without a synchronisation in between (the
    input copies run ahead on the layer's own stream and reuse one staging buffer) give the bits of
    the same calls with the copies on the caller's stream and a synchronisation after each."""
    H, kvh, dt, neox, theta, m, max_seq, steps = 12, 2, BF16, True, 1e6, 200, 256, 8
    width = (H + 2 * kvh) * D
    rows = [rnd_bits((m, width), dt, 70)] + [rnd_bits((1, width), dt, 71 + i) for i in range(steps)]
    ins = [torch.from_numpy(r.view(np.int16)).pin_memory() for r in rows]
    results = []
    side = torch.cuda.Stream()
    for overlap in (True, False):
        k_c = torch.zeros((1, kvh, max_seq, D), dtype=torch.bfloat16, device="cuda")   # caller-owned, adopted
        v_c = torch.zeros_like(k_c)
        lay = layer.AttentionLayer(layer.QWEN2, H, kvh, max_seq, 1, dt, theta, neox, layer.HEAD_MAJOR,
                                   k_cache=k_c, v_cache=v_c)
        lay.set_host_copy_overlap(overlap)
        outs = [torch.zeros((r.shape[0], H * D), dtype=torch.int16).pin_memory() for r in rows]
        pos = 0
        for x, o in zip(ins, outs):
            lay.forward_host(o, x, 1, pos + x.shape[0], pos, stream=side if overlap else None)
            pos += x.shape[0]
            if not overlap:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        results.append(([o.numpy().copy() for o in outs], host(k_c).copy(), host(v_c).copy()))
        lay.close()
    for a, b in zip(results[0][0], results[1][0]):
        assert np.array_equal(a, b)
    assert np.array_equal(results[0][1], results[1][1]) and np.array_equal(results[0][2], results[1][2])


@pytest.mark.parametrize("with_bias", [False, True])
def test_fused_projection_row_prefill_then_decode(layer, with_bias):
    """forward_fused on a packed q|k|v row (+ bias row) equals forward on the split, biased tensors bit for bit:
    prefill of a prompt, then ragged one-token steps of a batch of 3."""
    H, kvh, dt, neox, theta, max_seq, batch = 12, 2, BF16, True, 1e6, 256, 3
    width = (H + 2 * kvh) * D
    bias = rnd_bits((width,), dt, 40) if with_bias else None
    a = layer.AttentionLayer(layer.QWEN2, H, kvh, max_seq, batch, dt, theta, neox)
    b = layer.AttentionLayer(layer.QWEN2, H, kvh, max_seq, batch, dt, theta, neox)
    bias_d = dev(bias, dt) if with_bias else None

    def split_biased(rows):
        x = orc.bias_add(rows, bias, dt) if with_bias else rows
        return orc.split_qkv(x, H * D, kvh * D, kvh * D)

    m = 130
    rows = rnd_bits((batch, m, width), dt, 41)
    q, k, v = split_biased(rows)
    out_a = torch.empty((batch, m, H * D), dtype=torch.bfloat16, device="cuda")
    out_b = torch.empty_like(out_a)
    a.forward(out_a, dev(q, dt), dev(k, dt), dev(v, dt), batch, m, 0)
    b.forward_fused(out_b, dev(rows, dt), bias_d, batch, m, 0)
    torch.cuda.synchronize()
    assert torch.equal(out_a.view(torch.int16), out_b.view(torch.int16))
    lens = np.array([m, m, m], dtype=np.int32)
    for step in range(3):
        rows = rnd_bits((batch, 1, width), dt, 50 + step)
        q, k, v = split_biased(rows)
        o_a = torch.empty((batch, H * D), dtype=torch.bfloat16, device="cuda")
        o_b = torch.empty_like(o_a)
        a.decode_ragged(o_a, dev(q, dt), dev(k, dt), dev(v, dt), lens)
        b.forward_fused(o_b, dev(rows, dt), bias_d, batch, int(lens[0]) + 1, int(lens[0]), kv_len=lens)
        torch.cuda.synchronize()
        assert torch.equal(o_a.view(torch.int16), o_b.view(torch.int16)), "decode step %d" % step
        lens = lens + 1
    a.close()
    b.close()


def test_pooled_temporaries_are_recycled(layer):
    """A freed device block goes back to GPUAllocator's pool and serves the next request of that size."""
    L = layer.lib()
    L.gpu_allocator_trim()                     # start from an empty pool on this device
    size = 3 << 20
    p1 = L.gpu_allocator_allocate(size)
    assert p1
    L.gpu_allocator_deallocate(p1)
    before = layer.allocator_stats()
    p2 = L.gpu_allocator_allocate(size)
    after = layer.allocator_stats()
    assert p2 == p1 and after["pool_hits"] == before["pool_hits"] + 1
    assert after["backend_allocs"] == before["backend_allocs"]
    L.gpu_allocator_deallocate(p2)
    L.gpu_allocator_trim()
    assert layer.allocator_stats()["pooled_bytes"] == 0
