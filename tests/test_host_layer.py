"""CPU checks of the host layer: the pool policy of GPUAllocator (reference:
NPUAllocator, src/device_npu.cpp:22-67) on a host-memory backend, and the RoPE
table builder against the oracle's restatement of ModelBase::InitFreqCIS."""
import numpy as np
import pytest

from oracle import oracle as orc


@pytest.fixture()
def pool():
    from llm_simple_b200 import layer
    L = layer.lib()
    L.gpu_allocator_use_host_backend(1)
    L.gpu_allocator_set_limit(64 << 30)
    yield layer
    L.gpu_allocator_trim()
    L.gpu_allocator_use_host_backend(0)
    L.gpu_allocator_set_limit(64 << 30)


def test_freed_block_is_reused_and_smallest_fit_wins(pool):
    L = pool.lib()
    a = L.gpu_allocator_allocate(1000)      # rounded to 1024
    b = L.gpu_allocator_allocate(5000)      # 5120
    c = L.gpu_allocator_allocate(100000)
    assert len({a, b, c}) == 3
    s = pool.allocator_stats()
    assert s["backend_allocs"] == 3 and s["pooled_bytes"] == 0
    for p in (a, b, c):
        L.gpu_allocator_deallocate(p)
    s = pool.allocator_stats()
    assert s["pooled_bytes"] == s["backend_bytes"] == 1024 + 5120 + 100352
    # 3000 bytes: the 5120 block is the smallest that fits (the reference scans its size-sorted list)
    assert L.gpu_allocator_allocate(3000) == b
    assert L.gpu_allocator_allocate(900) == a
    assert L.gpu_allocator_allocate(900) == c   # only c is left and it fits
    s = pool.allocator_stats()
    assert s["pool_hits"] == 3 and s["backend_allocs"] == 3 and s["pooled_bytes"] == 0


def test_pool_is_trimmed_smallest_first_when_over_the_limit(pool):
    L = pool.lib()
    L.gpu_allocator_set_limit(300000)
    small = L.gpu_allocator_allocate(4096)
    mid = L.gpu_allocator_allocate(65536)
    big = L.gpu_allocator_allocate(200000)
    for p in (small, mid, big):
        L.gpu_allocator_deallocate(p)
    assert pool.allocator_stats()["backend_frees"] == 0
    # nothing pooled fits 250000: a new backend block pushes the total over the limit,
    # pooled blocks are released in ascending size until it is back under
    L.gpu_allocator_allocate(250000)
    s = pool.allocator_stats()
    assert s["backend_frees"] == 3 and s["pooled_bytes"] == 0
    assert s["backend_bytes"] == 250368


def test_trim_releases_everything_pooled(pool):
    L = pool.lib()
    ptrs = [L.gpu_allocator_allocate(n) for n in (512, 2048, 1 << 20)]
    for p in ptrs:
        L.gpu_allocator_deallocate(p)
    L.gpu_allocator_trim()
    s = pool.allocator_stats()
    assert s["pooled_bytes"] == 0 and s["backend_bytes"] == 0 and s["backend_frees"] == 3


@pytest.mark.parametrize("theta,dt", [(1e4, orc.DT_FLOAT16), (1e6, orc.DT_BFLOAT16), (1e6, orc.DT_FLOAT16)])
def test_init_freq_cis_is_bit_identical_to_the_oracle(theta, dt):
    from llm_simple_b200 import layer
    got = layer.init_freq_cis(128, 4100, theta, dt)
    want = orc.init_freq_cis(128, 4100, theta, dt)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_layer_rejects_positions_beyond_its_cache_before_any_launch(pool):
    """Every forward entry point checks prev_pos / cur_pos against the cache the layer was
    created for on the host, before a copy or a kernel is enqueued: a prefill that would append
    beyond the cache must not reach the device (the kernels carry no cache extent)."""
    table = np.zeros((64, 64, 2), dtype=np.float32)
    lay = pool.AttentionLayer(pool.QWEN2, 4, 2, 64, 2, orc.DT_BFLOAT16, 1e6, True, shared_freq_cis=table.ctypes.data)
    try:
        L = pool.lib()
        buf = np.zeros(1 << 20, dtype=np.uint8)
        p = buf.ctypes.data
        # cur_pos 65 > max_seq_len 64: prefill of 65 tokens, and a decode step at position 64
        for cur_pos, prev_pos in ((65, 0), (65, 64)):
            assert L.gpu_attention_layer_forward_host(lay.h, p, p, 1, cur_pos, prev_pos, None, None) == -1
            assert L.gpu_attention_layer_forward(lay.h, p, p, p, p, 1, cur_pos, prev_pos, None) == -1
            assert L.gpu_attention_layer_forward_fused(lay.h, p, p, None, 1, cur_pos, prev_pos, None, None) == -1
        # batch beyond max_batch, negative start
        assert L.gpu_attention_layer_forward_host(lay.h, p, p, 3, 8, 0, None, None) == -1
        assert L.gpu_attention_layer_forward_host(lay.h, p, p, 1, 8, -1, None, None) == -1
    finally:
        lay.close()


def test_kv_cache_layout_helper():
    from llm_simple_b200 import layer, ops
    d = ops.AttnDesc()
    assert layer.kv_cache_layout(d, layer.TOKEN_MAJOR, 8, 4096) == 8 * 4096 * 128
    assert (d.cache_seq_stride, d.cache_head_stride, d.cache_pos_stride) == (8 * 4096 * 128, 128, 8 * 128)
    assert layer.kv_cache_layout(d, layer.HEAD_MAJOR, 8, 4096) == 8 * 4096 * 128
    assert (d.cache_seq_stride, d.cache_head_stride, d.cache_pos_stride) == (8 * 4096 * 128, 4096 * 128, 128)
    ref = ops.make_desc(ops.DT_BFLOAT16, 1, 40, 8, 1, 4096, layout="head")
    assert (ref.cache_head_stride, ref.cache_pos_stride) == (d.cache_head_stride, d.cache_pos_stride)
    assert layer.kv_cache_layout(d, 2, 8, 4096) == 0
