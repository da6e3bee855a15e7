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
