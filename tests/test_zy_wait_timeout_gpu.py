"""Failure detection of the peer-memory exchange without any fault: on ONE GPU the
exchange kernel is told it has a peer whose buffer is a second local allocation that
nobody ever writes, so the flag it waits for never arrives.  Every wait in the library's
kernels is bounded: after about a second the merge blocks give up, record which rank they
were waiting for in the status word, leave their output rows unwritten and return; the
context stays usable.  (Runs late in the suite and clears the status word again, because
other tests assert that it is zero.)"""
import numpy as np
import pytest
import torch

from tests.gpu_util import BF16, D

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows", [8, 5])     # whole groups of four rows with 16-byte copies; a ragged group, unaligned slots
def test_exchange_wait_runs_out_and_reports(tmp_path, rows):
    from llm_simple_b200 import ops
    ops.lib()
    assert ops.gpu_ops_kernel_status() == 0
    world, rank = 2, 0
    nbytes = ops.gpu_attn_xchg_buffer_bytes(world, rows)
    local = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    silent_peer = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")       # stands in for rank 1; never written
    epoch = 1
    slot = ops.gpu_attn_xchg_local_slot(local.data_ptr(), world, rank, epoch, rows)
    part = torch.cat([torch.randn(rows * D, device="cuda"), torch.zeros(rows, device="cuda")]).float()
    # this rank's partial goes where the decode step would have put it
    off = slot - local.data_ptr()
    local[off:off + part.numel() * 4] = part.view(torch.uint8)
    out = torch.full((rows, D), 7.0, dtype=torch.bfloat16, device="cuda")
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    ops.gpu_attn_xchg_merge_layer(out, local.data_ptr(), [None, silent_peer.data_ptr()], world, rank, epoch, rows, D, BF16)
    t1.record()
    torch.cuda.synchronize()                      # returns: the kernel ended by itself
    try:
        ms = t0.elapsed_time(t1)
        assert 200.0 < ms < 5000.0, "the bounded wait took %.0f ms" % ms
        assert ops.gpu_ops_kernel_status() == 20 + 1          # gave up waiting for rank 1
        assert bool((out == 7.0).all())                       # no row was written from incomplete data
        # the push half of the kernel did its work: the silent peer's buffer now holds this rank's partial and flags
        peer_slot = silent_peer[off:off + part.numel() * 4].view(torch.float32)
        assert torch.equal(peer_slot, part)
        # and the context is intact: an ordinary launch still works
        x = torch.arange(1024, device="cuda").float()
        assert float((x * 2).sum()) == float(np.arange(1024).sum() * 2)
    finally:
        ops.gpu_ops_clear_kernel_status()
    assert ops.gpu_ops_kernel_status() == 0
