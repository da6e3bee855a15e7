"""CPU checks of the multi-rank host logic with gloo, world_size 2: the head and
position partitions, and the (O, LSE) exchange protocol -- per-rank partials
packed exactly as the GPU path packs them, all-gathered, merged -- against
attention over the whole cache."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from llm_simple_b200 import sharding
from oracle import oracle as orc

D = 128


def test_kv_head_range_and_position_slices():
    assert [sharding.kv_head_range(8, 4, r) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    with pytest.raises(ValueError):
        sharding.kv_head_range(2, 4, 0)
    s = sharding.position_slices(10, 4)
    assert s == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert sharding.position_slices(2, 4) == [(0, 1), (1, 2), (2, 2), (2, 2)]   # empty slices are legal
    for total in (0, 1, 32768, 32769):
        sl = sharding.position_slices(total, 8)
        assert sl[0][0] == 0 and sl[-1][1] == total and all(a[1] == b[0] for a, b in zip(sl, sl[1:]))
    assert sharding.packed_partial_floats(40) == 40 * 129


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _partial(q_r, k, v, lo, hi, H, kvh, dt):
    """Normalised attention of one token over positions [lo, hi) and its natural-log LSE per head."""
    g = H // kvh
    n = hi - lo
    if n == 0:
        return np.zeros((H, D), np.float32), np.full(H, -np.inf, np.float32)
    o = orc.attn(q_r, k[lo:hi], v[lo:hi], 1, n, n - 1, g, kvh, D, dt, orc.MODE_GOLDEN).reshape(H, D)
    lse = np.empty(H, np.float32)
    for h in range(H):
        qh = q_r.reshape(1, H, D)[:, h, :]
        kh = np.ascontiguousarray(k[lo:hi].reshape(n, kvh, D)[:, h // g, :])
        s, _ = orc.scores_one_head(qh, kh, 1, n, n - 1, D, dt, orc.MODE_GOLDEN)
        m = s.max()
        lse[h] = m + np.log(np.exp(s - m).sum())
    return o, lse


def _rank_main(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dt, H, kvh, total = orc.DT_BFLOAT16, 10, 2, 301
        rng = np.random.default_rng(5)                      # same data on every rank
        q = orc.to_bits(rng.standard_normal((1, H * D), dtype=np.float32), dt)
        k = orc.to_bits(rng.standard_normal((total, kvh * D), dtype=np.float32), dt)
        v = orc.to_bits(rng.standard_normal((total, kvh * D), dtype=np.float32), dt)
        lo, hi = sharding.position_slices(total, world)[rank]
        o, lse = _partial(q, k, v, lo, hi, H, kvh, dt)
        n = sharding.packed_partial_floats(H)
        send = torch.from_numpy(np.concatenate([o.reshape(-1), lse]).astype(np.float32))
        assert send.numel() == n
        recv = torch.empty(world * n, dtype=torch.float32)
        dist.all_gather_into_tensor(recv, send)
        parts = recv.numpy().reshape(world, n)
        o_p = parts[:, :H * D].reshape(world, H, D)
        lse_p = parts[:, H * D:]
        m = lse_p.max(axis=0)
        w = np.exp(lse_p - m)                               # out = sum_p e^(lse_p - M) o_p / sum_p e^(lse_p - M)
        merged = (w[:, :, None] * o_p).sum(axis=0) / w.sum(axis=0)[:, None]
        full = orc.attn(q, k, v, 1, total, total - 1, H // kvh, kvh, D, dt, orc.MODE_GOLDEN).reshape(H, D)
        ret[rank] = float(np.abs(merged - full).max())
    finally:
        dist.destroy_process_group()


def test_partial_exchange_over_gloo_two_ranks_equals_full_attention():
    world, port = 2, _free_port()
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_rank_main, args=(world, port, ret), nprocs=world, join=True)
    assert len(ret) == world and all(err < 2e-6 for err in ret.values()), dict(ret)


def test_reshard_plan_pairs_up():
    """Every chunk one rank sends is a chunk its peer expects, in the same order."""
    lens, kvh, world = [10, 3, 0, 17], 4, 4
    plans = [sharding.reshard_plan(lens, kvh, world, r) for r in range(world)]
    per = kvh // world
    for a in range(world):
        for b in range(world):
            sent = [(seq, a * per + h, hi - lo) for (peer, seq, h, lo, hi) in plans[a][0] if peer == b]
            got = [(seq, gh, n) for (peer, seq, gh, n) in plans[b][1] if peer == a]
            assert sent == got
    # all positions of all heads are covered exactly once
    total = sum(hi - lo for pl in plans for (_, _, _, lo, hi) in pl[0])
    assert total == sum(lens) * kvh


def _reshard_rank(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        batch, kvh, max_pos, lens = 3, 4, 40, [37, 5, 1]
        rng = np.random.default_rng(9)                      # the same full cache on every rank
        full_k = rng.integers(0, 65536, size=(batch, kvh, max_pos, D)).astype(np.int16)
        full_v = rng.integers(0, 65536, size=(batch, kvh, max_pos, D)).astype(np.int16)
        lo_h, hi_h = sharding.kv_head_range(kvh, world, rank)
        k_src = torch.from_numpy(full_k[:, lo_h:hi_h].copy())
        v_src = torch.from_numpy(full_v[:, lo_h:hi_h].copy())
        cap = 20
        k_dst = torch.full((batch, kvh, cap, D), -1, dtype=torch.int16)
        v_dst = torch.full((batch, kvh, cap, D), -1, dtype=torch.int16)
        sharding.reshard_heads_to_positions(k_src, v_src, k_dst, v_dst, lens)
        ok = True
        for b, total in enumerate(lens):
            lo, hi = sharding.position_slices(total, world)[rank]
            n = hi - lo
            ok &= np.array_equal(k_dst[b, :, :n].numpy(), full_k[b, :, lo:hi])
            ok &= np.array_equal(v_dst[b, :, :n].numpy(), full_v[b, :, lo:hi])
            ok &= bool((k_dst[b, :, n:] == -1).all()) and bool((v_dst[b, :, n:] == -1).all())
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_reshard_heads_to_positions_two_ranks_gloo():
    world, port = 2, _free_port()
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_reshard_rank, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}
