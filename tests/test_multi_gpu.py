"""Two ranks, one GPU each (NCCL): KV-head sharding reproduces the single-device
result bit for bit with no collective on the data path, and decode over a cache
sharded by position (the one exchange: an all-gather of (O, LSE) partials) agrees
with the oracle.  Skipped when fewer than two GPUs are visible."""
import os
import socket

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import BF16, D, assert_parity, dev, host, rnd_bits

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _case():
    dt, H, kvh, neox, theta = BF16, 40, 8, True, 1e6
    lens = [1500, 700, 2047, 33]
    max_pos = 2056
    table = orc.init_freq_cis(D, max_pos, theta, dt)
    batch = len(lens)
    q = rnd_bits((batch, H * D), dt, 1)
    k, v = rnd_bits((batch, kvh * D), dt, 2), rnd_bits((batch, kvh * D), dt, 3)
    kc = rnd_bits((batch, kvh, max_pos, D), dt, 4)      # head-major
    vc = rnd_bits((batch, kvh, max_pos, D), dt, 5)
    return dt, H, kvh, neox, lens, max_pos, table, q, k, v, kc, vc


def _decode(ops, dt, H, kvh, neox, lens, max_pos, table, q, k, v, kc, vc):
    batch = len(lens)
    desc = ops.make_desc(dt, batch, H, kvh, 1, max_pos, layout="head", is_neox=neox)
    ws_bytes = ops.gpu_attn_decode_workspace_bytes(desc, max(lens) + 1)
    ws = torch.zeros(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    out = torch.empty((batch, H * D), dtype=torch.bfloat16, device="cuda")
    ops.gpu_attn_decode_layer(desc, out, None, None, dev(q, dt), dev(k, dt), dev(v, dt), dev(kc, dt), dev(vc, dt),
                              torch.from_numpy(table).cuda(), torch.tensor(lens, dtype=torch.int32, device="cuda"),
                              None, True, max(lens) + 1, ws, ws_bytes)
    torch.cuda.synchronize()
    return host(out)


def _rank_main(rank, world, port, ret):
    import torch.distributed as dist
    from llm_simple_b200 import ops, sharding
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dt, H, kvh, neox, lens, max_pos, table, q, k, v, kc, vc = _case()
        batch, g = len(lens), H // kvh
        # ---- (1) KV-head sharding: this rank's heads only, no collective on the data path
        lo, hi = sharding.kv_head_range(kvh, world, rank)
        qs = np.ascontiguousarray(q.reshape(batch, H, D)[:, lo * g:hi * g].reshape(batch, -1))
        ks = np.ascontiguousarray(k.reshape(batch, kvh, D)[:, lo:hi].reshape(batch, -1))
        vs = np.ascontiguousarray(v.reshape(batch, kvh, D)[:, lo:hi].reshape(batch, -1))
        mine = _decode(ops, dt, (hi - lo) * g, hi - lo, neox, lens, max_pos, table, qs, ks, vs,
                       np.ascontiguousarray(kc[:, lo:hi]), np.ascontiguousarray(vc[:, lo:hi]))
        mine_d = dev(mine, dt)
        gathered = [torch.empty_like(mine_d) for _ in range(world)]
        dist.all_gather(gathered, mine_d)                                         # test plumbing only
        sharded = np.concatenate([host(t).reshape(batch, -1, D) for t in gathered], axis=1)
        # ---- (2) cache sharded by position, one sequence, partial (O, LSE) exchange
        total_old = lens[0]
        sl_lo, sl_hi = sharding.position_slices(total_old, world)[rank]
        local_max = sl_hi - sl_lo + 8
        kl = np.zeros((1, kvh, local_max, D), np.uint16)
        vl = np.zeros((1, kvh, local_max, D), np.uint16)
        kl[0, :, :sl_hi - sl_lo], vl[0, :, :sl_hi - sl_lo] = kc[0, :, sl_lo:sl_hi], vc[0, :, sl_lo:sl_hi]
        desc = ops.make_desc(dt, 1, H, kvh, 1, local_max, layout="head", is_neox=neox)
        dec = sharding.SplitKVDecoder(desc, dt)
        ws_bytes = ops.gpu_attn_decode_workspace_bytes(desc, local_max)
        ws = torch.zeros(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
        out = torch.empty((1, H * D), dtype=torch.bfloat16, device="cuda")
        dec.step(out, dev(q[:1], dt), dev(k[:1], dt), dev(v[:1], dt), dev(kl, dt), dev(vl, dt),
                 torch.from_numpy(table).cuda(), torch.tensor([sl_hi - sl_lo], dtype=torch.int32, device="cuda"),
                 torch.tensor([total_old], dtype=torch.int32, device="cuda"), sl_hi - sl_lo, ws, ws_bytes)
        torch.cuda.synchronize()
        # the same step on the planned decode kernel (the slice length is known on the host)
        out_p = torch.empty((1, H * D), dtype=torch.bfloat16, device="cuda")
        dec.step_planned(out_p, dev(q[:1], dt), dev(k[:1], dt), dev(v[:1], dt), dev(kl, dt), dev(vl, dt),
                         torch.from_numpy(table).cuda(), sl_hi - sl_lo,
                         torch.tensor([total_old], dtype=torch.int32, device="cuda"))
        torch.cuda.synchronize()
        # and the planned kernel in front of the exchange over peer memory
        dec_peer = sharding.SplitKVDecoder(desc, dt, exchange="peer")
        out_pp = torch.empty((1, H * D), dtype=torch.bfloat16, device="cuda")
        dec_peer.step_planned(out_pp, dev(q[:1], dt), dev(k[:1], dt), dev(v[:1], dt), dev(kl, dt), dev(vl, dt),
                              torch.from_numpy(table).cuda(), sl_hi - sl_lo,
                              torch.tensor([total_old], dtype=torch.int32, device="cuda"))
        torch.cuda.synchronize()
        dec_peer.close()
        assert ops.gpu_ops_kernel_status() == 0
        ret[rank] = (sharded, host(out), host(out_p), host(out_pp))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_head_sharding_and_split_kv_exchange():
    import torch.multiprocessing as mp
    from llm_simple_b200 import ops
    world, port = 2, _free_port()
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_rank_main, args=(world, port, ret), nprocs=world, join=True)
    dt, H, kvh, neox, lens, max_pos, table, q, k, v, kc, vc = _case()
    single = _decode(ops, dt, H, kvh, neox, lens, max_pos, table, q, k, v, kc, vc)
    sharded0, split0, planned0, planned_peer0 = ret[0]
    sharded1, split1, planned1, planned_peer1 = ret[1]
    # head-sharded vs single device: same kernel on disjoint heads.  Where a head's cache is cut
    # between CTAs depends on how many heads share the device, so the sums may be ordered
    # differently: equal within the parity tolerance, and both ranks gathered the same bytes.
    assert np.array_equal(sharded0, sharded1)
    diff = np.abs(orc.to_f32(sharded0.reshape(single.shape), dt) - orc.to_f32(single, dt))
    assert diff.max() <= 1e-2 and diff.mean() <= 1e-3
    # position-sharded decode of sequence 0 vs the oracle; both ranks hold the full result
    kc_t = np.ascontiguousarray(kc[0].transpose(1, 0, 2)).reshape(max_pos, kvh * D)
    vc_t = np.ascontiguousarray(vc[0].transpose(1, 0, 2)).reshape(max_pos, kvh * D)
    L = lens[0]
    q_r = orc.rope_single_layer(q[:1], table, L, H, neox, dt)
    k_r = orc.rope_single_layer(k[:1], table, L, kvh, neox, dt)
    orc.kv_append(kc_t, vc_t, k_r, v[:1], L, kvh, D)
    gold = orc.attn(q_r, kc_t, vc_t, 1, L + 1, L, H // kvh, kvh, D, dt, orc.MODE_GOLDEN, threads=8)
    assert_parity(split0, gold, dt, "rank 0")
    assert np.array_equal(split0, split1)
    assert_parity(planned0, gold, dt, "rank 0, planned kernel")
    assert np.array_equal(planned0, planned1)
    # the two exchanges merge the same partials in the same order
    assert np.array_equal(planned_peer0, planned0) and np.array_equal(planned_peer1, planned0)


def _flow_case():
    dt, H, kvh, neox, theta, prompt = BF16, 40, 8, True, 1e6, 700
    max_pos = 768
    table = orc.init_freq_cis(D, max_pos, theta, dt)
    q = rnd_bits((prompt + 1, H * D), dt, 11)           # prompt rows, then the first generated token
    k, v = rnd_bits((prompt + 1, kvh * D), dt, 12), rnd_bits((prompt + 1, kvh * D), dt, 13)
    return dt, H, kvh, neox, prompt, max_pos, table, q, k, v


def _flow_rank(rank, world, port, ret):
    """Prompt prefilled with the cache sharded by KV head, cache re-sharded by position over
    NCCL, first token decoded over the position shards with the (O, LSE) exchange."""
    import torch.distributed as dist
    from llm_simple_b200 import ops, sharding
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dt, H, kvh, neox, prompt, max_pos, table, q, k, v = _flow_case()
        g = H // kvh
        lo, hi = sharding.kv_head_range(kvh, world, rank)
        kvh_l, H_l = hi - lo, (hi - lo) * g
        tab_d = torch.from_numpy(table).cuda()
        qs = np.ascontiguousarray(q[:prompt].reshape(prompt, H, D)[:, lo * g:hi * g].reshape(prompt, -1))
        ks = np.ascontiguousarray(k[:prompt].reshape(prompt, kvh, D)[:, lo:hi].reshape(prompt, -1))
        vs = np.ascontiguousarray(v[:prompt].reshape(prompt, kvh, D)[:, lo:hi].reshape(prompt, -1))
        desc_p = ops.make_desc(dt, 1, H_l, kvh_l, prompt, max_pos, layout="head", is_neox=neox)
        k_src = torch.zeros((1, kvh_l, max_pos, D), dtype=torch.bfloat16, device="cuda")
        v_src = torch.zeros_like(k_src)
        q_emb = torch.empty((prompt, H_l * D), dtype=torch.bfloat16, device="cuda")
        out_p = torch.empty_like(q_emb)
        ops.gpu_rope_kv_append_layer(desc_p, q_emb, k_src, v_src, dev(qs, dt), dev(ks, dt), dev(vs, dt), tab_d, None,
                                     0, prompt)
        ops.gpu_attn_prefill_layer(desc_p, out_p, q_emb, k_src, v_src, prompt, 0)
        # ---- head shards -> position shards
        sl_lo, sl_hi = sharding.position_slices(prompt, world)[rank]
        cap = sl_hi - sl_lo + 8
        k_dst = torch.zeros((1, kvh, cap, D), dtype=torch.bfloat16, device="cuda")
        v_dst = torch.zeros_like(k_dst)
        torch.cuda.synchronize()
        sharding.reshard_heads_to_positions(k_src, v_src, k_dst, v_dst, [prompt])
        torch.cuda.synchronize()
        # ---- first generated token over the position shards
        desc_d = ops.make_desc(dt, 1, H, kvh, 1, cap, layout="head", is_neox=neox)
        dec = sharding.SplitKVDecoder(desc_d, dt)
        ws_bytes = ops.gpu_attn_decode_workspace_bytes(desc_d, cap)
        ws = torch.zeros(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
        out = torch.empty((1, H * D), dtype=torch.bfloat16, device="cuda")
        dec.step(out, dev(q[prompt:], dt), dev(k[prompt:], dt), dev(v[prompt:], dt), k_dst, v_dst, tab_d,
                 torch.tensor([sl_hi - sl_lo], dtype=torch.int32, device="cuda"),
                 torch.tensor([prompt], dtype=torch.int32, device="cuda"), sl_hi - sl_lo, ws, ws_bytes)
        torch.cuda.synchronize()
        # ---- the same step with the exchange done by one kernel over peer memory: same bits, three
        #      steps in a row (both halves of the exchange buffer; the tail rank rewrites the same row)
        dec2 = sharding.SplitKVDecoder(desc_d, dt, exchange="peer")
        same = True
        for _ in range(3):
            out2 = torch.zeros_like(out)
            dec2.step(out2, dev(q[prompt:], dt), dev(k[prompt:], dt), dev(v[prompt:], dt), k_dst, v_dst, tab_d,
                      torch.tensor([sl_hi - sl_lo], dtype=torch.int32, device="cuda"),
                      torch.tensor([prompt], dtype=torch.int32, device="cuda"), sl_hi - sl_lo, ws, ws_bytes)
            torch.cuda.synchronize()
            same = same and torch.equal(out2.view(torch.int16), out.view(torch.int16))
        dec2.close()
        # ---- the two-call form: decode into this rank's slot, then the exchange kernel with push blocks
        pe = sharding.PeerExchange(H)
        tail = rank == world - 1
        for _ in range(2):
            slot = pe.next_slot()
            ops.gpu_attn_decode_layer(desc_d, None, slot, slot + H * D * 4, dev(q[prompt:], dt),
                                      dev(k[prompt:], dt) if tail else None, dev(v[prompt:], dt) if tail else None,
                                      k_dst, v_dst, tab_d, torch.tensor([sl_hi - sl_lo], dtype=torch.int32, device="cuda"),
                                      torch.tensor([prompt], dtype=torch.int32, device="cuda"), tail,
                                      sl_hi - sl_lo + (1 if tail else 0), ws, ws_bytes)
            out3 = torch.zeros_like(out)
            pe.merge(out3, D, dt)
            torch.cuda.synchronize()
            same = same and torch.equal(out3.view(torch.int16), out.view(torch.int16))
        dist.barrier()
        pe.close()
        same = same and ops.gpu_ops_kernel_status() == 0
        ret[rank] = (host(k_dst[0, :, :sl_hi - sl_lo]), host(v_dst[0, :, :sl_hi - sl_lo]), host(out), host(out_p), same)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_prefill_reshard_decode_flow():
    import torch.multiprocessing as mp
    from llm_simple_b200 import sharding
    world, port = 2, _free_port()
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_flow_rank, args=(world, port, ret), nprocs=world, join=True)
    dt, H, kvh, neox, prompt, max_pos, table, q, k, v = _flow_case()
    g = H // kvh
    k_rot = orc.rope_single_layer(k[:prompt], table, 0, kvh, neox, dt).reshape(prompt, kvh, D)
    q_rot = orc.rope_single_layer(q[:prompt], table, 0, H, neox, dt)
    gold_p = orc.attn(q_rot, k_rot.reshape(prompt, -1), v[:prompt], prompt, prompt, 0, g, kvh, D, dt, orc.MODE_GOLDEN,
                      threads=8).reshape(prompt, H, D)
    for r in range(world):
        lo, hi = sharding.position_slices(prompt, world)[r]
        k_got, v_got, _, out_p, peer_same = ret[r]
        assert peer_same, "peer-memory exchange differs from the all-gather path on rank %d" % r
        # the re-sharded slices hold exactly the rotated K and the raw V of their positions, all heads
        assert np.array_equal(k_got, k_rot[lo:hi].transpose(1, 0, 2))
        assert np.array_equal(v_got, v[lo:hi].reshape(hi - lo, kvh, D).transpose(1, 0, 2))
        h_lo, h_hi = sharding.kv_head_range(kvh, world, r)
        assert_parity(out_p, gold_p[:, h_lo * g:h_hi * g].reshape(prompt, -1), dt, "prefill rank %d" % r)
    # the decoded token equals attention over the whole prompt + itself
    kc_t = np.zeros((prompt + 1, kvh * D), np.uint16)
    vc_t = np.zeros((prompt + 1, kvh * D), np.uint16)
    kc_t[:prompt], vc_t[:prompt] = k_rot.reshape(prompt, -1), v[:prompt]
    q_r = orc.rope_single_layer(q[prompt:], table, prompt, H, neox, dt)
    k_r = orc.rope_single_layer(k[prompt:], table, prompt, kvh, neox, dt)
    orc.kv_append(kc_t, vc_t, k_r, v[prompt:], prompt, kvh, D)
    gold = orc.attn(q_r, kc_t, vc_t, 1, prompt + 1, prompt, g, kvh, D, dt, orc.MODE_GOLDEN, threads=8)
    assert_parity(ret[0][2], gold, dt, "decode after re-shard, rank 0")
    assert np.array_equal(ret[0][2], ret[1][2])
