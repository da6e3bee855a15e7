"""Work partitioning of the attention path across the GPUs of one node, one
process per GPU (torch.distributed / NCCL for the plumbing).

Two partitions exist (the reference itself is single-device, so neither has a
counterpart there):

* by KV head: rank r owns KV heads [r*kvH/P, (r+1)*kvH/P) and their query
  heads -- of Q, of the cache and of the output columns.  Heads are independent
  in every formula of the path, so there is no collective.
* by cache position, for decode over very long contexts: rank r holds a
  contiguous slice of every sequence's positions, attends over it and returns a
  normalised partial output with its log-sum-exp; the partials are all-gathered
  into local memory and merged locally (gpu_attn_merge_packed_layer).  The owner
  of the tail slice appends the new token.

Moving from the first partition (how a prompt is prefilled) to the second (how a
very long context is decoded) is one exchange: reshard_heads_to_positions().
"""


def kv_head_range(n_kv_heads, world, rank):
    """[lo, hi) of the KV heads owned by `rank`."""
    if n_kv_heads % world:
        raise ValueError("%d KV heads do not divide over %d ranks" % (n_kv_heads, world))
    per = n_kv_heads // world
    return rank * per, (rank + 1) * per


def position_slices(total_len, world):
    """Contiguous [lo, hi) slices of `total_len` cached positions, one per rank,
    sizes differing by at most one; the last rank owns the tail (and the append)."""
    base, extra = divmod(total_len, world)
    out, lo = [], 0
    for r in range(world):
        hi = lo + base + (1 if r < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


def packed_partial_floats(rows, head_dim=128):
    """Floats one rank contributes to the (O, LSE) exchange: rows*head_dim outputs
    followed by rows log-sum-exps."""
    return rows * (head_dim + 1)


def reshard_plan(kv_lens, n_kv_heads, world, rank):
    """Chunks that move when a cache sharded by KV head becomes a cache sharded by position.

    Returns (sends, recvs).  A send is (peer, seq, local_head, lo, hi): positions [lo, hi) of
    one of this rank's heads, which `peer` owns after the exchange.  A recv is (peer, seq,
    head, n): n positions of global KV head `head` arriving from its old owner, stored at
    local positions [0, n).  Both lists are ordered by (peer, seq, head), the order in which
    the two sides post their transfers, so that they pair up."""
    h_lo, h_hi = kv_head_range(n_kv_heads, world, rank)
    per = h_hi - h_lo
    sends, recvs = [], []
    for peer in range(world):
        for b, total in enumerate(kv_lens):
            sl = position_slices(int(total), world)
            lo, hi = sl[peer]
            if hi > lo:
                for h in range(per):
                    sends.append((peer, b, h, lo, hi))
            mine = sl[rank][1] - sl[rank][0]
            if mine > 0:
                for h in range(per):
                    recvs.append((peer, b, peer * per + h, mine))
    return sends, recvs


def reshard_heads_to_positions(k_src, v_src, k_dst, v_dst, kv_lens, group=None):
    """Head-sharded caches -> position-sharded caches, in place in the destination tensors.

    k_src / v_src  [batch][kvH/P][max_pos][D]: this rank's KV heads, all positions (the layout a
                   head-sharded prefill leaves behind)
    k_dst / v_dst  [batch][kvH][cap][D]: all KV heads, this rank's position slice
                   (position_slices(kv_lens[b], P)[rank]) stored from local position 0
    kv_lens        cached positions per sequence, the same list on every rank
    Every chunk (one head, one sequence, one destination) is contiguous on both sides, so the
    exchange is a group of point-to-point transfers straight between the caches, with no staging
    copy; the chunk a rank keeps is a local copy.  Works on CUDA tensors (NCCL) and on CPU
    tensors (gloo)."""
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    n_kv_heads = k_dst.shape[1]
    if k_src.shape[1] * world != n_kv_heads:
        raise ValueError("source holds %d heads per rank, destination %d heads, %d ranks"
                         % (k_src.shape[1], n_kv_heads, world))
    sends, recvs = reshard_plan(kv_lens, n_kv_heads, world, rank)
    ops_list = []
    local = [(b, h, lo, hi) for (peer, b, h, lo, hi) in sends if peer == rank]
    for src, dst in ((k_src, k_dst), (v_src, v_dst)):
        for peer, b, h, lo, hi in sends:
            if peer != rank:
                ops_list.append(dist.P2POp(dist.isend, src[b, h, lo:hi], _global_rank(dist, group, peer), group))
        for peer, b, gh, n in recvs:
            if peer != rank:
                if n > dst.shape[2]:
                    raise ValueError("slice of %d positions does not fit a destination of %d" % (n, dst.shape[2]))
                ops_list.append(dist.P2POp(dist.irecv, dst[b, gh, :n], _global_rank(dist, group, peer), group))
        per = k_src.shape[1]
        for b, h, lo, hi in local:
            dst[b, rank * per + h, :hi - lo].copy_(src[b, h, lo:hi])
    if ops_list:
        for req in dist.batch_isend_irecv(ops_list):
            req.wait()


def _global_rank(dist, group, group_rank):
    return group_rank if group is None else dist.get_global_rank(group, group_rank)


class PeerExchange:
    """This rank's exchange buffer for the peer-memory (O, LSE) exchange, and its peers' buffers
    mapped into this process (CUDA IPC; one process per GPU of one node).  The 64-byte handles
    travel once, at construction, through the process group."""

    def __init__(self, rows, group=None):
        import torch.distributed as dist
        from . import ops
        self.ops, self.rows = ops, rows
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        nbytes = ops.gpu_attn_xchg_buffer_bytes(self.world, rows)
        self.local, handle = ops.gpu_peer_buffer_alloc(nbytes)
        handles = [None] * self.world
        dist.all_gather_object(handles, handle, group=group)
        self.peers = [self.local if r == self.rank else ops.gpu_peer_buffer_open(handles[r])
                      for r in range(self.world)]
        self.epoch = 0
        dist.barrier(group)          # every buffer exists and is zero before anyone pushes

    def next_slot(self):
        """Starts a step: returns the device address where this rank's packed partial of the step
        belongs (rows*128 fp32 outputs, then rows log-sum-exps)."""
        self.epoch += 1
        return self.ops.gpu_attn_xchg_local_slot(self.local, self.world, self.rank, self.epoch, self.rows)

    def merge(self, out, head_dim, dt, stream=None):
        self.ops.gpu_attn_xchg_merge_layer(out, self.local, self.peers, self.world, self.rank, self.epoch, self.rows,
                                           head_dim, dt, stream)

    def close(self):
        """Call on every rank, after a barrier that follows the last step."""
        for r, p in enumerate(self.peers):
            if r != self.rank and p:
                self.ops.gpu_peer_buffer_close(p)
        self.peers = []
        if self.local:
            self.ops.gpu_peer_buffer_free(self.local)
            self.local = None


class SplitKVDecoder:
    """Decode step over a cache sharded by position across the ranks of `group`.

    Each rank calls step() with its local slice of the cache; the result (all
    query heads, every rank gets the full output) is written to `out`."""

    def __init__(self, desc, dt, group=None, exchange="nccl"):
        """exchange: "nccl" = all-gather into local memory, then a merge kernel; "peer" = one kernel
        per rank that pushes its partial into the peers' buffers over NVLink, waits for theirs and
        merges (PeerExchange).  Both give the same bits."""
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.desc, self.dt, self.group = desc, dt, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.rows = desc.batch * desc.n_heads
        n = packed_partial_floats(self.rows, desc.head_dim)
        self.peer = None
        if exchange == "peer":
            self.peer = PeerExchange(self.rows, group)
        elif exchange == "nccl":
            self.send = torch.empty(n, dtype=torch.float32, device="cuda")
            self.recv = torch.empty(self.world * n, dtype=torch.float32, device="cuda")
        else:
            raise ValueError("exchange must be 'nccl' or 'peer'")

    def step(self, out, q_in, k_in, v_in, k_cache, v_cache, freqs_cis, local_len_dev, rope_pos_dev, max_local_len,
             workspace, workspace_bytes):
        from . import ops
        tail = self.rank == self.world - 1
        max_len = max_local_len + (1 if tail else 0)
        if self.peer:
            # two launches: the decode kernel, then the kernel that merges this rank's splits, pushes
            # the rows to the peers, waits for theirs and merges
            pe = self.peer
            pe.epoch += 1
            ops.gpu_attn_decode_xchg_layer(self.desc, out, q_in, k_in if tail else None, v_in if tail else None,
                                           k_cache, v_cache, freqs_cis, local_len_dev, rope_pos_dev, tail, max_len,
                                           workspace, workspace_bytes, pe.local, pe.peers, pe.world, pe.rank, pe.epoch)
            return
        o_ptr = self.send.data_ptr()
        lse_ptr = o_ptr + self.rows * self.desc.head_dim * 4
        ops.gpu_attn_decode_layer(self.desc, None, o_ptr, lse_ptr, q_in, k_in if tail else None,
                                  v_in if tail else None, k_cache, v_cache, freqs_cis, local_len_dev, rope_pos_dev,
                                  tail, max_len, workspace, workspace_bytes)
        self.dist.all_gather_into_tensor(self.recv, self.send, group=self.group)
        ops.gpu_attn_merge_packed_layer(out, self.recv, self.world, self.rows, self.desc.head_dim, self.dt)

    def step_planned(self, out, q_in, k_in, v_in, k_cache, v_cache, freqs_cis, local_len, rope_pos_dev, plan=None,
                     workspace=None):
        """The same step on the planned decode kernel (gpu_attn_decode_planned_layer): the length of this rank's
        slice is known on the host (a serving loop hands out the slices), so the work partition is built from it
        and the kernel writes (O, LSE) of every query row straight into the all-gather send buffer or, with the
        peer exchange, into this rank's slot of the exchange buffer.  `plan` / `workspace`: pass the ones of an
        earlier call with the same local_len to skip rebuilding them (returned by every call)."""
        from . import ops
        tail = self.rank == self.world - 1
        if plan is None:
            plan = ops.DecodePlan(self.desc, [int(local_len)] * self.desc.batch, tail)
            plan.upload()
        if workspace is None:
            workspace = self.torch.empty(max(plan.workspace_bytes, 16), dtype=self.torch.uint8, device="cuda")
        if self.peer:
            pe = self.peer
            pe.epoch += 1
            o_ptr = ops.gpu_attn_xchg_local_slot(pe.local, pe.world, pe.rank, pe.epoch, self.rows)
            lse_ptr = o_ptr + self.rows * self.desc.head_dim * 4
            ops.gpu_attn_decode_planned_layer(self.desc, None, plan, None, o_ptr, lse_ptr, q_in, k_in if tail else None,
                                              v_in if tail else None, k_cache, v_cache, freqs_cis, rope_pos_dev,
                                              workspace, plan.workspace_bytes)
            ops.gpu_attn_xchg_merge_layer(out, pe.local, pe.peers, pe.world, pe.rank, pe.epoch, self.rows,
                                          self.desc.head_dim, self.dt)
            return plan, workspace
        o_ptr = self.send.data_ptr()
        lse_ptr = o_ptr + self.rows * self.desc.head_dim * 4
        ops.gpu_attn_decode_planned_layer(self.desc, None, plan, None, o_ptr, lse_ptr, q_in, k_in if tail else None,
                                          v_in if tail else None, k_cache, v_cache, freqs_cis, rope_pos_dev, workspace,
                                          plan.workspace_bytes)
        self.dist.all_gather_into_tensor(self.recv, self.send, group=self.group)
        ops.gpu_attn_merge_packed_layer(out, self.recv, self.world, self.rows, self.desc.head_dim, self.dt)
        return plan, workspace

    def close(self):
        if self.peer:
            self.dist.barrier(self.group)
            self.peer.close()
            self.peer = None
