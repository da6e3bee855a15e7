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


class SplitKVDecoder:
    """Decode step over a cache sharded by position across the ranks of `group`.

    Each rank calls step() with its local slice of the cache; the result (all
    query heads, every rank gets the full output) is written to `out`."""

    def __init__(self, desc, dt, group=None):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.desc, self.dt, self.group = desc, dt, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.rows = desc.batch * desc.n_heads
        n = packed_partial_floats(self.rows, desc.head_dim)
        self.send = torch.empty(n, dtype=torch.float32, device="cuda")
        self.recv = torch.empty(self.world * n, dtype=torch.float32, device="cuda")

    def step(self, out, q_in, k_in, v_in, k_cache, v_cache, freqs_cis, local_len_dev, rope_pos_dev, max_local_len,
             workspace, workspace_bytes):
        from . import ops
        tail = self.rank == self.world - 1
        o_ptr = self.send.data_ptr()
        lse_ptr = o_ptr + self.rows * self.desc.head_dim * 4
        ops.gpu_attn_decode_layer(self.desc, None, o_ptr, lse_ptr, q_in, k_in if tail else None,
                                  v_in if tail else None, k_cache, v_cache, freqs_cis, local_len_dev, rope_pos_dev,
                                  tail, max_local_len + (1 if tail else 0), workspace, workspace_bytes)
        self.dist.all_gather_into_tensor(self.recv, self.send, group=self.group)
        ops.gpu_attn_merge_packed_layer(out, self.recv, self.world, self.rows, self.desc.head_dim, self.dt)
