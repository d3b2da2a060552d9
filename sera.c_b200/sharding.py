"""KV-head sharding of the attention path across the GPUs of one box.

Attention is independent per KV head (kv_head = head / 8,
ref: src/q3_forward.cu:228-229), so rank r of n owns KV heads
[r*Hkv/n, (r+1)*Hkv/n) and the 8 query heads of each; the only exchange is an
all-gather of the per-head outputs at the layer boundary. The reference is
single-device; this module is the whole multi-GPU host logic of the path.
"""
import torch
import torch.distributed as dist

GROUP = 8  # query heads per KV head


def head_shard(rank, world, n_kv_heads=8):
    """(kv_begin, kv_count, q_begin, q_count) of a rank."""
    if world < 1 or n_kv_heads % world:
        raise ValueError("world size %d does not divide %d KV heads" % (world, n_kv_heads))
    if not 0 <= rank < world:
        raise ValueError("rank %d outside world %d" % (rank, world))
    kv = n_kv_heads // world
    return rank * kv, kv, rank * kv * GROUP, kv * GROUP


def slice_heads(q, k, v, rank, world):
    """Per-rank slices of full-geometry q [T,H,D], k, v [T,Hkv,D]."""
    kb, kc, qb, qc = head_shard(rank, world, k.shape[1])
    return (q[:, qb:qb + qc].contiguous(), k[:, kb:kb + kc].contiguous(),
            v[:, kb:kb + kc].contiguous())


def all_gather_heads(out_local, gathered, group=None, async_op=False):
    """All-gather [T, H/n, D] shards into `gathered` [n, T, H/n, D]. Returns the
    work handle when async_op, so the next layer's attention can overlap it."""
    return dist.all_gather_into_tensor(gathered.view(-1), out_local.view(-1),
                                       group=group, async_op=async_op)


def gathered_to_full(gathered):
    """[n, T, H/n, D] -> [T, H, D] (a copy; a consumer that can read the
    rank-major layout, such as a column-sharded o_proj, does not need it)."""
    n, T, h, D = gathered.shape
    return gathered.permute(1, 0, 2, 3).reshape(T, n * h, D)


class PeerGather:
    """Gathered output buffers in symmetric memory for the per-layer exchange of
    q3_suffix_attention_layer_gathered.

    Each rank owns `depth` buffers [n, T, H/n, D] and one flag array per
    buffer; `peers(i)` returns the descriptor (peer-mapped base pointers of all
    ranks) the C ABI takes. The attention kernel writes this rank's slot of its
    own buffer; copy-engine copies (cudaMemcpyAsync over NVLink, no SM) push
    that slot into the other ranks' buffers and a one-thread kernel publishes
    the flags. Nothing loads from a peer: ranks only write to peers and read
    their own memory.
    """

    def __init__(self, tokens, n_heads_local, head_dim, dtype, device, group=None, depth=2):
        import torch.distributed._symmetric_memory as symm_mem
        from . import GatherPeers
        group = group or dist.group.WORLD
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks (one box)")
        self.shape = (self.world, tokens, n_heads_local, head_dim)
        self.depth = depth
        self.bufs, self.flags, self._desc, self._handles = [], [], [], []
        for _ in range(depth):
            buf = symm_mem.empty(self.shape, dtype=dtype, device=device)
            flg = symm_mem.empty((64,), dtype=torch.int32, device=device)
            buf.zero_()
            flg.zero_()
            hb = symm_mem.rendezvous(buf, group)
            hf = symm_mem.rendezvous(flg, group)
            d = GatherPeers()
            d.n_ranks, d.rank = self.world, self.rank
            for r in range(self.world):
                d.gathered[r] = hb.buffer_ptrs[r]
                d.flags[r] = hf.buffer_ptrs[r]
            self.bufs.append(buf)
            self.flags.append(flg)
            self._desc.append(d)
            self._handles += [hb, hf]
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def peers(self, i):
        return self._desc[i % self.depth]

    def full(self, i):
        """[T, H, D] view-copy of buffer i (after the wait for its layer)."""
        return gathered_to_full(self.bufs[i % self.depth])
