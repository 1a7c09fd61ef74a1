"""Sharding of one attention call over the GPUs of a box: by (batch, head), with no traffic
between GPUs inside the operator. Every (batch, head) pair is independent in the forward and
in the backward (grid axes 1 and 2 of every reference kernel, flash_triton.py:47-48, :197-198,
:344-345); the query heads of one kv head stay on one rank so that dK/dV need no cross-rank sum.
Collectives (all_gather) are used only to assemble results for validation.
"""
import torch
import torch.distributed as dist


def shard_slices(B, H, Hk, world_size, rank, prefer="heads"):
    """Returns (dim, q_slice, kv_slice): the tensor dimension that is split (1 = heads,
    0 = batch) and this rank's slice of it for q-shaped and k/v-shaped tensors.
    With prefer="heads" the kv heads are split when they divide evenly, otherwise the batches;
    with prefer="batch" the other way round."""
    assert 0 <= rank < world_size
    assert H % Hk == 0
    G = H // Hk

    def by_heads():
        per = Hk // world_size
        return 1, slice(rank * per * G, (rank + 1) * per * G), slice(rank * per, (rank + 1) * per)

    def by_batch():
        per = B // world_size
        s = slice(rank * per, (rank + 1) * per)
        return 0, s, s

    order = [(Hk, by_heads), (B, by_batch)]
    if prefer == "batch":
        order.reverse()
    for extent, make in order:
        if extent % world_size == 0:
            return make()
    raise ValueError(f"cannot split B={B}, Hk={Hk} evenly over {world_size} ranks by head or by batch")


def take_shard(x, dim, sl):
    """This rank's part of a [B, H, L(, D)] tensor (a view; ids keep their head stride 0)."""
    return x[sl] if dim == 0 else x[:, sl]


def gather_shards(x_local, dim, group=None):
    """all_gather of the per-rank results along `dim` (validation only, outside any timed region)."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(x_local) for _ in range(world)]
    dist.all_gather(parts, x_local.contiguous(), group=group)
    return torch.cat(parts, dim=dim)
