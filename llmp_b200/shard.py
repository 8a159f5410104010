"""One-box partitioning of the quantized products (host logic over
torch.distributed; NCCL on GPUs, gloo in the CPU tests).

Two partitionings, the ones the reference declares as data
(src/components/ffn.cc:67-81 columns; src/components/moe.cc:521-531 experts;
src/planner/partition.h:39-67) and whose collectives are IR ops there
(src/ir/op.h:246-250 kAllGather, kAllToAll):

* N-column sharding: rank r owns a contiguous range of every weight matrix's
  output rows (whole blocks run along K, so any row split is exact; MXFP8
  shards are multiples of 128 rows so that scale atoms split cleanly); the
  activations are replicated and the output shards all-gathered.
* Expert parallelism: rank r owns a contiguous range of whole experts; each
  (token, slot) row travels to its expert's owner (all-to-all), is computed
  there, travels back (all-to-all) and is combined on the token's home rank in
  slot order, so the weighted sum keeps the single-device order of additions.

Nothing here touches device memory layouts or launches kernels itself: the
expert computation is a callable the caller supplies (llmp_b200.moe_ffn on a
GPU; the CPU oracle in the tests).
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def row_shard(n: int, world: int, rank: int, multiple: int = 1) -> tuple[int, int]:
    """Rows [begin, end) of rank `rank`: `n` rows in units of `multiple`, split as evenly
    as whole units allow (the first ranks take the extra unit)."""
    if n % multiple != 0:
        raise ValueError(f"{n} rows are not whole units of {multiple}")
    units = n // multiple
    base, extra = divmod(units, world)
    begin = rank * base + min(rank, extra)
    end = begin + base + (1 if rank < extra else 0)
    return begin * multiple, end * multiple


def shard_rows(weights: torch.Tensor, world: int, rank: int, multiple: int = 1) -> torch.Tensor:
    """The rank's rows of a [n, row_bytes] block matrix (a view)."""
    b, e = row_shard(weights.shape[0], world, rank, multiple)
    return weights[b:e]


def all_gather_rows(shard: torch.Tensor, sizes: list[int], group=None) -> torch.Tensor:
    """All-gathers per-rank output shards [tokens, n_r] into [tokens, sum n_r] (rank order =
    row order).  Equal shards take one all_gather_into_tensor; ragged ones a list gather."""
    world = dist.get_world_size(group)
    tokens = shard.shape[0]
    if len(set(sizes)) == 1:
        full = torch.empty((world * tokens, sizes[0]), dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(full, shard.contiguous(), group=group)
        return full.view(world, tokens, sizes[0]).permute(1, 0, 2).reshape(tokens,
                                                                            world * sizes[0])
    parts = [torch.empty((tokens, s), dtype=shard.dtype, device=shard.device) for s in sizes]
    dist.all_gather(parts, shard.contiguous(), group=group)
    return torch.cat(parts, dim=1)


def expert_range(experts: int, world: int, rank: int) -> tuple[int, int]:
    return row_shard(experts, world, rank)


def expert_owner(ids: torch.Tensor, experts: int, world: int) -> torch.Tensor:
    """The rank owning each expert id (ids outside the experts map to rank 0 and are
    computed as NaN rows by the combine, as on one device)."""
    base, extra = divmod(experts, world)
    # ranks [0, extra) own base + 1 experts, the rest own base
    split = extra * (base + 1)
    ids = ids.clamp(0, experts - 1)
    low = ids // (base + 1) if base + 1 > 0 else torch.zeros_like(ids)
    high = extra + (ids - split) // max(base, 1)
    return torch.where(ids < split, low, high).to(torch.int64)


def ep_moe_ffn(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, experts: int,
               local_compute: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
               group=None) -> torch.Tensor:
    """Expert-parallel routed block.  x [tokens, hidden] (this rank's tokens), ids I32
    [tokens, used], weights F32 [tokens, used].  local_compute(rows [r, hidden], local expert
    ids I32 [r]) -> [r, hidden_out] runs this rank's experts on the rows it received.
    Returns [tokens, hidden_out]: sum over slots in slot order of row * weight."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    tokens, used = ids.shape
    slots = tokens * used
    flat = ids.reshape(-1)
    valid = (flat >= 0) & (flat < experts)
    owner = expert_owner(flat, experts, world)
    order = torch.sort(owner, stable=True).indices            # slots grouped by destination
    send_counts = torch.bincount(owner, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    send_split = send_counts.tolist()
    recv_split = recv_counts.tolist()
    rows_out = x[(order // used)].contiguous()
    begin, _ = expert_range(experts, world, 0)
    starts = torch.tensor([expert_range(experts, world, r)[0] for r in range(world)],
                          device=flat.device)
    local_ids = (flat.clamp(0, experts - 1) - starts[owner]).to(torch.int32)[order].contiguous()
    rows_in = torch.empty((sum(recv_split), x.shape[1]), dtype=x.dtype, device=x.device)
    ids_in = torch.empty((sum(recv_split),), dtype=torch.int32, device=x.device)
    dist.all_to_all_single(rows_in, rows_out, recv_split, send_split, group=group)
    dist.all_to_all_single(ids_in, local_ids, recv_split, send_split, group=group)
    y_in = local_compute(rows_in, ids_in) if rows_in.shape[0] > 0 else \
        torch.empty((0, 0), dtype=torch.float32, device=x.device)
    width = torch.tensor([y_in.shape[1] if rows_in.shape[0] > 0 else 0], device=x.device)
    dist.all_reduce(width, op=dist.ReduceOp.MAX, group=group)
    width = int(width.item())
    if rows_in.shape[0] == 0:
        y_in = torch.empty((0, width), dtype=torch.float32, device=x.device)
    y_back = torch.empty((slots, width), dtype=y_in.dtype, device=x.device)
    dist.all_to_all_single(y_back, y_in.contiguous(), send_split, recv_split, group=group)
    y = torch.empty_like(y_back)
    y[order] = y_back                                          # back to slot order
    y = y.view(tokens, used, width)
    nan = torch.full((), float("nan"), dtype=y.dtype, device=y.device)
    y = torch.where(valid.view(tokens, used, 1), y, nan)
    out = y[:, 0] * weights[:, 0:1]
    for j in range(1, used):                                   # slot order, as on one device
        out = out + y[:, j] * weights[:, j:j + 1]
    del rank, begin
    return out


# ------------------------------------------------------------------ fixed-capacity form
def ep_capacity(tokens: int, used: int, world: int, factor: float = 1.25, multiple: int = 128) -> int:
    """Rows a rank may send to one destination in a step: the mean load tokens * used / world
    times `factor`, rounded up to `multiple`.  Sizes are then known before the step, so nothing
    of the exchange waits on the host."""
    mean = -(-tokens * used // world)
    return max(multiple, -(-int(mean * factor) // multiple) * multiple)


def pack_reference(x, ids, experts: int, world: int, capacity: int):
    """What llmp_b200.moe_ep_pack computes, in plain torch (the CPU tests' stand-in): each
    (token, slot) row goes to lane i of its expert's owner, i counting that owner's rows in
    (token, slot) order.  Returns send rows [world * capacity, hidden], send ids I32 [world *
    capacity] (the local expert id, -1 for an unused lane), home I32 [tokens * used] (the
    row's index world * capacity-wide, -1 for an id outside the experts or a row past the
    capacity) and the number of rows dropped for capacity."""
    tokens, used = ids.shape
    per = experts // world
    flat = ids.reshape(-1).to(torch.int64)
    valid = (flat >= 0) & (flat < experts)
    owner = torch.where(valid, flat // per, torch.zeros_like(flat))
    send = torch.zeros((world * capacity, x.shape[1]), dtype=x.dtype, device=x.device)
    send_ids = torch.full((world * capacity,), -1, dtype=torch.int32, device=x.device)
    home = torch.full((tokens * used,), -1, dtype=torch.int32, device=x.device)
    count = [0] * world
    dropped = 0
    for s in range(tokens * used):
        if not bool(valid[s]):
            continue
        r = int(owner[s])
        i = count[r]
        count[r] += 1
        if i >= capacity:
            dropped += 1
            continue
        send[r * capacity + i] = x[s // used]
        send_ids[r * capacity + i] = int(flat[s]) - r * per
        home[s] = r * capacity + i
    return send, send_ids, home, dropped


def ep_moe_ffn_padded(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, experts: int,
                      capacity: int, pack: Callable, local_compute: Callable, combine: Callable,
                      group=None) -> torch.Tensor:
    """Expert-parallel routed block with exchanges of fixed size (no value reaches the host):
    pack(x, ids) -> (send rows [world * capacity, hidden], send ids I32 [world * capacity],
    home I32 [tokens * used]); an all-to-all of equal splits carries lane block r to rank r;
    local_compute(rows, local ids with -1 for unused lanes) -> [world * capacity, hidden_out]
    runs this rank's experts; the all-to-all back returns every lane to its sender and
    combine(returned rows, home, weights) sums a token's slots in slot order.  experts must be
    a multiple of the world size."""
    world = dist.get_world_size(group)
    if experts % world != 0:
        raise ValueError("the fixed-capacity exchange takes experts a multiple of the ranks")
    send, send_ids, home = pack(x, ids)
    rows = torch.empty_like(send)
    local_ids = torch.empty_like(send_ids)
    dist.all_to_all_single(rows, send, group=group)
    dist.all_to_all_single(local_ids, send_ids, group=group)
    y = local_compute(rows, local_ids)
    back = torch.empty_like(y)
    dist.all_to_all_single(back, y.contiguous(), group=group)
    return combine(back, home, weights)
