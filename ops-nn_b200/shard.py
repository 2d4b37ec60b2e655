"""Partition arithmetic for running the quantised matmul path on several GPUs of one box.

Every output element depends on one row of x1 and one column of x2 (with their scales), so the path shards without
any data-path collective: weight columns (n) for the decode and per-block workloads, the batch axis for the batched MX
workloads. The only collective is the optional gather of y for a caller that wants the whole output on every rank.

The reference has no multi-device code for these operators; the alignment rules below come from its data formats:
int4 weights are packed eight per int32 along n (matmul/weight_quant_batch_matmul_v2/op_host/op_api/
aclnn_weight_quant_batch_matmul_v2.cpp:1482-1524), per-block weight scales cover 128 columns
(matmul/quant_batch_matmul_v3/op_api/quant_matmul_checker.cpp:724-767).
"""


def split_range(total, world, rank, multiple=1):
    """[begin, end) of `rank`'s share of `total` items cut into `world` contiguous parts whose boundaries are multiples
    of `multiple`. Units of `multiple` are dealt as evenly as possible, the first ranks taking the extra ones; a
    ragged tail shorter than `multiple` goes to the last rank that owns anything."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("rank %r outside world %r" % (rank, world))
    if total < 0 or multiple < 1:
        raise ValueError("bad total/multiple")
    units = total // multiple
    base, extra = divmod(units, world)
    begin_u = rank * base + min(rank, extra)
    end_u = begin_u + base + (1 if rank < extra else 0)
    begin, end = begin_u * multiple, end_u * multiple
    tail = total - units * multiple
    if tail:
        last_owner = min(world, units) - 1 if units else 0
        if rank == last_owner:
            end += tail
        if units == 0 and rank != 0:
            begin = end = total
    return begin, end


def shard_w4a16(words, scale, offset, bias, world, rank, group_cols=8):
    """Column shard of a W4A16 problem. `words` is the int32 carrier (k, n/8); scale/offset are (groups, n) or (n,);
    bias is (n,) or None. Works on numpy arrays and torch tensors alike (basic slicing only: views, no copies).
    Returns (words, scale, offset, bias, (col_begin, col_end))."""
    n = words.shape[-1] * 8
    b, e = split_range(n, world, rank, max(8, group_cols))
    cut = lambda t: None if t is None else t[..., b:e]
    return words[..., b // 8:e // 8], cut(scale), cut(offset), cut(bias), (b, e)


def shard_perblock_weight(x2, x2_scale, world, rank, block=128):
    """Column shard of a per-block weight: x2 (k, n), x2_scale (ceil(k/block), ceil(n/block))."""
    n = x2.shape[-1]
    b, e = split_range(n, world, rank, block)
    return x2[..., b:e], x2_scale[..., b // block:(e + block - 1) // block], (b, e)


def shard_batch(tensors, world, rank):
    """Batch shard: every tensor in `tensors` whose leading dimension is the batch is cut; None entries and tensors
    marked as shared (wrapped in a 1-tuple) pass through."""
    first = next(t for t in tensors if t is not None and not isinstance(t, tuple))
    b, e = split_range(first.shape[0], world, rank)
    out = []
    for t in tensors:
        if t is None:
            out.append(None)
        elif isinstance(t, tuple):
            out.append(t[0])
        else:
            out.append(t[b:e])
    return out, (b, e)


def gather_columns(y_local, n_total, world, rank, multiple=8, group=None):
    """All ranks receive the full (m, n_total) output from (m, n_local) column shards (torch.distributed; NCCL for CUDA
    tensors, gloo for CPU tensors). Shards may differ in width, so every rank contributes a max-width padded block."""
    import torch
    import torch.distributed as dist

    widths = [split_range(n_total, world, r, multiple) for r in range(world)]
    wmax = max(e - b for b, e in widths)
    m = y_local.shape[0]
    send = torch.zeros((m, wmax), dtype=y_local.dtype, device=y_local.device)
    send[:, :y_local.shape[1]] = y_local
    recv = torch.empty((world * m, wmax), dtype=y_local.dtype, device=y_local.device)  # concatenated along dim 0
    dist.all_gather_into_tensor(recv, send, group=group)
    recv = recv.view(world, m, wmax)
    full = torch.empty((m, n_total), dtype=y_local.dtype, device=y_local.device)
    for r, (b, e) in enumerate(widths):
        full[:, b:e] = recv[r, :, :e - b]
    return full


def gather_batch(y_local, batch_total, world, rank, group=None):
    """All ranks receive the full (batch_total, ...) output from contiguous batch shards."""
    import torch
    import torch.distributed as dist

    parts = [split_range(batch_total, world, r) for r in range(world)]
    bmax = max(e - b for b, e in parts)
    send = torch.zeros((bmax,) + tuple(y_local.shape[1:]), dtype=y_local.dtype, device=y_local.device)
    send[:y_local.shape[0]] = y_local
    recv = torch.empty((world * bmax,) + tuple(y_local.shape[1:]), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(recv, send, group=group)
    recv = recv.view((world, bmax) + tuple(y_local.shape[1:]))
    return torch.cat([recv[r, :e - b] for r, (b, e) in enumerate(parts)], dim=0)
