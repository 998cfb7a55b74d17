"""Sharding one LUT-AMM across the GPUs of a box, one process per GPU.

The reference spreads one AMM over its DPUs as an input_parallelism x lut_parallelism
grid (inference-engine/src/host/parser.cpp:41-42; LUT slabs pim_lut_host.cpp:33, index
slabs :114).  The same two axes exist here:

* token sharding ("m"): rank r owns a contiguous run of tokens, weights are replicated,
  nothing is exchanged - the output stays sharded unless the caller asks for all rows;
* column sharding ("n"): rank r owns a run of output columns (a multiple of 16, the
  kernels' column granularity) of the LUT and the bias, every rank sees all tokens, and the
  [M][N/G] slabs are exchanged with one all-gather and interleaved into [M][N].

Only the plumbing lives here (ranges, the collective, the re-layout); the arithmetic is the
CUDA library's.  The functions take any torch.distributed backend, so the logic is tested
with gloo on CPU.
"""
from __future__ import annotations

COLUMN_GRANULE = 16


def token_range(M: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous, near-equal split; the first M % world ranks get one extra token."""
    base, extra = divmod(M, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def column_range(N: int, rank: int, world: int) -> tuple[int, int]:
    """Split N columns in units of 16; trailing ranks may get fewer (or zero) units."""
    assert N % COLUMN_GRANULE == 0, "output_feature_len must be a multiple of 16"
    units = N // COLUMN_GRANULE
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo * COLUMN_GRANULE, hi * COLUMN_GRANULE


def gather_rows(y_local, M: int, group=None):
    """All-gather token shards [m_r][N] into [M][N] on every rank (ragged shards allowed)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    N = y_local.shape[1]
    sizes = [token_range(M, r, world) for r in range(world)]
    pad = max(hi - lo for lo, hi in sizes)
    buf = torch.zeros(pad, N, dtype=y_local.dtype, device=y_local.device)
    buf[: y_local.shape[0]] = y_local
    out = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(out, buf, group=group)
    return torch.cat([o[: hi - lo] for o, (lo, hi) in zip(out, sizes)], dim=0)


def gather_columns(y_local, N: int, group=None):
    """All-gather column slabs [M][n_r] into row-major [M][N] on every rank."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    M = y_local.shape[0]
    ranges = [column_range(N, r, world) for r in range(world)]
    widths = [hi - lo for lo, hi in ranges]
    if len(set(widths)) == 1:
        stacked = torch.empty(world * M, widths[0], dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(stacked, y_local.contiguous(), group=group)
        return stacked.view(world, M, widths[0]).permute(1, 0, 2).reshape(M, N)
    pad = max(widths)
    buf = torch.zeros(M, pad, dtype=y_local.dtype, device=y_local.device)
    buf[:, : y_local.shape[1]] = y_local
    out = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(out, buf, group=group)
    return torch.cat([o[:, :w] for o, w in zip(out, widths)], dim=1)


def shard_weights_by_columns(lut, bias, rank: int, world: int):
    """LUT [CB][CT][N] and bias [N] -> this rank's column slab (numpy or torch)."""
    lo, hi = column_range(lut.shape[2], rank, world)
    return lut[:, :, lo:hi], bias[lo:hi]


def run_sharded(amm_fn, x, M: int, N: int, mode: str, group=None, gather: bool = True):
    """Drive one sharded AMM.  `amm_fn(x_rows)` computes this rank's slab: for mode "m" it is
    given the rank's tokens and returns [m_r][N]; for mode "n" it is given all tokens and
    returns [M][n_r] for the rank's columns."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if mode == "m":
        lo, hi = token_range(M, rank, world)
        y = amm_fn(x[lo:hi])
        return gather_rows(y, M, group) if gather else y
    if mode == "n":
        y = amm_fn(x)
        return gather_columns(y, N, group) if gather else y
    raise ValueError("mode must be 'm' (tokens) or 'n' (output columns)")
