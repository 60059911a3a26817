"""Tensor-parallel W4A16 linears: one process per GPU, torch.distributed for the exchange step.

Column-parallel: rank r owns output columns [r*N/W, (r+1)*N/W) (rows of qweight, columns of scales / zeros);
X is replicated; the per-rank outputs are all-gathered (or left sharded to feed a row-parallel linear).
Row-parallel: rank r owns input features [r*K/W, (r+1)*K/W) (columns of qweight, group rows of scales / zeros);
X arrives sharded along K (the output of a column-parallel linear); partial outputs are all-reduced (sum).

The shard helpers are pure indexing and work on any device; the compute is the CUDA operator
(`quantforge_b200.ops.w4a16_linear`) unless a test injects another callable.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import ops


def _codes_per_elem(qweight: torch.Tensor) -> int:
    return 8 if qweight.dtype == torch.int32 else 2


def check_shardable(N: int, K: int, group_size: int, world: int, mode: str) -> None:
    if mode == "column":
        if N % world or (N // world) % 16:
            raise ValueError(f"column-parallel needs N/world to be a multiple of 16 (N={N}, world={world})")
    elif mode == "row":
        if K % world or (K // world) % group_size or (K // world) % 128:
            raise ValueError(
                f"row-parallel needs K/world to be a multiple of the group size and of 128 (K={K}, world={world})")
    else:
        raise ValueError(mode)


def _own(t: torch.Tensor) -> torch.Tensor:
    """A shard in storage of its own. A slice of whole rows is already contiguous, so `.contiguous()` would hand back
    a view that starts in the middle of the parent's storage - for packed zero points with N/2 bytes per group at an
    address that is not a multiple of 16 whenever N is not a multiple of 32, which the kernels refuse."""
    return t.clone(memory_format=torch.contiguous_format)


def shard_column(qweight, scales, zeros, rank: int, world: int):
    """-> (qweight[N_r, :], scales[:, N_r], zeros[:, N_r]) for the column-parallel shard of `rank`."""
    N = qweight.shape[0]
    K = qweight.shape[1] * _codes_per_elem(qweight)
    check_shardable(N, K, K // scales.shape[0], world, "column")
    n0, n1 = rank * N // world, (rank + 1) * N // world
    z = None
    if zeros is not None:
        z = _own(zeros[:, n0 // 8:n1 // 8] if zeros.dtype == torch.int32 else zeros[:, n0:n1])
    return _own(qweight[n0:n1]), _own(scales[:, n0:n1]), z


def shard_row(qweight, scales, zeros, rank: int, world: int):
    """-> (qweight[:, K_r], scales[G_r, :], zeros[G_r, :]) for the row-parallel shard of `rank`."""
    N = qweight.shape[0]
    per = _codes_per_elem(qweight)
    K = qweight.shape[1] * per
    G = scales.shape[0]
    g = K // G
    check_shardable(N, K, g, world, "row")
    k0, k1 = rank * K // world, (rank + 1) * K // world
    z = _own(zeros[k0 // g:k1 // g]) if zeros is not None else None
    return _own(qweight[:, k0 // per:k1 // per]), _own(scales[k0 // g:k1 // g]), z


class ColumnParallelLinear:
    """y_r = x . W[N_r, :]^T ; gather_output=True all-gathers into [M, N].

    With `comm` (an `ops.Comm` of the same ranks), gather_output and M <= 64 the gather happens inside the kernel
    over NVLink peer memory and no NCCL collective is issued.
    """

    def __init__(self, qweight, scales, zeros=None, group_size: int = 128, zero_const: int = 8,
                 group: Optional[dist.ProcessGroup] = None, gather_output: bool = True,
                 compute: Optional[Callable] = None, prepack: bool = False, comm: Optional["ops.Comm"] = None,
                 slab: bool = False):
        """slab=True additionally prepacks the shard for the streaming GEMV kernel, which then serves batches of up
        to 32 rows (N/world must be a multiple of 64)."""
        self.comm = comm
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.gather_output = gather_output
        self.group_size, self.zero_const = group_size, zero_const
        self.qweight, self.scales, self.zeros = shard_column(qweight, scales, zeros, self.rank, self.world)
        self.N_local = self.qweight.shape[0]
        self.N = self.N_local * self.world
        self.weight_layout = ops.QF_LAYOUT_CANONICAL
        self.compute = compute
        self.slab = None
        if compute is None and slab:
            self.slab = ops.prepack_gemv_slab(self.qweight, self.scales, self.zeros, group_size, zero_const)
        if compute is None and prepack and self.N_local % 128 == 0:
            self.qweight = ops.prepack_w4(self.qweight)
            self.weight_layout = ops.QF_LAYOUT_INTERLEAVED

    def _local(self, x, out_dtype):
        if self.compute is not None:
            return self.compute(x, self.qweight, self.scales, self.zeros, self.group_size, self.zero_const, out_dtype)
        if self.slab is not None and x.shape[0] <= ops.QF_SLAB_MAX_M:
            return ops.w4a16_linear(x, self.slab, out_dtype=out_dtype)
        return ops.w4a16_linear(x, self.qweight, self.scales, self.zeros, self.group_size, self.zero_const, out_dtype,
                                weight_layout=self.weight_layout)

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        if (self.comm is not None and self.compute is None and self.gather_output and self.world > 1 and
                x.shape[0] <= 64):
            if self.slab is not None and x.shape[0] <= ops.QF_SLAB_MAX_M:
                return ops.w4a16_linear_allgather(x, self.slab, None, None, self.comm, out_dtype=out_dtype)
            return ops.w4a16_linear_allgather(x, self.qweight, self.scales, self.zeros, self.comm, self.group_size,
                                              self.zero_const, out_dtype, weight_layout=self.weight_layout)
        y = self._local(x, out_dtype)
        if not self.gather_output or self.world == 1:
            return y
        M = y.shape[0]
        gathered = torch.empty((self.world * M, self.N_local), dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(gathered, y.contiguous(), group=self.group)
        # [W*M, N/W] (rank-major) -> [M, N]
        return gathered.view(self.world, M, self.N_local).permute(1, 0, 2).reshape(M, self.N)


class RowParallelLinear:
    """y = sum_r x[:, K_r] . W[:, K_r]^T ; partial sums are all-reduced in fp32 (or `reduce_dtype`).

    With `comm` (an `ops.Comm` of the same ranks) and M <= 64 the sum over ranks happens inside the kernel
    over NVLink peer memory (fp32 partials, rank order, one rounding) and no NCCL collective is issued.
    """

    def __init__(self, qweight, scales, zeros=None, group_size: int = 128, zero_const: int = 8,
                 group: Optional[dist.ProcessGroup] = None, input_is_parallel: bool = True,
                 reduce_dtype: torch.dtype = torch.float32, compute: Optional[Callable] = None,
                 prepack: bool = False, comm: Optional["ops.Comm"] = None, slab: bool = False):
        """slab=True additionally prepacks the shard for the streaming GEMV kernel (batches of up to 32 rows; N must
        be a multiple of 64)."""
        self.comm = comm
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.input_is_parallel = input_is_parallel
        self.reduce_dtype = reduce_dtype
        self.group_size, self.zero_const = group_size, zero_const
        self.qweight, self.scales, self.zeros = shard_row(qweight, scales, zeros, self.rank, self.world)
        self.K_local = self.qweight.shape[1] * _codes_per_elem(self.qweight)
        self.weight_layout = ops.QF_LAYOUT_CANONICAL
        self.compute = compute
        self.slab = None
        if compute is None and slab:
            self.slab = ops.prepack_gemv_slab(self.qweight, self.scales, self.zeros, group_size, zero_const)
        if compute is None and prepack and self.qweight.shape[0] % 128 == 0:
            self.qweight = ops.prepack_w4(self.qweight)
            self.weight_layout = ops.QF_LAYOUT_INTERLEAVED

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        out_dtype = out_dtype or x.dtype
        if not self.input_is_parallel:
            x = x[:, self.rank * self.K_local:(self.rank + 1) * self.K_local].contiguous()
        use_slab = self.slab is not None and x.shape[0] <= ops.QF_SLAB_MAX_M
        if self.comm is not None and self.compute is None and x.shape[0] <= 64:
            if use_slab:
                return ops.w4a16_linear_allreduce(x, self.slab, None, None, self.comm, out_dtype=out_dtype)
            return ops.w4a16_linear_allreduce(x, self.qweight, self.scales, self.zeros, self.comm, self.group_size,
                                              self.zero_const, out_dtype, weight_layout=self.weight_layout)
        if self.compute is not None:
            y = self.compute(x, self.qweight, self.scales, self.zeros, self.group_size, self.zero_const,
                             self.reduce_dtype)
        elif use_slab:
            y = ops.w4a16_linear(x, self.slab, out_dtype=self.reduce_dtype)
        else:
            y = ops.w4a16_linear(x, self.qweight, self.scales, self.zeros, self.group_size, self.zero_const,
                                 self.reduce_dtype, weight_layout=self.weight_layout)
        if self.world > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y.to(out_dtype)
