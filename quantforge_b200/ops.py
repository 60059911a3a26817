"""Operators of the W4A16 path on torch CUDA tensors.

The names and argument meaning of `pack_int4`, `unpack_int4` and `gemv_int4` follow the
reference's python/quantforge/baseline.py (:17-31, :34-49, :52-72).  Every compute call goes
through the C ABI into hand-written sm_100a kernels; tensors on the CPU are rejected (there is
no CPU implementation in this package).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib
from ._lib import (QF_BF16, QF_EPI_NONE, QF_EPI_RESIDUAL_ADD, QF_EPI_SILU_MUL, QF_F16, QF_F32, QF_LAYOUT_CANONICAL,
                   QF_LAYOUT_GEMV_SLAB, QF_LAYOUT_INTERLEAVED, QF_LAYOUT_TILED, QF_PATH_AUTO, QF_PATH_GEMV,
                   QF_SLAB_MAX_M, QF_ZERO_CONST, QF_ZERO_I8, QF_ZERO_U4, LinearDesc, QuantForgeError)

_DT = {torch.float16: QF_F16, torch.bfloat16: QF_BF16, torch.float32: QF_F32}
_ctxs: dict[int, ctypes.c_void_p] = {}
_workspaces: dict[tuple[int, int], list] = {}


def _ctx(device: torch.device) -> ctypes.c_void_p:
    """The runtime context of `device` (created on first use; the caller's current device is left as it is)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _ctxs:
        lib = _lib.load()
        h = ctypes.c_void_p()
        with torch.cuda.device(idx):
            st = lib.qf_ctx_create(ctypes.byref(h), idx)
        if st != 0:
            raise QuantForgeError(st, _lib.status_name(st), f"qf_ctx_create(device={idx}) failed")
        _ctxs[idx] = h
    return _ctxs[idx]


def _check(st: int, ctx) -> None:
    if st != 0:
        raise QuantForgeError(st, _lib.status_name(st), _lib.load().qf_last_error(ctx).decode())


def _need_cuda(*tensors: Optional[torch.Tensor]) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("quantforge_b200 runs on CUDA tensors only (no CPU fallback)")
        if dev is not None and t.device != dev:
            raise ValueError("all tensors must live on the same device")
        dev = t.device
    return dev


def _stream(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def launch_count() -> int:
    """Kernel launches enqueued by the runtime library since it was loaded."""
    return int(_lib.load().qf_launch_count())


# --------------------------------------------------------------------------------------------
# packing helpers (layout only; any device)
# --------------------------------------------------------------------------------------------
def pack_int4(weights: torch.Tensor) -> torch.Tensor:
    """int8[..., 2n] codes in [0, 15] -> int8[..., n]; even index -> low nibble."""
    if weights.dtype != torch.int8:
        raise TypeError("pack_int4 expects an int8 tensor of codes")
    if weights.shape[-1] % 2 != 0:
        raise ValueError("last dim must be even")
    low = weights[..., 0::2] & 0x0F
    high = weights[..., 1::2] & 0x0F
    return (low | (high << 4)).to(torch.int8)


def pack_zeros_u4(zeros: torch.Tensor) -> torch.Tensor:
    """zero codes [G, N] in [0, 15] -> int32[G, N/8] holding 8 codes per word along N, LSB first."""
    G, N = zeros.shape
    if N % 8 != 0:
        raise ValueError("N must be a multiple of 8")
    z = zeros.to(torch.int64).reshape(G, N // 8, 8) & 0xF
    shifts = torch.arange(8, device=zeros.device, dtype=torch.int64) * 4
    words = (z << shifts).sum(dim=-1)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words)
    return words.to(torch.int32).contiguous()


# --------------------------------------------------------------------------------------------
# qf.unpack
# --------------------------------------------------------------------------------------------
def unpack_int4(packed: torch.Tensor) -> torch.Tensor:
    """int8[..., n] -> int8[..., 2n]: out[2i] = b & 0xF, out[2i+1] = (b >> 4) & 0xF (logical shift)."""
    dev = _need_cuda(packed)
    if packed.dtype not in (torch.int8, torch.uint8):
        raise TypeError("unpack_int4 expects int8 (or uint8) packed bytes")
    packed = packed.contiguous()
    out = torch.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=torch.int8, device=dev)
    rows = packed.numel() // packed.shape[-1] if packed.shape[-1] else 0
    ctx = _ctx(dev)
    with torch.cuda.device(dev):
        _check(_lib.load().qf_unpack_int4(ctx, _ptr(packed), _ptr(out), rows, packed.shape[-1], _stream(dev)), ctx)
    return out


# --------------------------------------------------------------------------------------------
# linear
# --------------------------------------------------------------------------------------------
def _make_desc(M, N, K, group_size, act_dtype, out_dtype, zeros, zero_const, path, split_k,
               weight_layout=QF_LAYOUT_CANONICAL, epilogue=QF_EPI_NONE) -> LinearDesc:
    d = LinearDesc()
    d.M, d.N, d.K = M, N, K
    d.group_size = group_size
    d.act_dtype = _DT[act_dtype]
    d.out_dtype = _DT[out_dtype]
    if zeros is None:
        d.zero_mode, d.zero_const = QF_ZERO_CONST, int(zero_const)
    elif zeros.dtype == torch.int8:
        d.zero_mode = QF_ZERO_I8
    elif zeros.dtype == torch.int32:
        d.zero_mode = QF_ZERO_U4
    else:
        raise TypeError("zeros must be None (constant), int8 [G,N] or packed int32 [G,N/8]")
    d.path = path
    d.split_k = split_k
    d.weight_layout = weight_layout
    d.epilogue = epilogue
    return d


def workspace_bytes(desc: LinearDesc) -> int:
    return int(_lib.load().qf_w4a16_workspace_bytes(ctypes.byref(desc)))


def _workspace(dev: torch.device, nbytes: int) -> Optional[torch.Tensor]:
    """Per (device, stream) zero-initialised scratch. Calls on one stream are ordered, so they share it.

    A call that needs more than any buffer made so far gets a NEW, larger buffer; the older ones stay alive and
    keep serving the smaller requests, because a CUDA graph captured earlier still holds their addresses."""
    if nbytes == 0:
        return None
    key = (dev.index if dev.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(dev).cuda_stream)
    bufs = _workspaces.setdefault(key, [])
    for ws in bufs:  # ascending sizes: the smallest buffer that fits, the same one every time for a given size
        if ws.numel() >= nbytes:
            return ws
    ws = torch.zeros(max(nbytes, 4 << 20), dtype=torch.uint8, device=dev)
    bufs.append(ws)
    return ws


def _check_linear_tensors(x, qweight, scales, zeros, group_size):
    if x.dim() != 2 or qweight.dim() != 2:
        raise ValueError("x must be [M, K] and qweight [N, K/2] (int8) or [N, K/8] (int32)")
    M, K = x.shape
    if qweight.dtype in (torch.int8, torch.uint8):
        N, kw = qweight.shape[0], qweight.shape[1] * 2
    elif qweight.dtype == torch.int32:
        N, kw = qweight.shape[0], qweight.shape[1] * 8
    else:
        raise TypeError("qweight must be int8/uint8 [N, K/2] or int32 [N, K/8]")
    if kw != K:
        raise ValueError(f"qweight holds {kw} codes per row but x has K={K}")
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("x must be float16 or bfloat16")
    if scales.dtype != x.dtype:
        raise TypeError("scales must have the dtype of x")
    G = K // group_size if group_size > 0 and K % group_size == 0 else -1
    if tuple(scales.shape) != (G, N):
        raise ValueError(f"scales must be [K/group_size, N] = [{G}, {N}], got {tuple(scales.shape)}")
    if zeros is not None:
        want = (G, N) if zeros.dtype == torch.int8 else (G, N // 8)
        if tuple(zeros.shape) != want:
            raise ValueError(f"zeros must be {want}, got {tuple(zeros.shape)}")
    return M, N, K


class SlabWeight:
    """Weights of one linear in QF_LAYOUT_GEMV_SLAB (codes, scales and zeros in one blob) and the facts needed to
    call the streaming GEMV kernel on them. Made by `prepack_gemv_slab`; serves batches of up to 32 rows."""

    def __init__(self, blob: torch.Tensor, N: int, K: int, group_size: int, act_dtype: torch.dtype, zero_mode: int,
                 zero_const: int):
        self.blob, self.N, self.K, self.group_size = blob, N, K, group_size
        self.act_dtype, self.zero_mode, self.zero_const = act_dtype, zero_mode, zero_const

    @property
    def device(self):
        return self.blob.device


def prepack_gemv_slab(qweight: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor] = None,
                      group_size: int = 128, zero_const: int = 8) -> SlabWeight:
    """One-time prepack of canonical weights (+ scales, zeros) for the streaming GEMV kernel (M <= 32)."""
    dev = _need_cuda(qweight, scales, zeros)
    N = qweight.shape[0]
    K = qweight.shape[1] * (8 if qweight.dtype == torch.int32 else 2)
    d = _make_desc(1, N, K, group_size, scales.dtype, scales.dtype, zeros, zero_const, QF_PATH_AUTO, 0,
                   QF_LAYOUT_GEMV_SLAB)
    lib = _lib.load()
    nbytes = int(lib.qf_prepack_bytes(QF_LAYOUT_GEMV_SLAB, N, K))
    if nbytes == 0:
        raise ValueError("QF_LAYOUT_GEMV_SLAB needs N % 64 == 0 and K % 128 == 0")
    qweight, scales = qweight.contiguous(), scales.contiguous()
    zeros = zeros.contiguous() if zeros is not None else None
    blob = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    ctx = _ctx(dev)
    with torch.cuda.device(dev):
        st = lib.qf_prepack_gemv_slab(ctx, ctypes.byref(d), _ptr(qweight), _ptr(scales), _ptr(zeros), _ptr(blob),
                                      _stream(dev))
    _check(st, ctx)
    return SlabWeight(blob, N, K, group_size, scales.dtype, d.zero_mode, int(zero_const))


def unpack_gemv_slab(w: SlabWeight) -> torch.Tensor:
    """The codes of a slab blob back as canonical int8 [N, K/2] (the inverse permutation of the prepack)."""
    out = torch.empty((w.N, w.K // 2), dtype=torch.int8, device=w.device)
    ctx = _ctx(w.device)
    with torch.cuda.device(w.device):
        st = _lib.load().qf_unpack_gemv_slab(ctx, w.N, w.K, _ptr(w.blob), _ptr(out), _stream(w.device))
    _check(st, ctx)
    return out


def repack_kn_to_canonical(w_kn: torch.Tensor, K: int, N: int) -> torch.Tensor:
    """W[K, N] as the reference's compiler half lays it out - int8 [K, N] (one code per byte) or int8 [K, N/2]
    (two codes per byte along N) - to the canonical int8 [N, K/2] the kernels read."""
    dev = _need_cuda(w_kn)
    if tuple(w_kn.shape) == (K, N):
        packed = 0
    elif tuple(w_kn.shape) == (K, N // 2):
        packed = 1
    else:
        raise ValueError(f"w_kn must be [{K}, {N}] or [{K}, {N // 2}], got {tuple(w_kn.shape)}")
    w_kn = w_kn.contiguous()
    out = torch.empty((N, K // 2), dtype=torch.int8, device=dev)
    ctx = _ctx(dev)
    with torch.cuda.device(dev):
        st = _lib.load().qf_repack_kn_to_canonical(ctx, _ptr(w_kn), packed, K, N, _ptr(out), _stream(dev))
    _check(st, ctx)
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, dim: int = 0) -> torch.Tensor:
    """Row order QF_EPI_SILU_MUL expects: groups of 8 gate rows followed by the matching 8 up rows, along `dim`
    (dim 0 for qweight [N, ...], the last dim for scales / int8 zeros [G, N])."""
    if gate.shape != up.shape or gate.shape[dim] % 8 != 0:
        raise ValueError("gate and up must have the same shape, a multiple of 8 long along `dim`")
    g = gate.movedim(dim, 0)
    u = up.movedim(dim, 0)
    n = g.shape[0]
    both = torch.stack([g.reshape(n // 8, 8, *g.shape[1:]), u.reshape(n // 8, 8, *u.shape[1:])], dim=1)
    return both.reshape(2 * n, *g.shape[1:]).movedim(0, dim).contiguous()


def w4a16_linear(x: torch.Tensor, qweight, scales: Optional[torch.Tensor] = None,
                 zeros: Optional[torch.Tensor] = None,
                 group_size: int = 128, zero_const: int = 8, out_dtype: Optional[torch.dtype] = None,
                 path: int = QF_PATH_AUTO, split_k: int = 0, out: Optional[torch.Tensor] = None,
                 weight_layout: int = QF_LAYOUT_CANONICAL, epilogue: int = QF_EPI_NONE,
                 residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Y[M,N] = X[M,K] . dequant(unpack(qweight))^T, fp32 accumulation, W never materialised.

    weight_layout: QF_LAYOUT_CANONICAL, or QF_LAYOUT_INTERLEAVED for weights passed through prepack_w4.
    qweight may also be a `SlabWeight` (prepack_gemv_slab): scales / zeros / group_size / weight_layout then come
    from it.
    epilogue: QF_EPI_SILU_MUL (weights are gate|up rows interleaved by `interleave_gate_up`; Y is [M, N/2]) or
    QF_EPI_RESIDUAL_ADD (Y = X.W^T + residual; residual [M, N] of out_dtype, may be `out` itself).

    x        f16|bf16 [M, K]
    qweight  int8 [N, K/2] (two codes per byte along K) or int32 [N, K/8]
    scales   same dtype as x, [K/group_size, N]
    zeros    None (constant `zero_const`), int8 [G, N] or packed int32 [G, N/8] (pack_zeros_u4)
    """
    if isinstance(qweight, SlabWeight):
        w = qweight
        dev = _need_cuda(x, w.blob, residual)
        if x.dim() != 2 or x.shape[1] != w.K:
            raise ValueError(f"x must be [M, {w.K}]")
        if x.dtype != w.act_dtype:
            raise TypeError("x must have the dtype the slab was built for")
        M, N, K = x.shape[0], w.N, w.K
        d = LinearDesc()
        d.M, d.N, d.K, d.group_size = M, N, K, w.group_size
        d.act_dtype, d.zero_mode, d.zero_const = _DT[x.dtype], w.zero_mode, w.zero_const
        d.path, d.split_k, d.weight_layout, d.epilogue = QF_PATH_AUTO, split_k, QF_LAYOUT_GEMV_SLAB, epilogue
        ptr_w, ptr_s, ptr_z = _ptr(w.blob), _ptr(None), _ptr(None)
        x = x.contiguous()
    else:
        if scales is None:
            raise ValueError("scales are required unless qweight is a SlabWeight")
        dev = _need_cuda(x, qweight, scales, zeros, residual)
        M, N, K = _check_linear_tensors(x, qweight, scales, zeros, group_size)
        x, qweight, scales = x.contiguous(), qweight.contiguous(), scales.contiguous()
        zeros = zeros.contiguous() if zeros is not None else None
        d = _make_desc(M, N, K, group_size, x.dtype, x.dtype, zeros, zero_const, path, split_k, weight_layout,
                       epilogue)
        ptr_w, ptr_s, ptr_z = _ptr(qweight), _ptr(scales), _ptr(zeros)
    out_dtype = out_dtype or x.dtype
    d.out_dtype = _DT[out_dtype]
    shape = (M, N // 2) if epilogue == QF_EPI_SILU_MUL else (M, N)
    if out is None:
        out = torch.empty(shape, dtype=out_dtype, device=dev)
    elif tuple(out.shape) != shape or out.dtype != out_dtype or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous {list(shape)} tensor of out_dtype")
    if epilogue == QF_EPI_RESIDUAL_ADD:
        if residual is None or tuple(residual.shape) != shape or residual.dtype != out_dtype or \
                not residual.is_contiguous():
            raise ValueError("QF_EPI_RESIDUAL_ADD needs a contiguous residual of the output's shape and dtype")
    ctx = _ctx(dev)
    with torch.cuda.device(dev):
        ws = _workspace(dev, workspace_bytes(d))
        st = _lib.load().qf_w4a16_linear_fused(ctx, ctypes.byref(d), _ptr(x), ptr_w, ptr_s, ptr_z, _ptr(out),
                                               _ptr(residual), _ptr(ws), ws.numel() if ws is not None else 0,
                                               _stream(dev))
    _check(st, ctx)
    return out


class Comm:
    """Exchange buffers of a group of ranks (one process per GPU of one node) for `w4a16_linear_allreduce`.

    `exchange(handle_bytes) -> list of every rank's handle bytes, in rank order` is how the 64-byte buffer handles
    travel; by default torch.distributed.all_gather_object over `group`. The constructor ends with a barrier.
    """

    def __init__(self, max_out_elems: int, device: Optional[torch.device] = None, group=None,
                 rank: Optional[int] = None, world: Optional[int] = None, exchange=None):
        import torch.distributed as dist
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        if self.device.type != "cuda":
            raise ValueError("Comm needs a CUDA device (no CPU fallback exists)")
        use_dist = (rank is None or world is None)
        self.group = group
        self.rank = dist.get_rank(group) if use_dist else rank
        self.world = dist.get_world_size(group) if use_dist else world
        self.max_out_elems = int(max_out_elems)
        self._ctx = _ctx(self.device)
        self._h = ctypes.c_void_p()
        lib = _lib.load()
        with torch.cuda.device(self.device):
            _check(lib.qf_comm_create(self._ctx, self.rank, self.world, self.max_out_elems, ctypes.byref(self._h)),
                   self._ctx)
            if self.world > 1:
                buf = ctypes.create_string_buffer(_lib.QF_COMM_HANDLE_BYTES)
                _check(lib.qf_comm_export(self._h, buf), self._ctx)
                mine = bytes(buf.raw)
                if exchange is not None:
                    handles = exchange(mine)
                else:
                    handles = [None] * self.world
                    dist.all_gather_object(handles, mine, group=group)
                blob = b"".join(handles)
                _check(lib.qf_comm_connect(self._h, blob, self.world), self._ctx)
                if exchange is None:
                    dist.barrier(group=group)

    def close(self, barrier: bool = True) -> None:
        """Unmap the peers and free the buffer. Every rank must have finished its calls: with `barrier` (default)
        the device is synchronised and the ranks meet in a torch.distributed barrier first."""
        if self._h:
            if self.world > 1 and barrier:
                import torch.distributed as dist
                torch.cuda.synchronize(self.device)
                dist.barrier(group=self.group)
            _lib.load().qf_comm_destroy(self._h)
            self._h = ctypes.c_void_p()


def _linear_exchange(fn_name, gather, x, qweight, scales, zeros, comm, group_size, zero_const, out_dtype, path,
                     split_k, out, weight_layout):
    if isinstance(qweight, SlabWeight):
        w = qweight
        dev = _need_cuda(x, w.blob)
        if x.dim() != 2 or x.shape[1] != w.K or x.dtype != w.act_dtype:
            raise ValueError(f"x must be [M, {w.K}] of the dtype the slab was built for")
        M, N, K = x.shape[0], w.N, w.K
        x = x.contiguous()
        d = LinearDesc()
        d.M, d.N, d.K, d.group_size = M, N, K, w.group_size
        d.act_dtype, d.zero_mode, d.zero_const = _DT[x.dtype], w.zero_mode, w.zero_const
        d.path, d.split_k, d.weight_layout = QF_PATH_AUTO, split_k, QF_LAYOUT_GEMV_SLAB
        out_dtype = out_dtype or x.dtype
        d.out_dtype = _DT[out_dtype]
        ptr_w, ptr_s, ptr_z = _ptr(w.blob), _ptr(None), _ptr(None)
    else:
        dev = _need_cuda(x, qweight, scales, zeros)
        M, N, K = _check_linear_tensors(x, qweight, scales, zeros, group_size)
        out_dtype = out_dtype or x.dtype
        x, qweight, scales = x.contiguous(), qweight.contiguous(), scales.contiguous()
        zeros = zeros.contiguous() if zeros is not None else None
        d = _make_desc(M, N, K, group_size, x.dtype, out_dtype, zeros, zero_const, path, split_k, weight_layout)
        ptr_w, ptr_s, ptr_z = _ptr(qweight), _ptr(scales), _ptr(zeros)
    shape = (M, N * comm.world) if gather else (M, N)
    if out is None:
        out = torch.empty(shape, dtype=out_dtype, device=dev)
    elif tuple(out.shape) != shape or out.dtype != out_dtype or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous {list(shape)} tensor of out_dtype")
    ctx = _ctx(dev)
    with torch.cuda.device(dev):
        ws = _workspace(dev, workspace_bytes(d))
        st = getattr(_lib.load(), fn_name)(ctx, comm._h, ctypes.byref(d), _ptr(x), ptr_w, ptr_s, ptr_z,
                                           _ptr(out), _ptr(ws), ws.numel() if ws is not None else 0,
                                           _stream(dev))
    _check(st, ctx)
    return out


def w4a16_linear_allreduce(x: torch.Tensor, qweight, scales: Optional[torch.Tensor],
                           zeros: Optional[torch.Tensor], comm: Comm, group_size: int = 128, zero_const: int = 8,
                           out_dtype: Optional[torch.dtype] = None, split_k: int = 0,
                           out: Optional[torch.Tensor] = None, path: int = QF_PATH_AUTO,
                           weight_layout: int = QF_LAYOUT_CANONICAL) -> torch.Tensor:
    """Row-parallel linear: this rank's K shard of X and of the weights in, the sum over all ranks out (on every
    rank, bit-identical), summed inside the kernel over NVLink peer memory. M <= 64."""
    return _linear_exchange("qf_w4a16_linear_allreduce", False, x, qweight, scales, zeros, comm, group_size,
                            zero_const, out_dtype, path, split_k, out, weight_layout)


def w4a16_linear_allgather(x: torch.Tensor, qweight, scales: Optional[torch.Tensor],
                           zeros: Optional[torch.Tensor], comm: Comm, group_size: int = 128, zero_const: int = 8,
                           out_dtype: Optional[torch.dtype] = None, split_k: int = 0,
                           out: Optional[torch.Tensor] = None, path: int = QF_PATH_AUTO,
                           weight_layout: int = QF_LAYOUT_CANONICAL) -> torch.Tensor:
    """Column-parallel linear: the whole X and this rank's shard of output columns in, Y[M, world*N_local] out on
    every rank (columns [r*N_local, (r+1)*N_local) from rank r), gathered inside the kernel. M <= 64."""
    return _linear_exchange("qf_w4a16_linear_allgather", True, x, qweight, scales, zeros, comm, group_size,
                            zero_const, out_dtype, path, split_k, out, weight_layout)


def w4a16_linear_host(x_host: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor,
                      zeros: Optional[torch.Tensor] = None, group_size: int = 128, zero_const: int = 8,
                      out_dtype: Optional[torch.dtype] = None, out_host: Optional[torch.Tensor] = None,
                      path: int = QF_PATH_AUTO, weight_layout: int = QF_LAYOUT_CANONICAL,
                      wait: bool = True) -> torch.Tensor:
    """Same linear with activations and result in HOST memory (pinned for speed); weights stay on the GPU.

    wait=False enqueues the copies and the kernel on the current stream and returns at once: out_host is valid
    after the stream has been synchronised (pinned buffers; x_host must not change until then)."""
    if x_host.is_cuda:
        raise ValueError("x_host must be a CPU tensor")
    dev = _need_cuda(qweight, scales, zeros)
    M, N, K = _check_linear_tensors(x_host, qweight, scales, zeros, group_size)
    out_dtype = out_dtype or x_host.dtype
    x_host = x_host.contiguous()
    if out_host is None:
        out_host = torch.empty((M, N), dtype=out_dtype, pin_memory=True)
    d = _make_desc(M, N, K, group_size, x_host.dtype, out_dtype, zeros, zero_const, path, 0, weight_layout)
    ctx = _ctx(dev)
    with torch.cuda.device(dev):
        ws = _workspace(dev, workspace_bytes(d))
        fn = _lib.load().qf_w4a16_linear_host if wait else _lib.load().qf_w4a16_linear_host_async
        st = fn(ctx, ctypes.byref(d), _ptr(x_host), _ptr(qweight), _ptr(scales), _ptr(zeros), _ptr(out_host),
                _ptr(ws), ws.numel() if ws is not None else 0, _stream(dev))
    _check(st, ctx)
    return out_host


def dequant_w4(qweight: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor] = None,
               group_size: int = 128, zero_const: int = 8) -> torch.Tensor:
    """qf.dequant(qf.unpack(qweight)) materialised: W[N, K] in the dtype of `scales`."""
    dev = _need_cuda(qweight, scales, zeros)
    N = qweight.shape[0]
    K = qweight.shape[1] * (8 if qweight.dtype == torch.int32 else 2)
    out = torch.empty((N, K), dtype=scales.dtype, device=dev)
    d = _make_desc(1, N, K, group_size, scales.dtype, scales.dtype, zeros, zero_const, QF_PATH_AUTO, 0)
    ctx = _ctx(dev)
    qweight, scales = qweight.contiguous(), scales.contiguous()
    zeros = zeros.contiguous() if zeros is not None else None
    with torch.cuda.device(dev):
        st = _lib.load().qf_dequant_w4(ctx, ctypes.byref(d), _ptr(qweight), _ptr(scales), _ptr(zeros), _ptr(out),
                                       _stream(dev))
    _check(st, ctx)
    return out


def prepack_w4(qweight: torch.Tensor, to_canonical: bool = False, layout: int = QF_LAYOUT_INTERLEAVED) -> torch.Tensor:
    """One-time weight permutation: canonical -> `layout` (QF_LAYOUT_INTERLEAVED or QF_LAYOUT_TILED), or back.

    The result has the shape and dtype of the input; only the order of the 4-bit codes changes.
    """
    dev = _need_cuda(qweight)
    qweight = qweight.contiguous()
    if layout == QF_LAYOUT_TILED:
        N = qweight.shape[0]
        K = qweight.shape[1] * (8 if qweight.dtype == torch.int32 else 2)
        out = torch.empty_like(qweight)
        ctx = _ctx(dev)
        with torch.cuda.device(dev):
            st = _lib.load().qf_prepack_w4_tiled(ctx, _ptr(qweight), _ptr(out), N, K, 1 if to_canonical else 0,
                                                 _stream(dev))
        _check(st, ctx)
        return out
    nbytes = qweight.numel() * qweight.element_size()
    if nbytes % 4 != 0:
        raise ValueError("qweight must hold whole 32-bit words")
    out = torch.empty_like(qweight)
    ctx = _ctx(dev)
    with torch.cuda.device(dev):
        st = _lib.load().qf_prepack_w4(ctx, _ptr(qweight), _ptr(out), nbytes // 4, 1 if to_canonical else 0,
                                       _stream(dev))
    _check(st, ctx)
    return out


def device_status(device: Optional[torch.device] = None) -> int:
    """Sticky device-side status of the context (0, or QF_ERR_TIMEOUT after a bounded wait expired). Synchronises."""
    dev = device or torch.device("cuda", torch.cuda.current_device())
    torch.cuda.synchronize(dev)
    return int(_lib.load().qf_ctx_status(_ctx(dev)))


def clear_device_status(device: Optional[torch.device] = None) -> None:
    dev = device or torch.device("cuda", torch.cuda.current_device())
    _lib.load().qf_ctx_clear_status(_ctx(dev))


def gemv_int4(x: torch.Tensor, w_packed: torch.Tensor, scale: torch.Tensor, zero_point: torch.Tensor) -> torch.Tensor:
    """Drop-in for the reference's `gemv_int4_baseline(x, w_packed, scale, zero_point)`.

    x (M, K) f16, w_packed (N, K/2) int8, per-output-channel scale (N,) f16 and zero_point (N,) int8.
    Per-channel quantisation is the group_size == K case of the group-wise kernel.
    """
    K = x.shape[1]
    return w4a16_linear(x, w_packed, scale.reshape(1, -1).to(x.dtype), zero_point.reshape(1, -1).to(torch.int8),
                        group_size=K, out_dtype=x.dtype)


class W4A16Linear:
    """A quantised linear layer whose weights live on one GPU: y = x . W^T."""

    def __init__(self, qweight: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor] = None,
                 group_size: int = 128, zero_const: int = 8, prepack: bool = False,
                 weight_layout: int = QF_LAYOUT_CANONICAL):
        """weight_layout: the layout `qweight` is already in (weights that went through prepack_w4 before);
        prepack=True converts canonical weights here instead."""
        _need_cuda(qweight, scales, zeros)
        self.qweight, self.scales, self.zeros = qweight.contiguous(), scales.contiguous(), zeros
        self.group_size, self.zero_const = group_size, zero_const
        self.weight_layout = weight_layout
        self._host_prep = {}
        if prepack and weight_layout == QF_LAYOUT_CANONICAL and qweight.shape[0] % 128 == 0:
            self.qweight = prepack_w4(self.qweight, layout=QF_LAYOUT_TILED)
            self.weight_layout = QF_LAYOUT_TILED
        self.N = qweight.shape[0]
        self.K = qweight.shape[1] * (8 if qweight.dtype == torch.int32 else 2)

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return w4a16_linear(x, self.qweight, self.scales, self.zeros, self.group_size, self.zero_const, out_dtype,
                            out=out, weight_layout=self.weight_layout)

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor, wait: bool = True) -> torch.Tensor:
        """Host activations in, host result out (both contiguous, ideally pinned), on the current stream of the
        weights' device, which must be the current device. Descriptor, workspace and weight pointers are prepared
        once per (batch, dtypes), so that a serving loop pays for little more than the C call.
        wait=False: returns after enqueueing; out_host is valid once the stream has been synchronised."""
        key = (x_host.shape[0], x_host.dtype, out_host.dtype)
        prep = self._host_prep.get(key)
        if prep is None:
            if x_host.is_cuda or out_host.is_cuda:
                raise ValueError("forward_host takes CPU tensors")
            dev = self.qweight.device
            M, N, K = _check_linear_tensors(x_host, self.qweight, self.scales, self.zeros, self.group_size)
            d = _make_desc(M, N, K, self.group_size, x_host.dtype, out_host.dtype, self.zeros, self.zero_const,
                           QF_PATH_AUTO, 0, self.weight_layout)
            with torch.cuda.device(dev):
                ws = _workspace(dev, workspace_bytes(d))
            lib = _lib.load()
            prep = (d, ctypes.byref(d), _ctx(dev), _ptr(self.qweight), _ptr(self.scales), _ptr(self.zeros), _ptr(ws),
                    ws.numel() if ws is not None else 0, ws, (M, N), lib.qf_w4a16_linear_host,
                    lib.qf_w4a16_linear_host_async, dev)
            self._host_prep[key] = prep
        d, dref, ctx, pw, ps, pz, pws, wsn, _ws, shape, fn_wait, fn_async, dev = prep
        if tuple(out_host.shape) != shape or not out_host.is_contiguous() or not x_host.is_contiguous():
            raise ValueError("x_host and out_host must be contiguous and out_host of shape [M, N]")
        st = (fn_wait if wait else fn_async)(ctx, dref, x_host.data_ptr(), pw, ps, pz, out_host.data_ptr(), pws, wsn,
                                             torch.cuda.current_stream(dev).cuda_stream)
        if st != 0:
            _check(st, ctx)
        return out_host
