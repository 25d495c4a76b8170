"""Grouped-affine matmul operator: Python host layer over the C ABI.

Names follow the reference: a *weight* is a `grouped_affine_u4/u8` tensor
`[N, K]` with `GroupedAffineMeta{scales, biases, group_size, scales_dtype}`
(core/src/dtype.zig:141-146); `linear` is the `MatmulFn` contract
`out[M,N] = a[M,K] @ b[N,K]^T` (core/src/compute/cpu/matmul_primitives.zig:101).
torch is used only for device memory and streams.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _capi

SCALES_F16, SCALES_BF16 = 0, 1
SHARD_NONE, SHARD_COL, SHARD_ROW = 0, 1, 2
DTYPE_F32, DTYPE_BF16 = 0, 1

_STATUS_INVALID_ARGUMENT = 1


class GafError(RuntimeError):
    """A non-zero status from libtalu_gaf (status 1 = the reference's InvalidArgument)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"tgaf status {status} ({_capi.load().tgaf_status_string(status).decode()}): {message}")
        self.status = status
        self.message = message

    @property
    def invalid_argument(self) -> bool:
        return self.status == _STATUS_INVALID_ARGUMENT


_CUDA_STREAM_LEGACY = 1  # cudaStreamLegacy: the handle of the default stream, usable where NULL means "none"


def _torch_current_stream(device: int) -> int:
    import torch
    if not torch.cuda.is_available():
        return 0
    h = torch.cuda.current_stream(device).cuda_stream
    return h if h else _CUDA_STREAM_LEGACY


def _vpw(bits: int) -> int:
    return 8 if bits == 4 else 4


class Context:
    """One device + one stream (tgaf_ctx).  Not re-entrant."""

    def __init__(self, device: int = 0, stream: int | None = None, own_stream: bool = False):
        """`stream`: a cudaStream_t handle.  Default: torch's current stream on `device`, so
        that calls are ordered with the torch ops around them; own_stream=True asks the
        library for a private non-blocking stream instead."""
        self._lib = _capi.load()
        h = C.c_void_p()
        if stream is None and not own_stream:
            stream = _torch_current_stream(device)
        st = self._lib.tgaf_ctx_create(int(device), C.c_void_p(stream or 0), C.byref(h))
        if st != 0:
            raise GafError(st, "tgaf_ctx_create failed (is a B200 visible?)")
        self._h = h
        self.device = int(device)

    def _check(self, st: int) -> None:
        if st != 0:
            raise GafError(st, self._lib.tgaf_last_error(self._h).decode())

    def set_stream(self, stream: int) -> None:
        self._check(self._lib.tgaf_ctx_set_stream(self._h, C.c_void_p(stream or _CUDA_STREAM_LEGACY)))

    def set_option(self, name: str, value: int) -> None:
        self._check(self._lib.tgaf_ctx_set_option(self._h, name.encode(), int(value)))

    def synchronize(self) -> None:
        self._check(self._lib.tgaf_synchronize(self._h))

    # -- tensor-parallel exchange --
    def comm_init(self, comm_id: bytes, rank: int, nranks: int) -> None:
        buf = (C.c_uint8 * _capi.COMM_ID_BYTES).from_buffer_copy(comm_id)
        self._check(self._lib.tgaf_comm_init(self._h, buf, rank, nranks))

    def allreduce(self, t) -> None:
        """In-place sum over ranks of a torch f32 / bf16 device tensor, on this context's stream."""
        import torch
        dt = {torch.float32: DTYPE_F32, torch.bfloat16: DTYPE_BF16}[t.dtype]
        self._check(self._lib.tgaf_allreduce(self._h, C.c_void_p(t.data_ptr()), t.numel(), dt))

    def uses_peer_memory(self) -> bool:
        """True when small all-reduces run as one kernel over NVLink peer memory (else NCCL)."""
        return bool(self._lib.tgaf_comm_uses_peer_memory(self._h))

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.tgaf_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def make_comm_id() -> bytes:
    lib = _capi.load()
    buf = (C.c_uint8 * _capi.COMM_ID_BYTES)()
    st = lib.tgaf_comm_make_id(buf)
    if st != 0:
        raise GafError(st, "tgaf_comm_make_id failed")
    return bytes(buf)


class Weight:
    """A gaf weight resident on the device (tgaf_weight)."""

    def __init__(self, ctx: Context, handle, N: int, K: int, group: int, bits: int, keep=None):
        self.ctx, self._h = ctx, handle
        self.N, self.K, self.group, self.bits = N, K, group, bits
        self._keep = keep

    @classmethod
    def from_host(cls, ctx: Context, packed, scales, biases, group: int, bits: int,
                  sdtype: int = SCALES_BF16, shard: int = SHARD_NONE, tp_rank: int = 0, tp_size: int = 1):
        """Upload the canonical layout: packed u32 [N, K/vpw], scales/biases u16 [N, K/G]."""
        packed = np.ascontiguousarray(packed)
        scales = np.ascontiguousarray(scales)
        biases = np.ascontiguousarray(biases)
        N = packed.shape[0]
        K = packed.shape[1] * packed.dtype.itemsize * 8 // bits if bits in (4, 8) else 0
        h = C.c_void_p()
        st = ctx._lib.tgaf_weight_upload(ctx._h, packed.ctypes.data, scales.ctypes.data, biases.ctypes.data,
                                         N, K, group, bits, sdtype, shard, tp_rank, tp_size, C.byref(h))
        ctx._check(st)
        n, k = C.c_uint64(), C.c_uint64()
        g, b = C.c_uint32(), C.c_uint32()
        ctx._check(ctx._lib.tgaf_weight_dims(h, C.byref(n), C.byref(k), C.byref(g), C.byref(b)))
        return cls(ctx, h, n.value, k.value, g.value, b.value)

    @classmethod
    def wrap_device(cls, ctx: Context, packed, scales, biases, group: int, bits: int, sdtype: int = SCALES_BF16):
        """Wrap torch device tensors (int32 packed [N, K/vpw], int16 scales/biases) without copying."""
        N = packed.shape[0]
        K = packed.shape[1] * _vpw(bits)
        h = C.c_void_p()
        st = ctx._lib.tgaf_weight_wrap_device(ctx._h, C.c_void_p(packed.data_ptr()), C.c_void_p(scales.data_ptr()),
                                              C.c_void_p(biases.data_ptr()), N, K, group, bits, sdtype, C.byref(h))
        ctx._check(st)
        return cls(ctx, h, N, K, group, bits, keep=(packed, scales, biases))

    def free(self) -> None:
        if getattr(self, "_h", None):
            self.ctx._lib.tgaf_weight_free(self.ctx._h, self._h)
            self._h = None

    def __del__(self):
        try:
            if getattr(self.ctx, "_h", None):
                self.free()
        except Exception:
            pass


def linear(ctx: Context, w: Weight, x, out=None):
    """y[M, N] = x[M, K] @ W^T on the device.  x: torch bf16 or f32, contiguous, on ctx's device."""
    import torch
    if x.dim() != 2 or x.shape[1] != w.K:
        raise GafError(_STATUS_INVALID_ARGUMENT, f"x must be [M, {w.K}], got {tuple(x.shape)}")
    if not x.is_contiguous():
        x = x.contiguous()
    M = x.shape[0]
    if out is None:
        out = torch.empty((M, w.N), dtype=x.dtype, device=x.device)
    if x.dtype == torch.bfloat16:
        st = ctx._lib.tgaf_linear_bf16(ctx._h, w._h, C.c_void_p(x.data_ptr()), M, C.c_void_p(out.data_ptr()))
    elif x.dtype == torch.float32:
        st = ctx._lib.tgaf_linear_f32(ctx._h, w._h, C.c_void_p(x.data_ptr()), M, C.c_void_p(out.data_ptr()))
    else:
        raise GafError(_STATUS_INVALID_ARGUMENT, f"unsupported activation dtype {x.dtype}")
    ctx._check(st)
    return out


def linear_bias(ctx: Context, w: Weight, x, bias, out=None):
    """`linear` followed by y[m, n] += bias[n] (the reference's Linear.forward with its optional bias,
    core/src/inference/backend/cpu/executor/model.zig:98-139).  bias: torch f32 [N] on the device, or None."""
    import torch
    if x.dim() != 2 or x.shape[1] != w.K:
        raise GafError(_STATUS_INVALID_ARGUMENT, f"x must be [M, {w.K}], got {tuple(x.shape)}")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != w.N):
        raise GafError(_STATUS_INVALID_ARGUMENT, f"bias must be f32 [{w.N}]")
    x = x.contiguous()
    M = x.shape[0]
    if out is None:
        out = torch.empty((M, w.N), dtype=x.dtype, device=x.device)
    fn = {torch.bfloat16: ctx._lib.tgaf_linear_bf16_bias, torch.float32: ctx._lib.tgaf_linear_f32_bias}.get(x.dtype)
    if fn is None:
        raise GafError(_STATUS_INVALID_ARGUMENT, f"unsupported activation dtype {x.dtype}")
    ctx._check(fn(ctx._h, w._h, C.c_void_p(x.data_ptr()), M, C.c_void_p(bias.data_ptr() if bias is not None else 0),
                  C.c_void_p(out.data_ptr())))
    return out


def linear_allreduce(ctx: Context, w: Weight, x, out=None):
    """`linear` on a row-parallel weight followed by the sum over the communicator's ranks
    (tgaf_linear_bf16_allreduce; one kernel for M <= 2 when the peer-memory path is up).  bf16 only."""
    import torch
    if x.dim() != 2 or x.shape[1] != w.K or x.dtype != torch.bfloat16:
        raise GafError(_STATUS_INVALID_ARGUMENT, f"x must be bf16 [M, {w.K}], got {x.dtype} {tuple(x.shape)}")
    if not x.is_contiguous():
        x = x.contiguous()
    M = x.shape[0]
    if out is None:
        out = torch.empty((M, w.N), dtype=x.dtype, device=x.device)
    ctx._check(ctx._lib.tgaf_linear_bf16_allreduce(ctx._h, w._h, C.c_void_p(x.data_ptr()), M, C.c_void_p(out.data_ptr())))
    return out


ACT_SILU, ACT_GELU = 1, 2


def ffn_swiglu(ctx: Context, w_gate_up: Weight, w_down: Weight, x, out=None, allreduce: bool = False,
               activation: int = ACT_SILU):
    """y = down(act(gate(x)) * up(x)) with the stacked gate|up weight (tgaf_ffn_swiglu_bf16[_allreduce];
    tgaf_ffn_gated_bf16 for ACT_GELU, the reference's use_gelu variant)."""
    import torch
    if x.dim() != 2 or x.shape[1] != w_gate_up.K or x.dtype != torch.bfloat16:
        raise GafError(_STATUS_INVALID_ARGUMENT, f"x must be bf16 [M, {w_gate_up.K}], got {x.dtype} {tuple(x.shape)}")
    if not x.is_contiguous():
        x = x.contiguous()
    M = x.shape[0]
    if out is None:
        out = torch.empty((M, w_down.N), dtype=x.dtype, device=x.device)
    if activation != ACT_SILU:
        if allreduce:
            raise GafError(_STATUS_INVALID_ARGUMENT, "the all-reduce form takes the silu activation only")
        ctx._check(ctx._lib.tgaf_ffn_gated_bf16(ctx._h, w_gate_up._h, w_down._h, C.c_void_p(x.data_ptr()), M, activation,
                                                C.c_void_p(out.data_ptr())))
        return out
    fn = ctx._lib.tgaf_ffn_swiglu_bf16_allreduce if allreduce else ctx._lib.tgaf_ffn_swiglu_bf16
    ctx._check(fn(ctx._h, w_gate_up._h, w_down._h, C.c_void_p(x.data_ptr()), M, C.c_void_p(out.data_ptr())))
    return out


def hint_next_weight(ctx: Context, w) -> None:
    """Names the weight the linear call AFTER the coming one will use (tgaf_hint_next_weight): the coming
    call's kernel then pulls the head of `w` into L2 while it drains.  One-shot; None clears it."""
    ctx._check(ctx._lib.tgaf_hint_next_weight(ctx._h, w._h if w is not None else None))


def linear_fixed_scratch(ctx: Context, w: Weight, x, out=None):
    """`linear` for bf16 activations through tgaf_linear_bf16_fixed_scratch: the library call
    allocates nothing (its split-K scratch is a fixed array inside the library image).  The
    output tensor is the caller's; pass `out` to keep this wrapper from allocating one."""
    import torch
    if x.dim() != 2 or x.shape[1] != w.K or x.dtype != torch.bfloat16:
        raise GafError(_STATUS_INVALID_ARGUMENT, f"x must be bf16 [M, {w.K}], got {x.dtype} {tuple(x.shape)}")
    if not x.is_contiguous():
        x = x.contiguous()
    M = x.shape[0]
    if out is None:
        out = torch.empty((M, w.N), dtype=x.dtype, device=x.device)
    ctx._check(ctx._lib.tgaf_linear_bf16_fixed_scratch(ctx._h, w._h, C.c_void_p(x.data_ptr()), M,
                                                       C.c_void_p(out.data_ptr())))
    return out


def linear_host(ctx: Context, w: Weight, x: np.ndarray, out: np.ndarray | None = None, wait: bool = True) -> np.ndarray:
    """Same through host buffers: x uint16 (bf16 bit patterns) or float32 [M, K].  wait=False (bf16 only,
    page-locked buffers) only enqueues: `out` is valid after ctx.synchronize()."""
    x = np.ascontiguousarray(x)
    if x.ndim != 2 or x.shape[1] != w.K:
        raise GafError(_STATUS_INVALID_ARGUMENT, f"x must be [M, {w.K}], got {x.shape}")
    M = x.shape[0]
    if out is None:
        out = np.empty((M, w.N), x.dtype)
    if x.dtype == np.uint16 and not wait:
        st = ctx._lib.tgaf_linear_bf16_host_async(ctx._h, w._h, x.ctypes.data, M, out.ctypes.data)
    elif x.dtype == np.uint16:
        st = ctx._lib.tgaf_linear_bf16_host(ctx._h, w._h, x.ctypes.data, M, out.ctypes.data)
    elif x.dtype == np.float32:
        st = ctx._lib.tgaf_linear_f32_host(ctx._h, w._h, x.ctypes.data, M, out.ctypes.data)
    else:
        raise GafError(_STATUS_INVALID_ARGUMENT, f"unsupported activation dtype {x.dtype}")
    ctx._check(st)
    return out


class Batch:
    """A launch list of device-buffer linears (tgaf_batch_*): `count` operations y_i = x_i @ W_i^T with the same
    number of rows, run by ONE call (one kernel launch when every weight is gaf4 of one scheme and M <= 8; M <= 4 for
    groups of 32 codes and for lists with sums over the ranks or dependent operations).
    depends[i]: x_i is written by an earlier operation of the list; reduce[i]: y_i is summed over the ranks."""

    def __init__(self, ctx: Context, weights, xs, ys, depends=None, reduce=None):
        import torch
        n = len(weights)
        if not (len(xs) == len(ys) == n) or n == 0:
            raise GafError(_STATUS_INVALID_ARGUMENT, "weights, xs and ys must have one entry per operation")
        m = xs[0].shape[0]
        for w, x, y in zip(weights, xs, ys):
            if x.dtype != torch.bfloat16 or y.dtype != torch.bfloat16 or tuple(x.shape) != (m, w.K) or tuple(y.shape) != (m, w.N):
                raise GafError(_STATUS_INVALID_ARGUMENT, "x must be bf16 [m, K] and y bf16 [m, N], the same m for all")
            if not (x.is_contiguous() and y.is_contiguous()):
                raise GafError(_STATUS_INVALID_ARGUMENT, "buffers must be contiguous")
        self.ctx, self.n = ctx, n
        self._keep = (list(weights), list(xs), list(ys))
        wp = (C.c_void_p * n)(*[w._h.value if isinstance(w._h, C.c_void_p) else w._h for w in weights])
        xp = (C.c_void_p * n)(*[x.data_ptr() for x in xs])
        yp = (C.c_void_p * n)(*[y.data_ptr() for y in ys])
        dep = (C.c_uint8 * n)(*[1 if d else 0 for d in depends]) if depends is not None else None
        red = (C.c_uint8 * n)(*[1 if r else 0 for r in reduce]) if reduce is not None else None
        h = C.c_void_p()
        ctx._check(ctx._lib.tgaf_batch_create(ctx._h, n, wp, xp, m, yp, dep, red, C.byref(h)))
        self._h = h

    @property
    def one_launch(self) -> bool:
        return bool(self.ctx._lib.tgaf_batch_uses_one_launch(self._h))

    def run(self) -> None:
        self.ctx._check(self.ctx._lib.tgaf_batch_run(self.ctx._h, self._h))

    def close(self) -> None:
        if getattr(self, "_h", None) and getattr(self.ctx, "_h", None):
            self.ctx._lib.tgaf_batch_destroy(self.ctx._h, self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class HostBatch:
    """A fixed list of (weight, x, out) host-buffer calls, submitted with one crossing of the C ABI
    (tgaf_linear_bf16_host_async_batch).  x / out: uint16 arrays (bf16 bit patterns) in page-locked memory; they
    are read / written when `submit` runs on the GPU, so refill x and read out between ctx.synchronize() calls."""

    def __init__(self, ctx: Context, weights, xs, outs, reduce=None):
        n = len(weights)
        if not (len(xs) == len(outs) == n):
            raise GafError(_STATUS_INVALID_ARGUMENT, "weights, xs and outs must have one entry per call")
        for w, x, o in zip(weights, xs, outs):
            if x.dtype != np.uint16 or o.dtype != np.uint16 or x.ndim != 2 or x.shape[1] != w.K or o.shape != (x.shape[0], w.N):
                raise GafError(_STATUS_INVALID_ARGUMENT, "x must be uint16 [M, K] and out uint16 [M, N]")
            if not (x.flags.c_contiguous and o.flags.c_contiguous):
                raise GafError(_STATUS_INVALID_ARGUMENT, "buffers must be contiguous")
        self.ctx, self.n = ctx, n
        self._keep = (list(weights), list(xs), list(outs))
        self._w = (C.c_void_p * n)(*[w._h.value if isinstance(w._h, C.c_void_p) else w._h for w in weights])
        self._x = (C.c_void_p * n)(*[x.ctypes.data for x in xs])
        self._y = (C.c_void_p * n)(*[o.ctypes.data for o in outs])
        self._m = (C.c_uint32 * n)(*[x.shape[0] for x in xs])
        self._red = (C.c_uint8 * n)(*[1 if r else 0 for r in reduce]) if reduce is not None else None
        self._g = None

    def record(self) -> "HostBatch":
        """Runs the list once and records it as a CUDA graph (tgaf_host_batch_create); `submit` then replays it."""
        h = C.c_void_p()
        self.ctx._check(self.ctx._lib.tgaf_host_batch_create_reduce(self.ctx._h, self.n, self._w, self._x, self._m, self._y,
                                                                    self._red, C.byref(h)))
        self._g = h
        return self

    @property
    def one_launch(self) -> bool:
        """True when the recorded list is two block copies around ONE kernel launch."""
        return self._g is not None and bool(self.ctx._lib.tgaf_host_batch_uses_one_launch(self._g))

    def submit(self) -> None:
        if self._g is not None:
            self.ctx._check(self.ctx._lib.tgaf_host_batch_submit(self.ctx._h, self._g))
        elif self._red is not None and any(self._red):
            raise GafError(_STATUS_INVALID_ARGUMENT, "a list with sums over the ranks must be recorded first")
        else:
            self.ctx._check(self.ctx._lib.tgaf_linear_bf16_host_async_batch(self.ctx._h, self.n, self._w, self._x, self._m, self._y))

    def close(self) -> None:
        if self._g is not None and getattr(self.ctx, "_h", None):
            self.ctx._lib.tgaf_host_batch_destroy(self.ctx._h, self._g)
        self._g = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def dequant_f32(ctx: Context, w: Weight):
    import torch
    out = torch.empty((w.N, w.K), dtype=torch.float32, device=f"cuda:{ctx.device}")
    ctx._check(ctx._lib.tgaf_dequant_f32(ctx._h, w._h, C.c_void_p(out.data_ptr())))
    return out


def dequant_f32_host(ctx: Context, w: Weight) -> np.ndarray:
    out = np.empty((w.N, w.K), np.float32)
    ctx._check(ctx._lib.tgaf_dequant_f32_host(ctx._h, w._h, out.ctypes.data))
    return out


def embedding_lookup_f32(ctx: Context, w: Weight, token_ids, multiplier: float = 1.0):
    """Rows `token_ids` (host integers) of a gaf table, dequantized to f32 and scaled: [count, K] on the device."""
    import torch
    ids = np.ascontiguousarray(token_ids, dtype=np.uint32)
    out = torch.empty((ids.size, w.K), dtype=torch.float32, device=f"cuda:{ctx.device}")
    ctx._check(ctx._lib.tgaf_embedding_lookup_f32(ctx._h, w._h, ids.ctypes.data, ids.size, multiplier,
                                                  C.c_void_p(out.data_ptr())))
    return out


def gaffine_matvec_f32(ctx: Context, bits: int, input, packed, scales, biases, out, in_dim: int, out_dim: int,
                       group_size: int, scales_dtype_tag: int, batch_rows: int) -> None:
    """Raw device-pointer launch with the reference wrapper's argument list
    (core/src/compute/cuda/gaffine_u4_matvec.zig:58-97).  Arguments are torch device tensors."""
    fn = ctx._lib.tgaf_gaffine_u4_matvec_f32 if bits == 4 else ctx._lib.tgaf_gaffine_u8_matvec_f32
    ptr = lambda t: C.c_void_p(t.data_ptr() if t is not None else 0)
    ctx._check(fn(ctx._h, ptr(input), ptr(packed), ptr(scales), ptr(biases), ptr(out), in_dim, out_dim,
                  group_size, scales_dtype_tag, batch_rows))
