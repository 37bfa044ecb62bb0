"""Python side of the sm_100a kernels: library loading, launch wrappers, autograd Functions.

The kernels live in ``axlearn_b200/csrc`` and are linked into ``axlearn_b200/lib/libaxb200.so``
with plain C entry points.  They are called through ``ctypes`` with raw device pointers and the
current CUDA stream, so a launch costs a few microseconds of host time and nothing here
depends on a PyTorch C++ ABI.  If the library is missing it is built on first use (``nvcc``
cross-compiles without a GPU); if that is impossible, the first GPU op raises — there is no
silent fallback to library kernels.

Kernels that wait on hardware barriers do so with a bounded number of polls and report a
timeout in a per-device status word instead of hanging; ``check_status()`` raises if it is set.
"""

from __future__ import annotations

import ctypes
import math
import os
import threading
from typing import Optional, Sequence, Union

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "libaxb200.so")
_lib_lock = threading.Lock()
_lib_handle: Optional[ctypes.CDLL] = None
launch_count = 0  # Kernels launched through this module (bench.py reports it).
# SMs left free for communication kernels that run concurrently with compute (NCCL or the
# peer-memory copy kernels). The persistent GEMM launches at most (SM count - this) CTAs, so
# that all of its CTAs stay resident and its static tile schedule has no second wave.
COMM_RESERVED_SMS = int(os.environ.get("AXB200_COMM_SMS", "0"))
# "2cta": large GEMMs run on CTA pairs (256 x 256 tiles); "1cta": always the single-CTA kernel.
GEMM_VARIANT = os.environ.get("AXB200_GEMM", "2cta")
# RMSNorm kernels: "warp" (rows in registers, one or more warps per row) or "plain" (one CTA per row).
RMSNORM_VARIANT = os.environ.get("AXB200_RMSNORM", "warp")


def reserve_sms_for_comm(n: int) -> None:
    global COMM_RESERVED_SMS
    COMM_RESERVED_SMS = max(COMM_RESERVED_SMS, int(n))

c_void_p, c_int, c_int64, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float


def lib() -> ctypes.CDLL:
    global _lib_handle
    if _lib_handle is not None:
        return _lib_handle
    with _lib_lock:
        if _lib_handle is None:
            if not os.path.exists(_LIB_PATH):
                from axlearn_b200.csrc import build as _build

                _build.build()
            h = ctypes.CDLL(_LIB_PATH)
            for name in dir(_Sigs):
                if name.startswith("axb_"):
                    fn = getattr(h, name)
                    fn.argtypes = getattr(_Sigs, name)
                    fn.restype = c_int
            _lib_handle = h
    return _lib_handle


class _Sigs:
    axb_gemm_bf16 = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                     c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p]
    axb_gemm_bf16_2cta = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                          c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p]
    axb_gemm_splitk_plan = [c_int, c_int, c_int]
    axb_multimem_allreduce = [ctypes.c_uint64, c_int64, c_int, c_int, c_void_p]
    axb_gemm_bf16_splitk = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                            c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
    axb_rmsnorm_fwd = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_void_p]
    axb_rmsnorm_bwd_ctas = [c_int64]
    axb_rmsnorm_fast_supported = [c_int]
    axb_rmsnorm_fwd_fast = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_void_p]
    axb_rmsnorm_bwd_fast = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_int64, c_int, c_void_p]
    axb_rmsnorm_bwd = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_int64, c_int, c_void_p]
    axb_swiglu_fwd = [c_void_p, c_void_p, c_void_p, c_int64, c_void_p]
    axb_swiglu_bwd = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]
    axb_rope = [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p]
    axb_ce_fwd_bwd = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                      c_float, c_int64, c_int, c_int, c_void_p]
    axb_adamw = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_float,
                 c_float, c_float, c_float, c_float, c_float, c_float, c_void_p]
    axb_sumsq_ctas = []
    axb_sumsq = [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_float, c_int, c_void_p]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _check(rc: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if rc != 0:
        raise RuntimeError(f"{what}: launcher returned {rc}")


# ------------------------------------------------------------------------------------------
# Status word.
# ------------------------------------------------------------------------------------------

_status: dict[int, torch.Tensor] = {}

_STATUS_TEXT = {
    1: "TMA producer gave up waiting for a free stage",
    2: "MMA issuer gave up waiting for operands / accumulator",
    3: "epilogue gave up waiting for an accumulator",
    4: "gave up waiting for a peer flag",
    5: "bad argument detected on device",
}


def status_word(device: Optional[torch.device] = None) -> torch.Tensor:
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status[idx]


def check_status(device: Optional[torch.device] = None, *, clear: bool = True) -> None:
    """Raises if any kernel on ``device`` reported a bounded-wait timeout (synchronises)."""
    w = status_word(device)
    code = int(w.item())
    if code != 0:
        if clear:
            w.zero_()
        raise RuntimeError(f"device kernel reported status {code}: {_STATUS_TEXT.get(code, 'unknown')}")


# ------------------------------------------------------------------------------------------
# GEMM.
# ------------------------------------------------------------------------------------------


_sm_counts: dict[int, int] = {}


def _sm_count(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _sm_counts:
        _sm_counts[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_counts[idx]


def _operand(t: torch.Tensor, contraction_dim: int) -> tuple[torch.Tensor, int, int]:
    """Returns (tensor, mn_major flag, leading dim) for a 2-D bf16 operand whose contraction
    dim is ``contraction_dim``; copies only if the layout is unusable."""
    other = 1 - contraction_dim

    def usable(x):
        if x.stride(contraction_dim) == 1 and x.stride(other) % 8 == 0 and x.stride(other) >= x.shape[contraction_dim]:
            return 0, x.stride(other)
        if x.stride(other) == 1 and x.stride(contraction_dim) % 8 == 0 and x.stride(contraction_dim) >= x.shape[other]:
            return 1, x.stride(contraction_dim)
        return None

    # Degenerate dims (size 1) can make both strides look contiguous; prefer K-major.
    u = usable(t) if t.data_ptr() % 16 == 0 else None
    if u is None:
        t = t.contiguous()
        u = usable(t)
        if u is None:
            raise ValueError(f"GEMM operand of shape {tuple(t.shape)} needs dims that are multiples of 8")
    return t, u[0], u[1]


_splitk_plans: dict[tuple, int] = {}
_splitk_ws: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def _splitk_plan(m: int, n: int, k: int) -> int:
    key = (m > 0, n, k)
    if key not in _splitk_plans:
        _splitk_plans[key] = lib().axb_gemm_splitk_plan(m, n, k)
    return _splitk_plans[key]


def _splitk_workspace(device: torch.device, floats: int) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 partials + tile counters of the split-K skinny GEMM, one pair per (device, stream):
    launches on one stream are ordered, so they can share it.  (Allocated through torch, so a
    first use during CUDA-graph capture lands in the graph's pool.)"""
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream())
    have = _splitk_ws.get(key)
    if have is None or have[0].numel() < floats:
        ws = torch.empty(max(floats, 1 << 21), dtype=torch.float32, device=device)
        counters = have[1] if have is not None else torch.zeros(4096, dtype=torch.int32, device=device)
        have = (ws, counters)
        _splitk_ws[key] = have
    return have


def gemm(a: torch.Tensor, b: torch.Tensor, *, out: Optional[torch.Tensor] = None,
         out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False,
         max_ctas: int = 0) -> torch.Tensor:
    """``a[M, K] @ b[K, N]`` on the tcgen05 kernel; operands may be transposed views."""
    assert a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[0], (a.shape, b.shape)
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    m, k = a.shape
    n = b.shape[1]
    a, a_mn, lda = _operand(a, 1)
    b, b_mn, ldb = _operand(b, 0)
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    else:
        assert out.shape == (m, n) and out.stride(1) == 1
    if m == 0 or n == 0:
        return out
    if k == 0:
        return out if accumulate else out.zero_()
    if max_ctas == 0 and COMM_RESERVED_SMS:
        max_ctas = max(8, _sm_count(a.device) - COMM_RESERVED_SMS)
    if m <= 128 and n % 32 == 0:
        split = _splitk_plan(m, n, k)
        if split > 1:
            ws, counters = _splitk_workspace(a.device, split * m * n)
            rc = lib().axb_gemm_bf16_splitk(
                a.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k, lda, ldb, out.stride(0), a_mn, b_mn,
                1 if out.dtype == torch.float32 else 0, 1 if accumulate else 0, split, ws.data_ptr(),
                counters.data_ptr(), status_word(a.device).data_ptr(), max_ctas, _stream())
            _check(rc, "axb_gemm_bf16_splitk")
            return out
    if GEMM_VARIANT == "2cta" and m >= 512 and n >= 256 and ((m + 255) // 256) * ((n + 255) // 256) >= 64:
        # Large problems: CTA pairs on 256 x 256 tiles.
        rc = lib().axb_gemm_bf16_2cta(a.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k, lda, ldb, out.stride(0),
                                      a_mn, b_mn, 1 if out.dtype == torch.float32 else 0, 1 if accumulate else 0,
                                      status_word(a.device).data_ptr(), max_ctas, _stream())
        if rc != -20:
            _check(rc, "axb_gemm_bf16_2cta")
            return out
    rc = lib().axb_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k, lda, ldb, out.stride(0),
                             a_mn, b_mn, 1 if out.dtype == torch.float32 else 0, 1 if accumulate else 0,
                             status_word(a.device).data_ptr(), max_ctas, _stream())
    _check(rc, "axb_gemm_bf16")
    return out


def _fused_fsdp_info(w: torch.Tensor):
    """The pending-gather record of ``w`` when it is a weight matrix managed by the fused FSDP
    runtime (gather fused into the forward GEMM, gradient scatter into the weight-gradient GEMM)."""
    from axlearn_b200.parallel import fsdp_fused

    return fsdp_fused.lookup(w)


def _is_nk_view(w: torch.Tensor) -> bool:
    """True when ``w [K, N]`` is a transposed view of a row-major ``[N, K]`` tensor."""
    return w.stride(0) == 1 and w.stride(1) != 1


class _SharedInputGrad:
    """Input-gradient buffer shared by the linears that read the same activation (q / k / v, the
    two halves of a gated feed-forward): the first backward allocates it, the others add their
    ``dy @ w^T`` into it from the GEMM epilogue, and only the first returns it to autograd -- no
    separate add kernels.  Valid only when the marked tensor feeds nothing but such linears."""

    __slots__ = ("buf",)

    def __init__(self):
        self.buf = None


def share_input_grad(x: torch.Tensor) -> torch.Tensor:
    """Marks ``x`` (a fresh alias of it) as the common input of several kernel linears; see
    ``_SharedInputGrad``.  A no-op for tensors the GEMM kernel does not take."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.requires_grad and x.shape[-1] % 8 == 0):
        return x
    y = x.view_as(x)
    y._axb_shared_dx = _SharedInputGrad()  # pylint: disable=protected-access
    return y


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):  # x: [..., K], w: [K, N] (any strides)
        ctx.save_for_backward(x, w)
        ctx.shared_dx = getattr(x, "_axb_shared_dx", None)
        x2 = x.reshape(-1, x.shape[-1])
        info = _fused_fsdp_info(w)
        if info is not None and not (info.gathered and info.carry is None):
            from axlearn_b200.ops import fused_comm

            carry = info.take_carry()  # the same matrix of the neighbouring layer, if not there yet
            if not info.gathered:
                y = fused_comm.ag_gemm(x2, shard_ptrs=info.shard_ptrs, state=info.state, rank=info.rank,
                                       weight_is_nk=_is_nk_view(w), carry=carry)
                info.gathered = True
                info.state.holds = info.layer
            else:
                y = fused_comm.gemm_carrying_gather(x2, w, shard_ptrs=carry[0], state=carry[1], rank=info.rank)
        else:
            y = gemm(x2, w)
        return y.reshape(x.shape[:-1] + (w.shape[1],))

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            shared = getattr(ctx, "shared_dx", None)
            if shared is None:
                dx = gemm(dy2, w.t()).reshape(x.shape)
            elif shared.buf is None:
                shared.buf = gemm(dy2, w.t())
                dx = shared.buf.reshape(x.shape)
            else:
                gemm(dy2, w.t(), out=shared.buf, accumulate=True)   # autograd already holds the buffer
        if ctx.needs_input_grad[1]:
            info = _fused_fsdp_info(w)
            if info is not None:
                # Rows of the weight gradient go straight to the staging slots of their owners.
                from axlearn_b200.ops import fused_comm

                if _is_nk_view(w):
                    fused_comm.gemm_rs(dy2.t(), x2, staging_ptrs=info.staging_ptrs, rank=info.rank)
                else:
                    fused_comm.gemm_rs(x2.t(), dy2, staging_ptrs=info.staging_ptrs, rank=info.rank)
            elif _is_nk_view(w):
                # w is a transposed view of a row-major [N, K] tensor: produce the gradient
                # directly in that layout so the view's backward is free.
                dw = gemm(dy2.t(), x2).t()
            else:
                dw = gemm(x2.t(), dy2)
        return dx, dw


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    if x.shape[-1] % 8 or w.shape[1] % 8:
        return torch.matmul(x, w)
    return _Linear.apply(x, w)


class _LinearKept(_Linear):
    """``_Linear`` whose forward result ``y`` is already known (kept by a remat policy): no GEMM
    in forward; the backward GEMMs are those of ``_Linear``."""

    @staticmethod
    def forward(ctx, x, w, y):  # pylint: disable=arguments-differ
        ctx.save_for_backward(x, w)
        ctx.shared_dx = getattr(x, "_axb_shared_dx", None)
        return y.view_as(y)

    @staticmethod
    def backward(ctx, dy):
        return _Linear.backward(ctx, dy) + (None,)


def linear_kept(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    return _LinearKept.apply(x, w, y)


def carries_gather(w: torch.Tensor) -> bool:
    """True when the forward GEMM on ``w`` also gathers parameters (fused FSDP)."""
    return _fused_fsdp_info(w) is not None


# ------------------------------------------------------------------------------------------
# RMSNorm.
# ------------------------------------------------------------------------------------------


def _rmsnorm_forward(x2, residual2, scale_b, eps):
    """``(y, sum, rstd)``; ``sum`` is ``x + residual`` (None without a residual)."""
    rows, d = x2.shape
    y = torch.empty_like(x2)
    total = torch.empty_like(x2) if residual2 is not None else None
    rstd = torch.empty(rows, dtype=torch.float32, device=x2.device)
    args = (x2.data_ptr(), None if residual2 is None else residual2.data_ptr(), scale_b.data_ptr(), y.data_ptr(),
            None if total is None else total.data_ptr(), rstd.data_ptr(), rows, d, eps)
    if RMSNORM_VARIANT != "plain" and lib().axb_rmsnorm_fast_supported(d):
        _check(lib().axb_rmsnorm_fwd_fast(*args, _stream()), "axb_rmsnorm_fwd_fast")
    else:
        _check(lib().axb_rmsnorm_fwd(*args, _stream()), "axb_rmsnorm_fwd")
    return y, total, rstd


def _rmsnorm_backward(x2, scale_b, rstd, dy2, dres2):
    """``(dx [+ dres], dscale fp32)`` in one pass over the rows."""
    rows, d = x2.shape
    dx = torch.empty_like(x2)
    ctas = lib().axb_rmsnorm_bwd_ctas(rows)
    partial = torch.empty((max(ctas, 1), d), dtype=torch.float32, device=x2.device)
    dscale = torch.empty(d, dtype=torch.float32, device=x2.device)
    args = (x2.data_ptr(), scale_b.data_ptr(), rstd.data_ptr(), dy2.data_ptr(),
            None if dres2 is None else dres2.data_ptr(), dx.data_ptr(), partial.data_ptr(), None, dscale.data_ptr(), rows, d)
    if RMSNORM_VARIANT != "plain" and lib().axb_rmsnorm_fast_supported(d):
        _check(lib().axb_rmsnorm_bwd_fast(*args, _stream()), "axb_rmsnorm_bwd_fast")
    else:
        _check(lib().axb_rmsnorm_bwd(*args, _stream()), "axb_rmsnorm_bwd")
    return dx, dscale


def _rows(t: torch.Tensor) -> torch.Tensor:
    t2 = t.reshape(-1, t.shape[-1])
    return t2 if t2.is_contiguous() else t2.contiguous()


class _RmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, eps):
        x2 = _rows(x)
        scale_b = scale.to(torch.bfloat16).contiguous()
        y, _, rstd = _rmsnorm_forward(x2, None, scale_b, eps)
        ctx.save_for_backward(x2, scale_b, rstd)
        ctx.scale_dtype = scale.dtype
        ctx.x_shape = x.shape
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, scale_b, rstd = ctx.saved_tensors
        dx, dscale = _rmsnorm_backward(x2, scale_b, rstd, _rows(dy), None)
        return dx.reshape(ctx.x_shape), dscale.to(ctx.scale_dtype), None


class _RmsNormKeepInput(torch.autograd.Function):
    """``(rms_norm(x), x)``: the second output is the input itself, for the residual branch of a
    pre-norm block.  The gradient arriving through that branch is added inside the backward
    kernel, so no separate add runs."""

    @staticmethod
    def forward(ctx, x, scale, eps):
        x2 = _rows(x)
        scale_b = scale.to(torch.bfloat16).contiguous()
        y, _, rstd = _rmsnorm_forward(x2, None, scale_b, eps)
        ctx.save_for_backward(x2, scale_b, rstd)
        ctx.scale_dtype = scale.dtype
        ctx.x_shape = x.shape
        return y.reshape(x.shape), x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dskip):
        x2, scale_b, rstd = ctx.saved_tensors
        if dy is None:
            return dskip, None, None
        dx, dscale = _rmsnorm_backward(x2, scale_b, rstd, _rows(dy), None if dskip is None else _rows(dskip))
        return dx.reshape(ctx.x_shape), dscale.to(ctx.scale_dtype), None


class _AddRmsNorm(torch.autograd.Function):
    """``s = x + r`` and ``rms_norm(s)`` in one pass; backward gives ``ds + d rms_norm`` (one
    tensor, the gradient of both ``x`` and ``r``) in one pass."""

    @staticmethod
    def forward(ctx, x, r, scale, eps):
        x2, r2 = _rows(x), _rows(r)
        scale_b = scale.to(torch.bfloat16).contiguous()
        y, total, rstd = _rmsnorm_forward(x2, r2, scale_b, eps)
        ctx.save_for_backward(total, scale_b, rstd)
        ctx.scale_dtype = scale.dtype
        ctx.x_shape = x.shape
        return total.reshape(x.shape), y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dsum, dy):
        total, scale_b, rstd = ctx.saved_tensors
        if dy is None:
            return dsum, dsum, None, None
        dx, dscale = _rmsnorm_backward(total, scale_b, rstd, _rows(dy), None if dsum is None else _rows(dsum))
        dx = dx.reshape(ctx.x_shape)
        return dx, dx, dscale.to(ctx.scale_dtype), None


def rms_norm(x: torch.Tensor, scale: torch.Tensor, eps: float) -> torch.Tensor:
    if x.dtype != torch.bfloat16:
        from axlearn_b200.ops import reference

        return reference.rms_norm(x, scale, eps, upcast=True)
    return _RmsNorm.apply(x, scale, float(eps))


def rms_norm_keep_input(x: torch.Tensor, scale: torch.Tensor, eps: float):
    """``(rms_norm(x), x)`` with the residual-branch gradient folded into the backward kernel."""
    return _RmsNormKeepInput.apply(x, scale, float(eps))


def add_rms_norm(x: torch.Tensor, r: torch.Tensor, scale: torch.Tensor, eps: float):
    """``(x + r, rms_norm(x + r))`` in one pass each way."""
    return _AddRmsNorm.apply(x, r, scale, float(eps))


# ------------------------------------------------------------------------------------------
# SwiGLU / RoPE.
# ------------------------------------------------------------------------------------------


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        gate, up = gate.contiguous(), up.contiguous()
        out = torch.empty_like(gate)
        _check(lib().axb_swiglu_fwd(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(), _stream()),
               "axb_swiglu_fwd")
        ctx.save_for_backward(gate, up)
        return out

    @staticmethod
    def backward(ctx, dout):
        gate, up = ctx.saved_tensors
        dout = dout.contiguous()
        dg, du = torch.empty_like(gate), torch.empty_like(up)
        _check(lib().axb_swiglu_bwd(gate.data_ptr(), up.data_ptr(), dout.data_ptr(), dg.data_ptr(),
                                    du.data_ptr(), gate.numel(), _stream()), "axb_swiglu_bwd")
        return dg, du


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    if gate.numel() % 8:
        from axlearn_b200.ops import reference

        return reference.swiglu(gate, up)
    return _SwiGLU.apply(gate, up)


_rope_tables: dict = {}


def _rope_table(device: torch.device, floats: int) -> torch.Tensor:
    """Per-device scratch for the (sin, cos) table of one RoPE call (T * H floats).  Calls on
    one stream run in order, so the table of a finished call may be overwritten by the next."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    t = _rope_tables.get(key)
    if t is None or t.numel() < floats:
        t = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device)
        _rope_tables[key] = t
    return t


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, positions, theta):
        x = x.contiguous()
        b, t, n, h = x.shape
        pos = positions.to(device=x.device, dtype=torch.int64).contiguous()
        y = torch.empty_like(x)
        _check(lib().axb_rope(x.data_ptr(), y.data_ptr(), pos.data_ptr(), b, t, n, h, theta, 0,
                              _rope_table(x.device, t * h).data_ptr(), _stream()), "axb_rope")
        ctx.save_for_backward(pos)
        ctx.theta = theta
        return y

    @staticmethod
    def backward(ctx, dy):
        (pos,) = ctx.saved_tensors
        dy = dy.contiguous()
        b, t, n, h = dy.shape
        dx = torch.empty_like(dy)
        _check(lib().axb_rope(dy.data_ptr(), dx.data_ptr(), pos.data_ptr(), b, t, n, h, ctx.theta, 1,
                              _rope_table(dy.device, t * h).data_ptr(), _stream()), "axb_rope")
        return dx, None, None


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    return _Rope.apply(x, positions, float(theta))


# ------------------------------------------------------------------------------------------
# Cross entropy.
# ------------------------------------------------------------------------------------------


def ce_chunk(logits: torch.Tensor, targets: torch.Tensor, live: torch.Tensor, z_loss_scale: float,
             inv_denom: torch.Tensor, need_grad: bool):
    """Statistics of one ``[n, V]`` chunk; with ``need_grad`` the logits buffer is overwritten by
    d(loss)/d(logits).  Returns ``(sum_ce, sum_z, sum_correct, dlogits | None)``."""
    assert logits.dim() == 2 and logits.is_contiguous()
    n, v = logits.shape
    tg = targets.to(torch.int64).contiguous()
    lv = live.to(torch.uint8).contiguous()
    stats = torch.empty((3, n), dtype=torch.float32, device=logits.device)
    inv = inv_denom.reshape(1).to(device=logits.device, dtype=torch.float32)
    _check(lib().axb_ce_fwd_bwd(logits.data_ptr(), 1 if logits.dtype == torch.float32 else 0, tg.data_ptr(),
                                lv.data_ptr(), stats[0].data_ptr(), stats[1].data_ptr(), stats[2].data_ptr(),
                                inv.data_ptr(), float(z_loss_scale), n, v, 1 if need_grad else 0, _stream()),
           "axb_ce_fwd_bwd")
    sums = stats.sum(dim=1)
    return sums[0], sums[1], sums[2], (logits if need_grad else None)


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, live, z_loss_scale, denom):
        v = logits.shape[-1]
        work = logits.reshape(-1, v).clone()  # The kernel writes the gradient in place.
        inv = (1.0 / denom).to(torch.float32)
        need = ctx.needs_input_grad[0]
        ce, z, correct, dl = ce_chunk(work, targets.reshape(-1), live.reshape(-1), z_loss_scale, inv, need)
        if need:
            ctx.save_for_backward(dl)
            ctx.shape = logits.shape
        loss = (ce + z_loss_scale * z) * inv
        ctx.mark_non_differentiable(ce, z, correct)
        return loss, ce * inv, z * inv, correct * inv

    @staticmethod
    def backward(ctx, g, *_):
        (dl,) = ctx.saved_tensors
        return (dl * g.to(dl.dtype)).reshape(ctx.shape), None, None, None, None


def cross_entropy(logits, targets, *, live_targets=None, z_loss_scale: float = 0.0, denominator=None):
    v = logits.shape[-1]
    if live_targets is None:
        live_targets = (targets >= 0) & (targets < v)
    num_live = live_targets.sum().to(torch.float32)
    denom = num_live.clamp_min(1.0) if denominator is None else denominator.to(torch.float32)
    loss, ce, z, acc = _CrossEntropy.apply(logits, targets, live_targets, float(z_loss_scale), denom)
    return loss, {"cross_entropy_loss": ce, "z_loss": z, "accuracy": acc, "num_live": num_live}


# ------------------------------------------------------------------------------------------
# Optimizer.
# ------------------------------------------------------------------------------------------

_scale_one: dict[int, torch.Tensor] = {}


def multi_tensor_adamw(params, grads, mus, nus, shadows, wd_scales, *, step: int, lr: float,
                       weight_decay: float, b1: float, b2: float, eps: float,
                       grad_scale: Union[float, torch.Tensor] = 1.0) -> None:
    dev = params[0].device
    if isinstance(grad_scale, torch.Tensor):
        gs = grad_scale.reshape(1).to(device=dev, dtype=torch.float32)
    else:
        gs = torch.full((1,), float(grad_scale), dtype=torch.float32, device=dev)
    bc1, bc2 = 1.0 - b1**step, 1.0 - b2**step
    h = lib()
    stream = _stream()
    for p, g, m, v, sh, ws in zip(params, grads, mus, nus, shadows, wd_scales):
        assert p.is_contiguous() and m.is_contiguous() and v.is_contiguous()
        g = g.contiguous()
        if g.dtype not in (torch.bfloat16, torch.float32):
            g = g.float()
        shadow_ptr = None
        if sh is not None and sh is not p:
            assert sh.dtype == torch.bfloat16 and sh.is_contiguous()
            shadow_ptr = sh.data_ptr()
        _check(h.axb_adamw(p.data_ptr(), g.data_ptr(), 1 if g.dtype == torch.bfloat16 else 0, m.data_ptr(),
                           v.data_ptr(), shadow_ptr, gs.data_ptr(), p.numel(), lr, weight_decay * ws, b1, b2,
                           eps, bc1, bc2, stream), "axb_adamw")


def sum_of_squares(tensors: Sequence[torch.Tensor], weights: Optional[Sequence[float]] = None) -> torch.Tensor:
    """Deterministic ``sum_i w_i * ||t_i||^2`` as a 0-d fp32 device tensor."""
    dev = tensors[0].device
    h = lib()
    out = torch.zeros(1, dtype=torch.float32, device=dev)
    partial = torch.empty(h.axb_sumsq_ctas(), dtype=torch.float32, device=dev)
    stream = _stream()
    for i, t in enumerate(tensors):
        if t.dtype not in (torch.bfloat16, torch.float32):
            t = t.float()
        t = t.contiguous()
        w = 1.0 if weights is None else float(weights[i])
        _check(h.axb_sumsq(t.data_ptr(), 1 if t.dtype == torch.bfloat16 else 0, t.numel(), partial.data_ptr(),
                           out.data_ptr(), w, 1, stream), "axb_sumsq")
    return out[0]


# ------------------------------------------------------------------------------------------
# Attention and KV-cache kernels are wired in axlearn_b200/ops/attention_ops.py.
# ------------------------------------------------------------------------------------------


def flash_supported(q, k, v, segment_ids) -> bool:
    from axlearn_b200.ops import attention_ops

    return attention_ops.flash_supported(q, k, v, segment_ids)


def flash_attention(q, k, v, *, causal: bool, softmax_scale: Optional[float], segment_ids=None, **masks):
    from axlearn_b200.ops import attention_ops

    return attention_ops.flash_attention(q, k, v, causal=causal, softmax_scale=softmax_scale, segment_ids=segment_ids,
                                         **masks)


def paged_kv_append(pages, new, page_ids, offsets):
    from axlearn_b200.ops import attention_ops

    return attention_ops.paged_kv_append(pages, new, page_ids, offsets)
