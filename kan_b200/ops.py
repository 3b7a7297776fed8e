"""Functional wrappers: torch CUDA tensors in, C-ABI calls underneath.

PyTorch provides device memory and streams only; all arithmetic happens in the
sm_100a kernels of libchebykan_b200.so.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib
from ._lib import MODES, OP_BWD_DCOEFF, OP_BWD_DX

_status = {}  # device index -> int32[1] tensor the tensor-core kernels report into

# KAN_B200_NVTX=1: every library call of this module runs inside an NVTX range named after the operation, so that a
# timeline shows pack / forward / dC / dx / optimizer / loss next to torch's own ranges (off by default: no overhead)
_NVTX = os.environ.get("KAN_B200_NVTX", "0") == "1"


class _Range:
    def __init__(self, name):
        self.name = name

    def __enter__(self):
        if _NVTX:
            torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        if _NVTX:
            torch.cuda.nvtx.range_pop()
        return False


def _mode(mode) -> int:
    if isinstance(mode, str):
        if mode not in MODES:
            raise ValueError(f"math_mode must be one of {sorted(MODES)}, got {mode!r}")
        return MODES[mode]
    return int(mode)


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _require(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: kan_b200 has no CPU path")
    if t.dtype != torch.float32:
        raise RuntimeError(f"expected scalar type Float but found {str(t.dtype).replace('torch.', '')} for {name}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.data_ptr() % 16 != 0 and t.numel() > 0:
        raise RuntimeError(f"{name} must be 16-byte aligned")


def status_tensor(device) -> torch.Tensor:
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status[idx]


def check_status(device=None) -> None:
    """Synchronise and raise if a tensor-core kernel reported a wait that gave up."""
    devs = list(_status) if device is None else [torch.device(device).index or 0]
    for idx in devs:
        if idx in _status:
            code = int(_status[idx].item())
            if code:
                _status[idx].zero_()
                raise RuntimeError(f"chebykan kernel on cuda:{idx} gave up a bounded wait (role code {code})")


def packed_bytes(in_dim: int, out_dim: int, degree: int, mode) -> int:
    n = _lib.load().chebykan_packed_bytes(in_dim, out_dim, degree, _mode(mode))
    _lib.check(n, "chebykan_packed_bytes")
    return n


def pack_coeffs(coeffs: torch.Tensor, mode, out: torch.Tensor | None = None) -> torch.Tensor:
    """cheby_coeffs[in,out,deg+1] -> the library's private GEMM operand layout."""
    _require(coeffs, "coeffs")
    if coeffs.dim() != 3:
        raise RuntimeError("coeffs must have shape [in, out, degree+1]")
    n_in, n_out, dp1 = coeffs.shape
    m = _mode(mode)
    nbytes = packed_bytes(n_in, n_out, dp1 - 1, m)
    if out is None:
        out = torch.empty(nbytes, dtype=torch.uint8, device=coeffs.device)
    elif out.numel() * out.element_size() < nbytes or out.device != coeffs.device:
        raise RuntimeError("packed buffer too small or on another device")
    with _Range("chebykan.pack"), torch.cuda.device(coeffs.device):
        rc = _lib.load().chebykan_pack_coeffs(coeffs.data_ptr(), out.data_ptr(), n_in, n_out, dp1 - 1, m,
                                              _stream(coeffs))
    _lib.check(rc, "chebykan_pack_coeffs")
    return out


def forward(x: torch.Tensor, packed: torch.Tensor, in_dim: int, out_dim: int, degree: int, mode,
            out: torch.Tensor | None = None) -> torch.Tensor:
    """y[B,out] from x[B,in] and a packed coefficient buffer of the same mode."""
    _require(x, "x")
    if x.dim() != 2 or x.shape[1] != in_dim:
        raise RuntimeError(f"x must have shape [B, {in_dim}]")
    m = _mode(mode)
    B = x.shape[0]
    if out is None:
        out = torch.empty(B, out_dim, dtype=torch.float32, device=x.device)
    else:
        _require(out, "out")
    with _Range("chebykan.forward"), torch.cuda.device(x.device):
        rc = _lib.load().chebykan_fwd(x.data_ptr(), packed.data_ptr(), out.data_ptr(), B, in_dim, out_dim,
                                      degree, m, status_tensor(x.device).data_ptr(), _stream(x))
    _lib.check(rc, "chebykan_fwd")
    return out


def forward_ln(x: torch.Tensor, packed: torch.Tensor, in_dim: int, out_dim: int, degree: int, mode,
               ln_in=None, stats_out: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Forward with a fused LayerNorm on the input (ln_in = (stats[B,2], gamma, beta, eps)) and/or
    row sums of y accumulated into `stats_out` ([B,2], zeroed by the caller).  Tensor-core modes only."""
    _require(x, "x")
    if x.dim() != 2 or x.shape[1] != in_dim:
        raise RuntimeError(f"x must have shape [B, {in_dim}]")
    B = x.shape[0]
    if out is None:
        out = torch.empty(B, out_dim, dtype=torch.float32, device=x.device)
    else:
        _require(out, "out")
    st_in = g = b = 0
    eps = 1e-5
    if ln_in is not None:
        stats, gamma, beta, eps = ln_in
        for t, n in ((stats, "ln stats"), (gamma, "ln gamma"), (beta, "ln beta")):
            _require(t, n)
        if stats.shape != (B, 2) or gamma.numel() != in_dim or beta.numel() != in_dim:
            raise RuntimeError("LayerNorm statistics must be [B, 2] and gamma/beta [in]")
        st_in, g, b = stats.data_ptr(), gamma.data_ptr(), beta.data_ptr()
    so = 0
    if stats_out is not None:
        _require(stats_out, "stats_out")
        if stats_out.shape != (B, 2):
            raise RuntimeError("stats_out must be [B, 2]")
        so = stats_out.data_ptr()
    with _Range("chebykan.forward_ln"), torch.cuda.device(x.device):
        rc = _lib.load().chebykan_fwd_ln(x.data_ptr(), packed.data_ptr(), out.data_ptr(), B, in_dim, out_dim, degree,
                                         _mode(mode), st_in, g, b, float(eps), so,
                                         status_tensor(x.device).data_ptr(), _stream(x))
    _lib.check(rc, "chebykan_fwd_ln")
    return out


def bwd_dcoeff(x: torch.Tensor, dy: torch.Tensor, in_dim: int, out_dim: int, degree: int, mode,
               out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """dC[in,out,deg+1] = sum_b T_d(tanh x[b,i]) dY[b,o]."""
    _require(x, "x")
    _require(dy, "dy")
    B = x.shape[0]
    if x.shape != (B, in_dim) or dy.shape != (B, out_dim):
        raise RuntimeError("x must be [B, in] and dy [B, out]")
    m = _mode(mode)
    lib = _lib.load()
    if out is None:
        out = torch.empty(in_dim, out_dim, degree + 1, dtype=torch.float32, device=x.device)
        accumulate = False
    else:
        _require(out, "out")
    ws_bytes = lib.chebykan_workspace_bytes(OP_BWD_DCOEFF, B, in_dim, out_dim, degree, m)
    _lib.check(ws_bytes, "chebykan_workspace_bytes")
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=x.device)
    with _Range("chebykan.dcoeff"), torch.cuda.device(x.device):
        rc = lib.chebykan_bwd_dcoeff(x.data_ptr(), dy.data_ptr(), out.data_ptr(), ws.data_ptr(), ws_bytes, B,
                                     in_dim, out_dim, degree, m, int(accumulate),
                                     status_tensor(x.device).data_ptr(), _stream(x))
    _lib.check(rc, "chebykan_bwd_dcoeff")
    return out


def bwd_dx(x: torch.Tensor, dy: torch.Tensor, coeffs: torch.Tensor, mode,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """dx[B,in] = (1-t^2) sum_d T_d'(t) sum_o dY[b,o] C[i,o,d]."""
    _require(x, "x")
    _require(dy, "dy")
    _require(coeffs, "coeffs")
    n_in, n_out, dp1 = coeffs.shape
    B = x.shape[0]
    if x.shape != (B, n_in) or dy.shape != (B, n_out):
        raise RuntimeError("x must be [B, in] and dy [B, out]")
    if out is None:
        out = torch.empty_like(x)
    else:
        _require(out, "out")
    lib = _lib.load()
    m = _mode(mode)
    ws_bytes = lib.chebykan_workspace_bytes(OP_BWD_DX, B, n_in, n_out, dp1 - 1, m)
    _lib.check(ws_bytes, "chebykan_workspace_bytes")
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=x.device)
    with _Range("chebykan.dx"), torch.cuda.device(x.device):
        rc = lib.chebykan_bwd_dx(x.data_ptr(), dy.data_ptr(), coeffs.data_ptr(), out.data_ptr(), ws.data_ptr(),
                                 ws_bytes, B, n_in, n_out, dp1 - 1, m,
                                 status_tensor(x.device).data_ptr(), _stream(x))
    _lib.check(rc, "chebykan_bwd_dx")
    return out


def jacobian(x: torch.Tensor, coeffs: torch.Tensor) -> torch.Tensor:
    """J[B, out, in] = d y / d x of the layer (the derivative autograd gives), fp32."""
    _require(x, "x")
    _require(coeffs, "coeffs")
    n_in, n_out, dp1 = coeffs.shape
    if x.dim() != 2 or x.shape[1] != n_in:
        raise RuntimeError(f"x must have shape [B, {n_in}]")
    B = x.shape[0]
    out = torch.empty(B, n_out, n_in, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().chebykan_jacobian(x.data_ptr(), coeffs.data_ptr(), out.data_ptr(), B, n_in, n_out, dp1 - 1,
                                           _stream(x))
    _lib.check(rc, "chebykan_jacobian")
    return out


def normalize_input(x: torch.Tensor) -> torch.Tensor:
    """t = tanh(x), the basis object's input normalisation (correctly rounded fp32)."""
    _require(x, "x")
    t = torch.empty_like(x)
    with torch.cuda.device(x.device):
        rc = _lib.load().chebykan_normalize_input(x.data_ptr(), t.data_ptr(), x.numel(), _stream(x))
    _lib.check(rc, "chebykan_normalize_input")
    return t


def basis_functions(t: torch.Tensor, degree: int) -> torch.Tensor:
    """Phi[..., d] = T_d(t) for d = 0..degree; `t` holds normalised inputs in [-1, 1]."""
    _require(t, "t")
    phi = torch.empty(*t.shape, degree + 1, dtype=torch.float32, device=t.device)
    with torch.cuda.device(t.device):
        rc = _lib.load().chebykan_basis_functions(t.data_ptr(), phi.data_ptr(), t.numel(), degree, _stream(t))
    _lib.check(rc, "chebykan_basis_functions")
    return phi


# ---------------------------------------------------------------------------------------------------------------
# Jacobi / Hermite layers: the fp32 kernels with the family's recurrence as a launch parameter
# ---------------------------------------------------------------------------------------------------------------
def make_family(kind: str, alpha: float = 0.0, beta: float = 0.0, scale: float = 0.0, affine: bool = False,
                shift: float = 0.0, offset: float = 0.0) -> "_lib.Family":
    """Host-side description of a polynomial family: kind in {'chebyshev', 'jacobi', 'hermite', 'hermite_prob'};
    u = scale * tanh(x) (scale 0 = the kind's default) or, with affine, u = scale * (x - shift) + offset."""
    kinds = {"chebyshev": _lib.FAMILY_CHEBYSHEV, "jacobi": _lib.FAMILY_JACOBI, "hermite": _lib.FAMILY_HERMITE,
             "hermite_prob": _lib.FAMILY_HERMITE_PROB}
    if kind not in kinds:
        raise ValueError(f"family must be one of {sorted(kinds)}, got {kind!r}")
    return _lib.Family(kinds[kind], float(alpha), float(beta), int(bool(affine)), float(scale), float(shift),
                       float(offset))


def family_table(family, degree: int):
    """(a, b, c) of P_d = (a[d] u + b[d]) P_{d-1} - c[d] P_{d-2} as the kernels use them: three CPU float32
    tensors of degree+1 entries (entry 0 unused).  Host only: needs no GPU."""
    bufs = [(ctypes.c_float * (degree + 1))() for _ in range(3)]
    rc = _lib.load().chebykan_family_table(ctypes.byref(family), degree, *[ctypes.addressof(b) for b in bufs])
    _lib.check(rc, "chebykan_family_table")
    return tuple(torch.tensor(list(b), dtype=torch.float32) for b in bufs)


def family_forward(family, x: torch.Tensor, packed: torch.Tensor, in_dim: int, out_dim: int, degree: int,
                   mode="fp32", out: torch.Tensor | None = None) -> torch.Tensor:
    """y[B,out] = sum_i sum_d C[i,o,d] P_d(u(x[b,i])) from coefficients packed for `mode` ('fp32', 'tf32' or 'bf16')."""
    _require(x, "x")
    if x.dim() != 2 or x.shape[1] != in_dim:
        raise RuntimeError(f"x must have shape [B, {in_dim}]")
    m = _mode(mode)
    need = packed_bytes(in_dim, out_dim, degree, m)
    if packed.numel() * packed.element_size() < need:
        raise RuntimeError("packed coefficient buffer is too small for this shape")
    B = x.shape[0]
    if out is None:
        out = torch.empty(B, out_dim, dtype=torch.float32, device=x.device)
    else:
        _require(out, "out")
        if out.shape != (B, out_dim):
            raise RuntimeError(f"out must have shape [{B}, {out_dim}]")
    with _Range("chebykan.family_forward"), torch.cuda.device(x.device):
        rc = _lib.load().chebykan_family_fwd(ctypes.byref(family), x.data_ptr(), packed.data_ptr(), out.data_ptr(), B,
                                             in_dim, out_dim, degree, m, status_tensor(x.device).data_ptr(), _stream(x))
    _lib.check(rc, "chebykan_family_fwd")
    return out


def family_bwd_dcoeff(family, x: torch.Tensor, dy: torch.Tensor, in_dim: int, out_dim: int, degree: int,
                      mode="fp32", out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """dC[in,out,deg+1] = sum_b P_d(u(x[b,i])) dY[b,o]; 'tf32' / 'bf16' contract on the tensor cores in tf32."""
    _require(x, "x")
    _require(dy, "dy")
    B = x.shape[0]
    if x.shape != (B, in_dim) or dy.shape != (B, out_dim):
        raise RuntimeError("x must be [B, in] and dy [B, out]")
    lib = _lib.load()
    m = _mode(mode)
    if out is None:
        out = torch.empty(in_dim, out_dim, degree + 1, dtype=torch.float32, device=x.device)
        accumulate = False
    else:
        _require(out, "out")
    ws_bytes = lib.chebykan_family_workspace_bytes(OP_BWD_DCOEFF, B, in_dim, out_dim, degree, m)
    _lib.check(ws_bytes, "chebykan_family_workspace_bytes")
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=x.device)
    with _Range("chebykan.family_dcoeff"), torch.cuda.device(x.device):
        rc = lib.chebykan_family_bwd_dcoeff(ctypes.byref(family), x.data_ptr(), dy.data_ptr(), out.data_ptr(),
                                            ws.data_ptr(), ws_bytes, B, in_dim, out_dim, degree, m, int(accumulate),
                                            status_tensor(x.device).data_ptr(), _stream(x))
    _lib.check(rc, "chebykan_family_bwd_dcoeff")
    return out


def family_bwd_dx(family, x: torch.Tensor, dy: torch.Tensor, coeffs: torch.Tensor, mode="fp32",
                  out: torch.Tensor | None = None) -> torch.Tensor:
    """dx[B,in] = du/dx * sum_d P_d'(u) sum_o dY[b,o] C[i,o,d]; 'tf32' / 'bf16' contract on the tensor cores in tf32."""
    _require(x, "x")
    _require(dy, "dy")
    _require(coeffs, "coeffs")
    n_in, n_out, dp1 = coeffs.shape
    B = x.shape[0]
    if x.shape != (B, n_in) or dy.shape != (B, n_out):
        raise RuntimeError("x must be [B, in] and dy [B, out]")
    if out is None:
        out = torch.empty_like(x)
    else:
        _require(out, "out")
    lib = _lib.load()
    m = _mode(mode)
    ws_bytes = lib.chebykan_family_workspace_bytes(OP_BWD_DX, B, n_in, n_out, dp1 - 1, m)
    _lib.check(ws_bytes, "chebykan_family_workspace_bytes")
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=x.device)
    with _Range("chebykan.family_dx"), torch.cuda.device(x.device):
        rc = lib.chebykan_family_bwd_dx(ctypes.byref(family), x.data_ptr(), dy.data_ptr(), coeffs.data_ptr(),
                                        out.data_ptr(), ws.data_ptr(), ws_bytes, B, n_in, n_out, dp1 - 1, m,
                                        status_tensor(x.device).data_ptr(), _stream(x))
    _lib.check(rc, "chebykan_family_bwd_dx")
    return out


def family_normalize(family, x: torch.Tensor) -> torch.Tensor:
    """u(x): the family's input normalisation, element-wise."""
    _require(x, "x")
    u = torch.empty_like(x)
    with torch.cuda.device(x.device):
        rc = _lib.load().chebykan_family_normalize(ctypes.byref(family), x.data_ptr(), u.data_ptr(), x.numel(), _stream(x))
    _lib.check(rc, "chebykan_family_normalize")
    return u


def family_basis(family, u: torch.Tensor, degree: int) -> torch.Tensor:
    """Phi[..., d] = P_d(u) for d = 0..degree at already normalised points u."""
    _require(u, "u")
    phi = torch.empty(*u.shape, degree + 1, dtype=torch.float32, device=u.device)
    with torch.cuda.device(u.device):
        rc = _lib.load().chebykan_family_basis(ctypes.byref(family), u.data_ptr(), phi.data_ptr(), u.numel(), degree,
                                               _stream(u))
    _lib.check(rc, "chebykan_family_basis")
    return phi


_mse_ws = {}  # device index -> per-block partial sums of the loss kernel


def mse_loss_grad(y: torch.Tensor, target: torch.Tensor, n_mean: int | None = None, grad_scale: float = 1.0):
    """(loss, dy): loss = sum (y - target)^2 / n_mean (a device scalar) and dy = 2 (y - target) / n_mean * grad_scale,
    from one pass over y and target.  n_mean defaults to y.numel()."""
    _require(y, "y")
    _require(target, "target")
    if y.shape != target.shape:
        raise RuntimeError("y and target must have the same shape")
    n = y.numel()
    if n == 0:
        raise RuntimeError("mse_loss_grad needs at least one element")
    lib = _lib.load()
    idx = y.device.index if y.device.index is not None else torch.cuda.current_device()
    ws = _mse_ws.get(idx)
    if ws is None:
        ws = _mse_ws[idx] = torch.empty(lib.chebykan_mse_workspace_bytes(), dtype=torch.uint8, device=y.device)
    dy = torch.empty_like(y)
    loss = torch.empty((), dtype=torch.float32, device=y.device)
    with _Range("chebykan.mse_loss"), torch.cuda.device(y.device):
        rc = lib.chebykan_mse_loss_grad(y.data_ptr(), target.data_ptr(), dy.data_ptr(), loss.data_ptr(), ws.data_ptr(),
                                        ws.numel(), n, int(n_mean or n), float(grad_scale), _stream(y))
    _lib.check(rc, "chebykan_mse_loss_grad")
    return loss, dy


def scale_by_device_scalar(dy: torch.Tensor, scalar: torch.Tensor) -> torch.Tensor:
    """dy *= scalar (a one-element CUDA tensor) in place; a scalar of exactly 1 leaves dy untouched."""
    _require(dy, "dy")
    _require(scalar, "scalar")
    if scalar.numel() != 1:
        raise RuntimeError("scalar must hold one element")
    with torch.cuda.device(dy.device):
        rc = _lib.load().chebykan_scale_by_device_scalar(dy.data_ptr(), scalar.data_ptr(), dy.numel(), _stream(dy))
    _lib.check(rc, "chebykan_scale_by_device_scalar")
    return dy


def sgd_step(param: torch.Tensor, grad: torch.Tensor, lr: float, grad_scale: float = 1.0) -> None:
    _require(param, "param")
    _require(grad, "grad")
    if grad.numel() != param.numel():
        raise RuntimeError("grad and param sizes differ")
    with _Range("chebykan.sgd"), torch.cuda.device(param.device):
        rc = _lib.load().chebykan_sgd_step(param.data_ptr(), grad.data_ptr(), param.numel(), lr, grad_scale,
                                           _stream(param))
    _lib.check(rc, "chebykan_sgd_step")


def adam_step(param: torch.Tensor, grad: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor,
              step: int, lr: float, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
              grad_scale: float = 1.0) -> None:
    for t, n in ((param, "param"), (grad, "grad"), (exp_avg, "exp_avg"), (exp_avg_sq, "exp_avg_sq")):
        _require(t, n)
        if t.numel() != param.numel():
            raise RuntimeError(f"{n} and param sizes differ")
    with _Range("chebykan.adam"), torch.cuda.device(param.device):
        rc = _lib.load().chebykan_adam_step(param.data_ptr(), grad.data_ptr(), exp_avg.data_ptr(),
                                            exp_avg_sq.data_ptr(), param.numel(), lr, beta1, beta2, eps, step,
                                            grad_scale, _stream(param))
    _lib.check(rc, "chebykan_adam_step")


def adam_step_graph(param: torch.Tensor, grad: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor,
                    step_dev: torch.Tensor, lr: float, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
                    grad_scale: float = 1.0) -> None:
    """Adam update with the step counter in device memory (int64[1]); safe to capture in a CUDA graph."""
    for t, n in ((param, "param"), (grad, "grad"), (exp_avg, "exp_avg"), (exp_avg_sq, "exp_avg_sq")):
        _require(t, n)
        if t.numel() != param.numel():
            raise RuntimeError(f"{n} and param sizes differ")
    if step_dev.dtype != torch.int64 or not step_dev.is_cuda or step_dev.numel() != 1:
        raise RuntimeError("step_dev must be a CUDA int64 tensor with one element")
    with _Range("chebykan.adam"), torch.cuda.device(param.device):
        rc = _lib.load().chebykan_adam_step_graph(param.data_ptr(), grad.data_ptr(), exp_avg.data_ptr(),
                                                  exp_avg_sq.data_ptr(), param.numel(), lr, beta1, beta2, eps,
                                                  step_dev.data_ptr(), grad_scale, _stream(param))
    _lib.check(rc, "chebykan_adam_step_graph")


def forward_host(x_host: torch.Tensor, coeffs_host: torch.Tensor, mode, scratch: torch.Tensor | None = None,
                 out: torch.Tensor | None = None):
    """Forward with HOST tensors through chebykan_fwd_host; returns (y_host, scratch).

    x_host / coeffs_host / out are CPU fp32 tensors (pinned memory makes the
    copies asynchronous DMA); `scratch` is a reusable device byte buffer.
    """
    if x_host.is_cuda or coeffs_host.is_cuda:
        raise RuntimeError("forward_host takes host tensors")
    if x_host.dtype != torch.float32 or coeffs_host.dtype != torch.float32:
        raise RuntimeError("expected scalar type Float")
    n_in, n_out, dp1 = coeffs_host.shape
    x2 = x_host.view(-1, n_in)
    B = x2.shape[0]
    m = _mode(mode)
    lib = _lib.load()
    need = lib.chebykan_fwd_host_scratch_bytes(B, n_in, n_out, dp1 - 1, m)
    _lib.check(need, "chebykan_fwd_host_scratch_bytes")
    if scratch is None or scratch.numel() < need:
        scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    if out is None:
        out = torch.empty(B, n_out, dtype=torch.float32, pin_memory=True)
    with torch.cuda.device(scratch.device):
        rc = lib.chebykan_fwd_host(x2.data_ptr(), coeffs_host.data_ptr(), out.data_ptr(), scratch.data_ptr(),
                                   scratch.numel(), B, n_in, n_out, dp1 - 1, m,
                                   torch.cuda.current_stream(scratch.device).cuda_stream)
    _lib.check(rc, "chebykan_fwd_host")
    return out, scratch


def forward_host_packed(x_host: torch.Tensor, packed: torch.Tensor, n_in: int, n_out: int, degree: int, mode,
                        out: torch.Tensor | None = None, chunk_rows: int = 8192,
                        scratch: torch.Tensor | None = None):
    """Pipelined forward with HOST x / y and device-resident packed coefficients (chebykan_fwd_host_packed):
    blocks of `chunk_rows` rows are copied in, computed and copied back concurrently.  Returns (y_host, scratch);
    `scratch` is a reusable device byte buffer.  Synchronous."""
    if x_host.is_cuda:
        raise RuntimeError("forward_host_packed takes a host tensor")
    if x_host.dtype != torch.float32:
        raise RuntimeError("expected scalar type Float")
    if not packed.is_cuda:
        raise RuntimeError("packed coefficients must live on the GPU")
    x2 = x_host.view(-1, n_in)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    B = x2.shape[0]
    rows = max(1, min(int(chunk_rows), max(B, 1)))
    lib = _lib.load()
    need = lib.chebykan_fwd_host_packed_scratch_bytes(rows, n_in, n_out)
    _lib.check(need, "chebykan_fwd_host_packed_scratch_bytes")
    if scratch is None or scratch.numel() < need or scratch.device != packed.device:
        scratch = torch.empty(need, dtype=torch.uint8, device=packed.device)
    if out is None:
        out = torch.empty(B, n_out, dtype=torch.float32, pin_memory=True)
    with _Range("chebykan.forward_host"), torch.cuda.device(packed.device):
        rc = lib.chebykan_fwd_host_packed(x2.data_ptr(), packed.data_ptr(), out.data_ptr(), scratch.data_ptr(),
                                          scratch.numel(), B, n_in, n_out, degree, _mode(mode), rows,
                                          torch.cuda.current_stream(packed.device).cuda_stream)
    _lib.check(rc, "chebykan_fwd_host_packed")
    return out, scratch
