"""Row-wise L2 normalisation of q/k and its gradient.

Same contract as the reference's ``flash_qla/utils/math.py:9-101`` (``l2norm_fwd`` returns the
normalised tensor in the input dtype and the fp32 reciprocal norm; ``l2norm_bwd`` maps the
gradient of the normalised tensor back).  An optional pre-op of the path
(``use_qk_l2norm_in_kernel``); on CUDA tensors both run as one-pass kernels of the library
(``csrc/l2norm.cu``).
"""

from __future__ import annotations

import torch

from .contiguous import input_guard


_DTYPE_CODE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _on_gpu_kernel(*tensors) -> bool:
    return all(t.is_cuda and t.dtype in _DTYPE_CODE for t in tensors)


def l2norm_fwd(x: torch.Tensor, eps: float = 1e-6, dim: int = -1):
    """``(y, rstd)``: ``y = x * rsqrt(sum(x^2) + eps)`` in the dtype of ``x``, ``rstd`` fp32 with
    the shape of ``x`` without its last axis.  CUDA tensors go through ``fqla_l2norm_fwd`` (one
    pass over the rows); tensors on the host are evaluated with torch ops, as the reference does
    everywhere."""
    assert dim == -1 or dim == x.dim() - 1
    assert x.stride(-1) == 1
    D = x.shape[-1]
    if _on_gpu_kernel(x) and D % 2 == 0 and D <= 512:
        from .. import _lib

        xc = x.contiguous()
        y = torch.empty_like(xc)
        rstd = torch.empty(xc.shape[:-1], dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            st = _lib.load().fqla_l2norm_fwd(
                xc.data_ptr(), y.data_ptr(), rstd.data_ptr(), xc.numel() // D, D,
                _DTYPE_CODE[x.dtype], float(eps), torch.cuda.current_stream(x.device).cuda_stream)
        _lib.check(st, "l2norm_fwd")
        return y, rstd
    xf = x.float()
    rstd = torch.rsqrt((xf * xf).sum(dim=-1, keepdim=True) + eps)
    y = (x * rstd).to(x.dtype)
    return y, rstd.squeeze(-1)


def l2norm_bwd(y: torch.Tensor, rstd: torch.Tensor, dy: torch.Tensor, eps: float = 1e-6, dim: int = -1):
    """Gradient of ``l2norm_fwd`` with respect to its input, fp32:
    ``(dy - <dy, y> y) * rstd``."""
    assert dim == -1 or dim == dy.dim() - 1
    D = dy.shape[-1]
    if _on_gpu_kernel(y, dy) and rstd.dtype == torch.float32 and D % 2 == 0 and D <= 512:
        from .. import _lib

        yc, dyc, rc = y.contiguous(), dy.contiguous(), rstd.contiguous()
        dx = torch.empty(dyc.shape, dtype=torch.float32, device=dy.device)
        with torch.cuda.device(dy.device):
            st = _lib.load().fqla_l2norm_bwd(
                yc.data_ptr(), rc.data_ptr(), dyc.data_ptr(), dx.data_ptr(), dyc.numel() // D, D,
                _DTYPE_CODE[y.dtype], _DTYPE_CODE[dy.dtype],
                torch.cuda.current_stream(dy.device).cuda_stream)
        _lib.check(st, "l2norm_bwd")
        return dx
    yf, dyf = y.float(), dy.float()
    dot = (dyf * yf).sum(dim=-1, keepdim=True)
    return (dyf - dot * yf) * rstd.unsqueeze(-1)


class L2NormFunction(torch.autograd.Function):
    @staticmethod
    @input_guard
    def forward(ctx, x, eps=1e-6):
        y, rstd = l2norm_fwd(x, eps)
        ctx.eps = eps
        ctx.save_for_backward(y, rstd)
        return y

    @staticmethod
    @input_guard
    def backward(ctx, dy):
        y, rstd = ctx.saved_tensors
        return l2norm_bwd(y, rstd, dy, ctx.eps).to(dy.dtype), None


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return L2NormFunction.apply(x, eps)
