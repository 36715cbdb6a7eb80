"""Row-wise L2 normalisation of q/k and its gradient.

Same contract as the reference's ``flash_qla/utils/math.py:9-101`` (``l2norm_fwd`` returns the
normalised tensor in the input dtype and the fp32 reciprocal norm; ``l2norm_bwd`` maps the
gradient of the normalised tensor back).  Plain torch ops on the input's device; this is an
optional pre-op of the path (``use_qk_l2norm_in_kernel``), not one of its kernels.
"""

from __future__ import annotations

import torch

from .contiguous import input_guard


def l2norm_fwd(x: torch.Tensor, eps: float = 1e-6, dim: int = -1):
    assert dim == -1 or dim == x.dim() - 1
    xf = x.float()
    rstd = torch.rsqrt((xf * xf).sum(dim=-1, keepdim=True) + eps)
    y = (x * rstd).to(x.dtype)
    return y, rstd.squeeze(-1)


def l2norm_bwd(y: torch.Tensor, rstd: torch.Tensor, dy: torch.Tensor, eps: float = 1e-6, dim: int = -1):
    assert dim == -1 or dim == dy.dim() - 1
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
