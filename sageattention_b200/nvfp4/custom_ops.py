"""`torch.library` registration of the NVFP4 operators, so that the path traces under
`torch.compile` / `torch.export` (fake-tensor shape inference) and takes part in autograd as
opaque ops.  The reference hints at this integration (`flash.py:268-273`) and upstream registers
its CUDA kernels the same way (`sageattention/sm80_compile.py:5-28, 98-132`).

Every op is a thin wrapper over the same host functions the eager API calls; nothing here adds a
second compute path.

    out = torch.ops.sageattention_b200.nvfp4_attn(q, k, v, scaling, causal, groups)     # differentiable
    nib, sc = torch.ops.sageattention_b200.nvfp4_quant(x, transpose, k_pad)
    out = torch.ops.sageattention_b200.nvfp4_decode(q, knv, ksc, vnv, vsc, s, s_pad, scaling, groups)
"""

from __future__ import annotations

from typing import Tuple

import torch

from . import flash

_NS = "sageattention_b200"


@torch.library.custom_op(f"{_NS}::nvfp4_attn_fwd", mutates_args=())
def nvfp4_attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scaling: float, causal: bool,
                   groups: int) -> Tuple[torch.Tensor, torch.Tensor]:
    out, lse = flash.nvfp4_flash_attention(q, k, v, scaling, causal=causal, num_key_value_groups=groups,
                                           return_lse=True)
    return out, lse


@nvfp4_attn_fwd.register_fake
def _(q, k, v, scaling, causal, groups):
    z, h, s_q, d = q.shape
    return q.new_empty(z, h, s_q, d), q.new_empty(z * h, s_q, dtype=torch.float32)


@torch.library.custom_op(f"{_NS}::nvfp4_attn_bwd", mutates_args=())
def nvfp4_attn_bwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, lse: torch.Tensor,
                   dout: torch.Tensor, scaling: float, causal: bool,
                   groups: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return flash._run_bwd_hp(q, k, v, out, lse, dout, scaling, causal, groups)


@nvfp4_attn_bwd.register_fake
def _(q, k, v, out, lse, dout, scaling, causal, groups):
    return (dout.new_empty(q.shape), dout.new_empty(k.shape), dout.new_empty(v.shape))


def _attn_setup(ctx, inputs, output):
    q, k, v, scaling, causal, groups = inputs
    out, lse = output
    ctx.save_for_backward(q, k, v, out, lse)
    ctx.meta = (scaling, causal, groups)


def _attn_backward(ctx, grad_out, grad_lse):
    q, k, v, out, lse = ctx.saved_tensors
    scaling, causal, groups = ctx.meta
    dq, dk, dv = nvfp4_attn_bwd(q, k, v, out, lse, grad_out.contiguous(), scaling, causal, groups)
    return dq, dk, dv, None, None, None


nvfp4_attn_fwd.register_autograd(_attn_backward, setup_context=_attn_setup)


def nvfp4_attn(q, k, v, scaling: float, causal: bool = False, groups: int = 1) -> torch.Tensor:
    """Differentiable attention through the registered ops (dense; `[Z,H,S,D]` layout)."""
    return nvfp4_attn_fwd(q, k, v, scaling, causal, groups)[0]


@torch.library.custom_op(f"{_NS}::nvfp4_quant", mutates_args=())
def nvfp4_quant(x: torch.Tensor, transpose: bool, k_pad: int) -> Tuple[torch.Tensor, torch.Tensor]:
    nib, sc = flash._quant_nvfp4(x, transpose=transpose, k_pad=k_pad if k_pad > 0 else None)
    return nib, sc.view(torch.uint8)


@nvfp4_quant.register_fake
def _(x, transpose, k_pad):
    b, a1, a2 = x.shape
    r, kk = (a2, a1) if transpose else (a1, a2)
    kp = k_pad if k_pad > 0 else kk
    return (x.new_empty(b, r, kp // 2, dtype=torch.uint8), x.new_empty(b, r, kp // 16, dtype=torch.uint8))


@torch.library.custom_op(f"{_NS}::nvfp4_decode", mutates_args=())
def nvfp4_decode(q: torch.Tensor, knv: torch.Tensor, ksc: torch.Tensor, vnv: torch.Tensor, vsc: torch.Tensor,
                 s: int, s_pad: int, scaling: float, groups: int) -> torch.Tensor:
    packed = (knv, ksc.view(torch.float8_e4m3fn), vnv, vsc.view(torch.float8_e4m3fn), s, s_pad)
    return flash.nvfp4_flash_decode_prequant(q, packed, scaling, groups)


@nvfp4_decode.register_fake
def _(q, knv, ksc, vnv, vsc, s, s_pad, scaling, groups):
    return q.new_empty(q.shape)
