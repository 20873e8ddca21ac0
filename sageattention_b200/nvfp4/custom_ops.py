"""`torch.library` registration of the NVFP4 operators, so that the path traces under
`torch.compile` / `torch.export` (fake-tensor shape inference) and takes part in autograd as
opaque ops.  The reference hints at this integration (`flash.py:268-273`) and upstream registers
its CUDA kernels the same way (`sageattention/sm80_compile.py:5-28, 98-132`).

Every op is a thin wrapper over the same host functions the eager API calls; nothing here adds a
second compute path.

    out = torch.ops.sageattention_b200.nvfp4_attn(q, k, v, scaling, causal, groups)     # differentiable
    nib, sc = torch.ops.sageattention_b200.nvfp4_quant(x, transpose, k_pad)
    out = torch.ops.sageattention_b200.nvfp4_decode(q, knv, ksc, vnv, vsc, s, s_pad, scaling, groups)
    out = nvfp4_attn_ex(q, k, v, scaling, causal, groups, key_pad_bias=..., cu_seqlens=..., out_layout=...,
                        backward_grad_dots=...)                                         # differentiable
    torch.ops.sageattention_b200.nvfp4_kv_append(k_new, v_new, knv, ksc, vnv, vsc, partial, rk, rv, pos)
    out = torch.ops.sageattention_b200.nvfp4_hybrid_decode(q, knv, ksc, vnv, vsc, rk, rv, length, window,
                                                           scaling, groups)
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import flash
from . import kv_cache as _kvc

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


# ---------------------------------------------------------------- attention with every forward option
def _varlen(cu_seqlens, s_q, device):
    return flash._varlen_seq_arrays(cu_seqlens, s_q, device) if cu_seqlens is not None else None


@torch.library.custom_op(f"{_NS}::nvfp4_attn_ex_fwd", mutates_args=())
def nvfp4_attn_ex_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scaling: float, causal: bool,
                      groups: int, key_pad_bias: Optional[torch.Tensor], cu_seqlens: Optional[torch.Tensor],
                      out_zshd: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    out, lse = flash.nvfp4_flash_attention(
        q, k, v, scaling, causal=causal, num_key_value_groups=groups, key_pad_bias=key_pad_bias,
        return_lse=True, out_layout="zshd" if out_zshd else "zhsd", _varlen_arrays=_varlen(cu_seqlens, q.shape[2], q.device))
    return out, lse


@nvfp4_attn_ex_fwd.register_fake
def _(q, k, v, scaling, causal, groups, key_pad_bias, cu_seqlens, out_zshd):
    z, h, s_q, d = q.shape
    out = q.new_empty(z, s_q, h, d) if out_zshd else q.new_empty(z, h, s_q, d)
    return out, q.new_empty(z * h, s_q, dtype=torch.float32)


@torch.library.custom_op(f"{_NS}::nvfp4_attn_ex_bwd", mutates_args=())
def nvfp4_attn_ex_bwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, lse: torch.Tensor,
                      dout: torch.Tensor, scaling: float, causal: bool, groups: int,
                      key_pad_bias: Optional[torch.Tensor], cu_seqlens: Optional[torch.Tensor], out_zshd: bool,
                      grad_mode: str) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    varlen = _varlen(cu_seqlens, q.shape[2], q.device)
    layout = "zshd" if out_zshd else "zhsd"
    if grad_mode == "bf16":
        return flash._run_bwd_hp(q, k, v, out, lse, dout, scaling, causal, groups, varlen, layout,
                                 key_pad_bias=key_pad_bias)
    return flash._run_bwd(q, k, v, out, lse, dout, scaling, causal, groups, varlen, layout, mode=grad_mode,
                          key_pad_bias=key_pad_bias)


@nvfp4_attn_ex_bwd.register_fake
def _(q, k, v, out, lse, dout, scaling, causal, groups, key_pad_bias, cu_seqlens, out_zshd, grad_mode):
    return (dout.new_empty(q.shape), dout.new_empty(k.shape), dout.new_empty(v.shape))


class _AttnEx(torch.autograd.Function):
    """Autograd over the two registered ops (the backward mode is not an input of the forward op,
    so it travels on the context instead of through ``register_autograd``)."""

    @staticmethod
    def forward(ctx, q, k, v, scaling, causal, groups, key_pad_bias, cu_seqlens, out_zshd, grad_mode):
        out, lse = nvfp4_attn_ex_fwd(q, k, v, scaling, causal, groups, key_pad_bias, cu_seqlens, out_zshd)
        ctx.save_for_backward(q, k, v, out, lse, key_pad_bias, cu_seqlens)
        ctx.meta = (scaling, causal, groups, out_zshd, grad_mode)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        q, k, v, out, lse, bias, cu = ctx.saved_tensors
        scaling, causal, groups, out_zshd, grad_mode = ctx.meta
        dq, dk, dv = nvfp4_attn_ex_bwd(q, k, v, out, lse, grad_out, scaling, causal, groups, bias, cu, out_zshd,
                                       grad_mode)
        return (dq, dk, dv) + (None,) * 7


def nvfp4_attn_ex(q, k, v, scaling: float, causal: bool = False, groups: int = 1, key_pad_bias=None,
                  cu_seqlens=None, out_layout: str = "zhsd", backward_grad_dots: Optional[str] = None) -> torch.Tensor:
    """Differentiable attention through the registered ops with the options of
    ``nvfp4_flash_attn_func``: additive key bias, packed varlen rows (``cu_seqlens``), ``zshd``
    output, and the backward mode ("bf16", "fp4_rownorm", "fp4_legacy" without stochastic
    rounding, "fp8_rownorm"; None resolves like the eager entry)."""
    if out_layout not in ("zhsd", "zshd"):
        raise ValueError(f"out_layout must be 'zhsd' or 'zshd', got {out_layout!r}")
    s_kv = k.shape[2]
    eff = s_kv if cu_seqlens is None else q.shape[2] / max(1, cu_seqlens.numel() - 1)
    mode = flash._resolve_backward_grad_dots(backward_grad_dots, eff, False, groups)
    if cu_seqlens is not None:
        assert causal and q.shape[0] == 1 and q.shape[2] == s_kv, "varlen needs causal packed self-attention with Z == 1"
    return _AttnEx.apply(q, k, v, float(scaling), bool(causal), int(groups), key_pad_bias, cu_seqlens,
                         out_layout == "zshd", mode)


# ---------------------------------------------------------------- KV cache: append and hybrid decode
@torch.library.custom_op(f"{_NS}::nvfp4_kv_append",
                         mutates_args=("knv", "ksc", "vnv", "vsc", "v_partial", "rk", "rv"))
def nvfp4_kv_append(k_new: torch.Tensor, v_new: torch.Tensor, knv: torch.Tensor, ksc: torch.Tensor,
                    vnv: torch.Tensor, vsc: torch.Tensor, v_partial: torch.Tensor, rk: Optional[torch.Tensor],
                    rv: Optional[torch.Tensor], pos: int) -> None:
    """``NVFP4KVCache.append`` on the cache's buffers (scale tensors as float8_e4m3fn or uint8)."""
    _kvc.append_token(k_new, v_new, knv, ksc, vnv, vsc, v_partial, rk, rv, pos)


@nvfp4_kv_append.register_fake
def _(k_new, v_new, knv, ksc, vnv, vsc, v_partial, rk, rv, pos):
    return None


@torch.library.custom_op(f"{_NS}::nvfp4_hybrid_decode", mutates_args=())
def nvfp4_hybrid_decode(q: torch.Tensor, knv: torch.Tensor, ksc: torch.Tensor, vnv: torch.Tensor,
                        vsc: torch.Tensor, rk: torch.Tensor, rv: torch.Tensor, length: int, recent_window: int,
                        scaling: float, groups: int) -> torch.Tensor:
    """``NVFP4KVCache.hybrid_decode`` on the cache's buffers."""
    f8 = torch.float8_e4m3fn
    return _kvc.hybrid_decode_buffers(q, knv, ksc.view(f8) if ksc.dtype != f8 else ksc, vnv,
                                      vsc.view(f8) if vsc.dtype != f8 else vsc, rk, rv, length, recent_window,
                                      scaling, groups)


@nvfp4_hybrid_decode.register_fake
def _(q, knv, ksc, vnv, vsc, rk, rv, length, recent_window, scaling, groups):
    return q.new_empty(q.shape)
