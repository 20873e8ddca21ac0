"""Decode demo: a small GQA decoder generating with per-layer ``NVFP4KVCache``s.

    python -m sageattention_b200.nvfp4.demo_decode [--layers 4] [--prompt 2048] [--new 64]

Stands in for the reference's ``example/nvfp4_decode_demo.py`` (which patches a pretrained Qwen2):
no checkpoint is assumed here, so the model is a randomly initialised pre-norm decoder with
rotary embeddings and grouped-query attention (default 8 query heads on 2 KV heads, head dim
128).  The prompt is prefilled once with plain bf16 attention; decoding then runs three ways from
the same prompt state --

  bf16    keys and values kept in bf16, ``scaled_dot_product_attention`` per step (the baseline);
  fp4     each layer appends the post-RoPE K and V to its ``NVFP4KVCache`` and attends with
          ``nvfp4_flash_decode_prequant`` over the packed cache;
  hybrid  ``NVFP4KVCache.hybrid_decode``: recent tokens in bf16, older prefix in NVFP4 --

and the demo reports what the reference's demo reports: greedy top-1 agreement with the bf16 run,
the teacher-forced logit cosine per step, cache memory per mode, and the per-step latency.
"""

from __future__ import annotations

import argparse
import math
import time

import torch
import torch.nn.functional as F

from . import NVFP4KVCache, nvfp4_flash_decode_prequant


class TinyGQADecoder(torch.nn.Module):
    """Pre-norm decoder: RMSNorm -> GQA attention with RoPE -> RMSNorm -> SiLU MLP."""

    def __init__(self, layers, hidden, heads, kv_heads, head_dim, vocab, dtype, device):
        super().__init__()
        self.h, self.hk, self.d, self.layers = heads, kv_heads, head_dim, layers
        g = torch.Generator(device="cpu").manual_seed(0)

        def w(o, i, gain=1.0):
            return (torch.randn(o, i, generator=g) * (gain / math.sqrt(i))).to(dtype).to(device)

        self.emb = (torch.randn(vocab, hidden, generator=g)).to(dtype).to(device)
        self.blocks = [dict(q=w(heads * head_dim, hidden), k=w(kv_heads * head_dim, hidden),
                            v=w(kv_heads * head_dim, hidden), o=w(hidden, heads * head_dim),
                            up=w(4 * hidden, hidden), down=w(hidden, 4 * hidden)) for _ in range(layers)]
        self.head = w(vocab, hidden, gain=4.0)
        self.inv_freq = 1.0 / (10000.0 ** (torch.arange(0, head_dim, 2, device=device).float() / head_dim))

    @staticmethod
    def _norm(x):
        return (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)).to(x.dtype)

    def _rope(self, x, pos):
        """x [Z, heads, S, D], pos [S] -> rotated (half-split convention)."""
        ang = pos.float()[:, None] * self.inv_freq[None, :]
        cos, sin = ang.cos()[None, None], ang.sin()[None, None]
        x1, x2 = x.float().chunk(2, dim=-1)
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)

    def qkv(self, blk, x, pos):
        z, s, _ = x.shape
        xn = self._norm(x)
        q = (xn @ blk["q"].T).view(z, s, self.h, self.d).transpose(1, 2)
        k = (xn @ blk["k"].T).view(z, s, self.hk, self.d).transpose(1, 2)
        v = (xn @ blk["v"].T).view(z, s, self.hk, self.d).transpose(1, 2)
        return self._rope(q, pos), self._rope(k, pos), v

    def finish(self, blk, x, attn):
        z, _, s, _ = attn.shape
        x = x + attn.transpose(1, 2).reshape(z, s, self.h * self.d) @ blk["o"].T
        return x + F.silu(self._norm(x) @ blk["up"].T) @ blk["down"].T

    def logits(self, x):
        return (self._norm(x[:, -1]) @ self.head.T).float()


@torch.no_grad()
def prefill(model, tokens):
    """bf16 prefill; returns last-position logits and per-layer post-RoPE (K, V)."""
    x = model.emb[tokens]
    pos = torch.arange(tokens.shape[1], device=tokens.device)
    kv = []
    g = model.h // model.hk
    for blk in model.blocks:
        q, k, v = model.qkv(blk, x, pos)
        attn = F.scaled_dot_product_attention(q, k.repeat_interleave(g, 1), v.repeat_interleave(g, 1),
                                              is_causal=True)
        x = model.finish(blk, x, attn)
        kv.append((k, v))
    return model.logits(x), kv


@torch.no_grad()
def decode_step(model, token, position, state, mode):
    """One decode step; ``state`` is per-layer: (K, V) bf16 tensors or an NVFP4KVCache."""
    x = model.emb[token][:, None]
    pos = torch.tensor([position], device=x.device)
    g = model.h // model.hk
    scaling = model.d ** -0.5
    for li, blk in enumerate(model.blocks):
        q, k, v = model.qkv(blk, x, pos)
        if mode == "bf16":
            kc, vc, n = state[li]
            kc[:, :, n:n + 1], vc[:, :, n:n + 1] = k, v
            state[li] = (kc, vc, n + 1)
            attn = F.scaled_dot_product_attention(q, kc[:, :, :n + 1].repeat_interleave(g, 1),
                                                  vc[:, :, :n + 1].repeat_interleave(g, 1))
        else:
            cache = state[li]
            cache.append(k, v)
            attn = (cache.hybrid_decode(q, scaling, g) if mode == "hybrid"
                    else nvfp4_flash_decode_prequant(q, cache.get_packed(), scaling, g))
        x = model.finish(blk, x, attn)
    return model.logits(x)


def fresh_state(model, kv, mode, capacity, window):
    z = kv[0][0].shape[0]
    if mode == "bf16":
        out = []
        for k, v in kv:
            kc = torch.empty(z, model.hk, capacity, model.d, dtype=k.dtype, device=k.device)
            vc = torch.empty_like(kc)
            n = k.shape[2]
            kc[:, :, :n], vc[:, :, :n] = k, v
            out.append((kc, vc, n))
        return out
    caches = []
    for k, v in kv:
        c = NVFP4KVCache(z, model.hk, model.d, capacity, k.device, k.dtype,
                         recent_window=window if mode == "hybrid" else 0)
        c.prefill(k, v)
        caches.append(c)
    return caches


@torch.no_grad()
def generate(model, kv, first_logits, n_new, mode, capacity, window, forced=None):
    """Greedy generation (or teacher-forced on ``forced`` tokens); returns tokens, logits, ms/step."""
    state = fresh_state(model, kv, mode, capacity, window)
    start = kv[0][0].shape[2]
    tok = first_logits.argmax(-1)
    toks, logs = [tok], []
    t0 = None
    for i in range(n_new):
        if i == 1:                       # the first step pays one-time library initialisation
            torch.cuda.synchronize()
            t0 = time.perf_counter()
        feed = tok if forced is None else forced[i]
        lg = decode_step(model, feed, start + i, state, mode)
        tok = lg.argmax(-1)
        toks.append(tok)
        logs.append(lg)
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / (n_new - 1) if n_new > 1 else float("nan")
    return torch.stack(toks, 1), torch.stack(logs, 1), ms, state


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=2)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--vocab", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--new", type=int, default=64)
    ap.add_argument("--window", type=int, default=128)
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise RuntimeError("the demo needs a CUDA device (the NVFP4 kernels have no CPU path)")
    dev, dt = "cuda", torch.bfloat16
    model = TinyGQADecoder(a.layers, a.hidden, a.heads, a.kv_heads, a.head_dim, a.vocab, dt, dev)
    tokens = torch.randint(0, a.vocab, (a.batch, a.prompt), generator=torch.Generator().manual_seed(1)).to(dev)
    first, kv = prefill(model, tokens)
    cap = a.prompt + a.new + 16
    ref_toks, ref_logits, ref_ms, _ = generate(model, kv, first, a.new, "bf16", cap, a.window)
    report = {"bf16_ms_per_step": ref_ms}
    print(f"model: {a.layers} layers, {a.heads} heads on {a.kv_heads} KV heads, head dim {a.head_dim}; "
          f"prompt {a.prompt} tokens x batch {a.batch}, {a.new} new tokens (greedy)")
    print(f"  bf16 cache : {ref_ms:.3f} ms/step")
    for mode in ("fp4", "hybrid"):
        toks, _, ms, state = generate(model, kv, first, a.new, mode, cap, a.window)
        agree = float((toks == ref_toks).float().mean())
        _, forced_logits, _, _ = generate(model, kv, first, a.new, mode, cap, a.window,
                                          forced=[ref_toks[:, i] for i in range(a.new)])
        cos = float(F.cosine_similarity(forced_logits.flatten(0, 1), ref_logits.flatten(0, 1), dim=-1).mean())
        mem = sum(c.hybrid_bytes() if mode == "hybrid" else c.fp4_bytes() for c in state)
        bf = sum(c.bf16_bytes() for c in state)
        report[mode] = {"agreement": agree, "logit_cos": cos, "ms_per_step": ms, "bytes": mem, "bf16_bytes": bf}
        print(f"  {mode:<6} cache: {ms:.3f} ms/step; free-running top-1 agreement with bf16 {agree * 100:.1f} %; "
              f"teacher-forced logit cosine {cos:.4f}; cache {mem / 1e6:.2f} MB vs bf16 {bf / 1e6:.2f} MB "
              f"({bf / mem:.2f}x)")
    return report


if __name__ == "__main__":
    main()
