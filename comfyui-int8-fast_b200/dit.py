"""Synthetic rectified-flow DiT denoising step (benchmark workload, random weights).

Stands in for the 9B-class Flux-style model the node pack's README timed (no checkpoint is
available offline): hidden 4096, 32 heads x 128, MLP ratio 3 with GELU, 8 double-stream and 24
single-stream blocks, 4096 image tokens (1024 x 1024 px) plus 512 text tokens.  Every q/k/v/o/MLP
linear is an int8 tensorwise-weight layer with dynamic per-token activation quantisation (the W8A8
hot path); input/output embedders, time embedding and the modulation linears stay bf16, mirroring
the layers the loader excludes for flux2.  Attention runs in bf16 through
torch.nn.functional.scaled_dot_product_attention.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as TF
from torch import Tensor, nn

from . import functional as F
from .ops import StandaloneInt8Ops as Ops


@dataclass(frozen=True)
class DiTConfig:
    hidden: int = 4096
    heads: int = 32
    mlp_ratio: int = 3
    double_blocks: int = 8
    single_blocks: int = 24
    img_tokens: int = 4096
    txt_tokens: int = 512
    in_channels: int = 64
    txt_dim: int = 4096

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @property
    def mlp_hidden(self) -> int:
        return self.hidden * self.mlp_ratio

    def int8_params(self) -> int:
        h, m = self.hidden, self.mlp_hidden
        per_stream = 3 * h * h + h * h + 2 * h * m
        return self.double_blocks * 2 * per_stream + self.single_blocks * ((3 * h + m) * h + (h + m) * h)

    def int8_ops(self, batch: int = 1) -> float:
        """2*M*N*K summed over the int8 linears of one step."""
        h, m = self.hidden, self.mlp_hidden
        per_stream = 3 * h * h + h * h + 2 * h * m
        tok = self.img_tokens + self.txt_tokens
        return 2.0 * batch * (self.double_blocks * per_stream * tok + self.single_blocks * ((3 * h + m) * h + (h + m) * h) * tok)

    def attention_flops(self, batch: int = 1) -> float:
        tok = self.img_tokens + self.txt_tokens
        return 4.0 * batch * (self.double_blocks + self.single_blocks) * tok * tok * self.hidden


def int8_linear(in_f: int, out_f: int, gen: torch.Generator, device, bias: bool = True) -> nn.Module:
    """An Int8 ops Linear with random N(0, 0.02) weights quantised tensorwise on the device."""
    from . import functional as F
    lin = Ops.Linear(in_f, out_f, bias=bias, device="meta")
    w = (torch.randn(out_f, in_f, generator=gen, device=device, dtype=torch.float32) * 0.02)
    q, scale = F.quantize_tensorwise(w)
    sd = {"weight": q, "weight_scale": scale.reshape(1).clone()}
    if bias:
        sd["bias"] = torch.zeros(out_f, device=device, dtype=torch.bfloat16)
    lin._load_from_state_dict(sd, "", {}, True, [], [], [])
    return lin


def bf16_linear(in_f: int, out_f: int, gen: torch.Generator, device) -> nn.Linear:
    lin = nn.Linear(in_f, out_f, bias=True, device=device, dtype=torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(out_f, in_f, generator=gen, device=device) * 0.02)
        lin.bias.zero_()
    return lin


def int8_gemm(lin, q: Tensor, q_scale: Tensor, out: Tensor | None = None) -> Tensor:
    """The GEMM half of an Int8 Linear on activations that a fused quantiser has already turned into int8."""
    return F.linear_w8a8(q, q_scale, lin.weight, lin._scale_on(q.device), lin.bias, torch.bfloat16, out=out)


def int8_gemm_gated_add_(lin, residual: Tensor, gate: Tensor, q: Tensor, q_scale: Tensor) -> Tensor:
    """residual += gate * lin(...) inside the GEMM epilogue (in place; the arithmetic of torch.addcmul)."""
    return F.linear_w8a8_gated_add_(residual, gate, q, q_scale, lin.weight, lin._scale_on(q.device), lin.bias)


def attention_prenormed(qkv: Tensor, heads: int) -> Tensor:
    """qkv [T, 3*h] whose q and k columns are already RMS-normalised per head -> attention output [T, h]."""
    t, h3 = qkv.shape
    h = h3 // 3
    q, k, v = qkv.view(1, t, 3, heads, h // heads).unbind(2)
    out = TF.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    return out.transpose(1, 2).reshape(t, h)


def rms_norm(x: Tensor, eps: float = 1e-6) -> Tensor:
    return TF.rms_norm(x, x.shape[-1:], eps=eps)


def modulate(x: Tensor, shift: Tensor, scale: Tensor) -> Tensor:
    """LayerNorm(x) * (1 + scale) + shift, the scale-and-shift as one pass over the normalised tensor."""
    return torch.addcmul(shift.unsqueeze(1), TF.layer_norm(x, x.shape[-1:]), 1 + scale.unsqueeze(1))


def gated_residual(x: Tensor, gate: Tensor, y: Tensor) -> Tensor:
    """x + gate * y in one pass."""
    return torch.addcmul(x, gate.unsqueeze(1), y)


def attention(qkv: Tensor, heads: int) -> Tensor:
    """qkv [B, T, 3*h] (q | k | v along the last axis) -> [B, T, h].  q and k are RMS-normalised per head; all three
    go to the attention kernel as [B, heads, T, d] views of the token-major buffers (no transposed copies)."""
    b, t, h3 = qkv.shape
    h = h3 // 3
    q, k, v = qkv.view(b, t, 3, heads, h // heads).unbind(2)
    out = TF.scaled_dot_product_attention(rms_norm(q).transpose(1, 2), rms_norm(k).transpose(1, 2), v.transpose(1, 2))
    return out.transpose(1, 2).reshape(b, t, h)


class StreamBlock(nn.Module):
    """One stream (image or text) of a double block."""

    def __init__(self, cfg: DiTConfig, gen, device):
        super().__init__()
        h, m = cfg.hidden, cfg.mlp_hidden
        self.mod = bf16_linear(h, 6 * h, gen, device)
        self.qkv = int8_linear(h, 3 * h, gen, device)
        self.proj = int8_linear(h, h, gen, device)
        self.mlp_up = int8_linear(h, m, gen, device)
        self.mlp_down = int8_linear(m, h, gen, device)


class DoubleBlock(nn.Module):
    def __init__(self, cfg: DiTConfig, gen, device):
        super().__init__()
        self.cfg = cfg
        self.img = StreamBlock(cfg, gen, device)
        self.txt = StreamBlock(cfg, gen, device)

    def forward_fused(self, img: Tensor, txt: Tensor, vec: Tensor):
        """The same block with the element-wise steps around the quantised linears folded into the library's kernels:
        LayerNorm + modulation and GELU run inside the activation quantiser, both streams' qkv projections write into
        one buffer, the per-head RMS norm of q and k is one in-place launch over it, and the gated residual updates
        happen in the GEMM epilogues.  img [Ti, h], txt [Tt, h]; both are updated in place and returned."""
        cfg = self.cfg
        h = cfg.hidden
        n_txt = txt.shape[0]
        qkv = torch.empty((n_txt + img.shape[0], 3 * h), dtype=torch.bfloat16, device=img.device)
        mods = {}
        for name, x, blk, rows in (("txt", txt, self.txt, qkv[:n_txt]), ("img", img, self.img, qkv[n_txt:])):
            mods[name] = [m.reshape(-1) for m in blk.mod(TF.silu(vec)).chunk(6, dim=-1)]
            q8, xs = F.quantize_rowwise_ln_modulate(x, mods[name][0], mods[name][1])
            int8_gemm(blk.qkv, q8, xs, out=rows)
        F.rmsnorm_heads_(qkv[:, : 2 * h])
        attn = attention_prenormed(qkv, cfg.heads)
        outs = []
        for name, x, blk, a in (("txt", txt, self.txt, attn[:n_txt]), ("img", img, self.img, attn[n_txt:])):
            sh1, sc1, g1, sh2, sc2, g2 = mods[name]
            int8_gemm_gated_add_(blk.proj, x, g1, *F.quantize_rowwise(a))          # x += g1 * proj(attention)
            q8, xs = F.quantize_rowwise_ln_modulate(x, sh2, sc2)
            q8, xs = F.quantize_rowwise_gelu(int8_gemm(blk.mlp_up, q8, xs))
            int8_gemm_gated_add_(blk.mlp_down, x, g2, q8, xs)                         # x += g2 * mlp(...)
            outs.append(x)
        return outs[1], outs[0]

    def forward(self, img: Tensor, txt: Tensor, vec: Tensor):
        cfg = self.cfg
        mods = {}
        qkv = {}
        for name, x, blk in (("txt", txt, self.txt), ("img", img, self.img)):
            mods[name] = blk.mod(TF.silu(vec)).chunk(6, dim=-1)
            qkv[name] = blk.qkv(modulate(x, mods[name][0], mods[name][1]))
        attn = attention(torch.cat([qkv["txt"], qkv["img"]], dim=1), cfg.heads)   # joint attention over text + image
        outs = []
        for name, x, blk, a in (("txt", txt, self.txt, attn[:, : txt.shape[1]]), ("img", img, self.img, attn[:, txt.shape[1]:])):
            sh1, sc1, g1, sh2, sc2, g2 = mods[name]
            x = gated_residual(x, g1, blk.proj(a))
            x = gated_residual(x, g2, blk.mlp_down(TF.gelu(blk.mlp_up(modulate(x, sh2, sc2)), approximate="tanh")))
            outs.append(x)
        return outs[1], outs[0]


class SingleBlock(nn.Module):
    def __init__(self, cfg: DiTConfig, gen, device):
        super().__init__()
        self.cfg = cfg
        h, m = cfg.hidden, cfg.mlp_hidden
        self.mod = bf16_linear(h, 3 * h, gen, device)
        self.linear1 = int8_linear(h, 3 * h + m, gen, device)
        self.linear2 = int8_linear(h + m, h, gen, device)

    def forward_fused(self, x: Tensor, vec: Tensor) -> Tensor:
        """x [T, h].  linear1's input is quantised with LayerNorm + modulation folded in; linear2's input row
        [ attention | GELU(mlp) ] is assembled and quantised in one pass, never stored in 16 bits."""
        h = self.cfg.hidden
        shift, scale, gate = [m.reshape(-1) for m in self.mod(TF.silu(vec)).chunk(3, dim=-1)]
        q8, xs = F.quantize_rowwise_ln_modulate(x, shift, scale)
        y = int8_gemm(self.linear1, q8, xs)
        F.rmsnorm_heads_(y[:, : 2 * h])
        attn = attention_prenormed(y[:, : 3 * h], self.cfg.heads)
        q8, xs = F.quantize_rowwise_gelu(y[:, 3 * h:], attn)
        return int8_gemm_gated_add_(self.linear2, x, gate, q8, xs)

    def forward(self, x: Tensor, vec: Tensor) -> Tensor:
        h = self.cfg.hidden
        shift, scale, gate = self.mod(TF.silu(vec)).chunk(3, dim=-1)
        y = self.linear1(modulate(x, shift, scale))
        # attention output and the activated MLP half go side by side into one buffer (no concatenation pass)
        z = torch.empty(y.shape[:-1] + (y.shape[-1] - 2 * h,), dtype=y.dtype, device=y.device)
        z[..., :h] = attention(y[..., :3 * h], self.cfg.heads)
        torch.ops.aten.gelu.out(y[..., 3 * h:], approximate="tanh", out=z[..., h:])
        return gated_residual(x, gate, self.linear2(z))


def timestep_embedding(t: Tensor, dim: int = 256) -> Tensor:
    half = dim // 2
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
    args = t.float()[:, None] * 1000.0 * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


class SyntheticDiT(nn.Module):
    def __init__(self, cfg: DiTConfig = DiTConfig(), seed: int = 0, device="cuda", fused: bool = True):
        """`fused` selects the block code that uses the library's fused quantiser prologues and the per-head RMS-norm
        kernel (batch 1, head size 128); otherwise every element-wise step is its own PyTorch call, which is how a
        model written against the node pack's Linear alone would run."""
        super().__init__()
        self.cfg = cfg
        self.fused = fused
        gen = torch.Generator(device=device)
        gen.manual_seed(seed)
        h = cfg.hidden
        self.img_in = bf16_linear(cfg.in_channels, h, gen, device)
        self.txt_in = bf16_linear(cfg.txt_dim, h, gen, device)
        self.time_in = nn.Sequential(bf16_linear(256, h, gen, device), nn.SiLU(), bf16_linear(h, h, gen, device))
        self.double_stream = nn.ModuleList([DoubleBlock(cfg, gen, device) for _ in range(cfg.double_blocks)])
        self.single_stream = nn.ModuleList([SingleBlock(cfg, gen, device) for _ in range(cfg.single_blocks)])
        self.final_mod = bf16_linear(h, 2 * h, gen, device)
        self.final = bf16_linear(h, cfg.in_channels, gen, device)

    @torch.no_grad()
    def forward(self, img: Tensor, txt: Tensor, t: Tensor) -> Tensor:
        """img [B, img_tokens, in_channels], txt [B, txt_tokens, txt_dim], t [B] in [0,1] -> velocity [B, img_tokens, in_channels]."""
        vec = self.time_in(timestep_embedding(t).to(torch.bfloat16))
        img, txt = self.img_in(img), self.txt_in(txt)
        if self.fused and img.shape[0] == 1 and self.cfg.head_dim == 128 and self.cfg.hidden % 8 == 0:
            img2, txt2 = img[0], txt[0]
            for blk in self.double_stream:
                img2, txt2 = blk.forward_fused(img2, txt2, vec)
            x2 = torch.cat([txt2, img2], dim=0)
            for blk in self.single_stream:
                x2 = blk.forward_fused(x2, vec)
            x = x2[None]
        else:
            for blk in self.double_stream:
                img, txt = blk(img, txt, vec)
            x = torch.cat([txt, img], dim=1)
            for blk in self.single_stream:
                x = blk(x, vec)
        x = x[:, txt.shape[1]:]
        shift, scale = self.final_mod(TF.silu(vec)).chunk(2, dim=-1)
        return self.final(modulate(x, shift, scale))
