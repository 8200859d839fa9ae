"""Vision tower of the Qwen2-VL family: patch embedding, transformer blocks with 2-D rotary positions and full attention inside
each frame, and the 2 x 2 patch merger that projects to the language model's width
(reference: model_executor/models/qwen2_vl.py ``Qwen2VisionTransformer``; HF ``Qwen2VisionTransformerPretrainedModel``; weight names
``visual.patch_embed.proj``, ``visual.blocks.N.{norm1,attn.qkv,attn.proj,norm2,mlp.fc1,mlp.fc2}``, ``visual.merger.{ln_q,mlp.0,mlp.2}``).

Input: ``pixel_values [t*h*w, C * temporal_patch * patch * patch]`` in the processor's order (patches of one 2 x 2 merge group
adjacent) and the grid ``(t, h, w)``; output ``[t*h*w / 4, out_hidden]``. The tower runs in PyTorch (the encoder runs once per image,
off the decode path); its output is cached by content hash."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class VisionBlock(nn.Module):
    def __init__(self, dim: int, heads: int, mlp_ratio: float, dtype):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim, eps=1e-6, dtype=dtype)
        self.norm2 = nn.LayerNorm(dim, eps=1e-6, dtype=dtype)
        self.qkv = nn.Linear(dim, 3 * dim, bias=True, dtype=dtype)
        self.proj = nn.Linear(dim, dim, bias=True, dtype=dtype)
        self.fc1 = nn.Linear(dim, int(dim * mlp_ratio), bias=True, dtype=dtype)
        self.fc2 = nn.Linear(int(dim * mlp_ratio), dim, bias=True, dtype=dtype)
        self.heads = heads

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, frames: list[int]) -> torch.Tensor:
        n, dim = x.shape
        h = self.norm1(x)
        q, k, v = self.qkv(h).view(n, 3, self.heads, dim // self.heads).unbind(1)

        def rot(t):
            tf = t.float()
            half = tf.shape[-1] // 2
            r = torch.cat([-tf[..., half:], tf[..., :half]], -1)
            return (tf * cos[:, None, :] + r * sin[:, None, :]).to(t.dtype)
        q, k = rot(q), rot(k)
        outs, o = [], 0
        for m in frames:  # full attention inside each frame
            a = F.scaled_dot_product_attention(q[o:o + m].transpose(0, 1), k[o:o + m].transpose(0, 1), v[o:o + m].transpose(0, 1))
            outs.append(a.transpose(0, 1).reshape(m, dim))
            o += m
        x = x + self.proj(torch.cat(outs, 0))
        h = self.fc1(self.norm2(x))
        return x + self.fc2(h * torch.sigmoid(1.702 * h))  # QuickGELU


class VisionTower(nn.Module):
    def __init__(self, vc: dict, dtype=torch.float32):
        super().__init__()
        self.embed_dim = int(vc.get("embed_dim", vc.get("hidden_size", 1280)))
        self.out_dim = int(vc.get("hidden_size", self.embed_dim)) if "embed_dim" in vc else int(vc.get("out_hidden_size", self.embed_dim))
        self.depth, self.heads = int(vc.get("depth", 32)), int(vc.get("num_heads", 16))
        self.patch, self.tpatch = int(vc.get("patch_size", 14)), int(vc.get("temporal_patch_size", 2))
        self.merge, self.in_ch = int(vc.get("spatial_merge_size", 2)), int(vc.get("in_channels", vc.get("in_chans", 3)))
        pdim = self.in_ch * self.tpatch * self.patch * self.patch
        self.patch_embed = nn.Linear(pdim, self.embed_dim, bias=False, dtype=dtype)  # the checkpoint's Conv3d with kernel = stride
        self.blocks = nn.ModuleList([VisionBlock(self.embed_dim, self.heads, float(vc.get("mlp_ratio", 4)), dtype) for _ in range(self.depth)])
        self.ln_q = nn.LayerNorm(self.embed_dim, eps=1e-6, dtype=dtype)
        md = self.embed_dim * self.merge * self.merge
        self.merger0 = nn.Linear(md, md, bias=True, dtype=dtype)
        self.merger2 = nn.Linear(md, self.out_dim, bias=True, dtype=dtype)

    def rotary(self, t: int, h: int, w: int, device) -> tuple[torch.Tensor, torch.Tensor]:
        m, hd = self.merge, self.embed_dim // self.heads
        hp = torch.arange(h, device=device).unsqueeze(1).expand(h, w)
        wp = torch.arange(w, device=device).unsqueeze(0).expand(h, w)

        def order(p):  # the processor emits the patches of one merge group next to each other
            return p.reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
        pos = torch.stack([order(hp), order(wp)], -1).repeat(t, 1)          # [t*h*w, 2]
        dim = hd // 2
        inv = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
        fr = torch.outer(torch.arange(max(h, w), dtype=torch.float32, device=device), inv)   # [max, dim/2]
        ang = fr[pos].flatten(1)                                             # [n, dim]  (h angles, then w angles)
        ang = torch.cat([ang, ang], -1)                                       # [n, head_dim]
        return ang.cos(), ang.sin()

    @torch.no_grad()
    def forward(self, pixel_values: torch.Tensor, grid_thw) -> torch.Tensor:
        t, h, w = (int(x) for x in grid_thw)
        dev, dt = self.patch_embed.weight.device, self.patch_embed.weight.dtype
        x = self.patch_embed(pixel_values.to(dev, dt))
        cos, sin = self.rotary(t, h, w, dev)
        frames = [h * w] * t
        for b in self.blocks:
            x = b(x, cos, sin, frames)
        x = self.ln_q(x).view(-1, self.embed_dim * self.merge * self.merge)
        return self.merger2(F.gelu(self.merger0(x)))

    # checkpoint names -> this module's parameters
    def load_weight(self, name: str, w: torch.Tensor) -> bool:
        name = name.split("visual.", 1)[-1]
        table = {"patch_embed.proj.weight": "patch_embed.weight", "merger.ln_q.weight": "ln_q.weight", "merger.ln_q.bias": "ln_q.bias",
                 "merger.mlp.0.weight": "merger0.weight", "merger.mlp.0.bias": "merger0.bias", "merger.mlp.2.weight": "merger2.weight",
                 "merger.mlp.2.bias": "merger2.bias"}
        tgt = table.get(name)
        if tgt is None and name.startswith("blocks."):
            tgt = name.replace(".attn.qkv.", ".qkv.").replace(".attn.proj.", ".proj.").replace(".mlp.fc1.", ".fc1.").replace(".mlp.fc2.", ".fc2.")
        if tgt is None:
            return False
        p = dict(self.named_parameters()).get(tgt)
        if p is None:
            return False
        p.data.copy_(w.reshape(p.shape).to(p.dtype))
        return True
