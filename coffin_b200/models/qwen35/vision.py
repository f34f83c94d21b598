"""Vision tower (ViT) that turns image patches into embeddings of the text model's width.

Pipeline: patch embedding as one GEMM over flattened ``3 x 2 x 16 x 16`` patches, learned
position embedding resampled bilinearly from its 48 x 48 grid, ``depth`` pre-LN blocks
(bidirectional attention over the patches of one image with axial 2-D rotary embedding, GELU-tanh
MLP), and a merger (LayerNorm, 2 x 2 spatial merge, two-layer MLP) producing one embedding per
merged patch.  Linear layers run on the tcgen05 GEMM (the bias rides in as a stride-0 residual),
attention on the paged flash kernel in its non-causal mode, LayerNorm / GELU as row kernels.
``OracleVision`` is the fp32 PyTorch definition the device tower is tested against.
Reference: ``models/qwen35/vision.py:220-854`` (torch matmul + fp32 softmax on the reference).
"""
from __future__ import annotations

import dataclasses
import math

import torch
import torch.nn.functional as F

V = "model.visual."


@dataclasses.dataclass
class VisionConfig:
    depth: int = 24
    hidden_size: int = 1024
    num_heads: int = 16
    intermediate_size: int = 4096
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    in_channels: int = 3
    out_hidden_size: int = 2560
    num_position_embeddings: int = 2304        # 48 x 48
    rope_theta: float = 10000.0
    eps: float = 1e-6

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size ** 2

    @classmethod
    def from_hf(cls, raw: dict, out_hidden: int) -> "VisionConfig":
        v = raw.get("vision_config", raw)
        return cls(depth=int(v.get("depth", 24)), hidden_size=int(v.get("hidden_size", 1024)),
                   num_heads=int(v.get("num_heads", 16)), intermediate_size=int(v.get("intermediate_size", 4096)),
                   patch_size=int(v.get("patch_size", 16)), temporal_patch_size=int(v.get("temporal_patch_size", 2)),
                   spatial_merge_size=int(v.get("spatial_merge_size", 2)), in_channels=int(v.get("in_channels", 3)),
                   out_hidden_size=int(v.get("out_hidden_size", out_hidden)),
                   num_position_embeddings=int(v.get("num_position_embeddings", 2304)))


def tiny_vision(out_hidden: int = 256) -> VisionConfig:
    return VisionConfig(depth=2, hidden_size=128, num_heads=2, intermediate_size=256, out_hidden_size=out_hidden,
                        num_position_embeddings=64)


def random_vision_state_dict(cfg: VisionConfig, seed: int = 0, std: float = 0.02) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g) * std
    h, m = cfg.hidden_size, cfg.spatial_merge_size ** 2
    sd = {V + "patch_embed.proj.weight": r(h, cfg.in_channels, cfg.temporal_patch_size, cfg.patch_size, cfg.patch_size),
          V + "patch_embed.proj.bias": r(h), V + "pos_embed.weight": r(cfg.num_position_embeddings, h),
          V + "merger.norm.weight": 1 + r(h), V + "merger.norm.bias": r(h),
          V + "merger.linear_fc1.weight": r(h * m, h * m), V + "merger.linear_fc1.bias": r(h * m),
          V + "merger.linear_fc2.weight": r(cfg.out_hidden_size, h * m), V + "merger.linear_fc2.bias": r(cfg.out_hidden_size)}
    for i in range(cfg.depth):
        p = f"{V}blocks.{i}."
        sd.update({p + "norm1.weight": 1 + r(h), p + "norm1.bias": r(h), p + "norm2.weight": 1 + r(h), p + "norm2.bias": r(h),
                   p + "attn.qkv.weight": r(3 * h, h), p + "attn.qkv.bias": r(3 * h),
                   p + "attn.proj.weight": r(h, h), p + "attn.proj.bias": r(h),
                   p + "mlp.linear_fc1.weight": r(cfg.intermediate_size, h), p + "mlp.linear_fc1.bias": r(cfg.intermediate_size),
                   p + "mlp.linear_fc2.weight": r(h, cfg.intermediate_size), p + "mlp.linear_fc2.bias": r(h)})
    return sd


# ----------------------------------------------------------------------------------------------
# geometry shared by oracle and device tower
def patch_order(t: int, h: int, w: int, merge: int) -> torch.Tensor:
    """Row-major patch index for every patch in merge-block order: patches of one ``merge x merge``
    block are consecutive, so the merger can view ``[N, hidden]`` as ``[N / merge^2, merge^2 * hidden]``."""
    idx = torch.arange(t * h * w).reshape(t, h // merge, merge, w // merge, merge)
    return idx.permute(0, 1, 3, 2, 4).reshape(-1)


def pos_embed_resample(table: torch.Tensor, h: int, w: int) -> torch.Tensor:
    """Bilinear resample of the ``[S*S, hidden]`` learned grid to ``[h*w, hidden]`` (row-major)."""
    S = int(math.isqrt(table.shape[0]))
    grid = table.float().reshape(S, S, -1).permute(2, 0, 1).unsqueeze(0)
    out = F.interpolate(grid, size=(h, w), mode="bilinear", align_corners=True)
    return out[0].permute(1, 2, 0).reshape(h * w, -1)


def axial_rope(h: int, w: int, head_dim: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin ``[h*w, head_dim]`` (row-major patches): the first half of the rotary frequencies
    turns with the row index, the second half with the column index; ``cat(half, half)`` layout."""
    quarter = head_dim // 4
    inv = 1.0 / (theta ** (torch.arange(0, quarter, dtype=torch.float32) / quarter))
    ys, xs = torch.meshgrid(torch.arange(h, dtype=torch.float32), torch.arange(w, dtype=torch.float32), indexing="ij")
    ang = torch.cat([ys.reshape(-1, 1) * inv[None], xs.reshape(-1, 1) * inv[None]], -1)     # [hw, head_dim/2]
    return torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    half = x.shape[-1] // 2
    rh = torch.cat([-x[..., half:], x[..., :half]], -1)
    return x * cos[:, None, :] + rh * sin[:, None, :]


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return F.gelu(x, approximate="tanh")


class OracleVision:
    """fp32 PyTorch tower. ``patches [N, patch_dim]`` in merge-block order, ``grid = (t, h, w)``."""

    def __init__(self, cfg: VisionConfig, sd: dict[str, torch.Tensor]) -> None:
        self.cfg = cfg
        self.sd = {k: v.float() for k, v in sd.items() if k.startswith(V)}

    def _geometry(self, grid):
        c = self.cfg
        t, h, w = grid
        order = patch_order(t, h, w, c.spatial_merge_size)
        pos = pos_embed_resample(self.sd[V + "pos_embed.weight"], h, w).repeat(t, 1)[order]
        cos, sin = axial_rope(h, w, c.head_dim, c.rope_theta)
        return pos, cos.repeat(t, 1)[order], sin.repeat(t, 1)[order]

    @torch.no_grad()
    def forward(self, patches: torch.Tensor, grid: tuple[int, int, int]) -> torch.Tensor:
        c, sd = self.cfg, self.sd
        N = patches.shape[0]
        pos, cos, sin = self._geometry(grid)
        x = patches.float() @ sd[V + "patch_embed.proj.weight"].reshape(c.hidden_size, -1).t() + sd[V + "patch_embed.proj.bias"]
        x = x + pos
        nh, hd = c.num_heads, c.head_dim
        for i in range(c.depth):
            p = f"{V}blocks.{i}."
            y = F.layer_norm(x, (c.hidden_size,), sd[p + "norm1.weight"], sd[p + "norm1.bias"], c.eps)
            qkv = (y @ sd[p + "attn.qkv.weight"].t() + sd[p + "attn.qkv.bias"]).reshape(N, 3, nh, hd)
            q, k, v = _rope(qkv[:, 0], cos, sin), _rope(qkv[:, 1], cos, sin), qkv[:, 2]
            att = torch.einsum("qhd,khd->hqk", q, k) * hd ** -0.5
            o = torch.einsum("hqk,khd->qhd", att.softmax(-1), v).reshape(N, -1)
            x = x + o @ sd[p + "attn.proj.weight"].t() + sd[p + "attn.proj.bias"]
            y = F.layer_norm(x, (c.hidden_size,), sd[p + "norm2.weight"], sd[p + "norm2.bias"], c.eps)
            y = gelu_tanh(y @ sd[p + "mlp.linear_fc1.weight"].t() + sd[p + "mlp.linear_fc1.bias"])
            x = x + y @ sd[p + "mlp.linear_fc2.weight"].t() + sd[p + "mlp.linear_fc2.bias"]
        m = c.spatial_merge_size ** 2
        y = F.layer_norm(x, (c.hidden_size,), sd[V + "merger.norm.weight"], sd[V + "merger.norm.bias"], c.eps)
        y = y.reshape(N // m, m * c.hidden_size)
        y = F.gelu(y @ sd[V + "merger.linear_fc1.weight"].t() + sd[V + "merger.linear_fc1.bias"])
        return y @ sd[V + "merger.linear_fc2.weight"].t() + sd[V + "merger.linear_fc2.bias"]


class VisionTower:
    """sm_100a tower: bf16 weights, tcgen05 GEMMs, flash attention (non-causal) per image."""

    def __init__(self, cfg: VisionConfig, sd: dict[str, torch.Tensor], device="cuda") -> None:
        from ...ops import kernels as K
        self.K = K
        self.cfg = cfg
        self.device = torch.device(device)
        bf, dev = torch.bfloat16, self.device
        W = lambda k: sd[k].to(dev, bf).contiguous()
        Fp = lambda k: sd[k].to(dev, torch.float32).contiguous()
        c = cfg
        self.patch_w = sd[V + "patch_embed.proj.weight"].reshape(c.hidden_size, -1).to(dev, bf).contiguous()
        self.patch_b = W(V + "patch_embed.proj.bias")
        self.pos_table = sd[V + "pos_embed.weight"].float()
        self.blocks = []
        for i in range(c.depth):
            p = f"{V}blocks.{i}."
            self.blocks.append(dict(n1w=Fp(p + "norm1.weight"), n1b=Fp(p + "norm1.bias"), n2w=Fp(p + "norm2.weight"),
                                    n2b=Fp(p + "norm2.bias"), qkv_w=W(p + "attn.qkv.weight"), qkv_b=W(p + "attn.qkv.bias"),
                                    proj_w=W(p + "attn.proj.weight"), proj_b=W(p + "attn.proj.bias"),
                                    fc1_w=W(p + "mlp.linear_fc1.weight"), fc1_b=W(p + "mlp.linear_fc1.bias"),
                                    fc2_w=W(p + "mlp.linear_fc2.weight"), fc2_b=W(p + "mlp.linear_fc2.bias")))
        self.mn_w, self.mn_b = Fp(V + "merger.norm.weight"), Fp(V + "merger.norm.bias")
        self.m1_w, self.m1_b = W(V + "merger.linear_fc1.weight"), W(V + "merger.linear_fc1.bias")
        self.m2_w, self.m2_b = W(V + "merger.linear_fc2.weight"), W(V + "merger.linear_fc2.bias")
        self._geo: dict[tuple, tuple] = {}

    def _bias(self, b: torch.Tensor, rows: int) -> torch.Tensor:
        return b.unsqueeze(0).expand(rows, -1)          # stride-0 rows: the GEMM epilogue adds it as a residual

    def _layernorm(self, x, w, b):
        out = torch.empty_like(x)
        self.K.call("layernorm", x, w, b, out, x.shape[0], x.shape[1], x.stride(0), out.stride(0), float(self.cfg.eps))
        self.K._count()
        return out

    def _gelu(self, x):
        self.K.call("gelu_tanh", x, x, x.numel())
        self.K._count()
        return x

    def _geometry(self, grid):
        g = self._geo.get(grid)
        if g is None:
            c = self.cfg
            t, h, w = grid
            order = patch_order(t, h, w, c.spatial_merge_size)
            pos = pos_embed_resample(self.pos_table, h, w).repeat(t, 1)[order]
            cos, sin = axial_rope(h, w, c.head_dim, c.rope_theta)
            g = (pos.to(self.device, torch.bfloat16), cos.repeat(t, 1)[order].to(self.device),
                 sin.repeat(t, 1)[order].to(self.device))
            self._geo[grid] = g
        return g

    @torch.no_grad()
    def forward(self, patches: torch.Tensor, grid: tuple[int, int, int]) -> torch.Tensor:
        """``patches [N, patch_dim]`` (merge-block order) of ONE image -> ``[N / merge^2, out_hidden]`` bf16."""
        K, c = self.K, self.cfg
        N = patches.shape[0]
        nh, hd, H = c.num_heads, c.head_dim, c.hidden_size
        pos, cos, sin = self._geometry(grid)
        x = K.gemm(patches.to(self.device, torch.bfloat16).contiguous(), self.patch_w, residual=self._bias(self.patch_b, N))
        x = x + pos
        npad = (N + 63) // 64 * 64
        table = torch.arange(npad // 64, dtype=torch.int32, device=self.device)
        kbuf = torch.zeros(npad, nh, hd, dtype=torch.bfloat16, device=self.device)
        vbuf = torch.zeros_like(kbuf)
        use_kernel = hd in (64, 256)
        for b in self.blocks:
            y = self._layernorm(x, b["n1w"], b["n1b"])
            qkv = K.gemm(y, b["qkv_w"], residual=self._bias(b["qkv_b"], N)).reshape(N, 3, nh, hd)
            q = _rope(qkv[:, 0].float(), cos, sin).to(torch.bfloat16).contiguous()
            k = _rope(qkv[:, 1].float(), cos, sin).to(torch.bfloat16)
            if use_kernel:
                kbuf[:N].copy_(k)
                vbuf[:N].copy_(qkv[:, 2])
                o = torch.empty(N, nh * hd, dtype=torch.bfloat16, device=self.device)
                K.attn_prefill(q, None, kbuf, vbuf, table, o, q_pos0=0, nh=nh, nkv=nh, hd=hd, causal=False, kv_len=N)
            else:   # head widths the flash kernel has no instance for
                att = torch.einsum("qhd,khd->hqk", q.float(), k.float()) * hd ** -0.5
                o = torch.einsum("hqk,khd->qhd", att.softmax(-1), qkv[:, 2].float()).reshape(N, -1).to(torch.bfloat16)
            x = K.gemm(o, b["proj_w"], residual=x + self._bias(b["proj_b"], N))
            y = self._layernorm(x, b["n2w"], b["n2b"])
            y = self._gelu(K.gemm(y, b["fc1_w"], residual=self._bias(b["fc1_b"], N)))
            x = K.gemm(y, b["fc2_w"], residual=x + self._bias(b["fc2_b"], N))
        m = c.spatial_merge_size ** 2
        y = self._layernorm(x, self.mn_w, self.mn_b).reshape(N // m, m * H)
        y = F.gelu(K.gemm(y, self.m1_w, residual=self._bias(self.m1_b, N // m)).float()).to(torch.bfloat16)
        return K.gemm(y, self.m2_w, residual=self._bias(self.m2_b, N // m))


# ----------------------------------------------------------------------------------------------
# image -> patches
def smart_resize(h: int, w: int, factor: int, min_pixels: int, max_pixels: int) -> tuple[int, int]:
    """Nearest size with both sides multiples of ``factor`` and area within the pixel budget."""
    hb = max(factor, round(h / factor) * factor)
    wb = max(factor, round(w / factor) * factor)
    if hb * wb > max_pixels:
        beta = math.sqrt(h * w / max_pixels)
        hb = max(factor, math.floor(h / beta / factor) * factor)
        wb = max(factor, math.floor(w / beta / factor) * factor)
    elif hb * wb < min_pixels:
        beta = math.sqrt(min_pixels / (h * w))
        hb = math.ceil(h * beta / factor) * factor
        wb = math.ceil(w * beta / factor) * factor
    return hb, wb


MEAN = (0.5, 0.5, 0.5)
STD = (0.5, 0.5, 0.5)


def patchify(image: torch.Tensor, cfg: VisionConfig, mean=MEAN, std=STD) -> tuple[torch.Tensor, tuple[int, int, int]]:
    """``image [3, H, W]`` float in [0, 1], sides multiples of ``patch * merge`` ->
    ``(patches [N, patch_dim] in merge-block order, (t, h, w))``.  A still image is repeated over
    the temporal patch.  ``mean`` / ``std``: per-channel normalisation (a checkpoint's own when it states one)."""
    C, Hh, Ww = image.shape
    p, tp = cfg.patch_size, cfg.temporal_patch_size
    mean = torch.tensor(tuple(mean)).reshape(3, 1, 1)
    std = torch.tensor(tuple(std)).reshape(3, 1, 1)
    img = ((image - mean) / std).unsqueeze(1).expand(C, tp, Hh, Ww)
    h, w = Hh // p, Ww // p
    x = img.reshape(C, tp, h, p, w, p).permute(2, 4, 0, 1, 3, 5).reshape(h * w, C * tp * p * p)
    return x[patch_order(1, h, w, cfg.spatial_merge_size)].contiguous(), (1, h, w)
