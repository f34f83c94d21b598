"""Quantised weight containers: per-output-channel int8 (W8A8) and group-128 int4 (W4A8).

In memory the device kernels want K-major ``[N, K]`` int8 (what tcgen05 ``kind::i8`` and the int8
GEMV read) and, for W4A8, the packed nibbles as they are on disk.  On disk the reference's
layouts are kept so checkpoints stay interchangeable: int8 ``[K, N]`` + fp32 ``[N]`` scale
(``coffin-int8-kn-v1``), packed uint8 ``[ceil(K/128)*64, N]`` (K padded to whole groups; low nibble = even k, code = q + 8) + fp32
``[ceil(K/128), N]`` scale (``coffin-w4a8-kn-v1``).  Reference: ``int8_weights.py:249-384``
(``QWeight.quantize``: absmax/127, scale floor 1e-8, chunked rows), ``w4a8_weights.py:28-222``,
``tools/quant_disk_w4a8.py:45-128``.
"""
from __future__ import annotations

import dataclasses

import torch

GROUP = 128


def is_quantizable(key: str, t: torch.Tensor) -> bool:
    """2-D projection weights of the text model are quantised; embeddings, norms, the router
    (``mlp.gate.weight``), the shared-expert gate and conv taps stay dense."""
    if t.dim() not in (2, 3) or not t.is_floating_point():
        return False
    if key.endswith(("embed_tokens.weight", "mlp.gate.weight", "shared_expert_gate.weight", "conv1d.weight")):
        return False
    if "norm" in key.rsplit(".", 2)[-2:][0] and key.endswith("norm.weight"):
        return False
    return key.endswith(("_proj.weight", "in_proj_qkv.weight", "in_proj_z.weight", "in_proj_b.weight",
                         "in_proj_a.weight", "out_proj.weight", "lm_head.weight", "fc.weight",
                         "experts.gate_up_proj", "experts.down_proj"))


def is_quantizable_qwen4(key: str, t: torch.Tensor) -> bool:
    """Qwen4-exp: the mixer projections (including the fused indexer projection), the routed and shared
    experts and the lm_head are quantised; the router, gates, norms, conv taps, the hyper-connection
    matrices (low rank, read in fp32 gates), the PLE projections and tables and the embedding stay dense
    (reference: ``tools/quant_disk_qwen4.py`` quantises the same families, ``models/qwen4exp/proj.py:524-722``
    loads them)."""
    if t.dim() not in (2, 3) or not t.is_floating_point():
        return False
    if "hyper_connection" in key or ".ple." in key or key.endswith(("embed_tokens.weight", "mlp.gate.weight",
                                                                      "shared_expert_gate.weight", "conv1d.weight")):
        return False
    return key.endswith(("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight", "index_qk_proj.weight",
                         "in_proj_qkv.weight", "in_proj_z.weight", "out_proj.weight", "gate_proj.weight",
                         "up_proj.weight", "down_proj.weight", "lm_head.weight", "experts.gate_up_proj",
                         "experts.down_proj"))


@dataclasses.dataclass
class QWeight:
    """Symmetric per-output-row int8: ``w[n, k] ~= wq[n, k] * scale[n]``. ``wq`` may carry a
    leading expert axis (``[E, N, K]`` with ``scale [E, N]``)."""
    wq: torch.Tensor
    scale: torch.Tensor

    @property
    def n(self) -> int:
        return self.wq.shape[-2]

    @property
    def k(self) -> int:
        return self.wq.shape[-1]

    @classmethod
    def quantize(cls, w: torch.Tensor, chunk_rows: int = 4096) -> "QWeight":
        flat = w.reshape(-1, w.shape[-1])
        wq = torch.empty(flat.shape, dtype=torch.int8, device=w.device)
        scale = torch.empty(flat.shape[0], dtype=torch.float32, device=w.device)
        for s in range(0, flat.shape[0], chunk_rows):
            blk = flat[s:s + chunk_rows].float()
            sc = (blk.abs().amax(-1) / 127.0).clamp_min(1e-8)
            scale[s:s + chunk_rows] = sc
            wq[s:s + chunk_rows] = (blk / sc[:, None]).round().clamp_(-127, 127).to(torch.int8)
        return cls(wq.reshape(w.shape), scale.reshape(w.shape[:-1]))

    def dequant(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        return (self.wq.float() * self.scale.unsqueeze(-1)).to(dtype)

    def to(self, device) -> "QWeight":
        return QWeight(self.wq.to(device), self.scale.to(device))

    # on-disk [K, N] layout
    def to_kn(self) -> tuple[torch.Tensor, torch.Tensor]:
        return self.wq.transpose(-1, -2).contiguous(), self.scale.contiguous()

    @classmethod
    def from_kn(cls, kn: torch.Tensor, scale: torch.Tensor) -> "QWeight":
        return cls(kn.transpose(-1, -2).contiguous(), scale)


@dataclasses.dataclass
class W4A8Weight:
    """Group-``GROUP`` symmetric int4: ``w[n, k] ~= (code - 8) * scale[k // GROUP, n]``.

    ``packed`` uint8 ``[..., R, N]``: low nibble = even k, high nibble = odd k; ``R`` is
    ``ceil(K/GROUP) * GROUP / 2`` as written by the quantisers (K padded to whole groups with zero
    codes) — a tensor of ``ceil(K/2)`` rows is read as well.  ``scale`` fp32 ``[..., ceil(K/GROUP), N]``.
    """
    packed: torch.Tensor
    scale: torch.Tensor
    k: int
    group_size: int = GROUP

    @property
    def n(self) -> int:
        return self.packed.shape[-1]

    @classmethod
    def quantize(cls, w: torch.Tensor, group: int = GROUP) -> "W4A8Weight":
        """``w [..., N, K]`` (checkpoint orientation)."""
        *lead, N, K = w.shape
        G = (K + group - 1) // group
        wf = w.float()
        pad = G * group - K
        if pad:
            wf = torch.nn.functional.pad(wf, (0, pad))
        grp = wf.reshape(*lead, N, G, group)
        scale = (grp.abs().amax(-1) / 7.0).clamp_min(1e-8)                  # [..., N, G]
        q = (grp / scale.unsqueeze(-1)).round().clamp_(-8, 7).to(torch.int16) + 8
        # K is padded to a whole number of groups before packing (the padding quantises to code 8 =
        # zero), which is what the reference's writer stores: ``ceil(K / group) * group / 2`` rows
        q = q.reshape(*lead, N, G * group)
        q = q.transpose(-1, -2)                                            # [..., G * group, N]
        packed = (q[..., 0::2, :] | (q[..., 1::2, :] << 4)).to(torch.uint8).contiguous()
        return cls(packed, scale.transpose(-1, -2).contiguous(), K, group)

    def codes(self) -> torch.Tensor:
        """int8 values in [-8, 7], ``[..., K, N]``."""
        lo = (self.packed & 0xF).to(torch.int8) - 8
        hi = (self.packed >> 4).to(torch.int8) - 8
        kn = torch.stack([lo, hi], -2).reshape(*self.packed.shape[:-2], -1, self.packed.shape[-1])
        return kn[..., :self.k, :]

    def dequant(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """Dense ``[..., N, K]``."""
        kn = self.codes().float()
        sc = self.scale.repeat_interleave(self.group_size, dim=-2)[..., :self.k, :]
        return (kn * sc).transpose(-1, -2).contiguous().to(dtype)

    def to(self, device) -> "W4A8Weight":
        return W4A8Weight(self.packed.to(device), self.scale.to(device), self.k, self.group_size)

    def to_nk(self) -> tuple[torch.Tensor, torch.Tensor]:
        """The layout the sm_100a kernels stream: codes ``[..., N, K/2]`` uint8 (byte ``j`` of a row =
        ``code(2j) | code(2j+1) << 4``) and scales ``[..., N, K/group]`` fp32.  ``K`` must be a multiple
        of the group size."""
        if self.k % self.group_size:
            raise ValueError(f"K={self.k} is not a multiple of the group size {self.group_size}")
        lo, hi = self.packed & 0xF, self.packed >> 4                               # [..., K/2, N] each
        kn = torch.stack([lo, hi], -2).reshape(*self.packed.shape[:-2], -1, self.packed.shape[-1])[..., :self.k, :]
        nk = kn.transpose(-1, -2)                                                  # [..., N, K]
        packed = (nk[..., 0::2] | (nk[..., 1::2] << 4)).to(torch.uint8).contiguous()
        return packed, self.scale.transpose(-1, -2).float().contiguous()


def quantize_state_dict(sd: dict[str, torch.Tensor], scheme: str = "int8") -> dict:
    """Replace every quantisable projection by its container (``int8`` or ``w4a8``)."""
    out = {}
    for k, v in sd.items():
        if isinstance(v, torch.Tensor) and is_quantizable(k, v):
            out[k] = QWeight.quantize(v) if scheme == "int8" else W4A8Weight.quantize(v)
        else:
            out[k] = v
    return out
