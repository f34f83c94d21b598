"""Model geometry for the Qwen3.5-style hybrid family.

The geometry is read from a checkpoint's ``config.json`` (``text_config`` block, the
same keys the reference reads in ``models/qwen35/model.py:107-130`` and
``models/qwen35/linear_attn.py:63-85``) or taken from one of the named presets below,
which restate the benchmark shapes.  One dataclass carries everything a layer needs,
so that the CPU oracle, the sm_100a model and the weight tools agree on shapes.
"""
from __future__ import annotations

import dataclasses
import json
from pathlib import Path
from typing import Any

LINEAR = "linear_attention"
FULL = "full_attention"


@dataclasses.dataclass
class ModelConfig:
    """Text-model geometry (one instance per checkpoint)."""

    vocab_size: int = 4096
    hidden_size: int = 256
    num_hidden_layers: int = 4
    layer_types: tuple[str, ...] = (LINEAR, LINEAR, LINEAR, FULL)
    # gated softmax attention
    num_attention_heads: int = 4
    num_key_value_heads: int = 2
    head_dim: int = 64
    partial_rotary_factor: float = 0.25
    rope_theta: float = 1e7
    mrope_section: tuple[int, int, int] = (11, 11, 10)
    # gated delta net
    linear_num_key_heads: int = 4
    linear_num_value_heads: int = 4
    linear_key_head_dim: int = 64
    linear_value_head_dim: int = 64
    linear_conv_kernel_dim: int = 4
    # FFN
    intermediate_size: int = 768
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    shared_expert_intermediate_size: int = 0
    norm_topk_prob: bool = True
    # misc
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = True
    mtp_num_hidden_layers: int = 0
    architecture: str = "qwen3_5"
    name: str = "tiny"

    # ---- derived -------------------------------------------------------
    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def lin_kdim(self) -> int:
        return self.linear_num_key_heads * self.linear_key_head_dim

    @property
    def lin_vdim(self) -> int:
        return self.linear_num_value_heads * self.linear_value_head_dim

    @property
    def lin_conv_dim(self) -> int:
        return 2 * self.lin_kdim + self.lin_vdim

    @property
    def lin_rep(self) -> int:
        return self.linear_num_value_heads // self.linear_num_key_heads

    @property
    def q_rep(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def full_layers(self) -> list[int]:
        return [i for i, t in enumerate(self.layer_types) if t != LINEAR]

    @property
    def linear_layers(self) -> list[int]:
        return [i for i, t in enumerate(self.layer_types) if t == LINEAR]

    def validate(self) -> None:
        if len(self.layer_types) != self.num_hidden_layers:
            raise ValueError(f"layer_types has {len(self.layer_types)} entries for "
                             f"{self.num_hidden_layers} layers")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.linear_num_value_heads % self.linear_num_key_heads:
            raise ValueError("linear value heads must be a multiple of key heads")
        if self.rotary_dim % 2:
            raise ValueError("rotary_dim must be even")

    # ---- (de)serialisation --------------------------------------------
    def to_hf(self) -> dict[str, Any]:
        """The ``config.json`` dict a checkpoint directory of this model carries."""
        text = {
            "model_type": "qwen3_5_text" if not self.is_moe else "qwen3_5_moe_text",
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "layer_types": list(self.layer_types),
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "rope_parameters": {"rope_theta": self.rope_theta,
                                "partial_rotary_factor": self.partial_rotary_factor,
                                "mrope_section": list(self.mrope_section),
                                "rope_type": "default"},
            "linear_num_key_heads": self.linear_num_key_heads,
            "linear_num_value_heads": self.linear_num_value_heads,
            "linear_key_head_dim": self.linear_key_head_dim,
            "linear_value_head_dim": self.linear_value_head_dim,
            "linear_conv_kernel_dim": self.linear_conv_kernel_dim,
            "intermediate_size": self.intermediate_size,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "mtp_num_hidden_layers": self.mtp_num_hidden_layers,
        }
        if self.is_moe:
            text.update({"num_experts": self.num_experts,
                         "num_experts_per_tok": self.num_experts_per_tok,
                         "moe_intermediate_size": self.moe_intermediate_size,
                         "shared_expert_intermediate_size": self.shared_expert_intermediate_size,
                         "norm_topk_prob": self.norm_topk_prob})
        return {"architectures": ["Qwen3_5ForConditionalGeneration"],
                "model_type": self.architecture, "text_config": text,
                "tie_word_embeddings": self.tie_word_embeddings}

    @classmethod
    def from_hf(cls, raw: dict[str, Any], name: str = "checkpoint") -> "ModelConfig":
        t = raw.get("text_config", raw)
        rp = t.get("rope_parameters") or {}
        n = int(t["num_hidden_layers"])
        types = t.get("layer_types")
        if types is None:
            interval = int(t.get("full_attention_interval", 4))
            types = [FULL if (i + 1) % interval == 0 else LINEAR for i in range(n)]
        cfg = cls(
            vocab_size=int(t["vocab_size"]), hidden_size=int(t["hidden_size"]),
            num_hidden_layers=n, layer_types=tuple(types),
            num_attention_heads=int(t["num_attention_heads"]),
            num_key_value_heads=int(t["num_key_value_heads"]),
            head_dim=int(t.get("head_dim", t["hidden_size"] // t["num_attention_heads"])),
            partial_rotary_factor=float(rp.get("partial_rotary_factor",
                                               t.get("partial_rotary_factor", 0.25))),
            rope_theta=float(rp.get("rope_theta", t.get("rope_theta", 1e7))),
            mrope_section=tuple(rp.get("mrope_section", (11, 11, 10))),
            linear_num_key_heads=int(t.get("linear_num_key_heads", 1)),
            linear_num_value_heads=int(t.get("linear_num_value_heads", 1)),
            linear_key_head_dim=int(t.get("linear_key_head_dim", 128)),
            linear_value_head_dim=int(t.get("linear_value_head_dim", 128)),
            linear_conv_kernel_dim=int(t.get("linear_conv_kernel_dim", 4)),
            intermediate_size=int(t.get("intermediate_size", 0)),
            num_experts=int(t.get("num_experts", 0) or 0),
            num_experts_per_tok=int(t.get("num_experts_per_tok", 0) or 0),
            moe_intermediate_size=int(t.get("moe_intermediate_size", 0) or 0),
            shared_expert_intermediate_size=int(t.get("shared_expert_intermediate_size", 0) or 0),
            norm_topk_prob=bool(t.get("norm_topk_prob", True)),
            rms_norm_eps=float(t.get("rms_norm_eps", 1e-6)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings",
                                             t.get("tie_word_embeddings", True))),
            mtp_num_hidden_layers=int(t.get("mtp_num_hidden_layers", 0) or 0),
            architecture=str(raw.get("model_type", "qwen3_5")),
            name=name,
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_dir(cls, model_dir: str | Path) -> "ModelConfig":
        p = Path(model_dir)
        return cls.from_hf(json.loads((p / "config.json").read_text()), name=p.name)


def _pattern(n: int, interval: int = 4) -> tuple[str, ...]:
    return tuple(FULL if (i + 1) % interval == 0 else LINEAR for i in range(n))


def preset(name: str) -> ModelConfig:
    """Named benchmark shapes.

    ``tiny``: 4-layer fp32 oracle model.  ``qwen35-4b``: dense 32-layer bf16 model.
    ``qwen35-27b``: dense 64-layer model for the int8 tensor-parallel run.
    ``qwen35-35b-a3b``: 40-layer routed-MoE model (256 experts, top-8, one shared expert).
    """
    if name == "tiny":
        return ModelConfig()
    if "qwen4" in name:
        from .models.qwen4exp.config import preset_qwen4
        return preset_qwen4(name)
    if name == "tiny-moe":
        return ModelConfig(name="tiny-moe", num_experts=8, num_experts_per_tok=2,
                           moe_intermediate_size=128, shared_expert_intermediate_size=128,
                           intermediate_size=0)
    if name == "qwen35-4b":
        return ModelConfig(name=name, vocab_size=151936, hidden_size=2560, num_hidden_layers=32,
                           layer_types=_pattern(32), num_attention_heads=16,
                           num_key_value_heads=4, head_dim=256, linear_num_key_heads=16,
                           linear_num_value_heads=32, linear_key_head_dim=128,
                           linear_value_head_dim=128, intermediate_size=9216)
    if name == "qwen35-27b":
        return ModelConfig(name=name, vocab_size=151936, hidden_size=5120, num_hidden_layers=64,
                           layer_types=_pattern(64), num_attention_heads=24,
                           num_key_value_heads=4, head_dim=256, linear_num_key_heads=16,
                           linear_num_value_heads=48, linear_key_head_dim=128,
                           linear_value_head_dim=128, intermediate_size=17408,
                           tie_word_embeddings=False)
    if name == "qwen35-35b-a3b":
        return ModelConfig(name=name, vocab_size=151936, hidden_size=2048, num_hidden_layers=40,
                           layer_types=_pattern(40), num_attention_heads=16,
                           num_key_value_heads=2, head_dim=256, linear_num_key_heads=16,
                           linear_num_value_heads=32, linear_key_head_dim=128,
                           linear_value_head_dim=128, intermediate_size=0, num_experts=256,
                           num_experts_per_tok=8, moe_intermediate_size=512,
                           shared_expert_intermediate_size=512, tie_word_embeddings=False)
    raise KeyError(f"unknown preset {name!r}")


PRESETS = ("tiny", "tiny-moe", "qwen35-4b", "qwen35-27b", "qwen35-35b-a3b")


def load_config(model_dir: str | Path):
    """Config object of a checkpoint directory, of whichever family its ``config.json`` names."""
    raw = json.loads((Path(model_dir) / "config.json").read_text())
    kind = str(raw.get("model_type", "")) + " " + " ".join(raw.get("architectures", []))
    if "qwen4" in kind.lower():
        from .models.qwen4exp.config import Qwen4Config
        return Qwen4Config.from_hf(raw, name=Path(model_dir).name)
    return ModelConfig.from_hf(raw, name=Path(model_dir).name)
