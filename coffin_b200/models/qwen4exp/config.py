"""Geometry of the Qwen4-exp family: hybrid delta-net / block-sparse ("QSA") attention layers on a
four-lane hyper-connected residual stream, a routed MoE in every layer and an optional n-gram
("PLE") injection.

The field names are the ``config.json`` keys of the family (``text_config`` block); what the
reference derives in ``models/qwen4exp/config.py:108-250`` (layer types from the interval, the QSA
block top-k from budget / ratio, the PLE conv state length, rotary width) is derived here as
properties.  One instance serves the fp32 oracle, the sm_100a model and the weight tools.
"""
from __future__ import annotations

import dataclasses
import json
from pathlib import Path
from typing import Any

LINEAR = "linear_attention"
INDEXED = "indexed_attention"
_ALIASES = {"full_attention": INDEXED}


@dataclasses.dataclass
class Qwen4Config:
    vocab_size: int = 248320
    hidden_size: int = 2560
    num_hidden_layers: int = 48
    layer_types: tuple[str, ...] = ()
    full_attention_interval: int = 4
    # gated block-sparse attention
    num_attention_heads: int = 16
    num_key_value_heads: int = 2
    head_dim: int = 256
    partial_rotary_factor: float = 1.0
    rope_theta: float = 10000.0
    mrope_section: tuple[int, ...] = ()
    indexer_n_heads: int = 4
    indexer_head_dim: int = 128
    indexer_budget: int = 2048
    indexer_compress_ratio: int = 64
    full_select_factor: int = 2
    # gated delta net
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4
    output_gate_type: str = "silu"
    # MoE
    num_experts: int = 512
    num_experts_per_tok: int = 10
    moe_intermediate_size: int = 512
    shared_expert_intermediate_size: int = 512
    norm_topk_prob: bool = True
    # hyper-connection
    hc_count: int = 4
    hc_lowrank: int = 320
    # n-gram embedding injection
    ple_layer_ids: tuple[int, ...] = ()          # one-based layer numbers
    ple_embed_dim: int = 0                       # 0: hidden_size
    ple_conv_kernel_size: int = 4
    ngram_size: int = 3
    heads_per_ngram: int = 8
    ngram_vocab_size_base: int = 20_000_000
    make_ngram_vocab_size_divisible_by: int = 128
    seed: int = 1234
    eos_token_id: int = 0
    # misc
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    mtp_num_hidden_layers: int = 0
    architecture: str = "qwen4_exp"
    name: str = "qwen4exp"

    def __post_init__(self) -> None:
        if not self.layer_types:
            k = self.full_attention_interval
            self.layer_types = tuple(LINEAR if (i + 1) % k else INDEXED for i in range(self.num_hidden_layers))
        self.layer_types = tuple(_ALIASES.get(t, t) for t in self.layer_types)
        self.mrope_section = tuple(self.mrope_section)
        self.ple_layer_ids = tuple(sorted(set(int(i) for i in self.ple_layer_ids)))
        if not self.ple_embed_dim:
            self.ple_embed_dim = self.hidden_size
        self.validate()

    # ---- derived -------------------------------------------------------------------------
    @property
    def hc_hidden(self) -> int:
        return self.hc_count * self.hidden_size

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def q_rep(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def block_topk(self) -> int:
        return self.indexer_budget // self.indexer_compress_ratio

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
    def linear_layers(self) -> list[int]:
        return [i for i, t in enumerate(self.layer_types) if t == LINEAR]

    @property
    def full_layers(self) -> list[int]:
        return [i for i, t in enumerate(self.layer_types) if t == INDEXED]

    @property
    def ngram_heads(self) -> int:
        return (self.ngram_size - 1) * self.heads_per_ngram

    @property
    def ngram_head_dim(self) -> int:
        return self.ple_embed_dim // self.ngram_heads

    @property
    def ple_conv_dilation(self) -> int:
        return self.ngram_size

    @property
    def ple_conv_state_len(self) -> int:
        return (self.ple_conv_kernel_size - 1) * self.ngram_size

    @property
    def ple_context_len(self) -> int:
        return self.ngram_size - 1

    @property
    def is_moe(self) -> bool:
        return True

    def ple_index(self, layer: int) -> int | None:
        """Rank of zero-based ``layer`` among the PLE layers, or ``None``."""
        return self.ple_layer_ids.index(layer + 1) if (layer + 1) in self.ple_layer_ids else None

    def validate(self) -> None:
        if len(self.layer_types) != self.num_hidden_layers:
            raise ValueError(f"layer_types has {len(self.layer_types)} entries for {self.num_hidden_layers} layers")
        bad = sorted(set(self.layer_types) - {LINEAR, INDEXED})
        if bad:
            raise ValueError(f"unsupported layer types {bad}")
        if self.hc_count < 2:
            raise ValueError("hc_count must be at least 2")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.linear_num_value_heads % self.linear_num_key_heads:
            raise ValueError("linear value heads must be a multiple of key heads")
        if self.indexer_budget % self.indexer_compress_ratio:
            raise ValueError("indexer_budget must be a multiple of indexer_compress_ratio")
        if self.rotary_dim % 2 or self.rotary_dim > self.indexer_head_dim:
            raise ValueError("rotary_dim must be even and fit the index head")
        if not 0 < self.num_experts_per_tok <= self.num_experts:
            raise ValueError("num_experts_per_tok out of range")
        if self.output_gate_type not in ("silu", "sigmoid"):
            raise ValueError(f"unsupported output gate {self.output_gate_type!r}")
        for one in self.ple_layer_ids:
            if not 1 <= one <= self.num_hidden_layers or self.layer_types[one - 1] != LINEAR:
                raise ValueError(f"PLE layer {one} must be an existing linear_attention layer")
        if self.mtp_num_hidden_layers not in (0, 1):
            # each draft step would use another layer; the head drives exactly one
            raise ValueError(f"the draft head has exactly one layer, the config declares {self.mtp_num_hidden_layers}")
        if self.ple_layer_ids and self.ple_embed_dim % self.ngram_heads:
            raise ValueError("ple_embed_dim must divide by the number of n-gram heads")

    # ---- (de)serialisation ----------------------------------------------------------------
    @classmethod
    def from_hf(cls, raw: dict[str, Any], name: str = "checkpoint") -> "Qwen4Config":
        t = dict(raw.get("text_config", raw))
        rope = t.pop("rope_parameters", None) or t.pop("rope_scaling", None) or {}
        for k in ("rope_theta", "partial_rotary_factor", "mrope_section"):
            if rope.get(k) is not None:
                t[k] = rope[k]
        eos = t.get("eos_token_id")
        if isinstance(eos, list):
            t["eos_token_id"] = int(eos[0]) if eos else 0
        if t.get("head_dim") is None and "hidden_size" in t and "num_attention_heads" in t:
            t["head_dim"] = t["hidden_size"] // t["num_attention_heads"]
        if t.get("output_gate_type") is None:
            t["output_gate_type"] = t.get("hidden_act", "silu") if t.get("hidden_act") in ("silu", "sigmoid") else "silu"
        known = {f.name for f in dataclasses.fields(cls)}
        kw = {k: (tuple(v) if isinstance(v, list) else v) for k, v in t.items() if k in known and v is not None}
        kw["name"] = name
        return cls(**kw)

    @classmethod
    def from_dir(cls, path: str | Path) -> "Qwen4Config":
        p = Path(path)
        return cls.from_hf(json.loads((p / "config.json").read_text()), name=p.name)

    def to_hf(self) -> dict[str, Any]:
        t = dataclasses.asdict(self)
        for k in ("architecture", "name", "full_select_factor"):
            t.pop(k)
        t["layer_types"] = list(self.layer_types)
        t["rope_parameters"] = {"rope_theta": t.pop("rope_theta"), "partial_rotary_factor": t.pop("partial_rotary_factor"),
                                "mrope_section": list(t.pop("mrope_section")), "rope_type": "default"}
        t["ple_layer_ids"] = list(self.ple_layer_ids)
        t["indexer_kv_heads"] = 1
        t["model_type"] = "qwen4_exp_text"
        return {"architectures": ["Qwen4ExpForConditionalGeneration"], "model_type": self.architecture, "text_config": t}


def tiny_qwen4(**over) -> Qwen4Config:
    """Eight-layer test geometry: 6 delta-net + 2 QSA layers, 16 experts top-2, PLE on layer 2,
    compress ratio 4 with a budget of 16 tokens so that a 100-token context is already sparse."""
    kw = dict(vocab_size=1024, hidden_size=128, num_hidden_layers=8, num_attention_heads=4, num_key_value_heads=2,
              head_dim=64, partial_rotary_factor=0.5, indexer_n_heads=2, indexer_head_dim=64, indexer_budget=16,
              indexer_compress_ratio=4, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=64,
              linear_value_head_dim=64, num_experts=16, num_experts_per_tok=2, moe_intermediate_size=64,
              shared_expert_intermediate_size=64, hc_count=4, hc_lowrank=32, ple_layer_ids=(2,), ple_embed_dim=64,
              heads_per_ngram=4, mrope_section=(6, 5, 5), ngram_vocab_size_base=500, make_ngram_vocab_size_divisible_by=8, eos_token_id=1,
              name="tiny-qwen4")
    kw.update(over)
    return Qwen4Config(**kw)


def preset_qwen4(name: str) -> Qwen4Config:
    """``tiny-qwen4``: the test geometry.  ``qwen4exp-a``: the family's default shape (48 layers,
    hidden 2560, 512 experts top-10, four residual lanes) without the n-gram table."""
    if name == "tiny-qwen4":
        return tiny_qwen4()
    if name == "qwen4exp-a":
        return Qwen4Config(name=name, vocab_size=151936, head_dim=256, partial_rotary_factor=0.25,
                           mrope_section=(11, 11, 10), rope_theta=1e7)
    raise KeyError(f"unknown Qwen4-exp preset {name!r}")
