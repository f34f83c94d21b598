"""Tensor plan and random initialisation of a Qwen4-exp checkpoint.

Key names are the ``model.language_model.*`` checkpoint names of the family (module tree of the
reference: ``models/qwen4exp/blocks.py:52-110`` for a layer, ``gated_residual.py:66-90`` for a
hyper-connection, ``qsa.py:436-460`` for the indexer, ``ngram.py:759-790`` for a PLE layer,
``model.py:250-262`` for the stem and the final mixer).  The model has no pre-norms and no final
norm: every normalisation sits inside a hyper-connection.
"""
from __future__ import annotations

import math

import torch

from ...weights.init import _draw
from .config import INDEXED, LINEAR, Qwen4Config
from .ngram import NGramHasher

LM = "model.language_model."


def _hyper(prefix: str, cfg: Qwen4Config, add, write_gate: bool = True) -> None:
    W, R = cfg.hc_hidden, cfg.hc_lowrank
    add(prefix + "hc_norm.weight", (W,), "norm0")
    add(prefix + "input_mix_weight_down.weight", (R, W), "w")
    add(prefix + "input_mix_weight_up.weight", (W, R), "wide")
    if write_gate:
        add(prefix + "block_inject_weight.weight", (cfg.hc_count, W), "w")


def _layer_plan(p: str, kind: str, cfg: Qwen4Config, add, ple: int | None) -> None:
    """Tensors of one decoder layer under prefix ``p`` (``ple``: index of its n-gram table, or None)."""
    H = cfg.hidden_size
    if kind == LINEAR:
        q = p + "linear_attn."
        add(q + "in_proj_qkv.weight", (cfg.lin_conv_dim, H), "w")
        add(q + "in_proj_z.weight", (cfg.lin_vdim, H), "w")
        add(q + "in_proj_b.weight", (cfg.linear_num_value_heads, H), "w")
        add(q + "in_proj_a.weight", (cfg.linear_num_value_heads, H), "w")
        add(q + "conv1d.weight", (cfg.lin_conv_dim, 1, cfg.linear_conv_kernel_dim), "conv")
        add(q + "A_log", (cfg.linear_num_value_heads,), "alog")
        add(q + "dt_bias", (cfg.linear_num_value_heads,), "dt")
        add(q + "norm.weight", (cfg.linear_value_head_dim,), "norm1")
        add(q + "out_proj.weight", (H, cfg.lin_vdim), "w")
    else:
        q = p + "self_attn."
        nh, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        add(q + "q_proj.weight", (nh * 2 * hd, H), "w")
        add(q + "k_proj.weight", (nkv * hd, H), "w")
        add(q + "v_proj.weight", (nkv * hd, H), "w")
        add(q + "o_proj.weight", (H, nh * hd), "w")
        add(q + "q_norm.weight", (hd,), "norm0")
        add(q + "k_norm.weight", (hd,), "norm0")
        add(q + "indexer.index_qk_proj.weight", ((cfg.indexer_n_heads + 1) * cfg.indexer_head_dim, H), "w")
        add(q + "indexer.q_layernorm.weight", (cfg.indexer_head_dim,), "norm0")
        add(q + "indexer.k_layernorm.weight", (cfg.indexer_head_dim,), "norm0")
    m = p + "mlp."
    E, I, S = cfg.num_experts, cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size
    add(m + "gate.weight", (E, H), "wide")
    add(m + "experts.gate_up_proj", (E, 2 * I, H), "w")
    add(m + "experts.down_proj", (E, H, I), "w")
    add(m + "shared_expert.gate_proj.weight", (S, H), "w")
    add(m + "shared_expert.up_proj.weight", (S, H), "w")
    add(m + "shared_expert.down_proj.weight", (H, S), "w")
    add(m + "shared_expert_gate.weight", (1, H), "w")
    _hyper(p + "attn_hyper_connection.", cfg, add)
    _hyper(p + "mlp_hyper_connection.", cfg, add)
    j = ple
    if j is not None:
        q = p + "ple."
        rows = NGramHasher(cfg, j).rows
        add(q + "ple_embedding.ngram_embedding.weight", (rows, cfg.ngram_head_dim), "wide")
        add(q + "key_proj.weight", (cfg.hc_hidden, cfg.ple_embed_dim), "wide")
        add(q + "value_proj.weight", (H, cfg.ple_embed_dim), "wide")
        for n in ("norm_key", "norm_query", "norm_conv"):
            add(q + n + ".weight", (cfg.hc_hidden,), "norm0")
        add(q + "conv1d.weight", (cfg.hc_hidden, 1, cfg.ple_conv_kernel_size), "conv")


def tensor_plan(cfg: Qwen4Config) -> list[tuple[str, tuple[int, ...], str]]:
    plan: list[tuple[str, tuple[int, ...], str]] = []
    add = lambda k, s, kind: plan.append((k, s, kind))
    H = cfg.hidden_size
    add(LM + "embed_tokens.weight", (cfg.vocab_size, H), "w")
    for i, kind in enumerate(cfg.layer_types):
        _layer_plan(f"{LM}layers.{i}.", kind, cfg, add, cfg.ple_index(i))
    _hyper(LM + "hyper_connection_mixer.", cfg, add, write_gate=False)
    if not cfg.tie_word_embeddings:
        add("lm_head.weight", (cfg.vocab_size, H), "w")
    if cfg.mtp_num_hidden_layers:
        # the draft head: two [H, H] projections with their pre-norms (the hidden one spans all lanes),
        # one QSA + MoE layer without n-gram injection, and a final mixer without write gate
        # (``models/qwen4exp/mtp.py:146-200`` of the reference)
        add("mtp.fc_embedding.weight", (H, H), "w")
        add("mtp.fc_hidden.weight", (H, H), "w")
        add("mtp.pre_fc_norm_embedding.weight", (H,), "norm0")
        add("mtp.pre_fc_norm_hidden.weight", (cfg.hc_hidden,), "norm0")
        _layer_plan("mtp.layers.0.", INDEXED, cfg, add, None)
        _hyper("mtp.hyper_connection_mixer.", cfg, add, write_gate=False)
    return plan


def random_state_dict(cfg: Qwen4Config, seed: int = 0, dtype: torch.dtype = torch.float32,
                      device: str | torch.device = "cpu", std: float = 0.02) -> dict[str, torch.Tensor]:
    """Every tensor of ``tensor_plan``.  "wide" matrices (router, read-gate up-projection, PLE
    projections) are drawn ten times wider so that gates and routing are not degenerate at the
    tiny test widths; the generator is seeded per tensor."""
    sd: dict[str, torch.Tensor] = {}
    dev = torch.device(device)
    for idx, (key, shape, kind) in enumerate(tensor_plan(cfg)):
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed * 1_000_003 + idx)
        if kind == "wide":
            sd[key] = _draw(shape, "w", gen, dev, dtype, std * 10)
        else:
            sd[key] = _draw(shape, kind, gen, dev, dtype, std)
    return sd


class LazyRandomStateDict:
    """The tensors of ``random_state_dict`` drawn one at a time, on access: a model constructor that
    quantises every projection as it reads it then never holds more than one bf16 tensor of the full-size
    shape (the 48-layer geometry has 96 G expert parameters - 193 GB in bf16, 48 GB as int4).  The same
    per-tensor seeds as ``random_state_dict``, so both give the same weights."""

    def __init__(self, cfg: Qwen4Config, seed: int = 0, dtype: torch.dtype = torch.bfloat16,
                 device: str | torch.device = "cuda", std: float = 0.02) -> None:
        self.cfg, self.seed, self.dtype, self.device, self.std = cfg, seed, dtype, torch.device(device), std
        self.plan = {key: (idx, shape, kind) for idx, (key, shape, kind) in enumerate(tensor_plan(cfg))}

    def __contains__(self, key) -> bool:
        return key in self.plan

    def __iter__(self):
        return iter(self.plan)

    def keys(self):
        return self.plan.keys()

    def get(self, key, default=None):
        return self[key] if key in self.plan else default

    def __getitem__(self, key: str) -> torch.Tensor:
        idx, shape, kind = self.plan[key]
        gen = torch.Generator(device=self.device)
        gen.manual_seed(self.seed * 1_000_003 + idx)
        if kind == "wide":
            return _draw(shape, "w", gen, self.device, self.dtype, self.std * 10)
        return _draw(shape, kind, gen, self.device, self.dtype, self.std)


def param_count(cfg: Qwen4Config) -> int:
    return sum(math.prod(s) for _, s, _ in tensor_plan(cfg))


# ---------------------------------------------------------------------------------------------------
# Streaming loader: shard index, plan check, rank-filtered reads.
#
# A real checkpoint of this family is dominated by two things a rank must not read whole: the routed
# expert stacks (512 experts per layer) and the n-gram table of the PLE layer (tens of GiB).  The
# loader therefore works from the safetensors shard index, checks every planned tensor's presence and
# shape BEFORE reading any data, then streams shard by shard; under expert parallelism it reads only
# this rank's expert range of every stack (``get_slice``) and marks the dict so that the MoE module does
# not cut again.  Reference: ``models/qwen4exp/checkpoint.py`` (shard index + mmap) and
# ``models/qwen4exp/weights.py`` (``plan / verify / load_into / slice_experts``).
def checkpoint_index(model_dir) -> dict[str, str]:
    """``{tensor name: shard file}`` of a checkpoint directory (``model.safetensors.index.json`` when it
    exists, else the names found by opening every shard's header)."""
    import json
    from pathlib import Path

    from safetensors import safe_open
    d = Path(model_dir)
    idx = d / "model.safetensors.index.json"
    if idx.exists():
        return dict(json.loads(idx.read_text())["weight_map"])
    out: dict[str, str] = {}
    for f in sorted(d.glob("*.safetensors")):
        if f.name.startswith("quant-"):
            continue
        with safe_open(str(f), framework="pt") as fh:
            for k in fh.keys():
                out[k] = f.name
    if not out:
        raise FileNotFoundError(f"no safetensors shards in {d}")
    return out


NGRAM_SHARD = __import__("re").compile(r"^(.*\.ngram_embedding)\.shard_(\d+)\.weight$")


class ShardList(list):
    """Equally sized row shards of one table, in order, as host views (see ``ngram.ShardedNGramTable``);
    ``keep`` holds the file mappings behind them."""
    keep = None

    @property
    def shape(self) -> tuple:
        return (sum(int(t.shape[0]) for t in self), int(self[0].shape[1])) if self else (0, 0)


def open_mapped(path, names: list[str]) -> tuple[list[torch.Tensor], object]:
    """Tensors ``names`` of one safetensors file as VIEWS of a private file mapping (no copy into anonymous
    memory: the pages come and go with the page cache).  Returns ``(views, mapping)``; the views are valid
    while ``mapping`` is alive."""
    import json
    import os
    import struct
    dt = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "I8": torch.int8, "U8": torch.uint8,
          "I32": torch.int32, "I64": torch.int64}
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        hlen = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(hlen))
    buf = torch.from_file(str(path), shared=False, size=size, dtype=torch.uint8)
    views = []
    for n in names:
        e = header[n]
        a, b = e["data_offsets"]
        views.append(buf[8 + hlen + a:8 + hlen + b].view(dt[e["dtype"]]).reshape(e["shape"]))
    return views, buf


def verify_plan(cfg: Qwen4Config, model_dir, index: dict[str, str] | None = None) -> dict:
    """Compare the checkpoint's headers with ``tensor_plan(cfg)`` without reading tensor data.  Returns
    ``{"missing": [...], "unexpected": [...], "shape": [(key, found, wanted), ...]}``; per-expert spellings
    (``experts.{e}.gate_proj.weight`` ...) count for their fused stack."""
    import re
    from pathlib import Path

    from safetensors import safe_open
    index = index or checkpoint_index(model_dir)
    want = {k: tuple(s) for k, s, _ in tensor_plan(cfg)}
    shapes: dict[str, tuple] = {}
    for fname in sorted(set(index.values())):
        with safe_open(str(Path(model_dir) / fname), framework="pt") as fh:
            for k in fh.keys():
                shapes[k] = tuple(fh.get_slice(k).get_shape())
    # a table stored as shard_0 .. shard_{n-1}: equal shards count as one [n * rows, width] tensor
    tables: dict[str, dict[int, tuple]] = {}
    for k in list(shapes):
        m = NGRAM_SHARD.match(k)
        if m:
            tables.setdefault(m.group(1), {})[int(m.group(2))] = shapes.pop(k)
    for prefix, parts in tables.items():
        ks = sorted(parts)
        if ks == list(range(len(ks))) and len(set(parts.values())) == 1 and len(parts[0]) == 2:
            shapes[prefix + ".weight"] = (len(ks) * parts[0][0], parts[0][1])
        else:
            shapes[prefix + ".weight"] = ("shards", tuple(ks), tuple(sorted(set(parts.values()))))   # reported as a shape mismatch
    per_expert = re.compile(r"^(.*\.mlp\.experts\.)(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")
    fused_seen: dict[str, set] = {}
    for k in list(shapes):
        m = per_expert.match(k)
        if m:
            fused_seen.setdefault(m.group(1), set()).add(int(m.group(2)))
    missing, bad = [], []
    for k, s in want.items():
        if k in shapes:
            if shapes[k] != s:
                bad.append((k, shapes[k], s))
        elif k.endswith(("experts.gate_up_proj", "experts.down_proj")) and \
                len(fused_seen.get(k.rsplit(".", 1)[0] + ".", ())) == cfg.num_experts:
            continue
        else:
            missing.append(k)
    known = set(want) | {k for k in shapes if per_expert.match(k)}
    unexpected = [k for k in shapes if k not in known and k.startswith((LM, "lm_head."))]
    return {"missing": missing, "unexpected": unexpected, "shape": bad}


def first_layers(cfg: Qwen4Config, n: int) -> Qwen4Config:
    """Geometry of the first ``n`` layers as a model of its own (PLE layers keep their rank, which the n-gram
    hashing depends on)."""
    import dataclasses
    if n >= cfg.num_hidden_layers:
        return cfg
    return dataclasses.replace(cfg, num_hidden_layers=n, layer_types=cfg.layer_types[:n],
                               ple_layer_ids=tuple(i for i in cfg.ple_layer_ids if i <= n))


def load_streaming(model_dir, cfg: Qwen4Config | None = None, device: str = "cpu", ep: tuple[int, int] | None = None,
                   strict: bool = True, layers: int | None = None) -> dict[str, torch.Tensor]:
    """State dict of a Qwen4-exp checkpoint read shard by shard.  ``ep=(rank, world)``: only this rank's
    contiguous expert range of every routed stack is read (and the dict is marked ``__ep_shard__``); all
    other tensors are read whole.  ``strict``: refuse a checkpoint whose headers do not match the plan.
    ``layers``: read only the first ``layers`` decoder layers (a staged check of a checkpoint too large to
    load whole; pair it with ``first_layers(cfg, layers)``)."""
    from pathlib import Path

    from safetensors import safe_open

    from ...config import load_config
    from ...weights.loader import fuse_experts
    d = Path(model_dir)
    cfg = cfg or load_config(d)
    index = checkpoint_index(d)
    if strict:
        rep = verify_plan(cfg, d, index)
        if rep["missing"] or rep["shape"]:
            raise ValueError(f"{d}: checkpoint does not match the tensor plan: missing {rep['missing'][:4]} "
                             f"shape {rep['shape'][:2]}")
    E = cfg.num_experts
    lo, hi = 0, E
    if ep is not None and ep[1] > 1:
        if E % ep[1]:
            raise ValueError(f"num_experts={E} is not divisible by expert-parallel world {ep[1]}")
        per = E // ep[1]
        lo, hi = ep[0] * per, (ep[0] + 1) * per
    sd: dict[str, torch.Tensor] = {}
    by_file: dict[str, list[str]] = {}
    for k, f in index.items():
        by_file.setdefault(f, []).append(k)
    import re
    per_expert = re.compile(r"\.mlp\.experts\.(\d+)\.")
    table_shards: dict[str, dict[int, tuple[str, str]]] = {}
    layer_no = re.compile(re.escape(LM) + r"layers\.(\d+)\.")
    for fname in sorted(by_file):
        with safe_open(str(d / fname), framework="pt", device=device) as fh:
            for k in by_file[fname]:
                if not k.startswith((LM, "lm_head.", "mtp.", "model.visual.")):
                    continue
                if layers is not None:
                    ml = layer_no.match(k)
                    if (ml and int(ml.group(1)) >= layers) or k.startswith(("mtp.", "model.visual.")):
                        continue
                ms = NGRAM_SHARD.match(k)
                if ms:                                          # mapped after the loop, never copied
                    table_shards.setdefault(ms.group(1), {})[int(ms.group(2))] = (fname, k)
                    continue
                if k.endswith(("experts.gate_up_proj", "experts.down_proj")) and (lo, hi) != (0, E):
                    sd[k] = fh.get_slice(k)[lo:hi]
                    continue
                m = per_expert.search(k)
                if m and not (lo <= int(m.group(1)) < hi):
                    continue                                   # another rank's expert
                sd[k] = fh.get_tensor(k)
    if (lo, hi) != (0, E):
        # per-expert spellings: renumber the kept experts from 0 so that they fuse into a local stack
        ren = {}
        for k, v in sd.items():
            m = per_expert.search(k)
            ren[k[:m.start(1)] + str(int(m.group(1)) - lo) + k[m.end(1):] if m else k] = v
        sd = ren
    sd = fuse_experts(sd)
    for prefix, parts in table_shards.items():
        ks = sorted(parts)
        if ks != list(range(len(ks))):
            raise ValueError(f"{prefix}: shards {ks[:4]}.. are not 0..{len(ks) - 1}; a missing shard would shift every later row")
        lst, keep = ShardList(), []
        by_f: dict[str, list[tuple[int, str]]] = {}
        for k in ks:
            by_f.setdefault(parts[k][0], []).append((k, parts[k][1]))
        got: dict[int, torch.Tensor] = {}
        for fname, items in by_f.items():
            views, mapping = open_mapped(d / fname, [name for _, name in items])
            keep.append(mapping)
            for (k, _), v in zip(items, views):
                got[k] = v
        lst.extend(got[k] for k in ks)
        lst.keep = keep
        sd[prefix + ".weight"] = lst
    if (lo, hi) != (0, E):
        sd["__ep_shard__"] = (ep[0], ep[1])
    return sd
