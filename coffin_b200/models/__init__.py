"""Model families. ``build_model`` maps a config to the sm_100a implementation.

Counterpart of the reference's family registry (``engine_api.py:210-361``): the architecture
string of ``config.json`` selects the class; here there is one backend, so the registry maps
names to classes only.
"""
from __future__ import annotations

from typing import Callable

from ..config import ModelConfig

_REGISTRY: dict[str, Callable] = {}


def register(name: str, factory: Callable) -> None:
    _REGISTRY[name] = factory


def registered() -> list[str]:
    _ensure_builtin()
    return sorted(_REGISTRY)


def _nccl_only() -> bool:
    """``COFFIN_TP_NCCL=1``: the prefill and wide-bucket all-reduces go through NCCL between kernels
    instead of the peer-memory exchange fused into the GEMM epilogue (the A/B baseline of the fused path)."""
    import os
    return os.environ.get("COFFIN_TP_NCCL") == "1"


def _ensure_builtin() -> None:
    if _REGISTRY:
        return

    def qwen35(cfg, sd, **kw):
        from .qwen35.model import Qwen35Model
        tp_world, tp_rank = kw.pop("tp_world", 1), kw.pop("tp_rank", 0)
        ep_world, ep_rank = kw.pop("ep_world", 1), kw.pop("ep_rank", 0)
        pp_world, pp_rank = kw.pop("pp_world", 1), kw.pop("pp_rank", 0)
        if pp_world > 1:
            from ..parallel.pp import build_stage
            return build_stage(cfg, sd, pp_rank, pp_world, lanes=kw.pop("pp_lanes", 2), **kw)
        if ep_world > 1:
            # expert parallel: attention / delta-net / dense weights replicated, routed experts split
            from ..parallel.tp import TpComm, make_exchange
            comm = TpComm(ep_rank, ep_world, cfg.hidden_size, 8, 2 * cfg.num_hidden_layers, exchange=make_exchange(),
                          prefill_rows=0 if _nccl_only() else kw.get("max_chunk", 2048))
            return Qwen35Model(cfg, sd, tp=comm, ep_rank=ep_rank, ep_world=ep_world, **kw)
        if tp_world > 1:
            from ..parallel.tp import TpComm, local_config, make_exchange, shard_state_dict
            lcfg = local_config(cfg, tp_world)
            lsd = shard_state_dict(cfg, sd, tp_rank, tp_world)
            n_sites = 2 * cfg.num_hidden_layers + 2      # two per layer + the vocabulary-parallel arg-max
            tp = TpComm(tp_rank, tp_world, cfg.hidden_size, 8, n_sites, exchange=make_exchange(),
                        prefill_rows=0 if _nccl_only() else kw.get("max_chunk", 2048))
            kw.pop("free_source", None)
            return Qwen35Model(lcfg, lsd, tp=tp, full_cfg=cfg, **kw)
        return Qwen35Model(cfg, sd, **kw)

    for n in ("qwen3_5", "qwen35", "qwen3_5_moe", "qwen3_5_text", "qwen3_next"):
        register(n, qwen35)

    def qwen4(cfg, sd, **kw):
        from .qwen4exp.model import Qwen4ExpModel
        if kw.pop("tp_world", 1) > 1 or kw.pop("pp_world", 1) > 1:
            raise NotImplementedError("the Qwen4-exp family runs on one GPU or expert parallel (ep_world), as its reference does")
        kw.pop("tp_rank", None), kw.pop("pp_rank", None)
        ep_world, ep_rank = kw.pop("ep_world", 1), kw.pop("ep_rank", 0)
        if ep_world > 1:
            from ..parallel.tp import TpComm, make_exchange
            comm = TpComm(ep_rank, ep_world, cfg.hidden_size, 8, 2, exchange=make_exchange(),
                          prefill_rows=0 if _nccl_only() else kw.get("max_chunk", 2048))
            return Qwen4ExpModel(cfg, sd, tp=comm, ep_rank=ep_rank, ep_world=ep_world, **kw)
        return Qwen4ExpModel(cfg, sd, **kw)

    for n in ("qwen4_exp", "qwen4exp"):
        register(n, qwen4)


def detect_architecture(cfg: ModelConfig) -> str:
    """Registry key for a config; unknown names fall back on geometry (a config that has
    delta-net heads is a Qwen3.5-style hybrid), as ``engine_api.py:295-297`` does."""
    _ensure_builtin()
    if cfg.architecture in _REGISTRY:
        return cfg.architecture
    if cfg.linear_num_value_heads > 0:
        return "qwen3_5"
    raise RuntimeError(f"no registered model family for architecture {cfg.architecture!r}")


def attach_vision(model, cfg, sd: dict, vision=None, model_dir=None) -> None:
    """Give ``model`` a ``vision`` tower when the checkpoint carries ``model.visual.*`` tensors, or
    when ``vision`` is a ``VisionConfig`` / the string ``"tiny"`` / ``"default"`` (random weights of
    that geometry - for benchmarks and tests; reference: the tower is optional and loaded on demand,
    ``models/qwen35/model.py:213-266``)."""
    from .qwen35.vision import V, VisionConfig, VisionTower, random_vision_state_dict, tiny_vision
    has = any(k.startswith(V) for k in sd)
    if not has and not vision:
        return
    if isinstance(vision, VisionConfig):
        vcfg = vision
    elif vision == "tiny":
        vcfg = tiny_vision(cfg.hidden_size)
    elif model_dir is not None:
        import json
        from pathlib import Path
        vcfg = VisionConfig.from_hf(json.loads((Path(model_dir) / "config.json").read_text()), cfg.hidden_size)
    else:
        vcfg = VisionConfig(out_hidden_size=cfg.hidden_size)
    vsd = sd if has else random_vision_state_dict(vcfg)
    if getattr(model, "device", None) is not None and str(model.device).startswith("cuda"):
        model.vision = VisionTower(vcfg, vsd, device=model.device)
    else:
        from .qwen35.vision import OracleVision
        model.vision = OracleVision(vcfg, {k: v.float() for k, v in vsd.items() if k.startswith(V)})


def build_model(cfg: ModelConfig, sd: dict, **kw):
    """``vision`` (``None`` / ``"tiny"`` / ``"default"`` / a ``VisionConfig``) and ``model_dir`` are
    consumed here: the tower is attached after the text model is built."""
    _ensure_builtin()
    vision, model_dir = kw.pop("vision", None), kw.pop("model_dir", None)
    has_visual = any(k.startswith("model.visual.") for k in sd)
    vsd = {k: v for k, v in sd.items() if k.startswith("model.visual.")} if has_visual else {}
    arch = detect_architecture(cfg)
    want_vision = bool(vision or has_visual) and vision is not False
    if want_vision and arch in ("qwen4_exp", "qwen4exp"):
        kw.setdefault("mrope_cache", True)     # image tokens rotate with 3-axis positions: the family keeps the rows per slot
    model = _REGISTRY[arch](cfg, sd, **kw)
    if want_vision:
        attach_vision(model, cfg, vsd, vision, model_dir)
    return model
