"""Reader and writer of pre-quantised checkpoint directories (``quant_index.json``).

Two formats, byte-compatible with the reference's tools:

* ``coffin-int8-kn-v1``: tensor ``key`` int8 ``[K, N]`` + ``key#scale`` fp32 ``[N]``; routed
  experts as stacks ``...experts.gate_up_stack`` / ``down_stack`` int8 ``[E, K, N]`` with
  ``#scale [E, N]`` and an ``#nk`` copy ``[E, N, K]``; shards ``quant-%05d-of-%05d.safetensors``.
* ``coffin-w4a8-kn-v1``: ``key`` uint8 ``[ceil(K/2), N]`` + ``key#scale`` fp32 ``[ceil(K/128), N]``
  (kind ``q4``; experts ``q4-moe`` ``[E, ceil(K/2), N]``); shards ``quant-w4a8-...``.

The index records per tensor its kind (``q8 | q8-moe | q4 | q4-moe | dense``), ``k``, ``n``, shape,
``scale_key``, ``nk_key`` and shard, plus the sha256 of the source ``config.json`` which the reader
checks.  Reference: ``quantized_load.py:46-51,190-454``, ``tools/quant_disk.py:147-177,229-383,533-554``,
``tools/quant_disk_w4a8.py:45-89,241-281``.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from .quant import GROUP, QWeight, W4A8Weight, is_quantizable

INDEX_NAME = "quant_index.json"
FORMAT = "coffin-int8-kn-v1"
W4A8_FORMAT = "coffin-w4a8-kn-v1"
# top level of a tree of per-rank directories (tools/quant_disk_qwen4.py --layout): a manifest, not loadable weights
MANIFEST_FORMAT = "coffin-qwen4-w4a8-manifest-v1"
DENSE_SUFFIXES = ("mlp.gate.weight", "shared_expert_gate.weight")


def is_quantized_dir(model_dir: str | Path) -> bool:
    return (Path(model_dir) / INDEX_NAME).is_file()


def read_index(model_dir: str | Path) -> dict:
    idx = json.loads((Path(model_dir) / INDEX_NAME).read_text())
    if idx.get("format") == MANIFEST_FORMAT:
        dirs = {lay: sorted(per.values()) for lay, per in idx.get("rank_dirs", {}).items()}
        raise ValueError(f"{model_dir}: this is the manifest of a per-rank tree, not a loadable directory; "
                         f"load one of its rank directories: {dirs}")
    if idx.get("format") not in (FORMAT, W4A8_FORMAT):
        raise ValueError(f"{model_dir}: unknown quantised format {idx.get('format')!r}")
    return idx


def config_digest(model_dir: str | Path) -> str:
    return hashlib.sha256((Path(model_dir) / "config.json").read_bytes()).hexdigest()


def _disk_key(key: str) -> str:
    if key.endswith("experts.gate_up_proj"):
        return key[:-len("gate_up_proj")] + "gate_up_stack"
    if key.endswith("experts.down_proj"):
        return key[:-len("down_proj")] + "down_stack"
    return key


def _mem_key(key: str) -> str:
    if key.endswith("experts.gate_up_stack"):
        return key[:-len("gate_up_stack")] + "gate_up_proj"
    if key.endswith("experts.down_stack"):
        return key[:-len("down_stack")] + "down_proj"
    return key


def write_quantized(model_dir: str | Path, sd, out_dir: str | Path, scheme: str = "int8",
                    shard_bytes: int = 4 << 30, weight_dtype: str = "bfloat16", is_q=None, generated_by: str | None = None) -> dict:
    """Quantise ``sd`` (dense, HF key layout) and write a pre-quantised directory next to a copy
    of ``config.json`` from ``model_dir``.  ``sd`` is a mapping or any iterable of ``(key, tensor)``
    pairs, consumed once in order (a streaming source never has to hold the whole model); ``is_q(key,
    tensor)`` replaces the default choice of which tensors are quantised."""
    from safetensors.torch import save_file
    src, out = Path(model_dir), Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_bytes((src / "config.json").read_bytes())
    w4 = scheme == "w4a8"
    tensors: dict[str, dict] = {}
    cur: dict[str, torch.Tensor] = {}
    tmp_files: list[Path] = []
    size = 0

    def flush() -> None:
        """Write the shard collected so far (under a temporary name: the final names carry the shard
        count, known only at the end) and drop its tensors, so memory stays at one shard."""
        nonlocal cur, size
        if cur:
            path = out / f"quant-part-{len(tmp_files) + 1:05d}.tmp"
            save_file(cur, str(path))
            tmp_files.append(path)
        cur, size = {}, 0

    def put(group: dict[str, torch.Tensor]) -> int:
        """Add the tensors of one logical weight (codes, scales, ...) to the SAME shard (the index records
        one shard per weight) and return its number."""
        nonlocal size
        nb = sum(t.numel() * t.element_size() for t in group.values())
        if size and size + nb > shard_bytes:
            flush()
        for name, t in group.items():
            cur[name] = t.contiguous().cpu()
        size += nb
        return len(tmp_files)

    kinds: dict[str, int] = {}
    has_visual = False
    pick = is_q or is_quantizable
    for key, t in (sd.items() if hasattr(sd, "items") else sd):
        dk = _disk_key(key)
        moe = t.dim() == 3
        has_visual = has_visual or key.startswith("model.visual.")
        if pick(key, t) and not key.endswith(DENSE_SUFFIXES):
            if w4:
                q = W4A8Weight.quantize(t)
                kind = "q4-moe" if moe else "q4"
                si = put({dk: q.packed, dk + "#scale": q.scale})
                meta = {"kind": kind, "k": q.k, "n": q.n, "shape": list(q.packed.shape), "scale_key": dk + "#scale",
                        "group_size": GROUP, "shard": si}
            else:
                q = QWeight.quantize(t)
                kn, sc = q.to_kn()
                kind = "q8-moe" if moe else "q8"
                group = {dk: kn, dk + "#scale": sc}
                if moe:
                    group[dk + "#nk"] = q.wq
                si = put(group)
                meta = {"kind": kind, "k": q.k, "n": q.n, "shape": list(kn.shape), "scale_key": dk + "#scale", "shard": si}
                if moe:
                    meta["nk_key"] = dk + "#nk"
        else:
            kind = "dense"
            si = put({dk: t})
            meta = {"kind": "dense", "shape": list(t.shape), "shard": si}
        kinds[kind] = kinds.get(kind, 0) + 1
        tensors[dk] = meta
    flush()
    pat = "quant-w4a8-%05d-of-%05d.safetensors" if w4 else "quant-%05d-of-%05d.safetensors"
    files = []
    for i, path in enumerate(tmp_files):
        name = pat % (i + 1, len(tmp_files))
        path.replace(out / name)
        files.append(name)
    for meta in tensors.values():
        meta["shard"] = files[meta["shard"]]
    index = {"format": W4A8_FORMAT if w4 else FORMAT, "generated_by": generated_by or "coffin_b200/tools/quant_disk.py",
             "source": str(src), "source_config_sha256": config_digest(src), "weight_dtype": weight_dtype,
             "act_dtype": "bfloat16",
             "scheme": ("group-128 symmetric int4: s = max|w|/7, round, clamp [-8, 7], code = q + 8, low nibble = even k"
                        if w4 else "per-output-column symmetric absmax: s = max|w|/127, round, clamp [-127, 127]; s floored at 1e-8"),
             "layout": "uint8 [ceil(K/2), N] + fp32 [ceil(K/128), N]" if w4 else "int8 [K, N] contiguous + fp32 [N]",
             "prefixes": ["model.language_model.", "mtp.", "lm_head."], "vision": has_visual,
             "files": files, "kinds": dict(sorted(kinds.items())),
             "totals": {"tensors": len(tensors), "bytes": sum((out / f).stat().st_size for f in files)},
             "tensors": tensors}
    (out / INDEX_NAME).write_text(json.dumps(index, indent=1))
    return index


def load_quantized(model_dir: str | Path, device: str = "cpu", quant: bool = True,
                   dense_dtype: torch.dtype = torch.bfloat16, check_config: bool = True, plan_of=None,
                   wanted=None) -> dict:
    """State dict (canonical keys) of a pre-quantised directory: projections as ``QWeight`` /
    ``W4A8Weight`` (or dequantised when ``quant`` is false), the rest dense.  ``plan_of(key)`` (a
    ``parallel.tp.slice_plan``) makes every tensor the slice of one tensor-parallel rank: the on-disk
    ``[K, N]`` tensors are read with ``get_slice`` (output rows = file columns, input columns = file
    rows), so a rank reads only its bytes.  ``wanted(key)`` filters keys (pipeline stages)."""
    from safetensors import safe_open
    model_dir = Path(model_dir)
    index = read_index(model_dir)
    if check_config and (model_dir / "config.json").is_file():
        if config_digest(model_dir) != index.get("source_config_sha256"):
            raise ValueError(f"{model_dir}: config.json does not match the one the weights were quantised from")
    entries = index["tensors"]
    sd: dict = {}
    handles: dict[str, object] = {}

    def cut(h, name: str, plan, layout: str):
        """Slice tensor ``name`` of file handle ``h``.  ``layout``: "kn" = [K(/2 or /group), N] file
        tensor of a projection, "n" = a per-output vector (scales), "nk" = [.., N, K], "dense"."""
        if plan is None:
            return h.get_tensor(name)
        kind, ranges = plan
        sl = h.get_slice(name)
        nd = len(sl.get_shape())
        lead = (slice(None),) * (nd - 2) if layout in ("kn", "nk", "kn_grp", "kn_half") and nd > 2 else ()
        if layout == "dense":
            if kind == "rows":
                return torch.cat([sl[a:b] for a, b in ranges]) if len(ranges) > 1 else sl[ranges[0][0]:ranges[0][1]]
            (a, b), = ranges
            return sl[:, a:b].contiguous()
        if layout == "n":                                   # per-output-row vector
            if kind == "rows":
                return torch.cat([sl[lead + (slice(a, b),)] if lead else sl[a:b] for a, b in ranges])
            return h.get_tensor(name)
        if layout == "nk":
            if kind == "rows":
                return torch.cat([sl[lead + (slice(a, b), slice(None))] for a, b in ranges], -2).contiguous()
            (a, b), = ranges
            return sl[lead + (slice(None), slice(a, b))].contiguous()
        div = {"kn": 1, "kn_half": 2, "kn_grp": GROUP}[layout]
        if kind == "rows":                                  # output rows are the file's last axis
            return torch.cat([sl[lead + (slice(None), slice(a, b))] for a, b in ranges], -1).contiguous()
        (a, b), = ranges
        if a % div or b % div:
            raise ValueError(f"{name}: column cut [{a}, {b}) is not aligned to {div}")
        return sl[lead + (slice(a // div, b // div), slice(None))].contiguous()

    def get(shard: str, name: str, plan=None, layout: str = "dense") -> torch.Tensor:
        path = model_dir / shard
        if not path.is_file():
            raise FileNotFoundError(f"{model_dir}: index names {shard}, which is missing")
        h = handles.get(shard)
        if h is None:
            h = handles[shard] = safe_open(str(path), framework="pt", device=device)
        if name not in h.keys():
            raise ValueError(f"{path}: index names {name}, shard does not hold it")
        return cut(h, name, plan, layout)

    def span(plan, full: int, kind: str) -> int:
        """Extent left of a dimension of ``full`` elements after ``plan`` cut it along ``kind``."""
        if plan is None or plan[0] != kind:
            return full
        return sum(b - a for a, b in plan[1])

    for dk, meta in entries.items():
        key, kind, shard = _mem_key(dk), meta["kind"], meta["shard"]
        if wanted is not None and not wanted(key):
            continue
        plan = plan_of(key) if plan_of is not None else None
        if kind == "dense":
            sd[key] = get(shard, dk, plan, "dense")
        elif kind in ("q8", "q8-moe"):
            k_loc, n_loc = span(plan, meta["k"], "cols"), span(plan, meta["n"], "rows")
            sc = get(shard, meta["scale_key"], plan, "n")
            if meta.get("nk_key"):
                q = QWeight(get(shard, meta["nk_key"], plan, "nk"), sc)
            else:
                kn = get(shard, dk, plan, "kn")
                if kn.dtype != torch.int8 or list(kn.shape[-2:]) != [k_loc, n_loc]:
                    raise ValueError(f"{dk}: tensor does not match its index entry")
                q = QWeight.from_kn(kn, sc)
            if list(q.wq.shape[-2:]) != [n_loc, k_loc] or sc.shape[-1] != n_loc:
                raise ValueError(f"{dk}: tensor does not match its index entry")
            sd[key] = q if quant else q.dequant(dense_dtype)
        elif kind in ("q4", "q4-moe"):
            gs = meta.get("group_size", GROUP)
            if gs != GROUP and plan is not None:
                raise ValueError(f"{dk}: sliced reads need group size {GROUP}")
            pk = get(shard, dk, plan, "kn_half")
            sc = get(shard, meta["scale_key"], plan, "kn_grp")
            k_loc, n_loc = span(plan, meta["k"], "cols"), span(plan, meta["n"], "rows")
            rows_ok = {(k_loc + 1) // 2, (k_loc + gs - 1) // gs * gs // 2}   # unpadded, or padded to whole groups
            if plan is not None and plan[0] == "cols":
                rows_ok = {k_loc // 2}
            if pk.dtype != torch.uint8 or pk.shape[-1] != n_loc or pk.shape[-2] not in rows_ok:
                raise ValueError(f"{dk}: tensor does not match its index entry")
            q = W4A8Weight(pk, sc, k_loc, gs)
            sd[key] = q if quant else q.dequant(dense_dtype)
        else:
            raise ValueError(f"{dk}: unknown kind {kind!r}")
    if index.get("ep_shard"):          # a per-rank directory: the routed stacks already hold this rank's experts only
        sd["__ep_shard__"] = tuple(int(x) for x in index["ep_shard"])
    return sd


def summary(model_dir: str | Path) -> dict:
    idx = read_index(model_dir)
    return {"format": idx["format"], "kinds": idx["kinds"], "files": len(idx["files"]), "totals": idx["totals"]}
