"""Write a pre-quantised checkpoint directory of a Qwen4-exp model, streaming.

    python -m coffin_b200.tools.quant_disk_qwen4 --model SRC --out DST --scheme w4a8
    python -m coffin_b200.tools.quant_disk_qwen4 --preset tiny-qwen4 --out DST --scheme int8 --verify

The source is read tensor by tensor from its shards and the output is written shard by shard, so the
tool needs memory for one tensor and one output shard - not for the model (the routed expert stacks
and the n-gram table of the PLE layer are each tens of GiB in the real geometry).  Per-expert source
spellings (``experts.{e}.gate_proj.weight`` ...) are fused into one stack per layer before quantisation,
one layer at a time.  What is quantised: the mixer projections (with the fused indexer projection),
routed and shared experts and the lm_head; the router, gates, norms, conv taps, hyper-connection
matrices, PLE tensors and the embedding stay in their source dtype.  The output carries
``quant_index.json`` in the same two formats as the Qwen3.5 tool (``coffin-int8-kn-v1`` /
``coffin-w4a8-kn-v1``) and is read back by ``weights.loader.load_checkpoint``.

``--layout epN`` (repeatable) writes a tree of per-rank directories instead, ``OUT/epN/rank-r/``: each holds
the replicated tensors and ONLY rank r's contiguous range of every routed expert stack, is loadable on its
own (its index carries ``ep_shard: [r, N]``, so the expert-parallel model does not cut again) and a rank
reads nothing it does not keep.  The top level gets a manifest (``quant_index.json`` with format
``coffin-qwen4-w4a8-manifest-v1``: layouts, rank directories, totals, whether the tree is complete) and
``quant_progress.json``, updated after every finished rank directory, from which an interrupted run resumes
(``--no-resume`` starts over).  Reference: ``tools/quant_disk_qwen4.py`` (streaming per-layer quantiser for
this family, per-rank ``ep4`` trees, manifest l.80, resumable progress l.1042-1160).
"""
from __future__ import annotations

import argparse
import json
import re
import sys
import time
from pathlib import Path


def stream_tensors(model_dir: Path, index: dict[str, str]):
    """Yield ``(key, tensor)`` shard by shard; per-expert tensors of a layer are collected and yielded as
    the two fused stacks as soon as the layer is complete."""
    import torch
    from safetensors import safe_open
    pat = re.compile(r"^(.*\.mlp\.experts\.)(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")
    n_exp: dict[str, int] = {}
    for k in index:
        m = pat.match(k)
        if m:
            n_exp[m.group(1)] = max(n_exp.get(m.group(1), 0), int(m.group(2)) + 1)
    pending: dict[str, dict] = {}
    by_file: dict[str, list[str]] = {}
    for k, f in index.items():
        by_file.setdefault(f, []).append(k)
    for fname in sorted(by_file):
        with safe_open(str(model_dir / fname), framework="pt") as fh:
            for k in sorted(by_file[fname]):
                m = pat.match(k)
                if not m:
                    yield k, fh.get_tensor(k)
                    continue
                base = m.group(1)
                slot = pending.setdefault(base, {"gate_proj": {}, "up_proj": {}, "down_proj": {}})
                slot[m.group(3)][int(m.group(2))] = fh.get_tensor(k)
                n = n_exp[base]
                if all(len(slot[x]) == n for x in slot):
                    yield base + "gate_up_proj", torch.stack([torch.cat([slot["gate_proj"][e], slot["up_proj"][e]]) for e in range(n)])
                    yield base + "down_proj", torch.stack([slot["down_proj"][e] for e in range(n)])
                    del pending[base]
    if pending:
        raise ValueError(f"incomplete expert sets: {sorted(pending)[:3]}")


_STACK = re.compile(r"\.mlp\.experts\.(gate_up_proj|down_proj)$")
PROGRESS_NAME = "quant_progress.json"


def expert_slice(stream, rank: int, world: int):
    """The tensor stream of one expert-parallel rank: routed stacks ``[E, ...]`` cut to the rank's range."""
    for k, t in stream:
        if _STACK.search(k) and t.dim() == 3:
            E = t.shape[0]
            if E % world:
                raise ValueError(f"{k}: {E} experts do not divide over {world} ranks")
            per = E // world
            yield k, t[rank * per:(rank + 1) * per].contiguous()
        else:
            yield k, t


def _write_json_atomic(path: Path, obj: dict) -> None:
    tmp = path.with_suffix(path.suffix + ".tmp")
    tmp.write_text(json.dumps(obj, indent=1))
    tmp.replace(path)                        # a run killed in the middle of a write leaves the previous file


def write_rank_trees(src: Path, index: dict, out: Path, layouts: list[str], scheme: str, shard_bytes: int, pick,
                     resume: bool = True) -> dict:
    """Per-rank directories for every layout in ``layouts`` (``epN``), the manifest and the progress file."""
    from ..weights.quant_io import INDEX_NAME, MANIFEST_FORMAT, config_digest, read_index, write_quantized
    out.mkdir(parents=True, exist_ok=True)
    for lay in layouts:
        if not re.fullmatch(r"ep[1-9]\d*", lay):
            raise ValueError(f"layout {lay!r}: only expert-parallel trees (epN) are written; this family runs expert "
                             "parallel, and a tensor-parallel load slices a plain quantised directory at read time")
    digest = config_digest(src)
    prog_path = out / PROGRESS_NAME
    done: dict[str, dict] = {}
    if resume and prog_path.is_file():
        old = json.loads(prog_path.read_text())
        if old.get("source_config_sha256") == digest and old.get("scheme") == scheme:
            done = {k: v for k, v in old.get("done", {}).items() if (out / v["dir"] / INDEX_NAME).is_file()}
    resumed = sorted(done)
    reports: dict[str, dict] = {}
    for lay in layouts:
        world = int(lay[2:])
        for r in range(world):
            unit, rel = f"{lay}/rank-{r}", f"{lay}/rank-{r}"
            if unit not in done:
                d = out / rel
                write_quantized(src, expert_slice(stream_tensors(src, index), r, world), d, scheme=scheme, is_q=pick,
                                shard_bytes=shard_bytes, generated_by="coffin_b200/tools/quant_disk_qwen4.py")
                idx = json.loads((d / INDEX_NAME).read_text())
                idx["ep_shard"] = [r, world]
                _write_json_atomic(d / INDEX_NAME, idx)
                done[unit] = {"dir": rel, "tensors": idx["totals"]["tensors"], "bytes": idx["totals"]["bytes"]}
                _write_json_atomic(prog_path, {"source": str(src), "source_config_sha256": digest, "scheme": scheme,
                                               "layouts": layouts, "done": done})
            reports.setdefault(lay, {})[str(r)] = done[unit]
    first = read_index(out / reports[layouts[0]]["0"]["dir"])
    manifest = {"format": MANIFEST_FORMAT, "generated_by": "coffin_b200/tools/quant_disk_qwen4.py", "source": str(src),
                "source_config_sha256": digest, "rank_format": first["format"], "scheme": first["scheme"], "layout": first["layout"],
                "world": {lay: int(lay[2:]) for lay in layouts}, "complete": True,
                "rank_dirs": {lay: {r: info["dir"] for r, info in per.items()} for lay, per in reports.items()},
                "layouts": reports, "kinds": first["kinds"], "resumed_units": resumed,
                "rank_index_hint": "quant_index.json of a loadable directory exists only under the rank directories; this file is the manifest"}
    _write_json_atomic(out / INDEX_NAME, manifest)
    return manifest


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", help="source checkpoint directory (HF safetensors)")
    ap.add_argument("--preset", help="draw a random-init source of this named geometry instead (e.g. tiny-qwen4)")
    ap.add_argument("--out", required=True)
    ap.add_argument("--scheme", choices=("int8", "w4a8"), default="w4a8")
    ap.add_argument("--shard-gb", type=float, default=4.0)
    ap.add_argument("--quant-embed", action="store_true",
                    help="int8 scheme only: store the embedding table as int8 rows + per-row scales (QuantizedEmbedding)")
    ap.add_argument("--verify", action="store_true", help="reload the output and report the worst dequantisation error")
    ap.add_argument("--layout", action="append", default=[], help="write per-rank trees instead of one directory: epN (repeatable)")
    ap.add_argument("--no-resume", action="store_true", help="ignore quant_progress.json of an earlier run")
    args = ap.parse_args(argv)
    if args.quant_embed and args.scheme != "int8":
        ap.error("--quant-embed needs --scheme int8 (one format per directory)")
    import torch
    from ..config import load_config, preset
    from ..models.qwen4exp.weights import checkpoint_index, random_state_dict, verify_plan
    from ..weights.init import save_checkpoint
    from ..weights.quant import QWeight, W4A8Weight, is_quantizable_qwen4
    from ..weights.quant_io import load_quantized, summary, write_quantized
    t0 = time.time()
    if args.model:
        src = Path(args.model)
    elif args.preset:
        import tempfile
        cfg = preset(args.preset)
        src = Path(tempfile.mkdtemp(prefix="coffin_q4src_"))
        save_checkpoint(cfg, random_state_dict(cfg, 0, dtype=torch.bfloat16), src)
    else:
        ap.error("give --model or --preset")
    cfg = load_config(src)
    index = checkpoint_index(src)
    rep = verify_plan(cfg, src, index)
    if rep["missing"] or rep["shape"]:
        print(json.dumps({"ok": False, "plan": {k: v[:8] for k, v in rep.items()}}, indent=1, default=str))
        return 2
    pick = is_quantizable_qwen4
    if args.quant_embed:
        pick = lambda k, t: is_quantizable_qwen4(k, t) or k.endswith("embed_tokens.weight")
    if args.layout:
        man = write_rank_trees(src, index, Path(args.out), args.layout, args.scheme, int(args.shard_gb * (1 << 30)), pick,
                               resume=not args.no_resume)
        rep_out = {"format": man["format"], "rank_dirs": man["rank_dirs"], "resumed_units": man["resumed_units"],
                   "bytes": {lay: sum(v["bytes"] for v in per.values()) for lay, per in man["layouts"].items()},
                   "seconds": round(time.time() - t0, 1)}
        if args.verify:
            from ..weights.loader import load_checkpoint
            dense = load_checkpoint(src)
            worst = 0.0
            for lay, per in man["rank_dirs"].items():
                world = int(lay[2:])
                for r, rel in per.items():
                    back = load_quantized(Path(args.out) / rel)
                    assert back.get("__ep_shard__") == (int(r), world)
                    for k, v in back.items():
                        if isinstance(v, (QWeight, W4A8Weight)):
                            ref = dense[k].float()
                            if _STACK.search(k):
                                per_e = ref.shape[0] // world
                                ref = ref[int(r) * per_e:(int(r) + 1) * per_e]
                            worst = max(worst, ((v.dequant() - ref).abs().max() / ref.abs().max().clamp_min(1e-9)).item())
            rep_out["worst_relative_error"] = round(worst, 4)
        json.dump(rep_out, sys.stdout, indent=1)
        print()
        return 0
    write_quantized(src, stream_tensors(src, index), args.out, scheme=args.scheme, is_q=pick,
                    shard_bytes=int(args.shard_gb * (1 << 30)), generated_by="coffin_b200/tools/quant_disk_qwen4.py")
    out = summary(args.out)
    out["seconds"] = round(time.time() - t0, 1)
    out["unexpected_source_tensors"] = rep["unexpected"][:8]
    if args.verify:
        from ..weights.loader import load_checkpoint
        dense = load_checkpoint(src)
        back = load_quantized(args.out)
        worst = 0.0
        for k, v in back.items():
            if isinstance(v, (QWeight, W4A8Weight)):
                ref = dense[k].float()
                worst = max(worst, ((v.dequant() - ref).abs().max() / ref.abs().max().clamp_min(1e-9)).item())
        out["worst_relative_error"] = round(worst, 4)
    json.dump(out, sys.stdout, indent=1)
    print()
    return 0


if __name__ == "__main__":
    sys.exit(main())
