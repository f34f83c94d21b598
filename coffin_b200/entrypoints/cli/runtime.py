"""Engine CLI: ``--serve`` starts the resident process; the other commands are socket clients.

    python -m coffin_b200.entrypoints.cli.runtime --serve --model /path/to/ckpt
    python -m coffin_b200.entrypoints.cli.runtime --serve --preset qwen35-4b        # random weights
    python -m coffin_b200.entrypoints.cli.runtime chat "hello"

Commands: ``ping reload reset stop generate chat bench profile ops spec`` (reference:
``entrypoints/cli/runtime.py:30-208``).  Multi-GPU: launch one process per GPU with
``RANK/WORLD_SIZE/MASTER_ADDR/MASTER_PORT`` set and ``COFFIN_PARALLEL=tp|pp|ep``; rank 0 owns the
socket.
"""
from __future__ import annotations

import argparse
import faulthandler
import json
import os
import sys

COMMANDS = ("ping", "reload", "reset", "stop", "generate", "chat", "bench", "profile", "ops", "spec", "tokenize")


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="coffin-b200", description=__doc__.split("\n")[0])
    ap.add_argument("--serve", action="store_true", help="run the engine process")
    ap.add_argument("cmd", nargs="?", choices=COMMANDS, default="ping")
    ap.add_argument("text", nargs="?", default="", help="prompt for generate/chat/bench/profile/ops/spec")
    ap.add_argument("--sock", default=os.environ.get("ENGINE_SOCK", "/tmp/coffin_b200.sock"))
    ap.add_argument("--model", default=os.environ.get("ENGINE_MODEL", ""), help="checkpoint directory")
    ap.add_argument("--preset", default="", help="serve a random-init model of a named shape")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--backend", default="", help="accepted for command-line compatibility: this engine has one backend "
                                                  "(sm_100a; `--device cpu` selects the fp32 oracle twin)")
    ap.add_argument("--max-seq", type=int, default=None)
    ap.add_argument("--quant", default=None, choices=["none", "int8", "w4a8"])
    ap.add_argument("--fp16", action="store_true", help="keep 16-bit weights (the default here; same as --quant none)")
    ap.add_argument("--block-size", type=int, default=64, help="KV block size in tokens (the kernels are built for 64)")
    ap.add_argument("--kv-dtype", default=None, choices=["bf16", "int8"], help="KV pool storage (int8: per-(token, head) scales)")
    ap.add_argument("--no-prefix-cache", action="store_true")
    ap.add_argument("--num-blocks", type=int, default=None)
    ap.add_argument("--snapshots", type=int, default=None)
    ap.add_argument("--snapshot-interval", type=int, default=None)
    ap.add_argument("--spec-k", type=int, default=None)
    ap.add_argument("--spec-batch", action="store_true")
    ap.add_argument("--spec-min-ctx", type=int, default=None,
                    help="rows with fewer cached tokens than this do not draft yet (0 = always)")
    ap.add_argument("--spec-sparse-k", type=int, default=0, help="approximate batched verify over the k best history blocks (refused when > 0: not built)")
    ap.add_argument("--chunk", type=int, default=None)
    ap.add_argument("--prefill-quantum", type=int, default=None)
    ap.add_argument("--max-num-seqs", type=int, default=None)
    ap.add_argument("--max-num-batched-tokens", type=int, default=None)
    ap.add_argument("--max-seconds", type=float, default=None)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-vision", action="store_true")
    ap.add_argument("--vision-int8", action="store_true",
                    help="accepted for compatibility: the tower stays bf16 here (0.6 GiB of 180)")
    ap.add_argument("--image-max-pixels", type=int, default=None, help="largest image served, in pixels (bigger ones are downsampled)")
    ap.add_argument("--image-min-pixels", type=int, default=None, help="smallest image after the upscale, in pixels")
    ap.add_argument("--max-images", type=int, default=None, help="images accepted in one request")
    ap.add_argument("--max-image-bytes", type=int, default=None, help="decoded bytes allowed per image")
    ap.add_argument("--no-bench", action="store_true", help="accepted for compatibility: the engine runs no benchmark at start")
    ap.add_argument("--vision", choices=("tiny", "default"), default=None,
                    help="attach a vision tower with random weights of this geometry (checkpoints with model.visual.* tensors get theirs)")
    ap.add_argument("-n", "--max-new", dest="n", type=int, default=64, help="tokens for generate/chat/bench")
    ap.add_argument("--prompt", default="", help="prompt for generate (same as the positional text)")
    ap.add_argument("--user", default="", help="user message for chat (same as the positional text)")
    ap.add_argument("--think", action="store_true", help="enable thinking mode (the default; --no-thinking turns it off)")
    ap.add_argument("--print-ids", action="store_true", help="print the generated token ids (accept rates are compared by id)")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--system", default="")
    ap.add_argument("--tools", default="", help="JSON file with an OpenAI tools array, or `demo` for the built-in demo tools")
    ap.add_argument("--no-thinking", action="store_true")
    return ap


def engine_config(args):
    from ...engine.config import EngineConfig
    if args.block_size != 64:
        raise SystemExit(f"--block-size {args.block_size}: the attention and cache kernels are built for blocks of 64 tokens")
    if args.backend and args.backend not in ("auto", "sm_100a", "cuda", "b200"):
        raise SystemExit(f"--backend {args.backend!r}: this engine has one backend (sm_100a); use --device cpu for the oracle twin")
    if args.fp16 and args.quant not in (None, "none"):
        raise SystemExit("--fp16 contradicts --quant " + args.quant)
    if args.vision_int8:
        print("[serve] --vision-int8 ignored: the vision tower stays bf16", flush=True)
    return EngineConfig.from_env(
        max_seq=args.max_seq, quant=args.quant, kv_dtype=args.kv_dtype, prefix_cache=False if args.no_prefix_cache else None,
        num_blocks=args.num_blocks, snapshots=args.snapshots, snapshot_interval=args.snapshot_interval,
        spec_k=args.spec_k, spec_batch=True if args.spec_batch else None, spec_sparse_k=args.spec_sparse_k or None,
        spec_min_ctx=args.spec_min_ctx, image_max_pixels=args.image_max_pixels, image_min_pixels=args.image_min_pixels,
        max_images=args.max_images, max_image_bytes=args.max_image_bytes, chunk=args.chunk,
        prefill_quantum=args.prefill_quantum, max_num_seqs=args.max_num_seqs,
        max_num_batched_tokens=args.max_num_batched_tokens, max_seconds=args.max_seconds,
        graph=False if args.no_graph else None, vision=False if args.no_vision else None)


def build_server(args):
    """Load (or draw) the weights once and return a ``Server`` whose ``reload`` rebuilds the model
    from the resident state dict."""
    import torch
    from ...config import load_config, preset
    from ...serving.runtime import Server
    cfg_e = engine_config(args)
    if cfg_e.max_seq > 32768 and args.max_seq is None:
        cfg_e.max_seq = 32768
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    mode = os.environ.get("COFFIN_PARALLEL", "tp")
    if args.model:
        from ...weights.loader import load_checkpoint
        mcfg = load_config(args.model)
        # a rank of a multi-rank engine reads only what it computes with: its tensor-parallel slices
        # (get_slice reads) or the layers of its pipeline stage
        if world > 1 and mode == "tp":
            sd = load_checkpoint(args.model, tp=(rank, world))
        elif world > 1 and mode == "pp":
            from ...parallel.pp import layer_range
            sd = load_checkpoint(args.model, layers=layer_range(mcfg.num_hidden_layers, rank, world))
        else:
            sd = load_checkpoint(args.model)
    else:
        from ...weights.init import random_state_dict
        mcfg = preset(args.preset or "tiny")
        dev = args.device if args.device == "cpu" else f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}"
        sd = random_state_dict(mcfg, 0, dtype=torch.float32 if args.device == "cpu" else torch.bfloat16, device=dev)

    def builder():
        if args.device == "cpu":
            from ...oracle.engine_model import OracleEngineModel
            twin = OracleEngineModel(mcfg, sd, max_seq=min(cfg_e.max_seq, 4096), num_slots=cfg_e.max_num_seqs,
                                     max_chunk=cfg_e.chunk)
            if not args.no_vision and (args.vision or any(k.startswith("model.visual.") for k in sd)):
                from ...models import attach_vision
                attach_vision(twin, mcfg, {k: v for k, v in sd.items() if k.startswith("model.visual.")},
                              args.vision, args.model or None)
            return twin
        from ...models import build_model
        kw = dict(vision=False if args.no_vision else args.vision, model_dir=args.model or None,
                  device=f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}", max_seq=cfg_e.max_seq,
                  num_slots=cfg_e.max_num_seqs, max_chunk=cfg_e.chunk,
                  num_blocks=cfg_e.num_blocks if cfg_e.num_blocks > 0 else None)
        if getattr(cfg_e, "kv_dtype", "bf16") != "bf16":
            kw["kv_dtype"] = cfg_e.kv_dtype
        if getattr(cfg_e, "quant", None) not in (None, "", "none"):
            kw["quant"] = cfg_e.quant
        if world > 1:
            if mode not in ("tp", "pp", "ep"):
                raise SystemExit(f"COFFIN_PARALLEL={mode!r}: expected tp, pp or ep")
            kw.update({f"{mode}_world": world, f"{mode}_rank": rank})
        return build_model(mcfg, sd, **kw)

    return Server(builder(), cfg_e, model_path=args.model, model_name=args.preset or "", builder=builder)


def _leave_group(srv) -> None:
    """End of a rank of a multi-rank engine: release the peer mappings, then a bounded teardown."""
    from ...parallel.control import shutdown
    comm = getattr(srv.model, "tp", None)
    graphs = getattr(srv.model, "_graphs", None)
    if graphs is not None:
        graphs.clear()
    if comm is not None:
        comm.close()
    shutdown(timeout_s=10.0)


def main(argv=None) -> int:
    args = parser().parse_args(argv)
    dump = float(os.environ.get("COFFIN_FAULT_DUMP", "0") or 0)
    if dump > 0:
        faulthandler.dump_traceback_later(dump, repeat=True)
    if args.serve:
        from ...serving.transport import serve
        world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
        fanout = None
        if world > 1:
            from ...parallel.control import init_control_plane, make_fanout, worker_loop
            init_control_plane()
            srv = build_server(args)
            if rank != 0:
                worker_loop(srv)
                _leave_group(srv)
                return 0
            fanout = make_fanout()
        else:
            srv = build_server(args)
        serve(srv, args.sock, fanout=fanout)
        if world > 1:
            _leave_group(srv)
        return 0
    from ...serving.transport import call
    req: dict = {"op": args.cmd}
    if args.cmd in ("generate", "bench", "profile", "ops", "spec", "tokenize"):
        req.update({"prompt": args.text or args.prompt or "Hello", "n": args.n, "max_new": args.n, "temperature": args.temperature})
        if args.spec_k:
            req["spec_k"] = args.spec_k
    elif args.cmd == "chat":
        msgs = ([{"role": "system", "content": args.system}] if args.system else []) + \
               [{"role": "user", "content": args.text or args.user or "Hello"}]
        req.update({"messages": msgs, "max_new": args.n, "temperature": args.temperature,
                    "enable_thinking": not args.no_thinking})
        if args.tools == "demo":            # the two demo tools of the agent loop (get_weather, multiply)
            from ..agent import DEMO_TOOLS
            req["tools"] = DEMO_TOOLS
        elif args.tools:
            req["tools"] = json.load(open(args.tools))
    try:
        rep = call(args.sock, req)
    except OSError as exc:
        print(f"engine not reachable on {args.sock}: {exc}", file=sys.stderr)
        return 2
    if args.cmd in ("generate", "chat") and rep.get("ok"):
        if rep.get("thinking"):
            print(f"[thinking] {rep['thinking']}")
        print(rep.get("text", ""))
        if args.print_ids:
            print(f"[ids] {rep.get('tokens')}")
        for c in rep.get("tool_calls") or []:
            print(f"[tool_call] {json.dumps(c, ensure_ascii=False)}")
        print(f"[{rep.get('n_prompt')} prompt, {rep.get('n_new')} new, cached {rep.get('cached_tokens')}, "
              f"prefill {rep.get('prefill_ms')} ms, {rep.get('decode_tok_s')} tok/s]")
    else:
        print(json.dumps(rep, indent=1, ensure_ascii=False))
    return 0 if rep.get("ok", True) else 1


if __name__ == "__main__":
    sys.exit(main())
