"""HTTP adapter CLI: ``python -m coffin_b200.entrypoints.openai.server --sock ... --port 18080``.

Several ``--sock`` values (or a comma list) put a least-loaded router over engine replicas.
Reference: ``entrypoints/cli/openai.py:34-113``.
"""
from __future__ import annotations

import argparse
import os
import sys
import time


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="coffin-b200-openai")
    ap.add_argument("--sock", action="append", default=None, help="engine socket (repeat for replicas)")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=18080)
    ap.add_argument("--served-model-name", default=None)
    ap.add_argument("--model", default=None, help="alias of --served-model-name")
    ap.add_argument("--default-max-tokens", type=int, default=8192)
    ap.add_argument("--enable-thinking", action=argparse.BooleanOptionalAction, default=True)
    ap.add_argument("--max-decode-seconds", type=float, default=180.0)
    ap.add_argument("--timeout", type=float, default=900.0)
    ap.add_argument("--max-images", type=int, default=int(os.environ.get("ENGINE_MAX_IMAGES", "4")))
    ap.add_argument("--max-image-bytes", type=int, default=int(os.environ.get("ENGINE_MAX_IMAGE_BYTES", str(10 << 20))))
    ap.add_argument("--max-image-total-bytes", type=int,
                    default=int(os.environ.get("ENGINE_MAX_IMAGE_TOTAL_BYTES", str(32 << 20))))
    return ap


def main(argv=None) -> int:
    from ..openai.app import ReplicaRouter, configure, make_server
    from ..openai.client import EngineClient
    args = parser().parse_args(argv)
    socks: list[str] = []
    for s in args.sock or [os.environ.get("ENGINE_SOCK", "/tmp/coffin_b200.sock")]:
        socks.extend(x for x in s.split(",") if x)
    clients = [EngineClient(s, args.timeout) for s in socks]
    name = args.served_model_name or args.model
    vision = True
    for c in clients:
        for attempt in range(3):
            try:
                p = c.ping()
                name = name or p.get("model")
                vision = vision and bool(p.get("vision", True))      # one replica without a tower closes the image path
                break
            except OSError as exc:
                if attempt == 2:
                    print(f"[http] engine {c.sock_path} not reachable: {exc}", file=sys.stderr)
                    return 2
                time.sleep(1.0)
    configure(ReplicaRouter(clients), served_model_name=name or "coffin-b200",
              default_max_tokens=args.default_max_tokens, enable_thinking=args.enable_thinking,
              max_decode_seconds=args.max_decode_seconds, max_images=args.max_images,
              max_image_bytes=args.max_image_bytes, max_image_total_bytes=args.max_image_total_bytes, vision=vision)
    srv = make_server(args.host, args.port)
    print(f"[http] serving {name} on http://{args.host}:{args.port} -> {', '.join(socks)}", flush=True)
    try:
        srv.serve_forever()
    except KeyboardInterrupt:
        pass
    return 0


if __name__ == "__main__":
    sys.exit(main())
