"""Single-process front door: load a checkpoint (or draw a named shape), generate greedily, print.

    python -m coffin_b200.entrypoints.run_chat --model /ckpt/Qwen3.5-4B --chat "introduce yourself" -n 64
    python -m coffin_b200.entrypoints.run_chat --preset qwen35-4b --raw "The capital of France is" -n 32
    python -m coffin_b200.entrypoints.run_chat --preset qwen35-4b --bench -n 128

No server, no scheduler: one model, one request, the check to run after touching a kernel ("does it
still produce text, and how fast").  Decoding is greedy so runs are reproducible; ``--bench`` prints
device-timed prefill / decode figures; ``--no-graph`` decodes eagerly instead of replaying the CUDA
graph.  The serving path is ``entrypoints/cli/runtime.py``.  Reference: ``run_chat.py:71-113``.
"""
from __future__ import annotations

import argparse
import sys
import time


def build_prompt(tok, args) -> list[int]:
    if args.raw:
        return tok.encode(args.raw)
    msgs = ([{"role": "system", "content": args.system}] if args.system else []) + \
           [{"role": "user", "content": args.chat or "Hello"}]
    text = tok.apply_chat_template(msgs, tokenize=False, add_generation_prompt=True,
                                   enable_thinking=not args.no_thinking)
    return tok.encode(text)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="")
    ap.add_argument("--preset", default="")
    ap.add_argument("--raw", default="")
    ap.add_argument("--chat", default="")
    ap.add_argument("--system", default="")
    ap.add_argument("-n", type=int, default=64)
    ap.add_argument("--bench", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-thinking", action="store_true")
    ap.add_argument("--quant", default="none", choices=["none", "int8", "w4a8"])
    ap.add_argument("--max-seq", type=int, default=8192)
    args = ap.parse_args(argv)
    import torch
    from ..config import preset
    from ..engine.llm import LLM
    from ..utils.tokenizer import load_tokenizer
    t0 = time.time()
    if args.model:
        llm = LLM.from_pretrained(args.model, max_seq=args.max_seq, graph=not args.no_graph)
    else:
        llm = LLM.from_random(preset(args.preset or "tiny"), max_seq=args.max_seq, graph=not args.no_graph,
                              quant=args.quant)
    tok = load_tokenizer(args.model or None, llm.cfg.vocab_size)
    print(f"[load] {llm.cfg.name}: {time.time() - t0:.1f} s", file=sys.stderr)
    prompt = build_prompt(tok, args) if not args.bench or args.raw or args.chat else list(range(1, 513))
    eos = () if args.bench else tuple(i for i in tok.eos_ids if i < llm.cfg.vocab_size)
    host = torch.tensor(prompt, dtype=torch.int64).pin_memory()
    if args.bench:
        llm.generate(host, max_new_tokens=8, ignore_eos=True)            # warm-up and graph capture
    out = llm.generate(host, max_new_tokens=args.n, eos=eos, ignore_eos=args.bench)
    if not args.bench:
        print(tok.decode(out.tokens, skip_special_tokens=True))
    print(f"[run] prompt {out.n_prompt} tok in {out.prefill_ms:.1f} ms ({out.n_prompt / out.prefill_ms * 1e3:.0f} tok/s); "
          f"{len(out.tokens)} new tok in {out.decode_ms:.1f} ms ({out.decode_tok_s:.1f} tok/s); stop: {out.stopped}",
          file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
