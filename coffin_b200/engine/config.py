"""``EngineConfig``: the single source of truth for engine behaviour.

CLI flags and server arguments are folded into this dataclass and everything below reads
it (the reference's three-tier scheme: argparse -> ``EngineConfig`` -> environment switches,
``engine/config.py:22-120``).  Defaults follow the reference where they are hardware
neutral; ``max_num_seqs`` defaults to 8 (one full decode bucket) because a B200 has room.
"""
from __future__ import annotations

import dataclasses
import os


@dataclasses.dataclass
class EngineConfig:
    max_seq: int = 262144              # context window (tokens) per sequence
    quant: str = "none"                # none | int8 | w4a8 : weight storage of the text model
    kv_dtype: str = "bf16"
    prefix_cache: bool = True
    block_size: int = 64
    num_blocks: int = -1               # -1: size the pool from max_seq * max_num_seqs
    snapshots: int = 8                 # delta-net state snapshots kept in the radix tree
    snapshot_interval: int = 2048      # tokens between snapshots during a long prefill
    spec_k: int = 0                    # default speculative draft length of greedy requests (0 = off; a request's own spec_k overrides)
    spec_batch: bool = False           # speculate also when several rows decode together (one verify pass over all rows)
    spec_min_ctx: int = 0              # rows shorter than this many tokens do not draft yet
    spec_sparse_k: int = 0             # approximate batched verify over the k best history blocks per row: accepted
                                       # as an option for parity with the reference, where it is also refused when
                                       # > 0 (no masked multi-query verify kernel, models/qwen35/model.py:1390-1401)
    group_prefill: bool = True         # chunks of several sequences share one forward (stacked rows)
    chunk: int = 2048                  # largest prefill chunk handed to the model
    prefill_quantum: int = 2048        # tokens of one sequence prefilled per engine step
    max_num_seqs: int = 8              # concurrent sequences (= state slots = decode rows)
    max_num_batched_tokens: int = 2048
    max_seconds: float = 0.0           # default per-request deadline (0 = none)
    graph: bool = True
    vision: bool = True
    image_max_pixels: int = 1024 * 1024
    image_min_pixels: int = 32 * 32
    max_images: int = 4
    max_image_bytes: int = 8 << 20     # decoded bytes allowed per image on the engine side
    batch_window_ms: float = 0.0       # hold a lone decode this long for companions
    warmup: bool = True                # serving: run a prefill chunk and capture every decode bucket before the first request

    @classmethod
    def from_env(cls, **overrides) -> "EngineConfig":
        """Apply ``COFFIN_*`` environment switches, then explicit overrides."""
        cfg = cls()
        env = os.environ
        if "COFFIN_BATCH_WINDOW" in env:
            cfg.batch_window_ms = float(env["COFFIN_BATCH_WINDOW"])
        if "COFFIN_MAX_SEQ" in env:
            cfg.max_seq = int(env["COFFIN_MAX_SEQ"])
        if env.get("COFFIN_NO_GRAPH") == "1":
            cfg.graph = False
        if env.get("COFFIN_NO_WARMUP") == "1":
            cfg.warmup = False
        for k, v in overrides.items():
            if v is not None:
                if not hasattr(cfg, k):
                    raise TypeError(f"unknown engine option {k!r}")
                setattr(cfg, k, v)
        return cfg

    def pool_blocks(self) -> int:
        if self.num_blocks > 0:
            return self.num_blocks
        per_seq = (self.max_seq + self.block_size - 1) // self.block_size
        return per_seq * self.max_num_seqs + 1
