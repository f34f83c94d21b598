"""``LLM``: the in-process front door (load a model, generate from token ids).

This is the single-process counterpart of the reference's ``run_chat.py:71-113`` /
``PrefixCacheEngine.generate`` (``engine/prefix_engine.py:480-506``): one call prefills a prompt
and decodes greedily or with a temperature, returning the tokens and per-phase timings.  It is
what the benchmark's end-to-end figure drives; the continuous-batching ``LLMEngine`` and the
socket server sit on the same model object.
"""
from __future__ import annotations

import dataclasses
import time
from pathlib import Path
from typing import Iterable, Sequence

import torch

from ..config import ModelConfig, load_config
from ..ops import kernels as K


@dataclasses.dataclass
class GenerationOutput:
    tokens: list[int]
    n_prompt: int
    prefill_ms: float
    decode_ms: float
    cached_tokens: int = 0
    stopped: str = "length"

    @property
    def decode_tok_s(self) -> float:
        return len(self.tokens) / (self.decode_ms / 1e3) if self.decode_ms > 0 else 0.0


class LLM:
    def __init__(self, model, graph: bool = True) -> None:
        self.model = model
        self.cfg: ModelConfig = model.cfg
        self.graph = graph
        self.graph_launches_replayed = 0
        self._graph_launches: dict[int, int] = {}
        self._graph_seen: set = set()
        self._slot = 0
        nblk = model.max_blocks_per_seq
        self._bt_list = list(range(nblk))
        self._bt = torch.arange(nblk, dtype=torch.int32, device=model.device)
        self._tok_host = torch.zeros(1, dtype=torch.int64).pin_memory()

    # ------------------------------------------------------------------ constructors
    @classmethod
    def from_random(cls, cfg: ModelConfig, seed: int = 0, max_seq: int = 4096, max_num_seqs: int = 1,
                    tp_world: int = 1, tp_rank: int = 0, graph: bool = True, pdl: bool = True,
                    max_chunk: int = 2048, device: str = "cuda", quant: str = "none",
                    ep_world: int = 1, ep_rank: int = 0, kv_dtype: str = "bf16") -> "LLM":
        """Random-init weights ~N(0, 0.02) of the given geometry, drawn on the device.  ``tp_world`` > 1
        shards every layer (tensor parallel); ``ep_world`` > 1 splits the routed experts by range instead
        (expert parallel, the dense part replicated)."""
        from ..models import build_model
        from ..weights.init import random_state_dict
        sd = random_state_dict(cfg, seed, dtype=torch.bfloat16, device=device)
        model = build_model(cfg, sd, device=device, max_seq=max_seq, num_slots=max_num_seqs,
                            max_chunk=max_chunk, pdl=pdl, tp_world=tp_world, tp_rank=tp_rank, free_source=True, quant=quant,
                            **({"ep_world": ep_world, "ep_rank": ep_rank} if ep_world > 1 else {}),
                            **({"kv_dtype": kv_dtype} if kv_dtype != "bf16" else {}))
        del sd
        torch.cuda.empty_cache()
        return cls(model, graph=graph)

    @classmethod
    def from_pretrained(cls, model_dir: str | Path, max_seq: int = 4096, max_num_seqs: int = 1,
                        graph: bool = True, device: str = "cuda", **kw) -> "LLM":
        from ..models import build_model
        from ..weights.loader import load_checkpoint
        cfg = load_config(model_dir)
        sd = load_checkpoint(model_dir)
        model = build_model(cfg, sd, device=device, max_seq=max_seq, num_slots=max_num_seqs, **kw)
        return cls(model, graph=graph)

    # ------------------------------------------------------------------ device-only path
    @torch.no_grad()
    def device_prefill(self, dev_prompt: torch.Tensor) -> torch.Tensor:
        """Prefill a prompt already on the device; returns the first sampled token (device)."""
        m = self.model
        m.zero_state(self._slot)
        T = dev_prompt.numel()
        logits = None
        for s in range(0, T, m.max_chunk):
            e = min(T, s + m.max_chunk)
            logits = m.prefill(dev_prompt[s:e], s, self._slot, self._bt, want_logits=e == T)
        self._n_ctx = T
        return K.argmax(logits.unsqueeze(0))

    @torch.no_grad()
    def device_decode(self, first: torch.Tensor, n: int) -> torch.Tensor:
        """``n`` greedy steps without a host round trip per token; returns the tokens (device)."""
        m = self.model
        b = m._row_buffers(1)
        b["tokens"].copy_(first)
        b["positions"].fill_(self._n_ctx)
        b["rope_pos"].fill_(self._n_ctx)
        b["slots"].fill_(self._slot)
        b["block_table"][0].copy_(self._bt)
        out = torch.empty(n, dtype=torch.int64, device=m.device)
        fused = hasattr(m, "_gkey")          # the step itself feeds the token back and advances the position
        if hasattr(m, "full_logits"):
            m.full_logits = False            # greedy: the arg-max is all a tensor-parallel step has to agree on
        if self.graph:
            self._ensure_graph(1, advance=fused)
        for i in range(n):
            if fused:
                nxt, _ = m.decode(1, graph=self.graph, advance=True)
                out[i:i + 1].copy_(nxt)
            else:
                nxt, _ = m.decode(1, graph=self.graph)
                out[i:i + 1].copy_(nxt)
                m.advance_rows(1)
            if self.graph:
                self.graph_launches_replayed += self._graph_launches[1]
        self._n_ctx += n
        return out

    def _ensure_graph(self, M: int, advance: bool = False) -> None:
        if (M, advance) not in self._graph_seen:
            self._graph_seen.add((M, advance))
            before = K.LAUNCHES
            if advance:
                self.model.capture(M, advance=True)
            else:
                self.model.capture(M)
            # capture() ran the body (warm-up + capture); one body's worth of launches per replay
            self._graph_launches[M] = self.model.launches_per_step(M)
            K.LAUNCHES = before

    # ------------------------------------------------------------------ public API
    @torch.no_grad()
    def generate(self, prompt: Sequence[int] | torch.Tensor, max_new_tokens: int = 32, temperature: float = 0.0,
                 eos: Iterable[int] = (), ignore_eos: bool = False, seed: int | None = None) -> GenerationOutput:
        """Prefill ``prompt`` (token ids; a pinned CPU tensor is copied asynchronously), then
        decode up to ``max_new_tokens``; each token is read back to the host as it is produced."""
        m = self.model
        host = prompt if isinstance(prompt, torch.Tensor) else torch.tensor(list(prompt), dtype=torch.int64)
        eos_set = set() if ignore_eos else set(eos)
        rng = torch.Generator().manual_seed(seed if seed is not None else 0)
        if hasattr(m, "full_logits"):
            m.full_logits = temperature > 0
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        dev = host.to(m.device, non_blocking=True)
        m.zero_state(self._slot)
        T = dev.numel()
        logits = None
        for s in range(0, T, m.max_chunk):
            e = min(T, s + m.max_chunk)
            logits = m.prefill(dev[s:e], s, self._slot, self._bt, want_logits=e == T)
        tok = self._pick(logits.unsqueeze(0), temperature, rng)
        t1 = time.perf_counter()
        out: list[int] = []
        pos = T
        stopped = "length"
        if self.graph:
            self._ensure_graph(1)
        while len(out) < max_new_tokens:
            if tok in eos_set:
                stopped = "eos"
                break
            out.append(tok)
            if len(out) == max_new_tokens or pos >= m.max_seq - 1:
                break
            m.set_rows(1, [tok], [pos], [self._slot], [self._bt_list])
            nxt, lg = m.decode(1, graph=self.graph)
            if self.graph:
                self.graph_launches_replayed += self._graph_launches[1]
            if temperature > 0:
                tok = self._pick(lg[:1], temperature, rng)
            else:
                self._tok_host.copy_(nxt, non_blocking=True)
                torch.cuda.current_stream().synchronize()
                tok = int(self._tok_host[0])
            pos += 1
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        return GenerationOutput(out, T, (t1 - t0) * 1e3, (t2 - t1) * 1e3, 0, stopped)

    def _pick(self, logits: torch.Tensor, temperature: float, rng: torch.Generator) -> int:
        if temperature <= 0:
            return int(K.argmax(logits)[0].item())
        t = torch.full((1,), float(temperature), device=logits.device)
        u = torch.rand(1, generator=rng).to(logits.device)
        return int(K.sample(logits, t, u)[0].item())
