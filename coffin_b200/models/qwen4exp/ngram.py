"""Hashed n-gram embedding ids and the embedding table behind the PLE layers.

Ids (reference ``models/qwen4exp/ngram.py:56-149`` for the constants, ``:530-757`` for the
hashing): for every token the 2-gram .. n-gram ending at it is hashed by multiplying each member
token by a per-layer odd 63-bit multiplier (a splitmix64 stream seeded per PLE layer), xor-ing the
products in wrapping 64-bit arithmetic, and reducing modulo a per-head prime; heads of one n-gram
order use consecutive primes above ``ngram_vocab_size_base`` and index disjoint row ranges of one
table.  History never crosses an end-of-sequence token: members before the latest EOS read as EOS.

Table: on the reference hardware the real table (~95 GiB of bf16 rows) lives in host memory and rows
are gathered per step (``HostNGramTable``, ``:152-470``).  A B200 has 180 GB of HBM, so
``NGramTable`` keeps the table on the device when it fits the given budget and otherwise keeps it
in pinned host memory and gathers rows with an asynchronous copy on a side stream (``prefetch`` /
``take``), so the gather of step ``n+1`` overlaps step ``n``.
"""
from __future__ import annotations

import math

import torch

MASK64 = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15
LAYER_STRIDE = 10007


def splitmix64(x: int) -> int:
    x = (x + GOLDEN) & MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & MASK64
    return (x ^ (x >> 31)) & MASK64


def _signed(x: int) -> int:
    x &= MASK64
    return x - (1 << 64) if x >> 63 else x


def layer_multipliers(vocab: int, ngram_size: int, ple_index: int, seed: int) -> list[int]:
    """One odd multiplier per n-gram member position, small enough that ``token * m`` of the
    first member cannot overflow a signed 64-bit integer by more than the wrap the hash accepts."""
    half = max(1, (((1 << 63) - 1) // max(vocab, 1)) // 2)
    base = seed + LAYER_STRIDE * ple_index
    return [2 * (splitmix64((base + GOLDEN * (i + 1)) & MASK64) % half) + 1 for i in range(ngram_size)]


def is_prime(n: int) -> bool:
    if n < 2:
        return False
    if n % 2 == 0:
        return n == 2
    return all(n % d for d in range(3, math.isqrt(n) + 1, 2))


def primes_after(start: int, count: int) -> list[int]:
    """The first ``count`` primes strictly greater than ``start``."""
    out, n = [], start
    while len(out) < count:
        n += 1
        if is_prime(n):
            out.append(n)
    return out


class NGramHasher:
    """Row ids of one PLE layer.  ``ids(tokens, context)`` -> int64 ``[T, heads]``."""

    def __init__(self, cfg, ple_index: int) -> None:
        self.n, self.per = cfg.ngram_size, cfg.heads_per_ngram
        self.eos = cfg.eos_token_id
        self.heads = cfg.ngram_heads
        self.mult = layer_multipliers(cfg.vocab_size, self.n, ple_index, cfg.seed)
        first = ple_index * self.heads
        self.sizes = primes_after(cfg.ngram_vocab_size_base - 1, first + self.heads)[first:]
        self.offsets = [sum(self.sizes[:i]) for i in range(self.heads)]
        total = sum(self.sizes)
        d = cfg.make_ngram_vocab_size_divisible_by
        self.rows = (total + d - 1) // d * d
        self.context_len = self.n - 1

    def ids(self, tokens: list[int], context: list[int] | None = None) -> torch.Tensor:
        ctx = list(context) if context is not None else [self.eos] * self.context_len
        hist = ctx + [int(t) for t in tokens]
        out = torch.empty(len(tokens), self.heads, dtype=torch.int64)
        seg_start = 0                                   # first index after the latest EOS before i
        starts = []
        for i, t in enumerate(hist):
            starts.append(seg_start)
            if t == self.eos:
                seg_start = i + 1
        for r in range(len(tokens)):
            i = len(ctx) + r
            members = [hist[i - s] if i - s >= starts[i] else self.eos for s in range(self.n)]
            mixed = 0
            row = []
            for order in range(2, self.n + 1):
                mixed = 0
                for s in range(order):
                    mixed ^= (members[s] * self.mult[s]) & MASK64
                sm = _signed(mixed)
                for h in range((order - 2) * self.per, (order - 1) * self.per):
                    row.append(sm % self.sizes[h] + self.offsets[h])
            out[r] = torch.tensor(row, dtype=torch.int64)
        return out


class NGramTable:
    """Embedding rows ``[rows, head_dim]`` on the device, or in pinned host memory with an
    asynchronous gather.  ``device_budget_bytes``: tables up to this size are moved to the device."""

    def __init__(self, weight: torch.Tensor, device, device_budget_bytes: int = 120 << 30) -> None:
        self.device = torch.device(device)
        self.rows, self.width = weight.shape
        nbytes = weight.numel() * weight.element_size()
        self.on_device = self.device.type != "cuda" or nbytes <= device_budget_bytes
        if self.on_device:
            self.weight = weight.to(self.device)
        else:
            self.weight = weight.cpu().contiguous()
            if not self.weight.is_pinned():
                self.weight = self.weight.pin_memory()
            self._stream = torch.cuda.Stream(device=self.device)
            self._stage: torch.Tensor | None = None
        self._pending: tuple | None = None

    def gather(self, ids: torch.Tensor) -> torch.Tensor:
        """``ids [T, heads]`` (host int64) -> ``[T, heads * width]`` on the device."""
        if int(ids.min()) < 0 or int(ids.max()) >= self.rows:
            raise ValueError(f"n-gram row ids outside [0, {self.rows})")
        flat = ids.reshape(-1)
        if self.on_device:
            return self.weight[flat.to(self.device)].reshape(ids.shape[0], -1)
        self.prefetch(ids)
        return self.take(ids)

    def prefetch(self, ids: torch.Tensor) -> None:
        """Start gathering the rows of the next step (host gather into a pinned stage, then an
        asynchronous copy on a side stream)."""
        if self.on_device:
            self._pending = (ids.clone(), None, None)
            return
        if self._pending is not None:
            raise RuntimeError("previous prefetch was not taken")
        flat = ids.reshape(-1)
        n = flat.numel()
        if self._stage is None or self._stage.shape[0] < n:
            self._stage = torch.empty(max(n, 4096), self.width, dtype=self.weight.dtype).pin_memory()
        stage = self._stage[:n]
        self._fill(flat, stage)
        with torch.cuda.stream(self._stream):
            dev = stage.to(self.device, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self._stream)
        self._pending = (ids.clone(), dev, ev)

    def _fill(self, flat: torch.Tensor, out: torch.Tensor) -> None:
        """Rows ``flat`` (host int64) of the host table into ``out [n, width]`` (pinned)."""
        torch.index_select(self.weight, 0, flat, out=out)

    def take(self, ids: torch.Tensor) -> torch.Tensor:
        if self._pending is None:
            return self.gather(ids)
        want, dev, ev = self._pending
        self._pending = None
        if want.shape != ids.shape or not torch.equal(want, ids):
            return self.gather(ids)             # the prefetch guessed another continuation
        if dev is None:
            return self.gather(ids)
        torch.cuda.current_stream().wait_event(ev)
        return dev.reshape(ids.shape[0], -1)


class ShardedNGramTable(NGramTable):
    """The table as the checkpoint stores it: equally sized shards ``...ngram_embedding.shard_{k}.weight``
    (128 x [2500012, 160] bf16 = 102 GB for the published geometry), kept as the VIEWS the loader hands over
    (file mappings of the safetensors shards) instead of one concatenated tensor - a copy would double the
    host footprint and cost a 100 GB pass at start-up for a table of which a step reads a few dozen rows.
    Row ``r`` lives in shard ``r // rows_per_shard`` at ``r % rows_per_shard``; a gather groups its ids by
    shard (one ``index_select`` per touched shard) and puts the rows back in request order.  Shards of unequal
    height would shift every later row and still look well-formed, so they are refused
    (reference: ``models/qwen4exp/ngram.py:363-470``).  ``keep``: whatever keeps the mappings alive."""

    def __init__(self, shards: list[torch.Tensor], device, device_budget_bytes: int = 120 << 30, keep=None) -> None:
        if not shards:
            raise ValueError("the sharded n-gram table needs at least one shard")
        first = shards[0]
        for k, t in enumerate(shards):
            if t.dim() != 2 or t.shape != first.shape or t.dtype != first.dtype:
                raise ValueError(f"n-gram shard {k} is {tuple(t.shape)}/{t.dtype}, shard 0 is {tuple(first.shape)}/{first.dtype}: "
                                 "unequal shards would shift the row mapping")
            if t.device.type != "cpu":
                raise ValueError(f"n-gram shard {k} is on {t.device}; the sharded table is the host-resident form")
        self.device = torch.device(device)
        self.rows_per_shard, self.width = int(first.shape[0]), int(first.shape[1])
        self.rows = self.rows_per_shard * len(shards)
        self.keep = keep
        nbytes = self.rows * self.width * first.element_size()
        self.on_device = self.device.type == "cuda" and nbytes <= device_budget_bytes
        if self.on_device:                      # small enough for HBM: one device tensor, filled shard by shard
            self.weight = torch.empty(self.rows, self.width, dtype=first.dtype, device=self.device)
            for k, t in enumerate(shards):
                self.weight[k * self.rows_per_shard:(k + 1) * self.rows_per_shard].copy_(t)
            self.shards = []
        else:
            self.shards = list(shards)
            self.weight = first                 # dtype / width holder for the staging buffer
            if self.device.type == "cuda":
                self._stream = torch.cuda.Stream(device=self.device)
            self._stage = None
        self._pending = None

    def gather(self, ids: torch.Tensor) -> torch.Tensor:
        if self.on_device or self.device.type == "cuda":
            return super().gather(ids)
        if int(ids.min()) < 0 or int(ids.max()) >= self.rows:
            raise ValueError(f"n-gram row ids outside [0, {self.rows})")
        out = torch.empty(ids.numel(), self.width, dtype=self.weight.dtype)
        self._fill(ids.reshape(-1), out)
        return out.reshape(ids.shape[0], -1)

    def prefetch(self, ids: torch.Tensor) -> None:
        if self.device.type != "cuda":          # nothing to overlap with on the host: the gather happens in take()
            self._pending = (ids.clone(), None, None)
            return
        super().prefetch(ids)

    def _fill(self, flat: torch.Tensor, out: torch.Tensor) -> None:
        if flat.numel() == 0:
            return
        flat = flat.to("cpu")
        shard_of = torch.div(flat, self.rows_per_shard, rounding_mode="floor")
        order = torch.argsort(shard_of, stable=True)
        local = (flat - shard_of * self.rows_per_shard)[order]          # grouped by shard, request order inside a group
        bounds = torch.cumsum(torch.bincount(shard_of, minlength=len(self.shards)), 0).tolist()
        grouped = torch.empty_like(out)
        start = 0
        for k, stop in enumerate(bounds):
            if stop > start:
                torch.index_select(self.shards[k], 0, local[start:stop], out=grouped[start:stop])
                start = stop
        out.index_copy_(0, order, grouped)

    def close(self) -> None:
        """Drop the shard views and whatever kept their mappings alive; the table cannot be read afterwards."""
        self.shards = []
        closer = getattr(self.keep, "close", None)
        if closer is not None:
            closer()
        self.keep = None
