"""Multimodal request payload: image embeddings, their token spans and mRoPE positions.

An image occupies a run of ``IMAGE_TOKEN_ID`` placeholders in the prompt; the vision tower's
merged patch embeddings replace the placeholder rows, and every token gets a 3-axis rotary
position (t, h, w): text tokens advance all three together, an image's tokens share one ``t`` and
enumerate the patch grid on ``h``/``w``, and the text after an image resumes at
``max(position) + 1``, which leaves ``rope_delta = next_position - token_index`` for decode.
Reference: ``utils/mm_input.py:50-260``.
"""
from __future__ import annotations

import dataclasses
import hashlib
from typing import Sequence

import torch

IMAGE_TOKEN_ID = 248056
VISION_START_ID = 248053
VISION_END_ID = 248054


def image_digest(data: bytes, extra: str = "") -> str:
    h = hashlib.sha256()
    h.update(data)
    h.update(extra.encode())
    return h.hexdigest()


def find_image_spans(tokens: Sequence[int], image_token_id: int = IMAGE_TOKEN_ID) -> list[tuple[int, int]]:
    spans, i, n = [], 0, len(tokens)
    while i < n:
        if tokens[i] == image_token_id:
            j = i
            while j < n and tokens[j] == image_token_id:
                j += 1
            spans.append((i, j))
            i = j
        else:
            i += 1
    return spans


def mrope_positions(n_tokens: int, spans: Sequence[tuple[int, int]], grids: Sequence[tuple[int, int, int]],
                    merge: int = 2) -> tuple[torch.Tensor, int]:
    """``positions [3, n_tokens]`` and ``rope_delta``.  ``grids[i] = (t, h, w)`` is the patch grid of
    image ``i`` before the ``merge x merge`` spatial merge."""
    pos = torch.zeros(3, n_tokens, dtype=torch.long)
    nxt, cur = 0, 0
    for (s, e), (t, h, w) in zip(spans, grids):
        n_text = s - cur
        pos[:, cur:s] = torch.arange(nxt, nxt + n_text)
        nxt += n_text
        gh, gw = h // merge, w // merge
        if t * gh * gw != e - s:
            raise ValueError(f"image span of {e - s} tokens does not match grid {t}x{gh}x{gw}")
        tt = torch.arange(t).repeat_interleave(gh * gw)
        hh = torch.arange(gh).repeat_interleave(gw).repeat(t)
        ww = torch.arange(gw).repeat(t * gh)
        pos[0, s:e], pos[1, s:e], pos[2, s:e] = nxt + tt, nxt + hh, nxt + ww
        nxt += max(t, gh, gw)
        cur = e
    pos[:, cur:] = torch.arange(nxt, nxt + n_tokens - cur)
    nxt += n_tokens - cur
    return pos, nxt - n_tokens


@dataclasses.dataclass
class MMInput:
    embeds: torch.Tensor | None          # [sum image tokens, hidden], prompt order
    grid_thw: list[tuple[int, int, int]]
    positions: torch.Tensor | None       # [3, L]
    rope_delta: int
    digests: list[str]
    spans: list[tuple[int, int]]

    @property
    def digest(self) -> str:
        return hashlib.sha256("".join(self.digests).encode()).hexdigest()

    def slice_positions(self, start: int, end: int) -> torch.Tensor:
        return self.positions[:, start:end]

    def scatter_into(self, x: torch.Tensor, start: int, end: int) -> torch.Tensor:
        """Overwrite the image rows of the chunk ``x`` (absolute prompt positions
        ``[start, end)``) with the matching embedding rows; returns ``x``."""
        if self.embeds is None:
            return x
        base = 0
        for s, e in self.spans:
            a, b = max(s, start), min(e, end)
            if a < b:
                x[a - start:b - start] = self.embeds[base + (a - s):base + (b - s)].to(dtype=x.dtype, device=x.device)
            base += e - s
        return x
