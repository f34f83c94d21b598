"""Image payloads of a chat request -> ``MMInput`` (embeddings, spans, mRoPE positions).

Images arrive as base64 (the HTTP adapter already refused remote URLs and enforced byte budgets).
Each one is decoded with PIL (EXIF orientation applied, decompression bombs and out-of-budget
sizes refused), resized to a multiple of ``patch * merge`` inside the pixel budget, cut into
patches, run through the vision tower, and its single ``<|image_pad|>`` placeholder in the prompt
is expanded to one placeholder per merged patch.  Reference: ``serving/runtime_support.py:184-242``
(``_decode_image``), ``serving/runtime_parts.py:553-700`` (``_prepare_mm``), ``utils/mm_input.py``.
"""
from __future__ import annotations

import base64
import binascii
import io

import torch

from ..utils.mm_input import MMInput, find_image_spans, image_digest, mrope_positions

MAX_DECODE_PIXELS = 64 * 1024 * 1024


def decode_image(b64: str, min_pixels: int, max_pixels: int, factor: int, max_bytes: int = 0) -> tuple[torch.Tensor, bytes]:
    """base64 -> ``[3, H, W]`` float tensor in [0, 1] (sides multiples of ``factor``) and the raw bytes.
    ``max_bytes`` > 0: decoded payloads above it are refused with 413 (the socket can be reached without the
    HTTP front, so the engine keeps its own limit)."""
    from .runtime import MMError
    from ..models.qwen35.vision import smart_resize
    if max_bytes > 0 and len(b64) * 3 // 4 - 2 > max_bytes:
        raise MMError(f"image larger than {max_bytes} bytes", 413)
    try:
        raw = base64.b64decode(b64, validate=True)
    except (binascii.Error, ValueError):
        raise MMError("image payload is not valid base64", 400) from None
    if max_bytes > 0 and len(raw) > max_bytes:
        raise MMError(f"image larger than {max_bytes} bytes", 413)
    try:
        from PIL import Image, ImageOps
        Image.MAX_IMAGE_PIXELS = MAX_DECODE_PIXELS
        img = Image.open(io.BytesIO(raw))
        if img.width * img.height > MAX_DECODE_PIXELS:
            raise MMError("image has too many pixels to decode", 413)
        img = ImageOps.exif_transpose(img).convert("RGB")
    except MMError:
        raise
    except Exception as exc:          # noqa: BLE001 - PIL raises many types on corrupt files
        raise MMError(f"cannot decode image: {type(exc).__name__}", 400) from None
    if min(img.width, img.height) < 4:
        raise MMError("image is too small", 400)
    h, w = smart_resize(img.height, img.width, factor, min_pixels, max_pixels)
    img = img.resize((w, h), Image.BICUBIC)
    t = torch.frombuffer(bytearray(img.tobytes()), dtype=torch.uint8).reshape(h, w, 3).permute(2, 0, 1).float() / 255.0
    return t, raw


def expand_placeholders(prompt: list[int], image_token_id: int, counts: list[int]) -> list[int]:
    """Replace the i-th run of image placeholders by ``counts[i]`` placeholders."""
    from .runtime import MMError
    spans = find_image_spans(prompt, image_token_id)
    if len(spans) != len(counts):
        raise MMError(f"prompt has {len(spans)} image placeholders for {len(counts)} images", 400)
    out, cur = [], 0
    for (s, e), n in zip(spans, counts):
        out.extend(prompt[cur:s])
        out.extend([image_token_id] * n)
        cur = e
    out.extend(prompt[cur:])
    return out


def build_mm_input(srv, images: list[dict], prompt: list[int]):
    """Run the tower on every image and return ``(MMInput, expanded prompt)``."""
    from ..models.qwen35.vision import patchify
    from .processor import ensure_recipe
    tower = srv.vision
    vc = tower.cfg
    recipe = ensure_recipe(srv)          # 503 (cached) when the checkpoint states an algorithm the engine does not implement
    image_token = getattr(srv.tok, "special", {}).get("<|image_pad|>") if hasattr(srv.tok, "special") else None
    if image_token is None:
        image_token = srv.tok.encode("<|image_pad|>")[0]
    embeds, grids, digests = [], [], []
    for im in images:
        t, raw = decode_image(im["b64"], recipe.min_pixels, recipe.max_pixels, recipe.factor,
                              getattr(srv.cfg, "max_image_bytes", 0))
        patches, grid = patchify(t, vc, recipe.mean, recipe.std)
        embeds.append(tower.forward(patches, grid))
        grids.append(grid)
        digests.append(image_digest(raw, f"{grid}"))
    m2 = vc.spatial_merge_size ** 2
    counts = [g[0] * g[1] * g[2] // m2 for g in grids]
    prompt = expand_placeholders(prompt, image_token, counts)
    spans = find_image_spans(prompt, image_token)
    positions, delta = mrope_positions(len(prompt), spans, grids, vc.spatial_merge_size)
    mm = MMInput(embeds=torch.cat(embeds), grid_thw=grids, positions=positions, rope_delta=delta,
                 digests=digests, spans=spans)
    return mm, prompt
