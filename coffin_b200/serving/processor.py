"""The image-processing recipe of a checkpoint, loaded lazily and checked before it is cached.

The engine cuts images into patches itself (resize inside a pixel budget to a multiple of
``patch * merge``, normalise, repeat over the temporal patch, merge-block order), which is the algorithm
of the Qwen2-VL / Qwen3-VL image processors.  A checkpoint states which algorithm it was trained with
in ``preprocessor_config.json``; this module reads that file, accepts it only when it names one of the
processors whose algorithm the engine implements, takes mean / std / pixel budgets / patch geometry
from it, and refuses everything else with a 503 that names the reason.  A refusal is cached: the file
is read once, a broken checkpoint answers 503 on every image request instead of failing somewhere
inside the prefill, and no half-initialised recipe is ever published on the service.

The reference loads a ``transformers`` processor for the same job and guards the same failure modes
(``serving/runtime_parts.py:_ensure_processor``: a tokenizer-only object must not be cached as a vision
processor, an unrecognised processor class is rejected, a failed load stays a 503).
"""
from __future__ import annotations

import dataclasses
import json
from pathlib import Path

KNOWN_IMAGE_PROCESSORS = frozenset({
    "Qwen2VLImageProcessor", "Qwen2VLImageProcessorFast", "Qwen3VLImageProcessor", "Qwen3VLImageProcessorFast",
})
KNOWN_PROCESSOR_CLASSES = frozenset({"Qwen2VLProcessor", "Qwen2_5_VLProcessor", "Qwen3VLProcessor"})
CONFIG_NAME = "preprocessor_config.json"


@dataclasses.dataclass(frozen=True)
class ImageRecipe:
    mean: tuple[float, float, float]
    std: tuple[float, float, float]
    min_pixels: int
    max_pixels: int
    patch_size: int
    merge_size: int
    temporal_patch_size: int
    source: str          # "builtin" (no file in the checkpoint) or the path of the file the values came from

    @property
    def factor(self) -> int:
        return self.patch_size * self.merge_size


def builtin_recipe(vc, min_pixels: int, max_pixels: int) -> ImageRecipe:
    """The recipe of a tower without a checkpoint file (random weights, tests): the tower's own geometry and
    the service's pixel budget."""
    from ..models.qwen35.vision import MEAN, STD
    return ImageRecipe(tuple(MEAN), tuple(STD), int(min_pixels), int(max_pixels), vc.patch_size, vc.spatial_merge_size,
                       vc.temporal_patch_size, "builtin")


def _triple(v, name: str) -> tuple[float, float, float]:
    if not isinstance(v, (list, tuple)) or len(v) != 3:
        raise ValueError(f"{name} must be three numbers, got {v!r}")
    out = tuple(float(x) for x in v)
    return out      # type: ignore[return-value]


def read_recipe(path: Path, vc, min_pixels: int, max_pixels: int) -> ImageRecipe:
    """Parse ``preprocessor_config.json``.  Raises ``ValueError`` with a readable reason when the file names an
    algorithm the engine does not implement or a geometry the tower was not built for."""
    raw = json.loads(Path(path).read_text(encoding="utf-8"))
    if not isinstance(raw, dict):
        raise ValueError("preprocessor config is not a JSON object")
    kind = raw.get("image_processor_type")
    cls = raw.get("processor_class")
    if kind is None and cls is None:
        raise ValueError("preprocessor config names neither image_processor_type nor processor_class")
    if kind is not None and kind not in KNOWN_IMAGE_PROCESSORS:
        raise ValueError(f"image processor {kind!r} is not one the engine implements ({', '.join(sorted(KNOWN_IMAGE_PROCESSORS))})")
    if cls is not None and cls not in KNOWN_PROCESSOR_CLASSES:
        raise ValueError(f"processor class {cls!r} is not one the engine implements ({', '.join(sorted(KNOWN_PROCESSOR_CLASSES))})")
    base = builtin_recipe(vc, min_pixels, max_pixels)
    mean = _triple(raw["image_mean"], "image_mean") if "image_mean" in raw else base.mean
    std = _triple(raw["image_std"], "image_std") if "image_std" in raw else base.std
    if any(s <= 0 for s in std):
        raise ValueError(f"image_std must be positive, got {std}")
    patch = int(raw.get("patch_size", base.patch_size))
    merge = int(raw.get("merge_size", base.merge_size))
    temporal = int(raw.get("temporal_patch_size", base.temporal_patch_size))
    if (patch, merge, temporal) != (base.patch_size, base.merge_size, base.temporal_patch_size):
        raise ValueError(f"preprocessor geometry patch={patch} merge={merge} temporal={temporal} differs from the tower's "
                         f"patch={base.patch_size} merge={base.merge_size} temporal={base.temporal_patch_size}")
    # the checkpoint's own budget ("size": shortest/longest edge are pixel COUNTS in this family, or
    # min_pixels/max_pixels), clipped by the service's: the service's limits bound the tower's memory per request
    size = raw.get("size") if isinstance(raw.get("size"), dict) else {}
    lo = raw.get("min_pixels", size.get("shortest_edge"))
    hi = raw.get("max_pixels", size.get("longest_edge"))
    lo = max(int(lo), int(min_pixels)) if lo is not None else int(min_pixels)
    hi = min(int(hi), int(max_pixels)) if hi is not None else int(max_pixels)
    if lo > hi:
        lo = hi
    if hi < (patch * merge) ** 2:
        raise ValueError(f"pixel budget {hi} is below one merged patch ({(patch * merge) ** 2} pixels)")
    return ImageRecipe(mean, std, lo, hi, patch, merge, temporal, str(path))


def ensure_recipe(srv) -> ImageRecipe:
    """The service's image recipe, loaded on the first image request and cached on ``srv.processor``; a failure
    is cached on ``srv._processor_failed`` and raised as a 503 on this and every later request."""
    from .runtime import MMError
    cached = getattr(srv, "processor", None)
    if cached is not None:
        return cached
    failed = getattr(srv, "_processor_failed", None)
    if failed:
        raise MMError(f"image processing is unavailable: {failed}", 503)
    vc = srv.vision.cfg
    lo, hi = srv.cfg.image_min_pixels, srv.cfg.image_max_pixels
    model_dir = getattr(srv, "model_path", "") or ""
    path = Path(model_dir) / CONFIG_NAME if model_dir else None
    try:
        recipe = read_recipe(path, vc, lo, hi) if path is not None and path.is_file() else builtin_recipe(vc, lo, hi)
    except (OSError, ValueError, KeyError, TypeError) as exc:
        srv._processor_failed = f"{type(exc).__name__}: {exc}"
        srv.processor = None
        raise MMError(f"image processing is unavailable: {srv._processor_failed}", 503) from None
    srv.processor = recipe            # published only when complete
    return recipe
