"""The image recipe of a checkpoint: read once, accepted only when it names an algorithm the engine implements,
a failure stays a cached 503 and nothing half-built is published (reference: tests/test_runtime_processor.py)."""
import json
from types import SimpleNamespace

import pytest

from coffin_b200.models.qwen35.vision import VisionConfig
from coffin_b200.serving import processor as P
from coffin_b200.serving.runtime import MMError

VC = VisionConfig(depth=1, hidden_size=32, num_heads=2, intermediate_size=64, out_hidden_size=32)


def service(tmp_path, cfg=None):
    if cfg is not None:
        (tmp_path / P.CONFIG_NAME).write_text(json.dumps(cfg), encoding="utf-8")
    return SimpleNamespace(model_path=str(tmp_path), processor=None, _processor_failed=None, vision=SimpleNamespace(cfg=VC),
                           cfg=SimpleNamespace(image_min_pixels=65536, image_max_pixels=1048576))


GOOD = {"processor_class": "Qwen3VLProcessor", "image_processor_type": "Qwen2VLImageProcessorFast",
        "image_mean": [0.48, 0.45, 0.40], "image_std": [0.26, 0.26, 0.27], "patch_size": 16, "merge_size": 2,
        "temporal_patch_size": 2, "size": {"shortest_edge": 3136, "longest_edge": 12845056}}


def test_checkpoint_recipe_is_read_once_and_keeps_the_service_budget(tmp_path):
    srv = service(tmp_path, GOOD)
    r = P.ensure_recipe(srv)
    assert r.mean == (0.48, 0.45, 0.40) and r.std == (0.26, 0.26, 0.27) and r.factor == 32
    assert (r.min_pixels, r.max_pixels) == (65536, 1048576)         # the wider checkpoint budget is clipped by the service's
    assert r.source.endswith(P.CONFIG_NAME)
    (tmp_path / P.CONFIG_NAME).unlink()
    assert P.ensure_recipe(srv) is r                                 # cached: the file is not read again


def test_a_tighter_checkpoint_budget_wins(tmp_path):
    srv = service(tmp_path, {**GOOD, "size": None, "min_pixels": 100000, "max_pixels": 500000})
    r = P.ensure_recipe(srv)
    assert (r.min_pixels, r.max_pixels) == (100000, 500000)


def test_no_file_means_the_builtin_recipe(tmp_path):
    srv = service(tmp_path)
    r = P.ensure_recipe(srv)
    assert r.source == "builtin" and r.mean == (0.5, 0.5, 0.5) and r.patch_size == VC.patch_size


@pytest.mark.parametrize("change, word", [
    ({"processor_class": "OtherProcessor"}, "OtherProcessor"),
    ({"image_processor_type": "CLIPImageProcessor"}, "CLIPImageProcessor"),
    ({"patch_size": 14}, "geometry"),
    ({"image_std": [0.5, 0.0, 0.5]}, "positive"),
    ({"image_mean": [0.5, 0.5]}, "three numbers"),
])
def test_unknown_algorithm_or_geometry_is_a_cached_503(tmp_path, change, word):
    srv = service(tmp_path, {**GOOD, **change})
    for _ in range(2):
        with pytest.raises(MMError) as e:
            P.ensure_recipe(srv)
        assert e.value.status == 503 and word in str(e.value)
        assert srv.processor is None and word in srv._processor_failed
    (tmp_path / P.CONFIG_NAME).write_text(json.dumps(GOOD))           # repaired on disk: still refused until a reload clears it
    with pytest.raises(MMError):
        P.ensure_recipe(srv)
    srv._processor_failed = None
    assert P.ensure_recipe(srv).source.endswith(P.CONFIG_NAME)


def test_unreadable_file_does_not_publish_a_partial_recipe(tmp_path):
    srv = service(tmp_path)
    (tmp_path / P.CONFIG_NAME).write_text("{ not json", encoding="utf-8")
    with pytest.raises(MMError) as e:
        P.ensure_recipe(srv)
    assert e.value.status == 503 and srv.processor is None and "JSONDecodeError" in srv._processor_failed


def test_patchify_uses_the_recipe_normalisation():
    import torch
    from coffin_b200.models.qwen35.vision import patchify
    img = torch.full((3, 32, 32), 0.75)
    a, grid = patchify(img, VC)
    b, _ = patchify(img, VC, (0.25, 0.25, 0.25), (0.25, 0.25, 0.25))
    assert grid == (1, 2, 2) and torch.allclose(a, torch.full_like(a, 0.5)) and torch.allclose(b, torch.full_like(b, 2.0))
