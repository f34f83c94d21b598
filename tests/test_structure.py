"""Structural gates, run on the sources without a GPU: the Python side and the kernel library agree on the
exported entry points, the package keeps its layering, and nothing reaches for a tracing compiler or a
second backend (the reference keeps the same kind of gates in tests/test_backends.py and
tests/test_backends_purity.py)."""
import ast
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
PKG = ROOT / "coffin_b200"
PY = sorted(p for p in PKG.rglob("*.py"))
CU = sorted((PKG / "_C").glob("*.cu"))


def _exports() -> set[str]:
    out = set()
    for f in CU:
        out |= set(re.findall(r"CB_EXPORT\s+[\w\s\*]+?\bcb_(\w+)\s*\(", f.read_text()))
    return out


def _called() -> dict[str, set[str]]:
    """Kernel entry points named from Python: the first string argument of call / call_nostream, and cb_ attributes."""
    used: dict[str, set[str]] = {}
    for f in PY + [ROOT / "bench.py", ROOT / "__graft_entry__.py"] + sorted((ROOT / "tests").glob("*.py")):
        src = f.read_text()
        names = set(re.findall(r"\bcall(?:_nostream)?\(\s*\"(\w+)\"", src)) | set(re.findall(r"\.cb_(\w+)\b", src))
        if f.name == "_lib.py":
            names.discard("name")                      # the docstring's placeholder
        for n in names:
            used.setdefault(n, set()).add(f.relative_to(ROOT).as_posix())
    return used


def test_every_entry_point_named_from_python_is_exported_by_the_library():
    exports, used = _exports(), _called()
    assert len(exports) > 60, "the export scan found too few symbols: the pattern no longer matches the sources"
    missing = {n: sorted(fs) for n, fs in used.items() if n not in exports}
    assert not missing, f"called from Python but not exported by any .cu: {missing}"


def test_exported_entry_points_are_reachable_from_python():
    """An export nobody calls is either dead or untested; the few that exist for other runtimes are listed."""
    allow = {"argmax_static",            # allocation-free entry point for embedding runtimes (no_alloc.h)
             "trace_register", "trace_name",
             # introspection / tuning hooks for callers that size their own scratch or sweep a variant
             "gemm_splitk_plan", "gemm_splitk_ws_bytes", "set_stream_opts", "tp_os_rows"}
    unused = sorted(_exports() - set(_called()) - allow)
    assert not unused, f"exported but never called from Python or the tests: {unused}"


def _imports(path: Path) -> set[str]:
    """Absolute module names a file imports from inside the package (relative imports resolved)."""
    tree = ast.parse(path.read_text())
    pkg_parts = path.relative_to(ROOT).with_suffix("").parts[:-1]
    out = set()
    for node in ast.walk(tree):
        if isinstance(node, ast.ImportFrom):
            if node.level:
                base = list(pkg_parts[:len(pkg_parts) - node.level + 1])
                mod = ".".join(base + ([node.module] if node.module else []))
            else:
                mod = node.module or ""
            out.add(mod)
            for a in node.names:
                out.add(f"{mod}.{a.name}")
        elif isinstance(node, ast.Import):
            out |= {a.name for a in node.names}
    return out


def test_no_tracing_compiler_second_backend_or_working_files_in_the_package():
    banned = ("triton", "tilelang", "jax", "_work", "tests")
    for f in PY:
        mods = _imports(f)
        hit = sorted(m for m in mods if m.split(".")[0] in banned)
        assert not hit, f"{f.relative_to(ROOT)} imports {hit}"
        src = f.read_text()
        assert "torch.compile(" not in src and "@torch.compile" not in src, f"{f.relative_to(ROOT)} uses torch.compile"


def test_layering_lower_layers_do_not_import_upward():
    """ops / weights / cache know nothing of the engine; the engine nothing of serving or the entry points;
    the CPU oracle is a test oracle and the CPU twin, not something the device model leans on."""
    rules = {
        "ops": ("engine", "serving", "entrypoints", "models"),
        "weights": ("engine", "serving", "entrypoints"),
        "cache": ("engine", "serving", "entrypoints", "models"),
        "engine": ("serving", "entrypoints"),
        "serving": ("entrypoints",),
        "parallel": ("serving", "entrypoints"),
    }
    bad = []
    for f in PY:
        rel = f.relative_to(PKG).parts
        layer = rel[0]
        for m in _imports(f):
            parts = m.split(".")
            if parts[0] != "coffin_b200" or len(parts) < 2:
                continue
            if parts[1] in rules.get(layer, ()):
                bad.append(f"{f.relative_to(ROOT)} -> {m}")
    # lazy imports inside functions of the debugging switches are the one sanctioned exception
    bad = [b for b in bad if "engine.debug" not in b and "engine/debug.py" not in b]
    assert not bad, "upward imports:\n" + "\n".join(sorted(set(bad)))
    for f in sorted((PKG / "models").rglob("*.py")):
        if f.name == "oracle.py":
            continue
        # oracle.ops holds the host-side table builders (rotary rows) both sides share; the oracle MODELS stay out
        leaned = [m for m in _imports(f) if m.startswith("coffin_b200.oracle") and not m.startswith("coffin_b200.oracle.ops")
                  and m != "coffin_b200.oracle"]
        assert not leaned, f"{f.relative_to(ROOT)} imports the CPU oracle: {leaned}"


def test_every_preset_resolves_and_validates():
    from coffin_b200.config import preset
    for name in ("tiny", "qwen35-4b", "qwen35-27b", "qwen35-35b-a3b", "tiny-qwen4", "qwen4exp-a"):
        cfg = preset(name)
        assert cfg.num_hidden_layers == len(cfg.layer_types)
        if hasattr(cfg, "validate"):
            cfg.validate()


def test_kernel_sources_are_built_for_sm_100a_only():
    src = (PKG / "_C" / "build.py").read_text()
    assert "arch=compute_100a,code=sm_100a" in src and "-lineinfo" in src
    assert not re.search(r"sm_(8\d|9\d)\b", src), "another architecture crept into the build flags"
