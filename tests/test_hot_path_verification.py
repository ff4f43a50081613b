"""Re-checks the finding this repository rests on: the reference project
(bat0001/peer-review-agents) contains no Expert-Threshold MoE token-routing
code -- no threshold router, CSR build, CSR scatter/gather, balanced
permutation, expert-parallel dispatch/combine or weighted combine -- and so no
oracle, no drop-in boundary and no CPU baseline can be derived from it.

The scan runs only where a checkout of the reference is present (directory given
by ``$REFERENCE_ROOT``, else the build container's mount point); elsewhere it is
skipped.
The remaining tests need nothing but this repository.
"""

import json
import os
import pathlib
import re
import subprocess
import sys

import pytest

REPO = pathlib.Path(__file__).resolve().parent.parent
REFERENCE = pathlib.Path(os.environ.get("REFERENCE_ROOT", "/root/reference"))

needs_reference = pytest.mark.skipif(
    not (REFERENCE / "cli" / "reva").is_dir(), reason="reference checkout not present"
)

# File types that could hold a kernel, a native extension or a packed archive of one.
NATIVE_SUFFIXES = {
    ".cu", ".cuh", ".cpp", ".cc", ".cxx", ".c", ".h", ".hpp", ".rs", ".go",
    ".so", ".a", ".whl", ".ipynb", ".pt", ".ptx", ".cubin", ".zip", ".gz", ".tar",
}

# Words any implementation of the named path would have to use somewhere.
PATH_TERMS = re.compile(
    r"triton|torch|\bmoe\b|mixture.of.experts|all_to_all|alltoall|nccl|\bcuda\b|"
    r"permut|scatter|top-?k|numpy|\bjax\b|\bcsr\b|expert|router|threshold|gather|tensor",
    re.IGNORECASE,
)

# The only files in the reference that match PATH_TERMS, and why each is unrelated:
# a cloud-console automation skill whose container templates are *named*
# "pytorch" / "tensorflow" / "cuda" (.claude/skills/access-fpt-cloud/fpt_manage.py:38-47,
# SKILL.md:95).
UNRELATED_MATCHES = {
    ".claude/skills/access-fpt-cloud/SKILL.md",
    ".claude/skills/access-fpt-cloud/fpt_manage.py",
}


def _reference_files():
    return [p for p in REFERENCE.rglob("*") if p.is_file()]


@needs_reference
def test_reference_has_no_native_or_kernel_files():
    native = [p for p in _reference_files() if p.suffix.lower() in NATIVE_SUFFIXES]
    assert native == []
    assert not (REFERENCE / ".gitmodules").exists()
    assert [p for p in REFERENCE.rglob("*") if p.is_symlink()] == []


@needs_reference
def test_reference_has_no_routing_or_tensor_code():
    hits = set()
    for p in _reference_files():
        try:
            text = p.read_text(encoding="utf-8")
        except (UnicodeDecodeError, OSError):
            continue
        if PATH_TERMS.search(text):
            hits.add(p.relative_to(REFERENCE).as_posix())
    assert hits <= UNRELATED_MATCHES, sorted(hits - UNRELATED_MATCHES)


@needs_reference
def test_reference_declares_no_numeric_dependency():
    numeric = re.compile(r"^name = \"(torch|triton|numpy|jax|jaxlib|cupy.*|nvidia-.*|cuda-.*)\"", re.M)
    assert numeric.findall((REFERENCE / "uv.lock").read_text()) == []
    for toml in ("pyproject.toml", "cli/pyproject.toml"):
        assert not re.search(r"torch|triton|numpy|jax|cupy", (REFERENCE / toml).read_text(), re.I)


def test_baseline_records_the_absence():
    v = json.loads((REPO / "BASELINE.json").read_text())["hot_path_verification"]
    assert v["status"] == "absent"
    assert v["module_path"] is None
    assert v["python_entry_points"] == []


def test_no_kernel_or_oracle_was_invented():
    """While the path is recorded absent, nothing here may pose as its product or oracle."""
    for pattern in ("**/*.cu", "**/*.cuh", "oracle/**/*", "include/*.h"):
        found = [p for p in REPO.glob(pattern) if "_work" not in p.parts and "gpurun_out" not in p.parts]
        assert found == [], found


@pytest.mark.parametrize("extra", [[], ["--impl", "reference"]])
def test_bench_reports_unavailable_and_exits_zero(extra):
    out = subprocess.run(
        [sys.executable, str(REPO / "bench.py"), "--gpus", "1", "--steps", "2", "--warmup", "3", *extra],
        capture_output=True, text=True, timeout=120, check=True,
    ).stdout.strip().splitlines()
    assert len(out) == 1
    line = json.loads(out[0])
    assert "unavailable" in line and line["unavailable"]
    assert line.get("value") is None
    assert line.get("gpu_launches", 0) == 0
    if extra:
        assert line["impl"] == "reference"


def test_bench_non_zero_ranks_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run(
        [sys.executable, str(REPO / "bench.py"), "--gpus", "2"],
        capture_output=True, text=True, timeout=120, env=env, check=True,
    )
    assert r.stdout.strip() == ""


def test_entry_points_state_that_nothing_is_built():
    sys.path.insert(0, str(REPO))
    try:
        import __graft_entry__ as entry
    finally:
        sys.path.pop(0)
    entry.build()  # nothing to compile; must not raise
    with pytest.raises(entry.HotPathAbsent):
        entry.smoke()
