"""Re-checks the finding this repository rests on: the reference project
(bat0001/peer-review-agents) contains no Expert-Threshold MoE token-routing
code -- no threshold router, CSR build, CSR scatter/gather, balanced
permutation, expert-parallel dispatch/combine or weighted combine -- and so no
oracle, no drop-in boundary and no CPU baseline can be derived from it.

Three groups of tests:

* the scan of the reference itself, run only where a checkout is present (the
  directory named by ``$REFERENCE_ROOT``, else a directory called ``reference``
  beside this repository); it starts with the tree's fingerprint, so a
  different reference announces itself before any other assertion;
* the scanner turned on scratch trees that *do* hide something, to show it is
  not blind (these need no reference);
* the state of this repository while the path is recorded absent and the
  operator has recorded no decision: nothing poses as product or oracle, and
  the entry points report "unavailable" rather than a number.
"""

import json
import os
import pathlib
import shutil
import subprocess
import sys

import pytest

import reference_scan as scan

REPO = pathlib.Path(__file__).resolve().parent.parent
REFERENCE = pathlib.Path(os.environ.get("REFERENCE_ROOT") or REPO.parent / "reference")

needs_reference = pytest.mark.skipif(
    not (REFERENCE / "cli" / "reva").is_dir(), reason="reference checkout not present"
)

STALE = (
    "reference tree changed - the absence finding is stale; "
    "redo the survey before anything else"
)


def _verification():
    return json.loads((REPO / "BASELINE.json").read_text())["hot_path_verification"]


def _stopped():
    """True while the path is recorded absent and no operator decision is on record.

    The only channel for that decision is BASELINE.json
    (``hot_path_verification.operator_decision``, or ``status`` itself).
    """
    v = _verification()
    return v["status"] == "absent" and not v.get("operator_decision")


while_stopped = pytest.mark.skipif(
    not _stopped(),
    reason="BASELINE.json no longer records the path as absent and undecided; "
    "the stopped-state checks do not apply",
)


# --------------------------------------------------------------------------
# 1. The reference itself
# --------------------------------------------------------------------------

@needs_reference
def test_reference_is_the_tree_that_was_verified():
    recorded = _verification()["reference_fingerprint"]
    found = scan.fingerprint(REFERENCE)
    assert found["file_count"] == recorded["file_count"], STALE
    assert found["sha256"] == recorded["sha256"], STALE


@needs_reference
def test_reference_has_no_native_or_kernel_files():
    assert scan.native_files(REFERENCE) == []
    assert not (REFERENCE / ".gitmodules").exists()
    assert scan.symlinks(REFERENCE) == []


@needs_reference
def test_every_reference_file_is_readable_text():
    """No file escapes the text search by not being text."""
    assert set(scan.undecodable_files(REFERENCE)) <= scan.UNDECODABLE_ALLOWED


@needs_reference
def test_reference_has_no_routing_or_tensor_code():
    hits = set(scan.text_hits(REFERENCE))
    assert hits <= scan.UNRELATED_TEXT_MATCHES, sorted(hits - scan.UNRELATED_TEXT_MATCHES)
    assert scan.name_hits(REFERENCE) == []


@needs_reference
def test_reference_declares_no_numeric_dependency():
    import re

    numeric = re.compile(r"^name = \"(torch|triton|numpy|jax|jaxlib|cupy.*|nvidia-.*|cuda-.*)\"", re.M)
    assert numeric.findall((REFERENCE / "uv.lock").read_text()) == []
    # declared dependencies: cli/pyproject.toml:21-28, pyproject.toml:6-8
    for toml in ("pyproject.toml", "cli/pyproject.toml"):
        assert not re.search(r"torch|triton|numpy|jax|cupy", (REFERENCE / toml).read_text(), re.I)


@needs_reference
@pytest.mark.parametrize(
    "name, payload",
    [
        ("x.bin", b"\x00\x01\x02\xff\xfe"),                   # opaque blob, listed suffix
        ("notes/blob.dat", b"\x93NUMPY\x01\x00\xff\xfe\x00"),  # opaque blob, unlisted suffix
        ("moe_router.txt", b"nothing to see\n"),               # innocent text, telling name
        ("cli/reva/extra.py", b"import torch\n"),              # telling text, innocent name
        ("vendor/src.tar.gz", b"\x1f\x8b\x08\x00"),            # archive with a double suffix
    ],
)
def test_a_payload_added_to_the_reference_is_caught(tmp_path, name, payload):
    """A copy of the reference with one file slipped in must fail the scan and the fingerprint."""
    tree = tmp_path / "reference"
    shutil.copytree(REFERENCE, tree)
    target = tree / name
    target.parent.mkdir(parents=True, exist_ok=True)
    target.write_bytes(payload)

    assert scan.fingerprint(tree)["sha256"] != _verification()["reference_fingerprint"]["sha256"]
    flagged = (
        set(scan.native_files(tree))
        | (set(scan.undecodable_files(tree)) - scan.UNDECODABLE_ALLOWED)
        | (set(scan.text_hits(tree)) - scan.UNRELATED_TEXT_MATCHES)
        | set(scan.name_hits(tree))
    )
    assert name in flagged


# --------------------------------------------------------------------------
# 2. The scanner on scratch trees (no reference needed)
# --------------------------------------------------------------------------

def _scratch(tmp_path, entries):
    root = tmp_path / "tree"
    for name, data in entries.items():
        p = root / name
        p.parent.mkdir(parents=True, exist_ok=True)
        p.write_bytes(data)
    return root


def test_scanner_passes_a_plain_text_tree(tmp_path):
    root = _scratch(tmp_path, {"a.py": b"print('hi')\n", "docs/b.md": "café\n".encode()})
    assert scan.native_files(root) == []
    assert scan.undecodable_files(root) == []
    assert scan.text_hits(root) == []
    assert scan.name_hits(root) == []
    assert scan.fingerprint(root)["file_count"] == 2


def test_scanner_reports_files_it_cannot_read_as_text(tmp_path):
    root = _scratch(tmp_path, {
        "ok.txt": b"fine\n",
        "latin1.txt": "café".encode("latin-1"),
        "nul.txt": b"abc\x00def",
    })
    assert scan.undecodable_files(root) == ["latin1.txt", "nul.txt"]


@pytest.mark.parametrize("name", [
    "k.cu", "w.safetensors", "a.npz", "a.npy", "m.pkl", "e.pyx", "l.pyd", "o.o",
    "s.tgz", "s.tar.bz2", "s.xz", "s.7z", "b.BIN",
])
def test_scanner_flags_native_binary_and_archive_suffixes(tmp_path, name):
    assert scan.native_files(_scratch(tmp_path, {name: b"x"})) == [name]


@pytest.mark.parametrize("name", [
    "moe_router.txt", "csr_build.md", "ops/all_to_all.txt", "Expert/readme", "topk.txt",
    "balanced_permutation.rst", "kernels/readme",
])
def test_scanner_matches_terms_in_file_and_directory_names(tmp_path, name):
    assert name in scan.name_hits(_scratch(tmp_path, {name: b"plain\n"}))


def test_scanner_matches_terms_in_text_even_in_partly_invalid_files(tmp_path):
    root = _scratch(tmp_path, {"half.txt": b"\xff\xfe import triton \xff"})
    assert scan.text_hits(root) == ["half.txt"]
    assert scan.undecodable_files(root) == ["half.txt"]


def test_fingerprint_changes_with_content_name_and_count(tmp_path):
    base = scan.fingerprint(_scratch(tmp_path / "0", {"a": b"1", "b": b"2"}))
    assert scan.fingerprint(_scratch(tmp_path / "1", {"a": b"1", "b": b"2"})) == base
    assert scan.fingerprint(_scratch(tmp_path / "2", {"a": b"1", "b": b"3"})) != base
    assert scan.fingerprint(_scratch(tmp_path / "3", {"a": b"1", "c": b"2"})) != base
    assert scan.fingerprint(_scratch(tmp_path / "4", {"a": b"1", "b": b"2", "c": b""})) != base
    # a path cannot be confused with content: "a\0..." boundaries are part of the digest
    assert scan.fingerprint(_scratch(tmp_path / "5", {"ab": b"", "c": b""})) != \
        scan.fingerprint(_scratch(tmp_path / "6", {"a": b"", "bc": b""}))


# --------------------------------------------------------------------------
# 3. This repository while the path is recorded absent and undecided
# --------------------------------------------------------------------------

def _ignored_directories():
    """Directory names the repository's ignore file excludes from history."""
    names = set()
    for line in (REPO / ".gitignore").read_text().splitlines():
        line = line.strip()
        if line and not line.startswith("#") and line.endswith("/"):
            names.add(line.strip("/").split("/")[-1])
    return names | {".git"}


@while_stopped
def test_baseline_records_the_absence():
    v = _verification()
    assert v["module_path"] is None
    assert v["python_entry_points"] == []
    assert v["reference_fingerprint"]["file_count"] > 0
    assert len(v["reference_fingerprint"]["sha256"]) == 64


@while_stopped
def test_no_kernel_or_oracle_was_invented():
    """While the path is recorded absent, nothing here may pose as its product or oracle."""
    skip = _ignored_directories()
    for pattern in ("**/*.cu", "**/*.cuh", "oracle/**/*", "include/*.h"):
        found = [p for p in REPO.glob(pattern) if not skip & set(p.relative_to(REPO).parts)]
        assert found == [], found


@while_stopped
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


@while_stopped
def test_bench_non_zero_ranks_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run(
        [sys.executable, str(REPO / "bench.py"), "--gpus", "2"],
        capture_output=True, text=True, timeout=120, env=env, check=True,
    )
    assert r.stdout.strip() == ""


@while_stopped
def test_entry_points_state_that_nothing_is_built(capsys):
    sys.path.insert(0, str(REPO))
    try:
        import __graft_entry__ as entry
    finally:
        sys.path.pop(0)
    entry.build()  # nothing to compile; must not raise
    capsys.readouterr()
    with pytest.raises(entry.HotPathAbsent):
        entry.smoke()
    # a stopped build is told apart from a broken one by one JSON status line
    status = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert status["status"] == "stopped"
    assert status["gpu_launches"] == 0
    assert status["reason"]
