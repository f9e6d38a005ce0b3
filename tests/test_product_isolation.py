"""The shipped package never touches the oracle, the reference checkout or working files."""

import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_package_does_not_import_oracle_or_reference():
    pattern = re.compile(r"^\s*(from|import)\s+(oracle|oal_attention|_work)\b", re.M)
    for path in (ROOT / "oal_b200").rglob("*.py"):
        text = path.read_text()
        assert not pattern.search(text), f"{path} imports test infrastructure"
        assert "/root/" + "reference" not in text, f"{path} names the reference checkout"


def test_runtime_files_do_not_read_reference_checkout():
    for name in ("bench.py", "__graft_entry__.py"):
        assert "/root/" + "reference" not in (ROOT / name).read_text()
    marker = "/root/" + "reference"
    for path in (ROOT / "tests").glob("test_*.py"):
        assert marker not in path.read_text(), path


def test_no_torch_fallback_ops_in_kernel_sources():
    """No vendor GEMM or alternative backend in the CUDA sources."""
    for path in (ROOT / "oal_b200" / "csrc").glob("*.cu*"):
        text = path.read_text()
        assert "cublas" not in text.lower() or "hd_cublas_compat" in text, path
        assert "#include <torch" not in text, path
