"""Copies the reference's own golden vectors for the decode path into this folder.

Run once in a container that has the reference tree mounted:
    python tests/golden/import_reference_goldens.py /path/to/reference
The vectors (little-endian raw arrays + a JSON sidecar with shape and dtype) were produced by the
reference's tests/generate_golden.py (Python MLX, mx.random.seed(42)) and are consumed by its
src/tests/golden_test.zig.  Only the four primitives on the decode path are taken.
"""
import shutil
import sys
from pathlib import Path

NAMES = ["rmsnorm_input", "rmsnorm_output", "rope_input", "rope_output", "sdpa_q", "sdpa_k", "sdpa_v",
         "sdpa_output", "embedding_weight", "embedding_indices", "embedding_output"]

if __name__ == "__main__":
    src = Path(sys.argv[1]) / "src" / "tests" / "golden"
    dst = Path(__file__).resolve().parent
    for n in NAMES:
        for ext in (".bin", ".bin.json"):
            shutil.copyfile(src / (n + ext), dst / (n + ext))
    print("copied", len(NAMES), "vectors")
