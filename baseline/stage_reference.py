"""Stage the reference's model runtime for the drop-in test: copies `model_hub/` and `config/` of the reference
checkout, unmodified, into `baseline/_ref/` (kept out of version control).  The GPU test
`tests/test_gpu_model_hub.py` decodes through that unchanged runtime with this package installed under the
reference's module names (`pariskv_b200.dropin`).

    python baseline/stage_reference.py [path to the reference checkout]
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def stage(reference_root: str) -> bool:
    """Returns True when the runtime is in place (freshly copied or already there)."""
    if not os.path.isdir(os.path.join(reference_root, "model_hub")):
        return os.path.isdir(os.path.join(DEST, "model_hub"))
    os.makedirs(DEST, exist_ok=True)
    for sub in ("model_hub", "config"):
        src, dst = os.path.join(reference_root, sub), os.path.join(DEST, sub)
        if os.path.isdir(src):
            if os.path.isdir(dst):
                shutil.rmtree(dst)
            shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__"))
    return True


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    print("staged" if stage(root) else "reference checkout not found; nothing staged")
