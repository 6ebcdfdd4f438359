"""Stage the reference's own CPU implementation of the hot path next to the oracle.

TEST / BENCHMARK INFRASTRUCTURE ONLY.  The reference's pytorch backend
(``src/cute_prism/_pytorch_backend.py``: ``pytorch_forward`` lines 78-176, ``pytorch_backward``
lines 179-321) is one self-contained Python file (torch + einops).  Where the reference tree is
present this script copies that file, unmodified, to ``oracle/_ref/cute_prism_pytorch_backend.py``.
``oracle/_ref/`` is git-ignored, so the reference's source never enters the history, but it travels
with the working tree to the GPU box, where ``bench.py --impl reference`` and the ``cpu_baseline``
leg time it on the host cores (``kind: "reference"``); without it they time the oracle port.

    python oracle/stage_ref.py [/path/to/reference]
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref", "cute_prism_pytorch_backend.py")


def stage(reference_root: str = "/root/reference") -> bool:
    src = os.path.join(reference_root, "src", "cute_prism", "_pytorch_backend.py")
    if not os.path.exists(src):
        return False
    os.makedirs(os.path.dirname(DEST), exist_ok=True)
    shutil.copyfile(src, DEST)
    return True


if __name__ == "__main__":
    ok = stage(*sys.argv[1:2])
    print("staged" if ok else "reference tree not found: nothing staged", DEST if ok else "")
