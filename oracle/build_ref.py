"""Recipe for ``oracle/_ref/``: the reference's own CPU implementation of the path, unmodified.

TEST INFRASTRUCTURE ONLY (see ``oracle/gdr_oracle.py``).  Run where the reference checkout is
present:

    python oracle/build_ref.py /path/to/reference

It copies, byte for byte, the reference's pure-PyTorch implementation ``tests/ref_gdr.py`` and
the two helper files its imports come from (``flash_qla/utils/pack.py``: ``pad_and_reshape``,
``pack``, ``unpack``, ``fill_last_chunk_of_g``; ``flash_qla/utils/index.py``:
``prepare_chunk_offsets``) into ``oracle/_ref/``.  That folder is listed in ``.gitignore``: the
copies never enter the history of this repository, they only travel next to it like other build
products, so that the CPU baseline of ``bench.py`` can time the reference's code itself
(``cpu_baseline.kind = "reference"``) on machines where the checkout is absent.
``oracle/ref_loader.py`` imports what was copied.
"""

from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
FILES = {
    "tests/ref_gdr.py": "ref_gdr.py",
    "flash_qla/utils/pack.py": "pack.py",
    "flash_qla/utils/index.py": "index.py",
}


def build(ref_root: str) -> str:
    os.makedirs(DEST, exist_ok=True)
    for src, dst in FILES.items():
        shutil.copyfile(os.path.join(ref_root, src), os.path.join(DEST, dst))
    return DEST


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else "/root/reference"))
