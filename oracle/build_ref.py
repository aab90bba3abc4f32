"""Stage the reference's own CPU implementation of the KDA path beside the oracle.

TEST / BASELINE INFRASTRUCTURE ONLY, like everything under ``oracle/``.

The reference is pure Python: its eager PyTorch implementation of ``chunk_kda`` / ``recurrent_kda``
(``impl="reference"``: attn_gym/linear/kda/naive.py, attn_gym/linear/kda/impl/reference.py) runs on
CPU cores with nothing but torch.  This script copies the ``attn_gym`` package, unmodified, from a
checkout of the reference into ``oracle/_ref/`` (kept out of version control), so that the
benchmark's reference arm and CPU baseline can time the reference itself where that folder
exists, and fall back to the restatement in ``kda_oracle.py`` where it does not.

    python oracle/build_ref.py path/to/reference/checkout

Nothing here is imported by the shipped library.
"""

from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def build_ref(source: str) -> str | None:
    """Copy <source>/attn_gym to oracle/_ref/attn_gym; returns the destination or None if the
    checkout is not there."""
    package = os.path.join(source, "attn_gym")
    if not os.path.isdir(package):
        return None
    target = os.path.join(DEST, "attn_gym")
    if os.path.isdir(target):
        shutil.rmtree(target)
    os.makedirs(DEST, exist_ok=True)
    shutil.copytree(package, target, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return target


def load_reference_chunk_kda():
    """The reference's ``chunk_kda`` from oracle/_ref, or None when it is not staged or does not
    import on this machine."""
    if not os.path.isdir(os.path.join(DEST, "attn_gym")):
        return None
    if DEST not in sys.path:
        sys.path.insert(0, DEST)
    try:
        from attn_gym.linear.kda import chunk_kda  # type: ignore
    except Exception:  # noqa: BLE001  (any import problem means: use the port)
        return None
    return chunk_kda


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(build_ref(sys.argv[1]) or "no reference checkout found there; nothing staged")
