"""Stage the reference's own Python sources into ``oracle/_ref/`` (git-ignored, never committed).

    python oracle/make_ref.py /path/to/reference

The staged tree is test infrastructure only.  It lets a GPU box, which has no checkout of the
reference, (1) run the reference's Triton attention ``fa_forward_colsum_fast_sub``
(stac/flash_attn_triton.py:900-1006) as the source of ``tests/golden/attention_ref.npz``,
(2) drive this library's managers from the reference's own callers
(causalvggt/layers/attention.py:113-161, causalvggt/models/aggregator.py:159-335,
stream_session.py:258-565) and (3) time the reference's CPU torch path as the baseline arm of
``bench.py``.  Nothing under ``stac_b200/`` imports it.
"""

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
PACKAGES = ("stac", "causalvggt")
FILES = ("stream_session.py", "model_wrapper.py")


def _only_python(_dir, names):
    return [n for n in names if n == "__pycache__" or (os.path.isfile(os.path.join(_dir, n))
                                                         and not n.endswith(".py"))]


def stage(reference_root, dest=DEST):
    """Copy the Python packages and the two driver modules; returns the destination."""
    if not os.path.isdir(os.path.join(reference_root, "stac")):
        raise FileNotFoundError(f"{reference_root} does not look like a checkout of the reference")
    os.makedirs(dest, exist_ok=True)
    for pkg in PACKAGES:
        target = os.path.join(dest, pkg)
        if os.path.isdir(target):
            shutil.rmtree(target)
        shutil.copytree(os.path.join(reference_root, pkg), target, ignore=_only_python)
    for f in FILES:
        shutil.copy2(os.path.join(reference_root, f), os.path.join(dest, f))
    return dest


def available(dest=DEST):
    return os.path.isfile(os.path.join(dest, "stac", "flash_attn_triton.py"))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    print(stage(sys.argv[1]))
