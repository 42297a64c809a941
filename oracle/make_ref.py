"""Installs the UNMODIFIED reference package into ``oracle/_ref/`` (git-ignored).

TEST INFRASTRUCTURE ONLY.  The reference is pure Python; where its source tree
is mounted this recipe installs it, as it is, with pip into ``oracle/_ref`` so
that the installed copy travels with the working tree to machines that do not
mount the reference.  Tests, ``__graft_entry__.smoke()`` and the CPU legs of
``bench.py`` import it from there (``oracle.ref.load()``); nothing under
``whisperdrz_b200/`` does.  No reference source is committed: ``oracle/_ref/``
is listed in ``.gitignore``.

    python oracle/make_ref.py [<reference checkout>]

The install is ``pip install --no-index --no-deps --no-build-isolation --target
oracle/_ref <copy of the checkout>`` (a copy, because the build writes an
egg-info directory into the source tree and the mount is read-only).  When pip
cannot build the wheel offline, the package directory ``src/whisperdrz`` is
copied verbatim instead, which gives the same importable files.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
DEFAULT_SRC = os.environ.get("WHISPERDRZ_REFERENCE", "/root/reference")


def install(src: str = DEFAULT_SRC, force: bool = False) -> str | None:
    """Returns the install directory, or None when no reference checkout is mounted."""
    marker = os.path.join(DEST, "whisperdrz", "__init__.py")
    if os.path.exists(marker) and not force:
        return DEST
    if not os.path.isdir(os.path.join(src, "src", "whisperdrz")):
        return None
    if os.path.isdir(DEST):
        shutil.rmtree(DEST)
    os.makedirs(DEST)
    with tempfile.TemporaryDirectory() as tmp:
        work = os.path.join(tmp, "reference")
        shutil.copytree(src, work, ignore=shutil.ignore_patterns("__pycache__", ".git"))
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-deps", "--no-build-isolation",
               "--quiet", "--target", DEST, work]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0 or not os.path.exists(marker):
            sys.stderr.write("pip install of the reference failed, copying the package directory instead:\n"
                             + r.stderr[-800:] + "\n")
            if os.path.isdir(DEST):
                shutil.rmtree(DEST)
            os.makedirs(DEST)
            shutil.copytree(os.path.join(work, "src", "whisperdrz"), os.path.join(DEST, "whisperdrz"),
                            ignore=shutil.ignore_patterns("__pycache__"))
    return DEST


if __name__ == "__main__":
    out = install(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_SRC, force=True)
    print(out or "no reference checkout found; nothing installed")
