"""Access to the unmodified reference package installed by ``oracle/make_ref.py``.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, ``__graft_entry__.smoke()``
and the CPU legs of ``bench.py``; never by the ``whisperdrz_b200`` package.
"""
from __future__ import annotations

import importlib
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def available() -> bool:
    return os.path.exists(os.path.join(REF_DIR, "whisperdrz", "__init__.py"))


def load():
    """Imports and returns the reference's top-level module (``whisperdrz``), or None when it was
    never installed here."""
    if not available():
        return None
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    return importlib.import_module("whisperdrz")


def model(dims, state_dict, dtype=None):
    """A reference ``WhisperDRZ`` (src/whisperdrz/model.py) of the given dimensions carrying ``state_dict``
    (fp32, eval mode), or None without the reference."""
    if load() is None:
        return None
    import torch
    from whisperdrz.config import Config, ModelDimensions as RefDims
    from whisperdrz.model import WhisperDRZ
    m = WhisperDRZ(RefDims(**dims.as_dict()), config=Config()).float().eval()
    missing, unexpected = m.load_state_dict(state_dict, strict=False)
    assert not unexpected, unexpected
    assert all("speaker" in k or "timing" in k for k in missing), missing
    return m if dtype is None else m.to(dtype)
