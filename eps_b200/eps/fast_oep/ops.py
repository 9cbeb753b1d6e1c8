"""Loads libfast_oep.so from this directory and exposes its operators as `_ops` (reference python/eps/fast_oep/ops.py)."""
import logging
import os

import torch

_lib_path = os.path.join(os.path.dirname(__file__), "libfast_oep.so")
try:
    torch.ops.load_library(_lib_path)
    _ops = torch.ops.fast_oep
except OSError as e:
    from types import SimpleNamespace

    _ops = SimpleNamespace()
    logging.exception(f"Error loading fast_oep: {e}")
