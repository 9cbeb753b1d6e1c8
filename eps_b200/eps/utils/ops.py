"""Loads libutils_.so from this directory and exposes its operators as `_ops` (reference python/eps/utils/ops.py)."""
import logging
import os

import torch

_lib_path = os.path.join(os.path.dirname(__file__), "libutils_.so")
try:
    torch.ops.load_library(_lib_path)
    _ops = torch.ops.utils
except OSError as e:
    from types import SimpleNamespace

    _ops = SimpleNamespace()
    logging.exception(f"Error loading utils: {e}")
