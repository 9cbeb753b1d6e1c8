"""Loads libcommunication_.so from this directory and exposes its operators as `_ops` (reference python/eps/communication/ops.py)."""
import logging
import os

import torch

_lib_path = os.path.join(os.path.dirname(__file__), "libcommunication_.so")
try:
    torch.ops.load_library(_lib_path)
    _ops = torch.ops.communication
except OSError as e:
    from types import SimpleNamespace

    _ops = SimpleNamespace()
    logging.exception(f"Error loading communication: {e}")
