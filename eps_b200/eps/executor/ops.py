"""Loads libexecutor_.so from this directory and exposes its operators as `_ops` (reference python/eps/executor/ops.py)."""
import logging
import os

import torch

_lib_path = os.path.join(os.path.dirname(__file__), "libexecutor_.so")
try:
    torch.ops.load_library(_lib_path)
    _ops = torch.ops.executor
except OSError as e:
    logging.exception(f"Error loading executor: {e}")
    raise
