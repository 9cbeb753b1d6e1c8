from . import ops as ops
