from . import ops as ops
from .all_to_all import AllToAll as AllToAll
