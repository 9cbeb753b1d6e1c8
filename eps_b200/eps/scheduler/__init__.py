from . import ops as ops
from .scheduler import Scheduler as Scheduler
