"""Drop-in `eps` package: the import paths, classes and torch ops of the reference's python/eps, served by the
B200 (sm_100a) libraries of this repository.  Put the directory that holds this package on sys.path
(`<repo>/eps_b200`) and `from eps.scheduler import Scheduler`, `from eps.executor import AokGroupedGemm, silu`,
`from eps.fast_ep import AllToAll`, `from eps.communication import MscclppCommunicator` work as with the reference.
Each sub-package loads `lib<name>.so` from its own directory (reference python/eps/<pkg>/ops.py:9-11)."""
from . import communication as communication
from . import executor as executor
from . import fast_ep as fast_ep
from . import fast_oep as fast_oep
from . import scheduler as scheduler
from . import utils as utils

__all__ = ["communication", "executor", "fast_ep", "fast_oep", "scheduler", "utils"]
