import torch

from . import ops as ops
from .aok_grouped_gemm import AokGroupedGemm as AokGroupedGemm
from .ffn import GemmExecutor as GemmExecutor
from .ffn import SharedExperts as SharedExperts
from .ffn import batched_gemm_fp8 as batched_gemm_fp8
from .ffn import dense_gemm_fp8 as dense_gemm_fp8
from .ffn import dense_silu as dense_silu
from .silu import silu as silu

# The reference imports AokGroupedGemm on Hopper (capability 9.0) only; this build is for Blackwell (10.0).
IS_BLACKWELL = torch.cuda.is_available() and torch.cuda.get_device_capability(torch.cuda.current_device())[0] == 10
