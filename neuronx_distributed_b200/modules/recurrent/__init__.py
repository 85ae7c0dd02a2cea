"""Recurrent sequence mixers: layers whose memory of the past is a fixed-size state carried from token to token (float), served by
the scan kernels of ``csrc/seqmix/linear_recurrence.cu``."""
from .gla import GatedLinearAttention  # noqa: F401
from .rglru import RealGatedLRUBlock  # noqa: F401
