"""gdn_chunk forward for NVIDIA B200 (sm_100a): TMA + tcgen05/TMEM kernels behind a C ABI."""

from .gdn_chunk_interface import (
    GDN_CHUNK,
    GDN_D,
    gdn_chunk,
    gdn_chunk_host,
    gdn_chunk_reference,
    gdn_chunk_twolevel,
    gdn_chunk_varlen,
    rmsnorm_gated,
)

__version__ = "0.1.0"
__all__ = ["rmsnorm_gated", "gdn_chunk_varlen", "gdn_chunk", "gdn_chunk_host", "gdn_chunk_twolevel", "gdn_chunk_reference", "GDN_D", "GDN_CHUNK"]
