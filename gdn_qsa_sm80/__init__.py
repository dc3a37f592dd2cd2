"""Drop-in import path: ``from gdn_qsa_sm80 import gdn_chunk`` resolves to the sm_100a
implementation in ``gdn_qsa_sm80_b200`` (same functional API as the reference package's
``gdn_qsa_sm80/__init__.py:3-7``; the reference's other operators are not part of this build)."""

from gdn_qsa_sm80_b200 import (  # noqa: F401
    GDN_CHUNK,
    GDN_D,
    gdn_chunk,
    gdn_chunk_host,
    gdn_chunk_reference,
    gdn_chunk_twolevel,
    gdn_chunk_varlen,
    rmsnorm_gated,
)

__all__ = ["rmsnorm_gated", "gdn_chunk_varlen", "gdn_chunk", "gdn_chunk_host", "gdn_chunk_twolevel", "gdn_chunk_reference"]
