"""Implementation constants (src/open_vc_attn/_dispatch.py of the reference).

There is one implementation: the hand-written sm_100a kernels in libovc.so.  The reference's
second backend (the FlashAttention-4 BF16 kernel selected by version="reference") is not part of
this build and asking for it raises.
"""

DEFAULT_VERSION = "open-vc"
DEFAULT_MID_WINDOW_BLOCKS = 4
VERSIONS = (DEFAULT_VERSION,)


def require_version(version):
    if version == "reference":
        raise ValueError(
            'version="reference" (the FlashAttention-4 BF16 backend) is not available in this build; '
            f"use version={DEFAULT_VERSION!r}"
        )
    if version != DEFAULT_VERSION:
        raise ValueError(f"Unknown implementation {version!r}; choose from {VERSIONS}")
