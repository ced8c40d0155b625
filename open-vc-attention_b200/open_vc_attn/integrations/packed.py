"""Validation of packed-sequence bounds on the host (no device synchronisation).

Same contract as src/open_vc_attn/integrations/packed.py of the reference.
"""


def segments(bounds, total, max_seqlen, *, trailing_padding=False):
    """Turn host-side cumulative bounds into ``(start, stop, is_padding)`` triples.

    ``bounds`` must start at 0, end at ``total`` and increase strictly.  With ``trailing_padding`` a
    two-segment layout whose first segment is exactly ``max_seqlen`` long marks the second as padding.
    """
    if bounds is None:
        raise ValueError("cu_seqlens_host is required; CUDA metadata is not copied to CPU")
    bounds = tuple(bounds)
    if len(bounds) < 2 or bounds[0] != 0 or bounds[-1] != total:
        raise ValueError("Packed bounds must start at zero and end at the tensor length")
    if not all(isinstance(x, int) for x in bounds) or not all(a < b for a, b in zip(bounds, bounds[1:])):
        raise ValueError("Packed bounds must be strictly increasing integers")
    pieces = [(a, b, False) for a, b in zip(bounds, bounds[1:])]
    if trailing_padding and len(bounds) == 3 and bounds[1] == max_seqlen:
        pieces[-1] = (bounds[1], bounds[2], True)
    if max_seqlen < 1 or any(b - a > max_seqlen for a, b, pad in pieces if not pad):
        raise ValueError("max_seqlen is inconsistent with packed bounds")
    return pieces
