"""Where the sequences of a packed ``[T, H, 128]`` tensor begin and end.

Everything is decided from the host copy of the cumulative lengths: reading the device copy would force a
synchronisation in the middle of a denoising step.  Behaviour of ``segments`` in
src/open_vc_attn/integrations/packed.py:4-19 of the reference, including the order in which faults are reported.
"""

from typing import NamedTuple


class Segment(NamedTuple):
    """Rows ``start:stop`` of the packed tensor; ``padding`` rows get zeros instead of attention."""

    start: int
    stop: int
    padding: bool


def _require(condition, message):
    if not condition:
        raise ValueError(message)


def segments(bounds, total, max_seqlen, *, trailing_padding=False):
    """Split ``total`` packed rows at the cumulative lengths ``bounds`` (host integers, ``bounds[0] == 0``).

    With ``trailing_padding`` a tensor of exactly two pieces whose first piece is ``max_seqlen`` long is one sequence
    followed by padding.  Returns a list of ``Segment`` (plain ``(start, stop, padding)`` tuples to a caller).
    """
    _require(bounds is not None, "cu_seqlens_host is required; CUDA metadata is not copied to CPU")
    edges = tuple(bounds)
    _require(
        len(edges) >= 2 and edges[0] == 0 and edges[-1] == total,
        "Packed bounds must start at zero and end at the tensor length",
    )
    ordered = all(isinstance(edge, int) for edge in edges) and all(
        left < right for left, right in zip(edges[:-1], edges[1:])
    )
    _require(ordered, "Packed bounds must be strictly increasing integers")

    pieces = [Segment(left, right, False) for left, right in zip(edges[:-1], edges[1:])]
    if trailing_padding and len(pieces) == 2 and pieces[0].stop == max_seqlen:
        pieces[1] = pieces[1]._replace(padding=True)
    longest = max((piece.stop - piece.start for piece in pieces if not piece.padding), default=0)
    _require(max_seqlen >= 1 and longest <= max_seqlen, "max_seqlen is inconsistent with packed bounds")
    return pieces
