"""Callers of ``attention`` for serving frameworks: a dense / packed diffusion adapter and, where the ``sglang``
package is installed, its backend registration (``integrations/`` of the reference, rebuilt on this package)."""

from .diffusion import DenseDiffusionAdapter
from .packed import Segment, segments

__all__ = ["DenseDiffusionAdapter", "Segment", "segments"]
