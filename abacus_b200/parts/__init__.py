from .base import BLOCKS, FEED_FORWARDS, FRAMES, MIXERS, NORMS, POSITIONS, BuildContext, Registry
from .workspace import Workspace
from .linear import Linear
from . import attention, block, delta, frame, latent, lightning, memory, mlp, moe, norm, position, side_by_side, streams, wkv  # noqa: F401  (register the built-in parts)

__all__ = ["BLOCKS", "FEED_FORWARDS", "FRAMES", "MIXERS", "NORMS", "POSITIONS", "BuildContext", "Registry", "Workspace", "Linear"]
