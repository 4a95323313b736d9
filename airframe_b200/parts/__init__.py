"""Parts of a layer and their registry; importing the package registers the
built-in kinds."""
from .base import (CATEGORIES, Block, BuildContext, FeedForward, Junction, KVNeed, Mixer, Norm, Part,
                   PositionEncoding, StateNeed, build_part, known_parts, register_part,
                   unregister_part)
from . import (attention, block, diff_attention, ends, hyper, junction, latent_attention, mlp, norm, parallel,  # noqa: F401
               recurrent, rope)  # noqa: F401  (registration)
from .linear import linear

__all__ = ["CATEGORIES", "Block", "BuildContext", "FeedForward", "Junction", "KVNeed", "Mixer", "Norm", "Part",
           "PositionEncoding", "StateNeed", "build_part", "known_parts", "register_part",
           "unregister_part", "linear"]
