from . import attention, feed_forward, norm, position  # noqa: F401  (register the built-in kinds)
from .base import (BuildContext, GroupView, LayerCache, PagedKvNeed, StateNeed,  # noqa: F401
                   StepContext)
from .block import Block, DecoderModel  # noqa: F401
from .registry import build_part, known, register_part, unregister_part  # noqa: F401
from .specs import (AttentionSpec, LayerSpec, ModelSpec, MoeSpec, RmsNormSpec,  # noqa: F401
                    RopeSpec, RunEntry, SwiGluSpec)
