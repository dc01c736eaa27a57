from . import attention, block, embedding, feed_forward, head, norm, rope  # registers the built-in parts
from .base import MODES, Mixer, Part, Prenormed, RunContext, Runtime, as_delta
from .linear import linear
from .registry import build_part, known_parts, register_part, unregister_part
