from .decoder import CacheLayout, DecoderModel

__all__ = ["CacheLayout", "DecoderModel"]
