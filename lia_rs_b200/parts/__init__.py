from .base import (ARRANGEMENTS, FEED_FORWARDS, JUNCTIONS, MIXERS, NORMS, POSITION_ENCODINGS, Arrangement, FeedForward,
                   Junction, KVCacheRequest, Mixer, Norm, Part, PartSpec, PositionEncoding, Runtime, StateRequest,
                   lookup, register_arrangement, register_feed_forward, register_junction, register_mixer, register_norm,
                   register_position_encoding)
from . import norm, rotary, attention, sigmoid_attention, softmax_attention, selective_scan, retention, gated_linear_attention, side_by_side, feed_forward, moe, block, hyper_connections, junction  # noqa: F401  (register the built-in parts)
from .block import LayerSpec, build_layer, check_layer, layer_tensor_specs

__all__ = ["ARRANGEMENTS", "FEED_FORWARDS", "JUNCTIONS", "Junction", "register_junction", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Arrangement",
           "FeedForward", "KVCacheRequest", "Mixer", "Norm", "Part", "PartSpec", "PositionEncoding",
           "Runtime", "StateRequest", "lookup", "register_arrangement", "register_feed_forward",
           "register_mixer", "register_norm", "register_position_encoding", "LayerSpec", "build_layer", "check_layer",
           "layer_tensor_specs"]
