from .decoder import Decoder, ModelSpec, LayerCall, CacheGroup
from . import llama
