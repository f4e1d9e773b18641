"""Models: the generic decoder and the architectures built on it."""
from .decoder import DecoderModel, Embedding, LMHead, ScheduleEntry
from .qwen2_moe import Qwen2MoeModel
