from . import qwen2  # noqa: F401  (registers Qwen2ForCausalLM)
from .decoder import DecoderModel
