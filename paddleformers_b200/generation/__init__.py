from .utils import GenerationConfig, GenerationMixin, KVCache, generate  # noqa: F401
