from .auto import AutoConfig, AutoModelForCausalLM, AutoModelForCausalLMPipe, AutoProcessor, AutoTokenizer  # noqa: F401
from .configuration_utils import LlmMetaConfig, PretrainedConfig  # noqa: F401
