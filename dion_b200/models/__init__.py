from .gpt import GPT, GPTConfig, parallelize_gpt_model  # noqa: F401
from .llama import Llama, LlamaConfig, make_llama_param_groups, parallelize_llama_model  # noqa: F401
