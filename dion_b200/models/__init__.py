from .gpt import GPT, GPTConfig, parallelize_gpt_model  # noqa: F401
