from b200moe.models.layers import *  # noqa: F401,F403
from b200moe.models.transformer import TransformerLM, TransformerLMPipelined  # noqa: F401
