from .layers import *  # noqa: F401,F403
from .transformer import TransformerLM, TransformerLMPipelined, default_d_ff  # noqa: F401
from .module_dev import ModuleStack  # noqa: F401
