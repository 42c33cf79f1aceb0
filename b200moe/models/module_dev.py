"""Small dense stack used by the module microbenchmark (reference
implementation/module_dev.py:5-23): three SwiGLU feed-forward layers of width
14336 named ``ffn1``..``ffn3`` (the names are the state-dict keys).  ``d_out`` is
accepted, as there, and not used: every layer maps ``d_in`` to ``d_in``."""
import torch.nn as nn

from .layers import PositionWiseFFLayer


class ModuleStack(nn.Module):
    def __init__(self, d_in: int = 4096, d_out: int = 4096, device=None, dtype=None, d_ff: int = 14336):
        super().__init__()
        self.ffn1 = PositionWiseFFLayer(d_in, d_ff, device=device, dtype=dtype)
        self.ffn2 = PositionWiseFFLayer(d_in, d_ff, device=device, dtype=dtype)
        self.ffn3 = PositionWiseFFLayer(d_in, d_ff, device=device, dtype=dtype)
        if dtype is not None:
            self.to(dtype)
        if device is not None:
            self.to(device)

    def forward(self, x):
        return self.ffn3(self.ffn2(self.ffn1(x)))
