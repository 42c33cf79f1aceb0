"""Small dense stack used by the module microbenchmark (reference
implementation/module_dev.py:5-23): three SwiGLU feed-forward layers of width
14336."""
import torch.nn as nn

from .layers import PositionWiseFFLayer


class ModuleStack(nn.Module):
    def __init__(self, d_model: int = 4096, d_out: int = 4096, d_ff: int = 14336, device=None, dtype=None):
        super().__init__()
        self.layers = nn.Sequential(*[PositionWiseFFLayer(d_model, d_ff, device=device, dtype=dtype)
                                      for _ in range(3)])
        if dtype is not None:
            self.to(dtype)
        if device is not None:
            self.to(device)

    def forward(self, x):
        return self.layers(x)
