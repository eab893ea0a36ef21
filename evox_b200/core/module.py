"""State containers: every piece of algorithm state is a registered buffer or parameter, so
`state_dict()` / `load_state_dict()` is the checkpoint format, exactly as in the reference
(evox/core/module.py:22-94)."""

from __future__ import annotations

import torch
from torch import nn


def Parameter(value, dtype: torch.dtype | None = None, device: torch.device | None = None, requires_grad: bool = False):
    """A hyper-parameter: a 0-d (or any) tensor stored as a non-trainable `nn.Parameter`.

    Kernels read hyper-parameters straight from device memory, so changing one never needs a
    host synchronisation (reference: evox/core/module.py:22-45)."""
    data = value.to(dtype=dtype, device=device) if isinstance(value, torch.Tensor) else torch.as_tensor(value, dtype=dtype, device=device)
    return nn.Parameter(data, requires_grad=requires_grad)


def Mutable(value: torch.Tensor, dtype: torch.dtype | None = None, device: torch.device | None = None):
    """State that changes from one generation to the next, stored as an `nn.Buffer`
    (reference: evox/core/module.py:48-58)."""
    return nn.Buffer(value.to(dtype=dtype, device=device))


class ModuleBase(nn.Module):
    """Base of algorithms, problems, workflows and monitors. Always in inference mode;
    `eval()` is refused to avoid confusion with fitness evaluation (evox/core/module.py:61-83)."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.train(False)

    def eval(self):  # noqa: A003 - mirrors the reference's refusal
        raise AssertionError("`ModuleBase.eval()` shall never be invoked to prevent ambiguity.")
