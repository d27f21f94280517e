"""Gate-activation registry of the MoE block (same names as src/model/utils.py:10-40)."""
from typing import Callable, Tuple, Union

import torch
import torch.nn.functional as F

Activation = Callable[[torch.Tensor], torch.Tensor]

# name -> callable; "swish" is an alias of "silu" (SwiGLU), "gelu" gives GEGLU, "relu" ReGLU,
# "sigmoid" the original GLU.
ACTIVATIONS = {
    "silu": F.silu,
    "swish": F.silu,
    "gelu": F.gelu,
    "relu": F.relu,
    "sigmoid": torch.sigmoid,
    "tanh": torch.tanh,
}


def resolve_activation(activation: Union[str, Activation]) -> Tuple[str, Activation]:
    """(name, fn) for a registered name (case-insensitive) or a callable passed through.

    Unknown names raise ValueError, like src/model/utils.py:25-40.
    """
    if callable(activation):
        return getattr(activation, "__name__", "custom"), activation
    if isinstance(activation, str):
        key = activation.lower()
        if key in ACTIVATIONS:
            return key, ACTIVATIONS[key]
    raise ValueError(
        f"Unknown activation {activation!r}. Use a callable or one of: "
        f"{', '.join(sorted(ACTIVATIONS))}."
    )
