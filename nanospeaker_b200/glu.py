"""GLU width rule and the pointwise GLU body (src/model/glu.py:16-47)."""
from .utils import Activation


def glu_hidden_dim(d_ff: int) -> int:
    """Hidden width of a GLU that replaces a d_ff-wide FFN at equal parameter count: 2*d_ff//3."""
    d_hidden = 2 * d_ff // 3
    if d_hidden < 1:
        raise ValueError(f"d_ff ({d_ff}) is too small: 2/3 * d_ff rounds down to {d_hidden}.")
    return d_hidden


def make_glu(act: Activation, fused: bool = True, dynamic=True):
    """(gate, up) -> act(gate) * up for the eager (non-kernel) path.

    `fused` and `dynamic` are accepted for signature compatibility; the CUDA path applies the GLU
    inside the up/gate GEMM epilogue, so nothing is compiled here.
    """
    def glu(gate, up):
        return act(gate) * up

    return glu
