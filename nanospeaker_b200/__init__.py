"""B200-native dropless MoE block: a drop-in for nanoSpeaker's `MoEBlock` whose GPU path is
hand-written sm_100a CUDA (tcgen05/TMEM grouped GEMMs fed by TMA, warp-level routing kernels)
behind a C ABI (include/moe_b200.h, nanospeaker_b200/libmoe_b200.so)."""
from .glu import glu_hidden_dim, make_glu
from .moe import AUTO_CAPACITY, MoEBlock
from .moe_kernel import (ALIGN_M, KERNEL_ACTIVATIONS, KERNEL_DTYPES, fused_moe_forward,
                         kernel_supported, moe_dispatch, moe_experts, router_topk,
                         shapes_supported)
from .expert_parallel import ep_block_forward, expert_partition
from .graphed import GraphedMoEBlock
from .muon import Muon, newton_schulz5
from .router import TopKRouter
from .sublayer import MoEFFNSublayer
from .utils import ACTIVATIONS, resolve_activation

__all__ = [
    "MoEBlock", "GraphedMoEBlock", "Muon", "newton_schulz5", "MoEFFNSublayer", "TopKRouter", "AUTO_CAPACITY", "ALIGN_M", "KERNEL_ACTIVATIONS", "KERNEL_DTYPES",
    "fused_moe_forward", "kernel_supported", "shapes_supported", "moe_dispatch", "moe_experts",
    "router_topk", "ep_block_forward", "expert_partition", "glu_hidden_dim", "make_glu", "ACTIVATIONS", "resolve_activation",
]
