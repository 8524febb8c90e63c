"""Process-wide quantisation settings (rounding mode and seed of the stochastic-rounding stream).

The reference has no such switch: its stand-alone quantizer rounds to nearest (cuda/src/quantization.cu:6-15) and its
fused forward GEMM truncates (cuda/src/iterator.h:155-164).  `reference` keeps exactly those per-call-site modes;
`nearest` and `stochastic` apply one mode everywhere.
"""
from __future__ import annotations

from ._lib import ROUND_NEAREST, ROUND_STOCHASTIC, ROUND_TRUNC

_state = {"rounding": "reference", "seed": 0, "share_quantized_inputs": False, "step_counter": None,
          "hub_block": 163840}


def set_rounding(mode: str = "reference", seed: int = 0) -> None:
    if mode not in ("reference", "nearest", "trunc", "stochastic"):
        raise ValueError(mode)
    _state["rounding"] = mode
    _state["seed"] = int(seed)


def get_rounding() -> str:
    return _state["rounding"]


def seed() -> int:
    return _state["seed"]


def mode_for(site: str) -> int:
    """Rounding mode for a call site: 'gemm_fwd' (the fused forward GEMM) or 'quantize' (everything else)."""
    r = _state["rounding"]
    if r == "reference":
        return ROUND_TRUNC if site == "gemm_fwd" else ROUND_NEAREST
    return {"nearest": ROUND_NEAREST, "trunc": ROUND_TRUNC, "stochastic": ROUND_STOCHASTIC}[r]


def share_quantized_inputs(enable: bool = True) -> None:
    """When on, consecutive QLinear layers that read the same activation tensor (HGT's q / k / v projections) share
    one absmax pass and one int8 copy of it instead of quantizing it once per layer.  The reference quantizes per
    layer (cuda/QLinear.py:28-35); with a deterministic rounding mode the results are bit-identical either way.
    The tensor is recognised by address, shape and autograd version counter, so writes that bypass the counter
    (`tensor.data`) are not seen; stochastic rounding never shares."""
    _state["share_quantized_inputs"] = bool(enable)
    if not enable:
        from .QLinear import clear_shared_input
        clear_shared_input()


def sharing_quantized_inputs() -> bool:
    return _state["share_quantized_inputs"]


def set_step_counter(counter) -> None:
    """A 1-element int64 CUDA tensor (or None) that the stochastic quantizers read on the device and add, shifted
    left by 32, to their per-call counter.  A loop that replays a captured CUDA graph increments it once per step
    (inside the graph: `counter.add_(1)`), so every replay draws new random numbers although the launch arguments
    are frozen; without it a replayed step repeats the rounding noise of the captured one."""
    if counter is not None:
        import torch
        assert counter.is_cuda and counter.dtype == torch.int64 and counter.numel() == 1
    _state["step_counter"] = counter


def step_counter():
    return _state["step_counter"]


def set_hub_block(side: int) -> None:
    """Largest side (rows and columns, rounded down to 128) of the dense hub region that graph_preprocess builds for
    the unweighted aggregation on large power-law graphs -- inside it only tiles dense enough to pay are taken; 0
    switches it off (every edge is gathered, as the reference's CSR SpMM does).  Results are bit-identical either
    way: the region's product is an exact int32 sum like the gathered one.  Applies to graphs preprocessed after
    the call."""
    if side < 0:
        raise ValueError(side)
    _state["hub_block"] = int(side)


def hub_block() -> int:
    return _state["hub_block"]
