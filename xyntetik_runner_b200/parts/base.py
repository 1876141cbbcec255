"""What every part of a layer looks like to the model that holds it.

A layer is put together from parts -- a mixer (attention here), a feed-forward,
norms, a position encoding -- arranged by a block.  A part takes all its sizes
and constants as constructor arguments, names the tensors it needs
(``tensors``), receives them (``bind``) and computes on the step's flat token
axis (``forward``).  No part knows which model it is in: the architecture's
builder chooses parts layer by layer and gives each its tensor-name prefix.

Registries map a kind name to a class, so that a configuration (or a test)
can choose a part by name and new kinds are added without touching this
package: ``register_mixer("my_kind", MyMixer)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from ..weights.loader import TensorSpec


class Part:
    """Something with named tensors."""
    prefix: str = ""
    # True when `forward` only launches kernels on the current stream with shapes that depend on the step's
    # sizes alone (no host reads of device data, no allocation): such a part may be captured in a CUDA graph.
    # The default is False, so a part that does not say so is always run plainly.
    graph_safe: bool = False

    def tensors(self) -> Dict[str, TensorSpec]:
        """Full tensor names (prefix included) this part reads, with shapes."""
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor], rt: "Runtime") -> None:
        """Receive the tensors (on the device, stored dtype) and prepare device-side constants."""

    def weight_bytes(self) -> int:
        """Bytes of weights a step reads from this part (for roofline accounting)."""
        return 0


@dataclass(frozen=True)
class Runtime:
    """What a part may need to know about the engine it runs in."""
    device: torch.device
    act_dtype: torch.dtype          # torch.bfloat16 (serving) or torch.float32 (true 32-bit path)
    page_size: int
    max_step_tokens: int
    max_requests: int


@dataclass(frozen=True)
class KVNeed:
    """A mixer that keeps keys and values per token: their geometry and how long they are needed."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None    # None: all keys; w: the last w keys


@dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps a fixed-size state per request (zeroed when a request gets the slot)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Norm(Part):
    def forward(self, ctx, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        """out[i] = norm(x[rows[i]]) (rows None: every row).  x is the float32 residual stream."""
        raise NotImplementedError


@dataclass(frozen=True)
class Rotary:
    """A position encoding that rotates pairs of query and key elements by angle = position * inv_freq[j]
    (src/model.c:3514-3532): everything the rotation kernels and a mixer need to know of it."""
    rotary_dim: int                        # leading elements of every head that are rotated (even; 0: none)
    inv_freq: Optional[torch.Tensor]       # float32 [rotary_dim / 2] on the device (None when rotary_dim is 0)
    pairing: str = "half"                  # "half": pair j = (j, j + rotary_dim/2); "adjacent": (2j, 2j + 1)
    mscale: float = 1.0                    # factor on every cosine and sine (src/model.c:283, 375)

    def __post_init__(self):
        if self.pairing not in ("half", "adjacent"):
            raise ValueError(f"pairing '{self.pairing}': choose half or adjacent")
        if self.rotary_dim % 2 or self.rotary_dim < 0:
            raise ValueError("rotary_dim must be even and not negative")


class PositionEncoding:
    """How positions enter a mixer.  Built once from the configuration; holds no model weights.

    The built-in mixer knows one family: rotations of query and key pairs, described by ``rotary()`` after
    ``prepare``.  A position encoding of another family (a bias on the scores, a scale on the query that depends
    on the position, learned vectors added to the embedding) needs a mixer or an embedding part written for it;
    it leaves ``rotary`` unimplemented and the built-in mixer refuses it by name."""

    def prepare(self, rt: Runtime) -> None:
        pass

    def rotary(self) -> Optional[Rotary]:
        """The rotation to apply to queries and keys, or None for no rotation at all."""
        raise NotImplementedError(f"{type(self).__name__} does not describe itself as a rotation of query and key pairs")


class Mixer(Part):
    """Mixes information between the tokens of a request (attention, or anything with state)."""

    def kv_need(self) -> Optional[KVNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor, lay) -> None:
        """h: normed input [n, width] in the activation dtype.  Adds the mixer's output into the
        float32 residual stream x.  `lay` (engine.model.LayerRuntime) says where this layer's cache
        and state are."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor) -> None:
        """Adds the feed-forward of h into the residual stream x."""
        raise NotImplementedError


class Block(Part):
    """The arrangement of a layer's parts around the residual stream."""
    mixer: Mixer

    def forward(self, ctx, x: torch.Tensor, lay) -> None:
        raise NotImplementedError


_REGISTRIES: Dict[str, Dict[str, type]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}}


def _register(family: str, name: str, cls: type, replace: bool) -> None:
    reg = _REGISTRIES[family]
    if name in reg and not replace:
        raise ValueError(f"{family} kind '{name}' is already registered")
    reg[name] = cls


def register_mixer(name, cls, replace=False): _register("mixer", name, cls, replace)
def register_feed_forward(name, cls, replace=False): _register("feed_forward", name, cls, replace)
def register_norm(name, cls, replace=False): _register("norm", name, cls, replace)
def register_position(name, cls, replace=False): _register("position", name, cls, replace)
def register_block(name, cls, replace=False): _register("block", name, cls, replace)


def make(family: str, kind: str, **params):
    """Build a part of `family` ("mixer", "feed_forward", "norm", "position", "block") by kind name."""
    try:
        cls = _REGISTRIES[family][kind]
    except KeyError:
        raise ValueError(f"unknown {family} kind '{kind}'; known: {sorted(_REGISTRIES[family])}") from None
    return cls(**params)


def kinds(family: str):
    return sorted(_REGISTRIES[family])
