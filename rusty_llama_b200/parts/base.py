"""The interfaces every part implements, and the registries that name them.

A model is put together from five families of parts:

  mixer          what mixes information across positions (attention here);
                 it may need cache storage and says so with `cache_need()`
  feed-forward   what acts on each position alone (a gated MLP here)
  norm           normalisation applied to the residual stream
  position       how positions reach the mixer (rotary here); owned by a mixer
  block          the arrangement of the above inside one layer (pre-norm here)

A part gets its sizes and constants from its `PartSpec.params` and nothing
else; no part knows which model it is in.  A new part is a subclass registered
under a new kind name; nothing in the library's files has to change for it.
The reference keeps the same seams as `Backend` trait methods
(src/backend/mod.rs:32-279) chosen by per-architecture predicates
(src/arch.rs:163-206).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Callable, Dict, Mapping, Optional, Tuple

import torch

from ..errors import ConfigError
from ..spec import PartSpec


# --------------------------------------------------------------------------- runtime
class Workspace:
    """Scratch tensors that live across steps and grow on demand.

    Kernels that need global memory beyond their inputs and outputs (the split
    partials of decode attention, the probabilities of the sampler) take it
    from here, so that a replayed CUDA graph always sees the same addresses.  A tensor that
    has to grow is replaced, but the old one is kept for good: graphs captured while it was
    current still write to its address when they are replayed."""

    def __init__(self, device: torch.device):
        self.device = device
        self._bufs: Dict[str, torch.Tensor] = {}
        self._retired: List[torch.Tensor] = []

    def get(self, name: str, numel: int, dtype: torch.dtype, zeroed: bool = False) -> torch.Tensor:
        """zeroed: the tensor starts as zeros and its users leave it as zeros (counters that the
        kernels reset themselves); such a name must always be asked for with zeroed=True."""
        buf = self._bufs.get(name)
        if buf is None or buf.numel() < numel or buf.dtype != dtype:
            if self.device.type == "cuda" and torch.cuda.is_current_stream_capturing():
                raise RuntimeError(f"workspace '{name}' would have to grow during graph capture")
            if buf is not None:
                self._retired.append(buf)
            make = torch.zeros if zeroed else torch.empty
            buf = make(max(numel, 1), dtype=dtype, device=self.device)
            self._bufs[name] = buf
        return buf


@dataclass
class Runtime:
    """Where and in which precision a model runs.

    dtype: torch.bfloat16 (the serving path) or torch.float32 (everything in
    true 32-bit: no tensor-core product, no reduced-precision matrix mode)."""

    device: torch.device
    dtype: torch.dtype
    workspace: Workspace

    @classmethod
    def create(cls, device, dtype) -> "Runtime":
        device = torch.device(device)
        if isinstance(dtype, str):
            try:
                dtype = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}[dtype]
            except KeyError:
                raise ConfigError(f"dtype '{dtype}' is neither bfloat16 nor float32") from None
        if dtype not in (torch.bfloat16, torch.float32):
            raise ConfigError(f"dtype {dtype} is neither bfloat16 nor float32")
        return cls(device, dtype, Workspace(device))


# --------------------------------------------------------------------------- parameters
@dataclass(frozen=True)
class ParamInfo:
    """One tensor a part expects in the checkpoint.

    kind "matrix": stored in the run's matrix type (bfloat16, or float32 on the
    32-bit path).  kind "vector": a tensor stored in 32-bit stays so; otherwise
    it follows the run.  kind "table": integers, kept as int32."""

    shape: Tuple[int, ...]
    kind: str = "matrix"


def runtime_dtype(info: ParamInfo, stored: torch.dtype, run: torch.dtype) -> torch.dtype:
    if info.kind == "table":
        return torch.int32
    if info.kind == "vector":
        return torch.float32 if (stored == torch.float32 or run == torch.float32) else run
    return run


# --------------------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class KVNeed:
    """Keys and values of every position (window 0) or of the last `window` positions."""

    num_kv_heads: int
    head_dim: int
    window: int = 0
    dtype: Optional[torch.dtype] = None  # None: the run's activation type


@dataclass(frozen=True)
class StateNeed:
    """A record of fixed shape per sequence, zero when the sequence starts."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


# --------------------------------------------------------------------------- part base classes
class Part:
    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        self.prefix = spec.prefix

    def param_infos(self) -> Dict[str, ParamInfo]:
        """Full checkpoint names of this part's tensors and what they must look like."""
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Receive the tensors named by `param_infos`, already on the device in their run types."""

    def children(self) -> Tuple["Part", ...]:
        """Parts that this part owns (an attention mixer's position encoding, extra norms): the model
        asks them for their tensors and loads them like its own parts."""
        return ()

    def _param(self, key: str):
        try:
            return self.spec.params[key]
        except KeyError:
            raise ConfigError(f"part '{self.spec.kind}' (prefix '{self.prefix}') lacks parameter '{key}'") from None


class ResidualStream:
    """The 32-bit residual stream x[T, d] plus what was returned last and not yet added.

    A mixer or feed-forward hands back `delta` ([T, d] or [parts, T, d] partial
    sums, in the activation type).  It is added when the next norm runs, inside
    the norm's kernel, or by `flush()`."""

    def __init__(self, x: torch.Tensor, act_dtype: torch.dtype):
        self.x = x
        self.act_dtype = act_dtype
        self.pending: Optional[torch.Tensor] = None

    def add(self, delta: torch.Tensor) -> None:
        if self.pending is not None:
            self.flush()
        self.pending = delta

    def flush(self) -> None:
        from ..kernels import ops

        if self.pending is not None:
            ops.add_rmsnorm(self.x, self.pending, None, 0.0, self.act_dtype)
            self.pending = None


class Norm(Part):
    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Add what is pending to the stream and return the normalised rows
        (all, or those named by `rows`) in the activation type."""
        raise NotImplementedError

    def rms_weight(self):
        """(weight, eps) if this norm is y = x / sqrt(mean(x^2) + eps) * weight, else None: an arrangement
        may then fold the norm into the products around it (the weight where the product before it stores its
        result, the row's scale where the product after it stores its own)."""
        return None


class PositionEncoding(Part):
    """How a mixer's queries and keys learn their positions.

    `write_qk` is what the attention mixer calls; the default does it in two
    steps from `rotate`, a fused implementation overrides it."""

    def rotate(self, q: torch.Tensor, k: torch.Tensor, step) -> None:
        """Encode positions into q[T, H, hd] and k[T, K, hd] in place."""
        raise NotImplementedError

    def decode_fusion(self):
        """None, or (inv_freq, rotary_dim, interleaved) if this encoding is a rotation by angles
        position * inv_freq[j] of `rotary_dim` leading dimensions (0 = none at all): a mixer may then
        leave `write_qk` out of a decode step and have its attention kernel do the same work."""
        return None

    def write_qk(self, qkv: torch.Tensor, step, kv, num_heads: int, num_kv_heads: int, head_dim: int, write_kv: bool) -> None:
        from ..kernels import ops

        T = qkv.shape[0]
        q = qkv[:, : num_heads * head_dim].view(T, num_heads, head_dim)
        k = qkv[:, num_heads * head_dim : (num_heads + num_kv_heads) * head_dim].view(T, num_kv_heads, head_dim)
        self.rotate(q, k, step)
        if write_kv:
            ops.rope_kv_write(
                qkv, step.tok_pos, step.tok_seq, kv.block_table, kv.k_pages, kv.v_pages, None,
                num_heads, num_kv_heads, head_dim, 0, False, write_kv=True,
            )


class Mixer(Part):
    def cache_need(self):
        """KVNeed, StateNeed or None."""
        return None

    def forward(self, xn: torch.Tensor, step, cache, shared_cache: bool = False) -> torch.Tensor:
        """xn[T, d] -> delta [T, d] (or partial sums [parts, T, d]).

        cache: this run's view of the cache (a KVView or StateView, or None).
        shared_cache: the view belongs to an earlier run of the schedule; read it, do not write it."""
        raise NotImplementedError

    def forward_unprojected(self, xn: torch.Tensor, step, cache, shared_cache: bool = False):
        """None, or (a[T, k], w[d, k]) such that forward(...) == a . w^T: a mixer whose last operation is a
        projection may leave it to the caller, who can then fuse it with what follows."""
        return None


class FeedForward(Part):
    def forward(self, xn: torch.Tensor, step) -> torch.Tensor:
        raise NotImplementedError

    def gated_weights(self):
        """None, or (w_gate_up[2 ff, d] with gate and up rows alternating, w_down[d, ff]) if this feed-forward
        is down(silu(gate(x)) * up(x)) with its weights in that form."""
        return None


class Block(Part):
    """The arrangement of one layer's parts.  Built by the model from a LayerSpec."""

    def __init__(self, spec: PartSpec, runtime: Runtime, mixer: Mixer, feed_forward: FeedForward, norms: Mapping[str, Norm]):
        super().__init__(spec, runtime)
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = dict(norms)

    def forward(self, stream: ResidualStream, step, cache, shared_cache: bool = False) -> None:
        raise NotImplementedError


# --------------------------------------------------------------------------- registries
class Registry:
    def __init__(self, family: str):
        self.family = family
        self._kinds: Dict[str, Callable] = {}

    def register(self, kind: str, cls=None, replace: bool = False):
        """`register("name", Class)` or `@register("name")` above the class."""

        def put(c):
            if kind in self._kinds and not replace:
                raise ConfigError(f"{self.family} '{kind}' is already registered")
            self._kinds[kind] = c
            return c

        return put(cls) if cls is not None else put

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def get(self, kind: str):
        try:
            return self._kinds[kind]
        except KeyError:
            raise ConfigError(f"unknown {self.family} '{kind}' (known: {', '.join(sorted(self._kinds)) or 'none'})") from None

    def build(self, spec: PartSpec, runtime: Runtime, *args, **kwargs):
        return self.get(spec.kind)(spec, runtime, *args, **kwargs)

    def kinds(self):
        return sorted(self._kinds)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")
