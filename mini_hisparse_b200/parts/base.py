"""What every part sees: the runtime (device, compute dtype, matrix products), the workspace,
and the step context (the batch's tokens, segments and cache views).

Interfaces, in short:

* ``Part.parameters()`` -> {local name: ParamSpec}; ``Part.load(tensors)`` receives them on the
  device in the dtype their role asks for and may fuse or re-lay them out.
* ``Norm.forward(x, ctx, delta=None, rows=None)``: x is the float32 residual [T, H]; with
  ``delta`` the sum x + delta is written back to x first; returns the normalised rows in the
  compute dtype.
* ``Mixer.cache_need()`` -> CacheNeed | None;
  ``Mixer.forward(h, ctx, cache)`` -> Product [T, H]; ``cache`` is a view of the entry's cache
  (``cache.writable`` is False when the entry only reads another entry's cache).
* ``Mixer.planner(page_size, sm_count)`` -> StepPlanner | None: the host-side plan of the mixer's
  work for one step (index arrays its kernels read).  The step function packs what the planner
  returns beside the block tables and hands the device views back in ``cache.meta``; it does not
  know what the arrays mean.
* ``FeedForward.forward(h, ctx)`` -> Product [T, H].
* ``Block.forward(x, pending, ctx, cache)`` -> pending: the block adds ``pending`` (the previous
  block's last output) into x where it normalises, and returns its own last output unadded.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch

from ..kernels import api as K
from .spec import CacheNeed, ParamSpec, PartSpec


# ---------------------------------------------------------------------------------------
@dataclass
class Product:
    """The result of a matrix product: one matrix, or ``nsplit`` float32 partial matrices
    [nsplit, M, N] that the consumer sums in order (split-K)."""

    tensor: torch.Tensor
    nsplit: int = 1

    @property
    def split_stride(self) -> int:
        return self.tensor.stride(0) if self.nsplit > 1 else 0

    @property
    def matrix(self) -> torch.Tensor:
        if self.nsplit > 1:
            raise ValueError("split product has not been reduced")
        return self.tensor

    def reduced(self) -> torch.Tensor:
        """The product as one float32 matrix (for inspection; the kernels sum the parts themselves)."""
        return self.tensor.float().sum(0) if self.nsplit > 1 else self.tensor.float()


class Workspace:
    """Named scratch buffers, reused layer after layer.  ``frozen`` forbids growth (a captured
    CUDA graph holds the addresses)."""

    def __init__(self, device):
        self.device = device
        self._buffers: dict[str, torch.Tensor] = {}
        self._zeroed: set[str] = set()
        self.frozen = False

    def get(self, name: str, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * dtype.itemsize
        buf = self._buffers.get(name)
        if buf is None or buf.numel() < nbytes:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would grow after it was frozen")
            cap = max(nbytes, 256)
            buf = torch.empty(cap, dtype=torch.uint8, device=self.device)
            self._buffers[name] = buf
        return buf[:nbytes].view(dtype).view(*shape)

    def get_zeroed(self, name: str, shape, dtype) -> torch.Tensor:
        """A buffer that is zero when first handed out; its users leave it zero (counters that
        reset themselves).  zero_self_resetting() puts all of them back after a fault."""
        n = 1
        for s in shape:
            n *= int(s)
        buf = self._buffers.get(name)
        if buf is None or buf.numel() < n * dtype.itemsize:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would grow after it was frozen")
            self._buffers[name] = torch.zeros(max(n * dtype.itemsize, 256), dtype=torch.uint8, device=self.device)
        self._zeroed.add(name)
        return self.get(name, shape, dtype)

    def zero_self_resetting(self) -> None:
        for name in self._zeroed:
            self._buffers[name].zero_()

    def nbytes(self) -> int:
        return sum(b.numel() for b in self._buffers.values())


class Runtime:
    """Device, compute dtype and the matrix product for that dtype."""

    def __init__(self, device="cuda:0", dtype=torch.bfloat16):
        self.device = torch.device(device)
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, not {dtype}")
        self.dtype = dtype
        if self.device.type != "cuda":
            raise K.KernelError(
                f"device {self.device} is not a CUDA device: this engine runs its own sm_100a "
                "kernels only and has no CPU path"
            )

    def kernel_modules(self) -> tuple[str, ...]:
        """The kernel libraries every model needs in this dtype; parts add their own."""
        return ("elementwise", "gemm_simt", "sampling")

    def linear(self, x: torch.Tensor, weight: torch.Tensor, ws: Workspace, name: str,
               out_dtype: torch.dtype | None = None, bias: torch.Tensor | None = None,
               allow_split: bool = True) -> Product:
        """x [M, K] times weight [N, K] transposed, float32 accumulation.  The result may come as
        split-K partial matrices unless ``allow_split`` is False."""
        M, N = x.shape[0], weight.shape[0]
        out = ws.get(name, (M, N), out_dtype or self.dtype)
        K.gemm_simt(x, weight, out, bias=bias)
        return Product(out)


    def swiglu_layout(self, gate: torch.Tensor, up: torch.Tensor):
        """The stacked gate/up weight [2 I, K] and the block size of its layout: rows of a block of
        gate are followed by the same rows of up.  Here: one block, [gate | up]."""
        return torch.cat((gate, up), 0).contiguous(), gate.shape[0]

    def qkv_rope_append(self, x, weight, bias, ctx, position, block_table, q_out, cache_storage, *,
                        nq: int, nkv: int, d: int, page_size: int, write_kv: bool) -> bool:
        """The stacked q/k/v product with bias, rotation and the append to the cache in ONE kernel,
        if this runtime has one for these sizes and this rotation (``position``: an object with
        rotary_dim, inv_freq and interleaved): then q_out and the cache are written and True is
        returned.  False: the caller runs the product and the rotary kernel one after the other."""
        return False

    def linear_swiglu(self, x, weight, block: int, ws: Workspace, name: str) -> torch.Tensor:
        """silu(x Wg^T) * (x Wu^T) in the compute dtype."""
        gu = self.linear(x, weight, ws, name + "_gu")
        out = ws.get(name, (x.shape[0], weight.shape[0] // 2), self.dtype)
        K.swiglu(gu.tensor, out, nsplit=gu.nsplit, split_stride=gu.split_stride, block=block)
        return out


# ---------------------------------------------------------------------------------------
@dataclass
class Segment:
    """Consecutive tokens of one request inside a step's batch."""

    request: Any          # the request's id
    slot: int             # its state slot
    start: int            # position of the first token
    count: int            # tokens in this step
    offset: int           # index of the first token in the batch


@dataclass
class CacheView:
    """What a mixer gets for its cache entry in one step."""

    need: CacheNeed | None
    group: int
    index: int                      # layer index inside the group
    writable: bool
    storage: torch.Tensor | None    # pages: [pages, 2, nkv, P, d]; state: [max_requests, *shape]
    page_size: int = 0
    meta: dict = field(default_factory=dict)   # device views of the group's per-step arrays


@dataclass
class StepContext:
    rt: Runtime
    ws: Workspace
    T: int
    segments: list[Segment]
    tokens: torch.Tensor            # [T] int32
    positions: torch.Tensor         # [T] int32
    tok_seg: torch.Tensor           # [T] int32: segment of each token
    seg_slot: torch.Tensor          # [S] int32: state slot of each segment
    status: torch.Tensor            # [1] int32 error bits set by kernels
    extras: dict = field(default_factory=dict)


# ---------------------------------------------------------------------------------------
class Part:
    """Base of all parts: a spec, stored tensors, nothing about the model around it."""

    def __init__(self, spec: PartSpec, rt: Runtime | None = None):
        self.spec = spec
        self.rt = rt

    def parameters(self) -> dict[str, ParamSpec]:
        return {}

    def kernel_modules(self) -> tuple[str, ...]:
        """Kernel libraries (csrc file stems) this part launches beyond the runtime's own: what a
        model's first step compiles is the union over its parts."""
        return ()

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        for k, v in tensors.items():
            setattr(self, k.replace(".", "_"), v)

    def nbytes(self) -> int:
        total = 0
        for v in vars(self).values():
            if isinstance(v, torch.Tensor):
                total += v.numel() * v.element_size()
        return total


class StepPlanner:
    """The host-side plan of a paged mixer's work for one step.

    A planner turns the step's segments into int32 index arrays (work items and the like) that
    the mixer's kernels read, and host facts (counts that size the launches).  The step function
    packs the arrays into the step's single host-to-device copy beside the block tables and gives
    the mixer their device views as ``cache.meta[name]``; facts arrive as ``cache.meta[name]`` too.
    Mixers of one page group whose ``plan_key()`` compare equal share one planner and one plan.

    ``fixed`` is what ``decode_fixed`` returned when a CUDA graph of single-token segments was
    captured: with it, the arrays' sizes and the facts must depend on the number of segments
    only, since a replayed graph launches what was captured.
    """

    def capacity(self, max_tokens: int, max_segments: int, fixed=None) -> dict[str, int]:
        """Upper bounds of the arrays' lengths (int32 words) for a step of that size."""
        raise NotImplementedError

    def plan(self, segments: list["Segment"], T: int, fixed=None) -> tuple[dict[str, np.ndarray], dict]:
        """(arrays, facts) of one step; every array no longer than its capacity."""
        raise NotImplementedError

    def decode_fixed(self, segments_count: int, max_positions: int):
        """What to hold constant in a captured graph of ``segments_count`` single-token segments
        with at most ``max_positions`` cached positions each (None: nothing)."""
        return None

    def decode_fixed_for(self, starts: np.ndarray, max_positions: int):
        """decode_fixed for a step whose single-token segments sit at positions ``starts``: a planner
        may choose by the histories it actually sees (a graph is captured per value, so the value
        should change seldom).  It must be hashable.  Default: decode_fixed."""
        return self.decode_fixed(len(starts), max_positions)

    def plan_decode(self, starts: np.ndarray, fixed) -> tuple[dict[str, np.ndarray], dict]:
        """plan() for single-token segments at positions ``starts`` (segment i = token i = slot
        row i), as a fast path without per-token loops.  Default: the general plan."""
        segments = [Segment(i, i, int(p), 1, i) for i, p in enumerate(starts)]
        return self.plan(segments, len(segments), fixed)


class Mixer(Part):
    def cache_need(self) -> CacheNeed | None:
        return None

    def plan_key(self):
        """Mixers of one page group with equal keys share a planner (None: no plan needed)."""
        return None

    def planner(self, page_size: int, sm_count: int) -> StepPlanner | None:
        return None

    def check_cache(self, page_size: int) -> None:
        """Raise ValueError if this mixer cannot work over pages of ``page_size`` positions: called
        when a model is paired with a cache, so that a step never finds out half-way."""

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None) -> Product:
        raise NotImplementedError

    #: False if forward() does host-side work that depends on the batch (no CUDA graph then)
    graph_safe = True


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx: StepContext) -> Product:
        raise NotImplementedError

    graph_safe = True


class Block:
    """Base of block arrangements: how a layer's parts are wired to the residual stream.

    A subclass builds its parts from ``spec.part(role)`` with the registries it wants, lists them
    in ``parts()`` (role -> part, the roles of its LayerSpec), and names the ONE part that owns
    per-request memory as ``self.mixer`` (or overrides the three methods below).
    ``forward(x, pending, ctx, cache) -> pending``: x is the float32 residual [T, H]; ``pending``
    is the previous block's last output, not yet added to x (None for the first block).
    """

    mixer: "Mixer | None" = None

    def parts(self) -> dict[str, Part]:
        raise NotImplementedError

    def cache_need(self) -> CacheNeed | None:
        return self.mixer.cache_need() if self.mixer is not None else None

    def plan_key(self):
        return self.mixer.plan_key() if self.mixer is not None else None

    def planner(self, page_size: int, sm_count: int) -> StepPlanner | None:
        return self.mixer.planner(page_size, sm_count) if self.mixer is not None else None

    def check_cache(self, page_size: int) -> None:
        if self.mixer is not None:
            self.mixer.check_cache(page_size)

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", True) for p in self.parts().values())

    def forward(self, x: torch.Tensor, pending: Product | None, ctx: StepContext,
                cache: CacheView | None) -> Product:
        raise NotImplementedError


class Norm(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext, delta: Product | None = None,
                rows: torch.Tensor | None = None, name: str = "h") -> torch.Tensor:
        raise NotImplementedError
