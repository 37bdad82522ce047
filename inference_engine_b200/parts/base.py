"""Interfaces that every part of a layer implements.

A part is built from a :class:`~inference_engine_b200.config.spec.PartSpec` (its sizes and
constants are parameters), says which tensors it reads (:meth:`Part.weights`), receives them
(:meth:`Part.bind`) and then runs on device tensors.  No part knows which model it is in:
it sees its own parameters, the step's :class:`StepContext` and, for a mixer, the binding
to its cache.

Categories and what each must provide
-------------------------------------
``norm``          ``add_norm(h, delta, ctx, rows=None, tag="norm", delta_scale=1.0) -> x``: add
                  ``delta_scale * delta`` to the 32-bit residual ``h`` in place (unless ``rows``
                  selects rows, then nothing is modified) and return the normalised activations.
``position``      a :class:`PositionEncoding`: ``rotary_table()``/``rotary_dim`` for encodings
                  applied to queries and keys, ``apply_to_embedding`` for additive ones.
``mixer``         ``cache_request()`` (what it keeps per request: pages of keys and values,
                  a fixed-size state, or nothing) and
                  ``forward(x, ctx, binding) -> delta`` (32-bit ``[N, hidden]``, or
                  ``[S, N, hidden]`` partial sums that the next norm adds in order).
``feed_forward``  ``forward(x, ctx) -> delta`` (32-bit ``[N, hidden]``).
``block``         the arrangement: ``forward(h, delta, ctx, binding, delta_scale=1.0) -> delta``
                  where ``h`` is the residual stream and ``delta`` the not-yet-added output of
                  the previous block, to be added times ``delta_scale``; ``residual_mult`` is the
                  factor its own returned delta is to be added with.
``embedding``     ``forward(token_ids, ctx) -> h`` (32-bit residual stream); one that keeps something
                  per request (the previous token) says so with ``cache_request()`` and is given
                  its binding as ``forward(token_ids, ctx, binding)``.
``stream``        an operation on the whole residual stream between layers, named by a run-order
                  entry's ``before``: ``forward(h, x0, ctx) -> None`` rewrites ``h`` in place
                  (``x0``: the embedding's output, kept when a stream part asks for it).
``head``          ``forward(x, ctx) -> logits`` (32-bit ``[rows, vocab]``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any


@dataclass(frozen=True)
class WeightDecl:
    """A tensor a part reads from the checkpoint.

    ``role``: ``matrix`` (used in a matrix product; kept in the compute dtype),
    ``vector`` (scales and biases; used in 32-bit), ``table`` (rows gathered by index) or
    ``int_table`` (integers, kept as int32).
    ``init`` says how the random-weights mode draws it: ``normal`` is N(0, std),
    ``ones_plus_normal`` is 1 + N(0, std), ``zeros`` and ``ones`` are constant.
    """

    shape: tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"


@dataclass(frozen=True)
class PagedKVRequest:
    """A mixer that keeps keys and values per token.  ``window`` = how many of the latest
    positions a query may see (``None`` = all): pages behind the window are given back."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None
    # Size of a cached value row: None = as large as a key row; 0 = no value rows are kept (a
    # mixer whose values are a part of its key rows, such as a shared latent vector).
    value_dim: int | None = None
    # A query sees only the keys of its own chunk of this many positions, counted from position 0
    # (``None`` = no chunks): pages that lie wholly before the current chunk are given back.
    chunk: int | None = None
    # With a window: the first ``keep_first`` positions stay visible to every later query, so the
    # pages that hold them are never given back while the request lives.
    keep_first: int = 0


@dataclass(frozen=True)
class StateRequest:
    """A mixer that keeps a state of fixed size per request (32-bit floats of ``shape``)."""

    shape: tuple[int, ...]


@dataclass(frozen=True)
class CacheBinding:
    """Where one run of a mixer finds its cache: the cache group, the layer's slot in the
    group's storage, and whether this run writes (a run that borrows another layer's cache
    only reads)."""

    group: int
    slot: int
    writes: bool = True


@dataclass
class BuildEnv:
    """What a part may look at while it is built."""

    hidden_size: int
    dtype: str  # "bfloat16" or "float32": the compute dtype of activations and matrices
    max_positions: int  # positions the engine will ever feed (tables are sized for it)
    positions: dict[str, Any]  # built position encodings by name
    device: Any = None

    @property
    def torch_dtype(self):
        import torch

        return torch.bfloat16 if self.dtype == "bfloat16" else torch.float32


class Part:
    category = "part"
    # Whether the part's step is a fixed sequence of kernel launches that reads lengths, slots and
    # tables from device memory, so that it can be captured once and replayed (a part that loops over
    # requests on the host, or reads device values there, says False).
    captures = True

    def weights(self) -> dict[str, WeightDecl]:
        """Full tensor names this part reads, with their shapes."""
        return {}

    def bind(self, tensors: dict[str, Any], env: BuildEnv) -> None:
        """Receive the tensors named by :meth:`weights`, already on the device in their
        stored dtype; cast and fuse them as the part needs."""

    def parts(self) -> list["Part"]:
        """Nested parts (a block returns its mixer, feed-forward and norms)."""
        return []


class PositionEncoding(Part):
    category = "position"
    rotary_dim = 0  # leading dims of each head that are rotated (0 = none)

    def rotary_table(self):
        """``[max_positions, 2, rotary_dim // 2]`` 32-bit cos and sin, or None."""
        return None

    def apply_to_embedding(self, h, ctx) -> None:
        """Additive encodings add to the embedded tokens here; default: nothing."""


class CarriesInputRows:
    """A sublayer whose first step is one matrix product over its input can carry the rows of another
    linear map of the same input in that product (a block's residual gate, for one): it says so
    with ``accepts_input_rows``, is handed the rows before its own ``bind`` (``take_input_rows``)
    and leaves their 32-bit products of the step, ``[N, rows]`` as columns of its product, in
    ``extra_out`` when it runs."""

    accepts_input_rows = False
    extra_out = None
    _extra_rows = None

    def take_input_rows(self, rows) -> None:
        if not self.accepts_input_rows:
            raise ValueError(f"{type(self).__name__} has no input product that could carry more rows")
        self._extra_rows = rows

    def _with_extra_rows(self, own_rows: list):
        """``(weight, first column of the extra rows' products)``: the part's own row blocks, zero
        rows up to a multiple of four (so that the extra columns can be read four at a time), then
        the rows it was handed."""
        import torch

        count = sum(r.shape[0] for r in own_rows)
        if self._extra_rows is None:
            return torch.cat(own_rows).contiguous(), count
        pad = -count % 4
        if pad:
            own_rows = own_rows + [own_rows[0].new_zeros(pad, own_rows[0].shape[1])]
        extra = self._extra_rows.to(own_rows[0].dtype)
        self._extra_count = extra.shape[0]
        return torch.cat(own_rows + [extra]).contiguous(), count + pad

    def _extra_columns(self, proj, at: int):
        return None if self._extra_rows is None else proj[:, at: at + self._extra_count]


class Mixer(CarriesInputRows, Part):
    category = "mixer"

    def cache_request(self) -> PagedKVRequest | StateRequest | None | tuple:
        """What the mixer keeps per request.  A mixer made of several (two side by side, one
        wrapped around another) returns a tuple of requests, and is then handed a tuple of
        bindings in the same order (``None`` where a request is ``None``)."""
        return None

    def forward(self, x, ctx, binding: CacheBinding | None):
        raise NotImplementedError


class FeedForward(CarriesInputRows, Part):
    category = "feed_forward"

    def forward(self, x, ctx):
        raise NotImplementedError


class Norm(Part):
    category = "norm"

    def add_norm(self, h, delta, ctx, rows=None, tag: str = "norm", delta_scale: float = 1.0):
        raise NotImplementedError


class Block(Part):
    category = "block"

    mixer: Mixer
    residual_mult: float = 1.0  # the factor with which the returned delta enters the residual stream

    def forward(self, h, delta, ctx, binding: CacheBinding | None, delta_scale: float = 1.0):
        raise NotImplementedError
