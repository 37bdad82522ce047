"""The engine's kernels as Python calls on torch tensors.

Each method hands raw device pointers and the current CUDA stream to a plain-C function of
the in-tree shared library (``ctypes``; nothing is allocated on the way).  There is no
fallback: if the library cannot be built or loaded, or a tensor is not on a CUDA device,
the call raises.  Matrix products in bfloat16 go to the vendor library through ``torch.mm``
(the reference uses cuBLAS for them through ``nn.Linear``, engine/model/layers.py:126-129);
32-bit matrix products, attention, norms, rotary encoding, the cache write, the activation,
the embedding gather and sampling are the kernels under ``csrc/``.
"""

from __future__ import annotations

import contextlib
import ctypes
import functools
import os
from ctypes import c_float, c_int, c_void_p

from .build import (ATTENTION_HEAD_DIMS, build_attention, build_core, build_part_library,
                    build_sigmoid_attention, build_sink_attention)

_ERRORS = {
    1: "a token id outside the vocabulary",
    2: "a page or slot outside the cache",
    3: "a position outside the rotary table",
    4: "a block-table entry that was already given back",
    5: "a bounded wait inside a kernel ran out (a copy never arrived)",
}


class KernelError(RuntimeError):
    pass


class KernelTimer:
    """Device time per kind of kernel, from CUDA events recorded around every launch made while
    the timer is active (``with ops.timed() as timer``).  The events sit between the kernels,
    so a kernel's start-up no longer overlaps its predecessor: the sum is a little more than
    the step takes untimed; the shares are what it is for."""

    def __init__(self, torch) -> None:
        self.torch = torch
        self.spans: list[tuple[str, object, object]] = []

    def begin(self, name: str):
        start = self.torch.cuda.Event(enable_timing=True)
        start.record()
        return name, start

    def end(self, span) -> None:
        stop = self.torch.cuda.Event(enable_timing=True)
        stop.record()
        self.spans.append((span[0], span[1], stop))

    def summary(self) -> dict[str, dict]:
        """kind -> {"launches": n, "ms": total device time}; waits for the device."""
        self.torch.cuda.synchronize()
        out: dict[str, dict] = {}
        for name, start, stop in self.spans:
            row = out.setdefault(name, {"launches": 0, "ms": 0.0})
            row["launches"] += 1
            row["ms"] += start.elapsed_time(stop)
        return out


def _kind(name):
    """Marks a kernel method with the kind its launches are counted under by a KernelTimer and
    shown under in a profiler's timeline (NVTX ranges, with IE_B200_NVTX=1).  ``name`` is a
    string or a function of the call's keyword arguments."""
    def decorate(method):
        def call(self, *args, **kwargs):
            timer, nvtx, recorder = self._timer, self.nvtx, self._recorder
            if timer is None and not nvtx and recorder is None:
                return method(self, *args, **kwargs)
            label = name if isinstance(name, str) else name(kwargs)
            if recorder is not None:
                recorder.append((label, functools.partial(method, self, *args, **kwargs)))
            if nvtx:
                self.torch.cuda.nvtx.range_push(label)
            span = timer.begin(label) if timer is not None else None
            try:
                return method(self, *args, **kwargs)
            finally:
                if span is not None:
                    timer.end(span)
                if nvtx:
                    self.torch.cuda.nvtx.range_pop()
        call.__name__, call.__doc__ = method.__name__, method.__doc__
        return call
    return decorate


def _dtype_code(t) -> int:
    import torch

    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {t.dtype}")


class CudaOps:
    name = "cuda-sm100a"

    def __init__(self, device="cuda") -> None:
        import torch

        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: the engine has no CPU path")
        self.torch = torch
        self.device = torch.device(device)
        self.lib_path = build_core()
        try:
            self.lib = ctypes.CDLL(str(self.lib_path))
        except OSError as exc:
            raise KernelError(f"the kernel library {self.lib_path} could not be loaded: {exc}") from exc
        self._declare()
        # programmatic dependent launch between the engine's own kernels (IE_B200_PDL=0: off)
        self.pdl = os.environ.get("IE_B200_PDL", "1") != "0"
        self.lib.ie_set_pdl(1 if self.pdl else 0)
        self.err = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._err_ptr = self.err.data_ptr()
        self._attn_libs: dict[int, object] = {}
        self._part_libs: dict[str, object] = {}
        self._sigattn_libs: dict[tuple[int, int], object] = {}
        self._sinkattn_libs: dict[tuple[int, int], object] = {}
        self.sink_mma = os.environ.get("IE_B200_SINK_MMA", "1") != "0"  # tensor-core sink attention
        # residual gates' products as partial sums: faster by themselves, slower inside a captured step
        self.gate_split = os.environ.get("IE_B200_GATE_SPLIT", "0") == "1"
        self.sigmoid_mma = os.environ.get("IE_B200_SIGMOID_MMA", "1") != "0"  # tensor-core sigmoid attention
        self._argmax_scratch = None
        self._tickets = None
        self._retired_tickets = []
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.attn_tc5 = os.environ.get("IE_B200_ATTN_TC5", "1") != "0"  # tcgen05 prefill attention
        self.latent_mma = os.environ.get("IE_B200_LATENT_MMA", "1") != "0"  # tensor-core latent attention
        self.prefill_key_splits = os.environ.get("IE_B200_PREFILL_KEY_SPLITS", "1") != "0"
        # up to this many query tiles x heads per SM a block takes two tiles of a request (a late and an early one)
        self.prefill_paired_max = float(os.environ.get("IE_B200_PREFILL_PAIRED_MAX", 4))
        # the decode kernel cuts contexts until about this many blocks run (one block per SM)
        self.decode_split_target = int(os.environ.get("IE_B200_DECODE_SPLIT_TARGET", 128))
        # up to this many parts of a context merge inside a thread-block cluster (2, 4, 8; 0: never),
        # for steps whose block tables hold at most `decode_cluster_tokens` tokens per request
        self.decode_cluster_max = int(os.environ.get("IE_B200_DECODE_PAIR", 8))
        self.decode_cluster_tokens = int(os.environ.get("IE_B200_DECODE_CLUSTER_TOKENS", 4096))
        # requests with at most 8 rows (tokens x query heads per key/value head) run the decode
        # kernels' swapped products: keys are the instruction's rows ("0": the 16-row layout for all)
        self.decode_narrow = os.environ.get("IE_B200_DECODE_NARROW", "1") != "0"
        # batches whose contexts differ much in length go to the decode kernel that deals key tiles
        # by length ("auto": when the step's context says so; "1": always; "0": never)
        self.decode_balanced = os.environ.get("IE_B200_DECODE_BALANCED", "auto")
        self.decode_balanced_blocks_per_pair = 32
        # by-request decode attention in two-warp blocks where that saves a round ("0": never)
        # ("2", "3": always blocks of as many warps when there are more blocks than SMs, for comparisons)
        small = os.environ.get("IE_B200_DECODE_SMALL", "1")
        self.decode_small = small != "0"
        self._force_small = int(small) if small in ("2", "3") else 0
        self._small_per_sm: dict[tuple[int, int], int] = {}
        self._dealing_look, self._dealing_answer = None, 0  # the last batch decode_dealing looked at, and its answer
        self.balanced_launches = 0
        # which kernel takes few-row bfloat16 products: "tma" (the TMA-fed weight-streaming kernel)
        # or "lib" (the vendor library, for comparisons)
        self.few_row_gemm = os.environ.get("IE_B200_FEW_ROW_GEMM", "tma")
        # ... up to this many 128-feature tiles (measured on the 1B shape: up to 8 rows the kernel
        # streams 67 MB in 12.0 us where the vendor library takes 12.7, and the 525 MB of the
        # head in 82 us against 79.5; from 9 rows on its second column tile makes it slower on
        # wide matrices, so only those that must be cut along k to fill the GPU go to it)
        self.tma_max_tiles = int(os.environ.get("IE_B200_TMA_MAX_TILES", 256))
        self.tma_max_tiles_wide = min(self.tma_max_tiles, self.sm_count // 2)  # 9 to 16 rows
        self.tma_max_blocks = int(os.environ.get("IE_B200_TMA_MAX_BLOCKS", 3 * self.sm_count // 2))
        # Products of 17 to `batch_gemm_rows` rows with a long inner dimension: the tcgen05
        # weight-streaming kernel (IE_B200_BATCH_GEMM=0: the vendor library).  Measured on the 1B
        # shape at 64 rows: the down projection (K = 8192) 11.0 us against the library's 13.0,
        # but QKV, output and gate-up (K = 2048) 7.3 / 6.3 / 16.3 against 5.7 / 5.5 / 13.5: every
        # block copies all tokens' activations through its SM's copy engine beside the weights,
        # which the library's kernels share within a cluster.  So only long inner dimensions, and
        # only where its blocks (feature tiles x cuts along k) fit the SMs in one round: at the 3B
        # shape the down projection (3072 x 8192) 13.5 against 14.2 us, at the 8B shape (4096 x
        # 14336: 224 blocks) 33.6 against 25.4, and its K = 4096 products 13 to 45 % behind.
        # the gated feed-forward's first product with the activation in its kernel (IE_B200_GATED_GEMM=0: off)
        self.gated_gemm = os.environ.get("IE_B200_GATED_GEMM", "1") != "0"
        # products of more than a few rows whose output is so narrow that the library's kernel would
        # leave most SMs idle are cut along the inner dimension and run as one strided batched product
        # (the parts are added by the consumer, like those of the few-row kernel)
        self.blas_split_k = os.environ.get("IE_B200_BLAS_SPLIT_K", "1") != "0"
        self.batch_gemm = os.environ.get("IE_B200_BATCH_GEMM", "1") != "0"
        self.batch_gemm_rows = int(os.environ.get("IE_B200_BATCH_GEMM_ROWS", 64))
        self.batch_gemm_max_tiles = int(os.environ.get("IE_B200_BATCH_GEMM_MAX_TILES", 256))
        self.batch_gemm_min_k = int(os.environ.get("IE_B200_BATCH_GEMM_MIN_K", 8192))
        # only where the kernel's blocks fit the SMs in one round
        self.batch_gemm_one_round = os.environ.get("IE_B200_BATCH_GEMM_ONE_ROUND", "1") != "0"
        self._device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
        self._timer: KernelTimer | None = None
        self._recorder: list | None = None
        self.nvtx = os.environ.get("IE_B200_NVTX", "0") == "1"  # an NVTX range around every kernel call
        self.launches = 0  # launches of this library's kernels (library matrix products not counted)
        self.launch_counts: dict[str, int] = {}  # the same, per kernel
        self._cluster_fit: dict[tuple[int, int], int] = {}  # (head size, parts) -> clusters the device runs at once

    def _declare(self) -> None:
        P, I, F, L = c_void_p, c_int, c_float, ctypes.c_longlong
        sigs = {
            "ie_embedding": [P, I, P, P, I, I, I, F, P, P],
            "ie_rmsnorm": [P, P, I, L, F, P, F, P, I, P, I, I, P],
            "ie_layernorm": [P, P, I, L, F, P, F, P, I, P, I, I, P],
            "ie_add_position_rows": [P, P, I, P, I, I, I, P, P],
            "ie_relu_squared": [P, P, I, L, P],
            "ie_scale": [P, F, L, P],
            "ie_rope_kv_write": [P, I, L, P, P, I, I, P, P, P, I, P, I, I, I, I, I, I, P, P],
            "ie_silu_mul": [P, I, I, L, P, I, I, I, I, P],
            "ie_gemm_tma_gated_bf16": [P, P, P, I, I, I, P, P],
            "ie_argmax": [P, I, I, I, P, P, P],
            "ie_gemm_f32": [P, P, P, I, I, I, P],
            "ie_gemm_tma_bf16": [P, P, P, I, I, I, I, I, I, P, P],
            "ie_gemm_tc5_bf16": [P, P, P, I, I, I, I, I, I, P, P],
            "ie_gemm_tc5_ok": [I, I, I],
            "ie_paged_attention_generic": [P, P, P, I, P, I, P, P, P, I, I, I, I, I, I, I, I, F, I, I, P, P, P, I, F, I, P, P],
            "ie_sample": [P, I, I, P, P, P, P, P, P, I, P, P, P, P, P],
            "ie_bigram_embedding": [P, P, I, P, P, P, P, P, P, L, I, P, I, I, I, I, L, L, P, P],
            "ie_sandwich_norm": [P, P, I, L, P, I, L, P, P, P, F, P, F, P, I, P, I, I, P],
            "ie_scale_softcap": [P, F, F, L, P],
            "ie_silu_mul_bias": [P, I, P, P, I, I, I, P],
            "ie_concat_cast": [P, P, P, I, I, I, P],
            "ie_weighted_sum": [P, F, P, F, P, L, P],
            "ie_gated_add_norm": [P, P, I, L, P, I, L, I, P, P, F, P, I, P, I, I, P],
            "ie_polynorm": [P, I, I, P, F, P, I, I, I, P],
        }
        for name, args in sigs.items():
            fn = getattr(self.lib, name)
            fn.argtypes, fn.restype = args, c_int
            setattr(self, "_" + name[3:], fn)

    # --- helpers ----------------------------------------------------------------------------

    def _stream(self) -> int:
        """The raw handle of torch's current stream on this device (asked on every launch, so
        through the cheap accessor when torch has it)."""
        if self._raw_stream is not None:
            return self._raw_stream(self._device_index)
        return self.torch.cuda.current_stream(self.device).cuda_stream

    def _check(self, code: int, what: str) -> None:
        self.launches += 1
        self.launch_counts[what] = self.launch_counts.get(what, 0) + 1
        if code != 0:
            raise KernelError(f"{what}: CUDA error {code} at launch")

    @staticmethod
    def _ptr(t) -> int | None:
        return None if t is None else t.data_ptr()

    def check_errors(self) -> None:
        """Read the device error word (this waits for the stream) and raise if a kernel saw
        an index out of range or gave up a wait."""
        self.raise_reported(self.err.tolist())

    def raise_reported(self, words) -> None:
        """``words``: a copy of the error word (code, value, where, spare).  A non-zero code
        clears the word on the device (the first report wins, so the next fault must find it
        empty) and raises."""
        code, value, where = words[:3]
        if code:
            self.err.zero_()
            raise KernelError(f"kernel check failed: {_ERRORS.get(code, code)} "
                              f"(value {value}, at row/token {where})")

    @contextlib.contextmanager
    def timed(self, lead_ms: float = 0.0):
        """``with ops.timed() as timer: ...; timer.summary()``: CUDA-event time per kind of kernel
        for everything launched inside the block (eager launches only: a replayed capture is one
        launch).  The host launches small kernels more slowly than the device runs them, and an
        event pair around a kernel that has not been launched yet measures the host; with
        ``lead_ms`` the device is first kept busy that long, so that the block's launches queue
        up behind it and the events see device time only."""
        timer = KernelTimer(self.torch)
        if lead_ms > 0:
            self.busy_wait(lead_ms)
        self._timer = timer
        try:
            yield timer
        finally:
            self._timer = None

    @contextlib.contextmanager
    def recording(self):
        """``with ops.recording() as calls``: every kernel call made inside the block is also kept
        as ``(kind, callable)``; calling the callable launches the same kernel on the same
        tensors again (for timing one kind of kernel by itself, back to back over a step's
        layers)."""
        calls: list = []
        self._recorder = calls
        try:
            yield calls
        finally:
            self._recorder = None

    def busy_wait(self, ms: float) -> None:
        """Keep the device busy for about ``ms``, so that what the host launches next queues up."""
        khz = self.torch.cuda.get_device_properties(self.device).clock_rate
        self.torch.cuda._sleep(int(ms * khz))

    # --- kernels ----------------------------------------------------------------------------

    @_kind("embedding")
    def embedding(self, table, ids, out, scale: float = 1.0) -> None:
        """``out[n] = table[ids[n]] * scale`` as 32-bit rows."""
        self._check(self._embedding(table.data_ptr(), _dtype_code(table), ids.data_ptr(),
                                    out.data_ptr(), ids.shape[0], table.shape[1], table.shape[0],
                                    float(scale), self._err_ptr, self._stream()), "embedding")

    @staticmethod
    def _partials(t) -> tuple[int, int]:
        """A 3-D tensor ``[S, rows, cols]`` stands for the sum of its S slices (the parts of a
        matrix product split along the inner dimension): (S, elements between slices)."""
        if t is None or t.dim() == 2:
            return 1, 0
        return t.shape[0], t.stride(0)

    @_kind("norm")
    def rmsnorm(self, h, delta, weight, eps, out, rows=None, delta_scale: float = 1.0) -> None:
        n = h.shape[0] if rows is None else rows.shape[0]
        parts, stride = self._partials(delta)
        self._check(self._rmsnorm(h.data_ptr(), self._ptr(delta), parts, stride, delta_scale, weight.data_ptr(),
                                  eps, out.data_ptr(), _dtype_code(out), self._ptr(rows), n,
                                  h.shape[1], self._stream()), "rmsnorm")

    @_kind("norm")
    def layernorm(self, h, delta, weight, eps, out, rows=None, delta_scale: float = 1.0) -> None:
        """Layer norm (weight, no bias) of ``h + delta_scale * delta``; the conventions of :meth:`rmsnorm`."""
        n = h.shape[0] if rows is None else rows.shape[0]
        parts, stride = self._partials(delta)
        self._check(self._layernorm(h.data_ptr(), self._ptr(delta), parts, stride, delta_scale, weight.data_ptr(),
                                    eps, out.data_ptr(), _dtype_code(out), self._ptr(rows), n,
                                    h.shape[1], self._stream()), "layernorm")

    @_kind("embedding")
    def add_position_rows(self, h, table, positions) -> None:
        """``h[n] += table[positions[n]]`` (a learned position vector per token)."""
        self._check(self._add_position_rows(h.data_ptr(), table.data_ptr(), _dtype_code(table),
                                            positions.data_ptr(), h.shape[0], h.shape[1], table.shape[0],
                                            self._err_ptr, self._stream()), "add_position_rows")

    @_kind("activation")
    def relu_squared(self, x, out) -> None:
        if x.dtype != out.dtype or not x.is_contiguous() or not out.is_contiguous():
            raise KernelError("relu_squared takes contiguous tensors of one dtype")
        self._check(self._relu_squared(x.data_ptr(), out.data_ptr(), _dtype_code(x), x.numel(), self._stream()),
                    "relu_squared")

    @_kind("head")
    def scale_(self, t, factor: float) -> None:
        """``t *= factor`` for a contiguous 32-bit tensor."""
        self._check(self._scale(t.data_ptr(), float(factor), t.numel(), self._stream()), "scale")

    @_kind("head")
    def scale_softcap_(self, t, factor: float, cap: float) -> None:
        """``t <- cap * tanh(t * factor / cap)`` for a contiguous 32-bit tensor."""
        self._check(self._scale_softcap(t.data_ptr(), float(factor), float(cap), t.numel(), self._stream()),
                    "scale_softcap")

    FEW_ROWS = 16  # up to this many rows a bfloat16 product runs the weight-streaming kernel

    def tma_split(self, n_out: int, k: int) -> tuple[int, int]:
        """(64-wide k blocks per split, splits) for the TMA-fed few-row product: one block of
        128 features per SM if there are enough features, else the inner dimension is cut so
        that about every SM has a block; a block takes at most 32 k blocks."""
        tiles = -(-n_out // 128)
        total = -(-k // 64)
        splits = max(1, min(total, self.sm_count // tiles))
        per = min(-(-total // splits), 32)
        # one copy brings up to four k blocks when they divide the slice: round the slice up to
        # a multiple of 4 (or 2) unless that leaves many SMs without a block
        for multiple in (4, 2):
            rounded = min(-(-per // multiple) * multiple, 32)
            if rounded != per and -(-total // rounded) * tiles * 10 >= -(-total // per) * tiles * 8:
                per = rounded
                break
            if rounded == per:
                break
        return per, -(-total // per)

    def blas_split(self, m: int, n: int, k: int) -> int:
        """Into how many parts along the inner dimension a bfloat16 product of ``m`` rows is cut before
        it goes to the library (1: not at all).  The library's kernels take about 128 x 128 outputs per
        block and do not cut the inner dimension themselves: the 64-row down projection of the 1B shape
        runs as 16 blocks on 148 SMs, 13 us where its 33.5 MB would stream in 5.  As a batched product
        over 8 slices of k it takes 8.5 us (measured, 1B shape, us: down at 17 / 64 / 256 / 512 rows
        13.0 / 13.2 / 13.8 / 18.9 -> 8.1 / 8.5 / 10.6 / 15.4; output projection at 17 / 64 rows 5.6 / 5.8
        -> 4.4 / 4.8; QKV 5.8 -> 5.0; products with many output features, gate-up and the head, lose).
        A power of two: at most 8 up to 32 rows, 4 up to 256, 2 up to 512 (the parts' sums are written and
        read again: 96 rows of the down projection take 9.6 us in 8 parts, 8.6 in 4); no more parts than
        bring the library's blocks to about 1.2 per SM; slices of at least 256.  The rule was set against
        `profile_gemm`'s tables of the 1B, 3B and 8B shapes' products at 9 to 512 rows: it is 0.6 %, 1.4 %
        and 1.8 % behind the best of 1, 2, 4, 8 parts on average, 4 %, 8 % and 15 % at worst."""
        if not self.blas_split_k or m > 512:
            return 1
        blocks = -(-m // 128) * -(-n // 128)
        parts = 1
        most = 8 if m <= 32 else 4 if m <= 256 else 2
        while parts * 2 <= min(1.2 * self.sm_count / blocks, most) and k % (parts * 2 * 64) == 0 and k // (parts * 2) >= 256:
            parts *= 2
        return parts

    @_kind(lambda kwargs: "linear:" + kwargs.get("tag", "linear"))
    def linear(self, x, w, out=None, *, ws=None, tag="linear", out_dtype=None, allow_split=False):
        """``x[M, K] @ w[N, K]^T``.  With ``out`` given the product is written there; otherwise a
        buffer named ``tag`` is taken from ``ws``.  With ``allow_split`` the result may come back
        as ``[S, M, N]`` partial sums (32-bit) that the consumer adds in order."""
        torch = self.torch
        m, k = x.shape
        n = w.shape[0]
        if out is not None:
            out_dtype = out.dtype
        if x.dtype == torch.float32:
            if out_dtype != torch.float32 or w.dtype != torch.float32:
                raise KernelError("the 32-bit matrix product takes and gives 32-bit tensors")
            if out is None:
                out = ws.buffer(tag, m, n, torch.float32)
            if m:
                self._check(self._gemm_f32(x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k,
                                           self._stream()), "gemm_f32")
            return out
        # The weight-streaming kernel pays where the library leaves SMs idle: few output
        # features (fewer 16-feature blocks than SMs) and a long inner dimension to split.
        few_rows = 0 < m <= self.FEW_ROWS and k % 8 == 0 and x.is_contiguous() and w.is_contiguous()
        splittable = (allow_split and out is None and out_dtype == torch.float32 and m > 0
                      and x.is_contiguous() and w.is_contiguous())
        library_parts = self.blas_split(m, n, k) if splittable else 1
        if few_rows and m > 8 and library_parts > 1 and (k >= 4096 or n * k >= 12 << 20):
            # (9 to 16 rows, a long inner dimension or a large matrix: the batched library product is ahead,
            # 8.0 against 9.5 us on the 1B shape's down projection, 7.9 against 9.1 on the 3B shape's QKV)
            few_rows = False
        if (few_rows and self.few_row_gemm == "tma"
                and -(-n // 128) <= (self.tma_max_tiles if m <= 8 else self.tma_max_tiles_wide)):
            kbps, splits = self.tma_split(n, k) if allow_split and out is None else (-(-k // 64), 1)
            # (more than one and a half rounds of blocks over the SMs: the library's kernels are
            # ahead there, 41.8 against 45.7 us on the 8B shape's gate-up matrix)
            if kbps <= 32 and -(-n // 128) * splits <= self.tma_max_blocks:
                if splits > 1:
                    out = ws.buffer(tag, splits * m, n, torch.float32).view(splits, m, n)
                elif out is None:
                    out = ws.buffer(tag, m, n, out_dtype)
                self._check(self._gemm_tma_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), _dtype_code(out),
                                                m, n, k, kbps, splits, self._err_ptr, self._stream()), "gemm_tma")
                return out
        if library_parts > 1:
            parts, ks = library_parts, k // library_parts
            out = ws.buffer(tag, parts * m, n, torch.float32).view(parts, m, n)
            # slice p of the inner dimension: x[:, p ks : (p + 1) ks] and w[:, p ks : (p + 1) ks]^T, as views
            torch.bmm(x.view(m, parts, ks).permute(1, 0, 2), w.view(n, parts, ks).permute(1, 2, 0),
                      out_dtype=torch.float32, out=out)
            return out
        # A batch of decode tokens (17 to 256 rows): still a stream of weights; the tcgen05
        # kernel with the operands' roles swapped, cut along k like the few-row kernel.
        if (self.batch_gemm and self.FEW_ROWS < m <= self.batch_gemm_rows and x.is_contiguous()
                and w.is_contiguous() and self._gemm_tc5_ok(m, n, k)
                and -(-n // 128) <= self.batch_gemm_max_tiles and k >= self.batch_gemm_min_k
                and (not self.batch_gemm_one_round or (
                    allow_split and out is None and -(-n // 128) * self.tma_split(n, k)[1] <= self.sm_count))):
            per, splits = self.tma_split(n, k) if allow_split and out is None else (k // 64, 1)
            if splits > 1:
                out = ws.buffer(tag, splits * m, n, torch.float32).view(splits, m, n)
            elif out is None:
                out = ws.buffer(tag, m, n, out_dtype)
            self._check(self._gemm_tc5_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), _dtype_code(out),
                                            m, n, k, per, splits, self._err_ptr, self._stream()), "gemm_tc5")
            return out
        if out is None:
            out = ws.buffer(tag, m, n, out_dtype)
        if m == 0:
            return out
        if out.dtype == x.dtype:
            torch.mm(x, w.t(), out=out)
        else:
            torch.mm(x, w.t(), out_dtype=out.dtype, out=out)
        return out

    @_kind("rotary+cache")
    def rope_kv_write(self, qkv, positions, table, rotary_dim, q_out, k_cache, v_cache,
                      slot_mapping, nh, nkv, hd, page_size) -> None:
        if table is not None and table.shape[2] * 2 != rotary_dim:
            raise KernelError("rotary table does not match rotary_dim")
        if rotary_dim > hd or rotary_dim % 2:
            raise KernelError(f"rotary_dim {rotary_dim} must be even and at most head_dim {hd}")
        parts, stride = self._partials(qkv)
        self._check(self._rope_kv_write(
            qkv.data_ptr(), parts, stride, positions.data_ptr(), self._ptr(table), rotary_dim,
            0 if table is None else table.shape[0], q_out.data_ptr(), k_cache.data_ptr(),
            v_cache.data_ptr(), _dtype_code(q_out), self._ptr(slot_mapping), q_out.shape[0],
            nh, nkv, hd, page_size, k_cache.shape[0], self._err_ptr, self._stream()), "rope_kv_write")

    def _attention_lib(self, hd: int):
        """The tensor-core attention library for head size ``hd`` (built on first use)."""
        lib = self._attn_libs.get(hd)
        if lib is None:
            lib = ctypes.CDLL(str(build_attention(hd)))
            lib.ie_set_pdl(1 if self.pdl else 0)
            lib.ie_set_decode_pair(self.decode_cluster_max)
            lib.ie_set_decode_narrow(1 if self.decode_narrow else 0)
            P, I, F = c_void_p, c_int, c_float
            lib.ie_attention_decode.argtypes = [P, P, P, P, I, P, P, P, P, P, I, I, I, I, I, F, I, I, P, P]
            lib.ie_attention_prefill.argtypes = [P, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, P, P]
            lib.ie_attention_prefill_tc5.argtypes = [P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, I, F, I, I, P, P, P, P]
            lib.ie_attention_prefill_tc5_scratch_floats.argtypes = [I, I, I]
            lib.ie_attention_prefill_tc5_scratch_floats.restype = ctypes.c_longlong
            lib.ie_attention_prefill_tc5_ok.argtypes = [I, I]
            lib.ie_attention_decode_scratch_floats.argtypes = [I, I, I]
            lib.ie_attention_decode_scratch_floats.restype = ctypes.c_longlong
            lib.ie_attention_decode_balanced.argtypes = [P, P, P, P, I, P, P, P, P, P, I, I, I, I, I, F, I, I, P, P]
            lib.ie_attention_decode_ordered.argtypes = [P, P, P, P, I, P, P, P, P, P, I, I, I, I, I, F, I, I, P, I, P, P]
            lib.ie_attention_decode_balanced_scratch_floats.argtypes = [I, I, I]
            lib.ie_attention_decode_balanced_scratch_floats.restype = ctypes.c_longlong
            lib.ie_attention_decode_max_clusters.argtypes = [I]
            self._attn_libs[hd] = lib
        return lib

    def _decode_tickets(self, count: int):
        """Zeroed counters for the decode kernel's split merge; every launch leaves them zero."""
        if self._tickets is None or self._tickets.numel() < count:
            if self._tickets is not None:
                self._retired_tickets.append(self._tickets)  # captured launches may still point at it
            self._tickets = self.torch.zeros(max(count, 16384), dtype=self.torch.int32, device=self.device)
        return self._tickets

    def _clusters_at_once(self, hd: int, parts: int) -> int:
        """How many clusters of ``parts`` decode attention blocks the device runs at one time for
        head size ``hd`` (a cluster's blocks must find room in one group of SMs at the same
        time, so this is less than the SMs over ``parts``); 0: unknown."""
        key = (hd, parts)
        if key not in self._cluster_fit:
            self._cluster_fit[key] = int(self._attention_lib(hd).ie_attention_decode_max_clusters(parts))
        return self._cluster_fit[key]

    def decode_splits(self, num_seqs: int, nkv: int, table_tokens: int = 0, hd: int | None = None) -> int:
        """Into how many parts the decode kernel cuts each context.  One block per (request,
        key/value head) streams at an SM's full rate, so contexts are only cut when there are
        few such blocks (small batches).  2, 4 or 8 parts run as one thread-block cluster and
        merge through shared memory, which is worth more than the last few blocks: the count is
        rounded down to one of those (and to one of which the device runs all clusters at one
        time, if the head size ``hd`` is given), except for long contexts (``table_tokens``: what
        the step's block tables can hold), where as many parts as give nearly every SM a block
        stream faster, whichever way they merge.  The number depends on the batch and the tables'
        width alone, never on the contexts' lengths, so that a captured launch stays valid."""
        pairs = max(num_seqs * nkv, 1)
        if table_tokens > self.decode_cluster_tokens:
            # long contexts: a block for nearly every SM counts for more than the way the parts merge
            # (2 requests x 8 heads x 32,768 tokens: 9 parts 30.5 us, 8 parts 55, 4 parts 51)
            parts = max(1, min(self.sm_count // pairs, 16 if pairs >= 8 else 32))
            # blocks of four warps run two to an SM: where that fills the device much better than one
            # block of eight warps per SM (10 to 12 requests of 8 heads: 96 blocks for 148 SMs, or 288
            # for 296 slots), it is worth their dearer merge (12 x 8,192 tokens: 47 -> 42 us)
            halves = (2 * self.sm_count) // pairs
            if 1 < halves <= 32 and pairs * halves / (2 * self.sm_count) > 1.25 * pairs * parts / self.sm_count:
                parts = halves
            return parts
        parts = max(1, min(self.decode_split_target // pairs, 32))
        if self.decode_cluster_max < 2 or parts < 2:
            return parts
        parts = min(8 if parts >= 8 else 4 if parts >= 4 else 2, self.decode_cluster_max)
        # all clusters have to run at one time (16 clusters of 8 do not: a second round of blocks
        # doubled the kernel's time at batch 2); else the next smaller size
        while hd is not None and parts > 2 and 0 < self._clusters_at_once(hd, parts) < pairs:
            parts //= 2
        return parts

    BY_REQUEST, BY_LENGTH, SMALL_2, SMALL_3 = 0, 1, 2, 3  # how a decode step's attention is dealt (StepContext.ragged)

    def _decode_blocks_per_sm(self, hd: int, warps: int) -> int:
        key = (hd, warps)
        if key not in self._small_per_sm:
            self._small_per_sm[key] = int(self._attention_lib(hd).ie_attention_decode_blocks_per_sm(warps))
        return self._small_per_sm[key]

    @staticmethod
    def _by_request_estimate(by_length, at_once: int, scale: float, setup: float) -> float:
        """How long blocks dealt by request take, in tokens a four-warp block walks: ``by_length`` the
        contexts, the longest first, ``at_once`` of them on the device at one time, a block's time
        ``setup + scale * length``.  The requests beyond the first round start as those of the round
        before end, the shortest of them first."""
        if by_length[0] <= 1.1 * by_length[-1]:  # (about one length: whole rounds)
            return -(-len(by_length) // at_once) * (setup + scale * by_length[0])
        finish = []
        for i, n in enumerate(by_length):
            r, k = divmod(i, at_once)
            finish.append((finish[r * at_once - 1 - k] if r else 0.0) + setup + scale * n)
        return max(finish)

    def decode_dealing(self, ctx_lens, nkv: int, hd: int | None = None) -> int:
        """How the decode attention of a step over contexts of these lengths is dealt: key tiles by
        length (:meth:`decode_by_length`), or by request, and then in blocks of 3 or 2 warps (3 or 4 of
        them to an SM at head size 64, against 2 of the four-warp blocks) where the step's blocks then
        need fewer rounds over the device.  A block of w warps takes a set-up worth 300 tokens and
        4 / w of its context (in tokens a four-warp block walks; measured at 1,024 tokens: a round of
        four-warp blocks 13 us, of three-warp blocks 18, of two-warp blocks 24); the rounds are
        estimated by :meth:`_by_request_estimate`, and smaller blocks must be 7 % ahead.  Measured at
        head size 64, us per layer, four-warp blocks -> the choice: 40 requests x 1,024 tokens 25.8 ->
        17.9 (3 warps), 55 x 1,024 26.9 -> 19.6 (0.90 of the copy rate), 64 x 1,024 27.3 -> 24.8 (2 warps),
        80 x 1,024 40.0 -> 35.9 (3), 128 x 1,024 54.6 -> 49.4 (2), 160 x 1,024 68.1 -> 56.4 (3), 64 x 4,096
        96.4 -> 90.4, 64 x 256 10.4 -> 8.3, 40 of 768 to 1,280 tokens 22.1 -> 19.8; kept in four-warp blocks,
        the longest first: 48 of 512 to 1,536 tokens (19.5; 23.1 in three-warp blocks), 64 of 64 to 2,048
        (27.1; 43.6 in two-warp blocks)."""
        # (the answer is kept while the batch looks the same: as many contexts, the same longest and the
        # same sum, each to 64 tokens per request; the estimates cost 60 us at 64 requests, 220 at 256)
        count = len(ctx_lens)
        look = (count, nkv, hd, max(ctx_lens) >> 6 if count else 0, sum(ctx_lens) // (64 * max(count, 1)),
                self.decode_balanced, self.decode_small, self._force_small)
        if look == self._dealing_look:
            return self._dealing_answer
        self._dealing_look, self._dealing_answer = look, self._decode_dealing(ctx_lens, nkv, hd)
        return self._dealing_answer

    def _decode_dealing(self, ctx_lens, nkv: int, hd: int | None = None) -> int:
        dealt_by_length = self.decode_by_length(ctx_lens, nkv, hd)
        first = self.BY_LENGTH if dealt_by_length else self.BY_REQUEST
        if not self.decode_small or hd is None or hd not in ATTENTION_HEAD_DIMS or not ctx_lens:
            return first
        pairs = len(ctx_lens) * nkv
        if self._force_small and pairs > self.sm_count:
            return self._force_small
        usual = self._decode_blocks_per_sm(hd, 4)
        if pairs <= max(usual, 1) * self.sm_count or self.decode_balanced == "1":
            return first  # (one round of the usual blocks anyway; up to one block per SM: eight warps)
        by_length = sorted(ctx_lens, reverse=True)
        setup = 300.0
        best, best_time = self.BY_REQUEST, 0.93 * self._by_request_estimate(
            by_length, max(1, usual * self.sm_count // nkv), 1.0, setup)
        if dealt_by_length:  # (the smaller blocks then have to beat that kernel: 48 requests x 4,096 tokens
            # take 75.9 us dealt by length, 64.4 in three-warp blocks)
            best, best_time = self.BY_LENGTH, self._dealt_estimates(ctx_lens, nkv, hd)[1]
        for warps, code in ((3, self.SMALL_3), (2, self.SMALL_2)):
            per_sm = self._decode_blocks_per_sm(hd, warps)
            if per_sm <= usual:
                continue
            time = self._by_request_estimate(by_length, max(1, per_sm * self.sm_count // nkv), 4.0 / warps, setup)
            if time < best_time:
                best, best_time = code, time
        return best

    def _dealt_estimates(self, ctx_lens, nkv: int, hd: int | None = None) -> tuple[float, float]:
        """(dealt by request, dealt by length): how long the two decode attention kernels take for
        contexts of these lengths, in tokens one block walks (a block of eight warps up to one (request,
        head) pair per SM, of four warps, two to an SM, beyond).  By request the step lasts as long as
        the longest context over its splits (twice that where the splits make more blocks than SMs:
        those blocks have four warps; and a set-up more where they merge through memory), or the whole
        work over the blocks the device runs at once, if that is more.  By length: what that kernel's own
        dealing gives the slowest block (below).  Measured, us per
        layer, by request / by length, with the estimate's answer: 12 requests x 4,096 tokens 25.8 / 33.4
        (by request), 11 x 2,048 12.8 / 19.5 (by request), 7 x 32,768 98.7 / 85.9 (by length), 10 x 8,192
        41.0 / 36.4 (by length), 24 x 8,192 92.8 / 74.4 (by length), 28 x 8,192 94.3 / 85.6 (by length),
        32 x 8,192 95.4 / 97.0 (by request), 20 x 4,096 47.6 / 37.3 (by length), 24 x 4,096 48.0 / 41.9 (by
        length), 28 x 4,096 48.5 / 47.8 (by request), 24 x 2,048 25.4 / 35.0 (by request), 40 of 128 to
        2,048 tokens 26 / 34 (by request), 9 x 4,096 25.1 / 18.5 (by length: two pieces per pair, one
        round); 14 x 8,192 49.5 / 47.1 is answered by request."""
        pairs = len(ctx_lens) * nkv
        work = sum(ctx_lens) * nkv
        longest = max(ctx_lens)
        slots = self.sm_count if pairs <= self.sm_count else 2 * self.sm_count
        table_tokens = 1024  # (what the step's block tables hold: widths double from 64 pages of 16 tokens)
        while table_tokens < longest:
            table_tokens *= 2
        splits = self.decode_splits(len(ctx_lens), nkv, table_tokens, hd)
        # blocks run in rounds over the slots; the last round is as long as a block even when few
        # blocks are in it (40 requests x 8 heads of 4,096 tokens, 320 blocks on 296 slots: 93 us by
        # request, 65 us by length)
        if pairs <= self.sm_count:
            by_request = longest / splits
            if pairs * splits > self.sm_count:   # (the splits' blocks have four warps)
                by_request = 2 * by_request * -(-pairs * splits // (2 * self.sm_count))
            if splits not in (1, 2, 4, 8):       # (merged through memory by the block that ends last)
                by_request += 1536
            by_request = max(by_request, work / slots)
        else:
            rounds = pairs * splits / slots
            last_round = (-(-pairs * splits // slots) - rounds) * work / (pairs * splits)
            by_request = max(longest / splits, work / slots + last_round)
        # By length, as that kernel deals (attention_mma.cu): every pair's tiles in pieces of about an
        # even share, dealt in rounds over the blocks, or, where the pieces would leave the slowest block
        # well behind, equal ranges of the list of all tiles, which lie in 1 + pairs / blocks stretches
        # of different pairs on average.  A piece or stretch costs six tiles per warp to set up.
        warps, keys = (8 if pairs <= self.sm_count else 4), (32 if hd is None or hd <= 64 else 16)  # (keys per tile)
        tiles = [-(-c // keys) for c in ctx_lens]
        share = max(-(-sum(tiles) * nkv // slots), warps)
        pieces = [max(1, min((n + share // 2) // share, n // warps)) for n in tiles]
        largest = max(-(-n // k) for n, k in zip(tiles, pieces))
        piece_rounds = -(-sum(pieces) * nkv // slots)
        setup = 6 * warps
        if piece_rounds * largest > share + setup:
            by_length = share + setup * (1 + pairs / slots)
        else:  # (the blocks that take a second piece are few when the pieces are few more than the blocks)
            by_length = max(1.0, sum(pieces) * nkv / slots) * (largest + setup)
        return by_request, by_length * keys

    def decode_by_length(self, ctx_lens, nkv: int, hd: int | None = None) -> bool:
        """Whether a decode step over contexts of these lengths should use the kernel that deals
        key tiles by length (:meth:`_dealt_estimates`)."""
        if self.decode_balanced in ("0", "1"):
            return self.decode_balanced == "1"
        by_request, by_length = self._dealt_estimates(ctx_lens, nkv, hd)
        return by_request > by_length

    def prefill_key_split(self, blocks: int, hd: int, max_ctx_len: int) -> int:
        """Among how many blocks the tcgen05 prefill kernel shares the keys of a query tile: the
        count that costs least by this estimate, in key tiles one block walks: rounds of blocks over
        the device, each block its share of the longest context's key tiles plus a start and end
        worth six, and for the block that adds the shares three key tiles and 1.1 per share
        (measured, a 128-token portion at 2,048 tokens, us for 1 / 2 / 4 / 8 shares: 23.9 / 18.5 / 17.0 /
        19.0; at 8,192 tokens: 81 / 47.6 / 36.8 / 29.5; a 512-token portion at 8,192: 103 / 65 / 72 / 82);
        if that saves a quarter of the time and leaves every block four key tiles; 1 when the tiles
        fill the device anyway."""
        slots = self.sm_count * (2 if hd == 64 else 1)
        if blocks <= 0 or blocks >= slots:
            return 1
        key_tiles = max(max_ctx_len // 64, 1)

        def cost(ks: int) -> float:
            rounds = -(-blocks * ks // slots)
            return rounds * (key_tiles / ks + 6.0) + (3.0 + 1.1 * ks if ks > 1 else 0.0)

        limit = max(1, min(16, max_ctx_len // 256))
        least = min(cost(ks) for ks in range(1, limit + 1))
        best = next(ks for ks in range(1, limit + 1) if cost(ks) <= 1.05 * least)  # (the fewest shares among the near-best)
        return best if cost(best) <= 0.75 * cost(1) else 1

    def paged_attention(self, q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, page_size,
                        scale, window, out, ragged: bool | None = None, value_dim: int | None = None) -> None:
        """Attention of every token of the step over its request's cached keys and values.
        bfloat16 with a head size the tensor-core kernels take and at most 16 query heads per
        key/value head: requests with few rows go to the split decode kernel, longer portions
        to the prefill kernel.  Everything else (32-bit, other head sizes) runs the general
        kernel, whose order of operations does not depend on the batch."""
        if nkv < 1 or nh % nkv:
            raise KernelError(f"{nh} query heads cannot share {nkv} key/value heads")
        if value_dim is not None and value_dim != hd:
            # value rows shorter than key rows (a shared latent row whose first entries are the value)
            return self.latent_paged_attention(q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, value_dim,
                                               page_size, scale, window, out)
        if hd % 8 or hd > 256:
            raise KernelError(f"head_dim {hd} is not supported: it must be a multiple of 8, at most 256")
        groups = nh // nkv
        if q.dtype == self.torch.bfloat16 and hd in ATTENTION_HEAD_DIMS and groups <= 16:
            lib = self._attention_lib(hd)
            # which requests go to which kernel: the same for every layer of the step
            # (kept on the step's context, one per (heads per key/value head, head size): mixers
            # of different shapes in one model each get their own)
            plans = getattr(ctx, "_attention_plans", None)
            if plans is None:
                plans = ctx._attention_plans = {}
            plan = plans.get((groups, hd))
            bounds = getattr(ctx, "bounds", None)
            if plan is None and bounds is not None:
                # a launch of fixed size (a captured step): both kernels, over as many query tiles
                # as any step within the bounds can have; each kernel skips the other's requests
                tokens, seqs, max_ctx = bounds
                rows = lib.ie_attention_prefill_rows()
                tiles = seqs + tokens // rows
                # (the keys of a tile may be shared among blocks here too: how many is decided from the
                # bounds alone, for the tiles a step of so many tokens usually has: one request's portion
                # and little else; blocks for tiles that a step does not have leave at once)
                likely = tokens // rows + min(seqs, 2)
                plan = plans[(groups, hd)] = {"any": True, "all": False, "tiles": tiles, "tile_pairs": tiles,
                                              "max_ctx": max_ctx, "likely_tiles": likely}
            if plan is None:
                small = [ql * groups <= 16 for ql in ctx.q_lens]
                plan = {"small": small, "any": any(small), "all": all(small)}
                if not plan["all"]:
                    rows = lib.ie_attention_prefill_rows()
                    per_seq = [-(-ql // rows) for ql, s in zip(ctx.q_lens, small) if not s]
                    plan["tiles"] = sum(per_seq)
                    plan["tile_pairs"] = sum(-(-t // 2) for t in per_seq)
                plans[(groups, hd)] = plan
            args = (q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, page_size, scale, window, out)
            if plan["any"]:
                if ragged is None:
                    ragged = max(getattr(ctx, "ragged", ()) or (0,))
                self._decode_attention(lib, int(ragged) if bounds is None else self.BY_REQUEST, *args)
            if not plan["all"]:
                self._prefill_attention(lib, plan, *args)
            return
        self.paged_attention_general(q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, page_size,
                                     scale, window, out)

    def _scratch(self, ctx, name: str, floats: int, device):
        ws = getattr(ctx, "ws", None)
        if ws is not None:
            # (one row of exactly what is asked for, rounded up so that it seldom has to grow: the
            # workspace's own floor of rows is for per-token buffers)
            size = max(1 << max(int(floats) - 1, 0).bit_length(), 1 << 22)  # (16 MB at least: most steps never outgrow it)
            return ws.buffer(name, 1, size, self.torch.float32, rows_cap=None)[:, :floats]
        return self.torch.empty(floats, dtype=self.torch.float32, device=device)

    @_kind("attention.decode")
    def _decode_attention(self, lib, ragged, q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, page_size, scale,
                          window, out) -> None:
        """The requests with few rows (the kernels skip the others): key tiles dealt by length
        when the step's context says its lengths differ much, else by request."""
        total_pages, stream = k_cache.shape[0], self._stream()
        by_length = self.decode_balanced == "1" or (self.decode_balanced == "auto" and ragged == self.BY_LENGTH)
        if by_length and ctx.num_seqs <= lib.ie_attention_decode_balanced_max_seqs():
            per_pair = self.decode_balanced_blocks_per_pair
            floats = lib.ie_attention_decode_balanced_scratch_floats(ctx.num_seqs, nkv, per_pair)
            scratch = self._scratch(ctx, "attn.partial", floats, q.device)
            tickets = self._decode_tickets(ctx.num_seqs * nkv)
            self._check(lib.ie_attention_decode_balanced(
                q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(),
                block_tables.shape[1], ctx.cu_q.data_ptr(), ctx.ctx_lens.data_ptr(), out.data_ptr(),
                scratch.data_ptr(), tickets.data_ptr(), ctx.num_seqs, nh, nkv, page_size,
                total_pages, scale, window, per_pair, self._err_ptr, stream), "attention_decode_balanced")
            self.balanced_launches += 1
            return
        splits = self.decode_splits(ctx.num_seqs, nkv, block_tables.shape[1] * page_size, hd)
        floats = lib.ie_attention_decode_scratch_floats(ctx.num_seqs, nkv, splits)
        scratch = tickets = None
        if floats:
            scratch = self._scratch(ctx, "attn.partial", floats, q.device)
            tickets = self._decode_tickets(ctx.num_seqs * nkv)
        self._check(lib.ie_attention_decode_ordered(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(),
            block_tables.shape[1], ctx.cu_q.data_ptr(), ctx.ctx_lens.data_ptr(), out.data_ptr(),
            self._ptr(scratch), self._ptr(tickets), ctx.num_seqs, nh, nkv, page_size,
            total_pages, scale, window, splits, self._ptr(getattr(ctx, "decode_order", None)),
            ragged if ragged in (self.SMALL_2, self.SMALL_3) and splits == 1 else 0, self._err_ptr, stream),
            "attention_decode")

    @_kind("attention.prefill")
    def _prefill_attention(self, lib, plan, q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, page_size,
                           scale, window, out) -> None:
        """The requests with more than 16 rows, in query tiles of `ie_attention_prefill_rows` tokens."""
        total_pages, stream = k_cache.shape[0], self._stream()
        tiles = plan["tiles"]
        fixed = "max_ctx" in plan  # a launch of fixed size: nothing is decided from the step's own lengths
        max_ctx = plan["max_ctx"] if fixed else ctx.max_ctx_len
        if self.attn_tc5 and lib.ie_attention_prefill_tc5_ok(page_size, max_ctx):
            # Head sizes 64 and 128, pages of 8 tokens or more: the tcgen05 / TMEM / TMA kernel.
            # While the blocks would fill the GPU less than about twice, a block takes two tiles
            # of a request, a late (long) and an early (short) one.  With so few tiles that even
            # then much of the GPU would idle (a short portion of a long prompt), the keys of
            # every tile are shared among several blocks instead.
            ksplit = 1
            if self.prefill_key_splits:
                ksplit = self.prefill_key_split((plan["likely_tiles"] if fixed else tiles) * nh, hd, max_ctx)
            # (pairs of tiles only where single tiles would take more than one round of blocks: two
            # prompts of 256 tokens took 11.2 us in pairs, 8.3 in single tiles; eight of them 14.9 and 17.5)
            slots = self.sm_count * (2 if hd == 64 else 1)
            paired = (not fixed and ksplit == 1 and slots < tiles * nh <= self.prefill_paired_max * self.sm_count)
            # (portions at the end of long contexts: their tiles see about as many keys each, and pairs
            # would only halve the blocks where those do not fill the device anyway: two 512-token
            # portions at 65,536 tokens took 1,602 us in 128 blocks of two tiles, 826 in 256 of one)
            if paired and ctx.max_ctx_len >= 2 * max(ctx.q_lens) and plan["tile_pairs"] * nh < slots:
                paired = False
            if paired:
                tiles = plan["tile_pairs"]
            scratch = tickets = None
            if ksplit > 1:
                floats = lib.ie_attention_prefill_tc5_scratch_floats(tiles, nh, ksplit)
                scratch = self._scratch(ctx, "attn.prefill_partial", floats, q.device)
                tickets = self._decode_tickets(max(tiles * nh, ctx.num_seqs * nkv))
            self._check(lib.ie_attention_prefill_tc5(
                q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(),
                block_tables.shape[1], ctx.cu_q.data_ptr(), ctx.ctx_lens.data_ptr(), out.data_ptr(),
                ctx.num_tokens, ctx.num_seqs, tiles, 1 if paired else 0, nh, nkv, page_size, total_pages,
                scale, window, ksplit, self._ptr(scratch), self._ptr(tickets), self._err_ptr, stream),
                "attention_prefill_tc5")
            return
        self._check(lib.ie_attention_prefill(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(),
            block_tables.shape[1], ctx.cu_q.data_ptr(), ctx.ctx_lens.data_ptr(), out.data_ptr(),
            ctx.num_seqs, tiles, nh, nkv, page_size, total_pages, scale, window,
            self._err_ptr, stream), "attention_prefill")

    @_kind("attention.general")
    def paged_attention_general(self, q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd,
                                page_size, scale, window, out) -> None:
        self._check(self._paged_attention_generic(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), _dtype_code(q),
            block_tables.data_ptr(), block_tables.shape[1], ctx.seq_of_token.data_ptr(),
            ctx.positions.data_ptr(), out.data_ptr(), ctx.num_tokens, nh, nkv, hd, hd, hd, page_size,
            k_cache.shape[0], scale, window, 0, None, None, None, 0, 0.0, 0, self._err_ptr, self._stream()), "paged_attention")

    @_kind("attention.latent")
    def latent_paged_attention(self, q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, value_dim,
                               page_size, scale, window, out) -> None:
        """Attention whose value rows are the first ``value_dim`` entries of ``v_cache``'s rows
        (``v_cache`` may be the key cache itself); ``out`` is ``[N, nh * value_dim]``."""
        if not 0 < value_dim <= 512:
            raise KernelError(f"value rows of {value_dim} entries are not supported (1 to 512)")
        if (q.dtype == self.torch.bfloat16 and nkv == 1 and window == 0 and v_cache is k_cache
                and self.latent_mma and self._part_lib("latent").ie_latent_attention_mma_ok(hd, value_dim)):
            # one shared row per token, values inside the key rows: the tensor-core kernel; a context is
            # cut into ranges of key tiles while the blocks are few (from the batch and the tables'
            # width alone, so that a captured launch stays valid)
            lib = self._part_lib("latent")
            bounds = getattr(ctx, "bounds", None)
            longest = bounds[0] if bounds is not None else ctx.max_q_len
            rows = lib.ie_latent_attention_rows(longest * nh)
            max_tiles = -(-longest * nh // rows)
            blocks = max_tiles * ctx.num_seqs
            table_tokens = block_tables.shape[1] * page_size
            splits = max(1, min(self.sm_count // blocks, table_tokens // 128, 16))
            scratch = None
            if splits > 1:
                scratch = self._scratch(ctx, "attn.latent_partial", ctx.num_tokens * nh * splits * (value_dim + 2), q.device)
            self._check(lib.ie_latent_attention_mma(
                q.data_ptr(), k_cache.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], ctx.cu_q.data_ptr(),
                ctx.ctx_lens.data_ptr(), out.data_ptr(), self._ptr(scratch), ctx.num_tokens, ctx.num_seqs, max_tiles,
                rows, nh, hd, value_dim, page_size, k_cache.shape[0], scale, splits, self._err_ptr, self._stream()),
                "latent_attention_mma")
            return
        self._check(self._paged_attention_generic(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), _dtype_code(q),
            block_tables.data_ptr(), block_tables.shape[1], ctx.seq_of_token.data_ptr(),
            ctx.positions.data_ptr(), out.data_ptr(), ctx.num_tokens, nh, nkv, hd, value_dim,
            v_cache.shape[-1], page_size, k_cache.shape[0], scale, window, 0, None, None, None, 0, 0.0, 0,
            self._err_ptr, self._stream()), "paged_attention_latent")

    # --- kernels of single mixers and feed-forwards (libraries built on first use) -------------

    _PART_SIGNATURES = {
        "latent": {
            "ie_latent_prep": "P I P P I I P F P P P P I P I I I I I I P P",
            "ie_headwise_linear": "P L L P P L L P I I I I I P",
            "ie_scale_head_rows": "P L L P I I I P",
            "ie_latent_attention_mma_ok": "I I",
            "ie_latent_attention_mma": "P P P I P P P P I I I I I I I I I F I P P",
            "ie_latent_attention_rows": "I",
        },
        "delta": {
            "ie_delta_prep": "P I P P P P P L P P P P P P P P I I I I I I I I P P",
            "ie_delta_rule": "P P P P P P L P P P I I I I I I P",
            "ie_gated_rms_heads": "P P F P P I L I P",
        },
        "routed": {
            "ie_route_topk": "P I P P I I I I I I I P I F P P P",
            "ie_routed_max_tiles": "I I",
            "ie_routed_align": "P I I P P P I P",
            "ie_routed_gate_up": "P P P I P P P I I I I F I F F P",
            "ie_routed_down": "P P P P I P P P I I I I I P",
        },
        "recurrent": {
            "ie_short_conv_residual": "P I P P L P P P P I I I I I P P",
            "ie_hgrn2_gates": "P I P P P I I P",
            "ie_mlstm_gates": "P P I P P F P L L P P P I I I P",
            "ie_gated_recurrence": "P I P I P I P P I P L P P P I I I I I F I P",
            "ie_recurrence_readout": "P I P P I F P I I P I L I I P",
            "ie_lowrank_decay": "P I P P F P I I I P",
        },
        "gated_attn": {
            "ie_qk_norm_rope_write": "P I P P I I P I I I P P F P P P I P I I I I I I I P P",
        },
    }

    def _part_lib(self, name: str):
        lib = self._part_libs.get(name)
        if lib is None:
            path = build_part_library(name)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as exc:
                raise KernelError(f"the kernel library {path} could not be loaded: {exc}") from exc
            kinds = {"P": c_void_p, "I": c_int, "F": c_float, "L": ctypes.c_longlong}
            for fn_name, sig in self._PART_SIGNATURES[name].items():
                fn = getattr(lib, fn_name)
                fn.argtypes, fn.restype = [kinds[k] for k in sig.split()], c_int
            self._part_libs[name] = lib
        return lib

    @_kind("latent.prep")
    def latent_prep(self, proj, positions, table, rot_dims, norm_w, eps, q_plain, q_abs, gate, cache,
                    slot_mapping, heads, dim, rot_dim, rank, page_size) -> None:
        """The latent attention's input stage (see ``csrc/latent_attention.cu``).  ``proj``: the fused
        projection's 32-bit output ``[N, heads * (dim + rot_dim) + rank + rot_dim + heads]``;
        ``cache``: ``[pages, 1, page_size, rank + rot_dim]``."""
        if table is not None and table.shape[2] * 2 != rot_dims:
            raise KernelError("rotary table does not match the rotated dims")
        if proj.dtype != self.torch.float32 or proj.dim() != 2 or not proj.is_contiguous():
            raise KernelError("latent_prep reads a contiguous 32-bit projection")
        if proj.shape[1] != heads * (dim + rot_dim) + rank + rot_dim + heads or cache.shape[-1] != rank + rot_dim:
            raise KernelError("latent_prep: the projection or the cache rows do not fit the sizes")
        total_slots = cache.shape[0] * page_size
        self._check(self._part_lib("latent").ie_latent_prep(
            proj.data_ptr(), proj.shape[1], positions.data_ptr(), self._ptr(table), rot_dims,
            0 if table is None else table.shape[0], norm_w.data_ptr(), eps, q_plain.data_ptr(), q_abs.data_ptr(),
            gate.data_ptr(), cache.data_ptr(), _dtype_code(q_abs), self._ptr(slot_mapping), proj.shape[0],
            heads, dim, rot_dim, rank, total_slots, self._err_ptr, self._stream()), "latent_prep")

    HEADWISE_LIBRARY_ROWS = 128  # from this many rows on the per-head products go to the library (bfloat16)

    @_kind("latent.headwise")
    def headwise_linear(self, x, w, out, row_scale=None) -> None:
        """``out[n, h, :] = w[h] @ x[n, h, :]`` (times ``row_scale[n, h]``): ``x`` ``[N, H, K]`` and
        ``out`` ``[N, H, O]`` may be views with any token and head strides (entries contiguous),
        ``w`` is ``[H, O, K]`` contiguous; 32-bit sums."""
        n, heads, k = x.shape
        o = w.shape[1]
        if (x.stride(2) != 1 or out.stride(2) != 1 or not w.is_contiguous() or w.shape != (heads, o, k)
                or out.shape != (n, heads, o) or x.dtype != w.dtype or out.dtype != w.dtype):
            raise KernelError("headwise_linear: shapes, strides or dtypes do not fit")
        if x.dtype == self.torch.bfloat16 and n >= self.HEADWISE_LIBRARY_ROWS and o % 8 == 0 and k % 8 == 0:
            # many rows: one strided batched product of the library over the heads, written in place
            # (both views are batches of row-major matrices with a leading dimension), then the factors
            self.torch.bmm(x.permute(1, 0, 2), w.transpose(1, 2), out=out.permute(1, 0, 2))
            if row_scale is not None:
                self._check(self._part_lib("latent").ie_scale_head_rows(
                    out.data_ptr(), out.stride(0), out.stride(1), row_scale.data_ptr(), n, heads, o,
                    self._stream()), "scale_head_rows")
            return
        self._check(self._part_lib("latent").ie_headwise_linear(
            x.data_ptr(), x.stride(0), x.stride(1), w.data_ptr(), out.data_ptr(), out.stride(0), out.stride(1),
            self._ptr(row_scale), _dtype_code(x), n, heads, o, k, self._stream()), "headwise_linear")

    @_kind("delta.prep")
    def delta_prep(self, qkvb, a, conv_w, A_log, dt_bias, state, slots, ctx, q_out, k_out, v_out, beta,
                   decay, heads, kv_heads, dim, vdim, taps) -> None:
        """Convolutions, unit norms, step sizes and decays of the gated delta rule, and the slots'
        kept convolution inputs moved on (see ``csrc/delta_rule.cu``).  ``state``: ``[slots, floats]``."""
        channels = 2 * kv_heads * dim + heads * vdim
        if qkvb.shape[1] != channels + heads or conv_w.shape != (channels, taps):
            raise KernelError("delta_prep: the projection or the convolution weights do not fit the sizes")
        self._check(self._part_lib("delta").ie_delta_prep(
            qkvb.data_ptr(), qkvb.shape[1], a.data_ptr(), conv_w.data_ptr(), A_log.data_ptr(), dt_bias.data_ptr(),
            state.data_ptr(), state.stride(0), slots.data_ptr(), ctx.seq_of_token.data_ptr(), ctx.cu_q.data_ptr(),
            q_out.data_ptr(), k_out.data_ptr(), v_out.data_ptr(), beta.data_ptr(), decay.data_ptr(),
            qkvb.shape[0], ctx.num_seqs, heads, kv_heads, dim, vdim, taps, state.shape[0], self._err_ptr,
            self._stream()), "delta_prep")
        self.launches += 1 if taps > 1 else 0

    @_kind("delta.rule")
    def delta_rule(self, q, k, v, beta, decay, state, slots, ctx, out, heads, kv_heads, dim, vdim) -> None:
        """The recurrence itself: every request's tokens of this step in order, from and to its slot."""
        if dim > 512:
            raise KernelError(f"the delta rule kernel takes key sizes up to 512, not {dim}")
        self._check(self._part_lib("delta").ie_delta_rule(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), beta.data_ptr(), decay.data_ptr(), state.data_ptr(),
            state.stride(0), slots.data_ptr(), ctx.cu_q.data_ptr(), out.data_ptr(), ctx.num_seqs, heads,
            kv_heads, dim, vdim, state.shape[0], self._stream()), "delta_rule")

    @_kind("delta.out")
    def gated_rms_heads(self, o, weight, eps, gate_pre, out, heads, vdim) -> None:
        """``out = o / rms(o) * weight * sigmoid(gate_pre)`` per (token, head) over ``vdim``."""
        self._check(self._part_lib("delta").ie_gated_rms_heads(
            o.data_ptr(), weight.data_ptr(), eps, gate_pre.data_ptr(), out.data_ptr(), _dtype_code(out),
            o.shape[0] * heads, vdim, self._stream()), "gated_rms_heads")

    @_kind("routed.route")
    def route_topk(self, x, w_router, groups, keep, ids, weights, bias=None, scoring: str = "softmax",
                   correction=None, group_top: int = 1, weight_scale: float = 1.0) -> None:
        """Softmax scores (of the router's logits plus ``bias``, if given), group limit and the ``top``
        experts per token with their normalised weights, times ``weight_scale``.  ``scoring="sigmoid"``:
        the scores are the logits' sigmoids; ``correction`` (one number per expert) is added to them
        for the choice of groups and experts only, and a group is ranked by its best ``group_top``
        (1 or 2) corrected scores added up."""
        if scoring not in ("softmax", "sigmoid"):
            raise KernelError(f"route_topk: no scoring {scoring!r}")
        if correction is not None and (correction.dtype != self.torch.float32 or correction.numel() != w_router.shape[0]):
            raise KernelError("route_topk: the correction is one 32-bit number per expert")
        self._check(self._part_lib("routed").ie_route_topk(
            x.data_ptr(), _dtype_code(x), w_router.data_ptr(), self._ptr(bias), x.shape[0], x.shape[1], w_router.shape[0],
            ids.shape[1], groups, keep, 1 if scoring == "sigmoid" else 0, self._ptr(correction), int(group_top),
            float(weight_scale), ids.data_ptr(), weights.data_ptr(), self._stream()), "route_topk")

    def routed_experts(self, x, ids, weights, w_gate_up, w_down, *, limit, alpha, up_offset, ws, tag="moe"):
        """The chosen experts' weighted outputs as ``[top, N, hidden]`` 32-bit slices (to be added in
        order).  ``w_gate_up``: ``[experts, 2, ff, hidden]``, ``w_down``: ``[experts, hidden, ff]``."""
        torch = self.torch
        lib = self._part_lib("routed")
        n, top = ids.shape
        experts, _, ff, hidden = w_gate_up.shape
        pairs = n * top
        max_tiles = lib.ie_routed_max_tiles(pairs, experts)
        rows = max_tiles * lib.ie_routed_tile_rows()
        index = ws.buffer(tag + ".index", 1, rows + max_tiles + 4, torch.int32, rows_cap=None)[0]
        sorted_pairs, tile_expert, meta = index[:rows], index[rows: rows + max_tiles], index[rows + max_tiles:]
        y = ws.buffer(tag + ".act", pairs, ff, x.dtype)
        out = ws.buffer(tag + ".delta", pairs, hidden, torch.float32).view(top, n, hidden)
        self._routed_align(lib, ids, pairs, experts, sorted_pairs, tile_expert, meta, max_tiles)
        self._routed_gate_up(lib, x, w_gate_up, y, sorted_pairs, tile_expert, meta, max_tiles, top, hidden, ff,
                             limit, alpha, up_offset)
        self._routed_down(lib, y, w_down, out, weights, sorted_pairs, tile_expert, meta, max_tiles, top, n, ff, hidden)
        return out

    @_kind("routed.align")
    def _routed_align(self, lib, ids, pairs, experts, sorted_pairs, tile_expert, meta, max_tiles) -> None:
        self._check(lib.ie_routed_align(ids.data_ptr(), pairs, experts, sorted_pairs.data_ptr(),
                                        tile_expert.data_ptr(), meta.data_ptr(), max_tiles, self._stream()),
                    "routed_align")

    @_kind("routed.gate_up")
    def _routed_gate_up(self, lib, x, w, y, sorted_pairs, tile_expert, meta, max_tiles, top, hidden, ff, limit,
                        alpha, up_offset) -> None:
        self._check(lib.ie_routed_gate_up(
            x.data_ptr(), w.data_ptr(), y.data_ptr(), _dtype_code(x), sorted_pairs.data_ptr(),
            tile_expert.data_ptr(), meta.data_ptr(), max_tiles, top, hidden, ff,
            0.0 if limit is None else float(limit), 0 if limit is None else 1, alpha, up_offset,
            self._stream()), "routed_gate_up")

    @_kind("routed.down")
    def _routed_down(self, lib, y, w, out, weights, sorted_pairs, tile_expert, meta, max_tiles, top, n, ff,
                     hidden) -> None:
        self._check(lib.ie_routed_down(
            y.data_ptr(), w.data_ptr(), out.data_ptr(), weights.data_ptr(), _dtype_code(y),
            sorted_pairs.data_ptr(), tile_expert.data_ptr(), meta.data_ptr(), max_tiles, top, n, ff, hidden,
            self._stream()), "routed_down")

    # --- residual-stream operations of models with norms on both sides of a sublayer ------------

    @_kind("embedding")
    def bigram_embedding(self, embed, bigram, ids, ctx, state, slots, out, buckets, mul_prev, mul_cur) -> None:
        """``out[n] = embed[id] + bigram[(prev * mul_prev + id * mul_cur) mod buckets]`` (row ``buckets``
        for a request's first token).  ``state``: ``[slots, 1]``, the request's last token as the
        integer's bits; moved on to the last token of this step."""
        if bigram.shape[0] != buckets + 1 or bigram.dtype != embed.dtype or state.dtype != self.torch.float32:
            raise KernelError("bigram_embedding: the table or the state does not fit")
        self._check(self._bigram_embedding(
            embed.data_ptr(), bigram.data_ptr(), _dtype_code(embed), ids.data_ptr(), ctx.positions.data_ptr(),
            ctx.seq_of_token.data_ptr(), ctx.cu_q.data_ptr(), slots.data_ptr(), state.data_ptr(), state.stride(0),
            state.shape[0], out.data_ptr(), ids.shape[0], embed.shape[1], embed.shape[0], buckets, mul_prev,
            mul_cur, self._err_ptr, self._stream()), "bigram_embedding")

    @_kind("norm")
    def sandwich_norm(self, h, delta, bias, post_weight, post_eps, weight, eps, out, rows=None, second=None,
                      extra=None) -> None:
        """``y = delta (+ second) (+ bias) (+ extra)``; ``y <- rms(y) * post_weight`` if given; ``h += y``
        (not with ``rows``); ``out = rms(h) * weight`` unless ``out`` is None.  ``delta`` may be None.
        ``second``: another sublayer's output, whole or in parts like ``delta``; ``extra``: a 32-bit array
        of the stream's shape, added row by row."""
        n = h.shape[0] if rows is None else rows.shape[0]
        parts, stride = self._partials(delta)
        parts2, stride2 = self._partials(second)
        if extra is not None and (extra.dtype != self.torch.float32 or tuple(extra.shape) != tuple(h.shape)
                                  or not extra.is_contiguous()):
            raise KernelError("sandwich_norm: the extra rows must be a 32-bit array like the stream")
        self._check(self._sandwich_norm(
            h.data_ptr(), self._ptr(delta), parts, stride, self._ptr(second), parts2 if second is not None else 0,
            stride2, self._ptr(extra), self._ptr(bias), self._ptr(post_weight), post_eps,
            self._ptr(weight), eps, self._ptr(out), _dtype_code(out) if out is not None else 0, self._ptr(rows), n,
            h.shape[1], self._stream()), "sandwich_norm")

    @_kind("activation")
    def silu_mul_bias(self, gate_up, bias, out) -> None:
        """``out = silu(g + bias_g) * (u + bias_u)`` from rows of gates, then ups (32-bit or ``out``'s
        dtype); biases and activation in 32-bit."""
        if gate_up.dtype not in (self.torch.float32, out.dtype) or gate_up.shape[1] != 2 * out.shape[1]:
            raise KernelError("silu_mul_bias reads rows of gates and ups, 32-bit or of the output's dtype")
        self._check(self._silu_mul_bias(gate_up.data_ptr(), _dtype_code(gate_up), self._ptr(bias), out.data_ptr(),
                                        _dtype_code(out), out.shape[0], out.shape[1], self._stream()), "silu_mul_bias")

    @_kind("stream")
    def concat_cast(self, a, b, out) -> None:
        """``out[n] = [a[n]; b[n]]`` from two 32-bit ``[N, width]`` arrays, in ``out``'s dtype."""
        self._check(self._concat_cast(a.data_ptr(), b.data_ptr(), out.data_ptr(), _dtype_code(out), a.shape[0],
                                      a.shape[1], self._stream()), "concat_cast")

    @_kind("stream")
    def weighted_sum(self, a, sa: float, b, sb: float, out) -> None:
        """``out = sa * a + sb * b`` for contiguous 32-bit tensors of one shape."""
        self._check(self._weighted_sum(a.data_ptr(), float(sa), b.data_ptr(), float(sb), out.data_ptr(), a.numel(),
                                       self._stream()), "weighted_sum")

    @_kind("norm")
    def gated_add_norm(self, h, delta, gate_pre, gate_bias, weight, eps, out, rows=None) -> None:
        """``h += sigmoid(gate_pre + gate_bias) * delta`` element by element (not with ``rows``, which
        selects rows and leaves ``h``); ``out = rms(h) * weight`` unless ``out`` is None.  ``delta`` may be
        the parts of a split product (``[S, N, hidden]``), and so may ``gate_pre`` (32-bit, ``[N, hidden]``
        or ``[S', N, hidden]``); a two-dimensional ``gate_pre`` may be some columns of a wider array."""
        if (gate_pre.dtype != self.torch.float32 or tuple(gate_pre.shape[-2:]) != tuple(h.shape)
                or gate_pre.stride(-1) != 1 or (gate_pre.dim() == 3 and not gate_pre.is_contiguous())):
            raise KernelError("gated_add_norm: the gate's pre-activation must be a 32-bit array like the stream")
        n = h.shape[0] if rows is None else rows.shape[0]
        parts, stride = self._partials(delta)
        gate_parts, gate_stride = self._partials(gate_pre)
        self._check(self._gated_add_norm(
            h.data_ptr(), delta.data_ptr(), parts, stride, gate_pre.data_ptr(), gate_parts, gate_stride,
            gate_pre.stride(-2), self._ptr(gate_bias),
            self._ptr(weight), eps, self._ptr(out), _dtype_code(out) if out is not None else 0, self._ptr(rows), n,
            h.shape[1], self._stream()), "gated_add_norm")

    @_kind("activation")
    def polynorm(self, z, coeff, eps, out) -> None:
        """``out = a N(z) + b N(z^2) + c N(z^3) + e`` per row with ``coeff = (a, b, c, e)`` and ``N`` the
        division by the root mean square over the row; ``z`` is 32-bit or has ``out``'s dtype, and may
        be the first columns of a wider array."""
        if z.dtype not in (self.torch.float32, out.dtype) or z.shape != out.shape or z.stride(1) != 1:
            raise KernelError("polynorm reads rows of unit stride, 32-bit or of the output's dtype")
        self._check(self._polynorm(z.data_ptr(), z.stride(0), _dtype_code(z), coeff.data_ptr(), eps, out.data_ptr(),
                                   _dtype_code(out), z.shape[0], z.shape[1], self._stream()), "polynorm")

    # --- recurrent mixers with a decaying matrix state -------------------------------------------

    @_kind("recurrent.conv")
    def short_conv_residual(self, x, w, state, slots, ctx, out) -> None:
        """``out = x + conv(x)``: a causal convolution over time per channel (``w``: ``[channels, taps]``,
        the last tap weighs the token itself); ``state``: ``[slots, (taps - 1) * channels]``, the
        request's last inputs, moved on by the step's tokens."""
        channels, taps = w.shape
        if x.shape[1] != channels or state.shape[1] < (taps - 1) * channels or x.dtype != out.dtype:
            raise KernelError("short_conv_residual: the sizes do not fit")
        self._check(self._part_lib("recurrent").ie_short_conv_residual(
            x.data_ptr(), _dtype_code(x), w.data_ptr(), state.data_ptr(), state.stride(0), slots.data_ptr(),
            ctx.seq_of_token.data_ptr(), ctx.cu_q.data_ptr(), out.data_ptr(), x.shape[0], ctx.num_seqs, channels,
            taps, state.shape[0], self._err_ptr, self._stream()), "short_conv_residual")
        self.launches += 1 if taps > 1 else 0

    @_kind("recurrent.gates")
    def hgrn2_gates(self, proj, bias, lower, write, size) -> None:
        """In the 32-bit projection ``[N, >= 2 size]``: ``q <- silu(q)``, ``f <- lower + (1 - lower) *
        sigmoid(f + bias)``; ``write = 1 - f``."""
        self._check(self._part_lib("recurrent").ie_hgrn2_gates(
            proj.data_ptr(), proj.stride(0), bias.data_ptr(), lower.data_ptr(), write.data_ptr(), proj.shape[0],
            size, self._stream()), "hgrn2_gates")

    @_kind("recurrent.gates")
    def mlstm_gates(self, gi, gf, bias_i, bias_f, cap, state, m_offset, slots, ctx, gates, heads) -> None:
        """The exponential gates of the matrix memory from their pre-activations (views ``[N, heads]`` of
        one projection), with the running maximum kept at ``state[slot, m_offset + head]``;
        ``gates``: ``[N, heads, 3]`` = (decay, write gate, exp(-maximum))."""
        if gi.stride(0) != gf.stride(0) or gi.stride(1) != 1 or gf.stride(1) != 1:
            raise KernelError("mlstm_gates: the gates' pre-activations must be views of one projection")
        self._check(self._part_lib("recurrent").ie_mlstm_gates(
            gi.data_ptr(), gf.data_ptr(), gi.stride(0), bias_i.data_ptr(), bias_f.data_ptr(), float(cap),
            state.data_ptr(), state.stride(0), m_offset, slots.data_ptr(), ctx.cu_q.data_ptr(), gates.data_ptr(),
            ctx.num_seqs, heads, state.shape[0], self._stream()), "mlstm_gates")

    @_kind("recurrent.rule")
    def gated_recurrence(self, q, a, w, gates, v, state, slots, ctx, out, heads, dim, vdim, cols, q_scale) -> None:
        """``S <- diag(a) S + w u^T; o = S^T q`` per head over every request's tokens of the step, from
        and to its slot (``[heads, cols, dim]``).  ``q``, ``a``, ``w``: views ``[N, heads * dim]``;
        ``v``: view ``[N, heads * vdim]``; with ``gates`` (``[N, heads, 3]``) ``a`` is the gates' decay,
        ``u = gate * v``, and column ``vdim`` (if ``cols = vdim + 1``) carries the value 1."""
        if dim > 512:
            raise KernelError(f"the recurrence kernel takes key sizes up to 512, not {dim}")
        self._check(self._part_lib("recurrent").ie_gated_recurrence(
            q.data_ptr(), q.stride(0), self._ptr(a), 0 if a is None else a.stride(0), w.data_ptr(), w.stride(0),
            self._ptr(gates), v.data_ptr(), v.stride(0), state.data_ptr(), state.stride(0), slots.data_ptr(),
            ctx.cu_q.data_ptr(), out.data_ptr(), ctx.num_seqs, heads, dim, vdim, cols, float(q_scale),
            state.shape[0], self._stream()), "gated_recurrence")

    @_kind("recurrent.out")
    def recurrence_readout(self, o, gates, weight, eps, gate_pre, out, heads, vdim, cols, gate_act="sigmoid") -> None:
        """Per (token, head): with ``gates`` divide by ``max(|o[vdim]|, exp(-m)) + 1e-6``; divide by the
        root mean square over ``vdim``; times ``weight`` (``[vdim]`` or ``[heads * vdim]``) and
        ``sigmoid(gate_pre)`` (``gate_act="silu"``: ``silu(gate_pre)``; a view ``[N, heads * vdim]``) if given."""
        if gate_act not in ("sigmoid", "silu"):
            raise KernelError(f"recurrence_readout: no gate activation {gate_act!r}")
        per_head = 1 if weight.numel() == heads * vdim and heads > 1 else 0
        if weight.numel() not in (vdim, heads * vdim):
            raise KernelError("recurrence_readout: the weight fits neither a head nor all heads")
        self._check(self._part_lib("recurrent").ie_recurrence_readout(
            o.data_ptr(), cols, self._ptr(gates), weight.data_ptr(), per_head, eps, self._ptr(gate_pre),
            0 if gate_pre is None else gate_pre.stride(0), 1 if gate_act == "silu" else 0, out.data_ptr(),
            _dtype_code(out), o.shape[0] * heads, heads, vdim, self._stream()), "recurrence_readout")

    @_kind("recurrent.gates")
    def lowrank_decay(self, y, w2, bias, tau: float, decay) -> None:
        """``decay = sigmoid(y @ w2^T + bias) ** (1 / tau)`` as ``exp(logsigmoid(.) / tau)``, all 32-bit.
        ``y``: a view ``[N, rank]`` of a projection; ``w2``: ``[channels, rank]``; ``decay``: ``[N, channels]``."""
        if y.dtype != self.torch.float32 or w2.dtype != self.torch.float32 or y.stride(1) != 1:
            raise KernelError("lowrank_decay reads a 32-bit projection and a 32-bit matrix")
        self._check(self._part_lib("recurrent").ie_lowrank_decay(
            y.data_ptr(), y.stride(0), w2.data_ptr(), self._ptr(bias), 1.0 / float(tau), decay.data_ptr(),
            y.shape[0], w2.shape[0], w2.shape[1], self._stream()), "lowrank_decay")

    # --- attention with normalised queries and keys and sigmoid weights ---------------------------

    @_kind("rotary+cache")
    def qk_norm_rope_write(self, proj, positions, table, rot_dims, q_weight, k_weight, eps, q_out, k_cache,
                           v_cache, slot_mapping, heads, kv_heads, dim, vdim, page_size, bias=None,
                           value_norm: bool = False, values_from_keys: bool = False,
                           interleaved: bool = False) -> None:
        """The input stage of an attention with per-head norms (see ``csrc/gated_attention.cu``).
        ``q_weight`` / ``k_weight`` None: queries and keys are not normalised; ``bias``: one row laid
        out like the projection's first columns, added first; ``value_norm``: value heads are divided
        by their root mean square.  ``proj`` may hold more columns behind the values.
        ``values_from_keys``: the projection holds queries and keys only, and the cached values are
        the keys as projected (with their bias, before any norm or rotation).  ``interleaved``: the
        rotation pairs entry ``2i`` with ``2i + 1`` instead of ``i`` with ``i + rot_dims / 2``."""
        if table is not None and table.shape[2] * 2 != rot_dims:
            raise KernelError("rotary table does not match the rotated dims")
        if values_from_keys and vdim != dim:
            raise KernelError("values that are the keys have the keys' size")
        need = (heads + kv_heads) * dim + (0 if values_from_keys else kv_heads * vdim)
        if proj.dtype != self.torch.float32 or proj.shape[1] < need or (q_weight is None) != (k_weight is None):
            raise KernelError("qk_norm_rope_write reads the fused 32-bit projection of queries, keys and values")
        if bias is not None and (bias.dtype != self.torch.float32 or bias.numel() < need):
            raise KernelError("qk_norm_rope_write: the bias must be a 32-bit row of the projection's width")
        self._check(self._part_lib("gated_attn").ie_qk_norm_rope_write(
            proj.data_ptr(), proj.stride(0), positions.data_ptr(), self._ptr(table), rot_dims,
            0 if table is None else table.shape[0], self._ptr(bias), 1 if value_norm else 0,
            1 if values_from_keys else 0, 1 if interleaved else 0,
            self._ptr(q_weight), self._ptr(k_weight), eps, q_out.data_ptr(),
            k_cache.data_ptr(), v_cache.data_ptr(), _dtype_code(q_out), self._ptr(slot_mapping), proj.shape[0],
            heads, kv_heads, dim, vdim, page_size, k_cache.shape[0], self._err_ptr, self._stream()),
            "qk_norm_rope_write")

    def _sigmoid_attention_lib(self, hd: int, vdim: int):
        lib = self._sigattn_libs.get((hd, vdim))
        if lib is None:
            path = build_sigmoid_attention(hd, vdim)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as exc:
                raise KernelError(f"the kernel library {path} could not be loaded: {exc}") from exc
            P, I, F = c_void_p, c_int, c_float
            lib.ie_sigmoid_attention_mma.argtypes = [P, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, P, P, P]
            lib.ie_sigmoid_attention_mma.restype = c_int
            self._sigattn_libs[(hd, vdim)] = lib
        return lib

    @_kind("attention.sigmoid")
    def sigmoid_attention(self, q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, vdim, page_size, scale,
                          chunk, head_bias, out) -> None:
        """Attention without a softmax: the weight of a visible key is ``sigmoid(score + head_bias[h])``;
        a query sees the keys at or before it in its own chunk of ``chunk`` positions (0: all).
        bfloat16 with key and value sizes that are multiples of 16 up to 256 runs the tensor-core
        kernel (a block per 64 positions of a request and head; lengths and tables are read on the
        device, and a captured step is launched for the most tokens a request can bring within its
        bounds); 32-bit and other sizes the general kernel.  Neither kernel's order of operations
        depends on the batch."""
        if (self.sigmoid_mma and q.dtype == self.torch.bfloat16 and hd % 16 == 0 and vdim % 16 == 0
                and 16 <= hd <= 256 and 16 <= vdim <= 256 and page_size & (page_size - 1) == 0):
            lib = self._sigmoid_attention_lib(hd, vdim)
            bounds = getattr(ctx, "bounds", None)
            longest = bounds[0] if bounds is not None else ctx.max_q_len  # (a captured step: its token bound)
            self._check(lib.ie_sigmoid_attention_mma(
                q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(),
                block_tables.shape[1], ctx.cu_q.data_ptr(), ctx.ctx_lens.data_ptr(), out.data_ptr(), ctx.num_seqs,
                longest, nh, nkv, page_size, k_cache.shape[0], scale, int(chunk or 0), head_bias.data_ptr(),
                self._err_ptr, self._stream()), "sigmoid_attention_mma")
            return
        self._check(self._paged_attention_generic(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), _dtype_code(q),
            block_tables.data_ptr(), block_tables.shape[1], ctx.seq_of_token.data_ptr(),
            ctx.positions.data_ptr(), out.data_ptr(), ctx.num_tokens, nh, nkv, hd, vdim, vdim, page_size,
            k_cache.shape[0], scale, 0, int(chunk or 0), head_bias.data_ptr(), None, None, 0, 0.0, 0, self._err_ptr,
            self._stream()), "sigmoid_attention")

    def _sink_attention_lib(self, hd: int, vdim: int):
        lib = self._sinkattn_libs.get((hd, vdim))
        if lib is None:
            path = build_sink_attention(hd, vdim)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as exc:
                raise KernelError(f"the kernel library {path} could not be loaded: {exc}") from exc
            P, I, F = c_void_p, c_int, c_float
            lib.ie_sink_attention_mma.argtypes = [P, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, P, P, I, P, I, I, I,
                                                  F, I, I, P, P]
            lib.ie_sink_attention_mma.restype = c_int
            self._sinkattn_libs[(hd, vdim)] = lib
        return lib

    # requests that bring at most so many tokens have their window's keys cut among blocks, each of
    # which serves the query heads of one key/value head (tokens x heads of a group: 64 rows at most)
    SINK_SPLIT_ROWS = 8
    SINK_SPLIT_MOST = 32  # ranges of key tiles per request where no window bounds them

    @_kind("attention.sink")
    def sink_attention(self, q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, vdim, page_size, scale,
                       window, sinks, gate, out, softcap: float | None = None, keep_first: int = 0) -> None:
        """Softmax attention over the paged cache whose denominator also holds ``exp(sinks[head])`` (a
        term without key or value; ``sinks`` None: a plain softmax), over the latest ``window``
        positions (None or 0: all), with value rows of ``vdim`` entries; ``gate`` (a 32-bit view
        ``[N, heads]``, or None): the head's result times ``sigmoid(gate)``.  bfloat16 with key and
        value sizes that are multiples of 16 up to 256 runs the tensor-core kernel (a block per 64
        positions of a request and head, for prompt portions and single tokens; lengths and tables
        are read on the device, and a captured step is launched for the most tokens a request can
        bring within its bounds; when no request brings more than a few tokens, the key tiles of the
        window (or, without one, of the positions the block tables hold) are cut among blocks and merged by a second kernel, so a
        decoded token's sums are the same numbers in another order than in a step that also holds
        a prompt portion); 32-bit and other sizes the general kernel, whose order of operations
        does not depend on the batch.  ``softcap``: a score ``s`` becomes ``softcap * tanh(s / softcap)``
        before the softmax.  ``keep_first`` (with a window): the keys at positions below it stay visible
        to every later query beside its window, at their own positions."""
        if gate is not None and (gate.dtype != self.torch.float32 or gate.stride(1) != 1):
            raise KernelError("sink_attention: the output gate must be a 32-bit view with unit stride")
        cap = float(softcap or 0.0)
        keep = int(keep_first or 0) if window else 0
        if cap < 0 or keep < 0:
            raise KernelError("sink_attention: the cap of the scores and the kept keys cannot be negative")
        if (self.sink_mma and q.dtype == self.torch.bfloat16 and hd % 16 == 0 and vdim % 16 == 0
                and 16 <= hd <= 256 and 16 <= vdim <= 256 and page_size & (page_size - 1) == 0):
            lib = self._sink_attention_lib(hd, vdim)
            bounds = getattr(ctx, "bounds", None)
            longest = bounds[0] if bounds is not None else ctx.max_q_len  # (a captured step: its token bound)
            scratch, splits, per_split, kept_splits = None, 1, 0, 0
            if longest <= self.SINK_SPLIT_ROWS and longest * (nh // nkv) <= 64:
                # the tiles between the first row's oldest key and the last row's own position, in
                # ranges of two: from the window and the row bound alone, so a captured launch stays valid;
                # the tiles of the kept first keys are ranges of their own in front of them.  Without a
                # window: the tiles of as many positions as the step's block tables hold, in at most
                # SINK_SPLIT_MOST ranges (a block whose range lies behind its request's end leaves at once).
                kept_tiles = -(-keep // 64)
                if window:
                    tiles = (int(window) + longest - 2) // 64 + 2
                    per_split = max(2, -(-(tiles + kept_tiles) // 1022))  # (the merge kernel takes up to 1,024 ranges)
                else:
                    tiles = -(-block_tables.shape[1] * page_size // 64)
                    per_split = max(2, -(-tiles // self.SINK_SPLIT_MOST))
                kept_splits = -(-kept_tiles // per_split)
                splits = -(-tiles // per_split) + kept_splits
                if splits > 1:
                    scratch = self._scratch(ctx, "attn.sink_partial", ctx.num_tokens * nh * splits * (vdim + 2), q.device)
            self._check(lib.ie_sink_attention_mma(
                q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(),
                block_tables.shape[1], ctx.cu_q.data_ptr(), ctx.ctx_lens.data_ptr(), out.data_ptr(), ctx.num_seqs,
                longest, nh, nkv, page_size, k_cache.shape[0], scale, int(window or 0), self._ptr(sinks),
                self._ptr(gate), 0 if gate is None else gate.stride(0), self._ptr(scratch), splits, per_split,
                ctx.num_tokens, cap, keep, kept_splits if scratch is not None else 0, self._err_ptr, self._stream()),
                "sink_attention_mma")
            if scratch is not None:  # (the call launched the merge kernel too)
                self.launches += 1
                self.launch_counts["sink_attention_merge"] = self.launch_counts.get("sink_attention_merge", 0) + 1
            return
        self._check(self._paged_attention_generic(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), _dtype_code(q),
            block_tables.data_ptr(), block_tables.shape[1], ctx.seq_of_token.data_ptr(),
            ctx.positions.data_ptr(), out.data_ptr(), ctx.num_tokens, nh, nkv, hd, vdim, vdim, page_size,
            k_cache.shape[0], scale, int(window or 0), 0, None, self._ptr(sinks), self._ptr(gate),
            0 if gate is None else gate.stride(0), cap, keep, self._err_ptr, self._stream()), "sink_attention")

    @_kind("activation")
    def silu_mul(self, gate_up, out, interleave: int = 0) -> None:
        """``out[n, i] = silu(gate_i) * up_i`` from rows that hold the gates and then the ups
        (``interleave`` 0) or gates and ups alternating in blocks of ``interleave`` values."""
        parts, stride = self._partials(gate_up)
        self._check(self._silu_mul(gate_up.data_ptr(), _dtype_code(gate_up), parts, stride,
                                   out.data_ptr(), _dtype_code(out), out.shape[0], out.shape[1],
                                   interleave, self._stream()), "silu_mul")

    GATE_BLOCK = 16  # rows of gates, then of ups, alternate in blocks of this many in a fused matrix

    def gated_linear(self, x, w_gate_up, interleave: int, *, ws, tag="ffn", out_dtype=None):
        """``silu(x @ gate^T) * (x @ up^T)`` with gate and up stacked in ``w_gate_up`` (halves, or
        alternating in blocks of ``interleave`` rows).  A step of few rows whose matrix is laid
        out in blocks of ``GATE_BLOCK`` runs one kernel that streams the weights and applies the
        activation to the sums it holds; everything else is the product followed by
        :meth:`silu_mul`."""
        torch = self.torch
        m, k = x.shape
        n = w_gate_up.shape[0]
        act = ws.buffer(tag + ".act", m, n // 2, out_dtype or x.dtype)
        tiles = -(-n // 128)
        if (self.gated_gemm and interleave == self.GATE_BLOCK and x.dtype == torch.bfloat16
                and act.dtype == torch.bfloat16 and 0 < m <= self.FEW_ROWS and self.few_row_gemm == "tma"
                and k % 8 == 0 and k <= 2048 and n % 32 == 0 and x.is_contiguous() and w_gate_up.is_contiguous()
                and tiles <= (self.tma_max_tiles if m <= 8 else self.tma_max_tiles_wide)
                and tiles <= self.tma_max_blocks):
            self._gated(x, w_gate_up, act)
            return act
        gate_up = self.linear(x, w_gate_up, ws=ws, tag=tag + ".gate_up", out_dtype=act.dtype, allow_split=True)
        self.silu_mul(gate_up, act, interleave)
        return act

    @_kind("linear:ffn.gate_up")
    def _gated(self, x, w, act) -> None:
        self._check(self._gemm_tma_gated_bf16(x.data_ptr(), w.data_ptr(), act.data_ptr(), x.shape[0], w.shape[0],
                                              x.shape[1], self._err_ptr, self._stream()), "gemm_tma_gated")

    def argmax(self, logits, out) -> None:
        """Greedy token of every row (lowest index on ties)."""
        rows = logits.shape[0]
        chunks = max(1, min(2 * self.sm_count // max(rows, 1), 64))
        need = 2 * rows * chunks
        if self._argmax_scratch is None or self._argmax_scratch.numel() < need:
            self._argmax_scratch = self.torch.empty(max(need, 4096), dtype=self.torch.int32, device=self.device)
        self._check(self._argmax(logits.data_ptr(), rows, logits.shape[1], chunks,
                                 self._argmax_scratch.data_ptr(), out.data_ptr(), self._stream()), "argmax")
        self.launches += 1

    @_kind("sampling")
    def sample(self, logits, out, temperature=None, top_k=None, top_p=None, min_p=None,
               penalty=None, seen_bits=None, seeds=None, draws=None, logprob=None) -> None:
        """One token per row of 32-bit ``logits``; the per-row tensors are optional (absent:
        greedy, no cut-off, no penalty).  ``seeds`` and ``draws`` (int64) are needed as soon
        as ``temperature`` is given."""
        if temperature is None and penalty is None and logprob is None:
            return self.argmax(logits, out)
        self._check(self._sample(
            logits.data_ptr(), logits.shape[0], logits.shape[1], self._ptr(temperature),
            self._ptr(top_k), self._ptr(top_p), self._ptr(min_p), self._ptr(penalty),
            self._ptr(seen_bits), 0 if seen_bits is None else seen_bits.shape[1],
            self._ptr(seeds), self._ptr(draws), out.data_ptr(), self._ptr(logprob),
            self._stream()), "sample")


_OPS: dict[str, CudaOps] = {}


def get_ops(device="cuda") -> CudaOps:
    """The process-wide kernel set for ``device``; built and loaded on first use."""
    key = str(device)
    if key not in _OPS:
        _OPS[key] = CudaOps(device)
    return _OPS[key]
