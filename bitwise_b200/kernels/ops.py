"""The kernel library as the parts see it: one object per precision, bound with ctypes.

``KernelOps("float32")`` loads the exact 32-bit kernels, ``KernelOps("bfloat16")`` the
serving kernels; both offer the same operations on torch tensors.  There is no CPU
implementation behind these names: if the CUDA library cannot be compiled or loaded the
constructor raises, and every call checks that its tensors live on a CUDA device.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build

_c_int = ctypes.c_int
_c_float = ctypes.c_float
_ptr = ctypes.c_void_p


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


class KernelError(RuntimeError):
    pass


class DeviceFailure(KernelError):
    """A kernel gave up a bounded wait: what the device computed since the last check is worthless."""


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _need(t: torch.Tensor, dtype, what: str, dims: Optional[int] = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what}: tensor is on {t.device}; the kernels run on a CUDA device only")
    if t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{what}: tensor is not contiguous")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{what}: expected {dims} dimensions, got {tuple(t.shape)}")


def _need_rows(t: torch.Tensor, dtype, what: str) -> None:
    """A matrix whose rows are contiguous; the rows may lie apart (columns sliced out of wider rows)."""
    if not t.is_cuda:
        raise KernelError(f"{what}: tensor is on {t.device}; the kernels run on a CUDA device only")
    if t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, got {t.dtype}")
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1) or t.stride(0) < t.shape[1]:
        raise KernelError(f"{what}: expected rows of contiguous entries, got shape {tuple(t.shape)} strides {t.stride()}")


class KernelOps:
    """Operations of one precision.  ``act_dtype`` is the dtype of activations between
    kernels (the residual stream, logits and norm weights are float32 in both)."""

    FUSED_ACTIVATIONS = ("silu", "gelu_tanh")  # what the gate/up product can apply in its epilogue, by index

    def __init__(self, dtype: str, verbose_build: bool = True):
        if dtype not in ("float32", "bfloat16"):
            raise KernelError(f"unknown dtype {dtype!r} (float32 or bfloat16)")
        self.dtype = dtype
        self.act_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
        self.kind = "f32" if dtype == "float32" else "bf16"
        # The step function hands contexts to the kernels rounded up to this many keys.  The
        # serving kernels derive grids and record strides from that bound, and a step replayed
        # as a CUDA graph keeps what its capture derived: with the bound in steps of 256 a graph
        # serves 256 positions, and a replay launches exactly what an eager step would.
        self.key_granule = 1 if dtype == "float32" else 256
        path = build.ensure_built(self.kind, (), verbose_build)
        try:
            self.lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the CUDA kernel library {path}: {e}") from None
        self.library_path = path
        self.lib.bw_last_error.restype = ctypes.c_char_p
        self.launches = 0  # kernels launched through this object (counted per call)
        self._attn_libs = {}
        self._verbose_build = verbose_build
        self._partials: Optional[torch.Tensor] = None  # scratch of the split products (bfloat16 path)
        self._counters: Optional[torch.Tensor] = None
        self._retired = []
        self._attn_scratch: Optional[torch.Tensor] = None
        self._fns = {}
        self._dev_index: Optional[int] = None
        self._scratch_sizes = {}
        self._kernel_counts = {}
        self._tc_tile_rows = {}
        self.legacy_attention = False  # tests set this to compare the attention kernels bit for bit
        if self.kind == "bf16":
            self.lib.bw_bf16_linear_scratch_floats.restype = ctypes.c_longlong
            self._split_rows = int(self.lib.bw_bf16_linear_split_rows())
        # One word of device memory that every kernel of this object's libraries raises when a
        # bounded wait runs out, and its pinned mirror on the host (filled by failure_poll).
        self._failure_word: Optional[torch.Tensor] = None
        self._failure_host: Optional[torch.Tensor] = None
        if torch.cuda.is_available():
            self._failure_words()  # before any kernel runs: captured graphs keep the word's address

    # -- plumbing ----------------------------------------------------------------------
    def _stream(self):
        # the raw handle of torch's current stream; the private getter skips the Stream object
        # that torch.cuda.current_stream() builds, which costs more than a kernel launch
        if _raw_stream is not None:
            return ctypes.c_void_p(_raw_stream(self._device_index()))
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def _device_index(self) -> int:
        if self._dev_index is None:
            self._dev_index = torch.cuda.current_device()
        return self._dev_index

    def _check(self, rc: int, name: str) -> None:
        if rc != 0:
            msg = self.lib.bw_last_error().decode("utf-8", "replace")
            raise KernelError(f"{name} failed ({rc}): {msg}")

    def _call(self, name: str, *args, lib=None, launches: int = 1) -> None:
        fn = self._fns.get(name) if lib is None else None
        if fn is None:
            fn = getattr(lib or self.lib, name)
            fn.restype = _c_int
            if lib is None:
                self._fns[name] = fn
        self._check(fn(*args), name)
        self.launches += launches

    # -- shared kernels ----------------------------------------------------------------
    def embed_rows(self, table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
        """out[r] = table[tokens[r]] widened to float32, times ``scale``."""
        n, width = out.shape
        _need(tokens, torch.int32, "embed_rows tokens")
        _need(out, torch.float32, "embed_rows out", 2)
        if table.dtype not in (torch.float32, torch.bfloat16) or table.shape[1] != width:
            raise KernelError("embed_rows: table must be float32 or bfloat16 of the output's width")
        _need(table, table.dtype, "embed_rows table", 2)
        self._call("bw_embed_rows", _p(table), _c_int(int(table.dtype == torch.bfloat16)), _p(tokens), _p(out),
                   _c_int(n), _c_int(width), _c_float(scale), self._stream())

    def patch_tokens(self, tokens: torch.Tensor, rows: torch.Tensor, src: torch.Tensor, values: torch.Tensor,
                     count: int) -> None:
        """tokens[rows[i]] = values[src[i]] for i < count: tokens that the step before sampled go
        into this step's token list on the device, unread by the host."""
        for t_, what in ((tokens, "tokens"), (rows, "rows"), (src, "src"), (values, "values")):
            _need(t_, torch.int32, "patch_tokens " + what)
        self._call("bw_patch_tokens", _p(tokens), _p(rows), _p(src), _p(values), _c_int(count), self._stream())

    def sample_rows(self, logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
                    out_tokens: torch.Tensor) -> None:
        rows, vocab = logits.shape
        _need(logits, torch.float32, "sample_rows logits", 2)
        _need(temperature, torch.float32, "sample_rows temperature")
        _need(uniform, torch.float64, "sample_rows uniform")
        _need(out_tokens, torch.int32, "sample_rows out")
        self._call("bw_sample_rows", _p(logits), _c_int(rows), _c_int(vocab), _p(temperature), _p(uniform),
                   _p(out_tokens), self._stream())

    def fingerprint_rows(self, logits: torch.Tensor, slot: torch.Tensor, state: torch.Tensor) -> None:
        """state[slot[r]] = chained hash of logits row r's raw bits (one row per slot per call)."""
        rows, vocab = logits.shape
        _need(logits, torch.float32, "fingerprint_rows logits", 2)
        _need(slot, torch.int32, "fingerprint_rows slot")
        _need(state, torch.int64, "fingerprint_rows state")
        self._call("bw_fingerprint_rows", _p(logits), _c_int(rows), _c_int(vocab), _p(slot), _p(state),
                   self._stream())

    # -- per-precision kernels ---------------------------------------------------------
    def rmsnorm(self, x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        """out[r] = rmsnorm(x[rows[r]] or x[r]) * weight; x and weight float32, out act_dtype."""
        n, width = out.shape
        _need(x, torch.float32, "rmsnorm x", 2)
        _need(weight, torch.float32, "rmsnorm weight", 1)
        _need(out, self.act_dtype, "rmsnorm out", 2)
        if x.shape[1] != width or weight.shape[0] != width:
            raise KernelError("rmsnorm: widths differ")
        if rows is not None:
            _need(rows, torch.int32, "rmsnorm rows")
        self._call(f"bw_{self.kind}_rmsnorm", _p(x), _p(weight), _p(out), _p(rows), _c_int(n), _c_int(width),
                   _c_float(eps), self._stream())

    def linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
               residual: Optional[torch.Tensor] = None, legacy: bool = False) -> None:
        """out = x @ w.T (+ residual).  x [M,K] and w [N,K] in act_dtype; out act_dtype or
        float32; with a float32 residual the sum is formed in 32-bit (out float32, may alias)."""
        m, k = x.shape
        n = w.shape[0]
        _need(x, self.act_dtype, "linear x", 2)
        _need(w, self.act_dtype, "linear w", 2)
        if w.shape[1] != k or tuple(out.shape) != (m, n):
            raise KernelError(f"linear: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
        if residual is not None:
            _need(residual, torch.float32, "linear residual", 2)
            _need(out, torch.float32, "linear out", 2)
            if tuple(residual.shape) != (m, n):
                raise KernelError("linear: residual shape differs from the output's")
        if self.kind == "f32":
            _need(out, torch.float32, "linear out", 2)
            self._call("bw_f32_linear", _p(x), _p(w), _p(out), _p(residual), _c_int(m), _c_int(n), _c_int(k),
                       self._stream())
        else:
            if out.dtype not in (torch.float32, torch.bfloat16):
                raise KernelError("linear: out must be float32 or bfloat16")
            _need(out, out.dtype, "linear out", 2)
            partials = counters = None
            if m <= self._split_rows:
                partials, counters = self._linear_scratch(x.device, n, k)
            self._call("bw_bf16_linear", _p(x), _p(w), _p(out), _c_int(int(out.dtype == torch.float32)),
                       _p(residual), _c_int(m), _c_int(n), _c_int(k), _p(partials), _p(counters),
                       _c_int(int(legacy)), self._stream(),
                       launches=1 if legacy else self._linear_kernels(m, n, k, False, partials is not None))

    def fuses_swiglu(self, width: int, intermediate: int, activation: str = "silu") -> bool:
        """Whether ``linear_swiglu`` can take a feed-forward of these sizes and this activation (then its
        gate/up weights are to be interleaved with ``interleave_gate_up``)."""
        return self.kind == "bf16" and intermediate % 64 == 0 and width % 8 == 0 and activation in self.FUSED_ACTIVATIONS

    @staticmethod
    def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        """Rows in blocks of 64: gate rows 64 b .. 64 b + 63, then the up rows of the same
        indices, so that a 128-row tile of the product holds both halves of 64 outputs."""
        inter, k = gate.shape
        g = gate.reshape(inter // 64, 64, k)
        u = up.reshape(inter // 64, 64, k)
        return torch.stack([g, u], dim=1).reshape(2 * inter, k).contiguous()

    def linear_swiglu(self, x: torch.Tensor, w_interleaved: torch.Tensor, out: torch.Tensor,
                      activation: str = "silu") -> None:
        """out[m][i] = act(x @ gate_i) * (x @ up_i) for interleaved gate/up weights, act SiLU or the tanh form
        of GELU; gate and up are rounded to act_dtype before they are combined, as if they had been stored."""
        if activation not in self.FUSED_ACTIVATIONS:
            raise KernelError(f"linear_swiglu: activation {activation!r}")
        m, k = x.shape
        n = w_interleaved.shape[0]
        _need(x, self.act_dtype, "linear_swiglu x", 2)
        _need(w_interleaved, self.act_dtype, "linear_swiglu w", 2)
        _need(out, self.act_dtype, "linear_swiglu out", 2)
        if self.kind != "bf16" or n % 128 or k % 8 or tuple(out.shape) != (m, n // 2) or w_interleaved.shape[1] != k:
            raise KernelError("linear_swiglu: unsupported shapes or precision")
        partials = None
        if m <= self._split_rows:
            partials, _ = self._linear_scratch(x.device, n, k)
        self._call("bw_bf16_linear_tc_swiglu", _p(x), _p(w_interleaved), _p(out), _c_int(m), _c_int(n), _c_int(k),
                   _p(partials), _c_int(self.FUSED_ACTIVATIONS.index(activation)), self._stream(),
                   launches=self._linear_kernels(m, n, k, True, partials is not None))

    def _linear_kernels(self, m: int, n: int, k: int, swiglu: bool, scratch: bool) -> int:
        """Kernels that a product of this shape launches (2 when it is split along k)."""
        key = (m, n, k, swiglu, scratch)
        c = self._kernel_counts.get(key)
        if c is None:
            c = int(self.lib.bw_bf16_linear_tc_kernels(_c_int(m), _c_int(n), _c_int(k), _c_int(int(swiglu)),
                                                       _c_int(int(scratch))))
            self._kernel_counts[key] = c
        return c

    def _linear_scratch(self, device, n: int, k: int):
        """Scratch of a product that is split along k: chunk sums for up to ``_split_rows``
        rows, and one counter per output tile (zero between launches).  It grows when a
        larger product appears and is otherwise reused by every product of the stream."""
        # sized for the largest batch that may be split, so that the address stays the same
        sizes = self._scratch_sizes.get((n, k))
        if sizes is None:
            sizes = (max(int(self.lib.bw_bf16_linear_scratch_floats(_c_int(r), _c_int(n), _c_int(k)))
                         for r in (64, self._split_rows)), int(self.lib.bw_bf16_linear_counters(_c_int(n))))
            self._scratch_sizes[(n, k)] = sizes
        floats, tiles = sizes
        if floats and (self._partials is None or self._partials.numel() < floats):
            self._retired.append(self._partials)  # a captured graph may still point at the old one
            self._partials = torch.empty(floats, dtype=torch.float32, device=device)
        if self._counters is None or self._counters.numel() < tiles:
            self._retired.append(self._counters)
            self._counters = torch.zeros(max(tiles, 1024), dtype=torch.int32, device=device)
        return self._partials, self._counters

    def force_linear_plan(self, width: int = 0, mode: int = 0) -> None:
        """Tests and measurements: force the tile width of small batches (16 .. 128 in steps of
        16, or 256; 0: chosen from the shape) and the mode (0 chosen, 1 one block walks k,
        2 split along k where possible).  Every combination gives the same bits."""
        if self.kind == "bf16":
            self._kernel_counts.clear()
            self.lib.bw_bf16_linear_tc_force(_c_int(width), _c_int(mode))

    def force_rows_plan(self, tile_cols: int = 0, stages: int = 0) -> None:
        """Tests and measurements of the 32-bit path: force the width of the streaming tile that
        products of up to 16 rows take (16, 32, 64 or 128 columns) and the stages of its ring
        (0: chosen from the shape).  Every combination gives the same bits."""
        if self.kind == "f32":
            self.lib.bw_f32_force_rows_plan(_c_int(tile_cols), _c_int(stages))

    def pair_tiles(self, on: bool) -> bool:
        """Large batches run two thread blocks per 256 x 256 tile of a product (the default) or
        one per 128 x 256 tile; same bits either way.  Returns the previous setting."""
        if self.kind != "bf16":
            return False
        return bool(self.lib.bw_bf16_linear_tc_pair_tiles(_c_int(int(on))))

    def rows_path(self, on: bool) -> bool:
        """Steps of up to 16 rows run their products on the streaming kernel (one kernel per
        product, chunk sums added inside it; the default) or on the tcgen05 kernel like larger
        steps; same bits either way.  Returns the previous setting."""
        if self.kind != "bf16":
            return False
        self._kernel_counts.clear()
        return bool(self.lib.bw_bf16_linear_rows_enable(_c_int(int(on))))

    def stream_attention(self, head_dim: int, mode: int) -> int:
        """How decode steps with head size 64 fetch the cache where TMA boxes fit (pages of 8 keys
        or more that divide 64): 0 never (a thread block per key tile that copies with cp.async),
        1 (the default) the streaming kernel (persistent blocks, TMA rings) for steps of 32 rows
        or more and a block per key tile fed by TMA boxes for fewer, 2 the streaming kernel
        whenever the shape allows.  Same bits every way.  Returns the previous setting."""
        if self.kind != "bf16":
            return 0
        return int(self._attention_lib(head_dim).bw_bf16_attention_stream_mode(_c_int(int(mode))))

    def _failure_words(self):
        if self._failure_word is None:
            dev = torch.device("cuda", self._device_index())
            self._failure_word = torch.zeros(1, dtype=torch.int32, device=dev)
            self._failure_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
            for lib in [self.lib] + list(self._attn_libs.values()) + [l for l in [getattr(self, "_parts", None), getattr(self, "_mixers", None), getattr(self, "_streamlib", None)] if l]:
                lib.bw_set_failure_word(_p(self._failure_word))
        return self._failure_word, self._failure_host

    def failure_poll(self) -> None:
        """Enqueue a copy of the failure word to the host on the current stream (four bytes,
        asynchronous).  ``failure_seen`` reads the copy once the stream has been waited for:
        callers that wait for the device anyway (for a step's tokens) learn of a failure
        without a wait of their own."""
        word, host = self._failure_words()
        host.copy_(word, non_blocking=True)

    def failure_seen(self) -> bool:
        """True (once) when the last ``failure_poll`` whose copy has arrived saw the word raised."""
        if self._failure_host is None or int(self._failure_host[0]) == 0:
            return False
        self._failure_host[0] = 0
        self._failure_word.zero_()
        return True

    def device_failure(self) -> bool:
        """True (once) when a kernel gave up a bounded wait since the last call.  This waits
        for the device and reads a word from it; steps use failure_poll / failure_seen."""
        word, _ = self._failure_words()
        bad = bool(int(word.item()))
        if bad:
            word.zero_()
        return bad

    def selftest_bounded_wait(self, polls: int = 4096) -> int:
        """Launch the check kernel of the bounded waits: one warp waits with the kernels' own
        helper for a barrier on which nothing arrives, gives up after ``polls`` polls and
        raises the failure word.  Returns 2 when the wait gave up (as it must), 1 when it
        reported success."""
        self._failure_words()
        out = torch.zeros(1, dtype=torch.int32, device=self._failure_word.device)
        self._call("bw_selftest_bounded_wait", ctypes.c_uint(polls), _p(out), self._stream())
        return int(out.item())

    def attention_tile_rows(self, heads: int, kv_heads: int) -> int:
        """Query rows per attention tile: the bfloat16 kernel stacks the heads of a group
        with the rows, 64 stacked rows per thread block."""
        if self.kind == "f32":
            return 16
        return max(1, 64 // max(1, heads // kv_heads))

    def attention_tile_heights(self, heads: int, kv_heads: int, head_dim: int):
        """The heights of query tiles (rows of one sequence per thread block) that this
        precision's attention kernels want prepared for a step."""
        if self.kind == "f32":
            return [16]
        group = max(1, heads // kv_heads)
        rows = [max(1, 64 // group)]
        if 128 % group == 0:
            rows.append(128 // group)  # the tcgen05 prefill kernel stacks 128 rows per block
        return rows

    def _attention_scratch(self, lib, device, n: int, heads: int, max_keys: int) -> torch.Tensor:
        """Scratch of the split attention: one (output, maximum, sum) record per row, head and
        tile of 64 keys.  Sized for contexts rounded up to 2048 keys so that it seldom grows."""
        lib.bw_bf16_attention_scratch_floats.restype = ctypes.c_longlong
        keys = (max_keys + 2047) // 2048 * 2048
        floats = int(lib.bw_bf16_attention_scratch_floats(_c_int(n), _c_int(heads), _c_int(keys)))
        if self._attn_scratch is None or self._attn_scratch.numel() < floats:
            self._retired.append(self._attn_scratch)  # a captured graph may still point at the old one
            self._attn_scratch = torch.empty(floats, dtype=torch.float32, device=device)
        return self._attn_scratch

    def _attention_lib(self, head_dim: int):
        lib = self._attn_libs.get(head_dim)
        if lib is None:
            path = build.ensure_built("bf16_attn", (f"BW_HEAD_DIM={head_dim}",), self._verbose_build)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load the attention library {path}: {e}") from None
            lib.bw_last_error.restype = ctypes.c_char_p
            if self._failure_word is not None:
                lib.bw_set_failure_word(_p(self._failure_word))
            self._attn_libs[head_dim] = lib
        return lib

    def rope_cache(self, qkv: torch.Tensor, pos: torch.Tensor, row_seq: torch.Tensor,
                   cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], block_table: torch.Tensor,
                   kcache: torch.Tensor, vcache: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                   write_kv: bool = True) -> None:
        """Rotate q (in place) and k by the table rows of ``pos``; store k and v in the pages
        ``block_table[row_seq[r]][pos[r] // page]``.  kcache / vcache: [pages, kv_heads, page, hd]."""
        n = qkv.shape[0]
        _need(qkv, self.act_dtype, "rope_cache qkv", 2)
        _need(pos, torch.int32, "rope_cache pos")
        _need(row_seq, torch.int32, "rope_cache row_seq")
        _need(block_table, torch.int32, "rope_cache block_table", 2)
        _need(kcache, self.act_dtype, "rope_cache kcache", 4)
        _need(vcache, self.act_dtype, "rope_cache vcache", 4)
        if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
            raise KernelError("rope_cache: row width is not (heads + 2 kv_heads) * head_dim")
        if tuple(kcache.shape[1:]) != (kv_heads, kcache.shape[2], head_dim) or kcache.shape != vcache.shape:
            raise KernelError("rope_cache: cache shape is not [pages, kv_heads, page, head_dim]")
        if cos is not None:
            _need(cos, torch.float32, "rope_cache cos", 2)
            _need(sin, torch.float32, "rope_cache sin", 2)
            if cos.shape[1] != head_dim // 2 or cos.shape != sin.shape:
                raise KernelError("rope_cache: table width is not head_dim / 2")
        self._call(f"bw_{self.kind}_rope_cache", _p(qkv), _c_int(qkv.shape[1]), _p(pos), _p(row_seq), _p(cos),
                   _p(sin), _p(block_table), _c_int(block_table.shape[1]), _p(kcache), _p(vcache), _c_int(n),
                   _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(kcache.shape[2]),
                   _c_int(int(write_kv)), self._stream())

    def fuses_rope(self, m: int, width: int, heads: int, kv_heads: int, head_dim: int) -> bool:
        """Whether ``linear_rope_cache`` takes a step of m rows: then the fused q/k/v product
        rotates q and k and stores k and v in the cache itself (steps of up to 16 rows on the
        serving precision)."""
        if self.kind != "bf16":
            return False
        key = ("rope", m, width, heads, kv_heads, head_dim)
        c = self._kernel_counts.get(key)
        if c is None:
            c = int(self.lib.bw_bf16_linear_rows_rope_usable(None, None, _c_int(m), _c_int((heads + 2 * kv_heads) * head_dim),
                                                             _c_int(width), _c_int(heads), _c_int(kv_heads),
                                                             _c_int(head_dim)))
            self._kernel_counts[key] = c
        return bool(c)

    def linear_rope_cache(self, x: torch.Tensor, w_qkv: torch.Tensor, qkv: torch.Tensor, pos: torch.Tensor,
                          row_seq: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                          block_table: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, heads: int,
                          kv_heads: int, head_dim: int, write_kv: bool = True) -> None:
        """``linear(x, w_qkv, qkv)`` followed by ``rope_cache(qkv, ...)`` in one kernel: the
        rotated q lands in qkv's first heads * head_dim columns, the rotated k and v in their
        pages; the k and v columns of qkv are NOT written.  Same bits as the two calls.  Only
        where ``fuses_rope`` says so."""
        m, k = x.shape
        n = w_qkv.shape[0]
        _need(x, self.act_dtype, "linear_rope_cache x", 2)
        _need(w_qkv, self.act_dtype, "linear_rope_cache w", 2)
        _need(qkv, self.act_dtype, "linear_rope_cache qkv", 2)
        _need(pos, torch.int32, "linear_rope_cache pos")
        _need(row_seq, torch.int32, "linear_rope_cache row_seq")
        _need(block_table, torch.int32, "linear_rope_cache block_table", 2)
        _need(kcache, self.act_dtype, "linear_rope_cache kcache", 4)
        _need(vcache, self.act_dtype, "linear_rope_cache vcache", 4)
        if self.kind != "bf16" or w_qkv.shape[1] != k or tuple(qkv.shape) != (m, n) or n != (heads + 2 * kv_heads) * head_dim:
            raise KernelError("linear_rope_cache: shapes do not fit the fused q/k/v projection")
        if tuple(kcache.shape[1:]) != (kv_heads, kcache.shape[2], head_dim) or kcache.shape != vcache.shape:
            raise KernelError("linear_rope_cache: cache shape is not [pages, kv_heads, page, head_dim]")
        if cos is not None:
            _need(cos, torch.float32, "linear_rope_cache cos", 2)
            _need(sin, torch.float32, "linear_rope_cache sin", 2)
            if cos.shape[1] != head_dim // 2 or cos.shape != sin.shape:
                raise KernelError("linear_rope_cache: table width is not head_dim / 2")
        self._call("bw_bf16_linear_rows_rope", _p(x), _p(w_qkv), _p(qkv), _c_int(m), _c_int(n), _c_int(k), _p(pos),
                   _p(row_seq), _p(cos), _p(sin), _p(block_table), _c_int(block_table.shape[1]), _p(kcache), _p(vcache),
                   _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(kcache.shape[2]), _c_int(int(write_kv)),
                   self._stream())

    def attention(self, qkv: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                  block_table: torch.Tensor, row_seq: torch.Tensor, pos: torch.Tensor, out: torch.Tensor,
                  heads: int, kv_heads: int, head_dim: int, window: int, max_keys: int, scale: float,
                  batch=None) -> None:
        """out[r, h] = softmax(q k^T * scale) v over the cached keys lo..pos[r] of row r's
        sequence (lo = max(0, pos - window + 1) when window > 0).  q is read from the first
        heads*head_dim columns of qkv.  ``batch`` carries the step's per-sequence arrays for
        kernels that tile queries by sequence."""
        n = qkv.shape[0]
        _need(qkv, self.act_dtype, "attention qkv", 2)
        _need(out, self.act_dtype, "attention out", 2)
        _need(kcache, self.act_dtype, "attention kcache", 4)
        _need(vcache, self.act_dtype, "attention vcache", 4)
        _need(block_table, torch.int32, "attention block_table", 2)
        _need(row_seq, torch.int32, "attention row_seq")
        _need(pos, torch.int32, "attention pos")
        if out.shape[1] != heads * head_dim or out.shape[0] != n:
            raise KernelError("attention: output shape is not [rows, heads * head_dim]")
        page = kcache.shape[2]
        if self.kind == "f32":
            # prompt portions run as tiles of 16 query rows that share their keys; a step of single
            # rows (a decode step, or a call without the step's arrays) spreads a row's scores over
            # many blocks and needs scratch for them
            tiles = batch.query_tiles(16) if batch is not None and 16 in getattr(batch, "tile_sets", {}) else None
            scratch, floats, launches = None, 0, 1
            if tiles is None or tiles[3] >= n:
                tiles = None
                self.lib.bw_f32_attention_scratch_floats.restype = ctypes.c_longlong
                floats = int(self.lib.bw_f32_attention_scratch_floats(_c_int(n), _c_int(heads), _c_int(max_keys)))
                if self._attn_scratch is None or self._attn_scratch.numel() < floats:
                    self._attn_scratch = torch.empty(floats, dtype=torch.float32, device=qkv.device)
                scratch, launches = self._attn_scratch, 2
            t_seq, t_row0, t_rows, t_count = tiles if tiles is not None else (None, None, None, 0)
            self._call("bw_f32_attention", _p(qkv), _c_int(qkv.shape[1]), _p(kcache), _p(vcache), _p(block_table),
                       _c_int(block_table.shape[1]), _p(row_seq), _p(pos), _p(t_seq), _p(t_row0), _p(t_rows),
                       _c_int(t_count), _p(batch.seq_pos0) if tiles is not None else None,
                       _p(batch.seq_row0) if tiles is not None else None, _p(out), _c_int(out.shape[1]), _c_int(n),
                       _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page), _c_int(window),
                       _c_int(max_keys), _c_float(scale), _p(scratch), ctypes.c_longlong(floats), self._stream(),
                       launches=launches)
        else:
            if batch is None:
                raise KernelError("attention (bfloat16): the step's sequence arrays are required")
            if head_dim % 16 or not (16 <= head_dim <= 256):
                raise KernelError(f"attention (bfloat16): head size {head_dim} is not a multiple of 16 up to 256")
            lib = self._attention_lib(head_dim)
            t_seq, t_row0, t_rows, t_count = batch.query_tiles(self.attention_tile_rows(heads, kv_heads))
            scratch = None
            split = t_count == n and max_keys > 128  # a decode step: one tile of keys per warp
            if not split and not self.legacy_attention:
                # prefill portions: the tcgen05 kernel, where it takes the shape (same bits)
                shape_key = (heads, kv_heads, head_dim, page, qkv.shape[1])
                rows_tc = self._tc_tile_rows.get(shape_key)
                if rows_tc is None:
                    rows_tc = int(lib.bw_bf16_attention_tc_tile_rows(_c_int(heads), _c_int(kv_heads),
                                                                     _c_int(head_dim), _c_int(page),
                                                                     _c_int(qkv.shape[1])))
                    self._tc_tile_rows[shape_key] = rows_tc
                sets = getattr(batch, "tile_sets", None)
                if rows_tc > 0 and (sets is None or rows_tc in sets) and n > t_count:
                    q_seq, q_row0, q_rows, q_count = batch.query_tiles(rows_tc)
                    fn = lib.bw_bf16_attention_tc
                    fn.restype = _c_int
                    rc = fn(_p(qkv), _c_int(qkv.shape[1]), _p(kcache), _p(vcache), _c_int(kcache.shape[0]),
                            _p(block_table), _c_int(block_table.shape[1]), _p(q_seq), _p(q_row0), _p(q_rows),
                            _c_int(q_count), _p(batch.seq_pos0), _p(batch.seq_row0), _p(out), _c_int(out.shape[1]),
                            _c_int(n), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page), _c_int(window),
                            _c_float(scale), self._stream())
                    if rc != 0:
                        raise KernelError(f"bw_bf16_attention_tc failed ({rc}): "
                                          + lib.bw_last_error().decode("utf-8", "replace"))
                    self.launches += 1
                    return
            if split:
                scratch = self._attention_scratch(lib, qkv.device, n, heads, max_keys)
                # head size 64: the cache streams through TMA rings, one block per SM (same bits)
                if lib.bw_bf16_attention_stream_usable(_c_int(n), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page),
                                                       _c_int(qkv.shape[1])):
                    fn = lib.bw_bf16_attention_stream
                    fn.restype = _c_int
                    rc = fn(_p(qkv), _c_int(qkv.shape[1]), _p(kcache), _p(vcache), _c_int(kcache.shape[0]),
                            _p(block_table), _c_int(block_table.shape[1]), _p(row_seq), _p(pos), _p(out),
                            _c_int(out.shape[1]), _c_int(n), _c_int(heads), _c_int(kv_heads), _c_int(head_dim),
                            _c_int(page), _c_int(window), _c_float(scale), _c_int(max_keys), _p(scratch), self._stream())
                    if rc != 0:
                        raise KernelError(f"bw_bf16_attention_stream failed ({rc}): "
                                          + lib.bw_last_error().decode("utf-8", "replace"))
                    self.launches += 2
                    return
            fn = lib.bw_bf16_attention
            fn.restype = _c_int
            rc = fn(_p(qkv), _c_int(qkv.shape[1]), _p(kcache), _p(vcache), _p(block_table),
                    _c_int(block_table.shape[1]), _p(t_seq), _p(t_row0), _p(t_rows), _c_int(t_count),
                    _p(batch.seq_pos0), _p(batch.seq_row0), _p(row_seq), _p(pos), _p(out), _c_int(out.shape[1]), _c_int(n),
                    _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page), _c_int(window), _c_float(scale),
                    _c_int(max_keys), _p(scratch), self._stream())
            if rc != 0:
                raise KernelError(f"bw_bf16_attention failed ({rc}): "
                                  + lib.bw_last_error().decode("utf-8", "replace"))
            self.launches += 2 if split else 1

    def swiglu(self, gate_up: torch.Tensor, out: torch.Tensor) -> None:
        """out = silu(gate) * up for rows laid out [gate | up]."""
        n, inter = out.shape
        _need(gate_up, self.act_dtype, "swiglu gate_up", 2)
        _need(out, self.act_dtype, "swiglu out", 2)
        if gate_up.shape[1] != 2 * inter or gate_up.shape[0] != n:
            raise KernelError("swiglu: input is not [rows, 2 * intermediate]")
        self._call(f"bw_{self.kind}_swiglu", _p(gate_up), _p(out), _c_int(n), _c_int(inter), self._stream())

    # -- parts that only some architectures have (their library is loaded at first use) ------
    def _parts_lib(self):
        lib = getattr(self, "_parts", None)
        if lib is None:
            path = build.ensure_built(f"{self.kind}_parts", (), self._verbose_build)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load the kernel library {path}: {e}") from None
            lib.bw_last_error.restype = ctypes.c_char_p
            if self._failure_word is not None:
                lib.bw_set_failure_word(_p(self._failure_word))
            self._parts = lib
            self._parts_fns = {}
        return lib

    def _pcall(self, name: str, *args, launches: int = 1) -> None:
        lib = self._parts_lib()
        fn = self._parts_fns.get(name)
        if fn is None:
            fn = getattr(lib, f"bw_{self.kind}_{name}")
            fn.restype = _c_int
            self._parts_fns[name] = fn
        rc = fn(*args)
        if rc != 0:
            raise KernelError(f"{name} failed ({rc}): " + lib.bw_last_error().decode("utf-8", "replace"))
        self.launches += launches

    def layernorm(self, x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                  rows: Optional[torch.Tensor] = None, weight2: Optional[torch.Tensor] = None,
                  out2: Optional[torch.Tensor] = None) -> None:
        """out[r] = (x[s] - mean) / sqrt(var + eps) * weight with s = rows[r] or r; x float32, out
        float32 (it may be x itself) or act_dtype.  With ``weight2`` and ``out2`` a second output
        of the same row statistics."""
        n, width = out.shape
        _need(x, torch.float32, "layernorm x", 2)
        _need(weight, torch.float32, "layernorm weight", 1)
        if out.dtype not in (torch.float32, self.act_dtype):
            raise KernelError(f"layernorm: out is {out.dtype}")
        _need(out, out.dtype, "layernorm out", 2)
        if x.shape[1] != width or weight.shape[0] != width:
            raise KernelError("layernorm: widths differ")
        if (weight2 is None) != (out2 is None):
            raise KernelError("layernorm: a second weight needs a second output")
        if out2 is not None:
            _need(weight2, torch.float32, "layernorm weight2", 1)
            _need(out2, out.dtype, "layernorm out2", 2)
            if tuple(out2.shape) != (n, width) or weight2.shape[0] != width:
                raise KernelError("layernorm: the second output's shape differs")
        if rows is not None:
            _need(rows, torch.int32, "layernorm rows")
        self._pcall("layernorm", _p(x), _p(weight), _p(weight2), _p(out), _p(out2),
                    _c_int(int(out.dtype == torch.float32)), _p(rows), _c_int(n), _c_int(width), _c_float(eps),
                    self._stream())

    def layernorm_residual(self, d: torch.Tensor, weight: torch.Tensor, eps: float, x: torch.Tensor,
                           next_weight: Optional[torch.Tensor] = None, next_eps: float = 0.0,
                           next_out: Optional[torch.Tensor] = None) -> None:
        """x[r] += (d[r] - mean) / sqrt(var + eps) * weight with the row statistics of d; d, weight and x
        float32.  With ``next_weight`` and ``next_out`` (act_dtype) also the layer norm of the summed row, with
        that weight and ``next_eps``: the norm before the next sublayer, in the same kernel."""
        n, width = x.shape
        _need(d, torch.float32, "layernorm_residual d", 2)
        _need(x, torch.float32, "layernorm_residual x", 2)
        _need(weight, torch.float32, "layernorm_residual weight", 1)
        if tuple(d.shape) != (n, width) or weight.shape[0] != width:
            raise KernelError("layernorm_residual: shapes differ")
        if (next_weight is None) != (next_out is None):
            raise KernelError("layernorm_residual: the next norm needs a weight and an output")
        if next_out is not None:
            _need(next_weight, torch.float32, "layernorm_residual next_weight", 1)
            _need(next_out, self.act_dtype, "layernorm_residual next_out", 2)
            if tuple(next_out.shape) != (n, width) or next_weight.shape[0] != width:
                raise KernelError("layernorm_residual: the next norm's shapes differ")
        self._pcall("layernorm_residual", _p(d), _p(weight), _p(x), _c_int(n), _c_int(width), _c_float(eps),
                    _p(next_weight), _c_float(next_eps), _p(next_out), self._stream())

    def add_rows(self, x: torch.Tensor, d: torch.Tensor) -> None:
        """x += d (float32, same shape)."""
        _need(x, torch.float32, "add_rows x")
        _need(d, torch.float32, "add_rows d")
        if x.shape != d.shape:
            raise KernelError("add_rows: shapes differ")
        self._pcall("add_rows", _p(x), _p(d), ctypes.c_longlong(x.numel()), self._stream())

    def latent_store(self, d: torch.Tensor, weight: torch.Tensor, eps: float, pos: torch.Tensor, row_seq: torch.Tensor,
                     cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], block_table: torch.Tensor,
                     cache: torch.Tensor, rank: int, rot_dim: int, half_layout: bool = False, q_latent=None) -> None:
        """For every row of ``d`` (float32 [n, >= rank + rot_dim], the row's first columns are used): the
        first ``rank`` entries divided by their root mean square (eps inside the root) times ``weight``, the
        next ``rot_dim`` turned pair by pair (2i with 2i+1; ``half_layout``: i with i + pairs) by row ``pos``
        of the tables, both stored at the row's place in ``cache`` [pages, page, rank + rot_dim].  With
        ``q_latent`` = (weight [q_rank], out act_dtype [n, q_rank]) the ``q_rank`` columns that follow in the
        same rows are normed as well, with that weight, into ``out``: the queries' latent, in the same kernel."""
        n = d.shape[0]
        _need_rows(d, torch.float32, "latent_store d")
        _need(weight, torch.float32, "latent_store weight", 1)
        _need(pos, torch.int32, "latent_store pos")
        _need(row_seq, torch.int32, "latent_store row_seq")
        _need(block_table, torch.int32, "latent_store block_table", 2)
        _need(cache, self.act_dtype, "latent_store cache", 3)
        if d.shape[1] < rank + rot_dim or cache.shape[2] != rank + rot_dim or weight.shape[0] != rank:
            raise KernelError("latent_store: widths do not fit rank + rot_dim")
        pairs = self._check_tables(cos, sin, rot_dim, "latent_store")
        q_w = q_out = None
        q_rank = 0
        if q_latent is not None:
            q_w, q_out = q_latent
            q_rank = q_w.shape[0]
            _need(q_w, torch.float32, "latent_store q weight", 1)
            _need(q_out, self.act_dtype, "latent_store q out", 2)
            if d.shape[1] < rank + rot_dim + q_rank or tuple(q_out.shape) != (n, q_rank):
                raise KernelError("latent_store: the queries' latent does not fit the rows")
        self._pcall("latent_store", _p(d), _c_int(d.stride(0)), _p(weight), _c_float(eps), _p(pos), _p(row_seq), _p(cos),
                    _p(sin), _c_int(pairs), _p(block_table), _c_int(block_table.shape[1]), _p(cache), _c_int(n),
                    _c_int(rank), _c_int(rot_dim), _c_int(cache.shape[1]), _c_int(int(bool(half_layout))), _p(q_w),
                    _c_int(q_rank), _p(q_out), self._stream())

    @staticmethod
    def _check_tables(cos, sin, rot_dim: int, what: str) -> int:
        if cos is None:
            return 0
        _need(cos, torch.float32, what + " cos", 2)
        _need(sin, torch.float32, what + " sin", 2)
        if cos.shape != sin.shape or 2 * cos.shape[1] > rot_dim:
            raise KernelError(f"{what}: the tables turn {2 * cos.shape[1]} entries of {rot_dim}")
        return int(cos.shape[1])

    def rotate_heads(self, q: torch.Tensor, heads: int, head_stride: int, offset: int, rot_dim: int, out: torch.Tensor,
                     out_head_stride: int, out_offset: int, pos: torch.Tensor, cos: Optional[torch.Tensor],
                     sin: Optional[torch.Tensor], half_layout: bool = False) -> None:
        """out[r, h * out_head_stride + out_offset + i] = the entries q[r, h * head_stride + offset + i],
        i < rot_dim, turned pair by pair (2i with 2i+1; ``half_layout``: i with i + pairs) by row pos[r] of
        the tables."""
        n = q.shape[0]
        _need(q, self.act_dtype, "rotate_heads q", 2)
        _need(out, self.act_dtype, "rotate_heads out", 2)
        _need(pos, torch.int32, "rotate_heads pos")
        if (heads - 1) * head_stride + offset + rot_dim > q.shape[1] or \
                (heads - 1) * out_head_stride + out_offset + rot_dim > out.shape[1] or out.shape[0] != n:
            raise KernelError("rotate_heads: the heads do not fit the rows")
        pairs = self._check_tables(cos, sin, rot_dim, "rotate_heads")
        self._pcall("rotate_heads", _p(q), _c_int(q.shape[1]), _c_int(head_stride), _c_int(offset), _p(out),
                    _c_int(out.shape[1]), _c_int(out_head_stride), _c_int(out_offset), _c_int(n), _c_int(heads),
                    _c_int(rot_dim), _c_int(pairs), _p(pos), _p(cos), _p(sin), _c_int(int(bool(half_layout))), self._stream())

    def latent_attention_tile_rows(self, heads: int) -> int:
        """Rows of one sequence per query tile that ``latent_attention`` wants prepared."""
        fn = getattr(self._parts_lib(), f"bw_{self.kind}_latent_attention_tile_rows")
        return int(fn(_c_int(heads)))

    def latent_attention_tile_heights(self, heads: int, rank: int, rot_dim: int):
        """The heights of query tiles that ``latent_attention`` may ask the step for: the plain
        kernel's, and on the serving precision the tensor-core kernel's where it takes the shape."""
        out = [self.latent_attention_tile_rows(heads)]
        tc = self._latent_tc_rows(heads, rank, rot_dim)
        if tc and tc not in out:
            out.append(tc)
        return out

    def _latent_tc_rows(self, heads: int, rank: int, rot_dim: int) -> int:
        if self.kind != "bf16":
            return 0
        fn = self._parts_lib().bw_bf16_latent_attention_tc_tile_rows
        return int(fn(_c_int(heads), _c_int(rank), _c_int(rot_dim), _c_int(heads * (rank + rot_dim))))

    def plain_parts(self, on: bool) -> None:
        """Tests: keep latent attention and the grouped products on the plain kernels (one chain of
        fused multiply-adds per output) also where the tensor-core kernels would take the shape."""
        self._plain_parts = bool(on)
        if self.kind == "bf16":
            lib = self._parts_lib()
            lib.bw_bf16_latent_attention_force_plain(_c_int(int(on)))
            lib.bw_bf16_grouped_force_plain(_c_int(int(on)))

    def _latent_scratch(self, floats: int, device) -> torch.Tensor:
        if self._attn_scratch is None or self._attn_scratch.numel() < floats:
            self._retired.append(self._attn_scratch)  # a captured graph may still point at the old one
            self._attn_scratch = torch.empty(floats, dtype=torch.float32, device=device)
        return self._attn_scratch

    def latent_attention(self, q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, out: torch.Tensor,
                         heads: int, rank: int, rot_dim: int, scale: float, batch, window: int = 0,
                         sinks: Optional[torch.Tensor] = None) -> None:
        """out[r, h] = sum_j softmax_j(q[r, h] . cache[j] * scale) cache[j][:rank] over the cached
        positions j <= pos[r] of row r's sequence (from pos - window + 1 on when window > 0).  ``sinks``
        (float32 [heads]): exp(sinks[h]) joins the softmax's denominator, with no key and no value.
        q: [n, heads * (rank + rot_dim)] (the heads' key maps folded in, the rotated part turned),
        cache: [pages, page, rank + rot_dim], out: [n, heads * rank]."""
        n = q.shape[0]
        dk = rank + rot_dim
        _need(q, self.act_dtype, "latent_attention q", 2)
        _need(cache, self.act_dtype, "latent_attention cache", 3)
        _need(out, self.act_dtype, "latent_attention out", 2)
        _need(block_table, torch.int32, "latent_attention block_table", 2)
        if q.shape[1] != heads * dk or cache.shape[2] != dk or tuple(out.shape) != (n, heads * rank):
            raise KernelError("latent_attention: shapes do not fit heads * (rank + rot_dim)")
        if sinks is not None:
            _need(sinks, torch.float32, "latent_attention sinks", 1)
            if sinks.shape[0] != heads:
                raise KernelError("latent_attention: one sink per head is needed")
        page = cache.shape[1]
        tc_rows = self._latent_tc_rows(heads, rank, rot_dim)
        if tc_rows and (not hasattr(batch, "tile_sets") or tc_rows in batch.tile_sets):
            # the serving precision's tensor-core kernel; steps of single rows with long contexts
            # spread every row's keys over several blocks and merge
            t_seq, t_row0, t_rows, t_count = batch.query_tiles(tc_rows)
            scratch, launches = None, 1
            if t_count == n and batch.max_keys > 256:
                span = _c_int(0)
                spans = int(self._parts_lib().bw_bf16_latent_attention_tc_spans(_c_int(t_count), _c_int(heads),
                                                                                _c_int(batch.max_keys), ctypes.byref(span)))
                scratch, launches = self._latent_scratch(n * heads * spans * (rank + 2), q.device), 2
            self._pcall("latent_attention_tc", _p(q), _c_int(q.shape[1]), _p(cache), _p(block_table),
                        _c_int(block_table.shape[1]), _p(t_seq), _p(t_row0), _p(t_rows), _c_int(t_count),
                        _p(batch.seq_pos0), _p(batch.seq_row0), _p(batch.pos), _p(out), _c_int(out.shape[1]), _c_int(n),
                        _c_int(heads), _c_int(rank), _c_int(rot_dim), _c_int(page), _c_int(window), _c_float(scale),
                        _c_int(batch.max_keys), _p(scratch), _p(sinks), self._stream(), launches=launches)
            return
        t_seq, t_row0, t_rows, t_count = batch.query_tiles(self.latent_attention_tile_rows(heads))
        if t_count == n and batch.max_keys > 256:
            # single rows with long contexts: spread every row's keys over many blocks
            lib = self._parts_lib()
            span = _c_int(0)
            spans = int(getattr(lib, f"bw_{self.kind}_latent_attention_spans")(_c_int(n), _c_int(heads),
                                                                               _c_int(batch.max_keys), ctypes.byref(span)))
            self._latent_scratch(n * heads * spans * (rank + 2), q.device)
            self._pcall("latent_attention_split", _p(q), _c_int(q.shape[1]), _p(cache), _p(block_table),
                        _c_int(block_table.shape[1]), _p(batch.row_seq), _p(batch.pos), _p(out), _c_int(out.shape[1]),
                        _c_int(n), _c_int(heads), _c_int(rank), _c_int(rot_dim), _c_int(page), _c_int(window),
                        _c_float(scale), _c_int(batch.max_keys), _p(self._attn_scratch), _p(sinks), self._stream(),
                        launches=2)
            return
        self._pcall("latent_attention", _p(q), _c_int(q.shape[1]), _p(cache), _p(block_table),
                    _c_int(block_table.shape[1]), _p(t_seq), _p(t_row0), _p(t_rows), _c_int(t_count), _p(batch.seq_pos0),
                    _p(batch.seq_row0), _p(out), _c_int(out.shape[1]), _c_int(heads), _c_int(rank), _c_int(rot_dim),
                    _c_int(page), _c_int(window), _c_float(scale), _p(sinks), self._stream())

    def route(self, logits: torch.Tensor, correction: Optional[torch.Tensor], groups: int, keep: int, top: int,
              weight_scale: float, chosen: torch.Tensor, weights: torch.Tensor, softmax_top: bool = False) -> None:
        """Per row of ``logits`` (float32 [n, experts]): scores sigmoid(z); the ``top`` experts with
        the largest score + correction among the experts of the ``keep`` best of ``groups`` equal
        groups of neighbours (a group counts as the sum of its two largest corrected scores);
        chosen int32 [n, top], weights float32 [n, top] = score * weight_scale.  ``softmax_top``: the choice
        is by the logits themselves (plus the correction) and the weights are the softmax over the chosen
        logits only, times weight_scale."""
        n, experts = logits.shape
        _need(logits, torch.float32, "route logits", 2)
        _need(chosen, torch.int32, "route chosen", 2)
        _need(weights, torch.float32, "route weights", 2)
        if correction is not None:
            _need(correction, torch.float32, "route correction", 1)
        if tuple(chosen.shape) != (n, top) or tuple(weights.shape) != (n, top):
            raise KernelError("route: outputs are not [rows, top]")
        self._pcall("route", _p(logits), _p(correction), _c_int(n), _c_int(experts), _c_int(groups), _c_int(keep),
                    _c_int(top), _c_float(weight_scale), _c_int(int(bool(softmax_top))), _p(chosen), _p(weights),
                    self._stream())

    def group_rows(self, chosen: torch.Tensor, experts: int, group_off: torch.Tensor, tile_prefix: torch.Tensor,
                   order: torch.Tensor, place: torch.Tensor) -> None:
        """The (row, choice) pairs of ``chosen`` listed expert by expert: group_off [experts + 1],
        tile_prefix [2, experts + 1] (tiles of the grouped product before each expert, for its
        two tile heights), order [pairs]
        (pair index = row * top + choice), place [pairs] (where a pair stands in ``order``)."""
        pairs = chosen.numel()
        for t_, what in ((chosen, "chosen"), (group_off, "group_off"), (tile_prefix, "tile_prefix"), (order, "order"),
                         (place, "place")):
            _need(t_, torch.int32, "group_rows " + what)
        if group_off.numel() < experts + 1 or tile_prefix.numel() < 2 * (experts + 1) or order.numel() < pairs or \
                place.numel() < pairs:
            raise KernelError("group_rows: an output is too small")
        self._pcall("group_rows", _p(chosen), _c_int(pairs), _c_int(experts), _p(group_off), _p(tile_prefix), _p(order),
                    _p(place), self._stream())

    def gather_rows(self, x: torch.Tensor, order: torch.Tensor, order_div: int, out: torch.Tensor, rows: int) -> None:
        """out[i] = x[order[i] // order_div] for i < rows."""
        _need(x, self.act_dtype, "gather_rows x", 2)
        _need(out, self.act_dtype, "gather_rows out", 2)
        _need(order, torch.int32, "gather_rows order")
        if out.shape[1] != x.shape[1] or out.shape[0] < rows or order.numel() < rows:
            raise KernelError("gather_rows: shapes differ")
        self._pcall("gather_rows", _p(x), _p(order), _c_int(order_div), _p(out), _c_int(rows), _c_int(x.shape[1]),
                    self._stream())

    def grouped_takes_tiles(self, rows: int, groups: int, n: int, k: int) -> bool:
        """Whether a grouped product over lists of this size runs on the tcgen05 kernel, which
        fetches tiles of consecutive rows (the caller then offers ``sorted_x`` to ``grouped_linear``):
        the serving precision, lists of on average a tile of 128 rows or more, n a multiple of 64."""
        return (self.kind == "bf16" and not getattr(self, "_plain_parts", False) and rows >= 128 * groups
                and n % 64 == 0 and k % 8 == 0)

    def grouped_linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: int, x_group_cols: int = 0,
                       o_group_cols: int = 0, lists=None, order_div: int = 1, gather: bool = True,
                       sorted_x: Optional[torch.Tensor] = None) -> None:
        """One product per group with w [groups, n, k].  Without ``lists`` every group g takes rows
        0 .. rows-1: out[r, g * o_group_cols + j] = sum_i x[r, g * x_group_cols + i] w[g, j, i].  With
        ``lists`` = (group_off, tile_prefix, order) from ``group_rows`` entry i of group g reads row
        order[i] // order_div of x (row i when ``gather`` is False) and writes row i of out; ``rows``
        is then the length of the list.  ``sorted_x``: scratch [rows, k] for the gathered rows, used
        where ``grouped_takes_tiles`` says so."""
        groups, n, k = w.shape
        _need(x, self.act_dtype, "grouped_linear x", 2)
        _need(w, self.act_dtype, "grouped_linear w", 3)
        if out.dtype not in (torch.float32, self.act_dtype):
            raise KernelError(f"grouped_linear: out is {out.dtype}")
        _need(out, out.dtype, "grouped_linear out", 2)
        if lists is None:
            if (groups - 1) * x_group_cols + k > x.shape[1] or (groups - 1) * o_group_cols + n > out.shape[1] or \
                    rows > x.shape[0] or rows > out.shape[0]:
                raise KernelError("grouped_linear: the groups' columns do not fit the rows")
            group_off = tile_prefix = order = None
        else:
            group_off, tile_prefix, order = lists
            if x.shape[1] != k or out.shape[1] != n or rows > out.shape[0]:
                raise KernelError("grouped_linear: widths differ from the weights'")
            if not gather:
                order = None
            if self.grouped_takes_tiles(rows, groups, n, k) and (order is None or sorted_x is not None):
                # long lists: the tcgen05 product over rows made contiguous group by group
                src = x
                if order is not None:
                    self.gather_rows(x, order, order_div, sorted_x, rows)
                    src = sorted_x
                if self.lib.bw_bf16_linear_tc_grouped_usable(_p(src), _p(w), _p(out), _c_int(n), _c_int(k)):
                    self._call("bw_bf16_linear_tc_grouped", _p(src), _p(w), _p(out), _c_int(int(out.dtype == torch.float32)),
                               _c_int(rows), _c_int(n), _c_int(k), _p(group_off), _p(tile_prefix[1]), _c_int(groups),
                               self._stream())
                    return
                x, order, order_div = src, None, 1
        self._pcall("grouped_linear", _p(x), _c_int(x.shape[1]), _c_int(x_group_cols), _p(order), _c_int(order_div),
                    _p(w), _p(out), _c_int(int(out.dtype == torch.float32)), _c_int(out.shape[1]), _c_int(o_group_cols),
                    _p(group_off), _p(tile_prefix), _c_int(rows), _c_int(groups), _c_int(n), _c_int(k), self._stream())

    def glu_clamped(self, gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> None:
        """out = g' * sigmoid(alpha * g') * (u' + 1) for rows laid out [gate | up], with
        g' = min(g, limit) and u' = clamp(u, -limit, limit)."""
        n, inter = out.shape
        _need(gate_up, self.act_dtype, "glu_clamped gate_up", 2)
        _need(out, self.act_dtype, "glu_clamped out", 2)
        if gate_up.shape[1] != 2 * inter or gate_up.shape[0] != n:
            raise KernelError("glu_clamped: input is not [rows, 2 * inner]")
        self._pcall("glu_clamped", _p(gate_up), _p(out), _c_int(n), _c_int(inter), _c_float(limit), _c_float(alpha),
                    self._stream())

    def combine(self, x: torch.Tensor, d: Optional[torch.Tensor], y: torch.Tensor, place: torch.Tensor,
                weights: torch.Tensor, top: int, scale: Optional[torch.Tensor] = None) -> None:
        """x[r] += d[r] + sum_j weights[r, j] * y[place[r * top + j]] (float32; d may be None); with ``scale``
        [width] what is added is multiplied by it column by column first."""
        n, width = x.shape
        _need(x, torch.float32, "combine x", 2)
        _need(y, torch.float32, "combine y", 2)
        _need(place, torch.int32, "combine place")
        _need(weights, torch.float32, "combine weights", 2)
        if d is not None:
            _need(d, torch.float32, "combine d", 2)
        if y.shape[1] != width or tuple(weights.shape) != (n, top) or (d is not None and d.shape != x.shape):
            raise KernelError("combine: shapes differ")
        if scale is not None:
            _need(scale, torch.float32, "combine scale", 1)
            if scale.shape[0] != width:
                raise KernelError("combine: one factor per column is needed")
        self._pcall("combine", _p(x), _p(d), _p(y), _p(place), _p(weights), _c_int(n), _c_int(top), _c_int(width),
                    _p(scale), self._stream())

    # -- element-wise steps of gated designs (their library is loaded at first use) ---------------------
    def _gated_lib(self):
        lib = getattr(self, "_gated", None)
        if lib is None:
            path = build.ensure_built(f"{self.kind}_gated", (), self._verbose_build)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load the kernel library {path}: {e}") from None
            lib.bw_last_error.restype = ctypes.c_char_p
            if self._failure_word is not None:
                lib.bw_set_failure_word(_p(self._failure_word))
            self._gated = lib
            self._gated_fns = {}
        return lib

    def _gcall(self, name: str, *args) -> None:
        lib = self._gated_lib()
        fn = self._gated_fns.get(name)
        if fn is None:
            fn = getattr(lib, f"bw_{self.kind}_{name}")
            fn.restype = _c_int
            self._gated_fns[name] = fn
        rc = fn(*args)
        if rc != 0:
            raise KernelError(f"{name} failed ({rc}): " + lib.bw_last_error().decode("utf-8", "replace"))
        self.launches += 1

    def sigmoid_gate(self, v: torch.Tensor, g: torch.Tensor, group: int = 1) -> None:
        """v[r, c] *= sigmoid(g[r, c // group]) in place; v: act_dtype [n, cols], g: float32 [n, cols / group]
        (its rows may be a slice of wider rows)."""
        n, cols = v.shape
        _need(v, self.act_dtype, "sigmoid_gate v", 2)
        _need_rows(g, torch.float32, "sigmoid_gate g")
        if group <= 0 or cols % group or tuple(g.shape) != (n, cols // group):
            raise KernelError(f"sigmoid_gate: {tuple(g.shape)} gate numbers do not fit {cols} columns in groups of {group}")
        self._gcall("sigmoid_gate", _p(v), _c_int(n), _c_int(cols), _p(g), _c_int(g.stride(0)), _c_int(group), self._stream())

    def glu_gelu(self, gate_up: torch.Tensor, out: torch.Tensor) -> None:
        """out = gelu_tanh(gate) * up for rows laid out [gate | up], gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2 / pi)
        (z + 0.044715 z^3)))."""
        n, inter = out.shape
        _need(gate_up, self.act_dtype, "glu_gelu gate_up", 2)
        _need(out, self.act_dtype, "glu_gelu out", 2)
        if gate_up.shape[1] != 2 * inter or gate_up.shape[0] != n:
            raise KernelError("glu_gelu: input is not [rows, 2 * inner]")
        self._gcall("glu_gelu", _p(gate_up), _p(out), _c_int(n), _c_int(inter), self._stream())

    def softcap_rows(self, z: torch.Tensor, cap: float) -> None:
        """z <- cap * tanh(z / cap) in place on float32 rows."""
        _need(z, torch.float32, "softcap_rows z")
        self._gcall("softcap_rows", _p(z), ctypes.c_longlong(z.numel()), _c_float(cap), self._stream())

    # -- mixers with state beside or instead of pages, and the norm after a sublayer (their library
    #    is loaded at first use) -------------------------------------------------------------------
    def _mixers_lib(self):
        lib = getattr(self, "_mixers", None)
        if lib is None:
            path = build.ensure_built(f"{self.kind}_mixers", (), self._verbose_build)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load the kernel library {path}: {e}") from None
            lib.bw_last_error.restype = ctypes.c_char_p
            if self._failure_word is not None:
                lib.bw_set_failure_word(_p(self._failure_word))
            self._mixers = lib
            self._mixers_fns = {}
        return lib

    def _mcall(self, name: str, *args, launches: int = 1) -> None:
        lib = self._mixers_lib()
        fn = self._mixers_fns.get(name)
        if fn is None:
            fn = getattr(lib, f"bw_{self.kind}_{name}")
            fn.restype = _c_int
            self._mixers_fns[name] = fn
        rc = fn(*args)
        if rc != 0:
            raise KernelError(f"{name} failed ({rc}): " + lib.bw_last_error().decode("utf-8", "replace"))
        self.launches += launches

    def rmsnorm_residual(self, d: torch.Tensor, weight: torch.Tensor, eps: float, x: torch.Tensor,
                         next_weight: Optional[torch.Tensor] = None, next_eps: float = 0.0,
                         next_out: Optional[torch.Tensor] = None) -> None:
        """x[r] += d[r] / sqrt(mean(d[r]^2) + eps) * weight; d, weight and x float32.  With ``next_weight``
        and ``next_out`` (act_dtype) also next_out[r] = x[r] / sqrt(mean(x[r]^2) + next_eps) * next_weight of
        the summed row: the norm before the next sublayer, in the same kernel."""
        n, width = x.shape
        _need(d, torch.float32, "rmsnorm_residual d", 2)
        _need(x, torch.float32, "rmsnorm_residual x", 2)
        _need(weight, torch.float32, "rmsnorm_residual weight", 1)
        if tuple(d.shape) != (n, width) or weight.shape[0] != width:
            raise KernelError("rmsnorm_residual: shapes differ")
        if (next_weight is None) != (next_out is None):
            raise KernelError("rmsnorm_residual: the next norm needs a weight and an output")
        if next_out is not None:
            _need(next_weight, torch.float32, "rmsnorm_residual next_weight", 1)
            _need(next_out, self.act_dtype, "rmsnorm_residual next_out", 2)
            if tuple(next_out.shape) != (n, width) or next_weight.shape[0] != width:
                raise KernelError("rmsnorm_residual: the next norm's shapes differ")
        self._mcall("rmsnorm_residual", _p(d), _p(weight), _p(x), _c_int(n), _c_int(width), _c_float(eps), _p(next_weight),
                    _c_float(next_eps), _p(next_out), self._stream())

    def scored_attention_tile_heights(self, group: int, dim: int, vdim: int):
        """The heights of query tiles (rows of one sequence per thread block) that ``scored_attention``
        wants prepared for ``group`` query heads on a key/value head."""
        fn = getattr(self._mixers_lib(), f"bw_{self.kind}_scored_attention_tile_rows")
        out = [int(fn(_c_int(group)))]
        tc = self._scored_mma_rows(group, dim, vdim)
        if tc and tc not in out:
            out.append(tc)
        return out

    def _scored_mma_rows(self, group: int, dim: int, vdim: int) -> int:
        """Rows per query tile of the tensor-core attention, 0 where it does not take the shape."""
        if self.kind != "bf16":
            return 0
        return int(self._mixers_lib().bw_bf16_scored_attention_mma_tile_rows(_c_int(group), _c_int(dim), _c_int(vdim)))

    def plain_mixers(self, on: bool) -> None:
        """Tests: keep scored attention on the CUDA-core kernel (one chain of fused multiply-adds per
        score and output) also where the tensor-core kernel would take the shape."""
        if self.kind == "bf16":
            self._mixers_lib().bw_bf16_scored_attention_force_plain(_c_int(int(on)))

    def qkv_prepare(self, u: torch.Tensor, conv_w: Optional[torch.Tensor], conv_state: Optional[torch.Tensor],
                    q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], eps: float,
                    cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], batch, block_table: torch.Tensor,
                    kcache: torch.Tensor, vcache: Optional[torch.Tensor], q_out: torch.Tensor, heads: int,
                    write_kv_heads: int, dim: int, vdim: int, conv_wt: Optional[torch.Tensor] = None,
                    bias: Optional[torch.Tensor] = None, vmix_src: Optional[torch.Tensor] = None,
                    vmix_lambda: Optional[torch.Tensor] = None, v_keep: Optional[torch.Tensor] = None) -> None:
        """From the projected rows ``u`` (float32 [n, cols]: ``heads`` query heads of ``dim``, then, when
        ``write_kv_heads`` > 0, that many key heads of ``dim`` and, with ``vcache``, value heads of
        ``vdim``): the convolution over time with ``conv_w`` [cols, taps] (inputs before the step's
        first row of a sequence from ``conv_state`` [slots, taps - 1, cols], zeros before position 0),
        the norm per head of q and k with ``q_norm`` / ``k_norm`` [dim], the rotation of the first 2 *
        pairs entries of q and k by the tables' row of the position; q into ``q_out`` [n, heads * dim],
        keys and values into their pages.  Each step may be absent (None).  ``conv_wt``: the taps
        transposed ([taps, cols]); with them, and sizes that are multiples of 4, the kernel reads four
        channels at a time.  ``bias`` [cols] is added to every projected row first.  ``vmix_src`` (float32 [n,
        kv_heads * vdim]) and ``vmix_lambda`` (one float32): the values become (1 - lambda) v + lambda vmix_src
        before they are stored; ``v_keep`` (same shape) receives the values as stored, in float32."""
        n, cols = u.shape
        _need_rows(u, torch.float32, "qkv_prepare u")
        _need(q_out, self.act_dtype, "qkv_prepare q_out", 2)
        _need(block_table, torch.int32, "qkv_prepare block_table", 2)
        _need(kcache, self.act_dtype, "qkv_prepare kcache", 4)
        taps = 0
        if conv_w is not None:
            _need(conv_w, torch.float32, "qkv_prepare conv_w", 2)
            taps = conv_w.shape[1]
            if conv_w.shape[0] != cols:
                raise KernelError("qkv_prepare: one row of taps per channel is needed")
        if conv_state is not None:
            _need(conv_state, torch.float32, "qkv_prepare conv_state", 3)
            if tuple(conv_state.shape[1:]) != (taps - 1, cols):
                raise KernelError("qkv_prepare: the state is not [slots, taps - 1, cols]")
        for w_, what in ((q_norm, "q_norm"), (k_norm, "k_norm")):
            if w_ is not None:
                _need(w_, torch.float32, "qkv_prepare " + what, 1)
                if w_.shape[0] != dim:
                    raise KernelError("qkv_prepare: a norm weight is not of the head's size")
        pairs = self._check_tables(cos, sin, dim, "qkv_prepare")
        want = heads * dim + write_kv_heads * dim + (write_kv_heads * vdim if vcache is not None else 0)
        if cols != want or tuple(q_out.shape) != (n, heads * dim):
            raise KernelError(f"qkv_prepare: rows of {cols} columns do not hold {want}")
        if write_kv_heads and (tuple(kcache.shape[1:]) != (write_kv_heads, kcache.shape[2], dim)):
            raise KernelError("qkv_prepare: key cache is not [pages, kv_heads, page, dim]")
        if vcache is not None:
            _need(vcache, self.act_dtype, "qkv_prepare vcache", 4)
            if write_kv_heads and tuple(vcache.shape[1:]) != (write_kv_heads, kcache.shape[2], vdim):
                raise KernelError("qkv_prepare: value cache is not [pages, kv_heads, page, vdim]")
        if bias is not None:
            _need(bias, torch.float32, "qkv_prepare bias", 1)
            if bias.shape[0] != cols:
                raise KernelError("qkv_prepare: one bias per projected column is needed")
        for t_, what in ((vmix_src, "vmix_src"), (v_keep, "v_keep")):
            if t_ is not None:
                _need(t_, torch.float32, "qkv_prepare " + what, 2)
                if vcache is None or not write_kv_heads or tuple(t_.shape) != (n, write_kv_heads * vdim):
                    raise KernelError(f"qkv_prepare: {what} is not [rows, kv_heads * vdim] of values that are stored")
        if (vmix_src is None) != (vmix_lambda is None):
            raise KernelError("qkv_prepare: mixing values needs both the other values and the factor")
        if vmix_lambda is not None:
            _need(vmix_lambda, torch.float32, "qkv_prepare vmix_lambda", 1)
        if conv_wt is not None:
            _need(conv_wt, torch.float32, "qkv_prepare conv_wt", 2)
            if conv_w is None or tuple(conv_wt.shape) != (taps, cols):
                raise KernelError("qkv_prepare: the transposed taps are not [taps, cols]")
        self._mcall("qkv_prepare", _p(u), _c_int(cols), _p(conv_w), _p(conv_wt), _c_int(taps), _p(conv_state), _p(q_norm), _p(k_norm),
                    _c_float(eps), _p(cos), _p(sin), _c_int(pairs), _p(batch.pos), _p(batch.row_seq), _p(batch.seq_row0),
                    _p(batch.seq_pos0), _p(batch.seq_slot), _p(block_table), _c_int(block_table.shape[1]), _p(kcache),
                    _p(vcache if write_kv_heads else None), _p(q_out), _c_int(n), _c_int(heads), _c_int(write_kv_heads),
                    _c_int(dim), _c_int(vdim), _c_int(kcache.shape[2]), _p(bias), _p(vmix_src), _p(vmix_lambda), _p(v_keep),
                    _c_int(u.stride(0)), self._stream())

    def conv_state_update(self, u: torch.Tensor, state: torch.Tensor, batch, taps: int, seq_tiles) -> None:
        """state[slot of s][i] = the projected row of position end_s - (taps - 1) + i for every sequence s
        of the step (``seq_tiles``: one tile per sequence), end_s its length after the step: from the
        step's rows ``u``, from the old state, or zero before position 0."""
        _need_rows(u, torch.float32, "conv_state_update u")
        _need(state, torch.float32, "conv_state_update state", 3)
        t_seq, t_row0, t_rows, t_count = seq_tiles
        if tuple(state.shape[1:]) != (taps - 1, u.shape[1]):
            raise KernelError("conv_state_update: the state is not [slots, taps - 1, cols]")
        self._mcall("conv_state_update", _p(u), _c_int(u.shape[1]), _p(state), _c_int(taps), _p(t_seq), _p(t_row0),
                    _p(t_rows), _c_int(t_count), _p(batch.seq_pos0), _p(batch.seq_slot), _c_int(u.stride(0)), self._stream())

    def scored_attention(self, q: torch.Tensor, kcache: torch.Tensor, vcache: Optional[torch.Tensor],
                         block_table: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int,
                         scale: float, softcap: float, sink: bool, slopes: Optional[torch.Tensor], window: int,
                         batch, dist_a: Optional[torch.Tensor] = None, dist_b: Optional[torch.Tensor] = None,
                         sinks: Optional[torch.Tensor] = None, keep_first: int = 0) -> None:
        """out[r, h] = sum_j p_j v_j over the cached positions j <= pos[r] of row r's sequence (from pos -
        window + 1 on when window > 0) with s_j = (q[r, h] . k_j) * scale, then s_j <- softcap * tanh(s_j /
        softcap) when softcap > 0, then s_j <- s_j - slopes[h] * (pos[r] - j) when slopes are given, and
        p_j = exp(s_j) / (sum exp(s) + (1 if sink else 0)).  ``vcache`` None: the values are the keys.
        ``dist_a``, ``dist_b`` [heads]: s_j <- s_j - dist_a[h] * ln(1 + dist_b[h] * (pos[r] - j)) as well.  ``sinks``
        [heads]: with ``sink``, exp(sinks[h]) joins the denominator instead of 1.  ``keep_first``: with a window,
        the keys j < keep_first are seen too."""
        n = q.shape[0]
        _need(q, self.act_dtype, "scored_attention q", 2)
        _need(out, self.act_dtype, "scored_attention out", 2)
        _need(kcache, self.act_dtype, "scored_attention kcache", 4)
        _need(block_table, torch.int32, "scored_attention block_table", 2)
        if vcache is not None:
            _need(vcache, self.act_dtype, "scored_attention vcache", 4)
        elif vdim != dim:
            raise KernelError("scored_attention: values that are the keys have the keys' size")
        if slopes is not None:
            _need(slopes, torch.float32, "scored_attention slopes", 1)
            if slopes.shape[0] != heads:
                raise KernelError("scored_attention: one slope per head is needed")
        if q.shape[1] != heads * dim or tuple(out.shape) != (n, heads * vdim) or kcache.shape[1] != kv_heads or \
                kcache.shape[3] != dim:
            raise KernelError("scored_attention: shapes do not fit the heads")
        if (dist_a is None) != (dist_b is None):
            raise KernelError("scored_attention: the distance term needs both numbers per head")
        for t_, what in ((dist_a, "dist_a"), (dist_b, "dist_b"), (sinks, "sinks")):
            if t_ is not None:
                _need(t_, torch.float32, "scored_attention " + what, 1)
                if t_.shape[0] != heads:
                    raise KernelError(f"scored_attention: {what} is not one number per head")
        tail = (_p(dist_a), _p(dist_b), _p(sinks), _c_int(int(keep_first)))
        tc_rows = self._scored_mma_rows(heads // kv_heads, dim, vdim)
        if tc_rows and (not hasattr(batch, "tile_sets") or tc_rows in batch.tile_sets):
            # The serving precision's tensor-core kernel.  Contexts beyond 256 keys are walked in spans
            # of 256 keys at fixed absolute positions, a block per query tile and span, and a second
            # kernel joins the spans' records: prompt portions and single rows alike, so that a
            # position's bits depend neither on the step's kind nor on what else is in it (a query
            # whose keys lie in the first span gets the same bits with and without the merge).
            t_seq, t_row0, t_rows, t_count = batch.query_tiles(tc_rows)
            spans, scratch, launches = 1, None, 1
            if batch.max_keys > 256:
                spans = int(self._mixers_lib().bw_bf16_scored_attention_spans(_c_int(batch.max_keys)))
                scratch, launches = self._latent_scratch(n * heads * spans * (vdim + 2), q.device), 2
            self._mcall("scored_attention_mma", _p(q), _c_int(q.shape[1]), _p(kcache), _p(vcache), _p(block_table),
                        _c_int(block_table.shape[1]), _p(t_seq), _p(t_row0), _p(t_rows), _c_int(t_count), _p(batch.seq_pos0),
                        _p(batch.seq_row0), _p(out), _c_int(out.shape[1]), _c_int(heads), _c_int(kv_heads), _c_int(dim),
                        _c_int(vdim), _c_int(kcache.shape[2]), _c_float(scale), _c_float(softcap), _c_int(int(bool(sink))),
                        _p(slopes), _c_int(window), _c_int(n), _c_int(spans), _p(scratch), *tail, self._stream(),
                        launches=launches)
            return
        fn = getattr(self._mixers_lib(), f"bw_{self.kind}_scored_attention_tile_rows")
        t_seq, t_row0, t_rows, t_count = batch.query_tiles(int(fn(_c_int(heads // kv_heads))))
        self._mcall("scored_attention", _p(q), _c_int(q.shape[1]), _p(kcache), _p(vcache), _p(block_table),
                    _c_int(block_table.shape[1]), _p(t_seq), _p(t_row0), _p(t_rows), _c_int(t_count), _p(batch.seq_pos0),
                    _p(batch.seq_row0), _p(out), _c_int(out.shape[1]), _c_int(heads), _c_int(kv_heads), _c_int(dim),
                    _c_int(vdim), _c_int(kcache.shape[2]), _c_float(scale), _c_float(softcap), _c_int(int(bool(sink))),
                    _p(slopes), _c_int(window), *tail, self._stream())

    def gla_scan(self, u: torch.Tensor, z: torch.Tensor, bias: torch.Tensor, tau: float, state: torch.Tensor,
                 norm_w: torch.Tensor, eps: float, out: torch.Tensor, heads: int, dim: int, vdim: int, q_scale: float,
                 batch, seq_tiles, scratch: Optional[torch.Tensor] = None) -> None:
        """The recurrence S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T (q_t * q_scale) per head over the
        rows of every sequence of the step (``seq_tiles``: one tile per sequence), from and into ``state``
        [slots, heads, dim, vdim] (zero at a request's first position), with a = sigmoid(z + bias) ** (1 /
        tau); out = o / rms(o) * norm_w * silu(gate).  ``u`` (float32) holds q | k | v | gate per row.
        ``scratch``: float32 [n, heads * vdim] for the outputs before their norm (allocated when absent)."""
        n = u.shape[0]
        _need(u, torch.float32, "gla_scan u", 2)
        _need(z, torch.float32, "gla_scan z", 2)
        _need(bias, torch.float32, "gla_scan bias", 1)
        _need(state, torch.float32, "gla_scan state", 4)
        _need(norm_w, torch.float32, "gla_scan norm_w", 1)
        _need(out, self.act_dtype, "gla_scan out", 2)
        if u.shape[1] != 2 * heads * (dim + vdim) or tuple(z.shape) != (n, heads * dim) or bias.shape[0] != heads * dim or \
                tuple(state.shape[1:]) != (heads, dim, vdim) or norm_w.shape[0] != vdim or tuple(out.shape) != (n, heads * vdim):
            raise KernelError("gla_scan: shapes do not fit the heads")
        t_seq, t_row0, t_rows, t_count = seq_tiles
        if scratch is None:
            scratch = torch.empty(n, heads * vdim, dtype=torch.float32, device=u.device)
        _need(scratch, torch.float32, "gla_scan scratch", 2)
        if tuple(scratch.shape) != (n, heads * vdim):
            raise KernelError("gla_scan: the scratch is not [rows, heads * vdim]")
        self._mcall("gla_scan", _p(u), _c_int(u.shape[1]), _p(z), _p(bias), _c_float(tau), _p(state), _p(norm_w),
                    _c_float(eps), _p(scratch), _p(out), _p(t_seq), _p(t_row0), _p(t_rows), _c_int(t_count),
                    _p(batch.seq_pos0), _p(batch.seq_slot), _c_int(n), _c_int(heads), _c_int(dim), _c_int(vdim),
                    _c_float(q_scale), self._stream(), launches=2)

    # -- kernels on the residual stream that only some blocks use (their library is loaded at first use) -------
    def _stream_lib(self):
        lib = getattr(self, "_streamlib", None)
        if lib is None:
            path = build.ensure_built(f"{self.kind}_stream", (), self._verbose_build)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load the kernel library {path}: {e}") from None
            lib.bw_last_error.restype = ctypes.c_char_p
            if self._failure_word is not None:
                lib.bw_set_failure_word(_p(self._failure_word))
            self._streamlib = lib
            self._stream_fns = {}
        return lib

    def _scall(self, name: str, *args, launches: int = 1) -> None:
        lib = self._stream_lib()
        fn = self._stream_fns.get(name)
        if fn is None:
            fn = getattr(lib, f"bw_{self.kind}_{name}")
            fn.restype = _c_int
            self._stream_fns[name] = fn
        rc = fn(*args)
        if rc != 0:
            raise KernelError(f"{name} failed ({rc}): " + lib.bw_last_error().decode("utf-8", "replace"))
        self.launches += launches

    def embed_pair(self, table: torch.Tensor, pair_table: torch.Tensor, batch, last_token: torch.Tensor, out: torch.Tensor,
                   scale: float, buckets: int, mul_prev: int, mul_cur: int) -> None:
        """out[r] = table[token] * scale + pair_table[row], row = (previous token * mul_prev + token * mul_cur) mod
        buckets, and row ``buckets`` at position 0.  The previous token of a sequence's first row of the step is
        ``last_token[slot]`` (int32 [slots, 1])."""
        n, width = out.shape
        _need(out, torch.float32, "embed_pair out", 2)
        _need(table, self.act_dtype, "embed_pair table", 2)
        _need(pair_table, self.act_dtype, "embed_pair pair_table", 2)
        _need(last_token, torch.int32, "embed_pair last_token")
        if table.shape[1] != width or tuple(pair_table.shape) != (buckets + 1, width):
            raise KernelError("embed_pair: the tables are not [vocab, width] and [buckets + 1, width]")
        self._scall("embed_pair", _p(table), _p(pair_table), _p(batch.tokens), _p(batch.pos), _p(batch.row_seq),
                    _p(batch.seq_row0), _p(batch.seq_slot), _p(last_token), _p(out), _c_int(n), _c_int(width), _c_float(scale),
                    _c_int(buckets), _c_int(mul_prev), _c_int(mul_cur), self._stream())

    def last_token_update(self, batch, last_token: torch.Tensor, seq_tiles) -> None:
        """last_token[slot of s] = the last token of every sequence s of the step (``seq_tiles``: one tile per sequence)."""
        _need(last_token, torch.int32, "last_token_update last_token")
        t_seq, t_row0, t_rows, t_count = seq_tiles
        self._scall("last_token_update", _p(batch.tokens), _p(t_seq), _p(t_row0), _p(t_rows), _c_int(t_count),
                    _p(batch.seq_slot), _p(last_token), self._stream())

    def norm_conv(self, x: torch.Tensor, weight: torch.Tensor, eps: float, taps_t: torch.Tensor, state: Optional[torch.Tensor],
                  state_col0: int, batch, out: torch.Tensor, normed: torch.Tensor, normed_col0: int) -> None:
        """h = rmsnorm(x) * weight; out = h + conv(h) with conv(h)_t = sum_j taps_t[j] * h_(t - taps + 1 + j) per channel
        (``taps_t`` float32 [taps, width]); rows before the step's first of a sequence are read from ``state``
        [slots, taps - 1, state columns] at columns state_col0 .., zeros before position 0.  ``normed`` (float32 [n,
        columns], written at columns normed_col0 ..) receives h of the last taps - 1 rows of every sequence's portion, which
        is what ``conv_state_update`` reads; its other rows are left as they are."""
        n, width = out.shape
        _need(x, torch.float32, "norm_conv x", 2)
        _need(weight, torch.float32, "norm_conv weight", 1)
        _need(taps_t, torch.float32, "norm_conv taps", 2)
        _need(out, self.act_dtype, "norm_conv out", 2)
        _need(normed, torch.float32, "norm_conv normed", 2)
        taps = taps_t.shape[0]
        if tuple(x.shape) != (n, width) or weight.shape[0] != width or taps_t.shape[1] != width or normed.shape[0] != n or \
                normed_col0 + width > normed.shape[1]:
            raise KernelError("norm_conv: shapes differ")
        state_cols = 0
        if state is not None:
            _need(state, torch.float32, "norm_conv state", 3)
            state_cols = state.shape[2]
            if state.shape[1] != taps - 1 or state_col0 + width > state_cols:
                raise KernelError("norm_conv: the state is not [slots, taps - 1, columns]")
        self._scall("norm_conv", _p(x), _p(weight), _c_float(eps), _p(taps_t), _c_int(taps), _p(state), _c_int(state_cols),
                    _c_int(state_col0), _p(batch.pos), _p(batch.row_seq), _p(batch.seq_row0), _p(batch.seq_slot), _p(out),
                    _p(normed), _c_int(normed.shape[1]), _c_int(normed_col0), _c_int(n), _c_int(width), self._stream())

    def scaled_add(self, x: torch.Tensor, scale: Optional[torch.Tensor], d: Optional[torch.Tensor],
                   rounded: Optional[torch.Tensor] = None) -> None:
        """x += scale * d column by column (float32; nothing is added without ``scale``); ``rounded``
        (act_dtype) receives the summed rows as well."""
        n, width = x.shape
        _need(x, torch.float32, "scaled_add x", 2)
        if (scale is None) != (d is None):
            raise KernelError("scaled_add: the factors and the rows come together")
        if scale is not None:
            _need(scale, torch.float32, "scaled_add scale", 1)
            _need(d, torch.float32, "scaled_add d", 2)
            if scale.shape[0] != width or tuple(d.shape) != (n, width):
                raise KernelError("scaled_add: shapes differ")
        if rounded is not None:
            _need(rounded, self.act_dtype, "scaled_add rounded", 2)
            if tuple(rounded.shape) != (n, width):
                raise KernelError("scaled_add: shapes differ")
        self._scall("scaled_add", _p(x), _p(scale), _p(d), _p(rounded), _c_int(n), _c_int(width), self._stream())

    def token_gate(self, t: torch.Tensor, table: torch.Tensor, col0: int, tokens: torch.Tensor, out: torch.Tensor) -> None:
        """out[r] = gelu_tanh(t[r]) * table[tokens[r], col0 : col0 + dim] (t float32 [n, dim], out act_dtype)."""
        n, dim = t.shape
        _need(t, torch.float32, "token_gate t", 2)
        _need(table, self.act_dtype, "token_gate table", 2)
        _need(tokens, torch.int32, "token_gate tokens")
        _need(out, self.act_dtype, "token_gate out", 2)
        if tuple(out.shape) != (n, dim) or col0 < 0 or col0 + dim > table.shape[1]:
            raise KernelError("token_gate: shapes differ")
        self._scall("token_gate", _p(t), _p(table), _c_int(table.shape[1]), _c_int(col0), _p(tokens), _p(out), _c_int(n),
                    _c_int(dim), self._stream())

    def normed_add_mix(self, x: torch.Tensor, y: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float,
                       mult: float, history: Optional[torch.Tensor], index: int, mix: Optional[torch.Tensor]) -> None:
        """x[r] += mult * y[r] / sqrt(mean(y[r]^2) + eps) * weight (skipped without ``y``); then, with ``history``
        (float32 [n, entries * width]): entry ``index`` of the row's history = x[r], and x[r] = sum_j mix[j] *
        history entry j, j = 0 .. index (mix float32 [index + 1])."""
        n, width = x.shape
        _need(x, torch.float32, "normed_add_mix x", 2)
        if y is not None:
            _need(y, torch.float32, "normed_add_mix y", 2)
            _need(weight, torch.float32, "normed_add_mix weight", 1)
            if tuple(y.shape) != (n, width) or weight.shape[0] != width:
                raise KernelError("normed_add_mix: shapes differ")
        entries = 0
        if history is not None:
            _need(history, torch.float32, "normed_add_mix history", 2)
            _need(mix, torch.float32, "normed_add_mix mix", 1)
            entries = history.shape[1] // width
            if history.shape[0] != n or history.shape[1] % width or mix.shape[0] != index + 1 or index >= entries:
                raise KernelError("normed_add_mix: the history does not fit")
        self._scall("normed_add_mix", _p(x), _p(y), _p(weight), _c_float(eps), _c_float(mult), _p(history), _c_int(entries),
                    _c_int(index), _p(mix), _c_int(n), _c_int(width), self._stream())

    def copy_history(self, x: torch.Tensor, history: torch.Tensor) -> None:
        """Entry 0 of every row's history (float32 [n, entries * width]) = x[r]."""
        n, width = x.shape
        _need(x, torch.float32, "copy_history x", 2)
        _need(history, torch.float32, "copy_history history", 2)
        if history.shape[0] != n or history.shape[1] % width:
            raise KernelError("copy_history: the history does not fit")
        self._scall("copy_history", _p(x), _p(history), _c_int(history.shape[1] // width), _c_int(n), _c_int(width),
                    self._stream())


_OPS = {}


def get_ops(dtype: str) -> KernelOps:
    """The shared KernelOps of a precision (libraries are loaded once per process)."""
    if dtype not in _OPS:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine has no CPU path")
        _OPS[dtype] = KernelOps(dtype)
    return _OPS[dtype]
