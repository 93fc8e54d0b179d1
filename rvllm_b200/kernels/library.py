"""The kernels of the product path, as methods that take torch tensors.

`CudaKernels` launches the hand-written sm_100a kernels of csrc/ on torch's current stream
through their exported C launchers.  bfloat16 matrix products with at least `TCGEN05_MIN_ROWS` rows
run on this project's tcgen05 / TMEM / TMA kernel (on pairs of CTAs where the rows fill its tiles);
with up to 32 rows, and with up to 64 where K need not be split, on its weight-streaming tcgen05
kernel; what lies between goes to the library GEMM behind `torch` (the reference calls cuBLASLt for
all its linear layers, v3/crates/rvllm-cutlass/src/cublaslt.rs).  Everything else is this project's
own code.  There is no CPU implementation: without a CUDA device, or when a kernel library cannot be
built, construction raises `KernelError`.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_void_p, c_int, c_float
from typing import Optional

import torch

from ..errors import KernelError
from . import build

_DT = {torch.float32: 0, torch.bfloat16: 1}
COUNTERS = {'launches': 0}   # kernels of this project launched so far (library GEMMs are not counted)
_STATUS = {-1: "a size is out of range", -2: "unsupported dtype", -3: "misaligned pointer or stride",
           -4: "size not supported by this kernel"}


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _check(name: str, status: int):
    if status == 0:
        COUNTERS['launches'] += 1
        return
    if status < 0:
        raise KernelError(f"{name}: refused, {_STATUS.get(status, 'code %d' % status)}")
    raise KernelError(f"{name}: CUDA launch failed with error {status}")


def _need(t: torch.Tensor, name: str, dtype=None, dims=None):
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous, got strides {t.stride()} for shape {tuple(t.shape)}")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, got shape {tuple(t.shape)}")


class AttentionMeta:
    """Per-step, per-cache-group arguments of the attention kernels (device int32 tensors) and
    the few host-side numbers that size their launches."""
    __slots__ = ("block_tables", "cu_seqlens", "ctx_lens", "token_seq", "slot_mapping", "num_seqs",
                 "max_q_len", "max_ctx_len", "max_blocks", "page_size", "num_decode")

    def __init__(self, block_tables, cu_seqlens, ctx_lens, token_seq, slot_mapping, num_seqs,
                 max_q_len, max_ctx_len, page_size, num_decode=0):
        self.num_decode = num_decode       # sequences that bring exactly one token
        self.block_tables, self.cu_seqlens, self.ctx_lens = block_tables, cu_seqlens, ctx_lens
        self.token_seq, self.slot_mapping = token_seq, slot_mapping
        self.num_seqs, self.max_q_len, self.max_ctx_len = num_seqs, max_q_len, max_ctx_len
        self.max_blocks = block_tables.shape[1]
        self.page_size = page_size


class CudaKernels:
    TCGEN05_MIN_ROWS = 128  # rows from which the tcgen05 GEMM of this project is used for bfloat16 ...
    TCGEN05_MIN_FILL = 0.0  # ... where its tiles keep its persistent workers busy for this share of their rounds
                            # (0: always.  With 0.8 the library's GEMM takes the partly filled shapes and is 20-140 %
                            # faster there, but its sums depend on the operands' addresses: the same request no longer
                            # gives the same bits in every run)
    PREFILL_SPLIT_MIN_KB = 32          # ... k blocks that a part keeps at least
    PREFILL_SPLIT_K = True             # ... or, where 2 or 4 CTAs per tile still fit the SMs, with K cut over a cluster of CTAs per tile
    NARROW_TILES = True                # ... with tiles of 128 columns where those of 256 would occupy at most half of the SMs
    PAIR_GEMM = True                   # the tcgen05 GEMM runs on pairs of CTAs (cta_group::2) where the rows fill its 256-row tiles
    TALKING_MMA = True                 # attention with mixed head weights: bfloat16 prompt portions go to the tensor-core kernel when it fits
    TALKING_SPLIT = True               # attention with mixed head weights: few tokens behind many keys go to the split-key kernels
    TALKING_SPLIT_MAX_TOKENS = 64      # ... up to this many tokens in the step
    TALKING_SPLIT_SPAN = 64            # ... in ranges of a multiple of this many keys
    TALKING_SPLIT_MAX_SCRATCH = 512 << 20   # ... while the scores of the step fit this many bytes of scratch
    TCGEN05_ATTENTION = True           # prompt portions go to the tcgen05 attention kernel when it fits
    TCGEN05_ATTENTION_MIN_TOKENS = 16  # ... from this many tokens in the longest portion of the step
    DECODE_MAX_ROWS = 64    # rows up to which the weight-streaming tcgen05 GEMM may be used
    DECODE_SPLIT_ROWS = 8   # ... when K has to be split over CTAs, only up to this many rows
    DECODE_BLOCK_MAX_ROWS = 256   # ... and, in blocks of 128 rows, for products of up to this many rows whose 128-feature
                                  # tiles x row blocks do not fill the SMs (q/k/v, o, down of a short prompt: the 256-row
                                  # tiles of the prefill GEMM would keep a fraction of the GPU busy)
    CLUSTER_REDUCE = True        # split-K partials of few rows are added up inside a thread-block cluster
    DECODE_K_ROTATE = 13         # tile t of a decode GEMM starts its K loop at block (t * this) mod its count, so that the CTAs of a
                                 # wave do not all read the same columns of the weights at a time (0: all start at the first block)
    DECODE_L2_AHEAD = 6          # k blocks of weights, beyond its stages, that a decode GEMM's CTA asks into L2 before its wait
    CLUSTER_MAX_ROWS = 64        # ... of up to this many rows (the whole range of the weight-streaming GEMM)
    CLUSTER_TARGET_CTAS = 225    # of such a product, tiles x splits (measured best at 8B, 7B and 32B layer sizes)
    TMA_DECODE = True       # decode attention's tiles come by TMA (head sizes 64 / 128, pages of 8 keys or more) ...
    TMA_DECODE_EARLY = True   # ... and keys older than the step's own are requested before the wait for the kernel before
    BALANCED_DECODE = True  # decode attention by the kernel that cuts all tiles evenly over resident CTAs ...
    BALANCED_MIN_PAIRS = 256  # ... from this many (sequence, kv head) pairs on
    LATENT_FLASH = True       # latent attention in bfloat16 runs on the tensor-core flash kernel where its sizes allow (else the plain kernel)
    LATENT_TCGEN05 = True     # ... and its prompt portions on the tcgen05 kernel's one-plane build (rows up to 256, values a multiple of 32)
    FUSED_QKV_PREFILL = True  # from TCGEN05_MIN_ROWS rows on the prefill GEMM rotates and writes the cache in its epilogue
    FUSED_NORM_MAX_ROWS = 0 # rows up to which an RMSNorm is applied inside the decode GEMM that consumes it
    FUSED_QKV_MAX_ROWS = 64 # rows up to which q/k/v product, rotation and cache write are one kernel
    pdl = os.environ.get("RVLLM_NO_PDL") != "1"   # programmatic dependent launch between kernels
    no_pdl_for = tuple(n for n in os.environ.get("RVLLM_NO_PDL_FOR", "").split(",") if n)   # ... but not for these source files
    num_sms = 148           # SMs of the device; asked from the device when the library is made

    def __init__(self, device="cuda:0"):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine has no CPU path")
        self.device = torch.device(device)
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise KernelError(f"the kernels are built for sm_100a; device {device} has compute capability {major}.{minor}")
        # the float32 path must never round operands to TF32 inside a library product
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        self.num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._libs = {}
        self._pdl_allowed = True     # a model may switch programmatic dependent launch off for its steps (`set_pdl`)
        self._decode_counters = None
        # one status word for every tcgen05 launch of the engine: a kernel whose bounded wait on an
        # mbarrier gave up writes a non-zero code here instead of hanging (see `raise_on_abort`)
        self._status = torch.zeros((1,), dtype=torch.int32, device=self.device)

    # ------------------------------------------------------------------ plumbing
    def _lib(self, source: str, defines=()):
        key = (source, tuple(defines))
        lib = self._libs.get(key)
        if lib is None:
            lib = build.load_library(source, defines)
            lib.rv_set_pdl(c_int(1 if (self.pdl and self._pdl_allowed and source not in self.no_pdl_for) else 0))
            if source == "gemm_tcgen05_decode.cu":
                lib.rv_gemm_decode_set_l2_ahead(c_int(self.DECODE_L2_AHEAD if (self.pdl and self._pdl_allowed) else 0))
                lib.rv_gemm_decode_set_k_rotate(c_int(self.DECODE_K_ROTATE))
            self._libs[key] = lib
        return lib

    def set_pdl(self, allowed: bool) -> None:
        """Allow or forbid programmatic dependent launch for every kernel launched from now on (the class switch `pdl`
        and the per-source exceptions still apply).  An engine calls this for its model before it runs a step."""
        allowed = bool(allowed)
        if allowed == self._pdl_allowed:
            return
        self._pdl_allowed = allowed
        for (source, _), lib in self._libs.items():
            on = self.pdl and allowed and source not in self.no_pdl_for
            lib.rv_set_pdl(c_int(1 if on else 0))
            if source == "gemm_tcgen05_decode.cu":
                lib.rv_gemm_decode_set_l2_ahead(c_int(self.DECODE_L2_AHEAD if on else 0))

    @staticmethod
    def _stream():
        return c_void_p(torch.cuda.current_stream().cuda_stream)

    @staticmethod
    def _dt(t: torch.Tensor, name: str) -> int:
        try:
            return _DT[t.dtype]
        except KeyError:
            raise KernelError(f"{name}: dtype {t.dtype} is not supported (float32, bfloat16)") from None

    # ------------------------------------------------------------------ aborted kernels
    @property
    def status_word(self) -> torch.Tensor:
        """int32 [1] on the device: 0, or the code of the first bounded wait that gave up in a tcgen05
        kernel launched without a status tensor of the caller's own."""
        return self._status

    def raise_on_abort(self, value: Optional[int] = None) -> None:
        """Raise `KernelError` if a kernel gave up a bounded wait since the last check: what it
        wrote is then not a result.  `value` is the status word as the caller has already read it
        (for instance copied to the host beside a step's sampled ids); None reads it now, which
        waits for the device.  After a non-zero value the word and the arrival counters of the
        split-K products are cleared, so that the next launches start clean (an aborted CTA skips
        its arrival, which would make a later launch take the wrong CTA for the last one)."""
        if value is None:
            value = int(self._status.item())
        if value == 0:
            return
        self._status.zero_()
        if self._decode_counters is not None:
            self._decode_counters.zero_()
        raise KernelError(f"a tcgen05 kernel gave up a bounded wait on an mbarrier (wait number {value} of the kernel's "
                          "source); what that step wrote is not a result")

    # ------------------------------------------------------------------ row kernels
    def gather_rows(self, table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """out[t] = table[ids[t]]; ids int32.  Used for the embedding and for picking logit rows."""
        _need(table, "table", dims=2); _need(ids, "ids", torch.int32, 1)
        if table.dtype == torch.int32:          # an integer table (which experts a token id uses): its rows are copied as 32-bit words
            return self.gather_rows(table.view(torch.float32), ids).view(torch.int32)
        out = torch.empty((ids.shape[0], table.shape[1]), dtype=table.dtype, device=table.device)
        st = self._lib("elementwise.cu").rv_gather_rows(
            _ptr(table), _ptr(ids), _ptr(out), c_int(ids.shape[0]), c_int(table.shape[1]),
            c_int(table.shape[0]), c_int(self._dt(table, "table")), self._stream())
        _check("gather_rows", st)
        return out

    def fill_normal(self, shape, dtype: torch.dtype, mean: float, std: float, seed: int, stream: int) -> torch.Tensor:
        """A new tensor of N(mean, std) values from the counter-based generator: element i depends
        on (seed, stream, i) only.  The engine's random-weights mode gives every tensor a stream of
        its own (its index among the sorted tensor names)."""
        out = torch.empty(tuple(shape), dtype=dtype, device=self.device)
        st = self._lib("elementwise.cu").rv_fill_normal(
            _ptr(out), ctypes.c_longlong(out.numel()), c_float(mean), c_float(std), ctypes.c_ulonglong(seed & (2 ** 64 - 1)),
            ctypes.c_ulonglong(stream), c_int(self._dt(out, "out")), self._stream())
        _check("fill_normal", st)
        return out

    def late_tokens(self, token_ids: torch.Tensor, cu_seqlens: torch.Tensor, source: torch.Tensor,
                    sampled: torch.Tensor) -> None:
        """token_ids[cu_seqlens[i]] = sampled[source[i]] for every sequence i with source[i] >= 0:
        tokens that the previous step sampled and the host has not read yet."""
        _need(token_ids, "token_ids", torch.int32, 1); _need(cu_seqlens, "cu_seqlens", torch.int32, 1)
        _need(source, "source", torch.int32, 1); _need(sampled, "sampled", torch.int32, 1)
        if cu_seqlens.shape[0] < source.shape[0]:
            raise KernelError(f"late_tokens: {source.shape[0]} sequences but {cu_seqlens.shape[0]} sequence starts")
        st = self._lib("elementwise.cu").rv_late_tokens(_ptr(token_ids), _ptr(cu_seqlens), _ptr(source), _ptr(sampled),
                                                        c_int(source.shape[0]), c_int(sampled.shape[0]), self._stream())
        _check("late_tokens", st)

    def rmsnorm(self, x: torch.Tensor, gamma: torch.Tensor, eps: float, out_dtype=None) -> torch.Tensor:
        _need(x, "x", dims=2); _need(gamma, "gamma", dims=1)
        if gamma.shape[0] != x.shape[1]:
            raise KernelError(f"rmsnorm: gamma has {gamma.shape[0]} entries for rows of {x.shape[1]}")
        if out_dtype is not None and out_dtype != x.dtype:      # a float32 stream normalised into the activations' type
            return self.residual_rmsnorm(x, gamma, eps, None, out_dtype, keep_residual=False)[1]
        out = torch.empty_like(x)
        st = self._lib("elementwise.cu").rv_rmsnorm(
            _ptr(x), _ptr(gamma), c_int(self._dt(gamma, "gamma")), _ptr(out), c_int(x.shape[0]),
            c_int(x.shape[1]), c_float(eps), c_int(self._dt(x, "x")), self._stream())
        _check("rmsnorm", st)
        return out

    def silu_mul(self, gate_up: torch.Tensor) -> torch.Tensor:
        """rows [gate | up] -> silu(gate) * up."""
        _need(gate_up, "gate_up", dims=2)
        inter = gate_up.shape[1] // 2
        if inter * 2 != gate_up.shape[1]:
            raise KernelError(f"silu_mul: row width {gate_up.shape[1]} is odd")
        out = torch.empty((gate_up.shape[0], inter), dtype=gate_up.dtype, device=gate_up.device)
        st = self._lib("elementwise.cu").rv_silu_mul(_ptr(gate_up), _ptr(out), c_int(gate_up.shape[0]),
                                                    c_int(inter), c_int(self._dt(gate_up, "gate_up")), self._stream())
        _check("silu_mul", st)
        return out

    def rope_cache_write(self, qkv, bias, positions, cos, sin, slot_mapping, cache_layer,
                         num_heads, num_kv_heads, head_dim, write_kv=True, out_dtype=None) -> torch.Tensor:
        """Add the q/k/v bias, rotate q and k, write k and v into their cache pages, return q
        [T, num_heads * head_dim].  qkv rows are [q | k | v], or q alone when `write_kv` is False.
        cache_layer: [num_pages, 2, num_kv_heads, page_size, head_dim].  `out_dtype` bfloat16 with
        float32 rows: the product stays in float until it has been biased and rotated."""
        _need(qkv, "qkv", dims=2); _need(positions, "positions", torch.int32, 1)
        out_dtype = out_dtype or qkv.dtype
        T = qkv.shape[0]
        width = (num_heads + (2 * num_kv_heads if write_kv else 0)) * head_dim
        if qkv.shape[1] != width:
            raise KernelError(f"rope_cache_write: qkv rows have {qkv.shape[1]} columns, expected {width}")
        if write_kv:
            _need(cache_layer, "cache_layer", out_dtype, 5); _need(slot_mapping, "slot_mapping", torch.int32, 1)
            if tuple(cache_layer.shape[1:3]) != (2, num_kv_heads) or cache_layer.shape[4] != head_dim:
                raise KernelError(f"rope_cache_write: cache layer of shape {tuple(cache_layer.shape)} does not "
                                  f"fit {num_kv_heads} kv heads of {head_dim}")
        rot = head_dim
        if cos is not None:
            _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
            rot = 2 * cos.shape[1]            # the leading `rot` elements of a head are rotated, the rest pass through
            if not 0 < rot <= head_dim or sin.shape != cos.shape:
                raise KernelError(f"rope_cache_write: cos/sin tables must be [rows, rotary_dim/2] with rotary_dim <= "
                                  f"head_dim {head_dim}, got {tuple(cos.shape)} and {tuple(sin.shape)}")
        if bias is not None:
            _need(bias, "bias", dims=1)
        q = torch.empty((T, num_heads * head_dim), dtype=out_dtype, device=qkv.device)
        page = cache_layer.shape[3] if write_kv else 1
        st = self._lib("elementwise.cu").rv_rope_cache_write(
            _ptr(qkv), _ptr(bias), c_int(self._dt(bias, "bias") if bias is not None else 0), _ptr(positions),
            _ptr(cos), _ptr(sin), _ptr(slot_mapping if write_kv else None), _ptr(cache_layer if write_kv else None),
            _ptr(q), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(page),
            c_int(1 if write_kv else 0), c_int(cos.shape[0] if cos is not None else 1), c_int(qkv.shape[1]),
            c_int(_DT[out_dtype]), c_int(rot), c_int(self._dt(qkv, "qkv")), self._stream())
        _check("rope_cache_write", st)
        return q

    # ------------------------------------------------------------------ attention
    def paged_attention(self, q, cache_layer, meta: AttentionMeta, num_heads, num_kv_heads, head_dim,
                        scale: float, window: Optional[int], softcap: Optional[float] = None,
                        sinks: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Attention of the step's tokens over the paged cache (keys of this step included).

        `softcap`: scaled scores pass c * tanh(s / c); `sinks` (float [heads]): exp(sink) joins each head's
        softmax denominator; `gate` (float [tokens, heads]): multiplies each head's output.

        bfloat16 with a head size that is a multiple of 16 and pages of a power of two go to the
        tensor-core flash kernel (one token per sequence: the decode tiling, keys split over CTAs
        when the batch alone cannot fill the GPU); everything else goes to the plain kernel."""
        page = cache_layer.shape[3]
        extras = softcap is not None or sinks is not None or gate is not None
        if q.dtype != torch.bfloat16 or head_dim % 16 or head_dim > 256 or (page & (page - 1)):
            return self.paged_attention_plain(q, cache_layer, meta, num_heads, num_kv_heads, head_dim, scale, window,
                                              softcap, sinks, gate)
        self._check_attention_extras(q, num_heads, sinks, gate)
        x = dict(softcap=softcap, sinks=sinks, gate=gate)
        out = torch.empty_like(q)
        group = num_heads // num_kv_heads
        # (the evenly cut decode kernel knows neither cap, sink nor gate: such layers stay with the split kernels)
        balanced = not extras and self._balanced_ok(meta, group, num_kv_heads)
        if self.TCGEN05_ATTENTION and meta.max_q_len >= self.TCGEN05_ATTENTION_MIN_TOKENS and head_dim in (64, 128) \
                and group <= 128 and page >= 8:
            self.attention_tcgen05(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window, **x)
            if meta.num_decode:
                if balanced:
                    self.flash_decode_balanced(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window)
                else:
                    self.decode_attention(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window, q_filter=1, **x)
            return out
        if meta.max_q_len == 1:
            if balanced:
                self.flash_decode_balanced(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window)
            else:
                self.decode_attention(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window,
                                      num_splits=self.decode_splits(meta, num_heads, num_kv_heads), **x)
        elif meta.num_decode == 0:
            self.flash_attention(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window, mode=0, **x)
        else:
            self.flash_attention(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window,
                                 mode=0, q_filter=2, **x)
            self.decode_attention(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window, q_filter=1, **x)
        return out

    def decode_attention(self, q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window,
                         num_splits=1, q_filter=0, status=None, tma=None, early=None, softcap=None, sinks=None, gate=None):
        """Attention of the step's one-token sequences (all of them, or with q_filter 1 those among
        longer ones) with the decode tiling, the keys split over `num_splits` CTAs: the tiles come by
        TMA where the kernel is built for the sizes (head size 64 or 128, pages of 8 keys or more),
        by cp.async otherwise; both give the same bits."""
        tma = self.TMA_DECODE if tma is None else tma
        if not tma or head_dim not in (64, 128) or cache_layer.shape[3] < 8:
            return self.flash_attention(q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window,
                                        mode=1, num_splits=num_splits, q_filter=q_filter, max_q_len=1,
                                        softcap=softcap, sinks=sinks, gate=gate)
        _need(q, "q", torch.bfloat16, 2); _need(cache_layer, "cache_layer", torch.bfloat16, 5)
        lib = self._lib("attention_flash.cu", (f"-DHEAD_DIM={head_dim}",))
        T = q.shape[0]
        scratch = None
        if num_splits > 1:
            scratch = torch.empty((num_splits * T * num_heads * (head_dim + 2),), dtype=torch.float32, device=q.device)
        early = self.TMA_DECODE_EARLY if early is None else early
        st = lib.rv_flash_decode_tma_ex(
            _ptr(q), _ptr(cache_layer), ctypes.c_longlong(cache_layer.shape[0]), _ptr(meta.block_tables), _ptr(meta.cu_seqlens),
            _ptr(meta.ctx_lens), _ptr(out), _ptr(scratch), c_int(T), c_int(meta.num_seqs), c_int(num_heads), c_int(num_kv_heads),
            c_int(head_dim), c_int(cache_layer.shape[3]), c_int(meta.max_blocks), c_float(scale), c_int(window or 0), c_int(1),
            c_int(num_splits), c_int(q_filter), _ptr(status if status is not None else self._status),
            c_int(1 if (early and self.pdl) else 0), c_float(softcap or 0.0), _ptr(sinks), _ptr(gate), self._stream())
        _check("flash_decode_tma", st)
        return out

    def decode_splits(self, meta: AttentionMeta, num_heads: int, num_kv_heads: int) -> int:
        """Into how many CTAs the keys of a sequence are split in a decode step.  Three CTAs of
        the kernel fit an SM (444 on a GPU of 148 SMs) and run in waves; a CTA costs about 4 us plus 2.25 us
        per 64-key tile (measured with all slots busy, where the tiles' bytes arrive at the speed
        of the memory), the merge kernel 2.5 us.  The split count with the least modelled time is
        taken: it fills one wave when the batch is small and keeps the last wave full when it is
        large."""
        self_max_splits = 64          # a long context at a small batch still fills the GPU (one sequence of 32,768 keys: 55)
        group = num_heads // num_kv_heads
        ctas = meta.num_seqs * num_kv_heads * ((group + 15) // 16)
        tiles = max(1, (meta.max_ctx_len + 63) // 64)
        best, best_t = 1, float("inf")
        for s in range(1, min(self_max_splits, tiles) + 1):
            per = -(-tiles // s)
            if s > 1 and per < 2:
                break
            # (the merge kernel reads eight splits per round trip)
            t = -(-ctas * s // (3 * self.num_sms)) * (4.0 + 2.25 * per) + (2.0 + 0.5 * -(-s // 8) if s > 1 else 0.0)
            if t < best_t - 1e-9:
                best, best_t = s, t
        return best

    def _balanced_tma_ctas(self, lib, num_heads: int, num_kv_heads: int) -> int:
        """CTAs of the TMA-fed evenly cut kernel that stay resident (asked from the device once per shape)."""
        key = (id(lib), num_heads, num_kv_heads)
        cache = self.__dict__.setdefault("_balanced_ctas", {})
        if key not in cache:
            cache[key] = int(lib.rv_flash_balanced_tma_ctas(c_int(num_heads), c_int(num_kv_heads)))
        return cache[key]

    def _balanced_ok(self, meta, group: int, num_kv_heads: int) -> bool:
        """The evenly cut decode kernel serves batches whose (sequence, kv head) pairs alone fill more
        than half of the resident CTAs: there the split kernel leaves waves half empty, and sequences
        of unequal length (continuous batching) unbalance it; smaller batches are faster split."""
        return (self.BALANCED_DECODE and group <= 16 and meta.num_seqs <= 256
                and meta.num_decode * num_kv_heads >= self.BALANCED_MIN_PAIRS)

    def flash_decode_balanced(self, q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window, ctas=0,
                              tma=None, status=None):
        """Decode attention for the sequences of the step that bring one token, the 64-key tiles of
        all (sequence, kv head) pairs cut evenly over a fixed number of resident CTAs; sequences
        with more tokens are left alone.  The tiles come by TMA where the kernel is built for the
        sizes (head size 64 or 128, pages of 8 keys or more, up to 240 sequences), by cp.async
        otherwise; both give the same bits."""
        _need(q, "q", torch.bfloat16, 2); _need(cache_layer, "cache_layer", torch.bfloat16, 5)
        lib = self._lib("attention_flash.cu", (f"-DHEAD_DIM={head_dim}",))
        T = q.shape[0]
        tma = self.TMA_DECODE if tma is None else tma
        if tma and head_dim in (64, 128) and cache_layer.shape[3] >= 8 and meta.num_seqs <= 240:
            grid = ctas or self._balanced_tma_ctas(lib, num_heads, num_kv_heads)
            if grid > 0:
                pieces = lib.rv_flash_balanced_max_pieces(c_int(meta.max_ctx_len), c_int(num_kv_heads), c_int(grid))
                scratch = torch.empty((pieces * T * num_heads * (head_dim + 2),), dtype=torch.float32, device=q.device)
                counts = torch.empty((meta.num_seqs * num_kv_heads,), dtype=torch.int32, device=q.device)
                st = lib.rv_flash_decode_balanced_tma(
                    _ptr(q), _ptr(cache_layer), ctypes.c_longlong(cache_layer.shape[0]), _ptr(meta.block_tables),
                    _ptr(meta.cu_seqlens), _ptr(meta.ctx_lens), _ptr(out), _ptr(scratch), _ptr(counts), c_int(pieces), c_int(T),
                    c_int(meta.num_seqs), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(cache_layer.shape[3]),
                    c_int(meta.max_blocks), c_float(scale), c_int(window or 0), c_int(grid),
                    _ptr(status if status is not None else self._status), self._stream())
                _check("flash_decode_balanced_tma", st)
                return out
        grid = ctas or 3 * self.num_sms
        pieces = lib.rv_flash_balanced_max_pieces(c_int(meta.max_ctx_len), c_int(num_kv_heads), c_int(grid))
        scratch = torch.empty((pieces * T * num_heads * (head_dim + 2),), dtype=torch.float32, device=q.device)
        counts = torch.empty((meta.num_seqs * num_kv_heads,), dtype=torch.int32, device=q.device)
        st = lib.rv_flash_decode_balanced(
            _ptr(q), _ptr(cache_layer), _ptr(meta.block_tables), _ptr(meta.cu_seqlens), _ptr(meta.ctx_lens), _ptr(out),
            _ptr(scratch), _ptr(counts), c_int(pieces), c_int(T), c_int(meta.num_seqs), c_int(num_heads),
            c_int(num_kv_heads), c_int(head_dim), c_int(cache_layer.shape[3]), c_int(meta.max_blocks), c_float(scale),
            c_int(window or 0), c_int(grid), self._stream())
        _check("flash_decode_balanced", st)
        return out

    def flash_attention(self, q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window,
                        mode=0, num_splits=1, q_filter=0, max_q_len=None, softcap=None, sinks=None, gate=None, value_dim=None):
        """The mma.sync flash kernel (mode 0: 64 rows per CTA, prompt portions; mode 1: 16 rows, warps and CTAs split the keys).
        `value_dim`: the build for one-plane caches, whose rows are keys in full and values in their leading `value_dim`
        elements; `out` then has rows of that width."""
        _need(q, "q", torch.bfloat16); _need(cache_layer, "cache_layer", torch.bfloat16, 5)
        defines = (f"-DHEAD_DIM={head_dim}",) if value_dim is None else (f"-DHEAD_DIM={head_dim}", f"-DV_DIM={value_dim}", "-DKV_PLANES=1")
        if cache_layer.shape[1] != (2 if value_dim is None else 1):
            raise KernelError(f"flash_attention: a cache layer of {cache_layer.shape[1]} planes for a kernel of {2 if value_dim is None else 1}")
        lib = self._lib("attention_flash.cu", defines)
        T = q.shape[0]
        scratch = None
        if num_splits > 1:
            scratch = torch.empty((num_splits * T * num_heads * ((value_dim or head_dim) + 2),), dtype=torch.float32, device=q.device)
        st = lib.rv_flash_attention_ex(
            _ptr(q), _ptr(cache_layer), _ptr(meta.block_tables), _ptr(meta.cu_seqlens), _ptr(meta.ctx_lens),
            _ptr(out), _ptr(scratch), c_int(T), c_int(meta.num_seqs), c_int(num_heads), c_int(num_kv_heads),
            c_int(head_dim), c_int(cache_layer.shape[3]), c_int(meta.max_blocks), c_float(scale), c_int(window or 0),
            c_int(mode), c_int(max_q_len or meta.max_q_len), c_int(num_splits), c_int(q_filter), c_float(softcap or 0.0),
            _ptr(sinks), _ptr(gate), self._stream())
        _check("flash_attention", st)
        if num_splits > 1:
            COUNTERS['launches'] += 1
        return out

    def attention_tcgen05(self, q, cache_layer, meta, out, num_heads, num_kv_heads, head_dim, scale, window, status=None,
                          softcap=None, sinks=None, gate=None, value_dim=None):
        """The tcgen05 flash-attention kernel for the sequences of a step that bring more than one
        token (bfloat16, head size 64 or 128, groups of up to 128 heads, pages of at least 8 keys).
        `value_dim`: the build for one-plane caches (rows of `head_dim` elements, up to 256, that are keys in full and
        values in their leading `value_dim` elements, a multiple of 32); `out` then has rows of that width."""
        _need(q, "q", torch.bfloat16); _need(cache_layer, "cache_layer", torch.bfloat16, 5)
        defines = (f"-DHEAD_DIM={head_dim}",) if value_dim is None else (f"-DLATENT_ROW={head_dim}", f"-DV_DIM={value_dim}")
        if cache_layer.shape[1] != (2 if value_dim is None else 1):
            raise KernelError(f"attention_tcgen05: a cache layer of {cache_layer.shape[1]} planes for a kernel of {2 if value_dim is None else 1}")
        lib = self._lib("attention_tcgen05.cu", defines)
        st = lib.rv_attention_tcgen05_ex(
            _ptr(q), _ptr(cache_layer), ctypes.c_longlong(cache_layer.shape[0]), _ptr(meta.block_tables),
            _ptr(meta.cu_seqlens), _ptr(meta.ctx_lens), _ptr(out), c_int(q.shape[0]), c_int(meta.num_seqs),
            c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(cache_layer.shape[3]), c_int(meta.max_blocks),
            c_float(scale), c_int(window or 0), c_int(meta.max_q_len), _ptr(status if status is not None else self._status),
            c_float(softcap or 0.0), _ptr(sinks), _ptr(gate), self._stream())
        _check("attention_tcgen05", st)
        return out

    def paged_attention_plain(self, q, cache_layer, meta, num_heads, num_kv_heads, head_dim, scale, window,
                              softcap=None, sinks=None, gate=None):
        _need(q, "q", dims=2); _need(cache_layer, "cache_layer", q.dtype, 5)
        self._check_attention_extras(q, num_heads, sinks, gate)
        out = torch.empty_like(q)
        st = self._lib("attention_ref.cu").rv_paged_attention_ref(
            _ptr(q), _ptr(cache_layer), _ptr(meta.block_tables), _ptr(meta.cu_seqlens), _ptr(meta.ctx_lens),
            _ptr(meta.token_seq), _ptr(out), c_int(q.shape[0]), c_int(num_heads), c_int(num_kv_heads),
            c_int(head_dim), c_int(cache_layer.shape[3]), c_int(meta.max_blocks), c_float(scale),
            c_int(window or 0), c_float(softcap or 0.0), _ptr(sinks), _ptr(gate), c_int(self._dt(q, "q")), self._stream())
        _check("paged_attention_plain", st)
        return out

    @staticmethod
    def _check_attention_extras(q, num_heads, sinks, gate):
        if sinks is not None:
            _need(sinks, "sinks", torch.float32, 1)
            if sinks.shape[0] != num_heads:
                raise KernelError(f"attention: {sinks.shape[0]} sinks for {num_heads} heads")
        if gate is not None:
            _need(gate, "gate", torch.float32, 2)
            if tuple(gate.shape) != (q.shape[0], num_heads):
                raise KernelError(f"attention: gate of shape {tuple(gate.shape)} for {q.shape[0]} tokens of {num_heads} heads")

    # ------------------------------------------------------------------ linear layers
    def linear(self, x, weight, bias=None, residual=None, out_dtype=None, norm=None) -> torch.Tensor:
        """x [M, K] . weight [N, K]^T (+ bias) (+ residual), accumulated in float.
        norm = (gamma, eps): x is normalised first (RMSNorm); few bfloat16 rows get it inside the GEMM.

        float32 operands: this project's FFMA kernel (no TF32 anywhere).  bfloat16 operands: the
        library GEMM; the residual is added in its float epilogue (beta = 1).  A weight kept in
        32 bits under a bfloat16 engine is multiplied in float32."""
        _need(x, "x", dims=2); _need(weight, "weight", dims=2)
        M, K = x.shape
        N = weight.shape[0]
        if weight.shape[1] != K:
            raise KernelError(f"linear: x has {K} columns, weight has {weight.shape[1]}")
        out_dtype = out_dtype or x.dtype
        if norm is not None:
            fuse = (self._can_fuse_norm(x, norm) and weight.dtype == torch.bfloat16 and self._use_decode_gemm(M, N, K, False)
                    and out_dtype in (torch.bfloat16, torch.float32)
                    and (residual is None or (residual.dtype == torch.bfloat16 and out_dtype == torch.bfloat16)))
            if fuse:
                return self.linear_decode(x, weight, bias, residual, out_dtype, norm=norm)
            x = self.rmsnorm(x, *norm, out_dtype=weight.dtype if x.dtype == torch.float32 else None)
        if weight.dtype == torch.float32:
            xf = x if x.dtype == torch.float32 else x.float()
            rf = None
            if residual is not None:
                rf = residual if residual.dtype == torch.float32 else residual.float()
                _need(rf, "residual", dims=2)
            if bias is not None:
                _need(bias, "bias", dims=1)
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
            st = self._lib("gemm_f32.cu").rv_gemm_f32(
                _ptr(xf), _ptr(weight), _ptr(bias), c_int(self._dt(bias, "bias") if bias is not None else 0),
                _ptr(rf), _ptr(out), c_int(M), c_int(N), c_int(K), self._stream())
            _check("gemm_f32", st)
            return out if out_dtype == torch.float32 else out.to(out_dtype)
        if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
            raise KernelError(f"linear: unsupported operand types {x.dtype} x {weight.dtype}")
        return self._linear_bf16(x, weight, bias, residual, out_dtype)

    def _linear_bf16(self, x, weight, bias, residual, out_dtype):
        M, K = x.shape
        if self._use_decode_gemm(M, weight.shape[0], K, False) and out_dtype in (torch.bfloat16, torch.float32) \
                and (residual is None or (residual.dtype == torch.bfloat16 and out_dtype == torch.bfloat16)):
            return self.linear_decode(x, weight, bias, residual, out_dtype)
        if self._tcgen05_fills(M, weight.shape[0]) and K % 8 == 0 and bias is None and out_dtype in (torch.bfloat16, torch.float32) \
                and (residual is None or (residual.dtype == torch.bfloat16 and out_dtype == torch.bfloat16)):
            return self.linear_tcgen05(x, weight, residual, out_dtype)
        if out_dtype == torch.float32:
            out = torch.mm(x, weight.t(), out_dtype=torch.float32)
            if bias is not None:
                out += bias.float()
            if residual is not None:
                out += residual.float()
            return out
        if residual is not None and bias is None:
            return torch.addmm(residual, x, weight.t())
        if residual is not None:
            # bias and residual: the sum is formed in float and rounded once
            out = torch.mm(x, weight.t(), out_dtype=torch.float32)
            out += bias.float()
            out += residual.float()
            return out.to(out_dtype)
        return torch.nn.functional.linear(x, weight, bias.to(x.dtype) if bias is not None else None)

    def _tcgen05_fills(self, M: int, N: int, gated: bool = False) -> bool:
        """Whether this project's tcgen05 GEMM is the one to use for M rows and N weight rows: from
        `TCGEN05_MIN_ROWS` rows on, and only where its persistent workers (one CTA per SM, or one pair per two SMs on
        tiles of 256 rows) are busy for at least `TCGEN05_MIN_FILL` of their rounds.  Where a last
        round stays mostly empty the library's GEMM, which cuts such shapes differently, measured
        20 to 140 % faster (o_proj at 512 rows: 22.6 against 41 us)."""
        if M < self.TCGEN05_MIN_ROWS:
            return False
        pair = self.PAIR_GEMM and (M % 256 == 0 or M % 256 > 128)
        rows, workers = (256, self.num_sms // 2) if pair else (128, self.num_sms)
        tiles = -(-M // rows) * (-(-(N // 2) // 128) if gated else -(-N // 256))
        rounds = -(-tiles // workers)
        return tiles >= self.TCGEN05_MIN_FILL * rounds * workers

    def _prefill_splits(self, M: int, N: int, K: int, gated: bool = False, head_dim: int = 0) -> int:
        """Into how many parts (1, 2 or 4) the prefill GEMM cuts K over a cluster of CTAs per tile of 128 rows x 256
        columns: as many as keep all CTAs within the SMs, with 32 k blocks each at least (the exchange of the partials
        through the cluster's shared memory costs about 7 us, as much as 16 k blocks); with the rotary epilogue only
        while a CTA's share of the columns holds whole heads."""
        if gated or not self.PREFILL_SPLIT_K or M < self.TCGEN05_MIN_ROWS:
            return 1
        tiles = -(-M // 128) * -(-N // 256)
        for s in (4, 2):
            if tiles * s <= self.num_sms and ((K + 63) // 64) // s >= self.PREFILL_SPLIT_MIN_KB and (head_dim == 0 or (256 // s) % head_dim == 0):
                return s
        return 1

    def _prefill_gemm_lib(self, M: int, pair=None, N: int = 0, gated: bool = False, head_dim: int = 0):
        """The tcgen05 GEMM library for M rows: built for pairs of CTAs (tiles of 256 rows) unless the
        last tile's second half would be empty, or for one CTA per tile (tiles of 128 rows); with
        tiles of 128 columns instead of 256 where the wide ones would leave half of the workers without
        a tile (N given: a few hundred rows of a product with few weight rows)."""
        if pair is None:
            pair = self.PAIR_GEMM and (M % 256 == 0 or M % 256 > 128)
        defines = ("-DRV_PAIR=1",) if pair else ()
        if N and self.NARROW_TILES and head_dim <= 128:        # (a head's rotation pairs lie in one tile)
            rows, workers = (256, self.num_sms // 2) if pair else (128, self.num_sms)
            tiles = -(-M // rows) * (-(-(N // 2) // 128) if gated else -(-N // 256))
            if 2 * tiles <= workers + workers // 8:
                defines = defines + ("-DBN=128",)
        return self._lib("gemm_tcgen05.cu", defines)

    def linear_tcgen05(self, x, weight, residual=None, out_dtype=None, gated=False, status=None, max_ctas=0, pair=None,
                       splits=None, activation="silu"):
        """The tcgen05 / TMEM / TMA GEMM for bfloat16 (any M; K a multiple of 8).  gated: weight rows
        are [gate | up] and the result is silu(x gate^T) * (x up^T).  `status`: optional int32 device
        tensor that receives a non-zero code if a bounded wait inside the kernel gave up.  `pair`:
        the build on pairs of CTAs (cta_group::2) or on single CTAs; default: by the number of rows."""
        _need(x, "x", torch.bfloat16, 2); _need(weight, "weight", torch.bfloat16, 2)
        M, K = x.shape
        N = weight.shape[0]
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
        if residual is not None:
            _need(residual, "residual", torch.bfloat16, 2)
        epilogue = (4 if activation == "gelu_tanh" else 2) if gated else (1 if residual is not None else 0)
        if splits is None:
            splits = self._prefill_splits(M, N, K, gated) if (max_ctas == 0 and pair is None) else 1
        if splits > 1:
            lib = self._lib("gemm_tcgen05.cu", ())          # K over a cluster: the build on single CTAs, wide tiles
        else:
            lib = self._prefill_gemm_lib(M, pair, N, gated)
        st = lib.rv_gemm_tcgen05_bf16(
            _ptr(x), _ptr(weight), _ptr(residual), _ptr(out), c_int(1 if out_dtype == torch.float32 else 0),
            c_int(M), c_int(N), c_int(K), c_int(epilogue), _ptr(status if status is not None else self._status), c_int(max_ctas),
            c_int(splits), self._stream())
        _check("gemm_tcgen05", st)
        return out

    def _use_decode_gemm(self, M: int, N: int, K: int, gated: bool) -> bool:
        """Whether the weight-streaming tcgen05 GEMM serves this product: few rows, and either
        enough 128-feature tiles to fill the GPU without splitting K, or so few rows that the
        split reduction is cheap."""
        if M <= 0 or K % 8:
            return False
        tiles = ((N // 2 + 63) // 64) if gated else (N + 127) // 128
        if M > self.DECODE_MAX_ROWS:
            return (not gated and self.CLUSTER_REDUCE and M <= self.DECODE_BLOCK_MAX_ROWS
                    and tiles * ((M + 127) // 128) <= self.num_sms)
        split_rows = self.CLUSTER_MAX_ROWS if (self.CLUSTER_REDUCE and not gated) else self.DECODE_SPLIT_ROWS
        return M <= max(split_rows, self.DECODE_SPLIT_ROWS) or self.gemm_splits(tiles, K) == 1

    def gemm_splits(self, n_tiles: int, K: int) -> int:
        """Into how many CTAs the K dimension of a decode GEMM is cut: about two CTAs per SM with
        at least four 64-wide k blocks each, three per SM where that still leaves sixteen (measured:
        cutting finer costs more in the merge than it gains in bandwidth)."""
        num_kb = (K + 63) // 64
        two, three = 2 * self.num_sms // max(n_tiles, 1), 3 * self.num_sms // max(n_tiles, 1)
        if three > two and num_kb // three >= 16:
            return min(three, 32)
        return max(1, min(two, num_kb // 4, 32))

    def _norm_args(self, norm, K):
        """ctypes arguments for a fused RMSNorm (gamma [K], eps), or the three nulls."""
        if norm is None:
            return c_void_p(0), c_int(0), c_float(0.0)
        gamma, eps = norm
        _need(gamma, "norm weight", dims=1)
        if gamma.shape[0] != K:
            raise KernelError(f"fused norm: gamma has {gamma.shape[0]} entries for rows of {K}")
        return _ptr(gamma), c_int(self._dt(gamma, "norm weight")), c_float(eps)

    def _can_fuse_norm(self, x, norm) -> bool:
        return (norm is not None and x.dtype == torch.bfloat16 and 0 < x.shape[0] <= self.FUSED_NORM_MAX_ROWS
                and x.shape[1] <= 8128)       # the kernel keeps gamma of its K range in shared memory

    def _cluster_policy(self, M, gated, splits, cluster, tiles, K, chosen):
        """(splits, cluster) of a decode GEMM.  Up to `CLUSTER_MAX_ROWS` rows of a product that is not
        gated are cut into at most 8 CTAs per tile, which add their partials up inside a cluster; where
        the caller left the cut open, about `CLUSTER_TARGET_CTAS` CTAs in all (measured: more CTAs
        than that delay the next kernel's first loads by more than they gain)."""
        if M > self.DECODE_MAX_ROWS and not gated:
            # blocks of 128 rows, one CTA per SM (four stages of 32 KB and the cluster's buffers fill one): K is
            # split so that tiles x row blocks x splits stay within the SMs, inside a cluster or not at all
            if not chosen:         # (clusters do not fill the last SMs of every GPC: an eighth of the SMs is left out of the count)
                splits = (self.num_sms - self.num_sms // 8) // max(tiles * ((M + 127) // 128), 1)
            splits = max(1, min(splits, 8, ((K + 63) // 64) // 4))
            return splits, splits >= 2 and cluster is not False
        if cluster is None:
            cluster = self.CLUSTER_REDUCE and not gated and 0 < M <= self.CLUSTER_MAX_ROWS and splits >= 2
            if cluster:
                if not chosen:
                    splits = max(2, min(self.CLUSTER_TARGET_CTAS // max(tiles, 1), ((K + 63) // 64) // 4))
                splits = min(splits, 8)
        return splits, bool(cluster)

    def linear_decode(self, x, weight, bias=None, residual=None, out_dtype=None, gated=False, splits=None, status=None,
                      norm=None, cluster=None, activation="silu"):
        """The weight-streaming tcgen05 GEMM for few rows of bfloat16 activations (beyond 128 rows:
        in blocks of 128, K split inside a cluster or not at all).
        norm = (gamma, eps): RMSNorm applied to x inside the kernel (at most 16 rows)."""
        _need(x, "x", torch.bfloat16, 2); _need(weight, "weight", torch.bfloat16, 2)
        M, K = x.shape
        N = weight.shape[0]
        lib = self._lib("gemm_tcgen05_decode.cu")
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
        tiles = lib.rv_gemm_decode_tiles(c_int(N), c_int(1 if gated else 0))
        chosen = splits is not None
        if splits is None:
            splits = self.gemm_splits(tiles, K)
        splits = max(1, min(splits, (K + 63) // 64))
        splits, cluster = self._cluster_policy(M, gated, splits, cluster, tiles, K, chosen)
        scratch = None
        if splits > 1 and not (cluster and M > self.DECODE_MAX_ROWS):
            if self._decode_counters is None or self._decode_counters.numel() < tiles:
                self._decode_counters = torch.zeros((max(tiles, 4096),), dtype=torch.int32, device=x.device)
            mb = lib.rv_gemm_decode_padded_rows(c_int(M))
            scratch = torch.empty((tiles * splits * mb * 128,), dtype=torch.float32, device=x.device)
        if bias is not None:
            _need(bias, "bias", dims=1)
        if residual is not None:
            _need(residual, "residual", torch.bfloat16, 2)
        st = lib.rv_gemm_tcgen05_decode_bf16(
            _ptr(x), _ptr(weight), _ptr(bias), c_int(self._dt(bias, "bias") if bias is not None else 0), _ptr(residual),
            _ptr(out), c_int(1 if out_dtype == torch.float32 else 0), c_int(M), c_int(N), c_int(K),
            c_int((2 if activation == "gelu_tanh" else 1) if gated else 0), c_int(splits), c_int(1 if cluster else 0), _ptr(scratch),
            _ptr(self._decode_counters if splits > 1 else None),
            _ptr(status if status is not None else self._status), *self._norm_args(norm, K), self._stream())
        _check("gemm_tcgen05_decode", st)
        return out

    def qkv_rope_cache_write(self, x, weight, bias, positions, cos, sin, slot_mapping, cache_layer,
                             num_heads, num_kv_heads, head_dim, norm=None) -> torch.Tensor:
        """The q/k/v product of the step's rows, then bias, rotation of q and k and the write of k
        and v into the rows' cache slots; returns q [T, num_heads * head_dim].  For few bfloat16
        rows this is one kernel (the decode GEMM's rotary epilogue); otherwise the product and
        `rope_cache_write` run one after the other, with the same result.  Tables narrower than
        head_dim / 2 (a rotation of the leading part of each head only) always take the latter.
        norm = (gamma, eps): x is normalised first (RMSNorm), inside the fused kernel where that runs."""
        M, K = x.shape
        full_rotation = cos is None or cos.shape[1] == head_dim // 2      # the rotary epilogues rotate whole heads
        few = 0 < M <= self.FUSED_QKV_MAX_ROWS or (M > self.DECODE_MAX_ROWS and self._use_decode_gemm(M, weight.shape[0], K, False))
        if (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and few and full_rotation
                and 128 % head_dim == 0 and K % 8 == 0 and weight.shape[0] == (num_heads + 2 * num_kv_heads) * head_dim):
            if norm is not None and not self._can_fuse_norm(x, norm):
                x, norm = self.rmsnorm(x, *norm), None
            return self._qkv_rope_fused(x, weight, bias, positions, cos, sin, slot_mapping, cache_layer,
                                        num_heads, num_kv_heads, head_dim, norm=norm)
        if norm is not None:
            x = self.rmsnorm(x, *norm)
        if (self.FUSED_QKV_PREFILL and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and full_rotation
                and self._tcgen05_fills(M, weight.shape[0]) and head_dim in (64, 128, 256) and K % 8 == 0
                and weight.shape[0] == (num_heads + 2 * num_kv_heads) * head_dim):
            return self._qkv_rope_tcgen05(x, weight, bias, positions, cos, sin, slot_mapping, cache_layer,
                                          num_heads, num_kv_heads, head_dim)
        # the product leaves its kernel in float and is rounded once, after bias and rotation
        qkv = self.linear(x, weight, out_dtype=torch.float32)
        return self.rope_cache_write(qkv, bias, positions, cos, sin, slot_mapping, cache_layer,
                                     num_heads, num_kv_heads, head_dim, out_dtype=x.dtype)

    def _qkv_rope_tcgen05(self, x, weight, bias, positions, cos, sin, slot_mapping, cache_layer,
                          num_heads, num_kv_heads, head_dim, status=None, max_ctas=0, pair=None, splits=None):
        """The prefill tcgen05 GEMM with the rotary epilogue (many rows, head sizes 64 / 128 / 256)."""
        _need(x, "x", torch.bfloat16, 2); _need(weight, "weight", torch.bfloat16, 2)
        _need(positions, "positions", torch.int32, 1); _need(slot_mapping, "slot_mapping", torch.int32, 1)
        _need(cache_layer, "cache_layer", torch.bfloat16, 5)
        M, K = x.shape
        if weight.shape[1] != K or positions.shape[0] < M or slot_mapping.shape[0] < M:
            raise KernelError("qkv_rope_cache_write: shapes of x, weight, positions and slot_mapping do not agree")
        if tuple(cache_layer.shape[1:3]) != (2, num_kv_heads) or cache_layer.shape[4] != head_dim:
            raise KernelError(f"qkv_rope_cache_write: cache layer of shape {tuple(cache_layer.shape)} does not "
                              f"fit {num_kv_heads} kv heads of {head_dim}")
        if cos is not None:
            _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
            if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
                raise KernelError("qkv_rope_cache_write: cos/sin tables must be [rows, head_dim/2]")
        if bias is not None:
            _need(bias, "bias", dims=1)
        q = torch.empty((M, num_heads * head_dim), dtype=torch.bfloat16, device=x.device)
        if splits is None:
            splits = self._prefill_splits(M, weight.shape[0], K, False, head_dim) if (max_ctas == 0 and pair is None) else 1
        if splits > 1:
            lib = self._lib("gemm_tcgen05.cu", ())
        else:
            lib = self._prefill_gemm_lib(M, pair, weight.shape[0], head_dim=head_dim)
        st = lib.rv_gemm_tcgen05_qkv_rope(
            _ptr(x), _ptr(weight), _ptr(bias), c_int(self._dt(bias, "bias") if bias is not None else 0),
            _ptr(positions), _ptr(cos), _ptr(sin), _ptr(slot_mapping), _ptr(cache_layer), _ptr(q), c_int(M), c_int(K),
            c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(cache_layer.shape[3]),
            c_int(cos.shape[0] if cos is not None else 1), _ptr(status if status is not None else self._status), c_int(max_ctas),
            c_int(splits), self._stream())
        _check("gemm_tcgen05_qkv_rope", st)
        return q

    def _qkv_rope_fused(self, x, weight, bias, positions, cos, sin, slot_mapping, cache_layer,
                        num_heads, num_kv_heads, head_dim, splits=None, status=None, norm=None, cluster=None):
        _need(x, "x", torch.bfloat16, 2); _need(weight, "weight", torch.bfloat16, 2)
        _need(positions, "positions", torch.int32, 1); _need(slot_mapping, "slot_mapping", torch.int32, 1)
        _need(cache_layer, "cache_layer", torch.bfloat16, 5)
        M, K = x.shape
        N = weight.shape[0]
        if weight.shape[1] != K or positions.shape[0] < M or slot_mapping.shape[0] < M:
            raise KernelError("qkv_rope_cache_write: shapes of x, weight, positions and slot_mapping do not agree")
        if tuple(cache_layer.shape[1:3]) != (2, num_kv_heads) or cache_layer.shape[4] != head_dim:
            raise KernelError(f"qkv_rope_cache_write: cache layer of shape {tuple(cache_layer.shape)} does not "
                              f"fit {num_kv_heads} kv heads of {head_dim}")
        if cos is not None:
            _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
            if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
                raise KernelError("qkv_rope_cache_write: cos/sin tables must be [rows, head_dim/2]")
        if bias is not None:
            _need(bias, "bias", dims=1)
        lib = self._lib("gemm_tcgen05_decode.cu")
        tiles = lib.rv_gemm_decode_tiles(c_int(N), c_int(0))
        chosen = splits is not None
        if splits is None:
            splits = self.gemm_splits(tiles, K)
        splits = max(1, min(splits, (K + 63) // 64))
        splits, cluster = self._cluster_policy(M, False, splits, cluster, tiles, K, chosen)
        scratch = None
        if splits > 1 and not (cluster and M > self.DECODE_MAX_ROWS):
            if self._decode_counters is None or self._decode_counters.numel() < tiles:
                self._decode_counters = torch.zeros((max(tiles, 4096),), dtype=torch.int32, device=x.device)
            mb = lib.rv_gemm_decode_padded_rows(c_int(M))
            scratch = torch.empty((tiles * splits * mb * 128,), dtype=torch.float32, device=x.device)
        q = torch.empty((M, num_heads * head_dim), dtype=torch.bfloat16, device=x.device)
        st = lib.rv_gemm_decode_qkv_rope(
            _ptr(x), _ptr(weight), _ptr(bias), c_int(self._dt(bias, "bias") if bias is not None else 0),
            _ptr(positions), _ptr(cos), _ptr(sin), _ptr(slot_mapping), _ptr(cache_layer), _ptr(q), c_int(M), c_int(K),
            c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(cache_layer.shape[3]),
            c_int(cos.shape[0] if cos is not None else 1), c_int(splits), c_int(1 if cluster else 0), _ptr(scratch),
            _ptr(self._decode_counters if splits > 1 else None), _ptr(status if status is not None else self._status), *self._norm_args(norm, K), self._stream())
        _check("gemm_decode_qkv_rope", st)
        return q

    def gate_up_silu(self, x, weight, norm=None) -> torch.Tensor:
        """silu(x Wg^T) * (x Wu^T) for weight rows [Wg | Wu]; see `gate_up_act`."""
        return self.gate_up_act(x, weight, "silu", norm=norm)

    def gate_up_act(self, x, weight, activation: str = "silu", norm=None) -> torch.Tensor:
        """act(x Wg^T) * (x Wu^T) for weight rows [Wg | Wu], act = "silu" or "gelu_tanh": one fused kernel for
        bfloat16 rows (the weight-streaming GEMM for few, the prefill GEMM for many; the activation is applied to the
        float accumulators in the epilogue), else the product followed by the activation kernel.  norm = (gamma, eps):
        x is normalised first (RMSNorm), inside the kernel for few rows."""
        if activation not in self.ACTIVATIONS:
            raise KernelError(f"gate_up_act: activation {activation!r} is not known ({', '.join(self.ACTIVATIONS)})")
        M, K = x.shape
        if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.shape[0] % 2 == 0 \
                and self._use_decode_gemm(M, weight.shape[0], K, True):
            if norm is not None and not self._can_fuse_norm(x, norm):
                x, norm = self.rmsnorm(x, *norm), None
            return self.linear_decode(x, weight, gated=True, norm=norm, activation=activation)
        if norm is not None:
            x = self.rmsnorm(x, *norm)
        if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and self._tcgen05_fills(M, weight.shape[0], True) \
                and K % 8 == 0 and weight.shape[0] % 2 == 0:
            return self.linear_tcgen05(x, weight, gated=True, activation=activation)
        if activation == "silu":
            return self.silu_mul(self.linear(x, weight))
        # the product leaves its kernel in float; the activation kernel rounds once
        return self.act_mul(self.linear(x, weight, out_dtype=torch.float32), activation, x.dtype)

    # ------------------------------------------------------------------ output-norm layers, gated attention, state-space mixer
    def residual_rmsnorm(self, y, gamma, eps: float, residual: Optional[torch.Tensor], rounded_dtype=None,
                         keep_residual: bool = True, next_norm=None):
        """r = residual + y / sqrt(mean(y^2) + eps) * gamma in float32 (residual None: zero).  Returns
        (r as float32 [rows, cols] or None without `keep_residual`, r rounded to `rounded_dtype` or None).
        `residual` is updated in place when given.  next_norm = (gamma', eps'): the second result is not r itself
        but r / sqrt(mean(r^2) + eps') * gamma' in `rounded_dtype`, the input of a sublayer that normalises what it reads."""
        _need(y, "y", dims=2); _need(gamma, "gamma", dims=1)
        rows, cols = y.shape
        if gamma.shape[0] != cols:
            raise KernelError(f"residual_rmsnorm: gamma has {gamma.shape[0]} entries for rows of {cols}")
        if residual is not None:
            _need(residual, "residual", torch.float32, 2)
            if residual.shape != y.shape:
                raise KernelError(f"residual_rmsnorm: residual {tuple(residual.shape)} against rows {tuple(y.shape)}")
        res_out = None
        if keep_residual:
            res_out = residual if residual is not None else torch.empty((rows, cols), dtype=torch.float32, device=y.device)
        rounded = None
        if next_norm is not None:
            if rounded_dtype is None or not keep_residual:
                raise KernelError("residual_rmsnorm: a following norm needs the stream kept and a type for its result")
            _need(next_norm[0], "next gamma", dims=1)
            if next_norm[0].shape[0] != cols:
                raise KernelError(f"residual_rmsnorm: the following norm has {next_norm[0].shape[0]} entries for rows of {cols}")
            rounded = torch.empty((rows, cols), dtype=rounded_dtype, device=y.device)
            st = self._lib("rowops.cu").rv_residual_rmsnorm_next(
                _ptr(y), c_int(self._dt(y, "y")), _ptr(gamma), c_int(self._dt(gamma, "gamma")), _ptr(residual), _ptr(res_out),
                _ptr(rounded), c_int(_DT[rounded_dtype]), c_int(rows), c_int(cols), c_float(eps), _ptr(next_norm[0]),
                c_int(self._dt(next_norm[0], "next gamma")), c_float(next_norm[1]), self._stream())
            _check("residual_rmsnorm", st)
            return res_out, rounded
        if rounded_dtype is not None and not (rounded_dtype == torch.float32 and keep_residual):
            rounded = torch.empty((rows, cols), dtype=rounded_dtype, device=y.device)
        st = self._lib("rowops.cu").rv_residual_rmsnorm(
            _ptr(y), c_int(self._dt(y, "y")), _ptr(gamma), c_int(self._dt(gamma, "gamma")), _ptr(residual), _ptr(res_out),
            _ptr(rounded), c_int(_DT[rounded_dtype] if rounded is not None else 0), c_int(rows), c_int(cols), c_float(eps),
            self._stream())
        _check("residual_rmsnorm", st)
        if rounded is None and rounded_dtype == torch.float32:
            rounded = res_out
        return res_out, rounded

    ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}

    def act_mul(self, gate_up: torch.Tensor, activation: str, out_dtype=None, limit: Optional[float] = None,
                alpha: Optional[float] = None) -> torch.Tensor:
        """rows [gate | up] -> act(gate) * up, computed in float.  "swiglu_clamp": g sigmoid(alpha g) (u + 1) with
        g = min(gate, limit), u = clamp(up, -limit, limit)."""
        _need(gate_up, "gate_up", dims=2)
        if activation not in self.ACTIVATIONS and activation != "swiglu_clamp":
            raise KernelError(f"act_mul: activation {activation!r} is not known ({', '.join(self.ACTIVATIONS)}, swiglu_clamp)")
        inter = gate_up.shape[1] // 2
        if inter * 2 != gate_up.shape[1]:
            raise KernelError(f"act_mul: row width {gate_up.shape[1]} is odd")
        out = torch.empty((gate_up.shape[0], inter), dtype=out_dtype or gate_up.dtype, device=gate_up.device)
        if activation == "swiglu_clamp":
            if limit is None or alpha is None:
                raise KernelError("act_mul: swiglu_clamp needs `limit` and `alpha`")
            st = self._lib("streamops.cu").rv_act_mul_clamp(_ptr(gate_up), c_int(self._dt(gate_up, "gate_up")), _ptr(out),
                                                           c_int(self._dt(out, "out")), c_int(gate_up.shape[0]), c_int(inter),
                                                           c_float(limit), c_float(alpha), self._stream())
            _check("act_mul", st)
            return out
        st = self._lib("rowops.cu").rv_act_mul(_ptr(gate_up), c_int(self._dt(gate_up, "gate_up")), _ptr(out), c_int(self._dt(out, "out")),
                                               c_int(gate_up.shape[0]), c_int(inter), c_int(self.ACTIVATIONS[activation]), self._stream())
        _check("act_mul", st)
        return out

    def qk_norm_rope_cache_write(self, proj, q_gamma, k_gamma, eps: float, positions, cos, sin, slot_mapping, cache_layer,
                                 num_heads, num_kv_heads, head_dim, out_dtype, with_gate: bool = False, write_kv: bool = True):
        """proj rows [q | k | gate logits]: q and k are each RMS-normalised over their whole part of the row
        (weights `q_gamma`, `k_gamma` of those widths), the leading 2 * cos.shape[1] elements of every head are
        rotated, k goes into the token's cache slot as the key and, as projected, as the value.
        Returns (q [T, heads * head_dim] in `out_dtype`, sigmoid(gate logits) float [T, heads] or None)."""
        _need(proj, "proj", dims=2); _need(positions, "positions", torch.int32, 1)
        _need(q_gamma, "q_gamma", dims=1); _need(k_gamma, "k_gamma", q_gamma.dtype, 1)
        T = proj.shape[0]
        qw, kw = num_heads * head_dim, num_kv_heads * head_dim
        if proj.shape[1] != qw + kw + (num_heads if with_gate else 0):
            raise KernelError(f"qk_norm_rope_cache_write: rows of {proj.shape[1]} columns, expected {qw} + {kw}"
                              + (f" + {num_heads}" if with_gate else ""))
        if q_gamma.shape[0] != qw or k_gamma.shape[0] != kw:
            raise KernelError("qk_norm_rope_cache_write: the norm weights do not have the widths of q and k")
        rot, table_rows = 0, 1
        if cos is not None:
            _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
            rot, table_rows = 2 * cos.shape[1], cos.shape[0]
            if not 0 < rot <= head_dim or sin.shape != cos.shape:
                raise KernelError(f"qk_norm_rope_cache_write: cos/sin tables must be [rows, rotary_dim/2] with rotary_dim <= {head_dim}")
        if write_kv:
            _need(cache_layer, "cache_layer", out_dtype, 5); _need(slot_mapping, "slot_mapping", torch.int32, 1)
            if tuple(cache_layer.shape[1:3]) != (2, num_kv_heads) or cache_layer.shape[4] != head_dim:
                raise KernelError(f"qk_norm_rope_cache_write: cache layer of shape {tuple(cache_layer.shape)} does not "
                                  f"fit {num_kv_heads} kv heads of {head_dim}")
        q = torch.empty((T, qw), dtype=out_dtype, device=proj.device)
        gate = torch.empty((T, num_heads), dtype=torch.float32, device=proj.device) if with_gate else None
        st = self._lib("rowops.cu").rv_qk_norm_rope_write(
            _ptr(proj), c_int(self._dt(proj, "proj")), c_int(proj.shape[1]), _ptr(q_gamma), _ptr(k_gamma),
            c_int(self._dt(q_gamma, "q_gamma")), _ptr(positions), _ptr(cos), _ptr(sin), c_int(rot), c_int(table_rows),
            _ptr(slot_mapping if write_kv else None), _ptr(cache_layer if write_kv else None), _ptr(q), c_int(_DT[out_dtype]),
            _ptr(gate), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
            c_int(cache_layer.shape[3] if write_kv else 1), c_float(eps), c_int(1 if write_kv else 0), self._stream())
        _check("qk_norm_rope_cache_write", st)
        return q, gate

    def causal_conv_silu(self, proj, col0: int, channels: int, weight, bias, token_seq, cu_seqlens, state_slots, state,
                         conv_off: int, out_dtype) -> torch.Tensor:
        """silu(causal convolution per channel) of columns col0 .. col0 + channels of `proj`, continued from and
        leaving behind each request's last taps - 1 inputs in `state` (float [slots, floats], at `conv_off`)."""
        _need(proj, "proj", dims=2); _need(weight, "weight", dims=2); _need(state, "state", torch.float32, 2)
        if weight.shape[0] != channels or (bias is not None and (bias.shape != (channels,) or bias.dtype != weight.dtype)):
            raise KernelError("causal_conv_silu: taps and bias do not fit the channels")
        T, taps = proj.shape[0], weight.shape[1]
        if conv_off + (taps - 1) * channels > state.shape[1]:
            raise KernelError("causal_conv_silu: the state rows are too short for the convolution's inputs")
        out = torch.empty((T, channels), dtype=out_dtype, device=proj.device)
        st = self._lib("ssm.cu").rv_causal_conv_silu(
            _ptr(proj), c_int(self._dt(proj, "proj")), c_int(proj.shape[1]), c_int(col0), _ptr(weight), _ptr(bias),
            c_int(self._dt(weight, "weight")), _ptr(token_seq), _ptr(cu_seqlens), _ptr(state_slots), _ptr(state),
            ctypes.c_longlong(state.shape[1]), ctypes.c_longlong(conv_off), _ptr(out), c_int(_DT[out_dtype]), c_int(T),
            c_int(state_slots.shape[0]), c_int(channels), c_int(taps), self._stream())
        _check("causal_conv_silu", st)
        COUNTERS['launches'] += 1 if taps > 1 else 0
        return out

    SCAN_SEGMENT_TOKENS = 256          # a sequence that brings more than twice as many tokens to a step is scanned in segments
    SCAN_SEGMENT_SCRATCH = 1 << 30     # ... of this many tokens side by side, while the segments' states fit these bytes of scratch
    SCAN_SEGMENT_ALWAYS = False        # ... and only where the one-pass walk would have fewer CTAs than the device has SMs (measured:
                                       # 128 CTAs, 64 heads of 64: the step's prefill 6.4 -> 5.5 ms; 256 CTAs, 128 heads: scan + carry +
                                       # correction 0.59 + 0.16 + 0.38 ms against 0.92 ms in one pass)

    def ssm_scan(self, xbc, proj, dt_col0: int, dt_bias, a_log, d_skip, cu_seqlens, state_slots, state, heads: int,
                 head_dim: int, state_size: int, groups: int, columns: int = 0, max_q_len: Optional[int] = None,
                 segment_tokens: Optional[int] = None) -> torch.Tensor:
        """The selective-state recurrence over the step's tokens, continued from and leaving behind each request's
        S in `state` (float [slots, floats], [heads][N][P] at offset 0).  xbc rows: [x | B | C]; raw dt is read
        from columns dt_col0 .. of `proj`.  Returns y float32 [T, heads * head_dim].  `columns`: columns of the
        state per thread (1 or 2); 0 lets the launcher choose by the size of the grid.  `max_q_len`: the most tokens any
        sequence brings (known on the host); long portions are then cut into segments of `segment_tokens` (default
        `SCAN_SEGMENT_TOKENS`) that are scanned side by side and joined by two small kernels."""
        _need(xbc, "xbc", dims=2); _need(proj, "proj", dims=2); _need(state, "state", torch.float32, 2)
        for name, p in (("dt_bias", dt_bias), ("a_log", a_log), ("d_skip", d_skip)):
            _need(p, name, dt_bias.dtype, 1)
            if p.shape[0] != heads:
                raise KernelError(f"ssm_scan: {name} has {p.shape[0]} entries for {heads} heads")
        if state.shape[1] < heads * state_size * head_dim:
            raise KernelError("ssm_scan: the state rows are too short")
        y = torch.empty((xbc.shape[0], heads * head_dim), dtype=torch.float32, device=xbc.device)
        seg = self.SCAN_SEGMENT_TOKENS if segment_tokens is None else segment_tokens
        n_seqs, max_segs, seg_state, seg_decay, dcum = state_slots.shape[0], 1, None, None, None
        few_ctas = self.SCAN_SEGMENT_ALWAYS or segment_tokens is not None or -(-head_dim // 32) * heads * n_seqs < self.num_sms
        if seg and few_ctas and max_q_len is not None and max_q_len > 2 * seg:
            max_segs = -(-max_q_len // seg)
            if n_seqs * max_segs * heads * state_size * head_dim * 4 <= self.SCAN_SEGMENT_SCRATCH and n_seqs * max_segs <= 65535:
                seg_state = torch.empty((n_seqs * max_segs, heads, state_size, head_dim), dtype=torch.float32, device=xbc.device)
                seg_decay = torch.empty((n_seqs * max_segs, heads), dtype=torch.float32, device=xbc.device)
                dcum = torch.empty((xbc.shape[0], heads), dtype=torch.float32, device=xbc.device)
            else:
                max_segs = 1
        if seg_state is None:
            seg = 0
        st = self._lib("ssm.cu").rv_ssm_scan(
            _ptr(xbc), c_int(self._dt(xbc, "xbc")), c_int(xbc.shape[1]), _ptr(proj), c_int(self._dt(proj, "proj")),
            c_int(proj.shape[1]), c_int(dt_col0), _ptr(dt_bias), _ptr(a_log), _ptr(d_skip), c_int(self._dt(dt_bias, "dt_bias")),
            _ptr(cu_seqlens), _ptr(state_slots), _ptr(state), ctypes.c_longlong(state.shape[1]), _ptr(y),
            c_int(state_slots.shape[0]), c_int(heads), c_int(head_dim), c_int(state_size), c_int(groups), c_int(columns),
            c_int(seg), c_int(max_segs), _ptr(seg_state), _ptr(seg_decay), _ptr(dcum), self._stream())
        _check("ssm_scan", st)
        COUNTERS['launches'] += 2 if seg else 0
        return y

    def gated_group_rmsnorm(self, y, proj, gamma, eps: float, parts: int, out_dtype) -> torch.Tensor:
        """(y * silu(z)) RMS-normalised in `parts` equal parts of a row, times gamma; z = the leading columns of `proj`."""
        _need(y, "y", torch.float32, 2); _need(proj, "proj", dims=2); _need(gamma, "gamma", dims=1)
        rows, width = y.shape
        if gamma.shape[0] != width or proj.shape[0] != rows or proj.shape[1] < width or width % parts:
            raise KernelError("gated_group_rmsnorm: shapes of y, z, gamma and the parts do not agree")
        out = torch.empty((rows, width), dtype=out_dtype, device=y.device)
        st = self._lib("rowops.cu").rv_gated_group_rmsnorm(
            _ptr(y), _ptr(proj), c_int(self._dt(proj, "proj")), c_int(proj.shape[1]), _ptr(gamma), c_int(self._dt(gamma, "gamma")),
            _ptr(out), c_int(_DT[out_dtype]), c_int(rows), c_int(width), c_int(parts), c_float(eps), self._stream())
        _check("gated_group_rmsnorm", st)
        return out


    # ------------------------------------------------------------------ stream additions, PolyNorm, capped logits
    def stream_add(self, x, emb: Optional[torch.Tensor], table: torch.Tensor, index: int) -> torch.Tensor:
        """x += (emb) + table[index] on the float32 stream, in place; returns x."""
        _need(x, "x", torch.float32, 2); _need(table, "table", dims=2)
        if table.shape[1] != x.shape[1] or not 0 <= index < table.shape[0]:
            raise KernelError(f"stream_add: row {index} of a table {tuple(table.shape)} for rows of {x.shape[1]}")
        if emb is not None:
            _need(emb, "emb", torch.float32, 2)
            if emb.shape != x.shape:
                raise KernelError(f"stream_add: {tuple(emb.shape)} added to {tuple(x.shape)}")
        row = table[index]
        st = self._lib("rowops.cu").rv_stream_add(_ptr(x), _ptr(emb), _ptr(row), c_int(self._dt(row, "table")), c_int(x.shape[0]),
                                                  c_int(x.shape[1]), self._stream())
        _check("stream_add", st)
        return x

    def polynorm(self, z, coef: torch.Tensor, eps: float, out_dtype=None) -> torch.Tensor:
        """a n(z) + b n(z^2) + c n(z^3) + e per row, n(v) = v / sqrt(mean(v^2) + eps); coef = float (a, b, c, e)."""
        _need(z, "z", dims=2); _need(coef, "coef", torch.float32, 1)
        if coef.shape[0] != 4:
            raise KernelError(f"polynorm: four coefficients, got {coef.shape[0]}")
        out = torch.empty(z.shape, dtype=out_dtype or z.dtype, device=z.device)
        st = self._lib("rowops.cu").rv_polynorm(_ptr(z), c_int(self._dt(z, "z")), _ptr(coef), _ptr(out), c_int(self._dt(out, "out")),
                                                c_int(z.shape[0]), c_int(z.shape[1]), c_float(eps), self._stream())
        _check("polynorm", st)
        return out

    def softcap(self, logits: torch.Tensor, cap: float) -> torch.Tensor:
        """logits <- cap * tanh(logits / cap), float32, in place; returns logits."""
        _need(logits, "logits", torch.float32)
        st = self._lib("rowops.cu").rv_softcap(_ptr(logits), c_float(cap), ctypes.c_longlong(logits.numel()), self._stream())
        _check("softcap", st)
        return logits

    # ------------------------------------------------------------------ float32 stream of pre-norm layers, small steps around mixers
    def scale_add_sinusoid(self, x, positions, frequencies, scale: float) -> torch.Tensor:
        """x * scale + pe(position), pe[2i] = sin(p w_i), pe[2i + 1] = cos(p w_i); `frequencies`: float64 w_i.  Float32 result."""
        _need(x, "x", dims=2); _need(positions, "positions", torch.int32, 1); _need(frequencies, "frequencies", torch.float64, 1)
        rows, cols = x.shape
        if positions.shape[0] != rows or frequencies.shape[0] != (cols + 1) // 2:
            raise KernelError(f"scale_add_sinusoid: {positions.shape[0]} positions and {frequencies.shape[0]} frequencies for {tuple(x.shape)}")
        out = torch.empty((rows, cols), dtype=torch.float32, device=x.device)
        st = self._lib("streamops.cu").rv_scale_add_sinusoid(_ptr(x), c_int(self._dt(x, "x")), _ptr(positions), _ptr(frequencies),
                                                            c_float(scale), _ptr(out), c_int(rows), c_int(cols), self._stream())
        _check("scale_add_sinusoid", st)
        return out

    def stream_add_norm(self, x, y: Optional[torch.Tensor], norm, out_dtype):
        """x += y on the float32 stream, in place (y None: nothing is added).  Returns (x, second result): None without
        `out_dtype`; the new x in `out_dtype`; or, with norm = (gamma, eps), the new x / sqrt(mean(x^2) + eps) * gamma."""
        _need(x, "x", torch.float32, 2)
        rows, cols = x.shape
        if y is not None:
            _need(y, "y", torch.float32, 2)
            if y.shape != x.shape:
                raise KernelError(f"stream_add_norm: {tuple(y.shape)} added to {tuple(x.shape)}")
        if out_dtype is None and y is None:
            return x, None
        gamma, eps = (norm if norm is not None else (None, 0.0))
        if gamma is not None:
            _need(gamma, "gamma", dims=1)
            if gamma.shape[0] != cols:
                raise KernelError(f"stream_add_norm: gamma has {gamma.shape[0]} entries for rows of {cols}")
        rounded = torch.empty((rows, cols), dtype=out_dtype, device=x.device) if out_dtype is not None else None
        st = self._lib("streamops.cu").rv_stream_add_norm(
            _ptr(x), _ptr(y), _ptr(gamma), c_int(self._dt(gamma, "gamma") if gamma is not None else 0), _ptr(rounded),
            c_int(_DT[out_dtype] if rounded is not None else 0), c_int(rows), c_int(cols), c_float(eps), self._stream())
        _check("stream_add_norm", st)
        return x, rounded

    def gelu_mul_columns(self, g, table_rows, col0: int, out_dtype) -> torch.Tensor:
        """gelu_tanh(g[t, c]) * table_rows[t, col0 + c]."""
        _need(g, "g", dims=2); _need(table_rows, "table_rows", dims=2)
        rows, cols = g.shape
        if table_rows.shape[0] != rows or col0 < 0 or col0 + cols > table_rows.shape[1]:
            raise KernelError(f"gelu_mul_columns: columns {col0}..{col0 + cols} of rows {tuple(table_rows.shape)} for {tuple(g.shape)}")
        out = torch.empty((rows, cols), dtype=out_dtype, device=g.device)
        st = self._lib("streamops.cu").rv_gelu_mul_columns(_ptr(g), c_int(self._dt(g, "g")), _ptr(table_rows),
                                                          c_int(self._dt(table_rows, "table_rows")), c_int(table_rows.shape[1]), c_int(col0),
                                                          _ptr(out), c_int(_DT[out_dtype]), c_int(rows), c_int(cols), self._stream())
        _check("gelu_mul_columns", st)
        return out

    def column_slice(self, x, col0: int, n: int, out_dtype) -> torch.Tensor:
        """A contiguous copy of columns col0 .. col0 + n of x, in `out_dtype`."""
        _need(x, "x", dims=2)
        if col0 < 0 or n <= 0 or col0 + n > x.shape[1]:
            raise KernelError(f"column_slice: columns {col0}..{col0 + n} of rows of {x.shape[1]}")
        out = torch.empty((x.shape[0], n), dtype=out_dtype, device=x.device)
        st = self._lib("streamops.cu").rv_column_slice(_ptr(x), c_int(self._dt(x, "x")), c_int(x.shape[1]), c_int(col0), _ptr(out),
                                                      c_int(_DT[out_dtype]), c_int(x.shape[0]), c_int(n), self._stream())
        _check("column_slice", st)
        return out

    def scaled_sum(self, a: Optional[torch.Tensor], sa: float, b, sb: float) -> torch.Tensor:
        """a <- sa * a + sb * b in place (float32); a None: a new tensor sb * b."""
        _need(b, "b", torch.float32)
        if a is not None:
            _need(a, "a", torch.float32)
            if a.shape != b.shape:
                raise KernelError(f"scaled_sum: {tuple(a.shape)} and {tuple(b.shape)}")
        out = a if a is not None else torch.empty_like(b)
        st = self._lib("streamops.cu").rv_scaled_sum(_ptr(a), c_float(sa), _ptr(b), c_float(sb), _ptr(out), ctypes.c_longlong(b.numel()),
                                                    self._stream())
        _check("scaled_sum", st)
        return out

    def head_norm_gate(self, o, gamma, eps: float, proj, g_col0: int, heads: int, value_dim: int, out_dtype) -> torch.Tensor:
        """Per head: o / sqrt(mean(o^2) + eps) * gamma * silu(z); gamma [value_dim] is shared by the heads, z = columns
        g_col0 .. g_col0 + heads * value_dim of `proj`."""
        _need(o, "o", torch.float32, 2); _need(gamma, "gamma", dims=1); _need(proj, "proj", dims=2)
        rows = o.shape[0]
        if o.shape[1] != heads * value_dim or gamma.shape[0] != value_dim or proj.shape[0] != rows or g_col0 + heads * value_dim > proj.shape[1]:
            raise KernelError("head_norm_gate: shapes of o, gamma and the gate do not agree")
        out = torch.empty((rows, heads * value_dim), dtype=out_dtype, device=o.device)
        st = self._lib("streamops.cu").rv_head_norm_gate(_ptr(o), _ptr(gamma), c_int(self._dt(gamma, "gamma")), _ptr(proj),
                                                        c_int(self._dt(proj, "proj")), c_int(proj.shape[1]), c_int(g_col0), _ptr(out),
                                                        c_int(_DT[out_dtype]), c_int(rows), c_int(heads), c_int(value_dim), c_float(eps),
                                                        self._stream())
        _check("head_norm_gate", st)
        return out

    # ------------------------------------------------------------------ recurrences with one state row per channel / per head
    def selective_scan(self, u, dt_raw, dt_bias, a, bc, b_col0: int, c_col0: int, d_skip, z, z_col0: int, cu_seqlens, state_slots,
                       state, out_dtype) -> torch.Tensor:
        """S[c, n] <- exp(dt_c a[c, n]) S[c, n] + dt_c u_c B_n; y_c = sum_n S[c, n] C_n + D_c u_c; returns y * silu(z) in
        `out_dtype`.  dt = softplus(dt_raw + dt_bias) per channel; B and C are float columns b_col0 .. and c_col0 .. of `bc`,
        z columns z_col0 .. of `z`; S lives as [inner][N] at offset 0 of the request's row of `state`."""
        _need(u, "u", dims=2); _need(dt_raw, "dt_raw", torch.float32, 2); _need(bc, "bc", torch.float32, 2); _need(z, "z", dims=2)
        _need(a, "a", torch.float32, 2); _need(state, "state", torch.float32, 2)
        T, inner = u.shape
        N = a.shape[1]
        for name, p in (("dt_bias", dt_bias), ("d_skip", d_skip)):
            _need(p, name, torch.float32, 1)
            if p.shape[0] != inner:
                raise KernelError(f"selective_scan: {name} has {p.shape[0]} entries for {inner} channels")
        if a.shape[0] != inner or dt_raw.shape != (T, inner) or bc.shape[0] != T or z.shape[0] != T:
            raise KernelError("selective_scan: shapes of u, dt, a, B | C and z do not agree")
        out = torch.empty((T, inner), dtype=out_dtype, device=u.device)
        st = self._lib("ssm.cu").rv_selective_scan1(
            _ptr(u), c_int(self._dt(u, "u")), _ptr(dt_raw), _ptr(dt_bias), _ptr(a), _ptr(bc), c_int(bc.shape[1]), c_int(b_col0),
            c_int(c_col0), _ptr(d_skip), _ptr(z), c_int(self._dt(z, "z")), c_int(z.shape[1]), c_int(z_col0), _ptr(cu_seqlens),
            _ptr(state_slots), _ptr(state), ctypes.c_longlong(state.shape[1]), _ptr(out), c_int(_DT[out_dtype]),
            c_int(state_slots.shape[0]), c_int(inner), c_int(N), self._stream())
        _check("selective_scan", st)
        return out

    def delta_rule(self, qkv, proj, b_col0: int, a_col0: int, a_log, dt_bias, cu_seqlens, state_slots, state, heads: int,
                   qk_heads: int, head_dim: int, value_dim: int, unit_eps: float) -> torch.Tensor:
        """The gated delta rule over the step's tokens, continued from and leaving behind each request's S ([heads][head_dim]
        [value_dim] at offset 0 of its row of `state`).  qkv rows: [q | k | v] after their convolution; the logits of beta and
        of the decay are float columns b_col0 .. and a_col0 .. of `proj`.  Returns o float32 [T, heads * value_dim]."""
        _need(qkv, "qkv", dims=2); _need(proj, "proj", torch.float32, 2); _need(state, "state", torch.float32, 2)
        _need(a_log, "a_log", torch.float32, 1); _need(dt_bias, "dt_bias", torch.float32, 1)
        T = qkv.shape[0]
        if qkv.shape[1] != 2 * qk_heads * head_dim + heads * value_dim or proj.shape[0] != T or a_log.shape[0] != heads or \
                dt_bias.shape[0] != heads:
            raise KernelError("delta_rule: shapes of q | k | v, the logits and the heads' constants do not agree")
        out = torch.empty((T, heads * value_dim), dtype=torch.float32, device=qkv.device)
        st = self._lib("ssm.cu").rv_delta_rule(
            _ptr(qkv), c_int(self._dt(qkv, "qkv")), c_int(qkv.shape[1]), _ptr(proj), c_int(proj.shape[1]), c_int(b_col0), c_int(a_col0),
            _ptr(a_log), _ptr(dt_bias), _ptr(cu_seqlens), _ptr(state_slots), _ptr(state), ctypes.c_longlong(state.shape[1]), _ptr(out),
            c_int(state_slots.shape[0]), c_int(heads), c_int(qk_heads), c_int(head_dim), c_int(value_dim), c_float(unit_eps),
            self._stream())
        _check("delta_rule", st)
        return out

    # ------------------------------------------------------------------ attention whose weights are mixed across the heads
    @staticmethod
    def _flat_page_size(cache_layer, num_kv_heads: int, head_dim: int, value_dim: int) -> int:
        per_page = cache_layer.numel() // cache_layer.shape[0]
        ps, rest = divmod(per_page, num_kv_heads * (head_dim + value_dim))
        if rest or ps <= 0:
            raise KernelError(f"a cache layer of shape {tuple(cache_layer.shape)} does not hold pages of {num_kv_heads} kv heads "
                              f"with keys of {head_dim} and values of {value_dim}")
        return ps

    def kv_prepare(self, proj, slot_mapping, cache_layer, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                   value_norm_eps: Optional[float], out_dtype, write_kv: bool = True) -> torch.Tensor:
        """proj rows [q | k | v]: returns q in `out_dtype`; k and v go into the token's cache slot, v first divided by its
        root mean square per head when `value_norm_eps` is given.  A page holds its key rows [kv heads][page][head_dim]
        and behind them its value rows [kv heads][page][value_dim]."""
        _need(proj, "proj", dims=2)
        T = proj.shape[0]
        qw = num_heads * head_dim
        if proj.shape[1] != qw + num_kv_heads * (head_dim + value_dim):
            raise KernelError(f"kv_prepare: rows of {proj.shape[1]} columns, expected {qw} + {num_kv_heads} x ({head_dim} + {value_dim})")
        ps = 1
        if write_kv:
            _need(cache_layer, "cache_layer"); _need(slot_mapping, "slot_mapping", torch.int32, 1)
            ps = self._flat_page_size(cache_layer, num_kv_heads, head_dim, value_dim)
        q = torch.empty((T, qw), dtype=out_dtype, device=proj.device)
        st = self._lib("talking_attention.cu").rv_kv_prepare(
            _ptr(proj), c_int(self._dt(proj, "proj")), c_int(proj.shape[1]), _ptr(slot_mapping if write_kv else None),
            _ptr(cache_layer if write_kv else None), c_int(self._dt(cache_layer, "cache_layer") if write_kv else 0), _ptr(q),
            c_int(_DT[out_dtype]), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(value_dim), c_int(ps),
            c_float(value_norm_eps if value_norm_eps is not None else 0.0), c_int(1 if value_norm_eps is not None else 0),
            c_int(1 if write_kv else 0), self._stream())
        _check("kv_prepare", st)
        return q

    def talking_attention(self, q, cache_layer, meta: AttentionMeta, positions, num_heads: int, num_kv_heads: int, head_dim: int,
                          value_dim: int, scale: float, r1, r2, talk, chunk: Optional[int]) -> torch.Tensor:
        """softmax attention over the paged cache whose weights are mixed across the heads (`talk` [heads, heads], float32)
        before they meet the values; r1, r2 (float32 per head): r1 ln(1 + r2 distance) is taken off the scores; `chunk`: a
        query sees the keys of its own block of that many positions only.  q, cache and result share one type."""
        _need(q, "q", dims=2); _need(cache_layer, "cache_layer", q.dtype)
        T = q.shape[0]
        if q.shape[1] != num_heads * head_dim:
            raise KernelError(f"talking_attention: q rows of {q.shape[1]} for {num_heads} heads of {head_dim}")
        ps = self._flat_page_size(cache_layer, num_kv_heads, head_dim, value_dim)
        if ps != meta.page_size:
            raise KernelError(f"talking_attention: the cache's pages hold {ps} tokens, the step's tables count {meta.page_size}")
        for name, p, n in (("r1", r1, num_heads), ("r2", r2, num_heads), ("talk", talk, num_heads * num_heads)):
            if p is not None:
                _need(p, name, torch.float32)
                if p.numel() != n:
                    raise KernelError(f"talking_attention: {name} has {p.numel()} entries, expected {n}")
        out = torch.empty((T, num_heads * value_dim), dtype=q.dtype, device=q.device)
        visible = min(meta.max_ctx_len, chunk) if chunk else meta.max_ctx_len
        if self.TALKING_SPLIT and 0 < T and (T <= self.TALKING_SPLIT_MAX_TOKENS or meta.max_q_len == 1) \
                and visible > self.TALKING_SPLIT_SPAN and num_heads * head_dim * 4 <= 48 * 1024 \
                and T * num_heads * (visible + 64) * 4 <= self.TALKING_SPLIT_MAX_SCRATCH:
            # few tokens behind many keys (or single tokens only): the keys of a token are cut over CTAs, into as many
            # ranges as give the GPU about two CTAs an SM (at most 64), each a multiple of TALKING_SPLIT_SPAN keys
            unit = self.TALKING_SPLIT_SPAN
            ranges = min(64, max(1, -(-2 * self.num_sms // T)))
            span = unit * -(-visible // (unit * ranges))
            nsplit = (visible + span - 1) // span
            lib = self._lib("talking_attention.cu")
            lib.rv_talking_attention_split_floats.restype = ctypes.c_longlong
            n = lib.rv_talking_attention_split_floats(c_int(T), c_int(num_heads), c_int(value_dim), c_int(span), c_int(nsplit))
            scratch = torch.empty((n,), dtype=torch.float32, device=q.device)
            st = lib.rv_talking_attention_split(
                _ptr(q), _ptr(cache_layer), _ptr(meta.block_tables), _ptr(meta.cu_seqlens), _ptr(meta.ctx_lens), _ptr(meta.token_seq),
                _ptr(out), _ptr(scratch), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(value_dim), c_int(ps),
                c_int(meta.max_blocks), c_float(scale), _ptr(r1), _ptr(r2), _ptr(talk), c_int(chunk or 0), c_int(span), c_int(nsplit),
                c_int(self._dt(q, "q")), self._stream())
            _check("talking_attention_split", st)
            return out
        if self.TALKING_MMA and q.dtype == torch.bfloat16 and T > 0:
            lib = self._lib("talking_attention_mma.cu")
            if lib.rv_talking_attention_mma_fits(c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(value_dim)):
                st = lib.rv_talking_attention_mma(
                    _ptr(q), _ptr(cache_layer), _ptr(meta.block_tables), _ptr(meta.cu_seqlens), _ptr(meta.ctx_lens), _ptr(out),
                    c_int(meta.num_seqs), c_int(meta.max_q_len), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(value_dim),
                    c_int(ps), c_int(meta.max_blocks), c_float(scale), _ptr(r1), _ptr(r2), _ptr(talk), c_int(chunk or 0), self._stream())
                if st != -4:            # (-4: the tiles of these sizes do not fit the shared memory; the plain kernel takes them)
                    _check("talking_attention_mma", st)
                    return out
        st = self._lib("talking_attention.cu").rv_talking_attention(
            _ptr(q), _ptr(cache_layer), _ptr(meta.block_tables), _ptr(meta.cu_seqlens), _ptr(meta.ctx_lens), _ptr(meta.token_seq),
            _ptr(out), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(value_dim), c_int(ps),
            c_int(meta.max_blocks), c_float(scale), _ptr(r1), _ptr(r2), _ptr(talk), c_int(chunk or 0), c_int(self._dt(q, "q")),
            self._stream())
        _check("talking_attention", st)
        return out

    # ------------------------------------------------------------------ latent attention
    def latent_prepare(self, proj, c_gamma, eps: float, positions, cos, sin, slot_mapping, cache_layer, num_heads: int,
                       head_dim: int, rot_dim: int, kv_rank: int, out_dtype, with_gate: bool = True, write_kv: bool = True,
                       halves: bool = False):
        """proj rows [q: heads x (head_dim + rot_dim) | c': kv_rank | r: rot_dim | gate logits: heads].  c' is RMS-normalised
        (weight `c_gamma`), the leading 2 * cos.shape[1] elements of r and of every head's rotated query part are turned in
        pairs (2i, 2i + 1) - with `halves`: (i, i + cos.shape[1]) -, [c | r] is written into the token's cache row.  Returns (q_plain [T, heads, head_dim],
        q_row [T, heads, kv_rank + rot_dim] with its last rot_dim columns filled, sigmoid(gate logits) float [T, heads] or None)."""
        _need(proj, "proj", dims=2); _need(positions, "positions", torch.int32, 1); _need(c_gamma, "c_gamma", dims=1)
        T, row = proj.shape[0], kv_rank + rot_dim
        if proj.shape[1] != num_heads * (head_dim + rot_dim) + row + (num_heads if with_gate else 0) or c_gamma.shape[0] != kv_rank:
            raise KernelError(f"latent_prepare: rows of {proj.shape[1]} columns do not fit {num_heads} heads of {head_dim} + {rot_dim}, "
                              f"a latent of {kv_rank} + {rot_dim}" + (f" and {num_heads} gates" if with_gate else ""))
        rot, table_rows = 0, 1
        if cos is not None:
            _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
            rot, table_rows = 2 * cos.shape[1], cos.shape[0]
            if not 0 < rot <= rot_dim or sin.shape != cos.shape:
                raise KernelError(f"latent_prepare: cos/sin tables must be [rows, dims/2] with dims <= {rot_dim}")
        if write_kv:
            _need(cache_layer, "cache_layer", out_dtype, 5); _need(slot_mapping, "slot_mapping", torch.int32, 1)
            if tuple(cache_layer.shape[1:3]) != (1, 1) or cache_layer.shape[4] != row:
                raise KernelError(f"latent_prepare: cache layer of shape {tuple(cache_layer.shape)} does not hold one row of {row} per token")
        q_plain = torch.empty((T, num_heads, head_dim), dtype=out_dtype, device=proj.device)
        q_row = torch.empty((T, num_heads, row), dtype=out_dtype, device=proj.device)
        gate = torch.empty((T, num_heads), dtype=torch.float32, device=proj.device) if with_gate else None
        st = self._lib("latent.cu").rv_latent_prepare(
            _ptr(proj), c_int(self._dt(proj, "proj")), c_int(proj.shape[1]), _ptr(c_gamma), c_int(self._dt(c_gamma, "c_gamma")),
            _ptr(positions), _ptr(cos), _ptr(sin), c_int(rot), c_int(table_rows), _ptr(slot_mapping if write_kv else None),
            _ptr(cache_layer if write_kv else None), _ptr(q_plain), _ptr(q_row), c_int(_DT[out_dtype]), _ptr(gate), c_int(T),
            c_int(num_heads), c_int(head_dim), c_int(rot_dim), c_int(kv_rank), c_float(eps), c_int(1 if write_kv else 0),
            c_int(1 if halves else 0), self._stream())
        _check("latent_prepare", st)
        return q_plain, q_row, gate

    def head_linear(self, x, weight, out: Optional[torch.Tensor] = None, out_dtype=None) -> torch.Tensor:
        """out[t, h, :] = weight[h] x[t, h, :] for x [T, heads, K], weight [heads, N, K]; float accumulation.  x and out may be
        slices of wider rows (their last dimension contiguous); without `out` a new [T, heads, N] tensor is returned."""
        _need(weight, "weight", dims=3)
        H, N, K = weight.shape
        if x.dim() != 3 or x.shape[1] != H or x.shape[2] != K or x.stride(2) != 1 or not x.is_cuda:
            raise KernelError(f"head_linear: x of shape {tuple(x.shape)} and strides {x.stride()} for weights {tuple(weight.shape)}")
        T = x.shape[0]
        if out is None:
            out = torch.empty((T, H, N), dtype=out_dtype or x.dtype, device=x.device)
        if tuple(out.shape) != (T, H, N) or out.stride(2) != 1:
            raise KernelError(f"head_linear: out of shape {tuple(out.shape)} and strides {out.stride()}, expected {(T, H, N)}")
        if self._head_linear_tcgen05(x, weight, out):
            return out
        st = self._lib("latent.cu").rv_head_linear(
            _ptr(x), c_int(self._dt(x, "x")), ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(x.stride(1)), _ptr(weight),
            c_int(self._dt(weight, "weight")), _ptr(out), c_int(self._dt(out, "out")), ctypes.c_longlong(out.stride(0)),
            ctypes.c_longlong(out.stride(1)), c_int(T), c_int(H), c_int(N), c_int(K), self._stream())
        _check("head_linear", st)
        return out

    HEAD_LINEAR_TCGEN05_MIN_ROWS = 128      # rows from which the per-head products run on the tcgen05 GEMM (batched over the heads)

    def _head_work(self, lib, T: int, H: int, N: int):
        """The work units of a per-head product of T rows on the device (made once per shape): every head's blocks of 128
        rows in pairs (the CTAs of a tile), and the order head by head, column tile by column tile, the head's units."""
        key = (T, H, N)
        cache = self.__dict__.setdefault("_head_work_cache", {})
        if key not in cache:
            if len(cache) > 64:
                cache.clear()
            R, ranks = int(lib.rv_gemm_tcgen05_block_rows()), int(lib.rv_gemm_tcgen05_ranks())
            nt = int(lib.rv_gemm_tcgen05_column_tiles(c_int(N), c_int(0)))
            blocks = -(-T // R)
            per_head = -(-blocks // ranks)
            group, rows, order = [], [], []
            for h in range(H):
                for u in range(per_head):
                    group.append(h)
                    rows.extend((u * ranks + r) * R if u * ranks + r < blocks else -1 for r in range(ranks))
                order.extend(((h * per_head + u) << 16) | t for t in range(nt) for u in range(per_head))
            as_dev = lambda v: torch.tensor(v, dtype=torch.int32).to(self.device)
            cache[key] = (as_dev(group), as_dev(rows), as_dev(order), H * per_head)
        return cache[key]

    def _head_linear_tcgen05(self, x, weight, out) -> bool:
        """`head_linear` on the tcgen05 GEMM where the operands allow: bfloat16, many rows, rows and head slices of x on
        16-byte boundaries.  A head is a group of the grouped product: its K elements are columns of x, its results
        columns of out.  False: not taken."""
        H, N, K = weight.shape
        T = x.shape[0]
        if not (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
                and T >= self.HEAD_LINEAR_TCGEN05_MIN_ROWS and K % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) % 8 == 0
                and x.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0 and x.stride(1) >= K and x.stride(0) >= (H - 1) * x.stride(1) + K
                and out.stride(0) >= (H - 1) * out.stride(1) + N and out.stride(1) >= N and H * (-(-T // 128)) <= 32767
                and not torch.cuda.is_current_stream_capturing()):
            return False
        lib = self._lib("gemm_tcgen05.cu", ("-DRV_PAIR=1",))
        group, rows, order, units = self._head_work(lib, T, H, N)
        st = lib.rv_gemm_tcgen05_batched(
            _ptr(x), _ptr(weight), _ptr(group), _ptr(rows), _ptr(order), _ptr(out), c_int(1 if out.dtype == torch.float32 else 0),
            c_int(T), c_int(N), c_int(K), c_int(H), c_int(units), c_int(x.stride(0)), c_int(x.stride(1)), c_int(out.stride(1)),
            c_int(out.stride(0)), _ptr(self._status), self._stream())
        _check("gemm_tcgen05_batched", st)
        return True

    def latent_attention(self, q_row, cache_layer, meta: AttentionMeta, num_heads: int, row: int, value_dim: int, scale: float,
                         gate: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Attention of the step's tokens over cached rows that are key and value at once: every head's query
        [T, heads, row] meets the whole row of a token, the weighted sum is taken over the rows' leading `value_dim`
        elements.  Causal, softmax in float; `gate` (float [T, heads]) multiplies each head's result; `sinks` (float [heads]):
        exp(sink) joins each head's softmax denominator.  Returns [T, heads, value_dim] in q's type."""
        _need(q_row, "q_row", dims=3); _need(cache_layer, "cache_layer", q_row.dtype, 5)
        T = q_row.shape[0]
        if q_row.shape[1] != num_heads or q_row.shape[2] != row or tuple(cache_layer.shape[1:3]) != (1, 1) or cache_layer.shape[4] != row:
            raise KernelError(f"latent_attention: queries {tuple(q_row.shape)} and cache {tuple(cache_layer.shape)} do not fit "
                              f"{num_heads} heads on rows of {row}")
        if not 0 < value_dim <= row:
            raise KernelError(f"latent_attention: a value of {value_dim} out of a row of {row}")
        self._check_attention_extras(q_row.view(T, -1), num_heads, sinks, gate)
        out = torch.empty((T, num_heads, value_dim), dtype=q_row.dtype, device=q_row.device)
        page = cache_layer.shape[3]
        flash_ok = (self.LATENT_FLASH and q_row.dtype == torch.bfloat16 and row % 16 == 0 and value_dim % 16 == 0 and row <= 256
                    and not (page & (page - 1)))
        if (self.LATENT_TCGEN05 and self.TCGEN05_ATTENTION and q_row.dtype == torch.bfloat16 and row % 8 == 0 and 32 <= row <= 256
                and value_dim % 32 == 0 and num_heads <= 128 and page >= 8 and not (page & (page - 1))
                and meta.max_q_len >= self.TCGEN05_ATTENTION_MIN_TOKENS and (flash_ok or meta.num_decode == 0)):
            # prompt portions on the tcgen05 kernel (all heads of a token side by side in a tile of 128 rows); the step's
            # one-token sequences, which it leaves alone, on the decode tiling of the mma.sync kernel
            self.attention_tcgen05(q_row, cache_layer, meta, out, num_heads, 1, row, scale, None, gate=gate, sinks=sinks, value_dim=value_dim)
            if meta.num_decode:
                self.flash_attention(q_row, cache_layer, meta, out, num_heads, 1, row, scale, None, mode=1, q_filter=1, max_q_len=1,
                                     gate=gate, sinks=sinks, value_dim=value_dim)
            return out
        if flash_ok:
            # the tensor-core kernel: all heads of a token are rows of one tile over the token's single "kv head"
            args = (q_row, cache_layer, meta, out, num_heads, 1, row, scale, None)
            if meta.max_q_len == 1:
                self.flash_attention(*args, mode=1, num_splits=self.decode_splits(meta, num_heads, 1), gate=gate, sinks=sinks, value_dim=value_dim)
            elif meta.num_decode == 0:
                self.flash_attention(*args, mode=0, gate=gate, sinks=sinks, value_dim=value_dim)
            else:
                self.flash_attention(*args, mode=0, q_filter=2, gate=gate, sinks=sinks, value_dim=value_dim)
                self.flash_attention(*args, mode=1, q_filter=1, max_q_len=1, gate=gate, sinks=sinks, value_dim=value_dim)
            return out
        st = self._lib("attention_ref.cu").rv_paged_attention_ref_ex(
            _ptr(q_row), _ptr(cache_layer), _ptr(meta.block_tables), _ptr(meta.cu_seqlens), _ptr(meta.ctx_lens),
            _ptr(meta.token_seq), _ptr(out), c_int(T), c_int(num_heads), c_int(1), c_int(row), c_int(cache_layer.shape[3]),
            c_int(meta.max_blocks), c_float(scale), c_int(0), c_float(0.0), _ptr(sinks), _ptr(gate), c_int(1), c_int(value_dim),
            c_int(self._dt(q_row, "q_row")), self._stream())
        _check("latent_attention", st)
        return out

    # ------------------------------------------------------------------ mixture of experts
    def moe_experts(self, x, chosen, gate_up, down, weight: float, add: Optional[torch.Tensor] = None, out_dtype=None,
                    weights: Optional[torch.Tensor] = None, activation: str = "silu") -> torch.Tensor:
        """out[t] = (add[t]) + weight * sum_k weights[t, k] down[e] a_e(x_t), e = chosen[t, k].
        activation "silu": gated experts, a_e(x) = silu(gate[e] x) * (up[e] x), gate_up [experts, 2 ff, width] (gate rows, then up
        rows); "relu2": plain experts, a_e(x) = relu(up[e] x)^2, `gate_up` is up [experts, ff, width].  down [experts, width, ff],
        chosen int32 [T, top], weights float32 [T, top] or None (all 1), add float32 [T, width] or None."""
        _need(x, "x", dims=2); _need(chosen, "chosen", torch.int32, 2)
        _need(gate_up, "gate_up", x.dtype, 3); _need(down, "down", x.dtype, 3)
        if activation not in ("silu", "relu2"):
            raise KernelError(f"moe_experts: activation {activation!r} is not known (silu, relu2)")
        gated = activation == "silu"
        T, width = x.shape
        E, ff2, _ = gate_up.shape
        ff, top = (ff2 // 2 if gated else ff2), chosen.shape[1]
        if weights is not None:
            _need(weights, "weights", torch.float32, 2)
            if weights.shape != chosen.shape:
                raise KernelError(f"moe_experts: weights {tuple(weights.shape)} against chosen {tuple(chosen.shape)}")
        if gate_up.shape[2] != width or tuple(down.shape) != (E, width, ff) or chosen.shape[0] != T or (gated and ff * 2 != ff2):
            raise KernelError(f"moe_experts: x {tuple(x.shape)}, gate_up {tuple(gate_up.shape)}, down {tuple(down.shape)}, "
                              f"chosen {tuple(chosen.shape)} do not fit together")
        if add is not None:
            _need(add, "add", torch.float32, 2)
            if add.shape != x.shape:
                raise KernelError(f"moe_experts: add {tuple(add.shape)} against x {tuple(x.shape)}")
        out_dtype = out_dtype or x.dtype
        if out_dtype not in (x.dtype, torch.float32):
            raise KernelError(f"moe_experts: result type {out_dtype} for operands of {x.dtype}")
        if x.dtype == torch.bfloat16 and T >= self.MOE_GROUPED_MIN_TOKENS and width % 8 == 0 and ff % 8 == 0 and E <= 4096:
            return self._moe_grouped(x, chosen, gate_up, down, weight, add, out_dtype, weights, gated)
        act = torch.empty((T * top, ff), dtype=x.dtype, device=x.device)
        out = torch.empty((T, width), dtype=out_dtype, device=x.device)
        st = self._lib("moe.cu").rv_moe_experts_ex(
            _ptr(x), _ptr(chosen), _ptr(weights), _ptr(gate_up), _ptr(down), _ptr(act), _ptr(add), _ptr(out),
            c_int(1 if out_dtype == torch.float32 else 0), c_int(T), c_int(top), c_int(E), c_int(ff), c_int(width), c_float(weight),
            c_int(1 if gated else 0), c_int(self._dt(x, "x")), self._stream())
        _check("moe_experts", st)
        COUNTERS['launches'] += 1
        return out

    MOE_GROUPED_MIN_TOKENS = 128      # tokens of a step from which the experts' products run grouped on the tcgen05 GEMM ...
    MOE_GROUPED_PAIRS = True          # ... on pairs of CTAs (cta_group::2): two blocks of 128 rows of one expert share every tile of its weights

    def _moe_grouped(self, x, chosen, gate_up, down, weight, add, out_dtype, weights=None, gated=True):
        """`moe_experts` for many bfloat16 tokens: the (token, slot) pairs sorted by expert, every expert's rows padded to
        whole blocks of 128, two grouped tcgen05 products over the sorted rows (gate/up with the SiLU epilogue - plain experts:
        up with the squared relu in its epilogue - then down with a float32 result), and the weighted sum per token.  Everything is decided on the device; the buffers are sized for the worst case (every
        expert's last block nearly empty)."""
        T, width = x.shape
        E, ff2, _ = gate_up.shape
        ff, top = (ff2 // 2 if gated else ff2), chosen.shape[1]
        epi = 2 if gated else 0
        lib = self._lib("gemm_tcgen05.cu", ("-DRV_PAIR=1",) if self.MOE_GROUPED_PAIRS else ())
        moe = self._lib("moe.cu")
        R, ranks = int(lib.rv_gemm_tcgen05_block_rows()), int(lib.rv_gemm_tcgen05_ranks())
        pairs = T * top
        max_blocks = (pairs + E * (R - 1)) // R         # every expert's last block of rows nearly empty
        units = max_blocks                               # (a unit holds at least one block)
        rows = max_blocks * R
        dev = x.device
        row_of = torch.empty((pairs,), dtype=torch.int32, device=dev)
        src_of = torch.empty((rows,), dtype=torch.int32, device=dev)
        tile_group = torch.empty((units,), dtype=torch.int32, device=dev)
        tile_rows = torch.empty((units * ranks,), dtype=torch.int32, device=dev)
        nt_a, nt_b = int(lib.rv_gemm_tcgen05_column_tiles(c_int(ff2), c_int(epi))), int(lib.rv_gemm_tcgen05_column_tiles(c_int(width), c_int(0)))
        order_a = torch.empty((units * nt_a,), dtype=torch.int32, device=dev)
        order_b = torch.empty((units * nt_b,), dtype=torch.int32, device=dev)
        _check("moe_route", moe.rv_moe_route(_ptr(chosen), c_int(pairs), c_int(top), c_int(E), c_int(R), c_int(rows), c_int(ranks),
                                             c_int(units), _ptr(row_of), _ptr(src_of), _ptr(tile_group), _ptr(tile_rows), c_int(nt_a),
                                             _ptr(order_a), c_int(nt_b), _ptr(order_b), self._stream()))
        xs = torch.empty((rows, width), dtype=torch.bfloat16, device=dev)
        _check("moe_gather", moe.rv_moe_gather(_ptr(x), _ptr(src_of), _ptr(xs), c_int(rows), c_int(width * 2), self._stream()))
        act = torch.empty((rows, ff), dtype=torch.bfloat16, device=dev)
        _check("gemm_tcgen05_grouped", lib.rv_gemm_tcgen05_grouped(
            _ptr(xs), _ptr(gate_up), _ptr(tile_group), _ptr(tile_rows), _ptr(order_a), _ptr(act), c_int(0), c_int(rows), c_int(ff2), c_int(width), c_int(E),
            c_int(units), c_int(2 if gated else 6), _ptr(self._status), self._stream()))      # (6: the plain epilogue with the squared relu)
        ys = torch.empty((rows, width), dtype=torch.float32, device=dev)
        _check("gemm_tcgen05_grouped", lib.rv_gemm_tcgen05_grouped(
            _ptr(act), _ptr(down), _ptr(tile_group), _ptr(tile_rows), _ptr(order_b), _ptr(ys), c_int(1), c_int(rows), c_int(width), c_int(ff), c_int(E),
            c_int(units), c_int(0), _ptr(self._status), self._stream()))
        out = torch.empty((T, width), dtype=out_dtype, device=dev)
        _check("moe_combine", moe.rv_moe_combine(_ptr(ys), _ptr(row_of), _ptr(add), _ptr(out), c_int(1 if out_dtype == torch.float32 else 0),
                                                 c_int(T), c_int(top), c_int(width), c_float(weight), _ptr(weights), self._stream()))
        return out

    def moe_route_top(self, scores, correction, experts: int, top: int, groups: int, keep: int, weight_eps: float,
                      shared_gate: bool = False):
        """A router's choice from its float32 logits [T, experts (+ 1)]: s = sigmoid(logits); the `top` experts with the largest
        s + correction among those of the `keep` best of `groups` equal groups of neighbouring experts (a group counts by the
        sum of its two largest corrected scores).  Returns (chosen int32 [T, top], weights float32 [T, top] = the chosen s over
        their sum + weight_eps, sigmoid of the last column float32 [T] with `shared_gate`, else None)."""
        _need(scores, "scores", torch.float32, 2); _need(correction, "correction", torch.float32, 1)
        T = scores.shape[0]
        if scores.shape[1] != experts + (1 if shared_gate else 0) or correction.shape[0] != experts:
            raise KernelError(f"moe_route_top: logits {tuple(scores.shape)} and {correction.shape[0]} corrections for {experts} experts")
        chosen = torch.empty((T, top), dtype=torch.int32, device=scores.device)
        weights = torch.empty((T, top), dtype=torch.float32, device=scores.device)
        gate = torch.empty((T,), dtype=torch.float32, device=scores.device) if shared_gate else None
        st = self._lib("moe.cu").rv_moe_route_top(
            _ptr(scores), c_int(scores.shape[1]), _ptr(correction), _ptr(chosen), _ptr(weights), _ptr(gate), c_int(T), c_int(experts),
            c_int(top), c_int(groups), c_int(keep), c_float(weight_eps), self._stream())
        _check("moe_route_top", st)
        return chosen, weights, gate

    # ------------------------------------------------------------------ Dynamic-Tanh norms and rows
    def dynamic_tanh(self, x, alpha, weight, bias, out_dtype=None) -> torch.Tensor:
        """tanh(alpha x) * weight + bias; alpha float32 [1] on the device, weight and bias float32 [cols]."""
        _need(x, "x", dims=2); _need(alpha, "alpha", torch.float32, 1)
        _need(weight, "weight", torch.float32, 1); _need(bias, "bias", torch.float32, 1)
        rows, cols = x.shape
        if weight.shape[0] != cols or bias.shape[0] != cols or alpha.shape[0] != 1:
            raise KernelError(f"dynamic_tanh: weight {tuple(weight.shape)}, bias {tuple(bias.shape)}, alpha {tuple(alpha.shape)} for rows of {cols}")
        out = torch.empty((rows, cols), dtype=out_dtype or x.dtype, device=x.device)
        st = self._lib("streamops.cu").rv_dynamic_tanh(_ptr(x), c_int(self._dt(x, "x")), _ptr(alpha), _ptr(weight), _ptr(bias), _ptr(out),
                                                       c_int(self._dt(out, "out")), c_int(rows), c_int(cols), self._stream())
        _check("dynamic_tanh", st)
        return out

    def residual_dynamic_tanh(self, y, norm, x, next_norm, out_dtype):
        """x += tanh(alpha y) * w + b on the float32 stream, in place; norm = (alpha [1], w, b).  With `next_norm` of the same
        form the second result is that norm of the new x in `out_dtype`.  Returns (x, second result or None)."""
        _need(x, "x", torch.float32, 2); _need(y, "y", torch.float32, 2)
        if y.shape != x.shape:
            raise KernelError(f"residual_dynamic_tanh: {tuple(y.shape)} added to {tuple(x.shape)}")
        rows, cols = x.shape
        for n in (norm, next_norm):
            if n is not None:
                _need(n[0], "alpha", torch.float32, 1); _need(n[1], "weight", torch.float32, 1); _need(n[2], "bias", torch.float32, 1)
                if n[0].shape[0] != 1 or n[1].shape[0] != cols or n[2].shape[0] != cols:
                    raise KernelError(f"residual_dynamic_tanh: a norm of {n[1].shape[0]} weights for rows of {cols}")
        out = torch.empty((rows, cols), dtype=out_dtype, device=x.device) if next_norm is not None else None
        a2, w2, b2 = next_norm if next_norm is not None else (None, None, None)
        st = self._lib("streamops.cu").rv_residual_dynamic_tanh(
            _ptr(x), _ptr(y), _ptr(norm[0]), _ptr(norm[1]), _ptr(norm[2]), _ptr(a2), _ptr(w2), _ptr(b2), _ptr(out),
            c_int(_DT[out_dtype] if out is not None else 0), c_int(rows), c_int(cols), self._stream())
        _check("residual_dynamic_tanh", st)
        return x, out

    def scale_rows(self, x, scale: float) -> torch.Tensor:
        """x * scale as a new float32 tensor."""
        _need(x, "x")
        out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        st = self._lib("streamops.cu").rv_scale_rows(_ptr(x), c_int(self._dt(x, "x")), c_float(scale), _ptr(out),
                                                     ctypes.c_longlong(x.numel()), self._stream())
        _check("scale_rows", st)
        return out

    def act_rows(self, u, activation: str, out_dtype, row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
        """relu(u)^2 ("relu2"), times row_scale[t] (float32 [rows]) where given, in `out_dtype`."""
        _need(u, "u", dims=2)
        if activation != "relu2":
            raise KernelError(f"act_rows: activation {activation!r} is not known (relu2)")
        rows, cols = u.shape
        if row_scale is not None:
            _need(row_scale, "row_scale", torch.float32, 1)
            if row_scale.shape[0] != rows:
                raise KernelError(f"act_rows: {row_scale.shape[0]} row scales for {rows} rows")
        out = torch.empty((rows, cols), dtype=out_dtype, device=u.device)
        st = self._lib("streamops.cu").rv_act_rows(_ptr(u), c_int(self._dt(u, "u")), _ptr(row_scale), _ptr(out), c_int(_DT[out_dtype]),
                                                   c_int(0), c_int(rows), c_int(cols), self._stream())
        _check("act_rows", st)
        return out

    # ------------------------------------------------------------------ unit-norm attention, mLSTM
    def qk_unit_prepare(self, proj, eps: float, positions, cos, sin, slot_mapping, cache_layer, num_heads: int, num_kv_heads: int,
                        head_dim: int, value_dim: int, slot_dim: int, out_dtype, halves: bool = False, with_gate: bool = True,
                        write_kv: bool = True):
        """proj float32 rows [q: heads x head_dim | k: kv heads x head_dim | v: kv heads x value_dim | gate logits: heads] (k and v
        only with `write_kv`).  q and k: the leading 2 * cos.shape[1] elements of every head turn in pairs (2i, 2i + 1) - with
        `halves`: (i, i + cos.shape[1]) -, then the head is divided by sqrt(mean(x^2) + eps).  k and v go into the token's
        cache slot, in heads of `slot_dim` elements whose tail is zeros.  Returns (q [T, heads * slot_dim] in `out_dtype`,
        sigmoid(gate logits) float32 [T, heads] or None)."""
        _need(proj, "proj", torch.float32, 2); _need(positions, "positions", torch.int32, 1)
        T = proj.shape[0]
        want = num_heads * head_dim + (num_kv_heads * (head_dim + value_dim) if write_kv else 0) + (num_heads if with_gate else 0)
        if proj.shape[1] != want or slot_dim < max(head_dim, value_dim):
            raise KernelError(f"qk_unit_prepare: rows of {proj.shape[1]} columns do not fit {num_heads} heads of {head_dim}"
                              + (f", {num_kv_heads} key/value heads of {head_dim} / {value_dim}" if write_kv else "")
                              + (f" and {num_heads} gates" if with_gate else "") + f" in slots of {slot_dim}")
        rot, table_rows = 0, 1
        if cos is not None:
            _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
            rot, table_rows = 2 * cos.shape[1], cos.shape[0]
            if not 0 < rot <= head_dim or sin.shape != cos.shape:
                raise KernelError(f"qk_unit_prepare: cos/sin tables must be [rows, dims/2] with dims <= {head_dim}")
        page = 1
        if write_kv:
            _need(cache_layer, "cache_layer", out_dtype, 5); _need(slot_mapping, "slot_mapping", torch.int32, 1)
            if cache_layer.shape[1] != 2 or cache_layer.shape[2] != num_kv_heads or cache_layer.shape[4] != slot_dim:
                raise KernelError(f"qk_unit_prepare: cache layer of shape {tuple(cache_layer.shape)} for {num_kv_heads} heads of {slot_dim}")
            page = cache_layer.shape[3]
        q = torch.empty((T, num_heads * slot_dim), dtype=out_dtype, device=proj.device)
        gate = torch.empty((T, num_heads), dtype=torch.float32, device=proj.device) if with_gate else None
        st = self._lib("qk_prepare.cu").rv_qk_unit_prepare(
            _ptr(proj), c_int(proj.shape[1]), _ptr(positions), _ptr(cos), _ptr(sin), c_int(rot), c_int(table_rows),
            c_int(1 if halves else 0), _ptr(slot_mapping if write_kv else None), _ptr(cache_layer if write_kv else None), _ptr(q),
            c_int(_DT[out_dtype]), _ptr(gate), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(value_dim),
            c_int(slot_dim), c_int(page), c_float(eps), c_int(1 if write_kv else 0), self._stream())
        _check("qk_unit_prepare", st)
        return q, gate

    def mlstm_scan(self, proj, i_col0: int, f_col0: int, i_bias, f_bias, cu_seqlens, state_slots, state, heads: int, head_dim: int,
                   value_dim: int, cap: float):
        """The mLSTM recurrence over the step's tokens, per sequence from the memory its state row holds ([heads][head_dim]
        [value_dim + 1] floats; the last column of a head is the normaliser) and back into it.  proj float32 rows
        [q | k | v | ...] with the raw input- and forget-gate columns at i_col0 and f_col0.  Returns (raw float32
        [T, heads * (value_dim + 1)]: per head the numerators S^T q and, last, n . q; top float32 [T, heads]: the running
        maximum m_t).  The m of the state row is left as it was: `mlstm_output` stores the new one."""
        _need(proj, "proj", torch.float32, 2); _need(state, "state", torch.float32, 2)
        _need(i_bias, "i_bias", torch.float32, 1); _need(f_bias, "f_bias", torch.float32, 1)
        T = proj.shape[0]
        raw = torch.empty((T, heads * (value_dim + 1)), dtype=torch.float32, device=proj.device)
        top = torch.empty((T, heads), dtype=torch.float32, device=proj.device)
        st = self._lib("mlstm.cu").rv_mlstm_scan(
            _ptr(proj), c_int(proj.shape[1]), c_int(i_col0), c_int(f_col0), _ptr(i_bias), _ptr(f_bias), _ptr(cu_seqlens), _ptr(state_slots),
            _ptr(state), ctypes.c_longlong(state.stride(0)), _ptr(raw), _ptr(top), c_int(cu_seqlens.shape[0] - 1), c_int(heads),
            c_int(head_dim), c_int(value_dim), c_float(cap), self._stream())
        _check("mlstm_scan", st)
        return raw, top

    def mlstm_output(self, raw, top, gamma, eps: float, den_eps: float, proj, g_col0: int, heads: int, head_dim: int, value_dim: int,
                     out_dtype, token_seq, cu_seqlens, state_slots, state) -> torch.Tensor:
        """o = numerators / (max(|n . q|, exp(-m)) + den_eps); per head o / sqrt(mean(o^2) + eps) * gamma * sigmoid(gate columns
        of proj from g_col0 on), in `out_dtype`; and the m of every sequence's last token into its state row."""
        _need(raw, "raw", torch.float32, 2); _need(top, "top", torch.float32, 2); _need(gamma, "gamma", torch.float32, 1)
        _need(proj, "proj", torch.float32, 2); _need(state, "state", torch.float32, 2)
        T = raw.shape[0]
        if raw.shape[1] != heads * (value_dim + 1) or tuple(top.shape) != (T, heads) or gamma.shape[0] != heads * value_dim:
            raise KernelError(f"mlstm_output: raw {tuple(raw.shape)}, top {tuple(top.shape)}, gamma {tuple(gamma.shape)} for {heads} heads of {value_dim}")
        out = torch.empty((T, heads * value_dim), dtype=out_dtype, device=raw.device)
        st = self._lib("mlstm.cu").rv_mlstm_output(
            _ptr(raw), _ptr(top), _ptr(gamma), _ptr(proj), c_int(proj.shape[1]), c_int(g_col0), _ptr(out), c_int(_DT[out_dtype]), c_int(T),
            c_int(heads), c_int(head_dim), c_int(value_dim), c_float(eps), c_float(den_eps), _ptr(token_seq), _ptr(cu_seqlens),
            _ptr(state_slots), _ptr(state), ctypes.c_longlong(state.stride(0)), self._stream())
        _check("mlstm_output", st)
        return out

    # ------------------------------------------------------------------ sampling
    def sample(self, logits, temperature=None, top_k=None, top_p=None, seeds=None, draw_index=None) -> torch.Tensor:
        """One token id per row of float logits.  All parameter tensors are per row; rows with
        temperature 0 (or `temperature` None) are greedy."""
        _need(logits, "logits", torch.float32, 2)
        R, V = logits.shape
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
        if temperature is not None:
            _need(temperature, "temperature", torch.float32, 1)
            _need(seeds, "seeds", torch.int64, 1); _need(draw_index, "draw_index", torch.int64, 1)
        if top_k is not None:
            _need(top_k, "top_k", torch.int32, 1)
        if top_p is not None:
            _need(top_p, "top_p", torch.float32, 1)
        st = self._lib("sampling.cu").rv_sample(_ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p),
                                                _ptr(seeds), _ptr(draw_index), _ptr(out), c_int(R), c_int(V),
                                                self._stream())
        _check("sample", st)
        return out
