"""The CUDA kernel set: ctypes bindings of the native library, with the interface the
parts call (`embed`, `add_rmsnorm`, `linear`, `qk_norm_rope_write`, `paged_attention`,
`short_conv`, `swiglu`, `add_bias`, `argmax`, `sample`).

Every kernel launches on torch's current stream, so captured graphs and ordinary
stream order both work.  Matrix products go to cuBLAS through `torch.mm`, as the
reference sends them to cuBLAS (src/cuda/cublas_ops.rs:44-92); with float32 operands
TF32 is switched off, so the float32 path is float32 throughout.  There is no CPU
path here: constructing `CudaOps` without a CUDA device or without the library raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..errors import KernelError
from .build import build, build_variant

_F32, _BF16 = 0, 1


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dtype}")


def _ptr(t):
    return c_void_p(0 if t is None else t.data_ptr())


class CudaOps:
    name = "cuda"

    def __init__(self, verbose_build: bool = True):
        if not torch.cuda.is_available():
            raise KernelError("rvllm_b200 needs a CUDA device: there is no CPU path")
        path = build(verbose=verbose_build)
        try:
            self.lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the kernel library {path}: {e}") from None
        self.library_path = path
        self.launches = 0
        self.lib.rv_last_error.restype = ctypes.c_char_p
        self.lib.rv_paged_attention_decode_scratch_bytes.restype = c_longlong
        self.lib.rv_gemm_tiled_bytes.restype = c_longlong
        self.lib.rv_gated_delta_scratch.restype = c_longlong
        self.lib.rv_mlstm_scratch.restype = c_longlong
        self.lib.rv_paged_attention_mixed_scratch_bytes.restype = c_longlong
        self._scratch = {}
        self._retired = []
        self._attn_libs = {}
        self._verbose_build = verbose_build
        # bfloat16 attention: "mma" = mma.sync tensor-core kernels (attention_mma.cu, head
        # sizes that are multiples of 16 up to 128), "simt" = the float32-arithmetic kernels;
        # prompt portions also "tcgen05" (attention_tcgen05.cu, head size 64) and "auto" =
        # tcgen05 where it applies, else mma
        self.prefill_attention = os.environ.get("RVLLM_PREFILL_ATTENTION", "auto")
        self.decode_attention = os.environ.get("RVLLM_DECODE_ATTENTION", "mma")
        # keys per block of the tensor-core decode kernel: 256 (four warps) or 128 (two)
        self.decode_split = int(os.environ.get("RVLLM_ATTN_DECODE_SPLIT", "256"))
        # "stream": one persistent block per SM whose warps each stream their work items'
        # tiles through a private ring; "block": one block per (request, head, split);
        # "auto": the stream kernel from `stream_min_items` work items of 256 keys on
        self.decode_kernel = os.environ.get("RVLLM_ATTN_DECODE_KERNEL", "auto")
        self.stream_min_items = int(os.environ.get("RVLLM_ATTN_STREAM_MIN_ITEMS", "384"))
        self._sm_count = torch.cuda.get_device_properties(
            torch.cuda.current_device()).multi_processor_count
        # bfloat16 products with at most `gemm_small_m` tokens go to the tcgen05
        # weight-streaming kernel (gemm_tcgen05.cu), whose weight copies start before the
        # previous kernel has finished; larger ones go to cuBLAS.  RVLLM_GEMM=cublas sends
        # everything to cuBLAS, =auto only the shapes with few output tiles and a long K.
        self.gemm_small_m = int(os.environ.get("RVLLM_GEMM_SMALL_M", "16"))
        self.gemm_mode = os.environ.get("RVLLM_GEMM", "tcgen05")
        self._gemm_state = {}
        self._tiled = {}
        self.gemm_tiled = os.environ.get("RVLLM_GEMM_TILED", "1") != "0"
        self.gemm_row_pad = int(os.environ.get("RVLLM_GEMM_ROW_PAD", "64"))
        # q/k norm + rotation + cache write inside the q|k|v product's epilogue (few bfloat16
        # tokens, head size 64); "0": always the separate kernel
        self.fuse_qkv_rope = os.environ.get("RVLLM_FUSE_QKV_ROPE", "1") == "1"
        self._check(self.lib.rv_gemm_tcgen05_init(), "gemm_tcgen05 set-up")
        self._check(self.lib.rv_moe_grouped_init(), "moe_grouped set-up")
        self.lib.rv_moe_grouped_scratch_bytes.restype = c_longlong
        # experts of a mixture: "grouped" = tokens sorted by expert through grouped tcgen05
        # products (bfloat16, widths in multiples of 8), "simple" = token by token; "auto" =
        # grouped from `moe_grouped_min` (token, expert) pairs on
        self.moe_mode = os.environ.get("RVLLM_MOE", "auto")
        self.moe_grouped_min = int(os.environ.get("RVLLM_MOE_GROUPED_MIN", "16"))
        # float32 products must be float32: no TF32, no reduced-precision accumulation
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        self.launches = 0

    # ---- plumbing --------------------------------------------------------------------

    def _check(self, rc: int, what: str) -> None:
        self.launches += 1
        if rc != 0:
            raise KernelError(f"{what}: {self.lib.rv_last_error().decode()}")

    @staticmethod
    def _stream() -> c_void_p:
        # the current stream of the current device; the raw query is a fraction of a microsecond
        # where `torch.cuda.current_stream()` builds a Python object in some 15 (and a step of a
        # small model makes some 140 launches)
        raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
        if raw is not None:
            return c_void_p(raw(torch._C._cuda_getDevice()))
        return c_void_p(torch.cuda.current_stream().cuda_stream)

    @staticmethod
    def _need(t: torch.Tensor, what: str, dtype=None, contiguous=True):
        if not t.is_cuda:
            raise KernelError(f"{what} must be a CUDA tensor")
        if contiguous and not t.is_contiguous():
            raise KernelError(f"{what} must be contiguous")
        if dtype is not None and t.dtype != dtype:
            raise KernelError(f"{what} must be {dtype}, got {t.dtype}")

    # ---- embedding -------------------------------------------------------------------

    def embed(self, table, ids, out, scale=None):
        self._need(table, "embedding table")
        self._need(ids, "token ids", torch.int32)
        self._need(out, "embedding output", torch.float32)
        n, hidden = out.shape
        self._check(self.lib.rv_embed(_ptr(table), _code(table.dtype), _ptr(ids), _ptr(out),
                                      c_int(n), c_int(hidden), c_int(table.shape[0]),
                                      c_float(1.0 if scale is None else scale), self._stream()),
                    "embed")

    # ---- residual add + RMSNorm ------------------------------------------------------

    def add_rmsnorm(self, resid, delta, weight, eps, out, rows=None, delta_scale=None, add=None):
        """`resid` None: the rows of `delta` alone are normalised (no stream involved).
        `delta_scale` float32 [hidden]: the pending rows are multiplied by it, channel by channel,
        before they are added; `add` float32 [hidden]: one vector added to every row."""
        if resid is not None:
            self._need(resid, "residual stream", torch.float32)
        elif delta is None or rows is not None:
            raise KernelError("add_rmsnorm: without a stream it takes rows to normalise, all of them")
        self._need(weight, "norm weight", torch.float32)
        self._need(out, "norm output")
        if delta is not None:
            self._need(delta, "pending sub-layer output")
            if resid is not None and delta.shape != resid.shape:
                raise KernelError("add_rmsnorm: the stream and the pending output differ in shape")
        if rows is not None:
            self._need(rows, "row list", torch.int32)
        n, hidden = out.shape
        if (resid if resid is not None else delta).shape[1] != hidden or weight.shape[0] != hidden:
            raise KernelError("add_rmsnorm: widths disagree")
        for vec, what in ((delta_scale, "scale of the pending rows"), (add, "added vector")):
            if vec is not None:
                self._need(vec, what, torch.float32)
                if vec.shape != (hidden,):
                    raise KernelError(f"add_rmsnorm: the {what} has another width")
        if delta_scale is not None and delta is None:
            raise KernelError("add_rmsnorm: a scale without pending rows")
        self._check(self.lib.rv_add_rmsnorm_ex(
            _ptr(resid), _ptr(delta), _code(delta.dtype) if delta is not None else _F32,
            _ptr(weight), _ptr(out), _code(out.dtype), _ptr(rows), c_int(n), c_int(hidden),
            c_float(eps), _ptr(delta_scale), _ptr(add), self._stream()), "add_rmsnorm")

    # ---- matrix product (library) -------------------------------------------------------

    def _gemm_status(self, device):
        device = torch.device(device)
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        st = self._gemm_state.get(device)
        if st is None:
            st = torch.zeros(1, dtype=torch.int32, device=device)
            self._gemm_state[device] = st
        return st

    def linear_tcgen05(self, x, w, out_dtype):
        """y = x . w^T for bfloat16 x [M <= 256, K] and w [N, K] on the tcgen05 kernel."""
        self._need(x, "activation rows", torch.bfloat16)
        self._need(w, "weight matrix", torch.bfloat16)
        m, k = x.shape
        n = w.shape[0]
        y = torch.empty((m, n), dtype=out_dtype, device=x.device)
        self._check(self.lib.rv_gemm_tcgen05(
            _ptr(x), _ptr(w), _ptr(y), _code(out_dtype), _ptr(self._gemm_status(x.device)),
            c_int(m), c_int(n), c_int(k), _ptr(self._tiled_weight(w)), self._stream()),
            "gemm_tcgen05")
        return y

    def _tiled_weight(self, w):
        """The weight matrix once more, laid out tile by tile for the streaming product
        (`rv_gemm_tile_weights`): made the first time a matrix is used with few tokens and
        kept as long as the matrix lives.  It doubles the memory of the matrices that decode
        steps multiply (2.3 GB at LFM2-1.2B sizes) and lets an SM copy a tile as one
        contiguous 16 KB instead of 128 strided rows.  RVLLM_GEMM_TILED=0: not made."""
        if not self.gemm_tiled:
            return None
        key = (w.data_ptr(), tuple(w.shape))
        hit = self._tiled.get(key)
        if hit is not None and hit[0]() is w:
            return hit[1]
        if torch.cuda.is_current_stream_capturing():
            return None                    # no allocation inside a capture: the box copies do
        n, k = w.shape
        nbytes = int(self.lib.rv_gemm_tiled_bytes(c_int(n), c_int(k)))
        tiled = torch.empty(nbytes, dtype=torch.uint8, device=w.device)
        self._check(self.lib.rv_gemm_tile_weights(_ptr(w), _ptr(tiled), c_int(n), c_int(k),
                                                  self._stream()), "gemm_tile_weights")
        import weakref
        # the copies of matrices that have died go first (a model that was unloaded)
        self._tiled = {kk: v for kk, v in self._tiled.items() if v[0]() is not None}
        self._tiled[key] = (weakref.ref(w), tiled)
        return tiled

    def status_word(self, device) -> torch.Tensor:
        """The int32 word in which kernels on `device` record a wait that ran out (0: none).
        A caller that already copies a step's result to the host can copy this word along
        and pass what it read to `raise_for_status`, which costs no synchronisation."""
        return self._gemm_status(device)

    def raise_for_status(self, code: int, device=None) -> None:
        if code != 0:
            if device is not None:
                self._gemm_status(device).zero_()
            raise KernelError(f"a kernel gave up waiting on an mbarrier (code {code}: 1-4 "
                              f"gemm_tcgen05, 12 decode attention, 21 prefill attention, 31-34 "
                              f"grouped experts); its output is not valid")

    def check_status(self) -> None:
        """Raise if a kernel recorded that one of its bounded waits ran out (this
        synchronises with the device)."""
        for device, st in self._gemm_state.items():
            code = int(st.item())
            if code != 0:
                st.zero_()
                raise KernelError(f"a kernel gave up waiting on an mbarrier (code {code}: 1-4 "
                                  f"gemm_tcgen05, 12 decode attention, 21 prefill attention) on {device}; its "
                                  f"output is not valid")

    def _small_product(self, x, w, out_dtype) -> bool:
        """Whether x . w^T goes to the tcgen05 weight-streaming kernel."""
        return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and 0 < x.shape[0] <= self.gemm_small_m and self.gemm_mode != "cublas"
                and x.shape[1] % 8 == 0 and x.is_contiguous() and w.is_contiguous()
                and out_dtype in (torch.bfloat16, torch.float32)
                and (self.gemm_mode == "tcgen05"
                     or (w.shape[0] <= 18 * 128 and x.shape[1] >= 4096)))

    def linear_qk_norm_rope_write(self, x, w_qkv, num_heads, num_kv_heads, head_dim, q_weight,
                                  k_weight, eps, table, positions, slot_mapping, k_cache, v_cache,
                                  out_dtype=None):
        """q|k|v = x . w_qkv^T, then per-head q/k norm, rotation and the cache write; returns
        the [tokens, (heads + 2 kv heads) * head_dim] buffer whose query columns attention
        reads.  Few bfloat16 tokens with head size 64 and a cache to write: one kernel (the
        product's epilogue does the rest); otherwise the product and `qk_norm_rope_write`."""
        out_dtype = out_dtype or x.dtype
        if (self.fuse_qkv_rope and k_cache is not None and num_kv_heads > 0 and head_dim == 64
                and out_dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
                and w_qkv.shape[0] == (num_heads + 2 * num_kv_heads) * 64
                and x.shape[0] <= 16 and self._small_product(x, w_qkv, out_dtype)):
            m, k = x.shape
            n = w_qkv.shape[0]
            qkv = torch.empty((m, n), dtype=out_dtype, device=x.device)
            cos, sin = table if table is not None else (None, None)
            self._check(self.lib.rv_gemm_tcgen05_qkv(
                _ptr(x), _ptr(w_qkv), _ptr(qkv), _ptr(self._gemm_status(x.device)), c_int(m),
                c_int(n), c_int(k), c_int(num_heads), c_int(num_kv_heads), _ptr(q_weight),
                _ptr(k_weight), c_float(eps), _ptr(cos), _ptr(sin), _ptr(positions),
                _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), _ptr(self._tiled_weight(w_qkv)),
                self._stream()), "gemm_tcgen05_qkv")
            return qkv
        qkv = self.linear(x, w_qkv, out_dtype=out_dtype)
        self.qk_norm_rope_write(qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps,
                                table, positions, slot_mapping, k_cache, v_cache)
        return qkv

    def linear(self, x, w, bias=None, out_dtype=None):
        out_dtype = out_dtype or x.dtype
        if x.dtype != w.dtype:
            # a matrix kept in 32 bits is multiplied in 32 bits
            wide = torch.float32 if torch.float32 in (x.dtype, w.dtype) else x.dtype
            x, w = x.to(wide), w.to(wide)
        if x.shape[0] == 0:
            return torch.empty((0, w.shape[0]), dtype=out_dtype, device=x.device)
        if self._small_product(x, w, out_dtype):
            y = self.linear_tcgen05(x, w, out_dtype)
        else:
            # The library chooses an algorithm per shape, and a shape it has not met costs it
            # some 70 us on the host: a prompt portion of 301 tokens, then 302, ... would pay
            # that in every product of every step.  So it is shown row counts in multiples of
            # 64 (RVLLM_GEMM_ROW_PAD): the rows beyond the real ones are whatever the buffer
            # holds (`new_rows` leaves room for them) and their results are dropped.
            m = x.shape[0]
            xp = self._padded_rows(x)
            if out_dtype == x.dtype:
                y = torch.mm(xp, w.t())
            elif x.dtype == torch.bfloat16 and out_dtype == torch.float32:
                y = torch.mm(xp, w.t(), out_dtype=torch.float32)
            else:
                y = torch.mm(xp, w.t()).to(out_dtype)
            if y.shape[0] != m:
                y = y[:m]
        if bias is not None:
            self.add_bias(y, bias)
        return y

    def new_rows(self, n, width, dtype, device):
        """An uninitialised [n, width] buffer for activation rows whose storage is a multiple
        of the row padding long, so that a library product can take it as it is."""
        pad = self._row_pad(n)
        if pad <= 1 or n % pad == 0:
            return torch.empty((n, width), dtype=dtype, device=device)
        return torch.empty((-(-n // pad) * pad, width), dtype=dtype, device=device)[:n]

    def _row_pad(self, n: int) -> int:
        """Rows are padded to multiples of 64, of 32 up to 64 rows (a replayed decode step of 32
        requests is 1 % slower with 64 rows than with its own 32)."""
        return min(self.gemm_row_pad, 32) if n <= 64 else self.gemm_row_pad

    def _padded_rows(self, x):
        m, k = x.shape
        pad = self._row_pad(m)
        if pad <= 1 or m % pad == 0 or not x.is_contiguous():
            return x
        mp = -(-m // pad) * pad
        if x.storage_offset() == 0 and x.untyped_storage().nbytes() >= mp * k * x.element_size():
            return x.as_strided((mp, k), (k, 1))          # the buffer has the room (`new_rows`)
        xp = torch.empty((mp, k), dtype=x.dtype, device=x.device)
        xp[:m].copy_(x)
        return xp

    def add_bias(self, x, bias):
        self._need(x, "add_bias input")
        self._need(bias, "bias", torch.float32)
        self._check(self.lib.rv_add_bias(_ptr(x), _code(x.dtype), _ptr(bias), c_int(x.shape[0]),
                                         c_int(x.shape[1]), self._stream()), "add_bias")

    # ---- q/k norm + rotation + cache write -------------------------------------------

    def qk_norm_rope_write(self, qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight,
                           eps, table, positions, slot_mapping, k_cache, v_cache):
        self._need(qkv, "q|k|v rows")
        if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
            raise KernelError("qk_norm_rope_write: row width and head counts disagree")
        if k_cache is not None:
            self._need(k_cache, "key pages", qkv.dtype)
            self._need(v_cache, "value pages", qkv.dtype)
        cos, sin = table if table is not None else (None, None)
        self._check(self.lib.rv_qk_norm_rope_write(
            _ptr(qkv), _code(qkv.dtype), c_int(qkv.shape[1]), c_int(qkv.shape[0]),
            c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), _ptr(q_weight),
            _ptr(k_weight), c_float(eps), _ptr(cos), _ptr(sin), _ptr(positions),
            _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), self._stream()),
            "qk_norm_rope_write")

    # ---- attention -------------------------------------------------------------------

    def _scratch_buffer(self, nbytes: int, device) -> torch.Tensor:
        """The split-KV scratch of `device`, at least `nbytes` long.  A captured launch
        sequence holds the raw address of the buffer it was captured with, so a buffer
        that is outgrown is never given back: it moves to `_retired` and stays valid for
        every graph that names it.  Growth doubles, so the retired ones together are
        smaller than the live one."""
        key = str(device)
        buf = self._scratch.get(key)
        if buf is None or buf.numel() < nbytes:
            size = max(nbytes, 1 << 20, 2 * buf.numel() if buf is not None else 0)
            if buf is not None:
                self._retired.append(buf)
            buf = torch.empty(size, dtype=torch.uint8, device=device)
            self._scratch[key] = buf
        return buf

    def attention_scratch_bytes(self, n_reqs: int, num_heads: int, head_dim: int,
                                max_ctx_len: int) -> int:
        """Bytes of split-KV scratch the decode attention kernels need at most for
        `n_reqs` single-token requests of up to `max_ctx_len` cached tokens (with the
        smallest split any of them uses, 128 keys)."""
        decode = int(self.lib.rv_paged_attention_decode_scratch_bytes(
            c_int(n_reqs), c_int(num_heads), c_int(head_dim), c_int(2 * max_ctx_len)))
        return max(decode, self._prefill_scratch_bytes(head_dim))

    def reserve_scratch(self, nbytes: int, device) -> None:
        """Size the scratch before any launch sequence is captured, so that it does not
        have to grow afterwards."""
        if nbytes > 0:
            self._scratch_buffer(nbytes, device)

    def _attn_lib(self, head_dim: int):
        """The tensor-core attention library for this head size, built at first use."""
        lib = self._attn_libs.get(head_dim)
        if lib is None:
            path = build_variant("attention_mma.cu", {"RV_HD": head_dim}, f"attn_hd{head_dim}",
                                 verbose=self._verbose_build)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load the kernel library {path}: {e}") from None
            getattr(lib, f"rv_attention_mma_last_error_hd{head_dim}").restype = ctypes.c_char_p
            self._attn_libs[head_dim] = lib
        return lib

    def _attn5_lib(self, head_dim: int):
        """The tcgen05 prefill attention library for this head size, built at first use."""
        key = ("tcgen05", head_dim)
        lib = self._attn_libs.get(key)
        if lib is None:
            path = build_variant("attention_tcgen05.cu", {"RV_HD": head_dim},
                                 f"attn5_hd{head_dim}", verbose=self._verbose_build)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load the kernel library {path}: {e}") from None
            getattr(lib, f"rv_attention_tcgen05_last_error_hd{head_dim}").restype = ctypes.c_char_p
            self._attn_libs[key] = lib
        return lib

    def _tcgen05_prefill_ok(self, qkv, out, num_heads, num_kv_heads, head_dim, page_size) -> bool:
        return (qkv.dtype == torch.bfloat16 and head_dim == 64
                and page_size in (8, 16, 32, 64) and num_heads // num_kv_heads <= 128
                and qkv.shape[1] % head_dim == 0 and qkv.data_ptr() % 16 == 0
                and out.data_ptr() % 16 == 0)

    def paged_attention_prefill_tcgen05(self, qkv, num_heads, num_kv_heads, head_dim, k_cache,
                                        v_cache, ctx, group, scale, window, out, sinks=None):
        """Requests [n_decode, n_reqs) -- the ones that bring more than one token -- on the
        tcgen05 kernel (bfloat16, head size 64)."""
        lib = self._attn5_lib(head_dim)
        nd = ctx.n_decode
        fn = getattr(lib, f"rv_paged_attention_prefill_tcgen05_hd{head_dim}")
        # scratch for the parts of a launch too small to fill the GPU (the kernel shares the key
        # tiles of its blocks out); never made or grown inside a stream capture
        need = self._prefill_scratch_bytes(head_dim)
        scratch = self._scratch.get(str(qkv.device))
        if scratch is None or scratch.numel() < need:
            scratch = (None if torch.cuda.is_current_stream_capturing()
                       else self._scratch_buffer(need, qkv.device))
        rc = fn(_ptr(qkv), c_int(qkv.shape[1]), c_int(qkv.shape[0]), _ptr(k_cache), _ptr(v_cache),
                c_longlong(k_cache.shape[0] * k_cache.shape[1]), _ptr(group.block_table),
                c_int(group.max_blocks), _ptr(ctx.q_start), _ptr(ctx.ctx_lens), _ptr(out),
                c_int(nd), c_int(ctx.n_reqs - nd), c_int(ctx.max_q_len), c_int(ctx.max_ctx_len),
                c_int(num_heads), c_int(num_kv_heads), c_int(group.page_size), c_float(scale),
                c_int(window if window else 0), _ptr(self._gemm_status(qkv.device)),
                _ptr(scratch), c_longlong(scratch.numel() if scratch is not None else 0),
                c_int(self._sm_count), _ptr(sinks), self._stream())
        self.launches += 1
        if rc != 0:
            msg = getattr(lib, f"rv_attention_tcgen05_last_error_hd{head_dim}")().decode()
            raise KernelError(f"paged_attention_prefill_tcgen05: {msg}")

    def _prefill_scratch_bytes(self, head_dim: int) -> int:
        """What the tcgen05 prefill attention may use for the parts of shared-out blocks."""
        if head_dim != 64 or self.prefill_attention not in ("auto", "tcgen05"):
            return 0
        # rv_paged_attention_prefill_tcgen05_scratch_bytes: six parts an SM, each 128 rows of
        # 64 float32 values, an offset and a sum (the kernel fits its parts to what it is given)
        return 6 * self._sm_count * 128 * (64 * 4 + 8)

    def _check_attn(self, lib, head_dim: int, rc: int, what: str) -> None:
        self.launches += 1
        if rc != 0:
            msg = getattr(lib, f"rv_attention_mma_last_error_hd{head_dim}")().decode()
            raise KernelError(f"{what}: {msg}")

    @staticmethod
    def _mma_ok(dtype, head_dim: int) -> bool:
        return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128

    def paged_attention(self, qkv, num_heads, num_kv_heads, head_dim, k_cache, v_cache,
                        ctx, group, scale, window, out, sinks=None, v_head_dim=None):
        """`sinks` float32 [heads]: one more term exp(sinks[h]) in head h's softmax denominator;
        `v_head_dim`: the size of a value head when it is not `head_dim`."""
        self._need(qkv, "query rows")
        self._need(out, "attention output", qkv.dtype)
        self._need(k_cache, "key pages", qkv.dtype)
        self._need(v_cache, "value pages", qkv.dtype)
        vd = v_head_dim or head_dim
        if sinks is not None:
            self._need(sinks, "sinks", torch.float32)
            if sinks.shape[0] != num_heads:
                raise KernelError("paged_attention: one sink per query head")
        if out.shape[1] != num_heads * vd:
            raise KernelError("paged_attention: output width and head sizes disagree")
        # the tensor-core kernels fetch query rows in 16-byte pieces: rows of another stride or
        # start take the float32-arithmetic kernels
        mma = (self._mma_ok(qkv.dtype, head_dim) and qkv.shape[1] % 8 == 0
               and qkv.data_ptr() % 16 == 0)
        if vd != head_dim or (sinks is not None and not mma):
            # a value size of its own, or sinks where no tensor-core kernel applies: the
            # float32-arithmetic kernels
            return self._paged_attention_options(qkv, num_heads, num_kv_heads, head_dim, vd,
                                                 k_cache, v_cache, ctx, group, scale, window, out,
                                                 sinks)
        code = _code(qkv.dtype)
        win = c_int(window if window else 0)
        nd = ctx.n_decode
        if nd > 0:
            if mma and self.decode_attention == "mma":
                self.paged_attention_decode_mma(qkv, num_heads, num_kv_heads, head_dim, k_cache,
                                                v_cache, group.block_table, ctx.q_start,
                                                ctx.ctx_lens, nd, ctx.max_ctx_len,
                                                group.page_size, scale, window, out, sinks=sinks)
            elif sinks is not None:
                self._paged_attention_options(qkv, num_heads, num_kv_heads, head_dim, vd, k_cache,
                                              v_cache, ctx, group, scale, window, out, sinks,
                                              prompts=False)
            else:
                self.paged_attention_decode(qkv, num_heads, num_kv_heads, head_dim, k_cache,
                                            v_cache, group.block_table, ctx.ctx_lens, nd,
                                            ctx.max_ctx_len, group.page_size, scale, window, out)
        if (ctx.n_tokens > nd and self.prefill_attention in ("auto", "tcgen05")
                and self._tcgen05_prefill_ok(qkv, out, num_heads, num_kv_heads, head_dim,
                                             group.page_size)):
            self.paged_attention_prefill_tcgen05(qkv, num_heads, num_kv_heads, head_dim, k_cache,
                                                 v_cache, ctx, group, scale, window, out,
                                                 sinks=sinks)
        elif ctx.n_tokens > nd and mma and self.prefill_attention in ("auto", "mma", "tcgen05"):
            lib = self._attn_lib(head_dim)
            fn = getattr(lib, f"rv_paged_attention_prefill_mma_hd{head_dim}")
            self._check_attn(lib, head_dim, fn(
                _ptr(qkv), c_int(qkv.shape[1]), _ptr(k_cache), _ptr(v_cache),
                _ptr(group.block_table), c_int(group.max_blocks), _ptr(ctx.q_start),
                _ptr(ctx.ctx_lens), _ptr(out), c_int(nd), c_int(ctx.n_reqs - nd),
                c_int(ctx.max_q_len), c_int(num_heads), c_int(num_kv_heads),
                c_int(group.page_size), c_float(scale), win, _ptr(sinks), self._stream()),
                "paged_attention_prefill_mma")
        elif ctx.n_tokens > nd:
            self._check(self.lib.rv_paged_attention_warp_ex(
                _ptr(qkv), code, c_int(qkv.shape[1]), _ptr(k_cache), _ptr(v_cache),
                _ptr(group.block_table), c_int(group.max_blocks), _ptr(ctx.q_start),
                _ptr(ctx.ctx_lens), _ptr(ctx.token_req), _ptr(out), c_int(nd),
                c_int(ctx.n_tokens - nd), c_int(num_heads), c_int(num_kv_heads),
                c_int(head_dim), c_int(group.page_size), c_float(scale), win, c_int(head_dim),
                _ptr(sinks), self._stream()), "paged_attention")

    def _paged_attention_options(self, qkv, num_heads, num_kv_heads, head_dim, vd, k_cache,
                                 v_cache, ctx, group, scale, window, out, sinks, prompts=True):
        """Attention with sinks or a value size of its own: single tokens on the split kernel
        with its merge, portions on the one-warp-per-(token, head) kernel, both in float32
        arithmetic."""
        nd = ctx.n_decode
        code = _code(qkv.dtype)
        win = c_int(window if window else 0)
        if nd > 0:
            need = self.lib.rv_paged_attention_decode_scratch_bytes(
                c_int(nd), c_int(num_heads), c_int(vd), c_int(ctx.max_ctx_len))
            scratch = self._scratch_buffer(need, qkv.device)
            self._check(self.lib.rv_paged_attention_decode_ex(
                _ptr(qkv), code, c_int(qkv.shape[1]), _ptr(k_cache), _ptr(v_cache),
                _ptr(group.block_table), c_int(group.block_table.shape[1]), _ptr(ctx.ctx_lens),
                _ptr(out), _ptr(scratch), c_longlong(scratch.numel()), c_int(nd),
                c_int(ctx.max_ctx_len), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
                c_int(group.page_size), c_float(scale), win, c_int(vd), _ptr(sinks),
                self._stream()), "paged_attention_decode")
            self.launches += 1
        if ctx.n_tokens > nd and prompts:
            self._check(self.lib.rv_paged_attention_warp_ex(
                _ptr(qkv), code, c_int(qkv.shape[1]), _ptr(k_cache), _ptr(v_cache),
                _ptr(group.block_table), c_int(group.max_blocks), _ptr(ctx.q_start),
                _ptr(ctx.ctx_lens), _ptr(ctx.token_req), _ptr(out), c_int(nd),
                c_int(ctx.n_tokens - nd), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
                c_int(group.page_size), c_float(scale), win, c_int(vd), _ptr(sinks),
                self._stream()), "paged_attention")

    def paged_attention_decode(self, qkv, num_heads, num_kv_heads, head_dim, k_cache, v_cache,
                               block_table, ctx_lens, n_reqs, max_ctx_len, page_size, scale,
                               window, out, scratch=None):
        """Split-KV attention for requests [0, n_reqs) that bring one token each."""
        need = self.lib.rv_paged_attention_decode_scratch_bytes(
            c_int(n_reqs), c_int(num_heads), c_int(head_dim), c_int(max_ctx_len))
        if scratch is None:
            scratch = self._scratch_buffer(need, qkv.device)
        self._check(self.lib.rv_paged_attention_decode(
            _ptr(qkv), _code(qkv.dtype), c_int(qkv.shape[1]), _ptr(k_cache), _ptr(v_cache),
            _ptr(block_table), c_int(block_table.shape[1]), _ptr(ctx_lens), _ptr(out),
            _ptr(scratch), c_longlong(scratch.numel() * scratch.element_size()),
            c_int(n_reqs), c_int(max_ctx_len), c_int(num_heads), c_int(num_kv_heads),
            c_int(head_dim), c_int(page_size), c_float(scale), c_int(window if window else 0),
            self._stream()), "paged_attention_decode")

    def paged_attention_decode_mma(self, qkv, num_heads, num_kv_heads, head_dim, k_cache, v_cache,
                                   block_table, q_start, ctx_lens, n_reqs, max_ctx_len,
                                   page_size, scale, window, out, scratch=None, sinks=None):
        """Tensor-core split-KV attention (bfloat16) for requests [0, n_reqs) that bring one
        token each; the splits are combined by the merge kernel."""
        stream = (self.decode_kernel in ("stream", "auto") and head_dim == 64
                  and page_size in (8, 16, 32, 64))
        lib = self._attn_lib(head_dim)
        if stream and self.decode_kernel == "auto":
            items = (n_reqs * -(-max_ctx_len // 256) * num_kv_heads
                     * -(-(num_heads // num_kv_heads) // 16))
            stream = items >= self.stream_min_items
        if stream:
            split = getattr(lib, f"rv_paged_attention_decode_stream_split_hd{head_dim}")(
                c_int(n_reqs), c_int(max_ctx_len), c_int(num_heads), c_int(num_kv_heads),
                c_int(self._sm_count))
        else:
            split = self.decode_split
        need = self.lib.rv_paged_attention_decode_scratch_bytes(
            c_int(n_reqs), c_int(num_heads), c_int(head_dim), c_int(max_ctx_len * (256 // split)))
        if scratch is None:
            scratch = self._scratch_buffer(need, qkv.device)
        win = c_int(window if window else 0)
        if stream:
            fn = getattr(lib, f"rv_paged_attention_decode_stream_hd{head_dim}")
            self._check_attn(lib, head_dim, fn(
                _ptr(qkv), c_int(qkv.shape[1]), _ptr(k_cache), _ptr(v_cache),
                c_longlong(k_cache.shape[0] * k_cache.shape[1]), _ptr(block_table),
                c_int(block_table.shape[1]), _ptr(ctx_lens), _ptr(scratch),
                c_longlong(scratch.numel() * scratch.element_size()), c_int(n_reqs),
                c_int(max_ctx_len), c_int(num_heads), c_int(num_kv_heads), c_int(page_size),
                c_float(scale), win, c_int(split), c_int(self._sm_count),
                _ptr(self._gemm_status(qkv.device)), self._stream()),
                "paged_attention_decode_stream")
            self._check(self.lib.rv_paged_attention_merge_ex(
                _ptr(scratch), _ptr(ctx_lens), _ptr(out), _code(out.dtype), c_int(n_reqs),
                c_int(max_ctx_len), c_int(num_heads), c_int(head_dim), win, c_int(split),
                _ptr(sinks), self._stream()), "paged_attention_merge")
            return
        fn = getattr(lib, f"rv_paged_attention_decode_mma_hd{head_dim}")
        self._check_attn(lib, head_dim, fn(
            _ptr(qkv), c_int(qkv.shape[1]), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
            c_int(block_table.shape[1]), _ptr(q_start), _ptr(ctx_lens), _ptr(scratch),
            c_longlong(scratch.numel() * scratch.element_size()), c_int(n_reqs),
            c_int(max_ctx_len), c_int(num_heads), c_int(num_kv_heads), c_int(page_size),
            c_float(scale), win, c_int(split), self._stream()), "paged_attention_decode_mma")
        self._check(self.lib.rv_paged_attention_merge_ex(
            _ptr(scratch), _ptr(ctx_lens), _ptr(out), _code(out.dtype), c_int(n_reqs),
            c_int(max_ctx_len), c_int(num_heads), c_int(head_dim), win, c_int(split),
            _ptr(sinks), self._stream()), "paged_attention_merge")

    def paged_attention_general(self, qkv, num_heads, num_kv_heads, head_dim, k_cache, v_cache,
                                ctx, group, scale, window, out):
        """Every token through the one-warp-per-(token, head) kernel."""
        self._check(self.lib.rv_paged_attention_warp(
            _ptr(qkv), _code(qkv.dtype), c_int(qkv.shape[1]), _ptr(k_cache), _ptr(v_cache),
            _ptr(group.block_table), c_int(group.max_blocks), _ptr(ctx.q_start),
            _ptr(ctx.ctx_lens), _ptr(ctx.token_req), _ptr(out), c_int(0), c_int(ctx.n_tokens),
            c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(group.page_size),
            c_float(scale), c_int(window if window else 0), self._stream()), "paged_attention")

    # ---- gated short convolution -----------------------------------------------------

    def short_conv(self, proj, filt, in_bias, conv_bias, state, ctx, out):
        self._need(proj, "in_proj rows")
        self._need(filt, "filter", torch.float32)
        self._need(out, "short_conv output", proj.dtype)
        hidden, taps = filt.shape
        if proj.shape[1] != 3 * hidden:
            raise KernelError("short_conv: in_proj rows must be three times the filter's width")
        if state is not None:
            self._need(state, "convolution state", torch.float32)
        self._check(self.lib.rv_short_conv(
            _ptr(proj), _code(proj.dtype), _ptr(filt), _ptr(in_bias), _ptr(conv_bias),
            _ptr(state), _ptr(ctx.q_start), _ptr(ctx.state_slot), _ptr(ctx.start_pos), _ptr(out),
            c_int(ctx.n_reqs), c_int(ctx.max_q_len), c_int(hidden), c_int(taps),
            self._stream()), "short_conv")

    # ---- SwiGLU ----------------------------------------------------------------------

    def swiglu(self, gate_up, out):
        self._need(gate_up, "gate|up rows")
        self._need(out, "swiglu output", gate_up.dtype)
        if gate_up.shape[1] != 2 * out.shape[1]:
            raise KernelError("swiglu: input rows must be twice the output's width")
        self._check(self.lib.rv_swiglu(_ptr(gate_up), _ptr(out), _code(out.dtype),
                                       c_int(out.shape[0]), c_int(out.shape[1]), self._stream()),
                    "swiglu")

    # ---- layer norm (alone, or with the addition into the stream) -----------------------

    def add_layernorm(self, resid, delta, weight, bias, eps, out, rows=None,
                      delta_weight=None, delta_bias=None, delta_eps=0.0):
        """out = LN(resid + d), d = delta or LN(delta; delta_weight, delta_bias, delta_eps);
        `resid` None: out = LN(delta).  The stream is updated unless `rows` selects rows."""
        if resid is not None:
            self._need(resid, "residual stream", torch.float32)
        elif delta is None or rows is not None or delta_weight is not None:
            raise KernelError("add_layernorm: without a stream it takes rows to normalise, all of them")
        self._need(weight, "norm weight", torch.float32)
        self._need(bias, "norm bias", torch.float32)
        self._need(out, "norm output")
        if delta is not None:
            self._need(delta, "pending sub-layer output")
            if resid is not None and delta.shape != resid.shape:
                raise KernelError("add_layernorm: the stream and the pending output differ in shape")
        if delta_weight is not None:
            self._need(delta_weight, "norm weight of the added rows", torch.float32)
            self._need(delta_bias, "norm bias of the added rows", torch.float32)
        if rows is not None:
            self._need(rows, "row list", torch.int32)
        n, hidden = out.shape
        if (resid if resid is not None else delta).shape[1] != hidden or weight.shape[0] != hidden \
                or bias.shape[0] != hidden:
            raise KernelError("add_layernorm: widths disagree")
        self._check(self.lib.rv_add_layernorm(
            _ptr(resid), _ptr(delta), _code(delta.dtype) if delta is not None else _F32,
            _ptr(delta_weight), _ptr(delta_bias), c_float(delta_eps), _ptr(weight), _ptr(bias),
            _ptr(out), _code(out.dtype), _ptr(rows), c_int(n), c_int(hidden), c_float(eps),
            self._stream()), "add_layernorm")

    # ---- xIELU -----------------------------------------------------------------------

    def xielu(self, z, act, out):
        self._need(z, "xielu input")
        self._need(out, "xielu output", z.dtype)
        self._need(act, "xielu constants", torch.float32)
        if z.shape != out.shape or act.numel() != 2:
            raise KernelError("xielu: shapes disagree")
        self._check(self.lib.rv_xielu_act(_ptr(z), _ptr(act), _ptr(out), _code(out.dtype),
                                          c_int(out.shape[0]), c_int(out.shape[1]),
                                          self._stream()), "xielu")

    # ---- minGRU scan -----------------------------------------------------------------

    def mingru_scan(self, proj, bias, state, ctx, out):
        self._need(proj, "z|x|g rows", torch.float32)
        self._need(bias, "z|x biases", torch.float32)
        self._need(state, "recurrent state", torch.float32)
        self._need(out, "mingru output")
        width = out.shape[1]
        if proj.shape[1] != 3 * width or bias.shape[0] != 2 * width or state.shape[1] != width:
            raise KernelError("mingru_scan: widths disagree")
        self._check(self.lib.rv_mingru_scan(
            _ptr(proj), _ptr(bias), _ptr(state), _ptr(ctx.q_start), _ptr(ctx.state_slot), _ptr(out),
            _code(out.dtype), c_int(ctx.n_reqs), c_int(ctx.max_q_len), c_int(width),
            self._stream()), "mingru_scan")

    # ---- partial rotation + cache write ------------------------------------------------

    def rope_partial_write(self, rows, num_heads, num_kv_heads, head_dim, v_head_dim, freq,
                           positions, slot_mapping, k_cache, v_cache):
        self._need(rows, "q|k|v rows")
        if k_cache is not None:
            self._need(k_cache, "key pages", rows.dtype)
            self._need(v_cache, "value pages", rows.dtype)
        inv, dims = freq if freq is not None else (None, 0)
        if inv is not None:
            self._need(inv, "rotation frequencies", torch.float32)
            if inv.shape[0] != dims // 2:
                raise KernelError("rope_partial_write: one frequency per pair of turning dimensions")
        self._check(self.lib.rv_rope_partial_write(
            _ptr(rows), _code(rows.dtype), c_int(rows.shape[1]), c_int(rows.shape[0]),
            c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(v_head_dim), _ptr(inv),
            c_int(dims), _ptr(positions), _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache),
            self._stream()), "rope_partial_write")

    # ---- attention with mixed heads ------------------------------------------------------

    def paged_attention_mixed(self, rows, gate_off, num_heads, num_kv_heads, head_dim, v_head_dim,
                              k_cache, v_cache, ctx, group, scale, window, chunk, head_mix, sinks,
                              out):
        self._need(rows, "query rows")
        self._need(out, "attention output", rows.dtype)
        self._need(k_cache, "key pages", rows.dtype)
        self._need(v_cache, "value pages", rows.dtype)
        if head_mix is not None:
            self._need(head_mix, "head mixing matrix", torch.float32)
        if sinks is not None:
            self._need(sinks, "sinks", torch.float32)
        if out.shape[1] != num_heads * v_head_dim:
            raise KernelError("paged_attention_mixed: output width and head sizes disagree")
        nd = ctx.n_decode
        # (the tensor-core kernel would take single tokens as portions of one token, but fifteen
        # of a tile's sixteen rows are then idle; measured slower than the split kernel)
        tensor = ctx.n_tokens > nd and self._mixed_mma_ok(rows, num_heads, num_kv_heads, head_dim,
                                                          v_head_dim, gate_off)
        # single tokens, and everything the tensor-core kernel does not take: one block a token
        def simt(first, count, scratch=None, span=0):
            self._check(self.lib.rv_paged_attention_mixed(
                _ptr(rows), _code(rows.dtype), c_int(rows.shape[1]), c_int(gate_off), _ptr(k_cache),
                _ptr(v_cache), _ptr(group.block_table), c_int(group.max_blocks), _ptr(ctx.q_start),
                _ptr(ctx.ctx_lens), _ptr(ctx.token_req), _ptr(out), c_int(first), c_int(count),
                c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(v_head_dim),
                c_int(group.page_size), c_float(scale), c_int(window if window else 0),
                c_int(chunk if chunk else 0), _ptr(head_mix), _ptr(sinks), _ptr(scratch),
                c_longlong(scratch.numel() if scratch is not None else 0), c_int(span),
                self._stream()), "paged_attention_mixed")

        el = rows.element_size()
        staged = (num_kv_heads * head_dim * el) % 8 == 0 and (num_kv_heads * v_head_dim * el) % 8 == 0 \
            and head_dim % 2 == 0 and v_head_dim % 2 == 0 \
            and 4 * (num_heads * (head_dim + num_heads + 110) + 8 * num_kv_heads
                     * (head_dim + v_head_dim) * el + 512) <= 200 * 1024
        if nd > 0 and staged:
            # single tokens: each split over the keys it sees, then put together
            span = self._mixed_span(ctx.max_ctx_len, window, chunk)
            need = self.attention_mixed_scratch_bytes(nd, num_heads, v_head_dim, span)
            simt(0, nd, self._scratch_buffer(need, rows.device), span)
            self.launches += 1
        elif nd > 0:
            simt(0, nd)                    # rows that cannot be staged: one block a token
        if ctx.n_tokens > nd and not tensor:
            simt(nd, ctx.n_tokens - nd)
        if tensor:
            lib = self._mixed_lib(head_dim, v_head_dim)
            tag = f"{head_dim}_{v_head_dim}"
            # too few blocks for the GPU (a block is 16 tokens): every block's keys are shared out
            # over `parts` blocks, one per stretch of positions, and a merge puts them together
            n_prompt = ctx.n_tokens - nd
            tiles = -(-n_prompt // 16)
            parts = min(16, -(-3 * self._sm_count // max(1, tiles)))
            scratch, stretch, n_stretch = None, 0, 0
            if parts >= 2 and os.environ.get("RVLLM_MIXED_SHARE", "1") != "0":
                span = self._mixed_span(ctx.max_ctx_len, window, chunk) + 15
                stretch = max(128, -(-(-(-span // parts)) // 32) * 32)
                n_stretch = -(-span // stretch) + 1
                need = n_prompt * n_stretch * (2 * num_heads + num_heads * v_head_dim) * 4
                have = self._scratch.get(str(rows.device))
                if n_stretch < 2:
                    pass
                elif have is not None and have.numel() >= need:
                    scratch = have
                elif not torch.cuda.is_current_stream_capturing():
                    scratch = self._scratch_buffer(need, rows.device)
            rc = getattr(lib, f"rv_attention_mixed_mma_d{tag}")(
                _ptr(rows), c_int(rows.shape[1]), c_int(gate_off), _ptr(k_cache), _ptr(v_cache),
                _ptr(group.block_table), c_int(group.max_blocks), _ptr(ctx.q_start),
                _ptr(ctx.ctx_lens), _ptr(out), c_int(nd), c_int(ctx.n_reqs - nd),
                c_int(ctx.max_q_len), c_int(num_heads), c_int(num_kv_heads),
                c_int(group.page_size), c_float(scale), c_int(window if window else 0),
                c_int(chunk if chunk else 0), _ptr(head_mix), _ptr(sinks), _ptr(scratch),
                c_int(stretch), c_int(n_stretch), c_int(nd), self._stream())
            self.launches += 1
            if rc != 0:
                msg = getattr(lib, f"rv_attention_mixed_mma_last_error_d{tag}")().decode()
                raise KernelError(f"paged_attention_mixed: {msg}")
            if scratch is not None:
                self._check(self.lib.rv_paged_attention_mixed_merge(
                    _ptr(scratch), c_int(n_stretch), _ptr(rows), _code(rows.dtype),
                    c_int(rows.shape[1]), c_int(gate_off), _ptr(ctx.q_start), _ptr(ctx.ctx_lens),
                    _ptr(ctx.token_req), _ptr(out), c_int(nd), c_int(n_prompt), c_int(num_heads),
                    c_int(v_head_dim), c_int(window if window else 0), c_int(chunk if chunk else 0),
                    _ptr(sinks), c_int(stretch), c_int(16), self._stream()),
                    "paged_attention_mixed_merge")

    @staticmethod
    def _mixed_span(max_ctx_len, window, chunk) -> int:
        """The most keys a token can see."""
        span = max(1, int(max_ctx_len))
        if window:
            span = min(span, window)
        if chunk:
            span = min(span, chunk)
        return span

    def attention_mixed_scratch_bytes(self, n_tokens, num_heads, v_head_dim, span) -> int:
        """Scratch of the split launch for `n_tokens` single tokens that see `span` keys at most."""
        return int(self.lib.rv_paged_attention_mixed_scratch_bytes(
            c_int(n_tokens), c_int(num_heads), c_int(v_head_dim), c_int(span)))

    def _mixed_mma_ok(self, rows, num_heads, num_kv_heads, head_dim, v_head_dim, gate_off) -> bool:
        """Whether prompt portions go to the tensor-core kernel (attention_mixed_mma.cu):
        bfloat16, head counts in multiples of 8 up to 32, sizes in multiples of 16, and a
        block's tiles within shared memory.  RVLLM_MIXED_ATTENTION=simt: never."""
        if os.environ.get("RVLLM_MIXED_ATTENTION", "auto") == "simt":
            return False
        if rows.dtype != torch.bfloat16 or num_heads % 8 or num_heads > 32:
            return False
        if head_dim % 16 or v_head_dim % 16 or head_dim > 256 or v_head_dim > 256:
            return False
        if rows.shape[1] % 2 or (gate_off >= 0 and gate_off % 2):
            return False
        smem = 32 * (num_kv_heads * (head_dim + v_head_dim) + 16) * 2 \
            + num_heads * 16 * 40 * 4 + 16 * (num_heads * head_dim + 8) * 2 \
            + num_heads * num_heads * 8 + num_heads * 192
        return smem <= 227 * 1024

    def _mixed_lib(self, head_dim: int, v_head_dim: int):
        """The tensor-core mixed-head attention library for these sizes, built at first use."""
        key = ("mixed", head_dim, v_head_dim)
        lib = self._attn_libs.get(key)
        if lib is None:
            tag = f"{head_dim}_{v_head_dim}"
            path = build_variant("attention_mixed_mma.cu", {"RV_D": head_dim, "RV_DV": v_head_dim},
                                 f"attnmix_d{tag}", verbose=self._verbose_build)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load the kernel library {path}: {e}") from None
            getattr(lib, f"rv_attention_mixed_mma_last_error_d{tag}").restype = ctypes.c_char_p
            self._attn_libs[key] = lib
        return lib

    # ---- unit norm of q and k, query temperature, cache write ---------------------------

    def qk_unit_write(self, rows, num_heads, num_kv_heads, head_dim, v_head_dim, eps, q_temp,
                      positions, slot_mapping, k_cache, v_cache):
        """`eps` None: no norm; `q_temp` = (coef, every) or None."""
        self._need(rows, "q|k|v rows")
        if k_cache is not None:
            self._need(k_cache, "key pages", rows.dtype)
            self._need(v_cache, "value pages", rows.dtype)
        coef, every = q_temp if q_temp is not None else (0.0, 0)
        self._check(self.lib.rv_qk_unit_write(
            _ptr(rows), _code(rows.dtype), c_int(rows.shape[1]), c_int(rows.shape[0]),
            c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(v_head_dim),
            c_int(0 if eps is None else 1), c_float(eps or 0.0), c_float(coef), c_int(every),
            _ptr(positions), _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), self._stream()),
            "qk_unit_write")

    # ---- latent rows: norm and cache write; the gate on the heads -------------------------

    def latent_norm_write(self, rows, offset, rank, weight, eps, slot_mapping, cache):
        self._need(rows, "q|gate|latent rows")
        self._need(weight, "latent norm weight", torch.float32)
        self._need(cache, "latent pages", rows.dtype)
        if weight.shape[0] != rank or cache.shape[-1] * cache.shape[-2] != rank:
            raise KernelError("latent_norm_write: the rank and the pages disagree")
        self._check(self.lib.rv_latent_norm_write(
            _ptr(rows), _code(rows.dtype), c_int(rows.shape[1]), c_int(rows.shape[0]),
            c_int(offset), c_int(rank), _ptr(weight), c_float(eps), _ptr(slot_mapping),
            _ptr(cache), self._stream()), "latent_norm_write")

    def sigmoid_gate(self, x, rows, gate_off):
        self._need(x, "heads to gate")
        self._need(rows, "rows with the gate", x.dtype)
        self._check(self.lib.rv_sigmoid_gate(
            _ptr(x), _code(x.dtype), c_int(x.shape[0]), c_int(x.shape[1]), _ptr(rows),
            c_int(rows.shape[1]), c_int(gate_off), self._stream()), "sigmoid_gate")

    def heads_product(self, rows, offset, heads, size, w, out, gate_rows=None, gate_off=-1):
        """out[n, h, :] = rows[n, offset + h * size : + size] . w[h] for w [heads, size, b]: one
        small product per head, as one batched library product straight from and into the
        [tokens, heads * size] layouts (a head is a batch entry whose rows are strided); with
        `gate_rows` the result is then multiplied by sigmoid(gate_rows[n, gate_off + ...]).
        (A kernel of this library for few tokens, one block per head and eight tokens with
        the gate in the same pass, measured 10 us a call inside a captured step where the
        library's product takes 2; it is not kept.)"""
        n = rows.shape[0]
        b = w.shape[2]
        if n == 0:
            return
        self._need(w, "per-head matrices", rows.dtype)
        x = rows.as_strided((heads, n, size), (size, rows.stride(0), 1),
                            rows.storage_offset() + offset)
        y = out.as_strided((heads, n, b), (b, out.stride(0), 1), out.storage_offset())
        torch.bmm(x, w, out=y)
        self.launches += 1
        if gate_rows is not None:
            self.sigmoid_gate(out, gate_rows, gate_off)

    # ---- mixture of experts ---------------------------------------------------------------

    SCORE_MODES = {"sigmoid": 0, "softmax": 1}
    EXPERT_ACTIVATIONS = {"swiglu": 0, "glu_clamp": 1, "relu2": 2}

    def _choice_bias(self, choice_bias, experts):
        if choice_bias is not None:
            self._need(choice_bias, "choice bias", torch.float32)
            if choice_bias.shape != (experts,):
                raise KernelError("the choice bias has one number per expert")
        return _ptr(choice_bias)

    def moe_select(self, logits, groups, keep, group_top, weight_eps, ids, weights,
                   score="sigmoid", renormalize=True, route_scale=1.0, choice_bias=None):
        """`score`: how logits become scores ("sigmoid", or "softmax" over all experts);
        `renormalize` false: the chosen scores are not divided by their sum; every weight is
        multiplied by `route_scale`; `choice_bias` float32 [experts] is added to the scores
        where experts are compared, not where they are weighed."""
        self._need(logits, "router logits", torch.float32)
        self._need(ids, "expert ids", torch.int32)
        self._need(weights, "expert weights", torch.float32)
        n, experts = logits.shape
        self._check(self.lib.rv_moe_select(
            _ptr(logits), c_int(n), c_int(experts), c_int(ids.shape[1]), c_int(groups),
            c_int(keep), c_int(group_top), c_float(weight_eps), _ptr(ids), _ptr(weights),
            c_int(self.SCORE_MODES[score]), c_int(1 if renormalize else 0), c_float(route_scale),
            self._choice_bias(choice_bias, experts), self._stream()), "moe_select")

    def moe_route(self, x, router, groups, keep, group_top, weight_eps, ids, weights,
                  score="sigmoid", renormalize=True, route_scale=1.0, choice_bias=None):
        """The router's product (float32 `router` [experts, width], float32 sums) and the
        choice of `moe_select`, in one kernel."""
        self._need(x, "feed-forward input")
        self._need(router, "router matrix", torch.float32)
        self._need(ids, "expert ids", torch.int32)
        self._need(weights, "expert weights", torch.float32)
        experts, width = router.shape
        if x.shape[1] != width:
            raise KernelError("moe_route: widths disagree")
        self._check(self.lib.rv_moe_route(
            _ptr(x), _code(x.dtype), _ptr(router), c_int(x.shape[0]), c_int(width), c_int(experts),
            c_int(ids.shape[1]), c_int(groups), c_int(keep), c_int(group_top), c_float(weight_eps),
            _ptr(ids), _ptr(weights), c_int(self.SCORE_MODES[score]),
            c_int(1 if renormalize else 0), c_float(route_scale),
            self._choice_bias(choice_bias, experts), self._stream()), "moe_route")

    def moe_experts(self, x, ids, weights, gate_up, down, out, activation="swiglu", limit=0.0,
                    alpha=1.0, addend=None):
        """out[t] = sum_k weights[t, k] * down[e](act(gate[e] x_t, up[e] x_t)), e = ids[t, k];
        gate_up [E, 2F, W] (gate and up rows alternating), down [E, W, F].  `activation`
        "swiglu": silu(gate) * up; "glu_clamp": g = min(gate, limit), u = clamp(up, -limit,
        limit), g * sigmoid(alpha g) * (u + 1); "relu2": experts without a gate, `gate_up` is
        the up matrices [E, F, W] and the activation max(., 0)^2.  `addend` [N, W]: rows each sum
        starts from."""
        act_mode = self.EXPERT_ACTIVATIONS[activation]
        if addend is not None:
            self._need(addend, "rows added to the experts' output", x.dtype)
            if addend.shape != out.shape:
                raise KernelError("moe_experts: the added rows and the output differ in shape")
        self._need(x, "feed-forward input")
        self._need(gate_up, "experts' gate and up matrices", x.dtype)
        self._need(down, "experts' down matrices", x.dtype)
        self._need(out, "feed-forward output", x.dtype)
        n, top = ids.shape
        experts, width, ffn = down.shape
        first_rows = ffn if activation == "relu2" else 2 * ffn
        if gate_up.shape != (experts, first_rows, width) or x.shape[1] != width:
            raise KernelError("moe_experts: shapes disagree")
        grouped = (x.dtype == torch.bfloat16 and width % 8 == 0 and ffn % 8 == 0
                   and self.moe_mode != "simple"
                   and (self.moe_mode == "grouped" or n * top >= self.moe_grouped_min))
        if grouped:
            # the token tile follows the rows an expert gets on average
            avg = n * top / experts
            tn = 16 if avg <= 8 else 32 if avg <= 24 else 64 if avg <= 48 else 128
            need = int(self.lib.rv_moe_grouped_scratch_bytes(
                c_int(n), c_int(top), c_int(experts), c_int(width), c_int(ffn), c_int(tn)))
            scratch = torch.empty(need, dtype=torch.uint8, device=x.device)
            self._check(self.lib.rv_moe_experts_grouped(
                _ptr(x), _ptr(ids), _ptr(weights), _ptr(gate_up), _ptr(down), _ptr(out),
                _ptr(scratch), c_longlong(need), _ptr(self._gemm_status(x.device)), c_int(n),
                c_int(top), c_int(experts), c_int(width), c_int(ffn), c_int(tn), c_int(act_mode),
                c_float(limit), c_float(alpha), _ptr(addend), self._stream()),
                "moe_experts_grouped")
            self.launches += 4
            return
        act = torch.empty((n * top, ffn), dtype=x.dtype, device=x.device)
        self._check(self.lib.rv_moe_experts_simple(
            _ptr(x), _code(x.dtype), _ptr(ids), _ptr(weights), _ptr(gate_up), _ptr(down),
            _ptr(act), _ptr(out), c_int(n), c_int(top), c_int(experts), c_int(width), c_int(ffn),
            c_int(act_mode), c_float(limit), c_float(alpha), _ptr(addend), self._stream()),
            "moe_experts")
        self.launches += 1

    # ---- hyper-connections -----------------------------------------------------------------

    def hyper_norm(self, src, dst, delta, mix, out_w, in_w, weight, eps, out, rows=None):
        """The step between two sub-layers of a block with several residual streams:
        x'_t = sum_s mix[s, t] x_s + out_w[t] delta (skipped without `delta`), written to `dst`
        [N, S, W] when given; u = sum_t in_w[t] x'_t (`in_w` None: the plain sum); `out` =
        RMSNorm(u) with `weight`.  `src` is [N, S, W] or, before the streams differ, [N, W].
        With `rows` only those rows are read and nothing is written back."""
        self._need(src, "residual streams", torch.float32)
        self._need(weight, "norm weight", torch.float32)
        self._need(out, "norm output")
        n_out, width = out.shape
        if dst is not None:
            self._need(dst, "residual streams", torch.float32)
            streams = dst.shape[1]
        else:
            streams = src.shape[1] if src.dim() == 3 else (in_w.shape[0] if in_w is not None else 1)
        for t, what in ((mix, "mixing matrix"), (out_w, "output weights"), (in_w, "input weights")):
            if t is not None:
                self._need(t, what, torch.float32)
        if delta is not None:
            self._need(delta, "pending sub-layer output")
        if rows is not None:
            self._need(rows, "row list", torch.int32)
        if src.shape[-1] != width or weight.shape[0] != width:
            raise KernelError("hyper_norm: widths disagree")
        self._check(self.lib.rv_hyper_norm(
            _ptr(src), c_int(streams if src.dim() == 3 else 1), _ptr(dst), _ptr(delta),
            _code(delta.dtype) if delta is not None else _F32, _ptr(mix), _ptr(out_w), _ptr(in_w),
            _ptr(weight), _ptr(out), _code(out.dtype), _ptr(rows), c_int(n_out), c_int(streams),
            c_int(width), c_float(eps), self._stream()), "hyper_norm")

    # ---- whole-projection q/k norm + pairwise rotation + value mixing + cache write --------

    def qkv_full_norm_rope_write(self, rows, bias, num_heads, num_kv_heads, head_dim, v_head_dim,
                                 q_weight, k_weight, eps, freq, rot_dims, positions, slot_mapping,
                                 q_out, k_cache, v_cache, v_first_in=None, v_first_out=None,
                                 lam=None):
        """`rows` float32 [N, (heads + kv) * head_dim + kv * v_head_dim] (+ `bias`): q and k are
        normalised over their whole projection (weights [heads * head_dim], [kv * head_dim]),
        the pairs (2i, 2i + 1) of each head's first `rot_dims` dimensions turn by position *
        freq[i]; v <- (1 - lam) v + lam v_first_in when given (`lam` a float32 scalar tensor);
        `v_first_out` receives this layer's own values.  q -> `q_out`, k and v -> the cache."""
        self._need(rows, "q|k|v rows", torch.float32)
        self._need(q_out, "query rows", k_cache.dtype)
        for t, what in ((bias, "bias"), (q_weight, "query norm weight"), (k_weight, "key norm weight"),
                        (freq, "rotation frequencies"), (v_first_in, "first values"),
                        (v_first_out, "first values"), (lam, "mixing weight")):
            if t is not None:
                self._need(t, what, torch.float32)
        total = (num_heads + num_kv_heads) * head_dim + num_kv_heads * v_head_dim
        if rows.shape[1] != total or q_out.shape[1] != num_heads * head_dim:
            raise KernelError("qkv_full_norm_rope_write: row width and head sizes disagree")
        self._check(self.lib.rv_qkv_full_norm_rope_write(
            _ptr(rows), _ptr(bias), _ptr(q_weight), _ptr(k_weight), c_float(eps), _ptr(freq),
            c_int(rot_dims), _ptr(positions), _ptr(slot_mapping), _ptr(q_out), _ptr(k_cache),
            _ptr(v_cache), _code(k_cache.dtype), _ptr(v_first_in), _ptr(v_first_out), _ptr(lam),
            c_int(rows.shape[0]), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
            c_int(v_head_dim), self._stream()), "qkv_full_norm_rope_write")

    # ---- gated delta rule ------------------------------------------------------------------

    def gated_delta_record(self, heads, kv_heads, dim, vdim, taps) -> int:
        """Floats of one request's record: convolution inputs, then the state."""
        return (taps - 1) * (2 * kv_heads * dim + heads * vdim) + heads * dim * vdim

    def gated_delta(self, proj, lowrank, filt, a_log, dt_bias, norm_w, state, ctx, out, heads,
                    kv_heads, dim, vdim, taps, unit_eps, eps):
        """The gated delta rule with a decay per key channel over the step's tokens; see
        csrc/gated_delta.cu for the layout of `proj`, `lowrank` and the record."""
        for t, what in ((proj, "projection rows"), (lowrank, "decay and gate rows"),
                        (filt, "convolution filters"), (a_log, "decay rates"),
                        (dt_bias, "decay bias"), (norm_w, "output norm weight"),
                        (state, "state records")):
            self._need(t, what, torch.float32)
        self._need(out, "mixer output")
        rec = self.gated_delta_record(heads, kv_heads, dim, vdim, taps)
        if state.shape[1] != rec or out.shape[1] != heads * vdim:
            raise KernelError("gated_delta: the record or the output has another size")
        n = proj.shape[0]
        need = self.lib.rv_gated_delta_scratch(c_int(n), c_int(heads), c_int(kv_heads), c_int(dim),
                                               c_int(vdim))
        if need < 0:
            raise KernelError(f"gated_delta: key heads of {dim} are not supported")
        scratch = torch.empty((need,), dtype=torch.float32, device=proj.device)
        self._check(self.lib.rv_gated_delta(
            _ptr(proj), c_int(proj.shape[1]), _ptr(lowrank), c_int(lowrank.shape[1]), _ptr(filt),
            _ptr(a_log), _ptr(dt_bias), _ptr(norm_w), _ptr(state), _ptr(ctx.token_req),
            _ptr(ctx.q_start), _ptr(ctx.state_slot), _ptr(scratch), _ptr(out), _code(out.dtype),
            c_int(n), c_int(ctx.n_reqs), c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim),
            c_int(taps), c_float(unit_eps), c_float(eps), self._stream()), "gated_delta")
        self.launches += 3

    # ---- clamped gated activation ----------------------------------------------------------

    def glu_clamp(self, gate_up, bias, out, limit, alpha):
        """out = g sigmoid(alpha g) (u + 1) with g = min(gate, limit), u = clamp(up, +-limit);
        `gate_up` [N, 2F] holds gate values then up values, `bias` float32 [2F] is added first."""
        self._need(gate_up, "gate|up rows")
        self._need(out, "activation output", gate_up.dtype)
        if bias is not None:
            self._need(bias, "bias", torch.float32)
        n, f = out.shape
        if gate_up.shape != (n, 2 * f):
            raise KernelError("glu_clamp: shapes disagree")
        self._check(self.lib.rv_glu_clamp(_ptr(gate_up), _ptr(bias), _ptr(out), _code(out.dtype),
                                          c_int(n), c_int(f), c_float(limit), c_float(alpha),
                                          self._stream()), "glu_clamp")

    # ---- relu squared; a sum of two mixers -------------------------------------------------

    def relu2(self, z, out):
        self._need(z, "activation input")
        self._need(out, "activation output", z.dtype)
        if z.shape != out.shape:
            raise KernelError("relu2: shapes disagree")
        self._check(self.lib.rv_relu2(_ptr(z), _ptr(out), _code(z.dtype), c_int(z.shape[0]),
                                      c_int(z.shape[1]), self._stream()), "relu2")

    def weighted_sum(self, a, sa, b, sb, out):
        """out = sa * a + sb * b, float32 arithmetic."""
        self._need(a, "first summand")
        self._need(b, "second summand", a.dtype)
        self._need(out, "sum", a.dtype)
        if a.shape != b.shape or a.shape != out.shape:
            raise KernelError("weighted_sum: shapes disagree")
        self._check(self.lib.rv_weighted_sum(_ptr(a), c_float(sa), _ptr(b), c_float(sb), _ptr(out),
                                             _code(a.dtype), c_longlong(a.numel()), self._stream()),
                    "weighted_sum")

    # ---- latent rows with a query latent and a turned key part ------------------------------

    def latent_prepare(self, rows, q_off, q_rank, q_weight, cq, kv_off, rank, rot, kv_weight, eps,
                       freq, positions, slot_mapping, cache):
        """Columns [q_off, +q_rank) of `rows` RMS-normed into `cq` (q_rank 0: none); columns
        [kv_off, +rank) RMS-normed and the `rot` columns after them turned by the position, both
        into the token's page slot [rank + rot]."""
        self._need(rows, "latent rows")
        self._need(kv_weight, "latent norm weight", torch.float32)
        self._need(cache, "latent pages", rows.dtype)
        if kv_weight.shape[0] != rank or cache.shape[-1] * cache.shape[-2] != rank + rot:
            raise KernelError("latent_prepare: the rank and the pages disagree")
        if q_rank:
            self._need(q_weight, "query latent norm weight", torch.float32)
            self._need(cq, "query latent rows", rows.dtype)
            if q_weight.shape[0] != q_rank or cq.shape != (rows.shape[0], q_rank):
                raise KernelError("latent_prepare: the query latent has another size")
        if rot:
            self._need(freq, "rotation frequencies", torch.float32)
            if freq.shape[0] != rot // 2:
                raise KernelError("latent_prepare: one frequency per turning pair")
        self._check(self.lib.rv_latent_prepare(
            _ptr(rows), _code(rows.dtype), c_int(rows.shape[1]), c_int(rows.shape[0]), c_int(q_off),
            c_int(q_rank), _ptr(q_weight), _ptr(cq), c_int(kv_off), c_int(rank), c_int(rot),
            _ptr(kv_weight), c_float(eps), _ptr(freq), _ptr(positions), _ptr(slot_mapping),
            _ptr(cache), self._stream()), "latent_prepare")

    def rope_heads(self, x, heads, size, off, rot, freq, positions):
        """In every head of x [N, heads * size] the `rot` values from `off` on turn by the
        token's position (dimension i with i + rot/2, angle position * freq[i])."""
        if not rot:
            return
        self._need(x, "rows to turn")
        self._need(freq, "rotation frequencies", torch.float32)
        if freq.shape[0] != rot // 2 or x.shape[1] < heads * size:
            raise KernelError("rope_heads: sizes disagree")
        self._check(self.lib.rv_rope_heads(
            _ptr(x), _code(x.dtype), c_int(x.shape[1]), c_int(x.shape[0]), c_int(heads), c_int(size),
            c_int(off), c_int(rot), _ptr(freq), _ptr(positions), self._stream()), "rope_heads")

    def head_gate(self, x, heads, size, rows, gate_off):
        """x[n, h, :] <- x[n, h, :] * sigmoid(rows[n, gate_off + h])."""
        self._need(x, "heads to gate")
        self._need(rows, "rows with the gates", x.dtype)
        if x.shape[1] != heads * size:
            raise KernelError("head_gate: sizes disagree")
        self._check(self.lib.rv_head_gate(
            _ptr(x), _code(x.dtype), c_int(x.shape[0]), c_int(heads), c_int(size), _ptr(rows),
            c_int(rows.shape[1]), c_int(gate_off), self._stream()), "head_gate")

    # ---- matrix memory with exponential gates ------------------------------------------------

    def mlstm_record(self, heads, dim, vdim) -> int:
        """Floats of one request's record: per head vdim + 1 columns of dim rows, then the maxima."""
        return heads * (vdim + 1) * dim + heads

    def mlstm(self, rows, in_bias, forget_bias, norm_w, state, ctx, out, heads, dim, vdim, cap, eps):
        """The matrix memory over the step's tokens; see csrc/mlstm.cu for the layout of `rows`
        (q | k | v | i | f | g, float32) and of the record."""
        for t, what in ((rows, "projection rows"), (in_bias, "input gate bias"),
                        (forget_bias, "forget gate bias"), (norm_w, "output norm weight"),
                        (state, "state records")):
            self._need(t, what, torch.float32)
        self._need(out, "mixer output")
        if state.shape[1] != self.mlstm_record(heads, dim, vdim) or out.shape[1] != heads * vdim:
            raise KernelError("mlstm: the record or the output has another size")
        n = rows.shape[0]
        need = self.lib.rv_mlstm_scratch(c_int(n), c_int(heads), c_int(vdim))
        scratch = torch.empty((need,), dtype=torch.float32, device=rows.device)
        self._check(self.lib.rv_mlstm(
            _ptr(rows), c_int(rows.shape[1]), _ptr(in_bias), _ptr(forget_bias), _ptr(norm_w),
            _ptr(state), _ptr(ctx.token_req), _ptr(ctx.q_start), _ptr(ctx.state_slot),
            _ptr(scratch), _ptr(out), _code(out.dtype), c_int(n), c_int(ctx.n_reqs), c_int(heads),
            c_int(dim), c_int(vdim), c_float(cap), c_float(eps), self._stream()), "mlstm")
        self.launches += 2

    def softcap(self, logits, cap):
        self._need(logits, "logits", torch.float32)
        self._check(self.lib.rv_softcap(_ptr(logits), c_longlong(logits.numel()), c_float(cap),
                                        self._stream()), "softcap")

    # ---- sampling --------------------------------------------------------------------

    def argmax(self, logits):
        self._need(logits, "logits", torch.float32)
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        scratch = torch.empty(logits.shape[0] * 64 * 2, dtype=torch.int32, device=logits.device)
        self._check(self.lib.rv_argmax(_ptr(logits), _ptr(out), _ptr(scratch),
                                       c_longlong(scratch.numel() * 4), c_int(logits.shape[0]),
                                       c_int(logits.shape[1]), self._stream()), "argmax")
        self.launches += 1
        return out

    def sample(self, logits, temperature, top_p, seed, counter):
        """Rows with temperature <= 0 are greedy."""
        self._need(logits, "logits", torch.float32)
        self._need(temperature, "temperatures", torch.float32)
        self._need(top_p, "top-p values", torch.float32)
        self._need(seed, "seeds", torch.int64)
        self._need(counter, "counters", torch.int64)
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        self._check(self.lib.rv_sample(_ptr(logits), _ptr(temperature),
                                       _ptr(top_p), _ptr(seed), _ptr(counter), _ptr(out),
                                       c_int(logits.shape[0]), c_int(logits.shape[1]),
                                       self._stream()), "sample")
        return out
