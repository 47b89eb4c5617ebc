"""ctypes bindings of the CUDA kernels.

Every method takes torch CUDA tensors, launches on torch's current stream and
raises `KernelError` when the entry point refuses its arguments or the launch
fails.  There is no CPU path: without a CUDA device, or without the compiled
library, `get_kernels()` raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_float, c_void_p, c_char_p
from typing import List, Optional

import torch

from . import build

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported element type {dt}; the kernels take float32 and bfloat16")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def token_tile(rows: int) -> int:
    """The token tile (UMMA N) of the tensor-core product for a step of `rows` tokens: the
    smallest of 16, 32, 64, 128, 256 that holds them, 256 beyond.  The one place the ladder
    is written: the kernel is told the tile, and whoever sizes work by it asks here."""
    for t in (16, 32, 64, 128):
        if rows <= t:
            return t
    return 256


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """The weight layout of the SwiGLU epilogue: blocks of 32 rows, each the gate rows
    [16t, 16t+16) followed by the up rows [16t, 16t+16); rows past the true size are zero."""
    inter, k = gate.shape
    blocks = -(-inter // 16)
    g = torch.zeros((blocks * 16, k), dtype=gate.dtype, device=gate.device)
    u = torch.zeros_like(g)
    g[:inter] = gate
    u[:inter] = up
    return torch.cat([g.view(blocks, 16, k), u.view(blocks, 16, k)], dim=1).reshape(blocks * 32, k).contiguous()


PAIR_TOKEN_TILE = 256        # the token tile of the kernel that runs on pairs of SMs


class RowScale:
    """A row scale still to be applied: an RMSNorm whose rows were left unscaled (csrc/rowscale.cuh).
    `shares` [n, stride >= rows] float32 holds each row's sum of squares in n shares, as the kernel that
    wrote the rows left them; the scale of row r is rsqrt(sum over shares[:, r] / width + eps).  The
    product that reads the unscaled rows applies the scale to its own results (`in_scale`)."""

    def __init__(self, shares: torch.Tensor, width: int, eps: float) -> None:
        self.shares, self.width, self.eps = shares, int(width), float(eps)

    def args(self):
        return (self.shares.data_ptr(), self.shares.shape[0], self.shares.stride(0), float(self.width), self.eps)

    def values(self) -> torch.Tensor:
        """The scales themselves (for tests and for parts written in torch)."""
        return torch.rsqrt(self.shares.sum(0) / self.width + self.eps)


_NO_SCALE = (None, 0, 0, 0.0, 0.0)
_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)      # torch's own quick way to the stream handle


def _scale_args(scale: Optional["RowScale"]):
    return scale.args() if scale is not None else _NO_SCALE


class PartialProduct:
    """Partial products of a stream-k GEMM waiting in the workspace to be added up."""

    def __init__(self, workspace: torch.Tensor, plan, n_rows: int, w_rows: int,
                 rs_rows: Optional[torch.Tensor] = None) -> None:
        self.workspace, self.plan, self.n_rows, self.w_rows = workspace, plan, n_rows, w_rows
        # the scale of every row that the product's input still wants (float32 [n_rows], written by the
        # product's kernel from the RowScale it was given): the adding-up has to apply it
        self.rs_rows = rs_rows


class Kernels:
    """The loaded kernel library.  One instance per process (`get_kernels`)."""

    def __init__(self, verbose: bool = True) -> None:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: braidinfer_b200 runs on an NVIDIA B200 (sm_100a) only "
                              "and has no CPU path")
        major, minor = torch.cuda.get_device_capability()
        if major != 10:
            raise KernelError(f"the kernels are built for sm_100a; this device is sm_{major}{minor}")
        path = build.core_library(verbose=verbose)
        self.lib = ctypes.CDLL(str(path))
        self.path = str(path)
        self.launches = 0          # kernels launched through this object (for measurements)
        self._declare()
        self._device_index = torch.cuda.current_device()
        self._error_flag = torch.zeros(8, dtype=torch.int32, device="cuda")
        self._tc_workspace: Optional[torch.Tensor] = None
        self._attn_libs = {}
        self.pending_partial = None     # the open PartialProduct, if any (it owns the GEMM workspace)
        self.workspace_generation = 0   # grows when a scratch buffer moves (captured graphs are stale then)
        self._attn_partial: Optional[torch.Tensor] = None
        self._verbose = verbose

    # ------------------------------------------------------------------ plumbing
    def _declare(self) -> None:
        L = self.lib
        L.braid_last_error.restype = c_char_p
        L.braid_embed.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        L.braid_rmsnorm.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p]
        L.braid_silu_mul.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        L.braid_residual_add.argtypes = [c_void_p, c_void_p, c_int, c_longlong, c_void_p]
        L.braid_rope_kv_write.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_void_p, c_void_p]
        L.braid_cast.argtypes = [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p]
        L.braid_gather_i32.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        L.braid_gather_i32.restype = c_int
        L.braid_attn_simple.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_float, c_void_p, c_void_p]
        L.braid_gemm_simt.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                      c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p]
        scale = [c_void_p, c_int, c_longlong, c_float, c_float]        # RowScale.args()
        L.braid_gemm_tc.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int,
                                    c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, c_int,
                                    c_void_p] + scale + [c_void_p, c_void_p, c_void_p]
        L.braid_streamk_reduce_prep.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                c_longlong, c_int, c_void_p]
        L.braid_gemm_tc2.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                     c_longlong, c_longlong, c_longlong, c_int, c_void_p, c_void_p]
        L.braid_streamk_reduce.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_longlong,
                                           c_int, c_int, c_void_p, c_void_p]
        L.braid_streamk_reduce_norm.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                                c_void_p, c_int, c_int, c_float, c_void_p]
        L.braid_streamk_reduce_rope_kv.argtypes = [c_void_p] * 8 + [c_int] * 9 + [c_void_p, c_void_p, c_void_p]
        L.braid_gemm_tc_workspace_bytes.argtypes = [c_int, c_int, c_int, c_int]
        L.braid_gemm_tc_workspace_bytes.restype = c_longlong
        L.braid_logit_hash.argtypes = [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p]
        L.braid_logit_hash.restype = c_int
        L.braid_argmax.argtypes = [c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p, c_void_p]
        L.braid_sample.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int] + [c_void_p] * 12 + \
                                  [c_void_p, c_void_p]
        for name in ("braid_embed", "braid_rmsnorm", "braid_silu_mul", "braid_residual_add",
                     "braid_rope_kv_write", "braid_cast", "braid_attn_simple", "braid_gemm_simt",
                     "braid_gemm_tc", "braid_gemm_tc2", "braid_argmax", "braid_sample", "braid_streamk_reduce",
                     "braid_streamk_reduce_norm", "braid_streamk_reduce_rope_kv", "braid_streamk_reduce_prep",
                     "braid_streamk_reduce_prep_cols"):
            getattr(L, name).restype = c_int

    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            msg = self.lib.braid_last_error().decode(errors="replace")
            raise KernelError(f"{what}: {msg} (code {rc})")

    def _stream(self):
        """The current stream's handle (inside a graph capture: the capturing stream).  Asked for at every
        launch, so through the quick route where this torch has it."""
        if _RAW_STREAM is not None:
            return _RAW_STREAM(self._device_index)
        return torch.cuda.current_stream().cuda_stream

    def check_device_errors(self) -> None:
        """Read the flags that kernels raise (a cache write outside its pages, a
        tensor-core kernel whose bounded wait ran out, NaN logits) and raise on any.
        It synchronises the stream, so the step calls it where it reads results."""
        flags = self._error_flag.tolist()
        if any(flags):
            self._error_flag.zero_()
            names = ["cache write outside the sequence's pages", "tensor-core GEMM wait ran out",
                     "NaN among the logits",
                     "tcgen05 attention gave up (a wait ran out, a visible position had no page, or its shared "
                     "memory was not 1024-byte aligned)",
                     "attention met a visible position whose page is absent or outside the cache (it read page 0 "
                     "instead; the result is wrong)"]
            raise KernelError("device error: " + "; ".join(n for n, f in zip(names, flags) if f))

    # ------------------------------------------------------------------ row-wise kernels
    def logit_hash(self, logits: torch.Tensor) -> List[int]:
        """One 64-bit hash a row of float32 logits (FNV-1a over the elements' 32-bit patterns, the hash the
        reference logs under BRAIDINFER_LOGIT_TRACE): equal logits, equal hash, so the first step at which
        two runs part is found by comparing two short text files.  Synchronises."""
        if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
            raise KernelError("logit_hash wants float32 rows [n, vocab] with contiguous elements")
        n, vocab = logits.shape
        out = torch.empty(max(n, 1), dtype=torch.int64, device=logits.device)
        self.launches += 1
        self._check(self.lib.braid_logit_hash(logits.data_ptr(), logits.stride(0), n, vocab, out.data_ptr(),
                                              self._stream()), "logit_hash")
        return [v & 0xFFFFFFFFFFFFFFFF for v in out[:n].tolist()]

    def embed(self, table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
        n, hidden = out.shape
        self.launches += 1
        self._check(self.lib.braid_embed(table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(), out.data_ptr(),
                                         n, hidden, table.shape[0], self._stream()), "embed")

    def rmsnorm(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float,
                row_index: Optional[torch.Tensor] = None) -> None:
        rows, width = out.shape
        if x.dtype != torch.float32:
            raise KernelError("rmsnorm reads the float32 residual stream")
        self.launches += 1
        self._check(self.lib.braid_rmsnorm(x.data_ptr(), w.data_ptr(), dtype_code(w.dtype), out.data_ptr(),
                                           dtype_code(out.dtype), _ptr(row_index), rows, width, float(eps),
                                           self._stream()), "rmsnorm")

    def silu_mul(self, gu: torch.Tensor, out: torch.Tensor) -> None:
        rows, inter = out.shape
        self.launches += 1
        self._check(self.lib.braid_silu_mul(gu.data_ptr(), out.data_ptr(), dtype_code(out.dtype), rows, inter,
                                            self._stream()), "silu_mul")

    def residual_add(self, h: torch.Tensor, delta: torch.Tensor) -> None:
        self.launches += 1
        self._check(self.lib.braid_residual_add(h.data_ptr(), delta.data_ptr(), dtype_code(delta.dtype),
                                                h.numel(), self._stream()), "residual_add")

    def cast(self, src: torch.Tensor, dst: torch.Tensor) -> None:
        self.launches += 1
        self._check(self.lib.braid_cast(src.data_ptr(), dtype_code(src.dtype), dst.data_ptr(),
                                        dtype_code(dst.dtype), src.numel(), self._stream()), "cast")

    def gather_i32(self, src: torch.Tensor, index: torch.Tensor, dst: torch.Tensor) -> None:
        self.launches += 1
        self._check(self.lib.braid_gather_i32(src.data_ptr(), index.data_ptr(), dst.data_ptr(), index.numel(),
                                              self._stream()), "gather_i32")

    def rope_kv_write(self, qkv: torch.Tensor, inv_freq: torch.Tensor, positions: torch.Tensor,
                      token_seq: torch.Tensor, page_table: Optional[torch.Tensor], cache: Optional[torch.Tensor],
                      nqh: int, nkh: int, hd: int, rope_dim: int, adjacent: bool, page_size: int) -> None:
        rows = qkv.shape[0]
        cols = page_table.shape[1] if page_table is not None else 0
        num_pages = cache.shape[0] if cache is not None else 0
        self.launches += 1
        self._check(self.lib.braid_rope_kv_write(
            qkv.data_ptr(), dtype_code(qkv.dtype), inv_freq.data_ptr(), positions.data_ptr(), token_seq.data_ptr(),
            _ptr(page_table), _ptr(cache), rows, nqh, nkh, hd, rope_dim, int(adjacent), page_size, cols, num_pages,
            self._error_flag.data_ptr(), self._stream()), "rope_kv_write")

    def attn_simple(self, q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, page_table: torch.Tensor,
                    positions: torch.Tensor, token_seq: torch.Tensor, nqh: int, nkh: int, hd: int,
                    page_size: int, window: Optional[int], scale: float) -> None:
        """q: [rows, >= nqh*hd] (a view of the qkv rows is fine), out: [rows, nqh*hd]."""
        rows = out.shape[0]
        self.launches += 1
        self._check(self.lib.braid_attn_simple(
            q.data_ptr(), out.data_ptr(), dtype_code(out.dtype), cache.data_ptr(), page_table.data_ptr(),
            positions.data_ptr(), token_seq.data_ptr(), q.stride(0), out.stride(0), rows, nqh, nkh, hd,
            page_size, page_table.shape[1], cache.shape[0], int(window or 0), float(scale),
            self._error_flag.data_ptr() + 16, self._stream()),
            "attn_simple")

    @staticmethod
    def attn_mma_supports(head_dim: int) -> bool:
        return head_dim % 16 == 0 and 16 <= head_dim <= 256

    def attn_mma_library(self, head_dim: int):
        """The attention library for one head size, compiled at first use."""
        lib = self._attn_libs.get(head_dim)
        if lib is None:
            if not self.attn_mma_supports(head_dim):
                raise KernelError(f"the tensor-core attention takes head sizes in steps of 16 up to 256, not {head_dim}")
            lib = ctypes.CDLL(str(build.attention_library(head_dim, verbose=self._verbose)))
            lib.braid_last_error.restype = c_char_p
            lib.braid_attn_mma.restype = c_int
            lib.braid_attn_mma.argtypes = [c_void_p] * 9 + [c_int] * 13 + [c_float, c_void_p, c_void_p]
            lib.braid_attn_mma_partial_floats.restype = c_longlong
            lib.braid_attn_mma_partial_floats.argtypes = [c_int, c_int, c_int]
            lib.braid_attn_tc_supported.restype = c_int
            lib.has_tc = bool(lib.braid_attn_tc_supported())
            if lib.has_tc:
                lib.braid_attn_tc.restype = c_int
                lib.braid_attn_tc.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong] + [c_void_p] * 4 + [c_int] * 10 + \
                                             [c_float, c_void_p, c_void_p]
            lib.braid_attn_mma_decode_slots.restype = c_int
            lib.braid_attn_mma_decode_slots.argtypes = [c_int]
            lib.decode_slots = lib.braid_attn_mma_decode_slots(1)     # CTAs of the few-token kernel held at once
            self._attn_libs[head_dim] = lib
        return lib

    @staticmethod
    def _check_pages(cache: torch.Tensor) -> None:
        """The tensor-core attention kernels tile pages at compile time (csrc/page.h)."""
        if cache.dim() != 5 or cache.shape[3] != build.page_size():
            raise KernelError(f"the tensor-core attention reads a cache [pages, 2, kv_heads, {build.page_size()}, "
                              f"head_dim]; got {tuple(cache.shape)}")

    @staticmethod
    def attn_tc_supports(head_dim: int) -> bool:
        return head_dim in (64, 128)

    def attn_tc(self, q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, page_table: torch.Tensor,
                q_start: torch.Tensor, q_len: torch.Tensor, kv_before: torch.Tensor, n_seqs: int, max_q_len: int,
                nqh: int, nkh: int, hd: int, window: Optional[int], scale: float) -> None:
        """bfloat16 attention of prompts over the cache on tcgen05 (head sizes 64 and 128)."""
        lib = self.attn_mma_library(hd)
        self._check_pages(cache)
        if not lib.has_tc:
            raise KernelError(f"the tcgen05 attention is built for head sizes 64 and 128, not {hd}")
        self.launches += 1
        cache_rows = cache.shape[0] * cache.shape[1] * cache.shape[2] * cache.shape[3]
        rc = lib.braid_attn_tc(q.data_ptr(), out.data_ptr(), cache.data_ptr(), cache_rows, page_table.data_ptr(),
                               q_start.data_ptr(), q_len.data_ptr(), kv_before.data_ptr(), q.stride(0), out.stride(0),
                               out.shape[0], n_seqs, max_q_len, nqh, nkh, hd, page_table.shape[1], int(window or 0),
                               float(scale), self._error_flag.data_ptr() + 12, self._stream())
        if rc != 0:
            raise KernelError(f"attn_tc: {lib.braid_last_error().decode(errors='replace')} (code {rc})")

    def attn_decode_slots(self, head_dim: int) -> int:
        return self.attn_mma_library(head_dim).decode_slots

    def attn_mma(self, q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, page_table: torch.Tensor,
                 q_start: torch.Tensor, q_len: torch.Tensor, kv_before: torch.Tensor, token_seq: torch.Tensor,
                 n_seqs: int, max_q_len: int, nqh: int, nkh: int, hd: int, window: Optional[int], scale: float,
                 n_splits: int = 1, few_tokens: bool = False) -> None:
        """bfloat16 attention over the cache on the tensor cores; `n_splits` > 1 slices the
        context (for steps of few tokens) and merges the slices in a second kernel."""
        lib = self.attn_mma_library(hd)
        self._check_pages(cache)
        rows = out.shape[0]
        partial = None
        if n_splits > 1:
            need = lib.braid_attn_mma_partial_floats(rows, nqh, n_splits)
            if self._attn_partial is None or self._attn_partial.numel() < need:
                self._attn_partial = torch.empty(max(need, 1 << 22), dtype=torch.float32, device="cuda")
                self.workspace_generation += 1
            partial = self._attn_partial
            self.launches += 1
        self.launches += 1
        rc = lib.braid_attn_mma(q.data_ptr(), out.data_ptr(), _ptr(partial), cache.data_ptr(), page_table.data_ptr(),
                                q_start.data_ptr(), q_len.data_ptr(), kv_before.data_ptr(), token_seq.data_ptr(),
                                q.stride(0), out.stride(0), rows, n_seqs, max_q_len, nqh, nkh, hd,
                                page_table.shape[1], cache.shape[0], int(window or 0), n_splits,
                                1 if few_tokens else 0, float(scale), self._error_flag.data_ptr() + 16, self._stream())
        if rc != 0:
            raise KernelError(f"attn_mma: {lib.braid_last_error().decode(errors='replace')} (code {rc})")

    # ------------------------------------------------------------------ matrix products
    def gemm_simt(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, residual: Optional[torch.Tensor] = None) -> None:
        n, k = x.shape
        m = w.shape[0]
        if x.dtype != w.dtype:
            # the kernel reads both operands as one element type: a mixed call would read the
            # narrower operand past its end
            raise KernelError(f"gemm_simt: x is {x.dtype} and w is {w.dtype}; both operands must have one element type")
        if w.shape[1] != k or tuple(out.shape) != (n, m):
            raise KernelError(f"gemm_simt: shapes x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
        mode = 1 if residual is not None else 0
        self.launches += 1
        self._check(self.lib.braid_gemm_simt(x.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(residual),
                                             dtype_code(x.dtype), dtype_code(out.dtype), mode, n, m, k,
                                             x.stride(0), w.stride(0), out.stride(0), self._stream()), "gemm_simt")

    def tc_workspace(self, nbytes: int) -> torch.Tensor:
        if self._tc_workspace is None or self._tc_workspace.numel() * 4 < nbytes:
            self._tc_workspace = torch.empty(max((nbytes + 3) // 4, 1 << 22), dtype=torch.float32, device="cuda")
            self.workspace_generation += 1
        return self._tc_workspace

    def _stream_k_workspace(self, n: int, w_rows: int, k: int, block_n: int) -> torch.Tensor:
        need = self.lib.braid_gemm_tc_workspace_bytes(n, w_rows, k, block_n)
        if need < 0:
            raise KernelError(f"gemm_tc: no stream-k plan for {n} rows x {w_rows} x {k} with token tile {block_n}")
        return self.tc_workspace(need)

    def gemm_tc(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, residual: Optional[torch.Tensor] = None,
                swiglu: bool = False, block_n: int = 0, stream_k: bool = False,
                in_scale: Optional[RowScale] = None) -> None:
        """bfloat16 x [n, k] times w [m, k]^T on the tensor cores.  With `swiglu`, w holds
        gate and up rows interleaved in blocks of 16 (`interleave_gate_up`) and out is [n, I].  `stream_k` spreads the weight stream
        evenly over all SMs whatever the shape (for up to a few hundred tokens) and adds a reduce kernel.
        Whole tiles of more than 128 tokens run on pairs of SMs (`gemm_tc_pair`: faster at every
        measured size, and bit for bit the same result) unless `block_n` names a token tile.
        `in_scale`: a row scale that x still wants; the store and SwiGLU epilogues apply it to their results."""
        n, k = x.shape
        if not stream_k and block_n == 0 and token_tile(n) == PAIR_TOKEN_TILE and in_scale is None:
            return self.gemm_tc_pair(x, w, out, residual=residual, swiglu=swiglu)
        w_rows = w.shape[0]
        m = out.shape[1] if swiglu else w_rows
        if swiglu and w_rows != 2 * (-(-m // 16) * 16):
            raise KernelError(f"the SwiGLU epilogue wants {2 * (-(-m // 16) * 16)} interleaved weight rows for "
                              f"{m} outputs, got {w_rows} (see interleave_gate_up)")
        mode = 2 if swiglu else (1 if residual is not None else 0)
        block_n = block_n or token_tile(n)
        ws = None
        if stream_k:
            if self.pending_partial is not None:
                raise KernelError("a deferred sum still lives in the GEMM workspace; resolve it before the next "
                                  "stream-k product")
            ws = self._stream_k_workspace(n, w_rows, k, block_n)
            self.launches += 1
        self.launches += 1
        self._check(self.lib.braid_gemm_tc(x.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(residual), _ptr(ws),
                                           ws.numel() * 4 if ws is not None else 0,
                                           dtype_code(out.dtype), mode, n, m, k, x.stride(0), w.stride(0),
                                           out.stride(0), block_n, int(stream_k), None, *_scale_args(in_scale),
                                           _ptr(self._rs_rows(n, x.device) if stream_k and in_scale is not None else None),
                                           self._error_flag.data_ptr() + 4, self._stream()), "gemm_tc")

    @staticmethod
    def _rs_rows(n: int, device) -> torch.Tensor:
        """Room for every row's scale (a stream-k product with a row scale writes them for the adding-up)."""
        return torch.empty(-(-n // 4) * 4, dtype=torch.float32, device=device)

    def gemm_tc_pair(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
                     residual: Optional[torch.Tensor] = None, swiglu: bool = False, direct_out: bool = False) -> None:
        """As `gemm_tc` with whole tiles, on pairs of SMs: tiles of 256 weight rows x 256 tokens, each CTA of
        a pair loading half of both operands (tcgen05.mma.cta_group::2).  For prompts.  The output leaves
        through TMA stores (a TMA reduce-add for a residual summed in place) where it can be addressed so;
        `direct_out` makes every thread store its own elements instead, as it does anyway otherwise."""
        n, k = x.shape
        w_rows = w.shape[0]
        m = out.shape[1] if swiglu else w_rows
        if swiglu and w_rows != 2 * (-(-m // 16) * 16):
            raise KernelError(f"the SwiGLU epilogue wants {2 * (-(-m // 16) * 16)} interleaved weight rows for "
                              f"{m} outputs, got {w_rows} (see interleave_gate_up)")
        mode = 2 if swiglu else (1 if residual is not None else 0)
        self.launches += 1
        self._check(self.lib.braid_gemm_tc2(x.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(residual),
                                            dtype_code(out.dtype), mode, n, m, k, x.stride(0), w.stride(0),
                                            out.stride(0), int(direct_out), self._error_flag.data_ptr() + 4,
                                            self._stream()),
                    "gemm_tc_pair")

    def gemm_tc_partial(self, x: torch.Tensor, w: torch.Tensor, in_scale: Optional[RowScale] = None) -> "PartialProduct":
        """The stream-k product without its reduce: the partial products stay in the
        workspace, and the returned handle lets one of the `streamk_reduce*` calls add
        them up together with what follows.  Only one such handle may be open at a time."""
        if self.pending_partial is not None:
            raise KernelError("a deferred sum still lives in the GEMM workspace; resolve it first")
        n, k = x.shape
        w_rows = w.shape[0]
        block_n = token_tile(n)
        ws = self._stream_k_workspace(n, w_rows, k, block_n)
        plan = (c_int * 8)()
        rs = self._rs_rows(n, x.device) if in_scale is not None else None
        self.launches += 1
        self._check(self.lib.braid_gemm_tc(x.data_ptr(), w.data_ptr(), None, None, ws.data_ptr(), ws.numel() * 4,
                                           F32, 0, n, w_rows, k, x.stride(0), w.stride(0), 0, block_n, 1, plan,
                                           *_scale_args(in_scale), _ptr(rs),
                                           self._error_flag.data_ptr() + 4, self._stream()), "gemm_tc_partial")
        p = PartialProduct(ws, plan, n, w_rows, rs)
        self.pending_partial = p
        return p

    def _close_partial(self, p: "PartialProduct") -> None:
        if self.pending_partial is not p:
            raise KernelError("this partial product is not the one that lives in the workspace")
        self.pending_partial = None

    def streamk_reduce(self, p: "PartialProduct", out: torch.Tensor, residual: Optional[torch.Tensor] = None,
                       swiglu: bool = False) -> None:
        m = out.shape[1] if swiglu else p.w_rows
        mode = 2 if swiglu else (1 if residual is not None else 0)
        self._close_partial(p)
        self.launches += 1
        self._check(self.lib.braid_streamk_reduce(p.workspace.data_ptr(), p.plan, p.n_rows, out.data_ptr(), _ptr(residual),
                                                  m, out.stride(0), dtype_code(out.dtype), mode, _ptr(p.rs_rows),
                                                  self._stream()),
                    "streamk_reduce")

    def streamk_reduce_norm(self, p: "PartialProduct", h: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float,
                            row_index: Optional[torch.Tensor] = None) -> None:
        """h += sum of the partial products (written back unless rows are gathered), then
        out = RMSNorm(h) * w, in one kernel."""
        rows_out, width = out.shape
        if p.rs_rows is not None:
            raise KernelError("this partial product carries a row scale, which reduce + norm does not apply")
        self._close_partial(p)
        self.launches += 1
        self._check(self.lib.braid_streamk_reduce_norm(p.workspace.data_ptr(), p.plan, p.n_rows, h.data_ptr(), w.data_ptr(),
                                                       dtype_code(w.dtype), out.data_ptr(), dtype_code(out.dtype),
                                                       _ptr(row_index), rows_out, width, float(eps), self._stream()),
                    "streamk_reduce_norm")

    def streamk_reduce_rope_kv(self, p: "PartialProduct", qkv: torch.Tensor, inv_freq: torch.Tensor,
                               positions: torch.Tensor, token_seq: torch.Tensor, page_table: Optional[torch.Tensor],
                               cache: Optional[torch.Tensor], nqh: int, nkh: int, hd: int, rope_dim: int,
                               adjacent: bool, page_size: int) -> None:
        """qkv = sum of the partial products, rotated, keys and values into the cache."""
        cols = page_table.shape[1] if page_table is not None else 0
        num_pages = cache.shape[0] if cache is not None else 0
        self._close_partial(p)
        self.launches += 1
        self._check(self.lib.braid_streamk_reduce_rope_kv(
            p.workspace.data_ptr(), p.plan, qkv.data_ptr(), inv_freq.data_ptr(), positions.data_ptr(),
            token_seq.data_ptr(), _ptr(page_table), _ptr(cache), qkv.shape[0], nqh, nkh, hd, rope_dim, int(adjacent),
            page_size, cols, num_pages, _ptr(p.rs_rows), self._error_flag.data_ptr(), self._stream()),
            "streamk_reduce_rope_kv")

    def streamk_reduce_prep(self, p: Optional["PartialProduct"], h: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
                            eps: float) -> RowScale:
        """h += sum of the partial products (p None: h is complete), out = bfloat16(h * w), and the returned
        RowScale completes the RMSNorm of h with weights w: whoever multiplies `out` by a matrix applies it
        to its results (`in_scale`).  Many small CTAs instead of one per row."""
        rows, width = h.shape
        if out.dtype != torch.bfloat16 or h.dtype != torch.float32 or out.shape != h.shape:
            raise KernelError("reduce_prep reads the float32 residual stream and writes bfloat16 of the same shape")
        cols = self.lib.braid_streamk_reduce_prep_cols()
        shares = torch.empty((-(-width // cols), -(-rows // 4) * 4), dtype=torch.float32, device=h.device)
        if p is not None:
            if p.rs_rows is not None:
                raise KernelError("this partial product carries a row scale, which the residual sum does not apply")
            self._close_partial(p)
        self.launches += 1
        self._check(self.lib.braid_streamk_reduce_prep(
            p.workspace.data_ptr() if p is not None else None, p.plan if p is not None else None, rows, h.data_ptr(),
            w.data_ptr(), dtype_code(w.dtype), out.data_ptr(), shares.data_ptr(), shares.stride(0), width,
            self._stream()), "streamk_reduce_prep")
        return RowScale(shares, width, eps)

    @staticmethod
    def gemm_tc_eligible(x: torch.Tensor, w: torch.Tensor) -> bool:
        return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
                and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    # ------------------------------------------------------------------ token choice
    def argmax(self, logits: torch.Tensor, out: torch.Tensor) -> None:
        rows, vocab = logits.shape
        self.launches += 1
        self._check(self.lib.braid_argmax(logits.data_ptr(), logits.stride(0), out.data_ptr(), rows, vocab,
                                          self._error_flag.data_ptr() + 8, self._stream()), "argmax")

    def sample(self, logits: torch.Tensor, work: torch.Tensor, out: torch.Tensor, temperature: torch.Tensor,
               uniform: torch.Tensor, top_k=None, top_p=None, min_p=None, rep_penalty=None,
               hist_off=None, hist_tok=None, hist_cnt=None, bias_off=None, bias_tok=None, bias_val=None) -> None:
        rows, vocab = logits.shape
        self.launches += 1
        self._check(self.lib.braid_sample(
            logits.data_ptr(), work.data_ptr(), logits.stride(0), out.data_ptr(), rows, vocab,
            temperature.data_ptr(), _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(rep_penalty), uniform.data_ptr(),
            _ptr(hist_off), _ptr(hist_tok), _ptr(hist_cnt), _ptr(bias_off), _ptr(bias_tok), _ptr(bias_val),
            self._error_flag.data_ptr() + 8, self._stream()), "sample")


_KERNELS: Optional[Kernels] = None


def get_kernels(verbose: bool = True) -> Kernels:
    global _KERNELS
    if _KERNELS is None:
        _KERNELS = Kernels(verbose=verbose)
    return _KERNELS
