"""Python face of the CUDA kernel library (``csrc/``), loaded with ctypes.

Every function takes torch tensors that already live on the GPU, passes their addresses and the
current CUDA stream to an ``extern "C"`` launcher, and raises ``KernelError`` if the launcher
refuses the sizes or the launch fails. There is no CPU implementation behind these functions and
no library stand-in: if the shared library cannot be built or loaded, the first call raises.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

STATUS_BITS = {1: "a token id outside the vocabulary", 2: "a cache slot or page id outside the pool",
               4: "a position outside the rotary table or beyond a block table", 8: "a bounded wait inside a kernel gave up"}


class KernelError(RuntimeError):
    pass


_lib = None
_lock = threading.Lock()
_c = ctypes
_P, _I, _LL, _F = _c.c_void_p, _c.c_int, _c.c_longlong, _c.c_float

_SIGNATURES = {
    "gb_embed": [_P, _I, _P, _P, _I, _I, _I, _P, _P],
    "gb_rmsnorm": [_P, _P, _P, _P, _I, _I, _I, _F, _P],
    "gb_rope_kv_write": [_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _LL, _I, _P, _P],
    "gb_swiglu": [_P, _P, _I, _I, _I, _P],
    "gb_copy_pages": [_P, _P, _P, _I, _LL, _LL, _I, _P],
    "gb_gemm_simt": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _LL, _LL, _LL, _P],
    "gb_attention_rows": [_P, _LL, _P, _LL, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _LL, _F, _I, _P, _P],
    "gb_sample": [_P, _LL, _P, _P, _P, _P, _I, _P, _P, _I, _I, _P],
    "gb_resolve_tokens": [_P, _P, _P, _I, _I, _P],
    "gb_attention_decode": [_P, _LL, _P, _LL, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _LL, _F, _I, _I, _P, _P,
                            _P, _P, _P],
    "gb_attention_decode_counters": [_I, _I, _I],
    "gb_gemm_stream_row_groups": [_I, _I, _I, _I],
    "gb_gemm_stream": [_P, _LL, _P, _LL, _P, _F, _P, _LL, _P, _LL, _I, _I, _I, _I, _P, _LL, _I, _P],
    "gb_gemm_stream_qkv": [_P, _LL, _P, _LL, _P, _F, _P, _LL, _P, _LL, _I, _I, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I,
                           _LL, _I, _P, _P, _LL, _I, _P],
    "gb_attention_decode_mma_pdl": [_P, _LL, _P, _LL, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _LL, _F, _I, _I, _P, _P,
                                    _P, _P, _I, _I, _I, _P],
    "gb_attention_decode_mma": [_P, _LL, _P, _LL, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _LL, _F, _I, _I, _P, _P, _P,
                                _P, _P],
    "gb_attention_decode_mma_supported": [_I, _I, _I],
    "gb_stream_marker": [_P],
    "gb_kv_prefetch": [_P, _P, _P, _I, _P, _P, _I, _I, _I, _LL, _LL, _I, _I, _P],
    "gb_attention_prefill": [_P, _LL, _P, _LL, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _LL, _F, _I, _P, _P],
    "gb_attention_prefill_supported": [_I, _I, _I, _I],
    "gb_gemm_tcgen05_qkv": [_P, _P, _P, _I, _I, _LL, _LL, _LL, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _LL, _I, _P, _P,
                            _P, _I, _F],
    "gb_gemm_tcgen05_qkv_supported": [_I],
    "gb_attention_prefill_tc": [_P, _LL, _I, _P, _LL, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _LL, _F, _I, _P, _P],
    "gb_attention_prefill_tc_supported": [_I, _I, _I, _I],
    "gb_gemm_tcgen05": [_P, _P, _P, _I, _I, _I, _I, _LL, _LL, _LL, _P, _P, _P, _P, _LL, _P, _P, _I, _F],
    "gb_gemm_tcgen05_column_tiles": [_I, _I, _I],
    "gb_gemm_tcgen05_supported": [_P, _P, _I, _I, _I, _LL, _LL],
    "gb_gemm_tcgen05_gated": [_P, _P, _P, _I, _I, _I, _LL, _LL, _LL, _P, _P, _P, _I, _F],
    "gb_program_encode_gemm": [_P, _P, _LL, _P, _LL, _P, _F, _P, _LL, _P, _LL, _I, _I, _I, _I],
    "gb_program_encode_gemm_qkv": [_P, _P, _LL, _P, _LL, _P, _F, _P, _LL, _P, _LL, _I, _I, _P, _I, _P, _P, _P, _P, _I, _I, _I,
                                   _I, _LL, _I, _P],
    "gb_program_encode_attention": [_P, _P, _LL, _P, _LL, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _LL, _F, _I, _I, _P, _P,
                                    _P, _P, _I],
    "gb_program_launch": [_P, _I, _I, _I, _I, _I, _I, _P, _P, _I, _P],
    "gb_program_launch_with_absent_blocks": [_P, _I, _I, _I, _I, _I, _I, _P, _P, _I, _LL, _P],
    "gb_program_launch_traced": [_P, _I, _I, _I, _I, _I, _I, _P, _P, _I, _P, _P],
    "gb_step_io": [_P, _P, _LL, _P, _P, _P, _LL, _P],
    "gb_program_op_bytes": [],
    "gb_program_max_rows": [],
}


def lib():
    """The loaded shared library; builds it at first use."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = _build.ensure_built()
            try:
                handle = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load the CUDA kernel library {path}: {e}") from None
            handle.gb_last_error.restype = ctypes.c_char_p
            handle.gb_last_error.argtypes = []
            for name, args in _SIGNATURES.items():
                fn = getattr(handle, name, None)
                if fn is None:
                    raise KernelError(f"{path} does not export {name}; rebuild it (csrc/build.py --force)")
                fn.argtypes = args
                fn.restype = ctypes.c_int
            handle.gb_set_pdl.argtypes = [ctypes.c_int]
            handle.gb_set_pdl.restype = None
            handle.gb_set_pdl(7 if USE_PDL else 0)
            _lib = handle
    return _lib


def step_io(host_meta_ptr: int, dev_meta: torch.Tensor, meta_bytes: int, graph_exec: int, sampled_dev: torch.Tensor,
            sampled_host: torch.Tensor, count: int, nodes: int) -> None:
    """A recorded decode step's traffic in one native call: metadata to the device, the graph, ``count`` sampled tokens
    back to pinned host memory; nothing is waited for. ``nodes``: the graph's kernel count, for ``launch_count``."""
    global launch_count
    rc = lib().gb_step_io(host_meta_ptr, dev_meta.data_ptr(), meta_bytes, graph_exec, sampled_dev.data_ptr(),
                          sampled_host.data_ptr(), 4 * count, _stream())
    if rc != 0:
        raise KernelError(lib().gb_last_error().decode("utf-8", "replace") or "gb_step_io failed")
    launch_count += nodes


def loaded_library_path() -> Optional[str]:
    return _build.library_path() if _lib is not None else None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


#: kernels launched through this module since import (graph replays add their node count)
launch_count = 0


def _call(name: str, *args) -> None:
    global launch_count
    if _program is not None:
        _program.flush()          # a kernel that is launched now must come after what was recorded before it
    launch_count += 1
    rc = getattr(lib(), name)(*args)
    if rc != 0:
        raise KernelError(lib().gb_last_error().decode("utf-8", "replace") or f"{name} failed with code {rc}")


# -------------------------------------------------------------------------------------- decode programs
BY_ROWS, BY_OPERATIONS = 0, 1
#: the default way in which a program's persistent kernel shares the work (see ``Program.how``)
PROGRAM_HOW = BY_ROWS


class Program:
    """A chain of small decode kernels written down as operations and run by one persistent kernel
    (``csrc/decode_program.cu``). While a program is open (``program_begin`` .. ``program_end``), the products of at
    most ``max_rows`` rows that ``gemm_stream`` / ``gemm_stream_qkv`` would launch and the attention that
    ``attention_decode_mma`` would launch are appended to it instead; any other kernel launched through this module
    first runs what has been recorded so far, so the order of the work never changes. Nothing here knows what the
    operations belong to: parts call the same functions as ever.

    A program object remembers the operation arrays it has run (one per flush of a step, in order). When a step
    records exactly the same operations again (same buffers, same shapes: the second run of a step that is being
    recorded into a CUDA graph, or the next step of the same shape), the copy on the device is reused."""

    def __init__(self):
        handle = lib()
        self.op_bytes = int(handle.gb_program_op_bytes())
        self.max_rows = int(handle.gb_program_max_rows())
        self.segments = []
        self.cursor = 0
        self.absent_blocks, self.wait_cycles = 0, 0
        self.trace_next, self.traces = False, []
        #: how the persistent kernel shares the work: BY_ROWS (a thread-block cluster per group of rows runs the whole
        #: program for them) or BY_OPERATIONS (all resident blocks share each operation and meet at a barrier)
        self.how = PROGRAM_HOW
        self._buf = ctypes.create_string_buffer(self.op_bytes)
        self._reset()

    def _reset(self):
        self._pending, self._n, self._rows, self._hd, self._bk, self._max_vblocks, self._max_k = [], 0, 0, 0, 0, 1, 8
        self._status = None

    def start_step(self):
        self.cursor = 0
        self._reset()

    def _add(self, name, vblocks, rows, k, *args):
        rc = getattr(lib(), name)(ctypes.addressof(self._buf), *args)
        if rc != 0:
            raise KernelError(lib().gb_last_error().decode("utf-8", "replace") or f"{name} failed with code {rc}")
        self._pending.append(self._buf.raw)
        self._n += 1
        self._rows = max(self._rows, rows)
        self._max_vblocks = max(self._max_vblocks, vblocks)
        self._max_k = max(self._max_k, k)

    #: a product whose weights are larger than this is launched by itself (all SMs stream it) instead of recorded: in a
    #: program shared by rows a cluster would have to stream it alone
    MAX_WEIGHT_BYTES = 12 << 20

    def takes_rows(self, rows: int) -> bool:
        return 1 <= rows <= self.max_rows

    def takes_product(self, rows: int, w: torch.Tensor) -> bool:
        return self.takes_rows(rows) and w.numel() * w.element_size() <= self.MAX_WEIGHT_BYTES

    def takes_attention(self, hd: int, block_keys: int) -> bool:
        """One program runs one attention variant; a second one waits for the next program."""
        bk = 16 if (hd == 64 and block_keys == 16) or hd == 128 else 32
        return self._hd in (0, hd) and (self._hd == 0 or self._bk == bk)

    def flush(self) -> None:
        """Run what has been recorded (one launch) and start an empty recording."""
        global launch_count
        if not self._n:
            return
        host = b"".join(self._pending)
        n, rows, hd, bk, max_vblocks, max_k, status = (self._n, self._rows, self._hd, self._bk, self._max_vblocks, self._max_k,
                                                        self._status)
        self._reset()
        k = self.cursor
        if k < len(self.segments) and self.segments[k]["host"] == host:
            seg = self.segments[k]
        else:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("a decode program changed between the run that prepared a CUDA graph and its recording")
            dev = torch.empty(len(host), dtype=torch.uint8, device=status.device)
            dev.copy_(torch.frombuffer(bytearray(host), dtype=torch.uint8))
            seg = {"host": host, "dev": dev, "barrier": torch.zeros(1, dtype=torch.int32, device=status.device)}
            del self.segments[k:]
            self.segments.append(seg)
        self.cursor = k + 1
        launch_count += 1
        if self.trace_next:        # (a measurement: per-operation clock values of the first and the last block)
            self.traces.append((n, torch.zeros(2 * n * 4, dtype=torch.int64, device=status.device), host))
            rc = lib().gb_program_launch_traced(seg["dev"].data_ptr(), n, rows, hd, bk, max_vblocks, max_k, seg["barrier"].data_ptr(),
                                                status.data_ptr(), self.how, self.traces[-1][1].data_ptr(), _stream())
        elif self.absent_blocks:     # (a test of the barrier's bounded wait)
            rc = lib().gb_program_launch_with_absent_blocks(seg["dev"].data_ptr(), n, rows, hd, bk, max_vblocks, max_k,
                                                            seg["barrier"].data_ptr(), status.data_ptr(), self.absent_blocks,
                                                            self.wait_cycles, _stream())
        else:
            rc = lib().gb_program_launch(seg["dev"].data_ptr(), n, rows, hd, bk, max_vblocks, max_k, seg["barrier"].data_ptr(),
                                         status.data_ptr(), self.how, _stream())
        if rc != 0:
            raise KernelError(lib().gb_last_error().decode("utf-8", "replace") or f"gb_program_launch failed with code {rc}")


_program: Optional[Program] = None


def program_begin(program: Program, status: torch.Tensor) -> None:
    """Start recording into ``program``; ``status`` is the device status word its kernel reports to."""
    global _program
    if _program is not None:
        raise KernelError("a decode program is already being recorded")
    program.start_step()
    program._status = status
    program._default_status = status
    _program = program


def program_end() -> None:
    """Run what is still recorded and stop recording."""
    global _program
    if _program is not None:
        try:
            _program.flush()
        finally:
            _program = None


def _program_for(status: Optional[torch.Tensor] = None) -> Optional[Program]:
    p = _program
    if p is not None and p._status is None:
        p._status = status if status is not None else p._default_status
    return p


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported tensor dtype {t.dtype}") from None


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel operands must be CUDA tensors; there is no CPU path")


def check_status(status: torch.Tensor) -> None:
    """Read the device status word (synchronises) and raise if a kernel recorded a bad index."""
    bits = int(status.item())
    if bits:
        status.zero_()
        what = [msg for bit, msg in STATUS_BITS.items() if bits & bit]
        raise KernelError("a kernel skipped an access: " + "; ".join(what))


# ------------------------------------------------------------------------------------------ ops
def embed(table: torch.Tensor, tokens: torch.Tensor, x: torch.Tensor, status: torch.Tensor) -> None:
    """x[i, :] = table[tokens[i], :] as float32."""
    _cuda(table, tokens, x, status)
    n, d = x.shape
    assert tokens.dtype == torch.int32 and x.dtype == torch.float32 and x.is_contiguous() and table.is_contiguous()
    _call("gb_embed", _ptr(table), _dt(table), _ptr(tokens), _ptr(x), n, d, table.shape[0], _ptr(status), _stream())


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r, :] = gain * x[rows[r] or r, :] / sqrt(mean(x^2) + eps); x and gain float32."""
    _cuda(x, gain, out, rows)
    assert x.dtype == torch.float32 and gain.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    n, d = out.shape
    assert x.shape[1] == d and gain.numel() == d
    _call("gb_rmsnorm", _ptr(x), _ptr(rows), _ptr(gain), _ptr(out), _dt(out), n, d, float(eps), _stream())


def rope_kv_write(qkv: torch.Tensor, cos_sin: Optional[torch.Tensor], positions: torch.Tensor, slots: torch.Tensor,
                  kcache: torch.Tensor, vcache: torch.Tensor, nh: int, nkv: int, hd: int, rot: int,
                  page_size: int, write_kv: bool, status: torch.Tensor) -> None:
    """Rotate q and k of each row at its position (in place) and store k, v at the row's slot.
    kcache/vcache: [pages, nkv, page_size, hd]; cos_sin: float32 [max_pos, rot/2, 2]."""
    _cuda(qkv, cos_sin, positions, slots, kcache, vcache, status)
    n = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * hd
    assert kcache.dtype == qkv.dtype and vcache.dtype == qkv.dtype and kcache.is_contiguous() and vcache.is_contiguous()
    max_pos = cos_sin.shape[0] if cos_sin is not None else 0
    _call("gb_rope_kv_write", _ptr(qkv), _dt(qkv), _ptr(cos_sin), _ptr(positions), _ptr(slots), _ptr(kcache),
          _ptr(vcache), n, nh, nkv, hd, rot if cos_sin is not None else 0, max_pos, page_size, kcache.shape[0],
          1 if write_kv else 0, _ptr(status), _stream())


def swiglu(gate_up: torch.Tensor, act: torch.Tensor) -> None:
    _cuda(gate_up, act)
    n, inter = act.shape
    assert gate_up.shape == (n, 2 * inter) and gate_up.dtype == act.dtype
    assert gate_up.is_contiguous() and act.is_contiguous()
    _call("gb_swiglu", _ptr(gate_up), _ptr(act), _dt(act), n, inter, _stream())


def copy_pages(kcache: torch.Tensor, vcache: torch.Tensor, pairs: torch.Tensor) -> None:
    """kcache/vcache: [layers, pages, ...]; pairs int32 [n, 2] of (source page, destination page)."""
    _cuda(kcache, vcache, pairs)
    layers = kcache.shape[0]
    layer_bytes = kcache.stride(0) * kcache.element_size()
    page_bytes = kcache.stride(1) * kcache.element_size()
    _call("gb_copy_pages", _ptr(kcache), _ptr(vcache), _ptr(pairs), pairs.shape[0], page_bytes, layer_bytes, layers,
          _stream())


def gemm_simt(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, accumulate: bool = False) -> None:
    """c[M, N] (+)= a[M, K] @ w[N, K]^T with float32 FMA on the CUDA cores (rows may be strided)."""
    _cuda(a, w, c)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    _call("gb_gemm_simt", _ptr(a), _dt(a), _ptr(w), _dt(w), _ptr(c), _dt(c), 1 if accumulate else 0, M, N, K,
          a.stride(0), w.stride(0), c.stride(0), _stream())


STREAM_MAX_ROWS = 64
#: above this many rows the norm is not folded into the stream kernels (every block would repeat
#: the normalisation of all rows) and QKV keeps one strip per block (twice the blocks) -- unless the
#: kernel takes the rows in groups of eight (``stream_folds``)
STREAM_FUSE_MAX_ROWS = 16


def stream_row_groups(rows: int, w: torch.Tensor) -> int:
    """In how many groups of eight rows the weight-streaming kernel runs a product of ``rows`` rows with ``w`` (1: all
    rows in one group). Small matrices are taken group by group: every block then works as for eight rows."""
    return int(lib().gb_gemm_stream_row_groups(rows, w.shape[0], w.shape[1], 0))


def stream_folds(rows: int, w: torch.Tensor) -> bool:
    """Whether a norm in front of this product (and rotation and the cache write behind a QKV product) is folded into
    the weight-streaming kernel: with few rows, or when the rows go in groups of eight."""
    return rows <= STREAM_FUSE_MAX_ROWS or (rows <= STREAM_MAX_ROWS and stream_row_groups(rows, w) > 1)


#: launch the decode-path kernels under programmatic stream serialisation (they wait for their
#: predecessor themselves, after work that does not depend on it)
USE_PDL = True


def gemm_stream_supported(a, w: torch.Tensor, rows: Optional[int] = None) -> bool:
    """Whether the weight-streaming kernel (few rows, bfloat16 weights) takes these operands. ``a``
    is a bfloat16 [M, K] tensor, or a float32 one that the kernel normalises on the way in."""
    M, K = a.shape
    if w.dtype != torch.bfloat16 or M > STREAM_MAX_ROWS or K % 8 or w.stride(0) % 8 or w.data_ptr() % 16:
        return False
    if a.dtype == torch.bfloat16:
        return a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
    return a.dtype == torch.float32 and a.stride(0) % 4 == 0 and a.data_ptr() % 16 == 0


def _stream_input(a: torch.Tensor, norm):
    """(x, ldx, xres, ldr, gain, eps) for the stream kernels: bfloat16 activations as they are, or
    float32 rows with the (gain, eps) of an RMSNorm to apply on the way in."""
    if norm is None:
        assert a.dtype == torch.bfloat16
        return _ptr(a), a.stride(0), 0, 0, 0, 0.0
    gain, eps = norm
    assert a.dtype == torch.float32 and gain.dtype == torch.float32 and gain.numel() == a.shape[1]
    return 0, 0, _ptr(a), a.stride(0), _ptr(gain), float(eps)


def _prefetch_args(t: Optional[torch.Tensor]):
    return (0, 0) if t is None else (t.data_ptr(), t.numel() * t.element_size())


def gemm_stream(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, accumulate: bool = False, gated: bool = False,
                norm=None, prefetch: Optional[torch.Tensor] = None) -> None:
    """c[M, N] (+)= a[M, K] @ w[N, K]^T for M <= 64 on the tensor cores, streaming w once. With
    ``gated``, w is [2I, K] (gate rows, then up rows) and c[M, I] = silu(a gate^T) * (a up^T). With
    ``norm`` = (gain, eps), ``a`` is the float32 residual and is RMS-normalised on the way in.
    ``prefetch`` names a tensor (a later kernel's weights) to pull into L2 meanwhile."""
    _cuda(a, w, c)
    M, K = a.shape
    N = w.shape[0] // 2 if gated else w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N) and a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    if gated:
        assert c.dtype == torch.bfloat16 and not accumulate
        mode = 3
    elif accumulate:
        assert c.dtype == torch.float32
        mode = 2
    else:
        mode = 0 if c.dtype == torch.bfloat16 else 1
        assert c.dtype in (torch.bfloat16, torch.float32)
    x, ldx, xres, ldr, gain, eps = _stream_input(a, norm)
    prog = _program_for()
    if prog is not None and prog.takes_product(M, w):
        prog._add("gb_program_encode_gemm", -(-N // 16), M, K, x, ldx, xres, ldr, gain, eps, _ptr(w), w.stride(0), _ptr(c),
                  c.stride(0), mode, M, N, K)
        return
    _call("gb_gemm_stream", x, ldx, xres, ldr, gain, eps, _ptr(w), w.stride(0), _ptr(c), c.stride(0), mode, M, N, K,
          *_prefetch_args(prefetch), 1 if USE_PDL else 0, _stream())


def gemm_stream_qkv_supported(a, w: torch.Tensor, hd: int, q_out: torch.Tensor) -> bool:
    return (gemm_stream_supported(a, w) and stream_folds(a.shape[0], w) and hd % 32 == 0
            and q_out.dtype == torch.bfloat16)


def gemm_stream_qkv(a: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, cos_sin: Optional[torch.Tensor],
                    positions: torch.Tensor, slots: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, nh: int,
                    nkv: int, hd: int, page_size: int, write_kv: bool, status: torch.Tensor, norm=None,
                    prefetch: Optional[torch.Tensor] = None) -> None:
    """Stacked QKV projection for M <= 64 with rotary encoding and the cache write in its epilogue:
    q_out[:, :nh*hd] receives the rotated queries, rotated keys and values go to each row's cache slot.
    Full rotary (table [max_pos, hd/2, 2]) or none (cos_sin None)."""
    _cuda(a, w, q_out, cos_sin, positions, slots, kcache, vcache, status)
    M, K = a.shape
    assert w.shape == ((nh + 2 * nkv) * hd, K) and q_out.stride(1) == 1 and q_out.shape[0] == M
    assert kcache.dtype == vcache.dtype == torch.bfloat16 and kcache.is_contiguous() and vcache.is_contiguous()
    if cos_sin is not None:
        assert cos_sin.shape[1] == hd // 2
    x, ldx, xres, ldr, gain, eps = _stream_input(a, norm)
    prog = _program_for(status)
    if prog is not None and prog.takes_product(M, w):
        prog._add("gb_program_encode_gemm_qkv", (nh + 2 * nkv) * (hd // 32), M, K, x, ldx, xres, ldr, gain, eps, _ptr(w),
                  w.stride(0), _ptr(q_out), q_out.stride(0), M, K, _ptr(cos_sin),
                  cos_sin.shape[0] if cos_sin is not None else 0, _ptr(positions), _ptr(slots), _ptr(kcache), _ptr(vcache),
                  nh, nkv, hd, page_size, kcache.shape[0], 1 if write_kv else 0, _ptr(status))
        return
    _call("gb_gemm_stream_qkv", x, ldx, xres, ldr, gain, eps, _ptr(w), w.stride(0), _ptr(q_out), q_out.stride(0), M, K,
          _ptr(cos_sin), cos_sin.shape[0] if cos_sin is not None else 0, _ptr(positions), _ptr(slots), _ptr(kcache),
          _ptr(vcache), nh, nkv, hd, page_size, kcache.shape[0], 1 if write_kv else 0, _ptr(status),
          *_prefetch_args(prefetch), 1 if USE_PDL else 0, _stream())


def gemm_tc_supported(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel takes these operands (bfloat16, TMA-aligned)."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or c.dtype not in (torch.bfloat16, torch.float32):
        return False
    return bool(lib().gb_gemm_tcgen05_supported(_ptr(a), _ptr(w), a.shape[0], w.shape[0], a.shape[1], a.stride(0),
                                                w.stride(0)))


_tc_status = {}


class RowScale:
    """The consumer half of an RMSNorm split between two tile-kernel products: ``ss`` float32 [M, parts] holds partial
    sums of squares of the residual rows, and each row of the product is multiplied by
    1 / sqrt(sum(ss[row]) / K + eps). The product's ``a`` operand is then bfloat16(residual * gain)."""
    __slots__ = ("ss", "eps")

    def __init__(self, ss: torch.Tensor, eps: float):
        assert ss.dtype == torch.float32 and ss.dim() == 2 and ss.is_contiguous()
        self.ss, self.eps = ss, float(eps)

    def args(self, rows: int):
        assert self.ss.shape[0] == rows
        return _ptr(self.ss), self.ss.shape[1], self.eps


_NO_SCALE = (None, 0, 0.0)


def gemm_tc_column_tiles(rows: int, n: int, k: int) -> int:
    """Column tiles of the output of a ``gemm_tc`` that adds [rows, k] x [n, k]^T into float32: the second extent of
    the partial sums of squares that a product with ``prepare`` writes."""
    return int(lib().gb_gemm_tcgen05_column_tiles(rows, n, k))


def gemm_tc(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, accumulate: bool = False,
            status: Optional[torch.Tensor] = None, prepare=None, row_scale: Optional[RowScale] = None) -> None:
    """c[M, N] (+)= a[M, K] @ w[N, K]^T with TMA + tcgen05.mma + TMEM. ``status`` receives the
    wait-timeout bit if a bounded wait inside the kernel ever gives up.

    ``prepare=(gain, pre, ss)`` (only with ``accumulate``) makes the epilogue the producer half of an RMSNorm of the
    rows it has just completed: ``pre`` bfloat16 [M, N] receives c * gain and ``ss`` float32
    [M, gemm_tc_column_tiles(M, N, K)] the partial sums of squares; a later product takes ``pre`` as its ``a`` with
    ``row_scale=RowScale(ss, eps)``."""
    _cuda(a, w, c, status)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N) and a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    prep = (None, None, 0, None)
    if prepare is not None:
        gain, pre, ss = prepare
        _cuda(gain, pre, ss)
        assert accumulate and gain.dtype == torch.float32 and gain.numel() == N and gain.is_contiguous()
        assert pre.dtype == torch.bfloat16 and pre.shape == (M, N) and pre.stride(1) == 1
        assert ss.dtype == torch.float32 and ss.is_contiguous() and ss.shape == (M, gemm_tc_column_tiles(M, N, K))
        prep = (_ptr(gain), _ptr(pre), pre.stride(0), _ptr(ss))
    if status is None:
        status = _tc_status.get(a.device)
        if status is None:
            status = _tc_status[a.device] = torch.zeros(1, dtype=torch.int32, device=a.device)
    if accumulate:
        assert c.dtype == torch.float32
        mode = 2
    else:
        mode = 0 if c.dtype == torch.bfloat16 else 1
    _call("gb_gemm_tcgen05", _ptr(a), _ptr(w), _ptr(c), mode, M, N, K, a.stride(0), w.stride(0), c.stride(0),
          _ptr(status), _stream(), *prep, *(row_scale.args(M) if row_scale is not None else _NO_SCALE))


def gemm_tc_qkv_supported(a: torch.Tensor, w: torch.Tensor, hd: int, q_out: torch.Tensor, kcache: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel can project, rotate and write the cache in one go for these operands."""
    return (q_out.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and q_out.stride(0) % 8 == 0
            and q_out.data_ptr() % 16 == 0 and bool(lib().gb_gemm_tcgen05_qkv_supported(hd)) and gemm_tc_supported(a, w, q_out))


def gemm_tc_qkv(a: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, cos_sin: Optional[torch.Tensor],
                positions: torch.Tensor, slots: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, nh: int, nkv: int,
                hd: int, page_size: int, write_kv: bool, status: torch.Tensor, row_scale: Optional[RowScale] = None) -> None:
    """Stacked QKV projection on the tcgen05 kernel with the rotation and the cache write in its epilogue:
    q_out[:, :nh*hd] receives the rotated queries, the cache slots of the rows the rotated keys and the
    values. ``cos_sin`` is float32 [max_pos, hd/2, 2] or None (no rotation). ``row_scale``: see ``RowScale``."""
    _cuda(a, w, q_out, cos_sin, positions, slots, kcache, vcache, status)
    M, K = a.shape
    assert w.shape == ((nh + 2 * nkv) * hd, K) and a.stride(1) == 1 and w.stride(1) == 1 and q_out.stride(1) == 1
    assert q_out.shape[0] == M and q_out.shape[1] >= nh * hd and kcache.is_contiguous() and vcache.is_contiguous()
    assert cos_sin is None or (cos_sin.dtype == torch.float32 and cos_sin.shape[1:] == (hd // 2, 2) and cos_sin.is_contiguous())
    _call("gb_gemm_tcgen05_qkv", _ptr(a), _ptr(w), _ptr(q_out), M, K, a.stride(0), w.stride(0), q_out.stride(0),
          _ptr(cos_sin), cos_sin.shape[0] if cos_sin is not None else 0, _ptr(positions), _ptr(slots), _ptr(kcache),
          _ptr(vcache), nh, nkv, hd, page_size, kcache.shape[0], 1 if write_kv else 0, _ptr(status), _stream(),
          *(row_scale.args(M) if row_scale is not None else _NO_SCALE))


def gemm_tc_gated(a: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor,
                  status: Optional[torch.Tensor] = None, row_scale: Optional[RowScale] = None) -> None:
    """act[M, I] = silu(a gate^T) * (a up^T) with w_gate_up = [gate rows; up rows], on the tcgen05
    kernel: gate and up columns of a tile sit side by side in one TMEM accumulator. ``row_scale``: see ``RowScale``."""
    _cuda(a, w_gate_up, act, status)
    M, K = a.shape
    inter = w_gate_up.shape[0] // 2
    assert w_gate_up.shape == (2 * inter, K) and act.shape == (M, inter) and act.dtype == torch.bfloat16
    assert a.stride(1) == 1 and w_gate_up.stride(1) == 1 and act.stride(1) == 1
    if status is None:
        status = _tc_status.get(a.device)
        if status is None:
            status = _tc_status[a.device] = torch.zeros(1, dtype=torch.int32, device=a.device)
    _call("gb_gemm_tcgen05_gated", _ptr(a), _ptr(w_gate_up), _ptr(act), M, inter, K, a.stride(0), w_gate_up.stride(0),
          act.stride(0), _ptr(status), _stream(), *(row_scale.args(M) if row_scale is not None else _NO_SCALE))


def attention_rows(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                   block_tables: torch.Tensor, row_seq: torch.Tensor, positions: torch.Tensor, nh: int, nkv: int,
                   hd: int, page_size: int, scale: float, window: Optional[int], status: torch.Tensor) -> None:
    """One warp per (row, head): softmax(q k^T * scale) v over the row's visible keys."""
    _cuda(q, out, kcache, vcache, block_tables, row_seq, positions, status)
    n = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == kcache.dtype
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    _call("gb_attention_rows", _ptr(q), q.stride(0), _ptr(out), out.stride(0), _dt(q), _ptr(kcache), _ptr(vcache),
          _ptr(block_tables), block_tables.shape[1], _ptr(row_seq), _ptr(positions), n, nh, nkv, hd, page_size,
          kcache.shape[0], float(scale), int(window or 0), _ptr(status), _stream())


DECODE_KEYS_PER_TILE = 64


def decode_splits(n: int, nh: int, nkv: int, max_context: int, target_blocks: int = 148 * 4) -> int:
    """How many blocks share the keys of one (row, kv head): enough to fill the GPU, never more than
    there are 64-key tiles. Depends on the batch shape only, so a captured graph can fix it."""
    per_split = lib().gb_attention_decode_counters(n, nh, nkv)
    tiles = max(1, -(-max_context // DECODE_KEYS_PER_TILE))
    return max(1, min(-(-target_blocks // max(per_split, 1)), tiles))


def attention_decode(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                     block_tables: torch.Tensor, row_seq: torch.Tensor, positions: torch.Tensor, nh: int, nkv: int,
                     hd: int, page_size: int, scale: float, window: Optional[int], splits: int,
                     part_acc: Optional[torch.Tensor], part_ml: Optional[torch.Tensor],
                     counters: Optional[torch.Tensor], status: torch.Tensor) -> None:
    """Split-key attention for rows with few queries per request. Scratch (needed when splits > 1):
    part_acc float32 [n, nh, splits, hd], part_ml float32 [n, nh, splits, 2], counters int32
    [gb_attention_decode_counters(n, nh, nkv)] that are zero on entry and left zero."""
    _cuda(q, out, kcache, vcache, block_tables, row_seq, positions, part_acc, part_ml, counters, status)
    n = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == kcache.dtype
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    if splits > 1:
        assert part_acc.numel() >= n * nh * splits * hd and part_ml.numel() >= n * nh * splits * 2
        assert counters.numel() >= lib().gb_attention_decode_counters(n, nh, nkv)
    _call("gb_attention_decode", _ptr(q), q.stride(0), _ptr(out), out.stride(0), _dt(q), _ptr(kcache), _ptr(vcache),
          _ptr(block_tables), block_tables.shape[1], _ptr(row_seq), _ptr(positions), n, nh, nkv, hd, page_size,
          kcache.shape[0], float(scale), int(window or 0), int(splits), _ptr(part_acc), _ptr(part_ml),
          _ptr(counters), _ptr(status), _stream())


def attention_decode_mma_supported(dtype: torch.dtype, nh: int, nkv: int, hd: int, page_size: int = 16) -> bool:
    return (dtype == torch.bfloat16 and page_size >= 16 and page_size & (page_size - 1) == 0
            and bool(lib().gb_attention_decode_mma_supported(nh, nkv, hd)))


DECODE_MMA_WAVE_SINGLE = 444        # blocks of the 16-key, four-warp variant that run at once: 148 SMs x 3
DECODE_MMA_WAVE_BLOCKS = 410        # the same in clusters of 2 to 4 (measured: 410 fit, 432 do not)
DECODE_MMA_BLOCK_US = 5.7           # a block's fixed cost, microseconds (measured)
DECODE_MMA_KEY_US = 0.0147          # and its cost per key


def decode_mma_plan(n: int, nkv: int, hd: int, max_context: int):
    """(splits, keys per warp iteration, warps per block) for the tensor-core decode kernel. A small batch needs
    many blocks per (row, kv head) to fill the GPU, but each block keeps at least 512 keys, below which the
    fixed cost of a block and of the merge outweighs the parallelism; where that leaves at most one block
    per SM, a block has eight warps instead of four, so that each warp walks through half as many keys (the
    splits are then rounded down: a second block of eight warps does not fit beside the first). A batch that
    fills the GPU by itself takes the 16-key variant (three blocks per SM instead of two) and the split count
    whose waves of resident blocks are estimated to end soonest.
    Depends on the batch shape and the longest context the step allows, never on the data, so a captured
    graph can fix it."""
    pairs = max(n * nkv, 1)
    most = max(1, -(-max_context // 512))
    if hd == 64 and pairs >= 96:
        # Blocks of the 16-key variant run three to an SM, in waves: all blocks of a wave take as long as one of them.
        # A block costs about 5.7 us of start, merge and hand-over and 14.7 ns a key; a wave holds about 410 blocks
        # (432 no longer fit one; without clusters, at one split, 416 still do: 71.3 us, 3 splits 92.0). The split count that this estimate likes best, among 1 to 4 (clusters of 5 and 7
        # place badly), is the one measured best at context 4096 for 96 to 2,048 pairs, within 1 %: 128 pairs 3 splits
        # 26.8 us (2: 34.6, 4: 37.3); 144 pairs 2 splits 35.6 (3: 45.6); 256 pairs 3 splits 51.6 (1: 66.1, 2: 66.3,
        # 4: 57.7); 320 pairs 1 split 68.4 (2: 72.9, 4: 79.0); 512 pairs 3 splits 99.0 (1: 123.1, 4: 98.2); 2,048 pairs
        # 1 split 338.7 (2: 354.7). (Filling two blocks per SM once, the rule before, took 2 splits at 256 pairs: a 1.7B
        # decode step at batch 8 2.85 ms, with 3 splits 2.56 ms.)
        best, best_cost = 1, None
        for splits in range(1, min(4, most) + 1):
            waves = -(-pairs * splits // (DECODE_MMA_WAVE_BLOCKS if splits > 1 else DECODE_MMA_WAVE_SINGLE))
            cost = waves * (DECODE_MMA_BLOCK_US + DECODE_MMA_KEY_US * -(-max_context // splits))
            if best_cost is None or cost < best_cost - 1e-9:
                best, best_cost = splits, cost
        return best, 16, 4
    if hd == 64 and pairs <= 74:
        # (measured at 9/3 heads, microseconds at context 4096 with 4 warps and the old split count against 8 warps:
        # batch 8 18.8 -> 12.4, batch 16 18.2 -> 15.1, batch 4 12.7 -> 11.3; eight warps want at least 256 keys a block
        # and at most 8 splits: context 1024, batch 8: 2 splits 9.3, 4 splits 8.6; context 4096, batch 1: 8 splits
        # 11.1, 16 splits 12.4)
        # 16 keys per iteration: 160 registers per thread instead of 251, so that a block no longer fills an SM's
        # register file and the product that follows finds room beside it while it waits for it (alone the two variants
        # take the same time; in a 135M decode step: batch 1 0.73 -> 0.65 ms, batch 8 0.80 -> 0.78 ms)
        # (with more than 1,024 keys per block the longer loop of the 16-key variant costs more than the room gains:
        # 360M shapes at batch 8, three splits of 1,365 keys: 1.23 ms with 32 keys per iteration, 1.27 ms with 16)
        splits = max(1, min(148 // pairs, 8, -(-max_context // 256)))
        return splits, (16 if max_context <= 1024 * splits else 0), 8
    return max(1, min(-(-148 // pairs), most)), 0, 4


def decode_mma_splits(n: int, nkv: int, hd: int, max_context: int) -> int:
    return decode_mma_plan(n, nkv, hd, max_context)[0]


def attention_decode_mma(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                         block_tables: torch.Tensor, row_seq: torch.Tensor, positions: torch.Tensor, nh: int, nkv: int,
                         hd: int, page_size: int, scale: float, window: Optional[int], splits: int,
                         part_acc: torch.Tensor, part_ml: torch.Tensor, counters: torch.Tensor,
                         status: torch.Tensor, block_keys: int = 0, warps: int = 4) -> None:
    """bfloat16 split-key decode attention on the tensor cores. Scratch: part_acc float32
    [n, nh, warps*splits, hd], part_ml float32 [n, nh, warps*splits, 2], counters int32 [n*nkv], zero on entry
    and left zero. ``warps`` per block: 4, or 8 (head size 64)."""
    _cuda(q, out, kcache, vcache, block_tables, row_seq, positions, part_acc, part_ml, counters, status)
    n = q.shape[0]
    assert q.dtype == out.dtype == kcache.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    assert part_acc.numel() >= n * nh * warps * splits * hd and part_ml.numel() >= n * nh * warps * splits * 2
    assert counters.numel() >= n * nkv
    prog = _program_for(status)
    if prog is not None and prog.takes_rows(n):
        if not prog.takes_attention(hd, block_keys):
            prog.flush()
            prog._status = status
        prog._add("gb_program_encode_attention", splits * nkv * n, n, 8, _ptr(q), q.stride(0), _ptr(out), out.stride(0),
                  _ptr(kcache), _ptr(vcache), _ptr(block_tables), block_tables.shape[1], _ptr(row_seq), _ptr(positions), n,
                  nh, nkv, hd, page_size, kcache.shape[0], float(scale), int(window or 0), int(splits), _ptr(part_acc),
                  _ptr(part_ml), _ptr(counters), _ptr(status), int(block_keys))
        prog._hd, prog._bk = hd, (16 if (hd == 64 and block_keys == 16) or hd == 128 else 32)
        return
    _call("gb_attention_decode_mma_pdl", _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache),
          _ptr(block_tables), block_tables.shape[1], _ptr(row_seq), _ptr(positions), n, nh, nkv, hd, page_size,
          kcache.shape[0], float(scale), int(window or 0), int(splits), _ptr(part_acc), _ptr(part_ml), _ptr(counters),
          _ptr(status), 1 if USE_PDL else 0, int(block_keys), int(warps), _stream())


def attention_prefill_supported(dtype: torch.dtype, nh: int, nkv: int, hd: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and bool(lib().gb_attention_prefill_supported(nh, nkv, hd, page_size))


def attention_prefill_tc_supported(q: torch.Tensor, out: torch.Tensor, nh: int, nkv: int, hd: int, page_size: int) -> bool:
    """Whether the tcgen05 flash-attention kernel takes these operands (bfloat16, head size 64, rows
    aligned for TMA)."""
    return (q.dtype == torch.bfloat16 and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
            and out.data_ptr() % 16 == 0 and bool(lib().gb_attention_prefill_tc_supported(nh, nkv, hd, page_size)))


def attention_prefill_tc(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                         block_tables: torch.Tensor, seq_first_row: torch.Tensor, seq_start_pos: torch.Tensor,
                         max_rows_per_seq: int, nh: int, nkv: int, hd: int, page_size: int, scale: float,
                         window: Optional[int], status: torch.Tensor) -> None:
    """bfloat16 flash attention on tcgen05 (TMA loads from the paged cache, S and PV in tensor memory) for
    batches whose requests bring runs of consecutive rows; arguments as ``attention_prefill``."""
    _cuda(q, out, kcache, vcache, block_tables, seq_first_row, seq_start_pos, status)
    assert q.dtype == out.dtype == kcache.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    assert kcache.is_contiguous() and vcache.is_contiguous() and kcache.shape[1:] == (nkv, page_size, hd)
    S = block_tables.shape[0]
    assert seq_first_row.numel() == S + 1 and seq_start_pos.numel() == S
    _call("gb_attention_prefill_tc", _ptr(q), q.stride(0), q.shape[0], _ptr(out), out.stride(0), _ptr(kcache),
          _ptr(vcache), _ptr(block_tables), block_tables.shape[1], _ptr(seq_first_row), _ptr(seq_start_pos), S,
          int(max_rows_per_seq), nh, nkv, hd, page_size, kcache.shape[0], float(scale), int(window or 0), _ptr(status),
          _stream())


def attention_prefill(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                      block_tables: torch.Tensor, seq_first_row: torch.Tensor, seq_start_pos: torch.Tensor,
                      max_rows_per_seq: int, nh: int, nkv: int, hd: int, page_size: int, scale: float,
                      window: Optional[int], status: torch.Tensor) -> None:
    """bfloat16 flash attention for batches whose requests bring runs of consecutive rows.
    seq_first_row int32 [S+1], seq_start_pos int32 [S]; block_tables int32 [S, max_pages]."""
    _cuda(q, out, kcache, vcache, block_tables, seq_first_row, seq_start_pos, status)
    assert q.dtype == out.dtype == kcache.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    S = block_tables.shape[0]
    assert seq_first_row.numel() == S + 1 and seq_start_pos.numel() == S
    _call("gb_attention_prefill", _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache),
          _ptr(block_tables), block_tables.shape[1], _ptr(seq_first_row), _ptr(seq_start_pos), S, int(max_rows_per_seq),
          nh, nkv, hd, page_size, kcache.shape[0], float(scale), int(window or 0), _ptr(status), _stream())


def kv_prefetch(kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor, row_seq: torch.Tensor,
                positions: torch.Tensor, nkv: int, hd: int, page_size: int, window: Optional[int],
                blocks_per_row: int) -> None:
    """Ask the memory system to bring the pages that each row's attention will read into L2."""
    _cuda(kcache, vcache, block_tables, row_seq, positions)
    tile_bytes = page_size * hd * kcache.element_size()
    if tile_bytes % 128:
        return
    _call("gb_kv_prefetch", _ptr(kcache), _ptr(vcache), _ptr(block_tables), block_tables.shape[1], _ptr(row_seq),
          _ptr(positions), positions.shape[0], nkv, page_size, kcache.shape[0], tile_bytes, int(window or 0),
          int(blocks_per_row), _stream())


def stream_marker() -> None:
    """An empty kernel on the current stream: a node of its own in a recorded step (see ``GqaAttention.prefetch``)."""
    _call("gb_stream_marker", _stream())


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           uniform: Optional[torch.Tensor] = None, want_slots: Optional[torch.Tensor] = None,
           state: Optional[torch.Tensor] = None, last_token: Optional[torch.Tensor] = None) -> None:
    """out[r] = argmax(logits[r]) where the row's temperature is <= 0 (or none is given), else a draw from
    softmax(logits[r] / temperature) with a uniform number in [0, 1). Temperature and number come from
    ``temperature[r]`` and ``uniform[r]``, or, for rows with ``want_slots[r] >= 0``, from the request's sampling
    state ``state[want_slots[r]]`` (int32 [slots, 4]: generator state low and high word, temperature bits, unused),
    whose xorshift64* generator the kernel advances by one draw. ``last_token`` (int32 [slots]) receives the chosen
    token of every row that names a slot (see ``resolve_tokens``)."""
    _cuda(logits, out, temperature, uniform, want_slots, state, last_token)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    if want_slots is not None:
        assert want_slots.dtype == torch.int32 and want_slots.numel() >= rows
        assert state is not None and state.dtype == torch.int32 and state.shape[1] == 4 and state.is_contiguous()
    _call("gb_sample", _ptr(logits), logits.stride(0), _ptr(temperature), _ptr(uniform), _ptr(want_slots), _ptr(state),
          state.shape[0] if state is not None else 0, _ptr(last_token), _ptr(out), rows, vocab, _stream())


def resolve_tokens(tokens: torch.Tensor, token_slots: torch.Tensor, last_token: torch.Tensor) -> None:
    """tokens[i] = last_token[token_slots[i]] where token_slots[i] >= 0 (in place): rows whose token is what the sampling
    kernel chose for their request in the step before, which the host had not read yet when it launched this step."""
    _cuda(tokens, token_slots, last_token)
    assert tokens.dtype == token_slots.dtype == last_token.dtype == torch.int32 and token_slots.numel() >= tokens.numel()
    _call("gb_resolve_tokens", _ptr(tokens), _ptr(token_slots), _ptr(last_token), tokens.numel(), last_token.numel(), _stream())
