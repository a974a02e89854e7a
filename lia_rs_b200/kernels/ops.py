"""Python faces of the CUDA entry points.  Every function takes CUDA tensors, checks what the
kernel assumes, launches on the current stream and raises on a refusal; there is no CPU or
library fallback here."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import torch

from . import build

F32, BF16 = 0, 1
GEMM_STORE, GEMM_ACCUM, GEMM_SWIGLU = 0, 1, 2

_ERRORS = {-1: "a size the kernel refuses", -2: "a pointer or stride that is not aligned as required",
           -3: "the launch failed (cudaGetLastError)", -4: "a driver entry point is missing or failed",
           -5: "no instantiation for this combination of element types"}


class KernelError(RuntimeError):
    pass


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = build.load()
        for name in dir(_Signatures):
            if name.startswith("lia_"):
                fn = getattr(_lib, name)
                fn.argtypes = getattr(_Signatures, name)
                fn.restype = c_int
    return _lib


class _Signatures:
    lia_embedding = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p]
    lia_rmsnorm = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p]
    lia_layernorm = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p]
    lia_rope_kv_write = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                         c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
    lia_gemm_simt = [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int,
                     c_int, c_int, c_float, c_void_p]
    lia_attention_generic = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p]
    lia_gather_rows = [c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.c_longlong, ctypes.c_longlong,
                       ctypes.c_longlong, c_void_p]
    lia_wait_probe = [c_int, c_void_p, c_void_p, c_void_p]
    lia_attention_decode = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                            c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]
    lia_attention_decode_cluster_splits = [c_int, c_int, c_int, c_int]
    lia_attention_decode_ctas_per_sm = [c_int, c_int]
    lia_gemm_tc = [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                   c_void_p, ctypes.c_longlong, c_int, c_void_p, c_void_p]
    lia_gemm_cluster = [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                        c_int, c_void_p, c_void_p]
    lia_gemm_cluster_splits = [c_int, c_int, c_int, c_int, c_int]
    lia_gemm_skinny = [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                       c_void_p, c_void_p]
    lia_gemm_stream = [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                       c_void_p, c_int, c_void_p, c_int, c_float, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    lia_gemm_stream_stages = [c_int, c_int, c_int, c_int, c_int, c_int]
    lia_attention_prefill = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                             c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p]
    lia_attention_prefill_tc = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                                c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_int, c_int,
                                c_float, c_void_p, c_void_p]
    lia_attention_prefill_tc_tokens_per_tile = [c_int, c_int]
    lia_select_tokens = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                         ctypes.c_longlong, c_void_p]
    lia_select_tokens_scratch_floats = [c_int, c_int]
    lia_select_candidates = [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p, ctypes.c_longlong, c_void_p]
    lia_select_candidates_scratch_floats = [c_int, c_int, c_int]
    lia_rotary_pairs_kv_write = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_int, c_int, c_int,
                                 c_void_p, c_void_p]
    lia_sigmoid_attention_generic = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                     c_void_p, c_int, c_int, c_void_p, c_void_p]
    lia_short_conv = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                      c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
    lia_embedding_positions = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                               c_int, c_float, c_void_p, c_void_p]
    lia_reinject_input = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p]
    lia_sigmoid_attention_tc_tokens_per_tile = [c_int, c_int, c_int]
    lia_sigmoid_attention_tc = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_float, c_int, c_int, c_void_p, c_int,
                                c_void_p, c_void_p]

    lia_norm_residual = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float,
                         c_void_p]
    lia_activation_rows = [c_void_p, ctypes.c_longlong, c_void_p, c_int, ctypes.c_longlong, c_int, c_int, c_int, c_int, c_void_p]
    lia_attention_general = [c_void_p, ctypes.c_longlong, ctypes.c_longlong, c_void_p, ctypes.c_longlong, ctypes.c_longlong,
                             c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                             c_int, c_void_p, c_void_p, ctypes.c_longlong, ctypes.c_longlong, c_int, c_int, c_int, c_int,
                             c_int, c_float, c_float, c_int, c_int, c_void_p, c_void_p]
    lia_qkv_prepare = [c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_float,
                       c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                       c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    lia_latent_prepare = [c_void_p, ctypes.c_longlong, c_void_p, ctypes.c_longlong, c_void_p, c_float, c_void_p, c_int,
                          c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                          c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    lia_causal_conv = [c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
    lia_conv_state_update = [c_void_p, ctypes.c_longlong, c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_int, c_int,
                             c_int, c_void_p]
    lia_selective_scan = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_longlong, c_int, c_int, c_void_p,
                          c_void_p, ctypes.c_longlong, c_void_p, ctypes.c_longlong, c_void_p, c_int, c_void_p, c_int, c_void_p,
                          c_void_p, c_int, c_int, c_int, c_int, c_void_p, ctypes.c_longlong, c_void_p]
    lia_selective_scan_chunk_floats = [c_int, c_int, c_int, c_int]
    lia_gemm_simt_batched = [c_int, c_void_p, c_int, c_int, ctypes.c_longlong, c_void_p, c_int, c_int, ctypes.c_longlong,
                             c_void_p, c_int, c_int, ctypes.c_longlong, c_int, c_int, c_int, c_int, c_float, c_void_p]

    lia_latent_attention_accepts = [c_int, c_int]
    lia_latent_attention = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                            c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p]
    lia_gemm_mma_batched_accepts = [c_void_p, ctypes.c_longlong, ctypes.c_longlong, c_void_p, ctypes.c_longlong, ctypes.c_longlong, c_void_p, ctypes.c_longlong, ctypes.c_longlong, c_int, c_int, c_int]
    lia_embedding_streams = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]
    lia_hyper_step = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                      c_int, c_int, c_float, c_void_p]
    lia_softcap_rows = [c_void_p, ctypes.c_longlong, c_int, c_int, c_float, c_void_p]
    lia_gate_rows = [c_void_p, c_int, ctypes.c_longlong, c_void_p, ctypes.c_longlong, c_int, c_int, c_int, c_int, c_void_p]
    lia_moe_tile_rows = []
    lia_moe_route = [c_void_p, c_int, ctypes.c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
                     c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
    lia_moe_plan = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
    lia_moe_gather = [c_void_p, ctypes.c_longlong, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p]
    lia_moe_gemm = [c_int, c_void_p, c_int, ctypes.c_longlong, c_void_p, c_int, c_void_p, c_void_p, ctypes.c_longlong,
                    c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lia_gemm_tc_grouped = [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                           c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]
    lia_moe_combine = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, ctypes.c_longlong,
                       c_int, c_int, c_int, c_float, c_int, c_void_p]
    lia_gla_encode = [c_void_p, ctypes.c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                      c_int, c_float, c_float, c_void_p]
    lia_gla = [c_void_p, ctypes.c_longlong, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_int, c_int, c_void_p, c_int,
               c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, ctypes.c_longlong, c_void_p, c_int,
               c_void_p, c_int, c_float, c_float, c_void_p]
    lia_retention_chunks = [c_int, c_int]
    lia_retention_encode = [c_void_p, ctypes.c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                            c_void_p]
    lia_retention = [c_void_p, ctypes.c_longlong, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_int, c_int, c_void_p,
                     c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, ctypes.c_longlong, c_void_p]
    lia_gemm_mma_batched = [c_void_p, ctypes.c_longlong, ctypes.c_longlong, c_void_p, ctypes.c_longlong, ctypes.c_longlong, c_void_p, ctypes.c_longlong, ctypes.c_longlong, c_int, c_int, c_int, c_int, c_void_p]

def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"element type {dtype} has no kernel")


def _cuda(*tensors):
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise KernelError("kernels need contiguous CUDA tensors (there is no CPU path)")


def _p(t):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream's handle.  Asked for at every launch (a graph capture runs on a stream of its own), so through
    torch's direct call where this torch has it: building a Stream object each time cost several microseconds a launch."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def kernel_launches() -> int:
    """Kernels this library has launched since it was loaded, counted at the launch sites in C.  A
    replay of a captured CUDA graph runs its kernels again without passing a launch site: the engine
    adds those (`Engine.stats['kernels']`)."""
    fn = lib().lia_kernel_launches
    fn.restype = ctypes.c_longlong
    fn.argtypes = []
    return int(fn())


def _check(code: int, what: str):
    if code != 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, code)}")


class Profiler:
    """Device time per kernel class, from CUDA events around every launch of this library while it is
    installed (`set_profiler`).  The reference's counterpart is LIA_PROFILE: a synchronisation and a host timer
    around every product, name, shape and seconds printed (src/inference/operations.rs:85-90,303-310); like it,
    this cannot run under a captured graph.  Events between launches also keep a kernel from starting under its
    predecessor's tail, so the times are those of a launch-by-launch step: read them as shares."""

    def __init__(self):
        self.records = []                        # (class, start event, end event, bytes, flops)

    def summary(self) -> dict:
        """class -> {calls, ms, bytes, flops} over what was recorded since the last call; waits for the device."""
        torch.cuda.synchronize()
        out = {}
        for key, start, end, nbytes, flops in self.records:
            entry = out.setdefault(key, {"calls": 0, "ms": 0.0, "bytes": 0, "flops": 0})
            entry["calls"] += 1
            entry["ms"] += start.elapsed_time(end)
            entry["bytes"] += int(nbytes)
            entry["flops"] += int(flops)
        self.records = []
        return out


class _Timed:
    __slots__ = ("key", "nbytes", "flops", "start")

    def __init__(self, key, nbytes, flops):
        self.key, self.nbytes, self.flops = key, nbytes, flops

    def __enter__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()

    def __exit__(self, *exc):
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        if _profiler is not None:
            _profiler.records.append((self.key, self.start, end, self.nbytes, self.flops))
        return False


class _NotTimed:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_profiler = None
_NOT_TIMED = _NotTimed()


def set_profiler(profiler) -> None:
    """Install (or, with None, remove) the profiler that every launch of this library reports to."""
    global _profiler
    _profiler = profiler


def _timed(kernel: str, label=None, nbytes=0, flops=0, work=None):
    """`work`: a function giving (bytes, flops), asked only while a profiler listens."""
    if _profiler is None:
        return _NOT_TIMED
    if work is not None:
        nbytes, flops = work()
    return _Timed(f"{kernel}:{label}" if label else kernel, nbytes, flops)


def _gemm_work(a, w, out):
    """(bytes, flops) of a product as the roofline counts them: every operand once."""
    return (a.numel() * a.element_size() + w.numel() * w.element_size() + out.numel() * out.element_size(),
            2 * a.shape[0] * w.shape[0] * a.shape[1])


def embedding(tokens, table, out, scale: float, error_flag=None):
    _cuda(tokens, table, out, error_flag)
    n, hidden = out.shape
    with _timed("embedding"):
        _check(lib().lia_embedding(_p(tokens), _p(table), dtype_code(table.dtype), _p(out), n, hidden,
                                   table.shape[0], scale, _p(error_flag), _stream()), "embedding")


def rmsnorm(x, weight, out, eps: float, out_scale: float = 1.0, rows_index=None):
    _cuda(x, weight, out, rows_index)
    rows, hidden = out.shape
    if x.dtype != torch.float32 or x.shape[1] != hidden:
        raise KernelError("rmsnorm takes 32-bit rows of the same width as its output")
    with _timed("rmsnorm"):
        _check(lib().lia_rmsnorm(_p(x), _p(rows_index), _p(weight), dtype_code(weight.dtype), _p(out),
                                 dtype_code(out.dtype), rows, hidden, eps, out_scale, _stream()), "rmsnorm")


def layernorm(x, weight, bias, out, eps: float, rows_index=None):
    """out[r] = (x[r] - mean) / sqrt(mean((x[r] - mean)^2) + eps) * weight + bias (bias may be None); x 32-bit rows, row
    r taken from rows_index[r] when an index is given; see csrc/elementwise.cu."""
    _cuda(x, weight, bias, out, rows_index)
    rows, hidden = out.shape
    if x.dtype != torch.float32 or x.shape[1] != hidden or (bias is not None and bias.dtype != weight.dtype):
        raise KernelError("layernorm takes 32-bit rows of the same width as its output, weight and bias of one element type")
    with _timed("layernorm"):
        _check(lib().lia_layernorm(_p(x), _p(rows_index), _p(weight), _p(bias), dtype_code(weight.dtype), _p(out),
                                   dtype_code(out.dtype), rows, hidden, float(eps), _stream()), "layernorm")


def rope_kv_write(qkv, positions, slots, block_table, q_out, k_pages, v_pages, nq, nkv, d, rotary_dim,
                  inv_freq, write_kv=True, error_flag=None):
    _cuda(qkv, positions, slots, block_table, q_out, k_pages, v_pages, inv_freq, error_flag)
    n = qkv.shape[0]
    if qkv.dtype != torch.float32 or qkv.shape[1] != (nq + 2 * nkv) * d:
        raise KernelError("rope_kv_write takes 32-bit q|k|v rows")
    if q_out.dtype != k_pages.dtype or k_pages.dtype != v_pages.dtype:
        raise KernelError("rope_kv_write: q and the cache must have one element type")
    num_pages, page_size = k_pages.shape[0], k_pages.shape[1]
    with _timed("rope_kv_write"):
        _check(lib().lia_rope_kv_write(_p(qkv), _p(positions), _p(slots), _p(block_table), block_table.shape[1],
                                       _p(q_out), _p(k_pages), _p(v_pages), dtype_code(q_out.dtype), n, nq, nkv, d,
                                       rotary_dim, _p(inv_freq), page_size, num_pages, 1 if write_kv else 0,
                                       _p(error_flag), _stream()), "rope_kv_write")


def gather_rows(src, index, dst):
    """dst[r] = src[index[r]] for 2-D tensors of one element type and width (rows copied as they are; a negative
    index gives zeros); see csrc/elementwise.cu."""
    _cuda(index)
    if not (src.is_cuda and dst.is_cuda) or src.dim() != 2 or dst.dim() != 2 or src.dtype != dst.dtype \
            or src.shape[1] != dst.shape[1] or src.stride(1) != 1 or dst.stride(1) != 1 or index.dtype != torch.int32 \
            or index.numel() < dst.shape[0]:
        raise KernelError("gather_rows: 2-D CUDA tensors of one type and width, int32 index of at least dst's rows")
    size = src.element_size()
    with _timed("gather_rows"):
        _check(lib().lia_gather_rows(_p(src), _p(index), _p(dst), dst.shape[0], src.shape[0], src.stride(0) * size,
                                     dst.stride(0) * size, src.shape[1] * size, _stream()), "gather_rows")


def wait_probe(polls: int, error_flag, gave_up=None):
    """One thread waits on an mbarrier that nobody arrives at, gives up after `polls` polls (at most 65,536) and
    raises error flag 3, exactly as the tensor-core kernels' bounded waits do; see csrc/library.cu."""
    _cuda(error_flag, gave_up)
    _check(lib().lia_wait_probe(int(polls), _p(error_flag), _p(gave_up), _stream()), "wait_probe")


def reset_scratch(device) -> None:
    """Zero the counters at the head of this device's split-K scratch: a product that gave up may have left
    them mid-count (every product that runs to its end leaves them at zero)."""
    key = torch.device(device).index or 0
    if key in _scratch:
        _scratch[key][:COUNTER_WORDS].zero_()


def gemm_simt(mode, a, w, out, alpha: float = 1.0, label=None, act: int = 0):
    """out[M, N] (op)= alpha * a[M, K] @ w[N, K]^T on the 32-bit pipes; see csrc/gemm_simt.cu."""
    _cuda(a, w, out)
    M, K = a.shape
    N = out.shape[1]
    rows_w = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or rows_w != (2 * N if mode == GEMM_SWIGLU else N):
        raise KernelError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    with _timed("gemm_simt", label, work=lambda: _gemm_work(a, w, out)):
        _check(lib().lia_gemm_simt(mode | (int(act) << 8), _p(a), dtype_code(a.dtype), a.stride(0), _p(w), dtype_code(w.dtype),
                                   w.stride(0), _p(out), dtype_code(out.dtype), out.stride(0), M, N, K, alpha,
                                   _stream()), "gemm_simt")


_SCRATCH_FLOATS = 16 << 20          # 64 MB of split-K scratch per device, allocated (zeroed) at first use
COUNTER_WORDS = 4096                # its first words are the split-K tile counters (csrc/gemm_tc.cu)
_scratch = {}
_sm_count = {}


def _device_scratch(device):
    key = (device.index if isinstance(device, torch.device) else torch.device(device).index) or 0
    if key not in _scratch:
        # zeroed: the first words are tile counters that every product leaves at zero again
        _scratch[key] = torch.zeros(_SCRATCH_FLOATS, dtype=torch.float32, device=device)
        _sm_count[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _scratch[key], _sm_count[key]


def gemm_tc_accepts(mode, a, w, out) -> bool:
    """Whether the tcgen05 kernel takes this product: bfloat16 operands, K and the row strides
    multiples of 8 elements (TMA needs 16-byte rows), 16-byte aligned bases."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype not in (torch.float32, torch.bfloat16):
        return False
    K = a.shape[1]
    return (K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc_tiles_fill_the_sms(a, out) -> bool:
    """Whether the product's output tiles (128 features each, all tokens of up to 256 in one) are at least
    three quarters as many as the device has SMs: the tcgen05 kernel then streams the weights with every SM at
    work without cutting K, whatever the number of tokens."""
    _, sms = _device_scratch(a.device)
    return 4 * ((out.shape[1] + 127) // 128) >= 3 * sms


def gemm_tc(mode, a, w, out, alpha: float = 1.0, error_flag=None, label=None, act: int = 0):
    """out[M, N] (op)= alpha * a[M, K] @ w[N, K]^T on the tensor cores; see csrc/gemm_tc.cu.  Products
    with few tiles split K and use this device's scratch, so calls on one device must not overlap.
    `act`: with GEMM_SWIGLU, ACT_RELU makes the gate a ReLU; with GEMM_STORE, ACT_RELU_SQUARED squares the result's ReLU."""
    M, K = a.shape
    N = out.shape[1]
    if w.shape[1] != K or out.shape[0] != M or w.shape[0] != (2 * N if mode == GEMM_SWIGLU else N):
        raise KernelError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    scratch, sms = _device_scratch(a.device)
    with _timed("gemm_tc", label, work=lambda: _gemm_work(a, w, out)):
        _check(lib().lia_gemm_tc(mode | (int(act) << 8), _p(a), a.stride(0), _p(w), w.stride(0), _p(out), dtype_code(out.dtype),
                                 out.stride(0), M, N, K, alpha, _p(scratch), scratch.numel(), sms, _p(error_flag),
                                 _stream()), "gemm_tc")


def gemm_cluster_accepts(mode, a, w, out) -> bool:
    """Whether the cluster kernel takes this product: what the tcgen05 kernel takes, and so few output
    tiles that at least two CTAs of a cluster can share each one's K."""
    if not gemm_tc_accepts(mode, a, w, out):
        return False
    _, sms = _device_scratch(a.device)
    return lib().lia_gemm_cluster_splits(mode, a.shape[0], out.shape[1], a.shape[1], sms) >= 2


def gemm_cluster(mode, a, w, out, alpha: float = 1.0, error_flag=None, label=None):
    """out[M, N] (op)= alpha * a[M, K] @ w[N, K]^T on the tensor cores with K cut over the CTAs of a
    thread-block cluster, partial sums meeting in distributed shared memory; see csrc/gemm_cluster.cu."""
    M, K = a.shape
    N = out.shape[1]
    if w.shape[1] != K or out.shape[0] != M or w.shape[0] != (2 * N if mode == GEMM_SWIGLU else N):
        raise KernelError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _, sms = _device_scratch(a.device)
    with _timed("gemm_cluster", label, work=lambda: _gemm_work(a, w, out)):
        _check(lib().lia_gemm_cluster(mode, _p(a), a.stride(0), _p(w), w.stride(0), _p(out), dtype_code(out.dtype),
                                      out.stride(0), M, N, K, alpha, sms, _p(error_flag), _stream()), "gemm_cluster")


SKINNY_MAX_TOKENS = 32


def gemm_skinny_accepts(mode, a, w, out) -> bool:
    """Whether the few-token kernel takes this product: bfloat16 operands, at most 32 tokens, K and the
    row strides multiples of 8 elements, 16-byte aligned bases (bulk copies and 16-byte loads)."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype not in (torch.float32, torch.bfloat16):
        return False
    M, K = a.shape
    return (M <= SKINNY_MAX_TOKENS and K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.stride(1) == 1 and w.stride(1) == 1 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny(mode, a, w, out, alpha: float = 1.0, error_flag=None, label=None):
    """out[M, N] (op)= alpha * a[M, K] @ w[N, K]^T for M <= 32 tokens: each CTA streams 16 rows of w over
    the whole of K; see csrc/gemm_skinny.cu."""
    M, K = a.shape
    N = out.shape[1]
    if w.shape[1] != K or out.shape[0] != M or w.shape[0] != (2 * N if mode == GEMM_SWIGLU else N):
        raise KernelError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    with _timed("gemm_skinny", label, work=lambda: _gemm_work(a, w, out)):
        _check(lib().lia_gemm_skinny(mode, _p(a), a.stride(0), _p(w), w.stride(0), _p(out), dtype_code(out.dtype),
                                     out.stride(0), M, N, K, alpha, _p(error_flag), _stream()), "gemm_skinny")


STREAM_MAX_TOKENS = 16
STREAM_NORM_MAX_K = 4096


def gemm_stream_accepts(mode, a, w, out, norm=False) -> bool:
    """Whether the persistent few-token kernel takes this product: bfloat16 weights, at most 16 tokens whose rows
    fit in shared memory beside a ring of two stages, K and the row strides multiples of 8 elements, 16-byte
    aligned bases.  `norm`: `a` is the 32-bit rows that the kernel norms itself (K at most 4,096)."""
    if w.dtype != torch.bfloat16 or out.dtype not in (torch.float32, torch.bfloat16):
        return False
    if a.dtype != (torch.float32 if norm else torch.bfloat16):
        return False
    M, K = a.shape
    if not (M <= STREAM_MAX_TOKENS and K % 64 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.stride(1) == 1 and w.stride(1) == 1 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        return False
    _, sms = _device_scratch(a.device)
    return lib().lia_gemm_stream_stages(mode, M, out.shape[1], K, 1 if norm else 0, sms) > 0


def gemm_stream(mode, a, w, out, alpha: float = 1.0, error_flag=None, label=None, norm_weight=None, eps: float = 0.0,
                stages_cap: int = 0, early_stages: int = 0, activation: int = 0):
    """out[M, N] (op)= alpha * x[M, K] @ w[N, K]^T for M <= 16 tokens, one persistent CTA per SM with the
    tokens' rows resident in shared memory; see csrc/gemm_stream.cu.  Without `norm_weight`, x = a (bfloat16);
    with it, a is 32-bit and x = RMSNorm(a; norm_weight, eps) rounded to bfloat16, computed inside the kernel.
    `activation` (STORE: ACT_GELU_TANH, ACT_SILU, ACT_RELU_SQUARED or ACT_RELU, applied to the 32-bit result before it is
    stored; SWIGLU: ACT_RELU makes the gate a ReLU)."""
    M, K = a.shape
    N = out.shape[1]
    if w.shape[1] != K or out.shape[0] != M or w.shape[0] != (2 * N if mode == GEMM_SWIGLU else N):
        raise KernelError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _, sms = _device_scratch(a.device)
    if norm_weight is None:
        x, ldx, src, ld_src, nw, nw_code = _p(a), a.stride(0), None, 0, None, 0
    else:
        if a.dtype != torch.float32 or norm_weight.numel() != K or not norm_weight.is_contiguous():
            raise KernelError("gemm_stream with a norm takes 32-bit rows and a weight of K elements")
        x, ldx, src, ld_src, nw, nw_code = None, 0, _p(a), a.stride(0), _p(norm_weight), dtype_code(norm_weight.dtype)
    with _timed("gemm_stream", label, work=lambda: _gemm_work(a, w, out)):
        _check(lib().lia_gemm_stream(mode, x, ldx, _p(w), w.stride(0), _p(out), dtype_code(out.dtype), out.stride(0),
                                     M, N, K, alpha, src, ld_src, nw, nw_code, eps, sms, stages_cap, early_stages, int(activation),
                                     _p(error_flag),
                                     _stream()), "gemm_stream")


ATTENTION_HEAD_DIM_STEP, ATTENTION_HEAD_DIM_MAX = 16, 256      # what csrc/attention_generic.cu takes


def attention_generic(q, k_pages, v_pages, positions, slots, block_table, out, nq, nkv, d, window, scale,
                      rows=None, error_flag=None, label=None, work_bytes=0):
    """Attention for every token of the batch, or for the tokens whose batch indices `rows` lists (row t of
    `out` is written for token t either way).  A visible key whose block-table entry names no page counts
    for nothing and raises error flag 2."""
    _cuda(q, k_pages, v_pages, positions, slots, block_table, out, rows, error_flag)
    if not (q.dtype == k_pages.dtype == v_pages.dtype == out.dtype):
        raise KernelError("attention: q, cache and out must have one element type")
    n = q.shape[0] if rows is None else rows.shape[0]
    with _timed("attention_generic", label, work_bytes):
        _check(lib().lia_attention_generic(_p(q), _p(k_pages), _p(v_pages), dtype_code(q.dtype), _p(positions),
                                           _p(slots), _p(block_table), block_table.shape[1], _p(rows), _p(out), n, nq,
                                           nkv, d, k_pages.shape[1], int(window or 0), scale, k_pages.shape[0],
                                           _p(error_flag), _stream()),
               "attention_generic")


DECODE_HEAD_DIMS = (32, 64, 128)       # head sizes the tensor-core attention kernels are built for


def attention_decode(q, k_pages, v_pages, rows, positions, slots, block_table, out, partial, nq, nkv, d, window,
                     scale, split_len, n_splits, counters=None, qkv=None, inv_freq=None, rotary_dim=0, write_kv=True,
                     error_flag=None, label=None, work_bytes=0, cluster=False, all_new=False, sink=False, softcap=None):
    """Split-key decode attention (bfloat16) for the single-token rows of the batch; see
    csrc/attention_decode.cu.  `partial` is 32-bit scratch for the ranges' partial results.
    `split_len` 0: every row cuts its own visible span into `n_splits` ranges.  `counters` (int32, at
    least rows * kv_heads * ceil(group / 16) words, zero before the first call; every call leaves them
    zero) lets the CTA that finishes a token last combine its ranges; without them (or with more than
    128 ranges) a second kernel does.  With `qkv` (32-bit q|k|v rows of the step, at most 16 query heads per
    kv head) `q` may be None: the kernel takes the queries from `qkv`, applies the rotary encoding
    (`inv_freq`, `rotary_dim`; 0: none) and, if `write_kv`, appends each token's key and value to the cache
    itself, so no separate position-encoding kernel runs.  `cluster`: `n_splits` came from
    `attention_decode_cluster_splits`; the ranges of a token then meet in distributed shared memory and neither
    `partial` nor `counters` is used.  `all_new`: the rows may be tokens of this step's prompt portions, so any of
    their keys may have been written by the kernels ahead (otherwise only a row's own key is taken to be of this step,
    and the kernel fetches older tiles before it waits for those kernels).  `sink`: one is added to the softmax's denominator
    (a key of score 0 without a value), once, where a token's ranges meet.  `softcap`: the scores pass
    cap * tanh(score / cap) ahead of the softmax (the hardware's tanh approximation)."""
    _cuda(q, k_pages, v_pages, rows, positions, slots, block_table, out, partial, counters, qkv, inv_freq, error_flag)
    if qkv is not None:
        if qkv.dtype != torch.float32 or qkv.shape[1] != (nq + 2 * nkv) * d:
            raise KernelError("attention_decode: qkv must be 32-bit q|k|v rows")
        q = out if q is None else q             # unused by the kernel then; only its element type is checked
    if counters is not None and (counters.dtype != torch.int32
                                 or counters.numel() < rows.shape[0] * nkv * ((nq // nkv + 15) // 16)):
        raise KernelError("attention_decode: counters must be int32, one per row and head group")
    if not (q.dtype == k_pages.dtype == v_pages.dtype == out.dtype == torch.bfloat16):
        raise KernelError("attention_decode is a bfloat16 kernel")
    with _timed("attention_decode", label, work_bytes):
        _check(lib().lia_attention_decode(_p(q), _p(k_pages), _p(v_pages), _p(rows), rows.shape[0], _p(positions),
                                          _p(slots), _p(block_table), block_table.shape[1], _p(out), _p(partial),
                                          0 if partial is None else partial.numel(), _p(counters), q.shape[0], nq, nkv, d,
                                          k_pages.shape[1], int(window or 0), scale, split_len, n_splits, _p(qkv), _p(inv_freq),
                                          int(rotary_dim), 1 if write_kv else 0, k_pages.shape[0], 1 if cluster else 0, 1 if all_new else 0,
                                          1 if sink else 0, float(softcap or 0.0), _p(error_flag),
                                          _stream()),
               "attention_decode")


def attention_decode_cluster_splits(d: int, group: int, clusters: int, wanted: int) -> int:
    """Ranges per token (2, 4, 8 or 16, at most `wanted`) with which `attention_decode(..., cluster=True)` can
    serve `clusters` (token, head group) pairs at once; 1: it cannot (one range, or too many clusters for the device)."""
    return int(lib().lia_attention_decode_cluster_splits(d, group, clusters, wanted))


def attention_decode_ctas_per_sm(d: int, group: int) -> int:
    """CTAs of `attention_decode` that one SM holds at once for this head size (0: unknown)."""
    return int(lib().lia_attention_decode_ctas_per_sm(d, group))


def attention_prefill_tokens_per_tile(group: int) -> int:
    """Tokens of a portion that one CTA of the prefill kernel takes (0: group size not supported)."""
    return 64 // group if 1 <= group <= 64 else 0


def attention_prefill(q, k_pages, v_pages, segments, n_segments, n_tiles, slots, block_table, out, nq, nkv, d,
                      window, scale, error_flag=None, label=None, work_flops=0, sink=False):
    """Tensor-core attention (bfloat16) for the prompt portions listed in `segments`
    ([n_segments, 3] int32: first batch index, first position, count); see csrc/attention_prefill.cu."""
    _cuda(q, k_pages, v_pages, segments, slots, block_table, out, error_flag)
    if not (q.dtype == k_pages.dtype == v_pages.dtype == out.dtype == torch.bfloat16):
        raise KernelError("attention_prefill is a bfloat16 kernel")
    with _timed("attention_prefill", label, 0, work_flops):
        _check(lib().lia_attention_prefill(_p(q), _p(k_pages), _p(v_pages), _p(segments), n_segments, n_tiles,
                                           _p(slots), _p(block_table), block_table.shape[1], _p(out), nq, nkv, d,
                                           k_pages.shape[1], int(window or 0), scale, k_pages.shape[0], 1 if sink else 0,
                                           _p(error_flag), _stream()), "attention_prefill")


def attention_prefill_tc_tokens_per_tile(group: int, d: int) -> int:
    """Tokens of a portion that one CTA of the tcgen05 prefill kernel takes (0: it does not take this group
    size or head size)."""
    return int(lib().lia_attention_prefill_tc_tokens_per_tile(group, d))


def attention_prefill_tc(q, k_pages, v_pages, segments, n_segments, n_tiles, slots, block_table, out, nq, nkv, d,
                         window, scale, error_flag=None, label=None, work_flops=0, splits=1, partial=None, sink=False,
                         softcap=None):
    """Prompt-portion attention on the tcgen05 tensor cores (bfloat16, head size 64 or 128, heads per kv head a
    divisor of 128); see csrc/attention_prefill_tc.cu.  Arguments as `attention_prefill`.  `splits` > 1 cuts every
    CTA's keys into that many ranges that run side by side and are merged by a second kernel; `partial` is their
    32-bit scratch, `attention_prefill_tc_partial_floats` words long."""
    _cuda(q, k_pages, v_pages, segments, slots, block_table, out, error_flag, partial)
    if not (q.dtype == k_pages.dtype == v_pages.dtype == out.dtype == torch.bfloat16):
        raise KernelError("attention_prefill_tc is a bfloat16 kernel")
    splits = int(splits)
    if splits > 1 and (partial is None or partial.dtype != torch.float32
                       or partial.numel() < attention_prefill_tc_partial_floats(q.shape[0], nq, d, splits)):
        raise KernelError("attention_prefill_tc: the ranges need 32-bit scratch of attention_prefill_tc_partial_floats words")
    with _timed("attention_prefill_tc", label, 0, work_flops):
        _check(lib().lia_attention_prefill_tc(_p(q), _p(k_pages), _p(v_pages), _p(segments), n_segments, n_tiles,
                                              _p(slots), _p(block_table), block_table.shape[1], _p(out), nq, nkv, d,
                                              k_pages.shape[1], int(window or 0), scale, k_pages.shape[0], splits,
                                              _p(partial) if splits > 1 else None, q.shape[0], 1 if sink else 0,
                                              float(softcap or 0.0), _p(error_flag), _stream()),
               "attention_prefill_tc")


def attention_prefill_tc_partial_floats(n_tokens: int, nq: int, d: int, splits: int) -> int:
    return int(splits) * int(n_tokens) * int(nq) * (int(d) + 2)


_select_scratch = {}


def select_tokens(logits, out, temperature=None, seeds=None, positions=None):
    _cuda(logits, out, temperature, seeds, positions)
    rows, vocab = logits.shape
    if logits.dtype != torch.float32 or out.dtype != torch.int32:
        raise KernelError("select_tokens takes 32-bit logits and writes int32 tokens")
    if temperature is not None and (seeds is None or positions is None):
        raise KernelError("select_tokens: temperature needs seeds and positions")
    key = torch.device(logits.device).index or 0
    fn = lib().lia_select_tokens_scratch_floats
    fn.restype = ctypes.c_longlong
    need = int(fn(rows, vocab))
    scratch = _select_scratch.get(key)
    if scratch is None or scratch.numel() < need:
        # zeroed: its head holds the rows' counters, which every call leaves at zero
        scratch = _select_scratch[key] = torch.zeros(max(need, 1 << 18), dtype=torch.float32, device=logits.device)
    with _timed("select_tokens"):
        _check(lib().lia_select_tokens(_p(logits), logits.stride(0), vocab, _p(temperature), _p(seeds),
                                       _p(positions), _p(out), rows, _p(scratch), scratch.numel(), _stream()), "select_tokens")


CANDIDATES_MAX = 32


def select_candidates(logits, k: int, out_values, out_ids, nonfinite, temperature=None, mass=None):
    """The best k logits of every row and their token ids, best first (larger logit, then larger id; minus
    infinity is no candidate, missing ones have id -1): what the host's sampling rule needs of a row when it
    keeps at most k tokens.  `nonfinite` (int32[1]) is increased by the number of NaN and infinite logits.
    With `temperature` (float64 [rows]) also `mass` (float64 [rows, 2]): the row's largest logit and the sum of
    exp((x - largest) / temperature) over the whole row in 64-bit, which bounds what the candidates leave out."""
    _cuda(logits, out_values, out_ids, nonfinite)
    rows, vocab = logits.shape
    if (temperature is None) != (mass is None):
        raise KernelError("select_candidates: temperature and mass come together")
    if temperature is not None:
        _cuda(temperature, mass)
        if temperature.dtype != torch.float64 or mass.dtype != torch.float64 or temperature.numel() != rows \
                or tuple(mass.shape) != (rows, 2) or not mass.is_contiguous() or not temperature.is_contiguous():
            raise KernelError("select_candidates: temperature is float64 [rows], mass float64 [rows, 2]")
    if logits.dtype != torch.float32 or out_values.dtype != torch.float32 or out_ids.dtype != torch.int32:
        raise KernelError("select_candidates takes 32-bit logits and writes float32 values and int32 ids")
    if tuple(out_values.shape) != (rows, k) or tuple(out_ids.shape) != (rows, k) or nonfinite.dtype != torch.int32:
        raise KernelError("select_candidates: outputs must be [rows, k]")
    key = torch.device(logits.device).index or 0
    fn = lib().lia_select_candidates_scratch_floats
    fn.restype = ctypes.c_longlong
    need = int(fn(rows, vocab, k))
    scratch = _select_scratch.get(key)
    if scratch is None or scratch.numel() < need:
        scratch = _select_scratch[key] = torch.zeros(max(need, 1 << 18), dtype=torch.float32, device=logits.device)
    with _timed("select_candidates"):
        _check(lib().lia_select_candidates(_p(logits), logits.stride(0), vocab, rows, k, _p(out_values), _p(out_ids),
                                           _p(nonfinite), _p(temperature), _p(mass), _p(scratch), scratch.numel(),
                                           _stream()), "select_candidates")


# ---- parts that other attention designs bring: pairwise rotary encoding, attention with sigmoid weights, a short
# ---- causal convolution behind the norm, learned positions, a re-injection of the embedding output

def embedding_positions(tokens, positions, table, position_table, out, scale: float, copy=None, error_flag=None):
    """out[t] = table[token_t] * scale + position_table[position_t] (32-bit); `copy` receives the same rows; see
    csrc/residual_ops.cu."""
    _cuda(tokens, positions, table, position_table, out, copy, error_flag)
    n, hidden = out.shape
    if table.dtype != position_table.dtype or position_table.shape[1] != hidden or table.shape[1] != hidden:
        raise KernelError("embedding_positions: both tables must have one element type and the stream's width")
    if out.dtype != torch.float32 or (copy is not None and (copy.dtype != torch.float32 or copy.shape != out.shape)):
        raise KernelError("embedding_positions writes 32-bit rows")
    with _timed("embedding"):
        _check(lib().lia_embedding_positions(_p(tokens), _p(positions), _p(table), _p(position_table),
                                             dtype_code(table.dtype), _p(out), _p(copy), n, hidden, table.shape[0],
                                             position_table.shape[0], scale, _p(error_flag), _stream()),
               "embedding_positions")


def reinject_input(x, x0, bias, side_by_side):
    """side_by_side[t] = [x[t], x0[t]] in its own element type, then x[t] = bias; see csrc/residual_ops.cu."""
    _cuda(x, x0, bias, side_by_side)
    n, hidden = x.shape
    if x.dtype != torch.float32 or x0.dtype != torch.float32 or x0.shape != x.shape or \
            tuple(side_by_side.shape) != (n, 2 * hidden) or (bias is not None and bias.numel() != hidden):
        raise KernelError("reinject_input: 32-bit streams of one shape, an output twice as wide, a bias of the width")
    with _timed("reinject_input"):
        _check(lib().lia_reinject_input(_p(x), _p(x0), _p(bias), dtype_code(bias.dtype) if bias is not None else F32,
                                        _p(side_by_side), dtype_code(side_by_side.dtype), n, hidden, _stream()),
               "reinject_input")


SHORT_CONV_MAX_TAPS = 8


def short_conv(x, norm_weight, taps0, taps1, positions, slots, state, tail, out0, out1, eps: float, single: bool):
    """RMSNorm of the 32-bit rows `x` and a short causal convolution of the normed rows for up to two readers
    (`taps0` -> `out0`, `taps1` -> `out1`; either pair may be None), carrying each request's last taps - 1 normed rows
    in `state` [slots, taps - 1, width]; see csrc/short_conv.cu.  `single`: every request of the step brings one
    token; otherwise `tail` ([tokens, width] 32-bit scratch) is needed."""
    _cuda(x, norm_weight, taps0, taps1, positions, slots, state, tail, out0, out1)
    n, width = x.shape
    given = [t for t in (taps0, taps1) if t is not None]
    outs = [o for o in (out0, out1) if o is not None]
    if not given or (taps0 is None) != (out0 is None) or (taps1 is None) != (out1 is None):
        raise KernelError("short_conv: taps and outputs come in pairs, at least one")
    taps = given[0].shape[1]
    if any(t.shape != (width, taps) or t.dtype != norm_weight.dtype for t in given) or x.dtype != torch.float32:
        raise KernelError("short_conv: taps are [width, taps] of the norm weight's element type, x is 32-bit")
    if any(o.shape != x.shape or o.dtype != outs[0].dtype for o in outs):
        raise KernelError("short_conv: outputs have the shape of x and one element type")
    if taps > 1 and (state is None or state.dtype != torch.float32 or tuple(state.shape[1:]) != (taps - 1, width)):
        raise KernelError("short_conv: state must be 32-bit [slots, taps - 1, width]")
    if taps > 1 and not single and (tail is None or tail.dtype != torch.float32 or tail.shape != x.shape):
        raise KernelError("short_conv: a step with runs of several tokens needs 32-bit scratch of x's shape")
    with _timed("short_conv", nbytes=x.numel() * 4 + sum(o.numel() * o.element_size() for o in outs)):
        _check(lib().lia_short_conv(_p(x), _p(norm_weight), _p(taps0), _p(taps1), dtype_code(norm_weight.dtype),
                                    _p(positions), _p(slots), _p(state), _p(tail), _p(out0), _p(out1),
                                    dtype_code(outs[0].dtype), n, width, taps, eps, 1 if single else 0,
                                    _device_scratch(x.device)[1], _stream()),
               "short_conv")


def rotary_pairs_kv_write(rows, positions, slots, block_table, q_out, k_pages, v_pages, nq, nkv, d, dv, rotary_dim, freq,
                          magnitude: float = 1.0, write_kv=True, error_flag=None):
    """Rotary encoding over adjacent pairs of q and k (rows: 32-bit [tokens, >= (nq + nkv) d + nkv dv]) and append
    of k and v to the pages; see csrc/rotary_pairs.cu."""
    _cuda(rows, positions, slots, block_table, q_out, k_pages, v_pages, freq, error_flag)
    if rows.dtype != torch.float32 or rows.shape[1] < (nq + nkv) * d + nkv * dv:
        raise KernelError("rotary_pairs_kv_write takes 32-bit rows of q, k and v heads")
    if q_out.dtype != k_pages.dtype or k_pages.dtype != v_pages.dtype:
        raise KernelError("rotary_pairs_kv_write: q and the cache must have one element type")
    if tuple(k_pages.shape[2:]) != (nkv, d) or tuple(v_pages.shape[2:]) != (nkv, dv):
        raise KernelError("rotary_pairs_kv_write: the pages do not have the heads' sizes")
    with _timed("rotary_pairs_kv_write"):
        _check(lib().lia_rotary_pairs_kv_write(_p(rows), rows.stride(0), _p(positions), _p(slots), _p(block_table),
                                               block_table.shape[1], _p(q_out), _p(k_pages), _p(v_pages),
                                               dtype_code(q_out.dtype), rows.shape[0], nq, nkv, d, dv, int(rotary_dim),
                                               _p(freq), float(magnitude), k_pages.shape[1], k_pages.shape[0],
                                               1 if write_kv else 0, _p(error_flag), _stream()),
               "rotary_pairs_kv_write")


def sigmoid_attention_generic(q, k_pages, v_pages, positions, slots, block_table, out, nq, nkv, d, dv, window, chunk,
                              scale, head_bias=None, gate=None, gate_stride=0, rows=None, error_flag=None, label=None,
                              work_bytes=0):
    """Attention with sigmoid weights (no softmax) for every token of the batch or for the batch indices in `rows`;
    see csrc/sigmoid_attention.cu.  `head_bias` [nq] 32-bit is added to every score of its head; `gate` is a 32-bit
    tensor in which token t's head h has its output-gate logit at flat index t * gate_stride + h."""
    _cuda(q, k_pages, v_pages, positions, slots, block_table, out, rows, head_bias, error_flag)
    if not (q.dtype == k_pages.dtype == v_pages.dtype == out.dtype):
        raise KernelError("attention: q, cache and out must have one element type")
    if head_bias is not None and (head_bias.dtype != torch.float32 or head_bias.numel() != nq):
        raise KernelError("sigmoid attention: head_bias must be 32-bit, one per query head")
    if gate is not None and (gate.dtype != torch.float32 or not gate.is_cuda):
        raise KernelError("sigmoid attention: gate logits must be 32-bit")
    n = q.shape[0] if rows is None else rows.shape[0]
    with _timed("sigmoid_attention_generic", label, work_bytes):
        _check(lib().lia_sigmoid_attention_generic(_p(q), _p(k_pages), _p(v_pages), dtype_code(q.dtype), _p(positions),
                                                   _p(slots), _p(block_table), block_table.shape[1], _p(rows), _p(out),
                                                   n, nq, nkv, d, dv, k_pages.shape[1], int(window or 0), int(chunk or 0),
                                                   scale, _p(head_bias), _p(gate), int(gate_stride), k_pages.shape[0],
                                                   _p(error_flag), _stream()),
               "sigmoid_attention_generic")


def sigmoid_attention_tc_tokens_per_tile(group: int, d: int, dv: int) -> int:
    """Tokens of a portion that one CTA of the tcgen05 sigmoid attention kernel takes (0: it does not take the sizes)."""
    return int(lib().lia_sigmoid_attention_tc_tokens_per_tile(int(group), int(d), int(dv)))


def sigmoid_attention_tc_accepts(group: int, d: int, dv: int) -> bool:
    """Whether the tensor-core kernel for sigmoid attention takes these sizes (bfloat16): head sizes of keys and of
    values that are multiples of 8 up to 128, and at most 128 query heads per kv head."""
    return sigmoid_attention_tc_tokens_per_tile(group, d, dv) > 0


def sigmoid_attention_tc_tiles(segments, per_tile: int) -> int:
    """CTAs per kv head that the portions of several tokens among `segments` ((slot, start, count, offset)) take."""
    return sum((count + per_tile - 1) // per_tile for _, _, count, _ in segments if count > 1)


def sigmoid_attention_tc(q, k_pages, v_pages, segments, n_segments, portion_tiles, single_rows, positions, slots,
                         block_table, out, nq, nkv, d, dv, window, chunk, scale, head_bias=None, gate=None, gate_stride=0,
                         error_flag=None, label=None, work_bytes=0, work_flops=0, fused_rows=None, freq=None, rotary_dim=0,
                         magnitude=1.0, write_kv=True, splits=1, partial=None):
    """Sigmoid attention on the tcgen05 tensor cores (bfloat16) for the portions listed in `segments` ([n_segments, 3]
    int32: first batch index, first position, count) and the single tokens whose batch indices `single_rows` lists;
    see csrc/sigmoid_attention_tc.cu.  With `fused_rows` (a step of single tokens only: the 32-bit rows of q, k and v
    heads that the product before left, `q` may be None) the kernel applies the pairwise rotary encoding (`freq`,
    `rotary_dim`, `magnitude`) to the queries and the key itself and, with `write_kv`, appends key and value to the pages:
    no position-encoding kernel runs.  `splits` > 1 (a step without portions): every token's key tiles are cut into that
    many ranges that run side by side and a second kernel adds them; `partial` is their 32-bit scratch of
    splits * out.shape[0] * nq * dv words."""
    _cuda(q, k_pages, v_pages, segments, single_rows, positions, slots, block_table, out, head_bias, error_flag, freq, partial)
    splits = int(splits)
    if splits > 1 and (partial is None or partial.dtype != torch.float32 or partial.numel() < splits * out.shape[0] * nq * dv):
        raise KernelError("sigmoid_attention_tc: the ranges need 32-bit scratch of splits * tokens * heads * head size words")
    if not (k_pages.dtype == v_pages.dtype == out.dtype == torch.bfloat16) or (q is not None and q.dtype != torch.bfloat16):
        raise KernelError("sigmoid_attention_tc is a bfloat16 kernel")
    if tuple(k_pages.shape[2:]) != (nkv, d) or tuple(v_pages.shape[2:]) != (nkv, dv) or out.shape[1] != nq * dv or \
            (q is not None and q.shape[1] != nq * d):
        raise KernelError("sigmoid_attention_tc: q, out and the pages do not have the heads' sizes")
    if head_bias is not None and (head_bias.dtype != torch.float32 or head_bias.numel() != nq):
        raise KernelError("sigmoid attention: head_bias must be 32-bit, one per query head")
    if gate is not None and (gate.dtype != torch.float32 or not gate.is_cuda):
        raise KernelError("sigmoid attention: gate logits must be 32-bit")
    if fused_rows is None and q is None:
        raise KernelError("sigmoid_attention_tc needs q or the rows to encode")
    if fused_rows is not None and (fused_rows.dtype != torch.float32 or not fused_rows.is_cuda or fused_rows.stride(1) != 1
                                   or (freq is not None and freq.dtype != torch.float32)):
        raise KernelError("sigmoid_attention_tc: the rows to encode and the frequencies must be 32-bit")
    n_single = 0 if single_rows is None else single_rows.numel()
    with _timed("sigmoid_attention_tc", label, work_bytes, work_flops):
        _check(lib().lia_sigmoid_attention_tc(_p(q), _p(k_pages), _p(v_pages), _p(segments), int(n_segments),
                                              int(portion_tiles), _p(single_rows), n_single, _p(positions), _p(slots),
                                              _p(block_table), block_table.shape[1], _p(out), nq, nkv, d, dv,
                                              k_pages.shape[1], int(window or 0), int(chunk or 0), scale, _p(head_bias),
                                              _p(gate), int(gate_stride), k_pages.shape[0], _p(fused_rows),
                                              0 if fused_rows is None else fused_rows.stride(0), _p(freq), int(rotary_dim),
                                              float(magnitude), 1 if write_kv else 0, splits, _p(partial) if splits > 1 else None,
                                              out.shape[0], _p(error_flag), _stream()),
               "sigmoid_attention_tc")


# ---- parts of decoders with a norm on both sides of a sublayer, attention through a latent, attention with a sink,
# ---- and a recurrent mixer with input-dependent decay

ACT_NONE, ACT_GELU_TANH, ACT_SILU, ACT_RELU_SQUARED, ACT_RELU = 0, 1, 2, 3, 4


def _f32(*tensors):
    for t in tensors:
        if t is not None and t.dtype != torch.float32:
            raise KernelError("this kernel takes its 32-bit operands as float32 tensors")


def norm_residual(y, weight, residual, eps: float, bias=None, next_weight=None, next_out=None, next_eps: float = 0.0):
    """residual += rms(y + bias) * weight; with `next_out` also next_out = rms(residual) * next_weight, in one pass over
    the rows; see csrc/norm_residual.cu.  y, residual, the weights and the bias are 32-bit."""
    _cuda(y, weight, residual, bias, next_weight, next_out)
    _f32(y, weight, residual, bias, next_weight)
    rows, hidden = residual.shape
    if tuple(y.shape) != (rows, hidden) or weight.numel() != hidden or (bias is not None and bias.numel() != hidden) or \
            (next_out is not None and (next_weight is None or next_weight.numel() != hidden or tuple(next_out.shape) != (rows, hidden))):
        raise KernelError("norm_residual: rows of one width, weights and bias of that width")
    with _timed("norm_residual", nbytes=(3 + (1 if next_out is not None else 0)) * rows * hidden * 4):
        _check(lib().lia_norm_residual(_p(y), _p(bias), _p(weight), _p(residual), _p(next_weight), _p(next_out),
                                       dtype_code(next_out.dtype) if next_out is not None else F32, rows, hidden, eps,
                                       next_eps, _stream()), "norm_residual")


def activation_rows(source, out, act: int = ACT_NONE, gated: bool = False):
    """out[r, :] = act(source[r, :]) for 32-bit rows `source` (any row stride); with `gated` the rows hold a gate half and
    then another half of out's width, out = act(gate) * the other half; see csrc/norm_residual.cu."""
    if not (source.is_cuda and out.is_cuda) or source.dtype != torch.float32 or source.dim() != 2 or out.dim() != 2 or \
            source.shape[0] != out.shape[0] or source.shape[1] != (2 if gated else 1) * out.shape[1] or \
            source.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("activation_rows: 32-bit rows in, rows of the same shape (gated: of half the width) out")
    with _timed("activation_rows", nbytes=source.numel() * 4 + out.numel() * out.element_size()):
        _check(lib().lia_activation_rows(_p(source), source.stride(0), _p(out), dtype_code(out.dtype), out.stride(0),
                                         out.shape[0], out.shape[1], int(act), 1 if gated else 0, _stream()),
               "activation_rows")


def attention_general(q1, q1_strides, q2, q2_strides, k1_pages, k2_pages, v_pages, v_stride, dv, positions, slots,
                      block_table, out, out_strides, n_tokens, nq, nkv, window, scale, sink=False, rows=None,
                      error_flag=None, label=None, work_bytes=0, softcap=None):
    """Softmax attention whose keys come in up to two parts (k1 [pages, page, nkv, dk1] with q1, k2 [.., dk2] with q2; k2
    and q2 may be None) and whose values are the first `dv` of every `v_stride` elements of `v_pages`; q1, q2 and out
    are addressed by (token stride, head stride) in elements; `sink` adds one to the denominator; `softcap`: the scores
    pass cap * tanh(score / cap) ahead of the softmax; see
    csrc/attention_generic.cu.  For every token of the batch, or for the batch indices `rows`."""
    _cuda(k1_pages, k2_pages, v_pages, positions, slots, block_table, rows, error_flag)
    for t in (q1, q2, out):
        if t is not None and not t.is_cuda:
            raise KernelError("kernels need CUDA tensors")
    if not (q1.dtype == k1_pages.dtype == v_pages.dtype == out.dtype) or (k2_pages is not None and
                                                                          (q2 is None or q2.dtype != q1.dtype or k2_pages.dtype != q1.dtype)):
        raise KernelError("attention: q, cache and out must have one element type")
    dk1 = k1_pages.shape[-1]
    dk2 = 0 if k2_pages is None else k2_pages.shape[-1]
    n = n_tokens if rows is None else rows.shape[0]
    q2s = q2_strides if q2 is not None else (0, 0)
    with _timed("attention_general", label, work_bytes):
        _check(lib().lia_attention_general(_p(q1), q1_strides[0], q1_strides[1], _p(q2), q2s[0], q2s[1], _p(k1_pages), dk1,
                                           _p(k2_pages), dk2, _p(v_pages), int(v_stride), int(dv), dtype_code(q1.dtype),
                                           _p(positions), _p(slots), _p(block_table), block_table.shape[1], _p(rows),
                                           _p(out), out_strides[0], out_strides[1], n, nq, nkv, k1_pages.shape[1],
                                           int(window or 0), scale, float(softcap or 0.0), 1 if sink else 0, k1_pages.shape[0], _p(error_flag),
                                           _stream()), "attention_general")


def qkv_prepare(rows, bias, q_norm, k_norm, eps, freq, rot_dims, vmix_mode, vmix_lambda, v_first, positions, slots,
                block_table, q_out, k_pages, v_pages, nq, nkv, d, dv, write_kv=True, error_flag=None, norm_whole=False):
    """Bias, per-head RMS norm of q and k, rotate-half encoding, value mixing and the append to the pages for the
    32-bit rows [q | k | v] of a product; see csrc/qk_prepare.cu.  `norm_whole`: one RMS norm over all of q's elements and
    one over all of k's instead (weights [nq d] and [nkv d])."""
    _cuda(bias, q_norm, k_norm, freq, v_first, positions, slots, block_table, q_out, k_pages, v_pages, error_flag)
    _f32(rows, bias, q_norm, k_norm, freq, v_first)
    if not rows.is_cuda or rows.stride(1) != 1 or rows.shape[1] < (nq + nkv) * d + nkv * dv:
        raise KernelError("qkv_prepare takes 32-bit rows of q, k and v heads")
    if not (q_out.dtype == k_pages.dtype == v_pages.dtype) or tuple(k_pages.shape[2:]) != (nkv, d) or \
            tuple(v_pages.shape[2:]) != (nkv, dv) or tuple(q_out.shape) != (rows.shape[0], nq * d):
        raise KernelError("qkv_prepare: q and the pages must have one element type and the heads' sizes")
    with _timed("qkv_prepare"):
        _check(lib().lia_qkv_prepare(_p(rows), rows.stride(0), _p(bias), _p(q_norm), _p(k_norm), float(eps), _p(freq),
                                     int(rot_dims), int(vmix_mode), float(vmix_lambda), _p(v_first), _p(positions),
                                     _p(slots), _p(block_table), block_table.shape[1], _p(q_out), _p(k_pages), _p(v_pages),
                                     dtype_code(q_out.dtype), rows.shape[0], nq, nkv, d, dv, k_pages.shape[1],
                                     k_pages.shape[0], 1 if write_kv else 0, 1 if norm_whole else 0, _p(error_flag), _stream()),
               "qkv_prepare")


def latent_prepare(q_rows, shared_rows, latent_norm, eps, freq, rot_dims, positions, slots, block_table, q_plain,
                   q_rotated, latent_pages, key_pages, heads, d, dr, rank, write_kv=True, error_flag=None, pairs=False):
    """For attention through a latent: norm and append of the latent, encoding and append of the shared key part,
    the queries' unrotated parts as planes [heads, tokens, d] and their rotated parts encoded [tokens, heads dr]; see
    csrc/qk_prepare.cu.  `pairs`: the rotation pairs element 2i with 2i + 1 (else i with i + rot_dims / 2).
    `shared_rows` None: only the queries are prepared (the pages are filled by another layer)."""
    _cuda(latent_norm, freq, positions, slots, block_table, q_plain, q_rotated, latent_pages, key_pages, error_flag)
    _f32(q_rows, shared_rows, latent_norm, freq)
    n = q_rows.shape[0]
    if q_rows.stride(1) != 1 or q_rows.shape[1] < heads * (d + dr):
        raise KernelError("latent_prepare takes 32-bit query rows of one step")
    if shared_rows is not None and (shared_rows.stride(1) != 1 or shared_rows.shape[1] < rank + dr or
                                    shared_rows.shape[0] != n or latent_norm is None):
        raise KernelError("latent_prepare takes 32-bit shared rows of the step and the latent's norm weight")
    if not (q_plain.dtype == q_rotated.dtype == latent_pages.dtype == key_pages.dtype) or q_plain.numel() != heads * n * d \
            or q_rotated.numel() != n * heads * dr or latent_pages.shape[-1] != rank or key_pages.shape[-1] != dr:
        raise KernelError("latent_prepare: outputs and pages must have one element type and the parts' sizes")
    with _timed("latent_prepare"):
        _check(lib().lia_latent_prepare(_p(q_rows), q_rows.stride(0), _p(shared_rows),
                                        0 if shared_rows is None else shared_rows.stride(0),
                                        _p(latent_norm), float(eps), _p(freq), int(rot_dims), _p(positions), _p(slots),
                                        _p(block_table), block_table.shape[1], _p(q_plain), _p(q_rotated),
                                        _p(latent_pages), _p(key_pages), dtype_code(q_plain.dtype), n, heads, d, dr, rank,
                                        latent_pages.shape[1], latent_pages.shape[0],
                                        1 if write_kv and shared_rows is not None else 0, 1 if pairs else 0,
                                        _p(error_flag), _stream()), "latent_prepare")


CONV_MAX_TAPS = 8
SCAN_MAX_STATES = 256


def causal_conv(x, taps_weight, bias, state, positions, slots, out, out_copy=None, act: int = 0, update_single: bool = False):
    """out[t, c] = act(bias[c] + sum_j taps[c, j] x[t - n + 1 + j, c]) along each request's run, earlier inputs from
    `state` [slots, n - 1, channels]; `x` 32-bit rows (any stride, the first `channels` columns); act 1: SiLU.  The
    state is read, not changed: `conv_state_update` follows; except with `update_single` (every run of the step is a
    single token), where the kernel leaves the new state itself.  See csrc/selective_scan.cu."""
    _cuda(taps_weight, bias, positions, slots, out, out_copy)
    _f32(x, taps_weight, bias, state, out)
    n, channels = out.shape
    taps = taps_weight.shape[1]
    if x.stride(1) != 1 or x.shape[0] != n or x.shape[1] < channels or taps_weight.shape[0] != channels or \
            (taps > 1 and (tuple(state.shape[1:]) != (taps - 1, channels) or not state[0].is_contiguous())):
        raise KernelError("causal_conv: rows of at least `channels` columns, taps [channels, n], state [slots, n - 1, channels]")
    with _timed("causal_conv", nbytes=2 * n * channels * 4):
        _check(lib().lia_causal_conv(_p(x), x.stride(0), _p(taps_weight), _p(bias), _p(state),
                                     state.stride(0) if state is not None else 0, _p(positions), _p(slots),
                                     _p(out), _p(out_copy), dtype_code(out_copy.dtype) if out_copy is not None else F32, n,
                                     channels, taps, int(act), 1 if update_single else 0, _stream()), "causal_conv")


def conv_state_update(x, state, positions, slots, channels: int):
    """state[slot] <- the last taps - 1 inputs of the slot's run in this step (older ones kept from the state)."""
    _cuda(positions, slots)
    _f32(x, state)
    taps = state.shape[1] + 1
    if not state[0].is_contiguous():
        raise KernelError("conv_state_update: a slot's state must be contiguous")
    with _timed("conv_state_update"):
        _check(lib().lia_conv_state_update(_p(x), x.stride(0), _p(state), state.stride(0), _p(positions), _p(slots),
                                           x.shape[0], channels, taps, _stream()), "conv_state_update")


def selective_scan_chunk_floats(n_tokens: int, n_segments: int, channels: int, states: int) -> int:
    """Words of 32-bit scratch with which `selective_scan` cuts a step's portions into chunks that run side by side."""
    fn = lib().lia_selective_scan_chunk_floats
    fn.restype = ctypes.c_longlong
    return int(fn(int(n_tokens), int(n_segments), int(channels), int(states)))


def selective_scan(x, dt_raw, dt_bias, A, bc, b_offset, c_offset, D, z, state, segments, n_segments, single_rows, slots, out,
                   chunk_scratch=None):
    """The recurrence S <- exp(dt A) S + dt x B, y = (S C + D x) silu(z) with dt = softplus(dt_raw + dt_bias), along the
    step's runs (`segments` [n, 3] and `single_rows`), state [slots, channels, states] 32-bit; see csrc/selective_scan.cu.
    With `chunk_scratch` (32-bit, `selective_scan_chunk_floats` words) the portions are cut into chunks of 64 tokens that
    run side by side: a pass from zero states, a carry along each portion, a pass from the true start states."""
    _cuda(x, dt_raw, dt_bias, A, D, segments, single_rows, slots, out, chunk_scratch)
    _f32(x, dt_raw, dt_bias, A, bc, D, z, state, chunk_scratch)
    n, channels = x.shape
    states = A.shape[1]
    n_single = 0 if single_rows is None else single_rows.numel()
    if tuple(dt_raw.shape) != (n, channels) or tuple(A.shape) != (channels, states) or bc.stride(1) != 1 or z.stride(1) != 1 \
            or tuple(state.shape[1:]) != (channels, states) or not state[0].is_contiguous() or tuple(out.shape) != (n, channels):
        raise KernelError("selective_scan: shapes do not agree")
    with _timed("selective_scan", nbytes=n * channels * (12 + out.element_size())):
        _check(lib().lia_selective_scan(_p(x), _p(dt_raw), _p(dt_bias), _p(A), _p(bc), bc.stride(0), int(b_offset),
                                        int(c_offset), _p(D), _p(z), z.stride(0), _p(state), state.stride(0), _p(segments), int(n_segments),
                                        _p(single_rows), n_single, _p(slots), _p(out), dtype_code(out.dtype), channels,
                                        states, n, _p(chunk_scratch), 0 if chunk_scratch is None else chunk_scratch.numel(),
                                        _stream()), "selective_scan")


def gemm_simt_batched(mode, a, w, out, alpha: float = 1.0, label=None):
    """out[b] (op)= alpha * a[b] @ w[b]^T for 3-D tensors a [B, M, K], w [B, N, K], out [B, M, N] (inner strides 1, any
    row and batch strides) on the 32-bit pipes; see csrc/gemm_simt.cu."""
    for t in (a, w, out):
        if not t.is_cuda or t.dim() != 3 or t.stride(2) != 1:
            raise KernelError("gemm_simt_batched takes 3-D CUDA tensors with contiguous rows")
    B, M, K = a.shape
    N = out.shape[2]
    if tuple(w.shape) != (B, N, K) or tuple(out.shape) != (B, M, N):
        raise KernelError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    with _timed("gemm_simt", label, work=lambda: _batched_work(a, w, out)):
        _check(lib().lia_gemm_simt_batched(mode, _p(a), dtype_code(a.dtype), a.stride(1), a.stride(0), _p(w),
                                           dtype_code(w.dtype), w.stride(1), w.stride(0), _p(out), dtype_code(out.dtype),
                                           out.stride(1), out.stride(0), B, M, N, K, alpha, _stream()), "gemm_simt_batched")


def latent_attention_accepts(rank: int, dr: int) -> bool:
    """Whether the tensor-core kernel for attention in a latent's space takes these sizes (bfloat16)."""
    return bool(lib().lia_latent_attention_accepts(int(rank), int(dr)))


def latent_attention(q1, q2, latent_pages, part_pages, positions, slots, block_table, out, heads, window, scale, splits=1,
                     partial=None, error_flag=None, label=None, work_bytes=0, work_flops=0):
    """Attention in a latent's space on the tensor cores (bfloat16): q1 [heads, tokens, rank] with the latents, q2
    [tokens, heads dr] with the rotated key parts, out [heads, tokens, rank]; see csrc/latent_attention_mma.cu.
    `splits` > 1 cuts every token's keys into that many ranges; `partial` is their 32-bit scratch of
    splits * heads * tokens * (rank + 2) words."""
    _cuda(q1, q2, latent_pages, part_pages, positions, slots, block_table, out, partial, error_flag)
    if not (q1.dtype == q2.dtype == latent_pages.dtype == part_pages.dtype == out.dtype == torch.bfloat16):
        raise KernelError("latent_attention is a bfloat16 kernel")
    rank, dr = latent_pages.shape[-1], part_pages.shape[-1]
    n = q2.shape[0]
    splits = int(splits)
    if tuple(q1.shape) != (heads, n, rank) or tuple(out.shape) != (heads, n, rank) or q2.shape[1] != heads * dr:
        raise KernelError("latent_attention: q1 and out are [heads, tokens, rank], q2 [tokens, heads dr]")
    if splits > 1 and (partial is None or partial.dtype != torch.float32 or partial.numel() < splits * heads * n * (rank + 2)):
        raise KernelError("latent_attention: the ranges need 32-bit scratch of splits * heads * tokens * (rank + 2) words")
    with _timed("latent_attention", label, work_bytes, work_flops):
        _check(lib().lia_latent_attention(_p(q1), _p(q2), _p(latent_pages), _p(part_pages), _p(positions), _p(slots),
                                          _p(block_table), block_table.shape[1], _p(out), _p(partial) if splits > 1 else None,
                                          n, heads, rank, dr, latent_pages.shape[1], int(window or 0), scale,
                                          latent_pages.shape[0], splits, _p(error_flag), _stream()), "latent_attention")


def _batched_work(a, w, out):
    """(bytes, flops) of B products as the roofline counts them: every operand once."""
    B, M, K = a.shape
    N = out.shape[2]
    return (B * (M * K * a.element_size() + N * K * w.element_size() + M * N * out.element_size()), 2 * B * M * N * K)


def _batched_arguments(a, w, out):
    for t in (a, w, out):
        if not t.is_cuda or t.dim() != 3 or t.stride(2) != 1:
            raise KernelError("a batched product takes 3-D CUDA tensors with contiguous rows")
    B, M, K = a.shape
    N = out.shape[2]
    if tuple(w.shape) != (B, N, K) or tuple(out.shape) != (B, M, N):
        raise KernelError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    return (_p(a), a.stride(1), a.stride(0), _p(w), w.stride(1), w.stride(0), _p(out), out.stride(1), out.stride(0)), (B, M, N, K)


def gemm_mma_batched_accepts(a, w, out) -> bool:
    """Whether the tensor-core kernel for many small products takes these tensors (bfloat16 [B, M, K], [B, N, K] ->
    [B, M, N]): K and the operands' strides multiples of 8 elements, N and the output's strides even, aligned bases."""
    if not (a.dtype == w.dtype == out.dtype == torch.bfloat16):
        return False
    pointers, (B, M, N, K) = _batched_arguments(a, w, out)
    return bool(lib().lia_gemm_mma_batched_accepts(*pointers, M, N, K))


def gemm_mma_batched(a, w, out, label=None):
    """out[b] = a[b] @ w[b]^T for every b in one launch on the tensor cores (bfloat16); see csrc/gemm_mma_batched.cu."""
    pointers, (B, M, N, K) = _batched_arguments(a, w, out)
    if not (a.dtype == w.dtype == out.dtype == torch.bfloat16):
        raise KernelError("gemm_mma_batched is a bfloat16 kernel")
    with _timed("gemm_mma_batched", label, work=lambda: _batched_work(a, w, out)):
        _check(lib().lia_gemm_mma_batched(*pointers, B, M, N, K, _stream()), "gemm_mma_batched")


# ---- several residual streams (hyper-connections), row-wise gates and the logits' soft cap: csrc/hyper_connections.cu ----
HYPER_MAX_STREAMS = 8
GATE_SIGMOID, GATE_SILU = 1, 2


def embedding_streams(tokens, table, out, streams: int, scale: float = 1.0, error_flag=None):
    """out [n, streams * hidden] 32-bit: every stream of a token starts as its row of the table times `scale`."""
    _cuda(tokens, table, out, error_flag)
    _f32(out)
    n, hidden = out.shape[0], table.shape[1]
    if out.shape[1] != streams * hidden:
        raise KernelError("embedding_streams: the rows hold `streams` copies of the table's width")
    with _timed("embedding_streams"):
        _check(lib().lia_embedding_streams(_p(tokens), _p(table), dtype_code(table.dtype), _p(out), n, hidden, int(streams),
                                           table.shape[0], float(scale), _p(error_flag), _stream()), "embedding_streams")


def hyper_step(x, streams: int, y=None, mix=None, out_weights=None, in_weights=None, rows_index=None, u=None,
               norm_weight=None, normed=None, eps: float = 0.0):
    """One pass over the rows of x [n, streams * hidden] (32-bit, the streams of a token side by side).  With y [n, hidden]:
    x_t <- sum_s mix[s, t] x_s + out_weights[t] y, in place.  With u [rows, hidden]: u = sum_s in_weights[s] x_s (the
    plain sum without `in_weights`) of the new streams, and with `normed` also normed = u / sqrt(mean(u^2) + eps) *
    norm_weight in normed's element type.  `rows_index` (without y): row r is read from row rows_index[r]."""
    _cuda(x, y, mix, out_weights, in_weights, rows_index, u, norm_weight, normed)
    _f32(x, y, mix, out_weights, in_weights, u, norm_weight)
    hidden = x.shape[1] // streams
    rows = (y if y is not None else u).shape[0]
    if x.shape[1] != streams * hidden or (y is not None and tuple(y.shape) != (rows, hidden)) or \
            (u is not None and tuple(u.shape) != (rows, hidden)) or (normed is not None and tuple(normed.shape) != (rows, hidden)) \
            or (mix is not None and mix.numel() != streams * streams) or (rows_index is None and x.shape[0] < rows):
        raise KernelError("hyper_step: shapes do not agree")
    with _timed("hyper_step", nbytes=rows * hidden * 4 * (streams * (2 if y is not None else 1) + 2)):
        _check(lib().lia_hyper_step(_p(x), _p(y), _p(mix), _p(out_weights), _p(in_weights), _p(rows_index), _p(u),
                                    _p(norm_weight), _p(normed), 0 if normed is None else dtype_code(normed.dtype), rows,
                                    hidden, int(streams), float(eps), _stream()), "hyper_step")


def softcap_rows(z, cap: float):
    """z <- cap * tanh(z / cap) on 32-bit rows, in place."""
    _f32(z)
    if not z.is_cuda or z.dim() != 2 or z.stride(1) != 1:
        raise KernelError("softcap_rows takes 32-bit CUDA rows")
    with _timed("softcap_rows"):
        _check(lib().lia_softcap_rows(_p(z), z.stride(0), z.shape[0], z.shape[1], float(cap), _stream()), "softcap_rows")


def gate_rows(o, g, act: int, span: int = 1):
    """o[r, i] <- o[r, i] * f(g[r, i // span]), f the logistic function (`GATE_SIGMOID`) or SiLU (`GATE_SILU`); g 32-bit
    rows (a slice of wider rows will do), o rows of the compute element type.  span 1: element by element; span = a
    head's size: one gate a head."""
    _f32(g)
    if not (o.is_cuda and g.is_cuda) or o.dim() != 2 or g.dim() != 2 or o.stride(1) != 1 or g.stride(1) != 1 or \
            o.shape[0] != g.shape[0] or o.shape[1] != g.shape[1] * int(span):
        raise KernelError("gate_rows: o's rows are span times as wide as g's")
    with _timed("gate_rows"):
        _check(lib().lia_gate_rows(_p(o), dtype_code(o.dtype), o.stride(0), _p(g), g.stride(0), o.shape[0], o.shape[1],
                                   int(act), int(span), _stream()), "gate_rows")


# ---- a mixture of gated experts: csrc/moe.cu ----
MOE_MAX_EXPERTS, MOE_MAX_TOP = 1024, 32


def moe_tile_rows() -> int:
    return int(lib().lia_moe_tile_rows())


def moe_max_tiles(pairs: int, experts: int, tile_rows: int = 0) -> int:
    """The most row tiles of `tile_rows` rows (0: the 32-bit product's) that `pairs` (token, choice) pairs grouped by expert
    can be cut into."""
    return pairs // (tile_rows or moe_tile_rows()) + min(experts, pairs)


def moe_grouped_tile_rows(pairs: int, experts: int) -> int:
    """Tokens per tile of the tensor-core product over the experts: the power of two from 16 to 128 that holds an expert's
    share of evenly spread pairs (a function of the step's numbers alone)."""
    rows = 16
    while rows < 128 and rows * experts < pairs:
        rows *= 2
    return rows


def moe_grouped_accepts(x, w_gate_up, w_down) -> bool:
    """Whether the tensor-core product takes the experts' matrices: bfloat16, both reduction lengths multiples of 8
    elements, 16-byte aligned bases (what TMA can address)."""
    return (x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and w_gate_up.shape[2] % 8 == 0 and
            w_down.shape[2] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1 and x.data_ptr() % 16 == 0 and
            w_gate_up.is_contiguous() and w_down.is_contiguous() and w_gate_up.data_ptr() % 16 == 0 and
            w_down.data_ptr() % 16 == 0)


def moe_route(x, router, top: int, scale: float, ids, weights, shared_gate=None, correction=None, groups: int = 0,
              keep: int = 0, renormalise: bool = False):
    """Router scores in 32-bit, the `top` largest chosen: ids, weights [n, top]; with one more row in `router` than
    outputs, shared_gate [n] = the logistic function of that row's product.  `correction` [outputs] is added to the
    scores for the choice only; `groups`/`keep`: only outputs of the best `keep` of `groups` equal groups can be chosen;
    `renormalise`: the weights are divided by their sum."""
    _cuda(x, router, ids, weights, shared_gate, correction)
    _f32(router, weights, shared_gate, correction)
    n, hidden = x.shape
    extra = 0 if shared_gate is None else 1
    experts = router.shape[0] - extra
    if router.shape[1] != hidden or tuple(ids.shape) != (n, top) or tuple(weights.shape) != (n, top) or ids.dtype != torch.int32:
        raise KernelError("moe_route: shapes do not agree")
    with _timed("moe_route"):
        _check(lib().lia_moe_route(_p(x), dtype_code(x.dtype), x.stride(0), _p(router), n, hidden, experts, int(top),
                                   float(scale), extra, _p(correction), int(groups), int(keep), 1 if renormalise else 0,
                                   _p(ids), _p(weights), _p(shared_gate), _stream()), "moe_route")


def moe_plan(ids, experts: int, offsets, order, inverse, tiles, n_tiles, tile_rows: int = 0, pad: bool = False):
    """The pairs grouped by expert: offsets [experts + 1], order (which pair a sorted row is) and inverse [pairs], the list
    of (expert, first row, rows) tiles of `tile_rows` rows (0: the 32-bit product's) and its length.  `pad`: every
    expert's rows begin at a multiple of tile_rows; `order` then has tile_rows * the most tiles entries, -1 on the rows
    of no pair."""
    _cuda(ids, offsets, order, inverse, tiles, n_tiles)
    pairs = ids.numel()
    tile_rows = tile_rows or moe_tile_rows()
    most = moe_max_tiles(pairs, experts, tile_rows)
    if offsets.numel() < experts + 1 or order.numel() < (most * tile_rows if pad else pairs) or inverse.numel() < pairs or \
            tiles.numel() < 3 * most:
        raise KernelError("moe_plan: a list is too short")
    with _timed("moe_plan"):
        _check(lib().lia_moe_plan(_p(ids), pairs, int(experts), int(tile_rows), 1 if pad else 0, order.numel(), _p(offsets),
                                  _p(order), _p(inverse), _p(tiles), _p(n_tiles), _stream()), "moe_plan")


def moe_gather(x, order, top: int, out):
    """out[r] = x[order[r] / top], zero where order[r] < 0: the sorted rows' inputs side by side (bfloat16)."""
    _cuda(x, order, out)
    if x.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or out.shape[1] != x.shape[1] or not out.is_contiguous() or \
            order.numel() < out.shape[0] or x.stride(1) != 1:
        raise KernelError("moe_gather: shapes or element types do not agree")
    with _timed("moe_gather"):
        _check(lib().lia_moe_gather(_p(x), x.stride(0), _p(order), int(top), _p(out), out.shape[0], out.shape[1], _stream()),
               "moe_gather")


def moe_gemm(gated, a, order, top: int, w, out, tiles, n_tiles, max_tiles: int, label=None):
    """The experts' products over the planned tiles, on the 32-bit pipes.  `gated` True (1): a = the tokens' rows, read
    through `order`; w [experts, 2 N, K] = [gate; up]; out [pairs, N] = up * silu(gate) in the compute element type.
    `gated` 2: a likewise, w [experts, N, K], out = relu(a w^T)^2 in the compute element type.  Else a = sorted rows
    [pairs, K], w [experts, N, K], out [pairs, N] 32-bit."""
    _cuda(a, order, w, out, tiles, n_tiles)
    N, K = out.shape[1], a.shape[1]
    gated = int(gated)
    if w.dim() != 3 or w.shape[1] != (2 * N if gated == 1 else N) or w.shape[2] != K or a.dtype != w.dtype or \
            out.dtype != (a.dtype if gated else torch.float32):
        raise KernelError("moe_gemm: shapes or element types do not agree")
    pairs = out.shape[0]
    with _timed("moe_gemm", label, nbytes=w.numel() * w.element_size(), flops=2 * pairs * w.shape[1] * K):
        _check(lib().lia_moe_gemm(gated, _p(a), dtype_code(a.dtype), a.stride(0), _p(order), int(top), _p(w),
                                  _p(out), out.stride(0), _p(tiles), _p(n_tiles), int(max_tiles), N, K, _stream()), "moe_gemm")


def gemm_tc_grouped(mode, a, w, out, tile_rows: int, tiles, n_tiles, max_tiles: int, pairs: int, error_flag=None, label=None,
                    act: int = 0):
    """out[r] = a[r] @ w[e(r)]^T on the tensor cores, rows sorted and padded by expert as `moe_plan(pad=True)` lists them:
    a [rows, K] bfloat16, w [experts, N or 2 N, K] bfloat16, out [rows, N]; GEMM_STORE or GEMM_SWIGLU (csrc/gemm_tc.cu).
    `pairs`: the rows that belong to a pair (for the profile's count of the work)."""
    _cuda(a, w, out, tiles, n_tiles)
    rows, K = a.shape
    N = out.shape[1]
    if w.dim() != 3 or w.shape[1] != (2 * N if mode == GEMM_SWIGLU else N) or w.shape[2] != K or out.shape[0] != rows or \
            not w.is_contiguous():
        raise KernelError("gemm_tc_grouped: shapes do not agree")
    _, sms = _device_scratch(a.device)
    with _timed("gemm_tc_grouped", label, nbytes=w.numel() * w.element_size(), flops=2 * pairs * w.shape[1] * K):
        _check(lib().lia_gemm_tc_grouped(mode | (int(act) << 8), _p(a), a.stride(0), rows, _p(w), K, w.shape[0], _p(out), dtype_code(out.dtype),
                                         out.stride(0), N, K, int(tile_rows), _p(tiles), _p(n_tiles), int(max_tiles), sms,
                                         _p(error_flag), _stream()), "gemm_tc_grouped")


def moe_combine(residual, y, inverse, weights, shared_y, shared_gate, top: int, alpha: float, store: bool, x=None):
    """residual (+)= alpha * (sum_c weights[t, c] y[inverse[t, c]] + shared_gate[t] shared_y[t]); a choice without a row
    (inverse < 0: an identity output) adds weights[t, c] x[t], x the tokens' inputs [n, hidden]."""
    _cuda(residual, y, inverse, weights, shared_y, shared_gate, x)
    _f32(residual, y, weights, shared_y, shared_gate)
    n, hidden = residual.shape
    with _timed("moe_combine"):
        _check(lib().lia_moe_combine(_p(residual), _p(y), _p(inverse), _p(weights), _p(shared_y), _p(shared_gate), _p(x),
                                     F32 if x is None else dtype_code(x.dtype), 0 if x is None else x.stride(0), n, hidden,
                                     int(top), float(alpha), 1 if store else 0, _stream()), "moe_combine")


# ---- retention (a decayed linear recurrence per head): csrc/retention.cu ----
RETENTION_MAX_HEAD = 256


def retention_chunks(portion_tokens: int, n_segments: int) -> int:
    return int(lib().lia_retention_chunks(int(portion_tokens), int(n_segments)))


def retention_scratch_floats(chunks: int, heads: int, d: int, dv: int) -> int:
    return chunks * heads * d * dv


def retention_encode(rows, freq, rot_dims: int, positions, slots, heads: int, d: int, k_scale: float):
    """rows [n, >= 2 heads d] 32-bit, q then k: both rotated in halves over the first rot_dims elements of each head, k
    then multiplied by k_scale, in place."""
    _cuda(freq, positions, slots)
    _f32(rows, freq)
    if rows.stride(1) != 1:
        raise KernelError("retention_encode takes 32-bit rows")
    with _timed("retention_encode"):
        _check(lib().lia_retention_encode(_p(rows), rows.stride(0), _p(freq), int(rot_dims), _p(positions), _p(slots),
                                          rows.shape[0], heads, d, float(k_scale), _stream()), "retention_encode")


def retention(rows, decay, state, segments, n_segments: int, max_chunks: int, single_rows, slots, out, heads: int, d: int,
              dv: int, eps: float, scratch=None):
    """S <- decay_h S + k v^T, o = S^T q, out = o / rms(o) * silu(g) along the step's runs; rows [n, 2 heads (d + dv)]
    32-bit = [q | k | v | g] as `retention_encode` left them, state [slots, heads, d, dv] 32-bit."""
    _cuda(decay, segments, single_rows, slots, out, scratch)
    _f32(rows, decay, state, scratch)
    n_single = 0 if single_rows is None else single_rows.numel()
    if rows.stride(1) != 1 or rows.shape[1] < 2 * heads * (d + dv) or tuple(out.shape) != (rows.shape[0], heads * dv) or \
            state[0].numel() != heads * d * dv or not state[0].is_contiguous():
        raise KernelError("retention: shapes do not agree")
    with _timed("retention", nbytes=rows.numel() * 4, flops=4 * rows.shape[0] * heads * d * dv):
        _check(lib().lia_retention(_p(rows), rows.stride(0), _p(decay), _p(state), state.stride(0), _p(segments),
                                   int(n_segments), int(max_chunks), _p(single_rows), n_single, _p(slots), _p(out),
                                   dtype_code(out.dtype), heads, d, dv, float(eps), _p(scratch),
                                   0 if scratch is None else scratch.numel(), _stream()), "retention")


# ---- gated linear attention (a linear recurrence with a decay per token and key channel): csrc/gated_linear_attention.cu ----
GLA_MAX_HEAD = 256


def gla_scratch_floats(chunks: int, heads: int, d: int, dv: int) -> int:
    return chunks * heads * d * (dv + 1)


def gla_encode(rows, w_a2, bias, log_decay, slots, heads: int, d: int, dv: int, q_scale: float, tau: float):
    """rows [n, >= 2 heads (d + dv) + rank] 32-bit = [q | k | v | g | a]: q times q_scale in place; log_decay [n, heads d]
    32-bit = log2(sigmoid(w_a2 a + bias)) / tau."""
    _cuda(w_a2, bias, log_decay, slots)
    _f32(rows, bias, log_decay)
    rank = w_a2.shape[1]
    if rows.stride(1) != 1 or rows.shape[1] < 2 * heads * (d + dv) + rank or tuple(w_a2.shape) != (heads * d, rank) or \
            not w_a2.is_contiguous() or tuple(log_decay.shape) != (rows.shape[0], heads * d) or not log_decay.is_contiguous():
        raise KernelError("gla_encode: shapes do not agree")
    with _timed("gla_encode"):
        _check(lib().lia_gla_encode(_p(rows), rows.stride(0), _p(w_a2), dtype_code(w_a2.dtype), _p(bias), _p(log_decay),
                                    _p(slots), rows.shape[0], heads, d, dv, rank, float(q_scale), float(tau), _stream()),
               "gla_encode")


def gla(rows, log_decay, state, segments, n_segments: int, max_chunks: int, single_rows, slots, norm_weight, out, heads: int,
        d: int, dv: int, eps: float, scratch=None, encode=None):
    """S <- diag(alpha) S + k v^T, o = S^T q, out = o / rms(o) * norm_weight * silu(g) along the step's runs; rows
    [n, 2 heads (d + dv) ..] 32-bit = [q | k | v | g ..] and log_decay = log2(alpha) as `gla_encode` left them, state
    [slots, heads, d, dv] 32-bit.  `encode` = (w_a2, bias, q_scale, tau), for a step of single tokens alone: the rows are as
    the product left them, `log_decay` may be None, and the kernel does what `gla_encode` does for each token's head."""
    _cuda(log_decay, segments, single_rows, slots, norm_weight, out, scratch)
    _f32(rows, log_decay, state, norm_weight, scratch)
    w_a2, bias, q_scale, tau = encode if encode is not None else (None, None, 1.0, 1.0)
    if encode is not None:
        _cuda(w_a2, bias)
        _f32(bias)
        if n_segments or tuple(w_a2.shape) != (heads * d, w_a2.shape[1]) or not w_a2.is_contiguous() or \
                rows.shape[1] < 2 * heads * (d + dv) + w_a2.shape[1]:
            raise KernelError("gla: the kernel encodes single tokens only, from rows that hold the decay's first product")
        log_decay = None
    n_single = 0 if single_rows is None else single_rows.numel()
    if rows.stride(1) != 1 or rows.shape[1] < 2 * heads * (d + dv) or tuple(out.shape) != (rows.shape[0], heads * dv) or \
            state[0].numel() != heads * d * dv or not state[0].is_contiguous() or \
            (log_decay is not None and (tuple(log_decay.shape) != (rows.shape[0], heads * d) or not log_decay.is_contiguous())) or \
            (log_decay is None and encode is None):
        raise KernelError("gla: shapes do not agree")
    with _timed("gla", nbytes=rows.numel() * 4, flops=4 * rows.shape[0] * heads * d * dv):
        _check(lib().lia_gla(_p(rows), rows.stride(0), _p(log_decay), _p(state), state.stride(0), _p(segments),
                             int(n_segments), int(max_chunks), _p(single_rows), n_single, _p(slots), _p(norm_weight), _p(out),
                             dtype_code(out.dtype), heads, d, dv, float(eps), _p(scratch),
                             0 if scratch is None else scratch.numel(), _p(w_a2), F32 if w_a2 is None else dtype_code(w_a2.dtype),
                             _p(bias), 0 if w_a2 is None else w_a2.shape[1], float(q_scale), float(tau), _stream()), "gla")
