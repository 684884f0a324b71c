"""ctypes bindings of the hand-written sm_100a kernels (`csrc/`, built by `ops/build.py`).

Every function here launches one of this repository's own CUDA kernels on the current
torch stream; there is no fallback: if the library is missing on a machine with a GPU
the import of the library raises.  Tensors are passed as raw device pointers.

`launch_count()` counts the kernels launched through this module (bench.py reports it).
"""
from __future__ import annotations

import ctypes
import math
import os
from ctypes import c_float, c_int, c_long, c_void_p
from pathlib import Path
from typing import Optional

import torch

_LIB_PATH = Path(__file__).resolve().parents[1] / "_C" / "libzorse_sm100.so"
_lib = None
_launches = 0
_status: dict[int, torch.Tensor] = {}

GEMM_OUT_F32 = 1
GEMM_ACCUMULATE = 2
GEMM_GELU = 4
GEMM_RELU = 8

GEMM_KERNEL = os.environ.get("ZORSE_GEMM", "2cta")
# candidate: accumulating GEMMs (weight gradients) request the old C tile before the tile's accumulators are ready
GEMM_ACC_PREFETCH = os.environ.get("ZORSE_GEMM_ACC_PREFETCH", "0") == "1"

ACT_GELU_TANH = 0
ACT_RELU = 1
ACT_GELU_ERF = 2


class KernelError(RuntimeError):
    pass


def available() -> bool:
    return _LIB_PATH.exists()


def lib():
    """Loads (building if needed) the kernel library. Raises if it cannot be had."""
    global _lib
    if _lib is None:
        path = _LIB_PATH
        if os.environ.get("ZORSE_DEBUG_BOUNDS", "0") == "1":
            # the checking build: same entry points, kernels verify their indices (see csrc/common/ptx.cuh)
            from . import build as _build

            path = _build.build(debug_bounds=True)
        elif not path.exists():
            from . import build as _build

            _build.build()
        _lib = ctypes.CDLL(str(path))
        _lib.zb_last_error.restype = ctypes.c_char_p
        if "ZORSE_RS_ADAM_VARIANT" in os.environ:      # 0 / 1 select a peer-load kernel (1 is the library default)
            _lib.zb_set_rs_adam_variant(c_int(int(os.environ["ZORSE_RS_ADAM_VARIANT"])))
    return _lib


def launch_count() -> int:
    return _launches


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def status_word(device=None) -> torch.Tensor:
    """Device int32 that kernels write a non-zero code to when a bounded wait runs out."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    if dev not in _status:
        _status[dev] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{dev}")
    return _status[dev]


_STATUS_NAMES = {
    1: "TMA stage never landed", 2: "stage never released", 3: "accumulator never completed",
    4: "accumulator never drained", 5: "flag wait ran out", 6: "bad argument", 7: "wait ran out",
}


_BOUNDS_SITES = {1: "GEMM tile origin", 2: "GEMM epilogue row / column", 3: "all-gather chunk", 4: "all-gather flag index",
                 5: "optimizer slice", 8: "attention tile"}


def check_status(device=None) -> None:
    """Synchronising read of the status word; raises KernelError if a kernel gave up."""
    s = status_word(device)
    v = int(s.item())
    if v != 0:
        s.zero_()
        code = v & 0xf
        if code == 8:
            site = (v >> 4) & 0xf
            raise KernelError(f"sm100 kernel (checking build) found an index outside its tensor: site {site} "
                              f"({_BOUNDS_SITES.get(site, '?')}) in block {v >> 8}; the access was skipped")
        raise KernelError(
            f"sm100 kernel reported status {v & 0xff} ({_STATUS_NAMES.get(v & 0xff, '?')}) in block {v >> 8}")


def _check(rc: int, what: str) -> None:
    global _launches
    if rc != 0:
        raise KernelError(f"{what}: {lib().zb_last_error().decode()}")
    _launches += 1


def _bf16(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.bfloat16 or not t.is_cuda:
        raise TypeError(f"{name} must be a CUDA bf16 tensor, got {t.dtype} on {t.device}")


# --------------------------------------------------------------------------- GEMM
def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         bias: Optional[torch.Tensor] = None, addend: Optional[torch.Tensor] = None, accumulate: bool = False,
         act: Optional[str] = None, bn: int = 0, max_ctas: int = 0, kernel: Optional[str] = None) -> torch.Tensor:
    """out[M,N] = A @ B^T (+bias) (+addend), or out += ... with accumulate.

    a: [M,K] (K-major) or [K,M] when a_mn; b: [N,K] (K-major) or [K,N] when b_mn.
    out: bf16 or fp32 [M,N]. kernel: "1cta" (128x{128,256} tile per CTA), "2cta" (256x256 tile per
    CTA pair, tcgen05 cta_group::2), "2cta_accpf" (candidate: as "2cta", bf16 `accumulate` reads the old C
    tile ahead of the accumulators) or None = GEMM_KERNEL default ("2cta" for M, N >= 256).
    """
    _bf16(a, "a"); _bf16(b, "b")
    M, N = out.shape
    K = a.shape[0] if a_mn else a.shape[1]
    assert (a.shape[1] if a_mn else a.shape[0]) == M, (a.shape, out.shape, a_mn)
    assert (b.shape == (K, N)) if b_mn else (b.shape == (N, K)), (b.shape, (N, K), b_mn)
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and out.stride(-1) == 1
    flags = 0
    if out.dtype == torch.float32:
        flags |= GEMM_OUT_F32
    elif out.dtype != torch.bfloat16:
        raise TypeError("gemm output must be bf16 or fp32")
    if accumulate:
        flags |= GEMM_ACCUMULATE
    if act == "gelu":
        flags |= GEMM_GELU
    elif act == "relu":
        flags |= GEMM_RELU
    kern = kernel or GEMM_KERNEL
    if kern in ("2cta", "2cta_accpf") and bn == 0 and M >= 256 and N >= 256:
        accpf = kern == "2cta_accpf" or (GEMM_ACC_PREFETCH and accumulate)
        fn = lib().zb_gemm2_accpf_bf16 if accpf else lib().zb_gemm2_bf16
        rc = fn(_p(a), _p(b), _p(out), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)),
                                 c_int(b.stride(0)), c_int(out.stride(0)), c_int(int(a_mn)), c_int(int(b_mn)),
                                 _p(bias), _p(addend), c_int(0 if addend is None else addend.stride(0)),
                                 c_int(flags), c_int(max_ctas), _p(status_word(a.device)), _stream())
        _check(rc, "gemm2")
        return out
    rc = lib().zb_gemm_bf16(_p(a), _p(b), _p(out), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)),
                            c_int(b.stride(0)), c_int(out.stride(0)), c_int(int(a_mn)), c_int(int(b_mn)),
                            _p(bias), _p(addend), c_int(0 if addend is None else addend.stride(0)),
                            c_int(flags), c_int(bn), c_int(max_ctas), _p(status_word(a.device)), _stream())
    _check(rc, "gemm")
    return out


# --------------------------------------------------------------------------- norms
NORM_FWD_VERSION = int(os.environ.get("ZORSE_NORM_FWD", "1"))


def norm_fwd(x, w, b, eps: float, layernorm: bool, version: Optional[int] = None):
    """version 1: one CTA per row; version 2 (candidate): one warp per row, no block barriers."""
    _bf16(x, "x")
    T, H = x.shape
    y = torch.empty_like(x)
    stats = torch.empty(T, 2, dtype=torch.float32, device=x.device)
    fn = lib().zb_norm_fwd2 if (version or NORM_FWD_VERSION) == 2 else lib().zb_norm_fwd
    _check(fn(_p(x), _p(w), _p(b), _p(y), _p(stats), c_int(T), c_int(H), c_float(eps),
              c_int(int(layernorm)), _stream()), "norm_fwd")
    return y, stats


NORM_BWD_VERSION = int(os.environ.get("ZORSE_NORM_BWD", "2"))


def norm_bwd(dy, x, w, stats, dres, dw, db, layernorm: bool, accumulate: bool = True, version: Optional[int] = None):
    """Returns dx (+dres). dw/db: gradient slots (fp32 or bf16) accumulated into.
    version 2: next-row prefetch, one barrier per row, parallel column reduction."""
    T, H = x.shape
    dx = torch.empty_like(x)
    P = lib().zb_norm_partial_rows(c_int(T))
    part_dw = torch.empty(P, H, dtype=torch.float32, device=x.device)
    part_db = torch.empty(P, H, dtype=torch.float32, device=x.device) if (layernorm and db is not None) else None
    gf32 = int(dw.dtype == torch.float32)
    fn = lib().zb_norm_bwd2 if (version or NORM_BWD_VERSION) == 2 else lib().zb_norm_bwd
    _check(fn(_p(dy), _p(x), _p(w), _p(stats), _p(dres), _p(dx), _p(part_dw), _p(part_db),
                             _p(dw), _p(db), c_int(T), c_int(H), c_int(int(layernorm)), c_int(gf32),
                             c_int(int(accumulate)), _stream()), "norm_bwd")
    return dx


def colsum_accumulate(dy, out, accumulate: bool = True):
    """out[n] (+)= sum_t dy[t, n] (bias gradients)."""
    T, N = dy.shape
    part = torch.empty(min(T, 64), N, dtype=torch.float32, device=dy.device)
    _check(lib().zb_colsum(_p(dy), c_int(T), c_int(N), c_int(dy.stride(0)), _p(part), _p(out),
                           c_int(int(out.dtype == torch.float32)), c_int(int(accumulate)), _stream()), "colsum")
    return out


# --------------------------------------------------------------------------- elementwise
def rope_(buf, cs, S: int, nheads: int, d: int, backward: bool = False):
    """In-place rotate-half RoPE on heads [0, nheads) of a packed [T, width] buffer."""
    T = buf.shape[0]
    _check(lib().zb_rope(_p(buf), _p(cs), c_int(T), c_int(S), c_int(nheads), c_int(d), c_int(buf.stride(0)),
                         c_int(int(backward)), _stream()), "rope")
    return buf


def swiglu_fwd(gu):
    T, F2 = gu.shape
    out = torch.empty(T, F2 // 2, dtype=gu.dtype, device=gu.device)
    _check(lib().zb_swiglu_fwd(_p(gu), _p(out), c_long(T), c_int(F2 // 2), _stream()), "swiglu_fwd")
    return out


def swiglu_bwd(gu, dout):
    dgu = torch.empty_like(gu)
    T, F2 = gu.shape
    _check(lib().zb_swiglu_bwd(_p(gu), _p(dout), _p(dgu), c_long(T), c_int(F2 // 2), _stream()), "swiglu_bwd")
    return dgu


def act_fwd(x, kind: int):
    y = torch.empty_like(x)
    _check(lib().zb_act_fwd(_p(x), _p(y), c_long(x.numel()), c_int(kind), _stream()), "act_fwd")
    return y


def act_bwd(x, dy, kind: int):
    dx = torch.empty_like(x)
    _check(lib().zb_act_bwd(_p(x), _p(dy), _p(dx), c_long(x.numel()), c_int(kind), _stream()), "act_bwd")
    return dx


def embedding_fwd(ids, table, pos_table=None, S: int = 1, pos_offset: int = 0):
    T = ids.numel()
    V, H = table.shape
    out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    _check(lib().zb_embedding_fwd(_p(ids), _p(table), _p(pos_table), _p(out), c_int(T), c_int(H), c_int(V),
                                  c_int(S), c_int(pos_offset), _stream()), "embedding_fwd")
    return out


def embedding_bwd(ids, dout, dtable, dpos=None, S: int = 1, pos_offset: int = 0):
    T = ids.numel()
    V, H = dtable.shape
    _check(lib().zb_embedding_bwd(_p(ids), _p(dout), _p(dtable), _p(dpos), c_int(T), c_int(H), c_int(V),
                                  c_int(S), c_int(pos_offset), c_int(int(dtable.dtype == torch.float32)),
                                  _stream()), "embedding_bwd")


# --------------------------------------------------------------------------- loss
def cross_entropy(logits, targets, grad_scale: float, dlogits=None, ignore_index: int = -100):
    """Returns per-row losses (fp32). Writes d(loss)/d(logits) * grad_scale into dlogits
    (may alias logits) when given."""
    T, V = logits.shape
    loss_rows = torch.empty(T, dtype=torch.float32, device=logits.device)
    _check(lib().zb_cross_entropy(_p(logits), _p(targets), _p(dlogits), _p(loss_rows), c_int(T), c_int(V),
                                  c_long(logits.stride(0)), c_float(grad_scale), c_long(ignore_index),
                                  _stream()), "cross_entropy")
    return loss_rows


# --------------------------------------------------------------------------- optimizer
def adam_step(p, m, v, g, p16, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0, zero_grad=False):
    n = p.numel()
    _check(lib().zb_adam(_p(p), _p(m), _p(v), _p(g), _p(p16), c_long(n), c_float(lr), c_float(beta1),
                         c_float(beta2), c_float(eps), c_float(weight_decay), c_int(step), c_float(grad_scale),
                         c_int(int(g.dtype == torch.float32)), c_int(int(zero_grad)), _stream()), "adam")


# --------------------------------------------------------------------------- attention
# 0 = by problem size: version 4 (two query tiles per CTA, 256 query rows) when that still gives every SM a
# CTA, version 1 (one 128-row tile per CTA) for smaller problems; 1 / 2 / 4 force a version.
ATTN_FWD_VERSION = int(os.environ.get("ZORSE_ATTN_FWD", "0"))


ATTN_FWD4_FLAGS = int(os.environ.get("ZORSE_ATTN_FWD4_FLAGS", "1"))


def _auto_fwd_version(B: int, S: int, Hq: int) -> int:
    return 4 if B * Hq * ((S + 255) // 256) >= 148 else 1


def flash_fwd(qkv, B: int, S: int, Hq: int, Hkv: int, D: int, causal: bool = True, window: int = 0,
              scale: Optional[float] = None, version: Optional[int] = None, flags: Optional[int] = None,
              trace: Optional[torch.Tensor] = None, trace_ctas: int = 0):
    """qkv: packed [B*S, (Hq+2Hkv)*D]. Returns (out [B*S, Hq*D], lse [B, Hq, S]).
    version 1: one query tile per CTA, S double-buffered in TMEM, P staged through shared memory (default
    for problems with fewer than 148 pairs of query tiles); version 2: two query tiles per CTA, P kept in
    TMEM; version 4 (default otherwise, 1.36-1.44x faster than version 1 on 4096-token sequences): two
    query tiles, one MMA issuer, score rows in registers (`flags` 1: two-wide
    fp32 math, 2: also a quarter of the exponentials as a polynomial on the fma pipe; `trace`: zeroed int64 buffer from `flash_fwd4_trace_buffer` for a phase timeline)."""
    _bf16(qkv, "qkv")
    assert qkv.shape == (B * S, (Hq + 2 * Hkv) * D) and qkv.is_contiguous()
    out = torch.empty(B * S, Hq * D, dtype=qkv.dtype, device=qkv.device)
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device=qkv.device)
    sc = (1.0 / math.sqrt(D)) if scale is None else scale
    ver = version or ATTN_FWD_VERSION or _auto_fwd_version(B, S, Hq)
    if ver == 4:
        fl = ATTN_FWD4_FLAGS if flags is None else flags
        _check(lib().zb_flash_fwd4(_p(qkv), _p(out), _p(lse), c_int(B), c_int(S), c_int(Hq), c_int(Hkv), c_int(D),
                                   c_int(int(causal)), c_int(window), c_float(sc), c_int(out.stride(0)),
                                   _p(status_word(qkv.device)), c_int(fl), _p(trace),
                                   c_int(trace_ctas if trace is not None else 0), _stream()), "flash_fwd4")
        return out, lse
    fn = {1: lib().zb_flash_fwd, 2: lib().zb_flash_fwd2}[ver]
    _check(fn(_p(qkv), _p(out), _p(lse), c_int(B), c_int(S), c_int(Hq), c_int(Hkv), c_int(D),
                              c_int(int(causal)), c_int(window), c_float(sc), c_int(out.stride(0)),
                              _p(status_word(qkv.device)), _stream()), "flash_fwd")
    return out, lse


_attn_scratch2: dict = {}


def _flash_bwd2(do, qkv, o, lse, B, S, Hq, Hkv, D, causal, window, scale, trace, trace_ctas):
    key = (qkv.device.index, B, S, Hq, D)
    if key not in _attn_scratch2:
        n = lib().zb_flash_bwd2_stats_floats(c_int(B), c_int(S), c_int(Hq))
        # zeroed once: the kernels never write the padding of the statistics rows
        _attn_scratch2[key] = (torch.zeros(n, dtype=torch.float32, device=qkv.device),
                               torch.zeros(B * S * Hq * D, dtype=torch.float32, device=qkv.device))
    stats, dq_acc = _attn_scratch2[key]
    dqkv = torch.empty_like(qkv)
    sc = (1.0 / math.sqrt(D)) if scale is None else scale
    _check(lib().zb_flash_bwd2(_p(do), _p(qkv), _p(o), _p(lse), _p(dqkv), _p(stats), _p(dq_acc), c_int(B), c_int(S),
                               c_int(Hq), c_int(Hkv), c_int(D), c_int(int(causal)), c_int(window), c_float(sc),
                               _p(status_word(qkv.device)), _p(trace), c_int(trace_ctas if trace is not None else 0),
                               _stream()), "flash_bwd2")
    global _launches
    _launches += 2  # statistics + finish kernels
    return dqkv


def _flash_bwd3(do, qkv, o, lse, B, S, Hq, Hkv, D, causal, window, scale, parts: int = 3, trace=None, trace_ctas: int = 0):
    key = (qkv.device.index, B, S, Hq)
    if key not in _attn_scratch3:
        n = lib().zb_flash_bwd2_stats_floats(c_int(B), c_int(S), c_int(Hq))
        _attn_scratch3[key] = torch.zeros(n, dtype=torch.float32, device=qkv.device)   # padding stays zero
    stats = _attn_scratch3[key]
    dqkv = torch.empty_like(qkv)
    sc = (1.0 / math.sqrt(D)) if scale is None else scale
    _check(lib().zb_flash_bwd3(_p(do), _p(qkv), _p(o), _p(lse), _p(dqkv), _p(stats), c_int(B), c_int(S), c_int(Hq),
                               c_int(Hkv), c_int(D), c_int(int(causal)), c_int(window), c_float(sc),
                               _p(status_word(qkv.device)), c_int(parts), _p(trace),
                               c_int(trace_ctas if trace is not None else 0), _stream()), "flash_bwd3")
    global _launches
    _launches += 2  # statistics + the second main kernel
    return dqkv


_attn_scratch3: dict = {}


def flash_bwd2_trace_buffer(device, ctas: int) -> torch.Tensor:
    w, e = lib().zb_flash_bwd2_trace_warps(), lib().zb_flash_bwd2_trace_events()
    return torch.zeros(ctas, w, e, dtype=torch.int64, device=device)


def flash_fwd4_trace_buffer(device, ctas: int) -> torch.Tensor:
    """Zeroed event buffer [ctas, warps, events] for `flash_fwd(version=4, trace=...)`; an event is
    (clock64 << 8) | code, 0 = unused slot."""
    w, e = lib().zb_flash_fwd4_trace_warps(), lib().zb_flash_fwd4_trace_events()
    return torch.zeros(ctas, w, e, dtype=torch.int64, device=device)


_attn_scratch: dict = {}


# 0 = default = version 3 (two kernels, no atomics: 1.46x faster than version 1 at 4096 tokens, d = 128);
# 1 / 2 / 3 force a version
ATTN_BWD_VERSION = int(os.environ.get("ZORSE_ATTN_BWD", "0"))


def flash_bwd(do, qkv, o, lse, B: int, S: int, Hq: int, Hkv: int, D: int, causal: bool = True, window: int = 0,
              scale: Optional[float] = None, version: Optional[int] = None, trace: Optional[torch.Tensor] = None,
              trace_ctas: int = 0):
    """Returns dqkv packed like qkv. Scratch (fp32 dQ accumulator, delta) is cached per shape
    and device; the accumulator is left zeroed by the kernel that converts it to bf16.
    version 1: scores with queries on the TMEM lanes, P and dS staged through shared
    memory; version 2: transposed scores, P^T / dS^T consumed from tensor memory, two Q/dO stages
    (`trace`: zeroed buffer from `flash_bwd2_trace_buffer`); version 3 (default): two kernels without atomics, dK / dV per
    key tile and dQ per query tile (scores are formed twice; no fp32 dQ accumulator)."""
    _bf16(do, "do"); _bf16(qkv, "qkv")
    assert do.is_contiguous() and qkv.is_contiguous() and o.is_contiguous()
    ver = version or ATTN_BWD_VERSION or 3
    if ver == 3:
        return _flash_bwd3(do, qkv, o, lse, B, S, Hq, Hkv, D, causal, window, scale, trace=trace, trace_ctas=trace_ctas)
    if ver == 2:
        return _flash_bwd2(do, qkv, o, lse, B, S, Hq, Hkv, D, causal, window, scale, trace, trace_ctas)
    key = (qkv.device.index, B, S, Hq, D)
    if key not in _attn_scratch:
        _attn_scratch[key] = (torch.empty(B * Hq * S, dtype=torch.float32, device=qkv.device),
                              torch.zeros(B * S * Hq * D, dtype=torch.float32, device=qkv.device))
    delta, dq_acc = _attn_scratch[key]
    dqkv = torch.empty_like(qkv)
    sc = (1.0 / math.sqrt(D)) if scale is None else scale
    _check(lib().zb_flash_bwd(_p(do), _p(qkv), _p(o), _p(lse), _p(dqkv), _p(delta), _p(dq_acc), c_int(B), c_int(S),
                              c_int(Hq), c_int(Hkv), c_int(D), c_int(int(causal)), c_int(window), c_float(sc),
                              _p(status_word(qkv.device)), _stream()), "flash_bwd")
    global _launches
    _launches += 2  # delta + finish kernels
    return dqkv


# --------------------------------------------------------------------------- fused collectives
def _ptr_array(ptrs):
    arr = (c_void_p * len(ptrs))(*[c_void_p(int(x)) for x in ptrs])
    return arr


def ag_gemm(a: torch.Tensor, full: torch.Tensor, w_offset: int, w_shape, out: torch.Tensor, *, shard_ptrs, R: int,
            r: int, shard_elems: int, chunk_bytes: int, chunk_flags: torch.Tensor, epoch: int,
            version_flags: torch.Tensor, need_version: int, bias=None, addend=None) -> torch.Tensor:
    """out = a @ W^T with W = full[w_offset : w_offset + N*K].view(N, K), while the same kernel
    pulls the other ranks' shards of the unit into `full` (all-gather fused with the GEMM).
    shard_ptrs: device addresses of every rank's bf16 shard (peer-mapped), by group rank."""
    _bf16(a, "a")
    N, K = w_shape
    M = a.shape[0]
    assert out.shape == (M, N) and a.shape[1] == K and out.dtype == torch.bfloat16
    # the 2-CTA core (256 x 256 tiles per CTA pair) when the problem has at least one such tile, like `gemm`
    two_cta = GEMM_KERNEL == "2cta" and M >= 256 and N >= 256 and os.environ.get("ZORSE_AG_GEMM", "2cta") != "1cta"
    fn = lib().zb_ag_gemm2_bf16 if two_cta else lib().zb_ag_gemm_bf16
    rc = fn(_p(a), _p(full), c_long(w_offset * 2), _p(out), c_int(M), c_int(N), c_int(K),
                               c_int(a.stride(0)), c_int(out.stride(0)), _p(bias), _p(addend),
                               c_int(0 if addend is None else addend.stride(0)), c_int(0), _ptr_array(shard_ptrs),
                               c_int(R), c_int(r), c_long(shard_elems * 2), c_int(chunk_bytes), _p(chunk_flags),
                               c_int(epoch), _p(version_flags), c_int(need_version), _p(status_word(a.device)),
                               _stream())
    _check(rc, "ag_gemm")
    return out


def gemm_rs(a: torch.Tensor, b: torch.Tensor, *, b_mn: bool, dst_ptrs, flag_ptrs, flag_index: int, epoch: int,
            counter: torch.Tensor, ldc: int, max_ctas: int = 0) -> None:
    """Partial product a @ b^T (b_mn: a @ b) whose rows are scattered for a row-wise reduce-scatter over
    R = len(dst_ptrs) processes: rows of chunk q are stored (bf16, row stride ldc) at dst_ptrs[q], a device
    address that may be in a peer's memory; afterwards `epoch` is stored to flag_ptrs[q][flag_index]."""
    _bf16(a, "a"); _bf16(b, "b")
    M, K = a.shape
    N = b.shape[1] if b_mn else b.shape[0]
    assert (b.shape[0] if b_mn else b.shape[1]) == K and a.stride(-1) == 1 and b.stride(-1) == 1
    R = len(dst_ptrs)
    rc = lib().zb_gemm2_rs_bf16(_p(a), _p(b), c_int(M), c_int(N), c_int(K), c_int(a.stride(0)), c_int(b.stride(0)),
                                c_int(ldc), c_int(int(b_mn)), _ptr_array(dst_ptrs), _ptr_array(flag_ptrs), c_int(R),
                                c_int(flag_index), c_int(epoch), _p(counter), c_int(max_ctas),
                                _p(status_word(a.device)), _stream())
    _check(rc, "gemm_rs")


def rs_finish(slots: torch.Tensor, flags: torch.Tensor, R: int, rows: int, H: int, epoch: int, out: torch.Tensor,
              resid: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, wait_seconds: float = 2.0):
    """out[rows, H] = sum over the R staging slots ([R, rows, H] bf16, filled by the peers' gemm_rs) (+ resid)
    (+ bias), after every sender's flag has reached `epoch` (bounded wait)."""
    rc = lib().zb_rs_finish(_p(slots), _p(flags), c_int(R), c_int(rows), c_int(H), c_int(H), c_int(epoch), _p(resid),
                            c_int(0 if resid is None else resid.stride(0)), _p(bias), _p(out), c_int(out.stride(0)),
                            ctypes.c_double(wait_seconds), _p(status_word(out.device)), _stream())
    _check(rc, "rs_finish")
    return out


def tp_norm_push(*, w, b, eps: float, layernorm: bool, y_local, dst_ptrs, flag_ptrs, flag_index: int, epoch: int,
                 stats, counter, x=None, slots=None, in_flags=None, in_epoch: int = 0, resid=None, bias=None, h_out=None,
                 wait_seconds: float = 2.0) -> None:
    """Row-wise norm whose output also goes to every lane member's gathered buffer (dst_ptrs: device addresses
    of this process's row block there).  Input rows: `x`, or the sum of the reduce-scatter `slots`
    ([R, rows, H], ready when in_flags reach in_epoch) + resid + bias, which is written to h_out."""
    rows, H = y_local.shape
    R_in = 0 if slots is None else slots.numel() // (rows * H)
    rc = lib().zb_tp_norm_push(_p(x), _p(slots), _p(in_flags), c_int(R_in), c_int(in_epoch), _p(resid),
                               c_int(0 if resid is None else resid.stride(0)), _p(bias), _p(h_out), _p(w), _p(b),
                               c_float(eps), c_int(int(layernorm)), _p(y_local), _ptr_array(dst_ptrs),
                               _ptr_array(flag_ptrs), c_int(len(dst_ptrs)), c_int(flag_index), c_int(epoch), _p(stats),
                               c_int(rows), c_int(H), _p(counter), ctypes.c_double(wait_seconds),
                               _p(status_word(y_local.device)), _stream())
    _check(rc, "tp_norm_push")


def tp_push(src: torch.Tensor, dst_ptrs, flag_ptrs, flag_index: int, epoch: int, counter) -> None:
    """Copies the contiguous tensor `src` to every device address in dst_ptrs, then stores `epoch` to
    flag_ptrs[q][flag_index] (all-gather by stores, for rows that need no arithmetic)."""
    assert src.is_contiguous()
    rc = lib().zb_tp_push(_p(src), _ptr_array(dst_ptrs), _ptr_array(flag_ptrs), c_int(len(dst_ptrs)), c_int(flag_index),
                          c_int(epoch), c_long(src.numel() * src.element_size()), _p(counter),
                          _p(status_word(src.device)), _stream())
    _check(rc, "tp_push")


def rs_adam(grad_ptrs, flag_ptrs, R: int, r: int, shard_elems: int, master, m, v, p16, *, lr, beta1, beta2, eps,
            weight_decay, step, grad_scale, grad_f32: bool, epoch: int, counter: torch.Tensor, max_blocks: int = 0,
            wait_seconds: float = 2.0):
    """Fused reduce-scatter + Adam: sums slice r of every rank's gradient bucket (peer loads)
    and updates master/m/v/p16 in one pass. grad_ptrs / flag_ptrs: device addresses by group rank."""
    rc = lib().zb_rs_adam(_ptr_array(grad_ptrs), _ptr_array(flag_ptrs), c_int(R), c_int(r), c_long(shard_elems),
                          _p(master), _p(m), _p(v), _p(p16), c_float(lr), c_float(beta1), c_float(beta2), c_float(eps),
                          c_float(weight_decay), c_int(step), c_float(grad_scale), c_int(int(grad_f32)), c_int(epoch),
                          _p(counter), c_int(max_blocks), ctypes.c_double(wait_seconds),
                          _p(status_word(master.device)), _stream())
    _check(rc, "rs_adam")


def rs_adam_nvls(grad_mc: int, flag_ptrs, R: int, r: int, shard_elems: int, master, m, v, p16, *, lr, beta1, beta2, eps,
                 weight_decay, step, grad_scale, grad_f32: bool, epoch: int, counter: torch.Tensor,
                 max_blocks: int = 0, wait_seconds: float = 2.0, p16_mc: int = 0):
    """rs_adam with the gradient slice summed inside NVSwitch: grad_mc is the multicast address of the
    group's gradient buckets (candidate; the switch's summation order, not the rank order).  With
    p16_mc (multicast address of this rank's shard inside the unsharded parameter buffers) the new
    bf16 shard is stored to every rank's buffer at once and p16 is left untouched."""
    rc = lib().zb_rs_adam_nvls(c_void_p(int(grad_mc)), c_void_p(int(p16_mc)), _ptr_array(flag_ptrs), c_int(R), c_int(r), c_long(shard_elems),
                               _p(master), _p(m), _p(v), _p(p16), c_float(lr), c_float(beta1), c_float(beta2),
                               c_float(eps), c_float(weight_decay), c_int(step), c_float(grad_scale),
                               c_int(int(grad_f32)), c_int(epoch), _p(counter), c_int(max_blocks),
                               ctypes.c_double(wait_seconds), _p(status_word(master.device)), _stream())
    _check(rc, "rs_adam_nvls")


def set_rs_adam_variant(variant: int) -> None:
    """0: measured kernel; 1: candidate that requests the optimizer state and all slices up front."""
    lib().zb_set_rs_adam_variant(c_int(variant))


def wait_flags(flags: torch.Tensor, R: int, which: int, epoch: int, wait_seconds: float = 2.0):
    """One-thread kernel that returns once flags[which*R + q] >= epoch for all q (bounded)."""
    _check(lib().zb_wait_flags(_p(flags), c_int(R), c_int(which), c_int(epoch), ctypes.c_double(wait_seconds),
                               _p(status_word(flags.device)), _stream()), "wait_flags")


def peer_pull(src_ptr: int, dst: torch.Tensor, nbytes: int, max_blocks: int = 0):
    """Copies nbytes from a peer-mapped device address into dst with plain peer loads."""
    _check(lib().zb_peer_pull(c_void_p(int(src_ptr)), _p(dst), c_long(nbytes), c_int(max_blocks), _stream()),
           "peer_pull")
