"""ctypes bindings of the in-tree sm_100a library ``b200moe/_C/libb200moe.so``.

Every function takes torch tensors, launches on the current CUDA stream and
returns torch tensors.  ``has(op)`` tells the op layer whether the kernel family
``op`` is loaded; ``require()`` raises if the library is missing, so a GPU run
can never fall back silently.  ``launch_count()`` counts launches of this
library's kernels (the benchmark reports it).
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# B200MOE_DEBUG=1 loads the checked build (``B200MOE_DEBUG=1 python -m b200moe.build``): data-dependent indices
# are range-checked in the kernels and ``check_status`` also raises on a recorded violation.
_DEBUG = os.environ.get("B200MOE_DEBUG", "0") not in ("", "0")
_LIB_PATH = (os.path.join(_HERE, "_C", "debug", "libb200moe_debug.so") if _DEBUG
             else os.path.join(_HERE, "_C", "libb200moe.so"))
_lib = None
_load_error = None
_launches = 0
_status = {}

_FAMILIES = {
    "gemm": "b2_gemm_nt", "rmsnorm": "b2_rmsnorm_fwd", "router": "b2_router_top2_fwd",
    "lmhead_ce": "b2_cross_entropy", "adamw": "b2_adamw", "embedding": "b2_embedding_fwd",
    "rope": "b2_rope", "moe": "b2_moe_plan", "attention": "b2_attention_fwd", "comm": "b2_comm_allreduce",
    "swiglu": "b2_swiglu_bwd",
}


def _load():
    global _lib, _load_error
    if _lib is not None or _load_error is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        _load_error = f"{_LIB_PATH} not found; run `python -m b200moe.build`"
        return None
    try:
        _lib = ctypes.CDLL(_LIB_PATH)
    except OSError as error:
        _load_error = str(error)
        _lib = None
        return None
    mode = os.environ.get("B200MOE_GEMM_TILE_MODE")
    if mode:          # A/B runs of whole programs: see set_gemm_tile_mode
        _lib.b2_gemm_set_tile_mode(ctypes.c_int(int(mode)))
    return _lib


def require():
    if _load() is None:
        raise RuntimeError(f"b200moe native library unavailable: {_load_error}")
    return _lib


def has(op: str) -> bool:
    lib = _load()
    if lib is None:
        return False
    symbol = _FAMILIES.get(op)
    return symbol is not None and hasattr(lib, symbol)


def available_ops() -> list:
    return sorted(op for op in _FAMILIES if has(op))


def launch_count() -> int:
    return _launches


def count_launch(n: int = 1) -> None:
    """For callers that launch through ``require()`` directly."""
    global _launches
    _launches += n


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def status_word(device=None) -> torch.Tensor:
    """Device int32 word that kernels set non-zero when a bounded wait ran out."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = _status.get(device)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _status[device] = word
    return word


def debug_records(clear: bool = False) -> dict:
    """Checked build only: the first range violation recorded by each source file, as
    ``{file: (code, value, bound, block)}``; empty in the normal build."""
    lib = _load()
    found = {}
    if lib is None:
        return found
    for name in ("moe", "comm", "moe_ep"):
        reader = getattr(lib, f"b2_{name}_debug_read", None) if _DEBUG else None
        if reader is None:
            continue
        record = (ctypes.c_int * 4)()
        if reader(record, ctypes.c_int(int(clear))) == 0 and record[0]:
            found[name] = tuple(record)
    return found


def set_wait_seconds(seconds: float) -> None:
    """Budget of every cross-GPU wait inside this library's kernels on the current device (default 10 s).  A wait
    that runs out makes its kernel skip the dependent work, set the status word and return."""
    rc = require().b2_comm_set_wait_ns(ctypes.c_longlong(int(float(seconds) * 1e9)))
    if rc != 0:
        raise RuntimeError(f"b2_comm_set_wait_ns failed with code {rc}")


def clear_status(device=None) -> None:
    """Reset the status word after a reported failure has been handled (tests; a trainer restarts instead)."""
    status_word(device).zero_()


def check_status() -> int:
    """Synchronising read of the status word; raises if a kernel gave up (or, in the checked build, if a kernel
    recorded an out-of-range index)."""
    value = int(status_word().item())
    if value:
        raise RuntimeError(f"b200moe kernel reported wait timeout code {value}")
    if _DEBUG:
        bad = debug_records()
        if bad:
            raise RuntimeError(f"b200moe checked build recorded out-of-range indices: {bad}")
    return value


_nvtx = False


def set_nvtx(enabled: bool) -> None:
    """Wrap every launch of this library in an NVTX range named after its entry point (for Nsight Systems
    timelines; the trainer switches it on with ``profile.enabled``)."""
    global _nvtx
    _nvtx = bool(enabled)


_timed = None      # list of (label, start event, end event) while launch timing is on


def start_launch_timing() -> None:
    """Bracket every launch of this library with a pair of CUDA events on its stream (``launch_times`` reads them).
    For per-kernel time tables of a whole step; it adds two event records per launch, so timed regions of a
    benchmark leave it off."""
    global _timed
    _timed = []


def launch_times() -> dict:
    """Stops launch timing and returns ``{label: (launches, total ms)}``; synchronises the device."""
    global _timed
    records, _timed = _timed or [], None
    torch.cuda.synchronize()
    table: dict = {}
    for label, begin, end in records:
        count, total = table.get(label, (0, 0.0))
        table[label] = (count + 1, total + begin.elapsed_time(end))
    return table


def _call(name, *args, n: int = 1, tag: str = ""):
    global _launches
    if _timed is not None:
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        rc = getattr(require(), name)(*args)
        end.record()
        _timed.append((f"{name} {tag}".strip(), begin, end))
        if rc != 0:
            raise RuntimeError(f"{name} failed with code {rc}")
        _launches += n
        return
    if _nvtx:
        torch.cuda.nvtx.range_push(name)
        try:
            rc = getattr(require(), name)(*args)
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        rc = getattr(require(), name)(*args)
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}{_failure_detail(name, rc)}")
    _launches += n


def _failure_detail(name: str, rc: int) -> str:
    """What else is known about a refused launch (the attention entry points keep the driver's result of a
    tensor-map encode that failed)."""
    if name.startswith("b2_attention") and -14 <= rc <= -11:
        reader = getattr(_lib, "b2_attention_last_encode_result", None)
        if reader is not None:
            return f" (tensor map {('q', 'k', 'v', 'dout')[-11 - rc]}: driver result {reader()})"
    return ""


_I, _L, _F = ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _bf16(t):
    if t.dtype != torch.bfloat16:
        raise TypeError(f"expected bfloat16, got {t.dtype}")
    return t


# ------------------------------------------------------------------------------ GEMM
def set_gemm_tile_mode(mode: int) -> None:
    """0: automatic among the single-CTA kinds (the default: fastest under the sustained power cap of a training
    step); 1: always 128x256 CTA tiles; 2: single-CTA 256x256 tiles wherever legal; 3: 256x256 tiles on CTA pairs
    (``cta_group::2``) wherever legal; 4: automatic with CTA pairs for problems that fill the machine (fastest for
    a kernel run in isolation).  The environment variable ``B200MOE_GEMM_TILE_MODE`` sets it at load time."""
    require().b2_gemm_set_tile_mode(_I(mode))


def gemm_nt(x, w, out_dtype=None, tile_expert=None, num_m_tiles=None, num_experts: int = 1, align256: bool = False):
    """``x [M,K] @ w[e] [N,K]ᵀ``.  Rows of ``w`` below 17: skinny path, fp32 result."""
    M, K = x.shape
    N = w.shape[-2]
    if N <= 16 and num_experts == 1:
        out = torch.empty(M, N, dtype=torch.float32, device=x.device)
        _call("b2_skinny_nt", _p(_bf16(x)), _p(_bf16(w)), _p(out), _I(M), _I(N), _I(K), _stream())
        return out
    out_dtype = out_dtype or torch.bfloat16
    out = torch.empty(M, N, dtype=out_dtype, device=x.device)
    assert x.stride(-1) == 1 and w.is_contiguous()
    _call("b2_gemm_nt", _p(_bf16(x)), _p(_bf16(w)), _p(out), _I(M), _I(N), _I(K), _L(x.stride(0)), _L(K), _L(N),
          _I(num_experts), _p(tile_expert), _p(num_m_tiles), _I(int(align256)),
          _I(0 if out_dtype == torch.bfloat16 else 4),
          _p(status_word(x.device)), _stream(), tag=f"{'grouped ' if tile_expert is not None else ''}N={N} K={K}")
    return out


def gemm_nt_rope(x, w, cos, sin, rope_cols: int, seq: int):
    """``x [M,K] @ w [N,K]ᵀ`` with the rotary embedding applied, in the GEMM epilogue, to output columns
    ``[0, rope_cols)``: heads of 128 columns, adjacent pairs, position ``row mod seq``; ``cos``/``sin`` fp32
    ``[>=seq, 64]``."""
    M, K = x.shape
    N = w.shape[0]
    if cos.shape[-1] != 64 or cos.dtype != torch.float32 or not cos.is_contiguous() or cos.shape[0] < seq:
        raise ValueError("rotary tables must be contiguous fp32 [>= seq, 64] (head_dim 128)")
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    assert x.stride(-1) == 1 and w.is_contiguous()
    _call("b2_gemm_nt_rope", _p(_bf16(x)), _p(_bf16(w)), _p(out), _I(M), _I(N), _I(K), _L(x.stride(0)), _L(N),
          _p(cos), _p(sin), _I(rope_cols), _I(seq), _p(status_word(x.device)), _stream())
    return out


def gemm_nn(dy, w, w2=None, tile_expert=None, num_m_tiles=None, num_experts: int = 1, align256: bool = False,
            out=None):
    """``dy [M,K] @ w[e] [K,N]`` (``w`` rows are the reduction index).  With ``w2``
    the reduction continues over ``w2``'s rows: ``dy = [a | b]``, result ``a w + b w2``."""
    M, K = dy.shape
    N = w.shape[-1]
    if K <= 16 and num_experts == 1 and w2 is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dy.device)
        _call("b2_skinny_nn", _p(dy.float().contiguous()), _p(_bf16(w)), _p(out), _I(M), _I(K), _I(N), _stream())
        return out
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dy.device)
    k_split = w.shape[-2] if w2 is not None else 0
    assert dy.stride(-1) == 1 and w.is_contiguous() and out.stride(-1) == 1 and out.shape == (M, N)
    _call("b2_gemm_nn", _p(_bf16(dy)), _p(_bf16(w)), _p(w2), _p(_bf16(out)), _I(M), _I(N), _I(K), _I(k_split),
          _L(dy.stride(0)), _L(N), _L(out.stride(0)), _I(num_experts), _p(tile_expert), _p(num_m_tiles), _I(int(align256)),
          _p(status_word(dy.device)), _stream(), tag=f"{'grouped ' if tile_expert is not None else ''}N={N} K={K}")
    return out


def gemm_tn(dy, x, out=None, accumulate: bool = False, out_dtype=None, expert_offsets=None, num_experts: int = 1):
    """``out[e] (+)= dy[rows_e]ᵀ @ x[rows_e]`` -> ``[E?, N_out, K_in]``; fp32 or bf16 output."""
    R, M = dy.shape
    N = x.shape[1]
    if M <= 16 and expert_offsets is None:
        if out is None:
            out = torch.zeros(M, N, dtype=torch.float32, device=dy.device)
            accumulate = True
        if out.dtype != torch.float32:
            raise TypeError("skinny weight gradients accumulate in fp32")
        if not accumulate:
            out.zero_()
        _call("b2_skinny_tn", _p(dy.float().contiguous()), _p(_bf16(x)), _p(out), _I(R), _I(M), _I(N), _stream())
        return out if out_dtype is None else out.to(out_dtype)
    want = None
    if out is None:
        want = out_dtype or torch.float32
        store = torch.float32 if want not in (torch.float32, torch.bfloat16) else want
        shape = (num_experts, M, N) if expert_offsets is not None else (M, N)
        out = torch.empty(shape, dtype=store, device=dy.device)
        accumulate = False
    kind = 1 if out.dtype == torch.float32 else 2
    assert dy.stride(-1) == 1 and x.stride(-1) == 1 and out.is_contiguous()
    _call("b2_gemm_tn", _p(_bf16(dy)), _p(_bf16(x)), _p(out), _I(M), _I(N), _I(R), _L(dy.stride(0)), _L(x.stride(0)),
          _L(N), _I(num_experts), _p(expert_offsets), _I(kind), _F(1.0 if accumulate else 0.0),
          _p(status_word(dy.device)), _stream(),
          tag=f"{'grouped ' if expert_offsets is not None else ''}{M}x{N} {'fp32' if kind == 1 else 'bf16'}")
    return out if want is None or want == out.dtype else out.to(want)


def gemm_swiglu(x, w1, w3, tile_expert=None, num_m_tiles=None, save_gate_up: bool = True, align256: bool = False):
    """``h = silu(x w1ᵀ) · (x w3ᵀ)`` per expert tile; optionally also the two pre-activations."""
    M, K = x.shape
    E, F = w1.shape[0], w1.shape[1]
    h = torch.empty(M, F, dtype=torch.bfloat16, device=x.device)
    gate = torch.empty_like(h) if save_gate_up else None
    up = torch.empty_like(h) if save_gate_up else None
    _call("b2_gemm_swiglu", _p(_bf16(x)), _p(_bf16(w1)), _p(_bf16(w3)), _p(h), _p(gate), _p(up), _I(M), _I(F), _I(K),
          _L(x.stride(0)), _I(E), _p(tile_expert), _p(num_m_tiles), _I(int(align256)), _p(status_word(x.device)),
          _stream())
    return h, gate, up


# ------------------------------------------------------------------------------ norms
def rmsnorm_fwd(x, weight, eps):
    x2 = _bf16(x).reshape(-1, x.shape[-1])
    y = torch.empty_like(x2)
    rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
    _call("b2_rmsnorm_fwd", _p(x2), _p(None), _p(weight), _p(None), _p(y), _p(rstd), _I(x2.shape[0]), _I(x2.shape[1]),
          _F(eps), _stream())
    return y.view(x.shape), rstd


def add_rmsnorm_fwd(x, delta, weight, eps):
    x2, d2 = _bf16(x).reshape(-1, x.shape[-1]), _bf16(delta).reshape(-1, x.shape[-1])
    summed, y = torch.empty_like(x2), torch.empty_like(x2)
    rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
    _call("b2_rmsnorm_fwd", _p(x2), _p(d2), _p(weight), _p(summed), _p(y), _p(rstd), _I(x2.shape[0]), _I(x2.shape[1]),
          _F(eps), _stream())
    return summed.view(x.shape), y.view(x.shape), rstd


def rmsnorm_bwd(dy, x, weight, rstd, residual_grad=None):
    x2 = x.reshape(-1, x.shape[-1])
    dy2 = _bf16(dy).reshape(-1, x.shape[-1])
    rows, D = x2.shape
    parts = require().b2_rmsnorm_bwd_parts(_I(rows))
    partial = torch.empty(parts, D, dtype=torch.float32, device=x.device)
    dx = torch.empty_like(x2)
    dw = torch.empty(D, dtype=torch.float32, device=x.device)
    res = None if residual_grad is None else _bf16(residual_grad).reshape(-1, D).contiguous()
    _call("b2_rmsnorm_bwd", _p(dy2), _p(x2), _p(weight), _p(rstd), _p(res), _p(dx), _p(partial), _p(dw), _I(rows), _I(D),
          _stream(), n=2)
    return dx.view(x.shape), dw


# ------------------------------------------------------------------------------ router
def router_top2_fwd(logits):
    logits = logits.float().contiguous()
    T, E = logits.shape
    weights = torch.empty(T, 2, dtype=torch.float32, device=logits.device)
    idx = torch.empty(T, 2, dtype=torch.int64, device=logits.device)
    probs = torch.empty(T, E, dtype=torch.float32, device=logits.device)
    _call("b2_router_top2_fwd", _p(logits), _p(weights), _p(idx), _p(probs), _I(T), _I(E), _stream())
    return weights, idx, probs


def router_top2_bwd(dweights, probs, idx, weights):
    T, E = probs.shape
    dlogits = torch.empty(T, E, dtype=torch.float32, device=probs.device)
    _call("b2_router_top2_bwd", _p(dweights.float().contiguous()), _p(probs), _p(idx), _p(weights), _p(dlogits), _I(T),
          _I(E), _stream())
    return dlogits


# ------------------------------------------------------------------------------ loss
def cross_entropy_fwd_bwd_(logits, targets):
    """Mean loss; ``logits`` (bf16 [T,V]) is overwritten with d(mean loss)/dlogits."""
    T, V = logits.shape
    loss = torch.zeros((), dtype=torch.float32, device=logits.device)
    _call("b2_cross_entropy", _p(_bf16(logits)), _p(targets.contiguous()), _p(loss), _I(T), _I(V), _F(1.0 / T), _stream())
    return loss


def cross_entropy_scaled_(logits, targets, loss, loss_scale: float, grad_scale: float):
    """Adds ``loss_scale · Σ_rows CE`` to ``loss`` (fp32 scalar tensor) and overwrites ``logits`` (bf16 [T,V]) with
    ``grad_scale · (softmax − onehot)``; rows up to 32768 entries are read once and written once."""
    T, V = logits.shape
    _call("b2_cross_entropy2", _p(_bf16(logits)), _p(targets.contiguous()), _p(loss), _I(T), _I(V), _F(loss_scale),
          _F(grad_scale), _stream())
    return loss


def scale_(x, factor):
    factor = factor.to(device=x.device, dtype=torch.float32).reshape(1)
    _call("b2_scale_bf16", _p(_bf16(x)), _p(factor), _L(x.numel()), _stream())
    return x


# ------------------------------------------------------------------------------ optimizer
_DT = {torch.float32: 0, torch.bfloat16: 1}


def adamw_(p, g, m, v, lr, beta1, beta2, eps, weight_decay, a_t, grad_scale=1.0, p_bf16=None):
    for t in (p, g, m, v):
        if not t.is_contiguous():
            raise ValueError("adamw_ needs contiguous tensors")
    _call("b2_adamw", _p(p), _p(g), _p(m), _p(v), _p(p_bf16), _L(p.numel()), _I(_DT[p.dtype]), _I(_DT[g.dtype]),
          _I(_DT[m.dtype]), _F(lr), _F(beta1), _F(beta2), _F(eps), _F(weight_decay), _F(a_t), _F(grad_scale), _stream())


def cast_f32_bf16(src, dst):
    _call("b2_cast_f32_bf16", _p(src), _p(dst), _L(src.numel()), _stream())


# ------------------------------------------------------------------------------ embedding / rope
def embedding_fwd(ids, table):
    flat = ids.reshape(-1).contiguous()
    out = torch.empty(flat.numel(), table.shape[1], dtype=table.dtype, device=table.device)
    _call("b2_embedding_fwd", _p(flat), _p(_bf16(table)), _p(out), _I(flat.numel()), _I(table.shape[1]), _stream())
    return out.view(*ids.shape, table.shape[1])


def embedding_bwd(flat_ids, dy2d, main_grad):
    _call("b2_embedding_bwd", _p(flat_ids.contiguous()), _p(_bf16(dy2d.contiguous())), _p(main_grad),
          _I(flat_ids.numel()), _I(dy2d.shape[1]), _stream())


def rope_inplace(buf, first_elem_offset, tokens, seq, heads, head_dim, pitch, cos, sin, sign):
    ptr = ctypes.c_void_p(buf.data_ptr() + first_elem_offset * buf.element_size())
    _call("b2_rope", ptr, _p(cos), _p(sin), _I(tokens), _I(seq), _I(heads), _I(head_dim), _L(pitch), _F(sign), _stream())


# ------------------------------------------------------------------------------ device clock
def device_timestamp(out=None, index: int = 0):
    """Enqueues a one-thread kernel that stores the GPU's ``globaltimer`` (nanoseconds, one clock for the whole
    device) into ``out[index]`` (int64, allocated if not given) when the stream reaches it."""
    if out is None:
        out = torch.zeros(2, dtype=torch.int64, device=torch.device("cuda", torch.cuda.current_device()))
    _call("b2_device_timestamp", ctypes.c_void_p(out.data_ptr() + 8 * index), _stream())
    return out


# ------------------------------------------------------------------------------ all-gather fused with its GEMM
def ag_gemm_grid() -> int:
    """CTAs per launch of ``ag_gemm_nt`` (its per-block counters advance by this much per launch)."""
    return int(require().b2_ag_gemm_grid())


def ag_gemm_plan(segments, world: int, rank: int):
    """Host-only: the schedule ``ag_gemm_nt`` uses for ``rank``.  Returns ``(order, n_local, owner)``: the column
    blocks (256 rows of ``W`` each) in launch order, how many of them (the leading ones) need no peer rows, and the
    owning rank of every row.  Needs no GPU."""
    segments = [int(v) for v in segments]
    total = sum(segments)
    blocks = (total + 255) // 256
    seg = (ctypes.c_int * len(segments))(*segments)
    order = (ctypes.c_int * max(blocks, 1))()
    owner = (ctypes.c_int * max(total, 1))()
    n_local = ctypes.c_int(0)
    rc = require().b2_ag_gemm_plan(seg, _I(len(segments)), _I(world), _I(rank), _I(total), order,
                                   ctypes.byref(n_local), owner)
    if rc != 0:
        raise ValueError(f"invalid row layout for the all-gather GEMM (code {rc})")
    return list(order[:blocks]), int(n_local.value), list(owner[:total])


def ag_gemm_nt(x, w_ptrs, n_rows: int, segments, world: int, rank: int, sig_ptrs, sig_slot: int, seq: int,
               block_flags, flag_epoch: int):
    """``x [M,K] @ W [n_rows,K]ᵀ`` where ``W`` is row-sharded over ``world`` ranks: ``w_ptrs`` holds every rank's
    copy of ``W`` (a ctypes array of ``MAX_RANKS`` addresses; in copy ``r`` the rows of rank ``r`` are current).
    ``segments``: row counts of the stacked parts of ``W`` that are sharded one by one (``[n_rows]`` for a plain
    layer, ``[q, k, v]`` rows for a fused projection); inside a part of ``S`` rows rank ``r`` owns rows
    ``[r·S/world, (r+1)·S/world)``.  The kernel pulls the peers' rows into this rank's copy while the tensor cores
    work on the local rows.  ``block_flags``: int32 ``[ceil(n_rows/256)]``, zero at first use; ``flag_epoch``:
    1, 2, ... per launch with those counters.  Returns ``None`` when the device cannot co-schedule the kernel
    (gather and multiply instead)."""
    M, K = x.shape
    if x.stride(1) != 1:
        raise ValueError("x must have unit inner stride")
    segments = [int(v) for v in segments]
    if sum(segments) != n_rows:
        raise ValueError("segments must add up to the rows of W")
    seg = (ctypes.c_int * len(segments))(*segments)
    y = torch.empty(M, n_rows, dtype=torch.bfloat16, device=x.device)
    rc = require().b2_ag_gemm_nt(_p(_bf16(x)), w_ptrs, _p(y), _I(M), _I(n_rows), _I(K), _L(x.stride(0)), _L(n_rows),
                                 seg, _I(len(segments)), _I(world), _I(rank), sig_ptrs, _I(sig_slot), _I(seq),
                                 _p(block_flags), _I(flag_epoch), _p(status_word(x.device)), _stream())
    if rc == -20:
        return None
    if rc != 0:
        raise RuntimeError(f"b2_ag_gemm_nt failed with code {rc}")
    global _launches
    _launches += 1
    return y


# ------------------------------------------------------------------------------ attention
def _token_pitch(t):
    B, S, H, hd = t.shape
    if hd != 128 or t.stride(3) != 1 or t.stride(2) != hd or t.stride(0) != S * t.stride(1):
        raise ValueError("attention tensors must be [B, S, H, 128] views with contiguous heads and uniform token pitch")
    return t.stride(1)


def attention_fwd(q, k, v, cos=None, sin=None, causal=True):
    """GQA attention, causal by default.  ``q [B,S,Hq,128]``, ``k, v [B,S,Hkv,128]`` bf16 (views of a fused projection are
    fine).  With ``cos``/``sin`` the rotation is applied to copies of q and k first.  Returns
    ``(out [B,S,Hq,128], lse fp32 [B,Hq,S], q_used, k_used)``."""
    B, S, Hq, hd = q.shape
    Hkv = k.shape[2]
    if cos is not None:
        q, k = q.contiguous().clone(), k.contiguous().clone()
        rope_inplace(q, 0, B * S, S, Hq, hd, Hq * hd, cos, sin, 1.0)
        rope_inplace(k, 0, B * S, S, Hkv, hd, Hkv * hd, cos, sin, 1.0)
    out = torch.empty(B, S, Hq, hd, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device)
    _call("b2_attention_fwd_ex", _p(_bf16(q)), _p(_bf16(k)), _p(_bf16(v)), _L(_token_pitch(q)), _L(_token_pitch(k)),
          _L(_token_pitch(v)), _p(out), _p(lse), _I(B), _I(S), _I(Hq), _I(Hkv), _F(hd ** -0.5), _I(int(causal)),
          _p(status_word(q.device)), _stream())
    return out, lse, q, k


def attention_bwd(dout, q, k, v, out, lse, cos=None, sin=None, grads=None, causal=True):
    """Gradients of ``attention_fwd``.  ``q`` and ``k`` are the tensors the forward kernel saw (rotated, if a
    rotation was applied); with ``cos``/``sin`` the kernels store dq and dk rotated back, i.e. as gradients of the
    unrotated q and k.  ``grads`` may give three preallocated ``[B,S,H,128]`` views (for instance slices of one
    fused buffer) to write into."""
    B, S, Hq, hd = q.shape
    Hkv = k.shape[2]
    if grads is None:
        grads = (torch.empty(B, S, Hq, hd, dtype=torch.bfloat16, device=q.device),
                 torch.empty(B, S, Hkv, hd, dtype=torch.bfloat16, device=q.device),
                 torch.empty(B, S, Hkv, hd, dtype=torch.bfloat16, device=q.device))
    dq, dk, dv = grads
    delta = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device)
    dout = _bf16(dout).contiguous()
    if cos is not None and (cos.shape[-1] != 64 or not cos.is_contiguous() or cos.shape[0] < S):
        raise ValueError("rotary tables must be contiguous fp32 [>= S, 64]")
    _call("b2_attention_bwd_rope", _p(dout), _p(q), _p(k), _p(v), _p(_bf16(out)), _p(lse), _L(_token_pitch(q)),
          _L(_token_pitch(k)), _L(_token_pitch(v)), _p(delta), _p(dq), _p(dk), _p(dv), _L(_token_pitch(dq)),
          _L(_token_pitch(dk)), _L(_token_pitch(dv)), _I(B), _I(S), _I(Hq), _I(Hkv), _F(hd ** -0.5),
          _I(int(causal)), _p(cos), _p(sin), _p(status_word(q.device)), _stream(), n=3)
    return dq, dk, dv


# ------------------------------------------------------------------------------ MoE routing
def moe_plan(idx, num_experts, capacity_rows):
    slots = idx.numel()
    dev = idx.device
    i32 = dict(dtype=torch.int32, device=dev)
    slot_row = torch.empty(slots, **i32)
    row_slot = torch.empty(capacity_rows, **i32)
    offs = torch.empty(num_experts, **i32)
    tile_expert = torch.empty(capacity_rows // 128, **i32)
    meta = torch.zeros(4, **i32)
    counts = torch.empty(num_experts, **i32)
    _call("b2_moe_plan", _p(idx.contiguous()), _I(slots), _I(num_experts), _p(slot_row), _p(row_slot), _p(offs),
          _p(tile_expert), _p(meta), _p(counts), _I(capacity_rows), _stream())
    return slot_row, row_slot, offs, tile_expert, meta, counts


def moe_gather(x, row_slot, meta, capacity_rows, scale=None, y_perm=None, dweights=None, out=None):
    D = x.shape[1]
    if out is None:
        out = torch.empty(capacity_rows, D, dtype=torch.bfloat16, device=x.device)
    _call("b2_moe_gather", _p(_bf16(x)), _p(row_slot), _p(meta), _p(scale), _p(y_perm), _p(dweights), _p(out), _I(D),
          _I(capacity_rows), _I(2 * x.shape[0]), _stream())
    return out


def moe_combine(y_perm, slot_row, weights, tokens, residual=None):
    D = y_perm.shape[1]
    out = torch.empty(tokens, D, dtype=torch.bfloat16, device=y_perm.device)
    _call("b2_moe_combine", _p(_bf16(y_perm)), _p(slot_row), _p(weights), _p(residual), _p(out), _I(tokens), _I(D),
          _I(y_perm.shape[0]), _stream())
    return out


def swiglu_bwd(dh, gate, up, live_rows=None, want_h: bool = True):
    rows, F = dh.shape
    dgu = torch.empty(rows, 2 * F, dtype=torch.bfloat16, device=dh.device)
    h = torch.empty(rows, F, dtype=torch.bfloat16, device=dh.device) if want_h else None
    _call("b2_swiglu_bwd", _p(_bf16(dh)), _p(gate), _p(up), _p(dgu), _p(h), _p(live_rows), _I(rows), _I(F), _stream())
    return dgu, h


# ------------------------------------------------------------------------------ expert-parallel return in the epilogue
def gemm_nt_push(a, w, tile_expert, num_m_tiles, num_experts, dst_table, row_tag, row_src, row_w, sig_table,
                 sig_slot: int, seq: int, rank: int, n: int, ticket):
    """Rows of ``a [M,K] @ w[e] [N,K]ᵀ``, scaled by ``row_w`` (or 1), stored as bf16 into row ``row_tag[r]`` of rank
    ``row_src[r]``'s buffer (``dst_table``: ctypes array of ``MAX_RANKS`` addresses, row pitch ``N``); afterwards
    flag ``seq`` is raised in slot ``sig_slot`` of every rank's signal pad."""
    M, K = a.shape
    N = w.shape[-2]
    assert a.stride(-1) == 1 and w.is_contiguous()
    _call("b2_gemm_nt_push", _p(_bf16(a)), _p(_bf16(w)), _I(M), _I(N), _I(K), _L(a.stride(0)), _I(num_experts),
          _p(tile_expert), _p(num_m_tiles), _I(1), dst_table, _p(row_tag), _p(row_src), _p(row_w), sig_table,
          _I(sig_slot), _I(seq), _I(rank), _I(n), _p(ticket), _p(status_word(a.device)), _stream())


def gemm_nn_push(a, w, w2, tile_expert, num_m_tiles, num_experts, dst_table, row_tag, row_src, row_w, sig_table,
                 sig_slot: int, seq: int, rank: int, n: int, ticket):
    """The same for ``a [M,K] @ [w[e]; w2[e]]`` (``w``, ``w2``: ``[E, K/2, N]``, the reduction runs over their rows)."""
    M, K = a.shape
    N = w.shape[-1]
    k_split = w.shape[-2] if w2 is not None else 0
    assert a.stride(-1) == 1 and w.is_contiguous()
    _call("b2_gemm_nn_push", _p(_bf16(a)), _p(_bf16(w)), _p(w2), _I(M), _I(N), _I(K), _I(k_split), _L(a.stride(0)),
          _I(num_experts), _p(tile_expert), _p(num_m_tiles), _I(1), dst_table, _p(row_tag), _p(row_src), _p(row_w),
          sig_table, _I(sig_slot), _I(seq), _I(rank), _I(n), _p(ticket), _p(status_word(a.device)), _stream())


def ep_swiglu_bwd(dh, gate_lo, up_lo, gate_hi, up_hi, split_row: int, dgu, meta, row_tag, row_src, row_w,
                  dw_table, n: int):
    """SwiGLU backward on expert-major rows with the routing weight folded in (see ``ep_swiglu_bwd_kernel``):
    ``dh`` is overwritten with ``w·h``, ``dgu`` receives ``w·[dgate | dup]``, the routing-weight gradient of every
    row goes to its source rank's ``dw_table`` entry."""
    rows, F = dh.shape
    _call("b2_ep_swiglu_bwd", _p(_bf16(dh)), _p(gate_lo), _p(up_lo), _p(gate_hi), _p(up_hi), _I(split_row), _p(dgu),
          _p(meta), _p(row_tag), _p(row_src), _p(row_w), dw_table, _I(rows), _I(F), _I(n), _stream())
