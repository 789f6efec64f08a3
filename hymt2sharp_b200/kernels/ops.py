"""Python face of the CUDA library: every function checks its tensors, passes raw
pointers and the current torch stream to one exported C function and raises
KernelError when that function refuses.  Nothing here computes; there is no
fallback to torch operators."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p

import torch

from .build import load_library

F32, BF16 = 0, 1
EPILOGUE_STORE, EPILOGUE_ACCUMULATE, EPILOGUE_SWIGLU = 0, 1, 2


class KernelError(RuntimeError):
    pass


def dtype_code(t: torch.dtype) -> int:
    if t == torch.float32:
        return F32
    if t == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {t} is not supported by the kernels (float32 and bfloat16 are)")


_library = None


def _lib():
    global _library
    if _library is None:
        _library = load_library()
    return _library


def _stream() -> c_void_p:
    # (the raw handle: torch.cuda.current_stream() builds a Stream object for it, ten times the cost, once per launch)
    return c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


launches = 0  # kernels of this library launched (or captured into a graph) so far

# The profiling switch (the counterpart of HunyuanDenseModel.ProfileEnabled and its tick counters,
# src/HyMT2Sharp/HunyuanDenseModel.cs:48-78): between profile_begin() and profile_end() every launch on the current
# stream is followed by a CUDA event, and the time between two events is booked under the launch's name, or under
# `tag` where a caller set one (a Linear names the product it is: "qkv", "o_proj", ...).  Kernels then run one after
# the other (an event between two launches keeps the second from starting early), so the sum is more than an
# unprofiled step takes; the shares are what it is for.  A step that is launched kernel by kernel from the host is
# timed truly only where its kernels outlast the host's work per launch (prompts); a decode step is therefore captured
# with a kernel between every two of its kernels that writes the device's clock (capture_begin/capture_end), and the
# stamps are read after each replay.
tag: str | None = None
_profile: list | None = None      # (name, event) in launch order, eager launches
_booked: dict | None = None       # {name: ms} already read from captured steps
_capturing: list | None = None    # the capture that is being made: [stamps, None, name, name, ...]
_suspended = False


def profile_begin() -> None:
    global _profile, _booked
    e = torch.cuda.Event(enable_timing=True)
    e.record()
    _profile = [(None, e)]
    _booked = {}


def profile_active() -> bool:
    return _profile is not None


def profile_end() -> dict:
    """{name: milliseconds} of everything launched since profile_begin(), in the order of first appearance."""
    global _profile, _booked
    events, _profile = _profile or [], None
    booked, _booked = _booked or {}, None
    torch.cuda.synchronize()
    out: dict = {}
    for (_, before), (name, after) in zip(events, events[1:]):
        if name is not None:
            out[name] = out.get(name, 0.0) + before.elapsed_time(after)
    for name, ms in booked.items():
        out[name] = out.get(name, 0.0) + ms
    return out


class profile_suspended:
    """Launches inside are not timed (a warm-up step in front of a capture)."""

    def __enter__(self):
        global _suspended
        self.was, _suspended = _suspended, True

    def __exit__(self, *exc):
        global _suspended
        _suspended = self.was
        if _profile is not None:   # what ran meanwhile is not booked to the next launch
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            _profile.append((None, e))


STAMPS = 8192   # kernels of one captured step that can be timed


def _stamp(stamps: torch.Tensor, index: int) -> None:
    rc = _lib().hymt2_stamp(ctypes.c_void_p(stamps.data_ptr() + 8 * index), _stream())
    if rc != 0:
        raise KernelError(f"stamp failed ({rc}): {_lib().hymt2_last_error().decode(errors='replace')}")


def capture_begin(device) -> None:
    """Inside a graph capture: from here on every launch is followed by a kernel that writes the device's clock."""
    global _capturing
    stamps = torch.zeros(STAMPS, dtype=torch.int64, device=device)
    _capturing = [stamps, None]
    _stamp(stamps, STAMPS - 2)   # two stamps with nothing between them: what a stamp itself costs
    _stamp(stamps, STAMPS - 1)
    _stamp(stamps, 0)


def capture_end() -> list:
    """[the stamps' tensor, None, name of launch 1, name of launch 2, ...]: what book_captured() wants."""
    global _capturing
    record, _capturing = _capturing or [], None
    return record


def book_captured(record: list) -> None:
    """After a replay of a graph captured between capture_begin() and capture_end(): waits for it and adds its kernels'
    times to the running profile (the time from the stamp in front of a kernel to the stamp behind it, less what a
    stamp costs)."""
    torch.cuda.synchronize()
    if _booked is None or not record:
        return
    names = record[2:]
    at = record[0].cpu().tolist()
    own = max(0, at[STAMPS - 1] - at[STAMPS - 2])
    for i, name in enumerate(names):
        _booked[name] = _booked.get(name, 0.0) + max(0, at[i + 1] - at[i] - own) * 1e-6


def profile_line(phase: str, times: dict) -> str:
    """One line in the manner of src/HyMT2Sharp.Benchmark/Program.cs:243-261."""
    body = " ".join(f"{k}={v:.2f}ms" for k, v in times.items())
    return f"profile {phase}: {body} accounted={sum(times.values()):.2f}ms"


def _check(rc: int, what: str, kernels: int = 1, timed: bool = True) -> None:
    global launches
    launches += kernels
    if rc != 0:
        msg = _lib().hymt2_last_error().decode(errors="replace")
        raise KernelError(f"{what} failed ({rc}): {msg}")
    if timed and kernels > 0 and not _suspended:
        if _capturing is not None:
            if len(_capturing) - 1 >= STAMPS - 2:
                raise KernelError(f"a captured step of more than {STAMPS - 3} kernels cannot be timed")
            _stamp(_capturing[0], len(_capturing) - 1)
            _capturing.append(tag or what)
        elif _profile is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            _profile.append((tag or what, e))


def _need(t: torch.Tensor, name: str, dtype=None, dims=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, got {t.dim()}")


# ---------------------------------------------------------------------------
def embed(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, status: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] = float32(table[ids[t]]) * scale; out is [T, hidden] float32."""
    _need(out, "out", torch.float32, 2); _need(table, "table", None, 2); _need(ids, "ids", torch.int32, 1)
    T, H = out.shape
    if table.shape[1] != H or ids.shape[0] < T:
        raise KernelError(f"embed: shapes out {tuple(out.shape)} table {tuple(table.shape)} ids {tuple(ids.shape)}")
    _check(_lib().hymt2_embed(_ptr(out), _ptr(table), c_int(dtype_code(table.dtype)), _ptr(ids), c_int(T),
                              c_int(H), c_int(table.shape[0]), c_float(scale), _ptr(status), _stream()), "embed")


def advance_decode(token_pos: torch.Tensor, kv_lens: torch.Tensor, slot_ids: torch.Tensor) -> None:
    """After a decode step: positions and lengths of the live rows (slot >= 0) grow by one."""
    _need(token_pos, "token_pos", torch.int32, 1); _need(kv_lens, "kv_lens", torch.int32, 1)
    _need(slot_ids, "slot_ids", torch.int32, 1)
    _check(_lib().hymt2_advance_decode(_ptr(token_pos), _ptr(kv_lens), _ptr(slot_ids), c_int(slot_ids.shape[0]),
                                       _stream()), "advance_decode")


PREFETCH_MAX_BYTES = 48 << 20   # of a larger tensor only the beginning is asked for: more would push too much else out of L2
_side = {}   # device index -> (side stream, event, whether the side stream has work that the main stream has not joined)


def prefetch_beside(t: torch.Tensor) -> None:
    """Asks for the beginning of `t` (at most PREFETCH_MAX_BYTES) to be brought into L2 by a small kernel on a
    stream BESIDE the current one, ordered after everything launched on the current stream so far.  The current
    stream does not wait for it (join_beside does, once, at the end of a step), so kernels that follow run while
    the memory fetches; in a captured step this is a branch of the graph."""
    if t is None or not t.is_contiguous() or t.data_ptr() % 16:
        return
    nbytes = min(t.numel() * t.element_size(), PREFETCH_MAX_BYTES)
    key = t.device.index if t.device.index is not None else torch.cuda.current_device()
    if key not in _side:
        _side[key] = [torch.cuda.Stream(device=t.device), torch.cuda.Event(), False]
    side, event, _ = _side[key]
    main = torch.cuda.current_stream(t.device)
    event.record(main)
    side.wait_event(event)
    with torch.cuda.stream(side):
        _check(_lib().hymt2_l2_prefetch(_ptr(t), c_long(nbytes), _stream()), "l2_prefetch", timed=False)
    _side[key][2] = True


def join_beside(device) -> None:
    """The current stream waits for what prefetch_beside put on the side stream (a step calls it at its end)."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _side.get(key)
    if st and st[2]:
        torch.cuda.current_stream(device).wait_stream(st[0])
        st[2] = False


def rmsnorm(out: torch.Tensor, x: torch.Tensor, gain: torch.Tensor, eps: float,
            rows_index: torch.Tensor | None = None, out_scale: float = 1.0) -> None:
    """out[r] = rmsnorm(x[rows_index[r]] or x[r]) * gain * out_scale, computed in float32."""
    _need(out, "out", None, 2); _need(x, "x", None, 2); _need(gain, "gain", None, 1)
    rows, dim = out.shape
    if x.shape[1] != dim or gain.shape[0] != dim:
        raise KernelError(f"rmsnorm: shapes out {tuple(out.shape)} x {tuple(x.shape)} gain {tuple(gain.shape)}")
    if rows_index is not None:
        _need(rows_index, "rows_index", torch.int32, 1)
        if rows_index.shape[0] < rows:
            raise KernelError("rmsnorm: rows_index is shorter than out")
    elif x.shape[0] < rows:
        raise KernelError("rmsnorm: x has fewer rows than out")
    _check(_lib().hymt2_rmsnorm(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(x), c_int(dtype_code(x.dtype)),
                                _ptr(gain), c_int(dtype_code(gain.dtype)), _ptr(rows_index), c_int(rows),
                                c_int(dim), c_float(eps), c_float(out_scale), _stream()), "rmsnorm")


def silu_mul(out: torch.Tensor, gate_up: torch.Tensor) -> None:
    """out[r, c] = silu(gate_up[r, c]) * gate_up[r, width + c]."""
    _need(out, "out", None, 2); _need(gate_up, "gate_up", out.dtype, 2)
    rows, width = out.shape
    if gate_up.shape != (rows, 2 * width):
        raise KernelError(f"silu_mul: shapes out {tuple(out.shape)} gate_up {tuple(gate_up.shape)}")
    _check(_lib().hymt2_silu_mul(_ptr(out), _ptr(gate_up), c_int(dtype_code(out.dtype)), c_int(rows), c_int(width),
                                 _stream()), "silu_mul")


def gemm_simt(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, epilogue: int = EPILOGUE_STORE) -> None:
    """out[M, N] = epilogue(a[M, K] @ w[N, K]^T) on CUDA cores, float32 accumulation in K order.
    With EPILOGUE_SWIGLU w has 2N rows (gate rows, then up rows)."""
    for t, n in ((out, "out"), (a, "a"), (w, "w")):
        if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm: {n} must be a CUDA matrix with contiguous rows")
    M, N = out.shape
    K = a.shape[1]
    rows_w = 2 * N if epilogue == EPILOGUE_SWIGLU else N
    if a.shape[0] != M or w.shape != (rows_w, K):
        raise KernelError(f"gemm: shapes out {tuple(out.shape)} a {tuple(a.shape)} w {tuple(w.shape)} epilogue {epilogue}")
    _check(_lib().hymt2_gemm_simt(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(a), c_int(dtype_code(a.dtype)),
                                  _ptr(w), c_int(dtype_code(w.dtype)), c_int(M), c_int(N), c_int(K),
                                  c_long(a.stride(0)), c_long(w.stride(0)), c_long(out.stride(0)),
                                  c_int(epilogue), _stream()), "gemm_simt")


_status: dict = {}
_status_of: dict = {}   # the same by what callers pass (a torch.device with an index)


def device_status(device) -> torch.Tensor:
    """The int32[4] status word of a device: kernels set [0] when a device-side check fails or a
    bounded wait gives up (1: token id outside the table; 2: a sequence longer than the split attention was given
    room for; 101-106: a wait of the tensor-core GEMM (106: for the partial sums of a tile's other CTAs); 108-119: of the prompt attention; 120-129: of the decode
    attention)."""
    hit = _status_of.get(device)
    if hit is not None:
        return hit
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(4, dtype=torch.int32, device=dev)
    if dev.index is not None:          # ("cuda" without an index means the current device, which may change)
        _status_of[device] = _status[key]
    return _status[key]


_tc_scratch: dict = {}   # device index -> (workspace float32, counters int32, earlier tensors kept alive)


def _tc_workspace(device: torch.device, floats: int, counters: int):
    """Scratch of the split-K tensor-core GEMM: partial tiles and per-tile arrival counters.  One
    pair per device, shared by all calls (they run in stream order); it only ever grows, and what it
    replaced stays alive because captured graphs may still point at it."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    ws, cnt, old = _tc_scratch.get(key, (None, None, []))
    if ws is None or ws.numel() < floats or cnt.numel() < counters:
        if ws is not None:
            old = old + [ws, cnt]
        ws = torch.empty(max(floats, 8 << 20), dtype=torch.float32, device=device)
        cnt = torch.zeros(max(counters, 1 << 14), dtype=torch.int32, device=device)
        _tc_scratch[key] = (ws, cnt, old)
    return ws, cnt


def gemm_tc_supported(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, epilogue: int) -> bool:
    """Whether the tcgen05 kernel takes these operands (types, alignment, the epilogue's output type)."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    if a.dim() != 2 or w.dim() != 2 or out.dim() != 2 or a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        return False
    K = a.shape[1]
    if K % 8 or a.stride(0) % 8 or w.stride(0) % 8 or a.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    if epilogue == EPILOGUE_STORE:
        return out.dtype in (torch.bfloat16, torch.float32)
    if epilogue == EPILOGUE_ACCUMULATE:
        return out.dtype == torch.float32
    return out.dtype == torch.bfloat16


def gemm_tc_norm_tiles(tokens: int, out_features: int, inner: int, epilogue: int) -> int:
    """How many partial sums of squares per token gemm_tc leaves behind when it is asked to prepare the norm that follows it
    (`norm_after`); 0: this shape's plan cannot, and the norm runs as a kernel of its own."""
    key = (tokens, out_features, inner, epilogue)
    hit = _norm_tiles.get(key)
    if hit is None:
        hit = _norm_tiles[key] = int(_lib().hymt2_gemm_tc_norm_tiles(c_int(tokens), c_int(out_features), c_int(inner), c_int(epilogue)))
    return hit


# What the library answered about a shape (its plan depends on the sizes and the device's SMs only): asked once a shape,
# since a step asks the same questions layer after layer.
_norm_tiles: dict = {}
_plans: dict = {}
_rope_plans: dict = {}


def _plan_scratch(T: int, N: int, K: int, epilogue: int) -> tuple:
    """(floats of workspace, counters) that the tensor-core product of this shape wants."""
    key = (T, N, K, epilogue)
    hit = _plans.get(key)
    if hit is None:
        floats, counters = ctypes.c_long(0), c_int(0)
        _check(_lib().hymt2_gemm_tc_plan(c_int(T), c_int(N), c_int(K), c_int(epilogue), ctypes.byref(floats),
                                         ctypes.byref(counters)), "gemm_tc_plan", 0)
        hit = _plans[key] = (floats.value, counters.value)
    return hit


def gemm_tc(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, epilogue: int, status: torch.Tensor,
            row_scale: tuple | None = None, norm_after: tuple | None = None, checked: bool = False) -> None:
    """out[T, N] = epilogue(a[T, K] @ w[N, K]^T) on the tcgen05 tensor cores (bfloat16 operands,
    float32 accumulation in tensor memory).  With EPILOGUE_SWIGLU w has 2N rows.

    An RMSNorm can be folded into the products around it.  `row_scale` = (ss [T, tiles] float32, width, eps): `a` holds
    bf16(x * gain) and the sums are multiplied by 1 / sqrt(sum(ss[t]) / width + eps) (store and SwiGLU epilogues).
    `norm_after` = (normed [T, N] bfloat16, gain [N], ss [T, gemm_tc_norm_tiles(...)] float32), accumulate epilogue only:
    bf16(out_new * gain) and the partial sums of squares of the new rows are written for the product that comes next.
    `checked`: the caller has just asked gemm_tc_supported about these very operands."""
    T, N = out.shape
    K = a.shape[1]
    rows_w = 2 * N if epilogue == EPILOGUE_SWIGLU else N
    if a.shape[0] != T or w.shape != (rows_w, K) or not (checked or gemm_tc_supported(out, a, w, epilogue)):
        raise KernelError(f"gemm_tc: operands out {tuple(out.shape)} {out.dtype} a {tuple(a.shape)} {a.dtype} "
                          f"w {tuple(w.shape)} {w.dtype} epilogue {epilogue} are not taken")
    floats, counters = _plan_scratch(T, N, K, epilogue)
    ws = cnt = None
    if floats:
        ws, cnt = _tc_workspace(out.device, floats, counters)
    ss_in = normed = gain = ss_out = None
    tiles_in, width, eps = 0, 0, 0.0
    if row_scale is not None:
        ss_in, width, eps = row_scale
        _need(ss_in, "row_scale sums", torch.float32, 2)
        if ss_in.shape[0] < T or epilogue == EPILOGUE_ACCUMULATE:
            raise KernelError("gemm_tc: row_scale needs sums for every token and a store or SwiGLU epilogue")
        tiles_in = ss_in.shape[1]
    if norm_after is not None:
        normed, gain, ss_out = norm_after
        tiles = gemm_tc_norm_tiles(T, N, K, epilogue)
        _need(normed, "normed", torch.bfloat16, 2); _need(gain, "gain", None, 1); _need(ss_out, "ss_out", torch.float32, 2)
        if tiles == 0 or normed.shape != (T, N) or gain.shape[0] != N or ss_out.shape != (T, tiles) or out.dtype != torch.float32:
            raise KernelError(f"gemm_tc: norm_after does not fit T={T} N={N} K={K} epilogue {epilogue} (tiles {tiles})")
    _check(_lib().hymt2_gemm_tc_norm(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(a), _ptr(w), c_int(T), c_int(N), c_int(K),
                                     c_long(a.stride(0)), c_long(w.stride(0)), c_long(out.stride(0)), c_int(epilogue),
                                     _ptr(ws), c_long(ws.numel() if ws is not None else 0), _ptr(cnt),
                                     c_int(cnt.numel() if cnt is not None else 0), _ptr(status), _stream(),
                                     _ptr(ss_in), c_int(tiles_in), c_int(width), c_float(eps), _ptr(normed), _ptr(gain),
                                     c_int(dtype_code(gain.dtype) if gain is not None else F32), _ptr(ss_out)), "gemm_tc")


def gemm_tc_debug(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, epilogue: int, status: torch.Tensor,
                  wait_limit: int, withhold_block: int) -> None:
    """gemm_tc with a fault put in on purpose: the copies of k block `withhold_block` are announced and never made,
    and every wait gives up after `wait_limit` tries.  The kernel must set status[0] = 102, free what it holds and
    return; `out` is then not a product.  Only products of few tokens whose K is not cut are taken."""
    T, N = out.shape
    K = a.shape[1]
    if a.shape[0] != T or w.shape != (N, K) or not gemm_tc_supported(out, a, w, epilogue):
        raise KernelError("gemm_tc_debug: operands are not taken")
    _check(_lib().hymt2_gemm_tc_debug(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(a), _ptr(w), c_int(T), c_int(N), c_int(K),
                                      c_long(a.stride(0)), c_long(w.stride(0)), c_long(out.stride(0)), c_int(epilogue),
                                      _ptr(status), _stream(), c_int(wait_limit), c_int(withhold_block)), "gemm_tc_debug")


def gemm_tc_rope_kv_supported(x: torch.Tensor, w: torch.Tensor, nh: int, nkv: int, d: int, cache_dtype, rope_dim: int) -> bool:
    """Whether the fused projection + rotation + cache append takes these operands: bfloat16, head_dim 128, and
    either few enough tokens that the product is cut over K among clusters (any even rope_dim), or more than 128
    tokens, which are the accumulator's rows (rope_dim 0 or 128)."""
    if d != 128 or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or cache_dtype != torch.bfloat16:
        return False
    if x.dim() != 2 or w.dim() != 2 or x.stride(1) != 1 or w.stride(1) != 1 or w.shape != ((nh + 2 * nkv) * d, x.shape[1]):
        return False
    K = x.shape[1]
    if K % 8 or x.stride(0) % 8 or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    key = (x.shape[0], w.shape[0], K, rope_dim)
    hit = _rope_plans.get(key)
    if hit is None:
        hit = _rope_plans[key] = bool(_lib().hymt2_gemm_tc_rope_kv_supported(c_int(key[0]), c_int(key[1]), c_int(K), c_int(rope_dim)))
    return hit


def gemm_tc_rope_kv(x: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, k_plane: torch.Tensor | None,
                    v_plane: torch.Tensor | None, block_table: torch.Tensor, block_tokens: int, token_seq: torch.Tensor,
                    token_pos: torch.Tensor, slot_ids: torch.Tensor, inv_freq: torch.Tensor | None, rope_dim: int,
                    q_gain: torch.Tensor | None, k_gain: torch.Tensor | None, eps: float, nh: int, nkv: int,
                    status: torch.Tensor, angles: torch.Tensor | None = None, row_scale: tuple | None = None,
                    checked: bool = False) -> None:
    """q_out[T, nh*128] = rotation and per-head norm of the query part of x @ w^T; the key part, rotated and
    normed, and the value part go to the rows of the cache planes that (slot, position) of every token name
    (k_plane None: nothing is written).  One tcgen05 kernel; head_dim 128; see rope_kv for the arguments.
    `angles`: what rope_angles(token_pos, inv_freq) gave, where gemm_tc_rope_kv_wants_angles says so.
    `row_scale` = (ss [T, tiles] float32, width, eps): x holds bf16(h * gain) of an RMSNorm whose row scale is applied to the
    projection's sums here (see gemm_tc).  `checked`: the caller has just asked gemm_tc_rope_kv_supported about these operands."""
    d = 128
    T = x.shape[0]
    if gemm_tc_rope_kv_wants_angles(T, rope_dim):
        if angles is None:
            raise KernelError(f"gemm_tc_rope_kv: {T} tokens need the table of their angles (rope_angles)")
        _need(angles, "angles", torch.float32, 3)
        if angles.shape != (T, rope_dim // 2, 2) or not angles.is_contiguous():
            raise KernelError(f"gemm_tc_rope_kv: angles is {tuple(angles.shape)}, expected {(T, rope_dim // 2, 2)}")
    else:
        angles = None
    if not (checked or gemm_tc_rope_kv_supported(x, w, nh, nkv, d, (k_plane if k_plane is not None else q_out).dtype, rope_dim)):
        raise KernelError(f"gemm_tc_rope_kv: operands x {tuple(x.shape)} {x.dtype} w {tuple(w.shape)} {w.dtype} are not taken")
    _need(q_out, "q_out", torch.bfloat16, 2)
    if q_out.shape != (T, nh * d) or not q_out.is_contiguous():
        raise KernelError(f"gemm_tc_rope_kv: q_out is {tuple(q_out.shape)}, expected {(T, nh * d)}")
    write = k_plane is not None
    if write:
        for t, n in ((k_plane, "k_plane"), (v_plane, "v_plane")):
            _need(t, n, torch.bfloat16, 4)
            if t.shape[1:] != (nkv, block_tokens, d):
                raise KernelError(f"gemm_tc_rope_kv: {n} is {tuple(t.shape)}, expected [blocks, {nkv}, {block_tokens}, {d}]")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((token_seq, "token_seq"), (token_pos, "token_pos"), (slot_ids, "slot_ids")):
        _need(t, n, torch.int32, 1)
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] != rope_dim // 2:
            raise KernelError("gemm_tc_rope_kv: inv_freq must hold rope_dim/2 values")
    gain_dtype = F32
    if q_gain is not None:
        _need(q_gain, "q_gain", None, 1); _need(k_gain, "k_gain", q_gain.dtype, 1)
        if q_gain.shape[0] != d or k_gain.shape[0] != d:
            raise KernelError("gemm_tc_rope_kv: the gains must hold head_dim values")
        gain_dtype = dtype_code(q_gain.dtype)
    _check(_lib().hymt2_gemm_tc_rope_kv(_ptr(x), _ptr(w), c_int(T), c_int(x.shape[1]), c_long(x.stride(0)), c_long(w.stride(0)),
                                        _ptr(q_out), _ptr(k_plane), _ptr(v_plane), _ptr(block_table),
                                        c_int(block_table.stride(0)), c_int(block_tokens), _ptr(token_seq), _ptr(token_pos),
                                        _ptr(slot_ids), _ptr(inv_freq), _ptr(angles), c_int(rope_dim), _ptr(q_gain), _ptr(k_gain),
                                        c_int(gain_dtype), c_float(eps), c_int(nh), c_int(nkv), c_int(1 if write else 0),
                                        _ptr(status), _stream(), _ptr(row_scale[0] if row_scale else None),
                                        c_int(row_scale[0].shape[1] if row_scale else 0), c_int(row_scale[1] if row_scale else 0),
                                        c_float(row_scale[2] if row_scale else 0.0)), "gemm_tc_rope_kv")


def gemm_tc_describe(tokens: int, out_features: int, inner: int, epilogue: int, sm_count: int = 0) -> dict:
    """How the tensor-core kernel would run this product (nothing is launched; works without a GPU when sm_count
    is given): orientation, kernel, tile width, ring depth, splits of K and how they fold, tiles and CTAs.
    epilogue: EPILOGUE_STORE / _ACCUMULATE / _SWIGLU, or 3 for the q/k/v projection with rotation."""
    out = (ctypes.c_int * 8)()
    rc = _lib().hymt2_gemm_tc_describe(c_int(tokens), c_int(out_features), c_int(inner), c_int(epilogue), c_int(sm_count), out)
    if rc != 0:
        raise KernelError(f"gemm_tc_describe failed ({rc}): {_lib().hymt2_last_error().decode(errors='replace')}")
    keys = ("swapped", "persistent", "tile_width", "stages", "k_splits", "cluster", "tiles", "ctas")
    return {k: (bool(v) if k in ("swapped", "persistent", "cluster") else int(v)) for k, v in zip(keys, out)}


def protocol_numbers() -> dict:
    """The numbers that the barrier protocols of the tcgen05 kernels are built on, as compiled (stages, slots, barriers
    per purpose, issuers): what an exploration of the protocols has to be run with.  Works without a GPU."""
    def ask(fn, names):
        out = (ctypes.c_int * 8)()
        getattr(_lib(), fn)(out)
        return dict(zip(names, out))
    return {"prefill": ask("hymt2_attention_prefill_tc_protocol", ("kv_stages", "k_slots", "p_bars", "o_bars", "stage_holders", "s_buffers")),
            "decode": ask("hymt2_attention_decode_tc_protocol", ("stages", "accumulators")),
            "gemm": ask("hymt2_gemm_tc_protocol", ("max_stages", "accumulators", "issuers", "issuers_own_stages", "epilogue_groups"))}


def gemm_tc_rope_kv_wants_angles(tokens: int, rope_dim: int) -> bool:
    """Whether gemm_tc_rope_kv of this many tokens wants the table of their angles: where tokens are the
    accumulator's rows, a thread owns a whole token and would compute every angle once per head."""
    key = ("angles", tokens, rope_dim)
    hit = _rope_plans.get(key)
    if hit is None:
        hit = _rope_plans[key] = bool(_lib().hymt2_gemm_tc_rope_kv_wants_angles(c_int(tokens), c_int(rope_dim)))
    return hit


def rope_angles(token_pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """[T, rope_dim/2, 2] float32: (cos, sin) of float32(position) * inv_freq, the product and the functions of
    the rotation kernels; once per step and frequency table, for every layer that uses that table."""
    _need(token_pos, "token_pos", torch.int32, 1)
    _need(inv_freq, "inv_freq", torch.float32, 1)
    out = torch.empty((token_pos.shape[0], inv_freq.shape[0], 2), dtype=torch.float32, device=token_pos.device)
    _check(_lib().hymt2_rope_angles(_ptr(out), _ptr(token_pos), _ptr(inv_freq), c_int(token_pos.shape[0]),
                                    c_int(inv_freq.shape[0]), _stream()), "rope_angles")
    return out


def rope_kv(qkv: torch.Tensor, q_out: torch.Tensor, k_plane: torch.Tensor | None, v_plane: torch.Tensor | None,
            block_table: torch.Tensor, block_tokens: int, token_seq: torch.Tensor, token_pos: torch.Tensor,
            slot_ids: torch.Tensor, inv_freq: torch.Tensor | None, rope_dim: int, q_gain: torch.Tensor | None,
            k_gain: torch.Tensor | None, eps: float, nh: int, nkv: int, d: int) -> None:
    """Rotation, per-head norm and cache append for the fused projection qkv[T, (nh+2nkv)*d].
    k_plane/v_plane are one layer's cache planes [blocks, nkv, block_tokens, d], or None to
    write no keys and values (a layer that reads another layer's cache)."""
    _need(qkv, "qkv", None, 2); _need(q_out, "q_out", qkv.dtype, 2)
    T = q_out.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * d or q_out.shape[1] != nh * d or qkv.shape[0] < T:
        raise KernelError(f"rope_kv: shapes qkv {tuple(qkv.shape)} q_out {tuple(q_out.shape)} for nh={nh} nkv={nkv} d={d}")
    write = k_plane is not None
    if write:
        for t, n in ((k_plane, "k_plane"), (v_plane, "v_plane")):
            _need(t, n, qkv.dtype, 4)
            if t.shape[1:] != (nkv, block_tokens, d):
                raise KernelError(f"rope_kv: {n} is {tuple(t.shape)}, expected [blocks, {nkv}, {block_tokens}, {d}]")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((token_seq, "token_seq"), (token_pos, "token_pos"), (slot_ids, "slot_ids")):
        _need(t, n, torch.int32, 1)
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] != rope_dim // 2:
            raise KernelError("rope_kv: inv_freq must hold rope_dim/2 values")
    gain_dtype = F32
    if q_gain is not None:
        _need(q_gain, "q_gain", None, 1); _need(k_gain, "k_gain", q_gain.dtype, 1)
        if q_gain.shape[0] != d or k_gain.shape[0] != d:
            raise KernelError("rope_kv: the q and k gains must have head_dim entries")
        gain_dtype = dtype_code(q_gain.dtype)
    _check(_lib().hymt2_rope_kv(_ptr(qkv), _ptr(q_out), _ptr(k_plane), _ptr(v_plane), c_int(dtype_code(qkv.dtype)),
                                _ptr(block_table), c_int(block_table.stride(0)), c_int(block_tokens),
                                _ptr(token_seq), _ptr(token_pos), _ptr(slot_ids), _ptr(inv_freq), c_int(rope_dim),
                                _ptr(q_gain), _ptr(k_gain), c_int(gain_dtype), c_float(eps), c_int(T), c_int(nh),
                                c_int(nkv), c_int(d), c_int(1 if write else 0), _stream()), "rope_kv")


def attention_simt_scratch(tokens: int, nh: int, d: int, max_splits: int) -> tuple[int, int]:
    """Floats of scratch (partial outputs, partial max/sum) that a split run needs."""
    return tokens * nh * max_splits * d, tokens * nh * max_splits * 2


def attention_simt(out: torch.Tensor, q: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                   block_table: torch.Tensor, cu_seqlens: torch.Tensor, slot_ids: torch.Tensor,
                   kv_lens: torch.Tensor, batch: int, max_new_tokens: int, nh: int, nkv: int, d: int,
                   scale: float, window: int = 0, split_keys: int = 0, max_splits: int = 0,
                   part_acc: torch.Tensor | None = None, part_ml: torch.Tensor | None = None,
                   status: torch.Tensor | None = None) -> None:
    """Causal grouped-query attention of the new tokens over the paged cache (CUDA cores).  With a split, a row
    longer than max_splits * split_keys is left as it was and status[0] (the device's status word unless another is
    given) becomes 2."""
    if status is None:
        status = device_status(out.device)
    _need(out, "out", None, 2); _need(q, "q", out.dtype, 2)
    _need(k_plane, "k_plane", out.dtype, 4); _need(v_plane, "v_plane", out.dtype, 4)
    T = out.shape[0]
    block_tokens = k_plane.shape[2]
    if out.shape[1] != nh * d or q.shape[1] != nh * d or q.shape[0] < T or k_plane.shape[1] != nkv \
            or k_plane.shape[3] != d or v_plane.shape != k_plane.shape:
        raise KernelError(f"attention: shapes out {tuple(out.shape)} q {tuple(q.shape)} k {tuple(k_plane.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    if split_keys > 0:
        need_acc, need_ml = attention_simt_scratch(T, nh, d, max_splits)
        _need(part_acc, "part_acc", torch.float32); _need(part_ml, "part_ml", torch.float32)
        if part_acc.numel() < need_acc or part_ml.numel() < need_ml:
            raise KernelError("attention: the split scratch is too small")
    _check(_lib().hymt2_attention_simt(_ptr(out), _ptr(q), _ptr(k_plane), _ptr(v_plane), c_int(dtype_code(out.dtype)),
                                       _ptr(block_table), c_int(block_table.stride(0)), c_int(block_tokens),
                                       _ptr(cu_seqlens), _ptr(slot_ids), _ptr(kv_lens), c_int(batch), c_int(T),
                                       c_int(max_new_tokens), c_int(nh), c_int(nkv), c_int(d), c_float(scale),
                                       c_int(window), c_int(split_keys), c_int(max_splits), _ptr(part_acc),
                                       _ptr(part_ml), _stream(), _ptr(status)), "attention_simt", 2 if split_keys > 0 else 1)


def attention_decode_tc_scratch(rows: int, nh: int, nkv: int, d: int, max_splits: int) -> tuple[int, int, int]:
    """What attention_decode_tc needs: floats of partial outputs, floats of partial (maximum, sum), one
    copy for each quarter of d, and zeroed int32 counters."""
    return rows * nh * max_splits * d, rows * nh * max_splits * 8, rows * nkv * 4


def attention_decode_tc(out: torch.Tensor, q: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                        block_table: torch.Tensor, slot_ids: torch.Tensor, kv_lens: torch.Tensor, nh: int, nkv: int,
                        d: int, scale: float, window: int, max_splits: int, part_acc: torch.Tensor,
                        part_ml: torch.Tensor, counters: torch.Tensor, status: torch.Tensor) -> None:
    """bfloat16 decode attention on the tcgen05 tensor cores with the keys on the 128-row side;
    head_dim 128, cache blocks of 64 tokens, at most 16 heads per kv head.  Chunks of 128 keys:
    max_splits >= ceil(longest length / 128); scratch and counters as attention_decode_tc_scratch
    says, the counters zeroed (the kernel leaves them zeroed)."""
    _need(out, "out", torch.bfloat16, 2); _need(q, "q", torch.bfloat16, 2)
    _need(k_plane, "k_plane", torch.bfloat16, 4); _need(v_plane, "v_plane", torch.bfloat16, 4)
    rows = out.shape[0]
    if out.shape[1] != nh * d or q.shape != out.shape or k_plane.shape[1] != nkv or k_plane.shape[3] != d \
            or v_plane.shape != k_plane.shape:
        raise KernelError(f"attention_decode_tc: shapes out {tuple(out.shape)} q {tuple(q.shape)} k {tuple(k_plane.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    _need(slot_ids, "slot_ids", torch.int32, 1); _need(kv_lens, "kv_lens", torch.int32, 1)
    need_acc, need_ml, need_counters = attention_decode_tc_scratch(rows, nh, nkv, d, max_splits)
    if part_acc.numel() < need_acc or part_ml.numel() < need_ml or counters.numel() < need_counters:
        raise KernelError("attention_decode_tc: the scratch for the partials is too small")
    _check(_lib().hymt2_attention_decode_tc(_ptr(out), _ptr(q), _ptr(k_plane), _ptr(v_plane), c_long(k_plane.shape[0]),
                                            _ptr(block_table), c_int(block_table.stride(0)), c_int(k_plane.shape[2]),
                                            _ptr(slot_ids), _ptr(kv_lens), c_int(rows), c_int(nh), c_int(nkv), c_int(d),
                                            c_float(scale), c_int(window), c_int(max_splits), _ptr(part_acc),
                                            _ptr(part_ml), _ptr(counters), _ptr(status), _stream()), "attention_decode_tc")


def attention_prefill_tc(out: torch.Tensor, q: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                         block_table: torch.Tensor, cu_seqlens: torch.Tensor, slot_ids: torch.Tensor,
                         kv_lens: torch.Tensor, batch: int, max_new_tokens: int, nh: int, nkv: int, d: int,
                         scale: float, window: int, status: torch.Tensor) -> None:
    """bfloat16 causal attention of the new tokens over the paged cache on the tcgen05 tensor cores
    (flash attention with S and O in tensor memory); head_dim 64 or 128, cache blocks of 64 tokens."""
    _need(out, "out", torch.bfloat16, 2); _need(q, "q", torch.bfloat16, 2)
    _need(k_plane, "k_plane", torch.bfloat16, 4); _need(v_plane, "v_plane", torch.bfloat16, 4)
    T = out.shape[0]
    if out.shape[1] != nh * d or q.shape != out.shape or k_plane.shape[1] != nkv or k_plane.shape[3] != d \
            or v_plane.shape != k_plane.shape:
        raise KernelError(f"attention_prefill_tc: shapes out {tuple(out.shape)} q {tuple(q.shape)} k {tuple(k_plane.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    _check(_lib().hymt2_attention_prefill_tc(_ptr(out), _ptr(q), _ptr(k_plane), _ptr(v_plane), c_long(k_plane.shape[0]),
                                             _ptr(block_table), c_int(block_table.stride(0)), c_int(k_plane.shape[2]),
                                             _ptr(cu_seqlens), _ptr(slot_ids), _ptr(kv_lens), c_int(batch), c_int(T),
                                             c_int(max_new_tokens), c_int(nh), c_int(nkv), c_int(d), c_float(scale),
                                             c_int(window), _ptr(status), _stream()), "attention_prefill_tc")


_counters: dict = {}


def zeroed_counters(device, n: int) -> torch.Tensor:
    """A per-device int32 array that is zero between kernels: arrival counters of kernels whose
    last-arriving block finishes the work (each such kernel leaves its counters at zero)."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    old = _counters.get(key)
    if old is None or old[-1].numel() < n:
        _counters[key] = (old or []) + [torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)]
    return _counters[key][-1]


def reset_counters(device) -> None:
    """Zeroes every arrival counter that kernels of this device share between launches (the split products'
    and the attention kernels'), on the current stream: after a kernel gave up in mid-count."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    for t in _counters.get(key) or []:
        t.zero_()
    ws, cnt, old = _tc_scratch.get(key, (None, None, []))
    for t in [cnt] + [o for o in old if o.dtype == torch.int32]:
        if t is not None:
            t.zero_()


def attention_decode(out: torch.Tensor, q: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                     block_table: torch.Tensor, cu_seqlens: torch.Tensor, slot_ids: torch.Tensor, kv_lens: torch.Tensor,
                     nh: int, nkv: int, d: int, scale: float, window: int, max_splits: int,
                     part_acc: torch.Tensor, part_ml: torch.Tensor, counters: torch.Tensor) -> None:
    """bfloat16 decode attention (one new token per row) that streams the cache once per kv head;
    head_dim 64 or 128.  The partials go through part_acc / part_ml (sizes as attention_simt_scratch);
    `counters` holds rows*nh zeroed ints (the kernel leaves them zero)."""
    _need(out, "out", torch.bfloat16, 2); _need(q, "q", torch.bfloat16, 2)
    _need(k_plane, "k_plane", torch.bfloat16, 4); _need(v_plane, "v_plane", torch.bfloat16, 4)
    rows = out.shape[0]
    if out.shape[1] != nh * d or q.shape[1] != nh * d or q.shape[0] < rows or k_plane.shape[1] != nkv \
            or k_plane.shape[3] != d or v_plane.shape != k_plane.shape:
        raise KernelError(f"attention_decode: shapes out {tuple(out.shape)} q {tuple(q.shape)} k {tuple(k_plane.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    need_acc, need_ml = attention_simt_scratch(rows, nh, d, max_splits)
    _need(part_acc, "part_acc", torch.float32); _need(part_ml, "part_ml", torch.float32)
    _need(counters, "counters", torch.int32, 1)
    if part_acc.numel() < need_acc or part_ml.numel() < need_ml or counters.numel() < rows * nh:
        raise KernelError("attention_decode: the scratch for the partials is too small")
    _check(_lib().hymt2_attention_decode(_ptr(out), _ptr(q), _ptr(k_plane), _ptr(v_plane), _ptr(block_table),
                                         c_int(block_table.stride(0)), c_int(k_plane.shape[2]), _ptr(cu_seqlens),
                                         _ptr(slot_ids), _ptr(kv_lens), c_int(rows), c_int(nh), c_int(nkv), c_int(d),
                                         c_float(scale), c_int(window), c_int(max_splits), _ptr(part_acc),
                                         _ptr(part_ml), _ptr(counters), _stream()), "attention_decode")


# ---------------------------------------------------------------------------
def _logits_ok(logits: torch.Tensor, what: str) -> None:
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError(f"{what}: logits must be a float32 CUDA matrix with contiguous rows")


ARGMAX_PIECE = 4096


def argmax(out: torch.Tensor, logits: torch.Tensor, row_map: torch.Tensor | None = None,
           scratch: tuple | None = None) -> None:
    """out[r] = first index of the maximum of logits[r]; rows with row_map[r] < 0 are skipped.
    `scratch` = (float32, int32) tensors of rows * ceil(vocab / 4096) entries lets a wide
    vocabulary be scanned by many blocks per row."""
    _need(out, "out", torch.int32, 1)
    _logits_ok(logits, "argmax")
    rows, vocab = logits.shape
    val = idx = None
    if scratch is not None:
        val, idx = scratch
        need = rows * (-(-vocab // ARGMAX_PIECE))
        _need(val, "scratch values", torch.float32); _need(idx, "scratch indices", torch.int32)
        if val.numel() < need or idx.numel() < need:
            raise KernelError("argmax: the scratch is too small")
    two_stage = scratch is not None and vocab > 2 * ARGMAX_PIECE
    _check(_lib().hymt2_argmax(_ptr(out), _ptr(logits), c_long(logits.stride(0)), c_int(rows), c_int(vocab),
                               _ptr(row_map), _ptr(val), _ptr(idx), _stream()), "argmax", 2 if two_stage else 1)


def seed_rng(states: torch.Tensor, rows: torch.Tensor, seeds: torch.Tensor) -> None:
    """states[rows[i]] = xoshiro256** state seeded with seeds[i] through SplitMix64."""
    _need(states, "states", torch.int64, 2); _need(rows, "rows", torch.int32, 1); _need(seeds, "seeds", torch.int64, 1)
    _check(_lib().hymt2_seed_rng(_ptr(states), _ptr(rows), _ptr(seeds), c_int(rows.shape[0]), _stream()), "seed_rng")


def sample(out: torch.Tensor, logits: torch.Tensor, inv_temperature: torch.Tensor, rng_states: torch.Tensor,
           row_map: torch.Tensor | None = None) -> None:
    """Temperature sampling of one token for every logits row whose sequence has a temperature
    above 0; advances that sequence's random stream by one draw.  row_map[r] is the row of the
    per-sequence arrays (inv_temperature, rng_states) that logits row r belongs to; < 0 skips."""
    _need(out, "out", torch.int32, 1); _need(inv_temperature, "inv_temperature", torch.float32, 1)
    _need(rng_states, "rng_states", torch.int64, 2)
    _logits_ok(logits, "sample")
    rows, vocab = logits.shape
    _check(_lib().hymt2_sample(_ptr(out), _ptr(logits), c_long(logits.stride(0)), c_int(rows), c_int(vocab),
                               _ptr(inv_temperature), _ptr(rng_states), _ptr(row_map), _stream()), "sample")


def filter_logits(logits: torch.Tensor, inv_temperature: torch.Tensor, top_k: torch.Tensor | None,
                  top_p: torch.Tensor | None, min_p: torch.Tensor | None, penalty: torch.Tensor | None,
                  history: torch.Tensor | None, row_map: torch.Tensor | None = None) -> None:
    """In place: repetition penalty, then (temperature > 0 only) top-k / min-p / top-p drops;
    dropped entries become -inf."""
    _logits_ok(logits, "filter")
    rows, vocab = logits.shape
    hs = 0
    if history is not None:
        _need(history, "history", torch.int32, 2)
        hs = history.shape[1]
    _check(_lib().hymt2_filter_logits(_ptr(logits), c_long(logits.stride(0)), c_int(rows), c_int(vocab),
                                      _ptr(inv_temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(penalty),
                                      _ptr(history), c_int(hs), _ptr(row_map), _stream()), "filter_logits")


def record_history(history: torch.Tensor, counts: torch.Tensor, tokens: torch.Tensor,
                   row_map: torch.Tensor | None, rows: int) -> None:
    """history[sequence, count % width] = tokens[r]; count += 1, for every logits row r."""
    _need(history, "history", torch.int32, 2); _need(counts, "counts", torch.int32, 1)
    _need(tokens, "tokens", torch.int32, 1)
    _check(_lib().hymt2_record_history(_ptr(history), _ptr(counts), c_int(history.shape[1]), _ptr(tokens),
                                       _ptr(row_map), c_int(rows), _stream()), "record_history")


# ---------------------------------------------------------------------------
# grouped norm, short convolution, recurrence, small element-wise steps, shared-vector attention
# ---------------------------------------------------------------------------
def _f32(t: torch.Tensor | None, name: str, n: int | None = None) -> None:
    if t is not None:
        _need(t, name, torch.float32)
        if n is not None and t.numel() != n:
            raise KernelError(f"{name} must hold {n} values, got {t.numel()}")


def rmsnorm_groups(out: torch.Tensor, x: torch.Tensor, gain: torch.Tensor, eps: float, groups: int,
                   rows_index: torch.Tensor | None = None, out_scale: float = 1.0, add: bool = False) -> None:
    """RMSNorm in `groups` equal consecutive parts of every row, each part with its own root mean square, the whole
    times gain, in float32.  `add`: out (float32) += the result instead of out = the result."""
    _need(out, "out", None, 2); _need(x, "x", None, 2); _need(gain, "gain", None, 1)
    rows, dim = out.shape
    if x.shape[1] != dim or gain.shape[0] != dim or groups <= 0 or dim % groups:
        raise KernelError(f"rmsnorm_groups: shapes out {tuple(out.shape)} x {tuple(x.shape)} gain {tuple(gain.shape)} groups {groups}")
    if rows_index is not None:
        _need(rows_index, "rows_index", torch.int32, 1)
        if rows_index.shape[0] < rows:
            raise KernelError("rmsnorm_groups: rows_index is shorter than out")
    elif x.shape[0] < rows:
        raise KernelError("rmsnorm_groups: x has fewer rows than out")
    if add and out.dtype != torch.float32:
        raise KernelError("rmsnorm_groups: adding needs float32 rows")
    _check(_lib().hymt2_rmsnorm_groups(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(x), c_int(dtype_code(x.dtype)), _ptr(gain),
                                       c_int(dtype_code(gain.dtype)), _ptr(rows_index), c_int(rows), c_int(dim), c_int(groups),
                                       c_float(eps), c_float(out_scale), c_int(1 if add else 0), _stream()), "rmsnorm_groups")


def _rows_view(t: torch.Tensor, name: str, dtype=None) -> int:
    """A matrix whose rows are contiguous (it may be a view of some columns of a wider one); returns its row stride."""
    if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be a CUDA matrix with contiguous rows")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    return t.stride(0)


def causal_conv(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, state: torch.Tensor,
                state_offset: int, cu_seqlens: torch.Tensor, slot_ids: torch.Tensor, kv_lens: torch.Tensor, batch: int,
                max_new_tokens: int, add_input: bool, silu: bool = False) -> None:
    """Causal convolution over time on each channel: out_t = act((x_t if add_input) + bias + sum_j w[:, j] x_(t - taps + 1 + j)),
    zeros before a sequence's start; act is SiLU if `silu`, else nothing.  `state` is the cache's byte matrix [slots, bytes]; from byte `state_offset` of a
    slot's row lie float32 [taps - 1, channels], the sequence's last inputs, which the kernel reads and renews."""
    ldx, ldo = _rows_view(x, "x"), _rows_view(out, "out", x.dtype)
    T, C = x.shape
    _f32(w, "w"); _f32(bias, "bias", C)
    if out.shape != x.shape or w.dim() != 2 or w.shape[0] != C:
        raise KernelError(f"causal_conv: shapes out {tuple(out.shape)} x {tuple(x.shape)} w {tuple(w.shape)}")
    taps = w.shape[1]
    if state.dtype != torch.uint8 or state.dim() != 2 or state_offset + 4 * (taps - 1) * C > state.shape[1]:
        raise KernelError("causal_conv: the state rows are too short for this convolution")
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    stride = state.stride(0)
    if taps == 1:      # a filter of one tap remembers nothing: the state rows are not touched, whatever their size and alignment
        stride, state_offset = 0, 0
    _check(_lib().hymt2_causal_conv(_ptr(out), _ptr(x), c_int(dtype_code(x.dtype)), _ptr(w), _ptr(bias), _ptr(state),
                                    c_long(state_offset), c_long(stride), _ptr(cu_seqlens), _ptr(slot_ids), _ptr(kv_lens),
                                    c_int(batch), c_int(max_new_tokens), c_int(C), c_int(taps), c_int(ldx), c_int(ldo),
                                    c_int((1 if add_input else 0) | (2 if silu else 0)), _stream()), "causal_conv")


def rglru_scan(out: torch.Tensor, gates: torch.Tensor, u: torch.Tensor, y: torch.Tensor, br: torch.Tensor, bi: torch.Tensor,
               lam: torch.Tensor, decay: float, state: torch.Tensor, state_offset: int, cu_seqlens: torch.Tensor,
               slot_ids: torch.Tensor, kv_lens: torch.Tensor, batch: int, max_new_tokens: int) -> None:
    """The real-gated linear recurrence over every sequence's new tokens, in float32: r = sigmoid(gates[:, :W] + br),
    i = sigmoid(gates[:, W:] + bi), a = exp(-decay * r * softplus(lam)), S <- a S + sqrt(1 - a^2) i u, out = S * y.
    S (float32 [W]) lies at byte `state_offset` of the sequence's state row.  Portions longer than two chunks of 64 tokens
    run in two passes over chunks (the recurrence composes), every chunk a thread of its own per channel."""
    T, W = u.shape
    ldu, ldy, ldo = _rows_view(u, "u"), _rows_view(y, "y", u.dtype), _rows_view(out, "out", u.dtype)
    _need(gates, "gates", torch.float32, 2)
    if gates.shape != (T, 2 * W) or y.shape != u.shape or out.shape != u.shape:
        raise KernelError(f"rglru_scan: shapes gates {tuple(gates.shape)} u {tuple(u.shape)} y {tuple(y.shape)} out {tuple(out.shape)}")
    _f32(br, "br", W); _f32(bi, "bi", W); _f32(lam, "lam", W)
    if state.dtype != torch.uint8 or state.dim() != 2 or state_offset + 4 * W > state.shape[1]:
        raise KernelError("rglru_scan: the state rows are too short")
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    lib = _lib()
    lib.hymt2_rglru_scan_scratch.restype = c_long
    floats = int(lib.hymt2_rglru_scan_scratch(c_int(batch), c_int(max_new_tokens), c_int(W)))
    scratch = torch.empty(floats, dtype=torch.float32, device=u.device) if floats else None
    _check(lib.hymt2_rglru_scan(_ptr(out), _ptr(gates), _ptr(u), _ptr(y), c_int(dtype_code(u.dtype)), _ptr(br), _ptr(bi), _ptr(lam),
                                c_float(decay), _ptr(state), c_long(state_offset), c_long(state.stride(0)), _ptr(cu_seqlens),
                                _ptr(slot_ids), _ptr(kv_lens), c_int(batch), c_int(W), c_int(ldu), c_int(ldy), c_int(ldo),
                                c_int(max_new_tokens), _ptr(scratch), c_long(floats), _stream()), "rglru_scan", 2 if floats else 1)


def bias_act(x: torch.Tensor, bias: torch.Tensor | None, act_cols: int) -> None:
    """In place: x += bias; the first `act_cols` columns then go through the tanh form of GELU."""
    ld = _rows_view(x, "x")
    _f32(bias, "bias", x.shape[1])
    _check(_lib().hymt2_bias_act(_ptr(x), c_int(dtype_code(x.dtype)), _ptr(bias), c_int(x.shape[0]), c_int(x.shape[1]), c_long(ld),
                                 c_int(act_cols), _stream()), "bias_act")


def xielu(out: torch.Tensor, x: torch.Tensor, pq: torch.Tensor) -> None:
    """out = xIELU(x) with pq = (p, q) float32 on the device: z > 0: softplus(p) z^2 + z/2; else (1/2 + softplus(q)) (e^z - 1 - z) + z/2."""
    _need(out, "out", x.dtype); _need(x, "x"); _f32(pq, "pq", 2)
    if out.shape != x.shape:
        raise KernelError("xielu: shapes differ")
    _check(_lib().hymt2_xielu(_ptr(out), _ptr(x), c_int(dtype_code(x.dtype)), _ptr(pq), c_long(x.numel()), _stream()), "xielu")


def sigmoid_gate(x: torch.Tensor, g: torch.Tensor, heads: int, vdim: int, per_head: bool) -> None:
    """In place on x [T, heads * vdim]: times sigmoid(g), where g has one column per head or one per entry."""
    _need(x, "x", None, 2)
    ldg = _rows_view(g, "g", x.dtype)
    if x.shape[1] != heads * vdim or g.shape != (x.shape[0], heads if per_head else heads * vdim):
        raise KernelError(f"sigmoid_gate: shapes x {tuple(x.shape)} g {tuple(g.shape)}")
    _check(_lib().hymt2_sigmoid_gate(_ptr(x), _ptr(g), c_int(dtype_code(x.dtype)), c_int(x.shape[0]), c_int(heads), c_int(vdim),
                                     c_long(ldg), c_int(1 if per_head else 0), _stream()), "sigmoid_gate")


def softcap(logits: torch.Tensor, cap: float) -> None:
    """In place: logits = cap * tanh(logits / cap)."""
    _need(logits, "logits", torch.float32)
    _check(_lib().hymt2_softcap(_ptr(logits), c_float(cap), c_long(logits.numel()), _stream()), "softcap")


def gemm_simt_batched(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, batch: int, a_step: int, out_step: int,
                      epilogue: int = EPILOGUE_STORE) -> None:
    """`batch` products in one launch: product z is out[:, z*out_step : z*out_step + N] = a[:, z*a_step : z*a_step + K] @ w[z]^T
    with w [batch, N, K]; a and out are matrices with contiguous rows (columns of wider buffers are fine)."""
    lda, ldc = _rows_view(a, "a"), _rows_view(out, "out")
    _need(w, "w", None, 3)
    if w.shape[0] != batch or a.shape[0] != out.shape[0]:
        raise KernelError(f"gemm_simt_batched: shapes out {tuple(out.shape)} a {tuple(a.shape)} w {tuple(w.shape)}")
    N, K = w.shape[1], w.shape[2]
    if (batch - 1) * a_step + K > a.shape[1] or (batch - 1) * out_step + N > out.shape[1]:
        raise KernelError("gemm_simt_batched: the steps run past a row")
    _check(_lib().hymt2_gemm_simt_batched(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(a), c_int(dtype_code(a.dtype)), _ptr(w),
                                          c_int(dtype_code(w.dtype)), c_int(out.shape[0]), c_int(N), c_int(K), c_long(lda), c_long(K),
                                          c_long(ldc), c_int(batch), c_long(a_step), c_long(N * K), c_long(out_step), c_int(epilogue),
                                          _stream()), "gemm_simt_batched")


def latent_prep(proj: torch.Tensor, q_cols: int, q_out: torch.Tensor | None, cache_plane: torch.Tensor | None, block_table: torch.Tensor,
                block_tokens: int, token_seq: torch.Tensor, token_pos: torch.Tensor, slot_ids: torch.Tensor, gain: torch.Tensor,
                inv_freq: torch.Tensor | None, rot_dims: int, amplitude: float, eps: float, heads: int, dim: int, rot: int,
                rank: int, rows_out: torch.Tensor | None = None) -> None:
    """From a token's fused projection [heads * (dim + rot) query entries | rank latent entries | rot shared key entries]:
    the normed latent vector and the rotated shared key part go to the token's cache row [rank + rot]; every head's
    rotated query part goes to q_out[t, h, rank : rank + rot].  Pairs (2i, 2i+1) turn by position * inv_freq[i], cosine
    and sine times `amplitude`.  cache_plane None: nothing is cached.  q_out None: the rotated query parts are written
    back into proj, in place.  rows_out [T, rank + rot]: the cache rows once more, side by side for all tokens.  With neither a
    cache plane nor rows_out the projection need not hold a compressed row at all (only the queries are read)."""
    ldp = _rows_view(proj, "proj")
    T = proj.shape[0]
    dl = rank + rot
    if q_out is not None:
        _need(q_out, "q_out", proj.dtype, 2)
    if rows_out is not None:
        _need(rows_out, "rows_out", proj.dtype, 2)
    # a run without a compressed row of its own (it reads another run's cache) brings the queries alone
    rowless = cache_plane is None and rows_out is None
    if proj.shape[1] < q_cols + (0 if rowless else dl) or q_cols != heads * (dim + rot) or (q_out is not None and q_out.shape != (T, heads * dl)) \
            or (rows_out is not None and rows_out.shape != (T, dl)):
        raise KernelError(f"latent_prep: shapes proj {tuple(proj.shape)} do not fit {heads} heads of {dim} + {rot} and a row of {dl}")
    if cache_plane is not None:
        _need(cache_plane, "cache_plane", proj.dtype, 4)
        if cache_plane.shape[1:] != (1, block_tokens, dl):
            raise KernelError(f"latent_prep: the cache plane is {tuple(cache_plane.shape)}, expected [blocks, 1, {block_tokens}, {dl}]")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((token_seq, "token_seq"), (token_pos, "token_pos"), (slot_ids, "slot_ids")):
        _need(t, n, torch.int32, 1)
    _f32(gain, "gain", rank); _f32(inv_freq, "inv_freq", rot_dims // 2)
    _check(_lib().hymt2_latent_prep(_ptr(proj), c_long(ldp), c_int(q_cols), _ptr(q_out), _ptr(rows_out), _ptr(cache_plane), c_int(dtype_code(proj.dtype)),
                                    _ptr(block_table), c_int(block_table.stride(0)), c_int(block_tokens), _ptr(token_seq),
                                    _ptr(token_pos), _ptr(slot_ids), _ptr(gain), _ptr(inv_freq), c_int(rot_dims), c_float(amplitude),
                                    c_float(eps), c_int(T), c_int(heads), c_int(dim), c_int(rot), c_int(rank), _stream()), "latent_prep")


def attention_shared_vector(out: torch.Tensor, q: torch.Tensor, cache_plane: torch.Tensor, block_table: torch.Tensor,
                            cu_seqlens: torch.Tensor, slot_ids: torch.Tensor, kv_lens: torch.Tensor, batch: int,
                            max_new_tokens: int, nh: int, d: int, dv: int, scale: float, window: int = 0, split_keys: int = 0,
                            max_splits: int = 0, part_acc: torch.Tensor | None = None, part_ml: torch.Tensor | None = None,
                            status: torch.Tensor | None = None) -> None:
    """Causal attention of the new tokens over a cache of ONE vector [d] per token that all heads share: it is every
    head's key, and its first dv entries are every head's value.  q [T, nh * d], out [T, nh * dv]; CUDA cores, float32
    scores and softmax.  Splits as attention_simt (the partials are [T, nh, splits, dv])."""
    if status is None:
        status = device_status(out.device)
    _need(out, "out", None, 2); _need(q, "q", out.dtype, 2); _need(cache_plane, "cache_plane", out.dtype, 4)
    T = out.shape[0]
    if out.shape[1] != nh * dv or q.shape[1] != nh * d or q.shape[0] < T or cache_plane.shape[1] != 1 or cache_plane.shape[3] != d:
        raise KernelError(f"attention_shared_vector: shapes out {tuple(out.shape)} q {tuple(q.shape)} cache {tuple(cache_plane.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    if split_keys > 0:
        _need(part_acc, "part_acc", torch.float32); _need(part_ml, "part_ml", torch.float32)
        if part_acc.numel() < T * nh * max_splits * dv or part_ml.numel() < T * nh * max_splits * 2:
            raise KernelError("attention_shared_vector: the split scratch is too small")
    _check(_lib().hymt2_attention_shared_vector(_ptr(out), _ptr(q), _ptr(cache_plane), c_int(dtype_code(out.dtype)), _ptr(block_table),
                                                c_int(block_table.stride(0)), c_int(cache_plane.shape[2]), _ptr(cu_seqlens),
                                                _ptr(slot_ids), _ptr(kv_lens), c_int(batch), c_int(T), c_int(max_new_tokens),
                                                c_int(nh), c_int(d), c_int(dv), c_float(scale), c_int(window), c_int(split_keys),
                                                c_int(max_splits), _ptr(part_acc), _ptr(part_ml), _stream(), _ptr(status)),
           "attention_shared_vector", 2 if split_keys > 0 else 1)


_mma_ok: dict = {}


def latent_attention_mma_supported(dtype: torch.dtype, d: int, dv: int, block_tokens: int) -> bool:
    """Whether the tensor-core kernel of the shared-vector attention takes these sizes (bfloat16, rows in pieces of 16)."""
    if dtype != torch.bfloat16:
        return False
    key = (d, dv, block_tokens)
    hit = _mma_ok.get(key)
    if hit is None:
        hit = _mma_ok[key] = bool(_lib().hymt2_latent_attention_mma_supported(c_int(d), c_int(dv), c_int(block_tokens)))
    return hit


def latent_attention_mma(out: torch.Tensor, q: torch.Tensor, cache_plane: torch.Tensor, block_table: torch.Tensor,
                         cu_seqlens: torch.Tensor, slot_ids: torch.Tensor, kv_lens: torch.Tensor, batch: int, max_new_tokens: int,
                         nh: int, d: int, dv: int, scale: float, window: int = 0, split_keys: int = 0, max_splits: int = 0,
                         part_acc: torch.Tensor | None = None, part_ml: torch.Tensor | None = None,
                         status: torch.Tensor | None = None) -> None:
    """attention_shared_vector in bfloat16 on the tensor cores (16x16x16 fragments, float32 sums and softmax): the same
    arguments and the same partials when split."""
    if status is None:
        status = device_status(out.device)
    _need(out, "out", torch.bfloat16, 2); _need(q, "q", torch.bfloat16, 2); _need(cache_plane, "cache_plane", torch.bfloat16, 4)
    T = out.shape[0]
    if out.shape[1] != nh * dv or q.shape != (T, nh * d) or cache_plane.shape[1] != 1 or cache_plane.shape[3] != d:
        raise KernelError(f"latent_attention_mma: shapes out {tuple(out.shape)} q {tuple(q.shape)} cache {tuple(cache_plane.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    if split_keys > 0:
        _need(part_acc, "part_acc", torch.float32); _need(part_ml, "part_ml", torch.float32)
        if part_acc.numel() < T * nh * max_splits * dv or part_ml.numel() < T * nh * max_splits * 2:
            raise KernelError("latent_attention_mma: the split scratch is too small")
    _check(_lib().hymt2_latent_attention_mma(_ptr(out), _ptr(q), _ptr(cache_plane), _ptr(block_table), c_int(block_table.stride(0)),
                                             c_int(cache_plane.shape[2]), _ptr(cu_seqlens), _ptr(slot_ids), _ptr(kv_lens), c_int(batch),
                                             c_int(T), c_int(max_new_tokens), c_int(nh), c_int(d), c_int(dv), c_float(scale),
                                             c_int(window), c_int(split_keys), c_int(max_splits), _ptr(part_acc), _ptr(part_ml),
                                             _ptr(status), _stream()), "latent_attention_mma", 2 if split_keys > 0 else 1)


SKINNY_MAX_ROWS = 16


def gemm_skinny_batched(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, a_step: int, out_step: int) -> None:
    """gemm_simt_batched for at most 16 rows (a decode step): one warp per output column, the weights read once.
    a and w have one type; out may be float32."""
    lda, ldc = _rows_view(a, "a"), _rows_view(out, "out")
    _need(w, "w", a.dtype, 3)
    batch, N, K = w.shape
    if a.shape[0] != out.shape[0] or a.shape[0] > SKINNY_MAX_ROWS or (batch - 1) * a_step + K > a.shape[1] or (batch - 1) * out_step + N > out.shape[1]:
        raise KernelError(f"gemm_skinny_batched: shapes out {tuple(out.shape)} a {tuple(a.shape)} w {tuple(w.shape)}")
    _check(_lib().hymt2_gemm_skinny_batched(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(a), _ptr(w), c_int(dtype_code(a.dtype)),
                                            c_int(a.shape[0]), c_int(N), c_int(K), c_long(lda), c_long(ldc), c_int(batch),
                                            c_long(a_step), c_long(N * K), c_long(out_step), _stream()), "gemm_skinny_batched")


def latent_attention_expanded_supported(dtype: torch.dtype, dim: int, rot: int, dv: int) -> bool:
    """Whether the per-head form of the tensor-core latent attention takes these head sizes."""
    if dtype != torch.bfloat16:
        return False
    key = ("expanded", dim, rot, dv)
    hit = _mma_ok.get(key)
    if hit is None:
        hit = _mma_ok[key] = bool(_lib().hymt2_latent_attention_expanded_supported(c_int(dim), c_int(rot), c_int(dv)))
    return hit


def latent_attention_expanded(out: torch.Tensor, q: torch.Tensor, kexp: torch.Tensor, vexp: torch.Tensor, krot: torch.Tensor,
                              cu_seqlens: torch.Tensor, slot_ids: torch.Tensor, kv_lens: torch.Tensor, batch: int,
                              max_new_tokens: int, nh: int, dim: int, rot: int, dv: int, scale: float, window: int = 0) -> None:
    """Causal attention of whole prompts that start at position 0, bfloat16 on the tensor cores, with keys and values per
    head: q [T, >= nh * (dim + rot)] (head h at column h * (dim + rot), its last rot entries rotated), kexp [T, nh * dim],
    vexp [T, nh * dv], krot [T, rot] the rotated key part of all heads; out [T, nh * dv].  All may be columns of wider
    matrices."""
    T = out.shape[0]
    for t, n in ((out, "out"), (q, "q"), (kexp, "kexp"), (vexp, "vexp"), (krot, "krot")):
        _rows_view(t, n, torch.bfloat16)
        if t.shape[0] != T:
            raise KernelError(f"latent_attention_expanded: {n} has {t.shape[0]} rows, expected {T}")
    if out.shape[1] != nh * dv or q.shape[1] < nh * (dim + rot) or kexp.shape[1] != nh * dim or vexp.shape[1] != nh * dv or krot.shape[1] != rot:
        raise KernelError("latent_attention_expanded: the matrices do not fit the head sizes")
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    _check(_lib().hymt2_latent_attention_expanded(_ptr(out), c_long(out.stride(0)), _ptr(q), c_long(q.stride(0)), _ptr(kexp),
                                                  c_long(kexp.stride(0)), _ptr(vexp), c_long(vexp.stride(0)), _ptr(krot),
                                                  c_long(krot.stride(0)), _ptr(cu_seqlens), _ptr(slot_ids), _ptr(kv_lens), c_int(batch),
                                                  c_int(max_new_tokens), c_int(nh), c_int(dim), c_int(rot), c_int(dv), c_float(scale),
                                                  c_int(window), _stream()), "latent_attention_expanded")



def rmsnorm_groups_add_norm(residual: torch.Tensor, x: torch.Tensor, gain_a: torch.Tensor, eps_a: float, out: torch.Tensor,
                            gain_b: torch.Tensor, eps_b: float, groups: int) -> None:
    """residual (float32) += norm_a(x); out = norm_b(residual), both norms in `groups` parts: the norm after one sublayer and the
    norm in front of the next in one kernel."""
    _need(residual, "residual", torch.float32, 2); _need(x, "x", torch.float32, 2); _need(out, "out", None, 2)
    _need(gain_a, "gain_a", None, 1); _need(gain_b, "gain_b", gain_a.dtype, 1)
    rows, dim = residual.shape
    if x.shape != residual.shape or out.shape != residual.shape or gain_a.shape[0] != dim or gain_b.shape[0] != dim or dim % groups:
        raise KernelError(f"rmsnorm_groups_add_norm: shapes residual {tuple(residual.shape)} x {tuple(x.shape)} out {tuple(out.shape)}")
    _check(_lib().hymt2_rmsnorm_groups_add_norm(_ptr(residual), _ptr(x), _ptr(gain_a), _ptr(out), c_int(dtype_code(out.dtype)), _ptr(gain_b),
                                                c_int(dtype_code(gain_a.dtype)), c_int(rows), c_int(dim), c_int(groups), c_float(eps_a),
                                                c_float(eps_b), _stream()), "rmsnorm_groups_add_norm")


# -- grouped-query attention in its general form: values of another width than keys, norms before the rotation, a sink ------
NORM_NONE, NORM_HEAD_AFTER, NORM_HEAD_BEFORE, NORM_ALL_BEFORE = 0, 1, 2, 3


def rope_kv_general(proj: torch.Tensor, q_out: torch.Tensor, k_plane: torch.Tensor | None, v_plane: torch.Tensor | None,
                    block_table: torch.Tensor, block_tokens: int, token_seq: torch.Tensor, token_pos: torch.Tensor,
                    slot_ids: torch.Tensor, inv_freq: torch.Tensor | None, rope_dim: int, q_gain: torch.Tensor | None,
                    k_gain: torch.Tensor | None, norm_mode: int, eps: float, nh: int, nkv: int, d: int, dv: int, has_kv: bool) -> None:
    """Norm, rotation and cache append for a projection proj[T, nh*d + nkv*(d + dv)] (queries, keys, values), or
    proj[T, nh*d] with `has_kv` False (queries only).  norm_mode: NORM_NONE; NORM_HEAD_AFTER (per head, after the rotation, gains
    of d entries); NORM_HEAD_BEFORE (per head, before it); NORM_ALL_BEFORE (over the token's whole q or k projection, before
    the rotation, gains as wide as the projection).  k_plane [blocks, nkv, block_tokens, d] and v_plane [.., dv], or None to
    append nothing."""
    _need(proj, "proj", None, 2); _need(q_out, "q_out", proj.dtype, 2)
    T = q_out.shape[0]
    cols = nh * d + (nkv * (d + dv) if has_kv else 0)
    if proj.shape[1] != cols or q_out.shape[1] != nh * d or proj.shape[0] < T:
        raise KernelError(f"rope_kv: shapes proj {tuple(proj.shape)} q_out {tuple(q_out.shape)} for nh={nh} nkv={nkv} d={d} dv={dv}")
    write = k_plane is not None and has_kv
    if write:
        for t, n, w in ((k_plane, "k_plane", d), (v_plane, "v_plane", dv)):
            _need(t, n, proj.dtype, 4)
            if t.shape[1:] != (nkv, block_tokens, w):
                raise KernelError(f"rope_kv: {n} is {tuple(t.shape)}, expected [blocks, {nkv}, {block_tokens}, {w}]")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((token_seq, "token_seq"), (token_pos, "token_pos"), (slot_ids, "slot_ids")):
        _need(t, n, torch.int32, 1)
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] != rope_dim // 2:
            raise KernelError("rope_kv: inv_freq must hold rope_dim/2 values")
    gain_dtype = F32
    if norm_mode != NORM_NONE:
        _need(q_gain, "q_gain", None, 1)
        gain_dtype = dtype_code(q_gain.dtype)
        wide = norm_mode == NORM_ALL_BEFORE
        if q_gain.shape[0] != (nh * d if wide else d):
            raise KernelError(f"rope_kv: the q gain holds {q_gain.shape[0]} entries")
        if has_kv:
            _need(k_gain, "k_gain", q_gain.dtype, 1)
            if k_gain.shape[0] != (nkv * d if wide else d):
                raise KernelError(f"rope_kv: the k gain holds {k_gain.shape[0]} entries")
    _check(_lib().hymt2_rope_kv_general(_ptr(proj), _ptr(q_out), _ptr(k_plane if write else None), _ptr(v_plane if write else None),
                                        c_int(dtype_code(proj.dtype)), _ptr(block_table), c_int(block_table.stride(0)),
                                        c_int(block_tokens), _ptr(token_seq), _ptr(token_pos), _ptr(slot_ids), _ptr(inv_freq),
                                        c_int(rope_dim), _ptr(q_gain), _ptr(k_gain if has_kv else None), c_int(gain_dtype), c_float(eps),
                                        c_int(T), c_int(nh), c_int(nkv), c_int(d), c_int(dv), c_int(norm_mode), c_int(1 if has_kv else 0),
                                        c_int(1 if write else 0), _stream()), "rope_kv")


def attention_simt_kv(out: torch.Tensor, q: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                      block_table: torch.Tensor, cu_seqlens: torch.Tensor, slot_ids: torch.Tensor, kv_lens: torch.Tensor, batch: int,
                      max_new_tokens: int, nh: int, nkv: int, d: int, dv: int, scale: float, window: int = 0, sink: bool = False,
                      split_keys: int = 0, max_splits: int = 0, part_acc: torch.Tensor | None = None,
                      part_ml: torch.Tensor | None = None, status: torch.Tensor | None = None) -> None:
    """attention_simt with keys of d and values of dv entries a head (out [T, nh * dv]), and optionally a sink: one more
    term in the softmax's denominator, of score 0 and without a value.  Scratch of a split run: attention_simt_scratch with dv."""
    if status is None:
        status = device_status(out.device)
    _need(out, "out", None, 2); _need(q, "q", out.dtype, 2)
    _need(k_plane, "k_plane", out.dtype, 4); _need(v_plane, "v_plane", out.dtype, 4)
    T = out.shape[0]
    block_tokens = k_plane.shape[2]
    if out.shape[1] != nh * dv or q.shape[1] != nh * d or q.shape[0] < T or k_plane.shape[1] != nkv or k_plane.shape[3] != d \
            or v_plane.shape != (*k_plane.shape[:3], dv):
        raise KernelError(f"attention: shapes out {tuple(out.shape)} q {tuple(q.shape)} k {tuple(k_plane.shape)} v {tuple(v_plane.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    if split_keys > 0:
        need_acc, need_ml = attention_simt_scratch(T, nh, dv, max_splits)
        _need(part_acc, "part_acc", torch.float32); _need(part_ml, "part_ml", torch.float32)
        if part_acc.numel() < need_acc or part_ml.numel() < need_ml:
            raise KernelError("attention: the split scratch is too small")
    _check(_lib().hymt2_attention_simt_kv(_ptr(out), _ptr(q), _ptr(k_plane), _ptr(v_plane), c_int(dtype_code(out.dtype)),
                                          _ptr(block_table), c_int(block_table.stride(0)), c_int(block_tokens), _ptr(cu_seqlens),
                                          _ptr(slot_ids), _ptr(kv_lens), c_int(batch), c_int(T), c_int(max_new_tokens), c_int(nh),
                                          c_int(nkv), c_int(d), c_int(dv), c_float(scale), c_int(window), c_int(1 if sink else 0),
                                          c_int(split_keys), c_int(max_splits), _ptr(part_acc), _ptr(part_ml), _stream(), _ptr(status)),
           "attention_simt", 2 if split_keys > 0 else 1)


# -- small steps ---------------------------------------------------------------------------------------------------------------
def relu_squared(out: torch.Tensor, x: torch.Tensor) -> None:
    """out = max(x, 0)^2."""
    _need(out, "out", x.dtype); _need(x, "x")
    if out.shape != x.shape:
        raise KernelError("relu_squared: shapes differ")
    _check(_lib().hymt2_relu_squared(_ptr(out), _ptr(x), c_int(dtype_code(x.dtype)), c_long(x.numel()), _stream()), "relu_squared")


def convert(out: torch.Tensor, x: torch.Tensor) -> None:
    """out = x rounded to out's type."""
    _need(out, "out"); _need(x, "x")
    if out.shape != x.shape:
        raise KernelError("convert: shapes differ")
    _check(_lib().hymt2_convert(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(x), c_int(dtype_code(x.dtype)), c_long(x.numel()), _stream()),
           "convert")


def rmsnorm_add_then_rows(residual: torch.Tensor, x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor, groups: int = 1) -> None:
    """residual (float32) += norm(x); out = the new rows rounded to out's type: the norm behind one sublayer, and the input of a
    next sublayer that reads the residual as it is."""
    _need(residual, "residual", torch.float32, 2); _need(x, "x", torch.float32, 2); _need(out, "out", None, 2); _need(gain, "gain", None, 1)
    rows, dim = residual.shape
    if x.shape != residual.shape or out.shape != residual.shape or gain.shape[0] != dim or dim % groups:
        raise KernelError(f"rmsnorm_add_then_rows: shapes residual {tuple(residual.shape)} x {tuple(x.shape)} out {tuple(out.shape)}")
    _check(_lib().hymt2_rmsnorm_groups_add_norm(_ptr(residual), _ptr(x), _ptr(gain), _ptr(out), c_int(dtype_code(out.dtype)), _ptr(None),
                                                c_int(dtype_code(gain.dtype)), c_int(rows), c_int(dim), c_int(groups), c_float(eps),
                                                c_float(eps), _stream()), "rmsnorm_groups_add_norm")


# -- a mixture of experts ---------------------------------------------------------------------------------------------------------
EPILOGUE_RELU_SQUARED = 3
_group_tiles: dict = {}


def moe_route(chosen: torch.Tensor, weight: torch.Tensor, logits: torch.Tensor, correction: torch.Tensor | None,
              bias: torch.Tensor | None = None, renormalise: bool = False) -> None:
    """From router outputs logits [T, R] (float32), plus `bias` [R] where one is given: scores = softmax over all R; chosen [T, top]
    (int32) = the `top` largest of score + correction, best first, ties to the lower index; weight [T, top] (float32) = their
    scores, as they are, or (`renormalise`) divided by their sum: the softmax over the chosen outputs alone."""
    _need(logits, "logits", torch.float32, 2); _need(chosen, "chosen", torch.int32, 2); _need(weight, "weight", torch.float32, 2)
    T, R = logits.shape
    top = chosen.shape[1]
    if chosen.shape[0] != T or weight.shape != chosen.shape or not (0 < top <= R):
        raise KernelError(f"moe_route: shapes logits {tuple(logits.shape)} chosen {tuple(chosen.shape)} weight {tuple(weight.shape)}")
    _f32(correction, "correction", R); _f32(bias, "bias", R)
    _check(_lib().hymt2_moe_route(_ptr(chosen), _ptr(weight), _ptr(logits), _ptr(correction), _ptr(bias), c_int(1 if renormalise else 0),
                                  c_int(T), c_int(R), c_int(top), _stream()), "moe_route")


def moe_tiles(tokens: int, top: int, experts: int, tile: int) -> int:
    """Row tiles that the sorted list of a step can need at most: every expert's segment is padded to whole tiles."""
    return -(-(tokens * top + experts * (tile - 1)) // tile) if experts else 1


def moe_place(pair_row: torch.Tensor, row_token: torch.Tensor, tile_group: torch.Tensor, counts: torch.Tensor, chosen: torch.Tensor,
              experts: int, tile: int) -> None:
    """Sorts the (token, choice) pairs of chosen [T, top] by expert, tokens in order inside an expert, each expert's rows padded
    to whole tiles: pair_row [T, top] = a pair's row in the sorted list (-1: it names an identity expert, index >= experts),
    row_token [tiles * tile] = the token of a sorted row (-1: padding), tile_group [tiles + 1] = the expert of a row tile (-1: not
    in use; the tiles in use come first) and, in its last entry, the number of tiles in use.  counts [max(experts, 1)] is scratch."""
    for t, n in ((pair_row, "pair_row"), (row_token, "row_token"), (tile_group, "tile_group"), (counts, "counts"), (chosen, "chosen")):
        _need(t, n, torch.int32)
    T, top = chosen.shape
    tiles = tile_group.numel() - 1
    if pair_row.shape != chosen.shape or row_token.numel() < tiles * tile or tiles < moe_tiles(T, top, experts, tile) \
            or counts.numel() < max(experts, 1):
        raise KernelError("moe_place: a buffer is too small")
    _check(_lib().hymt2_moe_place(_ptr(pair_row), _ptr(row_token), _ptr(tile_group), _ptr(counts), _ptr(chosen), c_int(T), c_int(top),
                                  c_int(experts), c_int(tile), c_int(tiles), _stream()), "moe_place", 2)


GROUPED_KERNELS = ("simt", "skinny", "tc")


def gemm_group_tile(kernel: str = "simt") -> int:
    """Rows of a row tile of a grouped product (an expert's segment of sorted rows is padded to whole tiles): 64 for the
    CUDA-core kernel, 8 for the one for few rows, 128 for the tensor-core kernel."""
    if kernel not in _group_tiles:
        _group_tiles[kernel] = 128 if kernel == "tc" else int(getattr(_lib(), f"hymt2_gemm_{kernel}_group_tile")())
    return _group_tiles[kernel]


def gemm_grouped(kernel: str, out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, row_token: torch.Tensor,
                 gather: bool, epilogue: int = EPILOGUE_STORE) -> None:
    """out[r] = epilogue(a[source(r)] @ w[tile_group[r // tile]]^T) for the sorted rows r of moe_place: w [experts, N, K];
    source(r) = row_token[r] with `gather` (a holds one row per token), r itself otherwise (a holds sorted rows); padding
    rows and unused tiles are skipped ("tc": computed and never read).  Epilogues: EPILOGUE_STORE, EPILOGUE_RELU_SQUARED.
    kernel "simt": CUDA cores, any sizes and types; "skinny": CUDA cores, tiles of 8 rows, a and w of one type, the time of
    reading the weights once; "tc": tcgen05, bfloat16, no gather (see moe_gather), K and N multiples of 8."""
    _need(out, "out", None, 2); _need(a, "a", None, 2); _need(w, "w", None, 3)
    _need(tile_group, "tile_group", torch.int32, 1); _need(row_token, "row_token", torch.int32, 1)
    tiles, tile = tile_group.numel() - 1, gemm_group_tile(kernel)
    N, K = w.shape[1], w.shape[2]
    if out.shape != (tiles * tile, N) or a.shape[1] != K or row_token.numel() < tiles * tile or (not gather and a.shape[0] < tiles * tile):
        raise KernelError(f"gemm_grouped: shapes out {tuple(out.shape)} a {tuple(a.shape)} w {tuple(w.shape)} tiles {tiles} of {tile}")
    if kernel == "simt":
        _check(_lib().hymt2_gemm_simt_grouped(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(a), c_int(dtype_code(a.dtype)), _ptr(w),
                                              c_int(dtype_code(w.dtype)), _ptr(tile_group), _ptr(row_token), c_int(1 if gather else 0),
                                              c_int(tiles), c_int(N), c_int(K), c_long(a.stride(0)), c_long(out.stride(0)), c_long(N * K),
                                              c_int(epilogue), _stream()), "gemm_simt_grouped")
    elif kernel == "skinny":
        if a.dtype != w.dtype:
            raise KernelError("gemm_grouped: the kernel for few rows wants a and w of one type")
        _check(_lib().hymt2_gemm_skinny_grouped(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(a), _ptr(w), c_int(dtype_code(w.dtype)),
                                                _ptr(tile_group), _ptr(row_token), c_int(1 if gather else 0), c_int(tiles), c_int(N), c_int(K),
                                                c_long(a.stride(0)), c_long(out.stride(0)), c_long(N * K), c_int(epilogue), _stream()),
               "gemm_skinny_grouped")
    else:
        if gather or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            raise KernelError("gemm_grouped: the tensor-core kernel wants sorted bfloat16 rows")
        _check(_lib().hymt2_gemm_tc_grouped(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(a), _ptr(w), _ptr(tile_group), c_int(tiles),
                                            c_int(w.shape[0]), c_int(N), c_int(K), c_long(a.stride(0)), c_long(out.stride(0)),
                                            c_int(1 if epilogue == EPILOGUE_RELU_SQUARED else 0), _ptr(device_status(out.device)), _stream()),
               "gemm_tc_grouped")


def gemm_simt_grouped(out, a, w, tile_group, row_token, gather: bool, epilogue: int = EPILOGUE_STORE) -> None:
    gemm_grouped("simt", out, a, w, tile_group, row_token, gather, epilogue)


def moe_gather(xs: torch.Tensor, x: torch.Tensor, row_token: torch.Tensor) -> None:
    """xs[r] = x[row_token[r]] (zeros where row_token[r] < 0): the sorted rows side by side, for a product that cannot gather."""
    _need(xs, "xs", x.dtype, 2); _need(x, "x", None, 2); _need(row_token, "row_token", torch.int32, 1)
    if xs.shape[1] != x.shape[1] or row_token.numel() < xs.shape[0]:
        raise KernelError(f"moe_gather: shapes xs {tuple(xs.shape)} x {tuple(x.shape)} rows {row_token.numel()}")
    _check(_lib().hymt2_moe_gather(_ptr(xs), _ptr(x), c_int(dtype_code(x.dtype)), _ptr(row_token), c_int(xs.shape[0]), c_int(x.shape[1]),
                                   _stream()), "moe_gather")


def moe_combine(out: torch.Tensor, y: torch.Tensor, x: torch.Tensor, pair_row: torch.Tensor, weight: torch.Tensor, add: bool = False) -> None:
    """out[t] (float32) = (out[t] if `add`) + sum_k weight[t, k] * (y[pair_row[t, k]] if pair_row[t, k] >= 0 else x[t]), k in order."""
    _need(out, "out", torch.float32, 2); _need(y, "y", torch.float32, 2); _need(x, "x", None, 2)
    _need(pair_row, "pair_row", torch.int32, 2); _need(weight, "weight", torch.float32, 2)
    T, H = out.shape
    if x.shape != out.shape or y.shape[1] != H or pair_row.shape[0] != T or weight.shape != pair_row.shape:
        raise KernelError(f"moe_combine: shapes out {tuple(out.shape)} y {tuple(y.shape)} x {tuple(x.shape)} pairs {tuple(pair_row.shape)}")
    _check(_lib().hymt2_moe_combine(_ptr(out), _ptr(y), _ptr(x), c_int(dtype_code(x.dtype)), _ptr(pair_row), _ptr(weight), c_int(T), c_int(H),
                                    c_int(pair_row.shape[1]), c_int(1 if add else 0), _stream()), "moe_combine")


def _attention_kv_shapes(what: str, out, q, k_plane, v_plane, nh, nkv, d, dv) -> None:
    _need(out, "out", torch.bfloat16, 2); _need(q, "q", torch.bfloat16, 2)
    _need(k_plane, "k_plane", torch.bfloat16, 4); _need(v_plane, "v_plane", torch.bfloat16, 4)
    if out.shape[1] != nh * dv or q.shape[1] != nh * d or q.shape[0] < out.shape[0] or k_plane.shape[1] != nkv or k_plane.shape[3] != d \
            or v_plane.shape != (*k_plane.shape[:3], dv):
        raise KernelError(f"{what}: shapes out {tuple(out.shape)} q {tuple(q.shape)} k {tuple(k_plane.shape)} v {tuple(v_plane.shape)}")


def attention_prefill_tc_kv(out: torch.Tensor, q: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor, block_table: torch.Tensor,
                            cu_seqlens: torch.Tensor, slot_ids: torch.Tensor, kv_lens: torch.Tensor, batch: int, max_new_tokens: int,
                            nh: int, nkv: int, d: int, dv: int, scale: float, window: int, sink: bool, status: torch.Tensor) -> None:
    """attention_prefill_tc with keys of d and values of dv entries a head (64 or 128 each; out [T, nh * dv]) and optionally a
    sink in the softmax."""
    _attention_kv_shapes("attention_prefill_tc", out, q, k_plane, v_plane, nh, nkv, d, dv)
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    _check(_lib().hymt2_attention_prefill_tc_kv(_ptr(out), _ptr(q), _ptr(k_plane), _ptr(v_plane), c_long(k_plane.shape[0]),
                                                _ptr(block_table), c_int(block_table.stride(0)), c_int(k_plane.shape[2]),
                                                _ptr(cu_seqlens), _ptr(slot_ids), _ptr(kv_lens), c_int(batch), c_int(out.shape[0]),
                                                c_int(max_new_tokens), c_int(nh), c_int(nkv), c_int(d), c_int(dv), c_float(scale),
                                                c_int(window), c_int(1 if sink else 0), _ptr(status), _stream()), "attention_prefill_tc")


def attention_decode_kv(out: torch.Tensor, q: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor, block_table: torch.Tensor,
                        cu_seqlens: torch.Tensor, slot_ids: torch.Tensor, kv_lens: torch.Tensor, nh: int, nkv: int, d: int, dv: int,
                        scale: float, window: int, sink: bool, max_splits: int, part_acc: torch.Tensor, part_ml: torch.Tensor,
                        counters: torch.Tensor) -> None:
    """attention_decode with keys of d and values of dv entries a head (64 or 128 each) and optionally a sink; the scratch is
    sized as attention_simt_scratch with dv."""
    _attention_kv_shapes("attention_decode", out, q, k_plane, v_plane, nh, nkv, d, dv)
    rows = out.shape[0]
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    need_acc, need_ml = attention_simt_scratch(rows, nh, dv, max_splits)
    _need(part_acc, "part_acc", torch.float32); _need(part_ml, "part_ml", torch.float32); _need(counters, "counters", torch.int32, 1)
    if part_acc.numel() < need_acc or part_ml.numel() < need_ml or counters.numel() < rows * nh:
        raise KernelError("attention_decode: the scratch for the partials is too small")
    _check(_lib().hymt2_attention_decode_kv(_ptr(out), _ptr(q), _ptr(k_plane), _ptr(v_plane), _ptr(block_table),
                                            c_int(block_table.stride(0)), c_int(k_plane.shape[2]), _ptr(cu_seqlens), _ptr(slot_ids),
                                            _ptr(kv_lens), c_int(rows), c_int(nh), c_int(nkv), c_int(d), c_int(dv), c_float(scale),
                                            c_int(window), c_int(1 if sink else 0), c_int(max_splits), _ptr(part_acc), _ptr(part_ml),
                                            _ptr(counters), _stream()), "attention_decode")


MOE_SMALL_PAIRS = 64   # up to this many (token, choice) pairs one block routes and sorts a step


def moe_route_place(chosen: torch.Tensor, weight: torch.Tensor, pair_row: torch.Tensor, row_token: torch.Tensor, tile_group: torch.Tensor,
                    logits: torch.Tensor, correction: torch.Tensor | None, experts: int, tile: int, bias: torch.Tensor | None = None,
                    renormalise: bool = False) -> None:
    """moe_route and moe_place in one launch, for a step of at most MOE_SMALL_PAIRS (token, choice) pairs."""
    _need(logits, "logits", torch.float32, 2); _need(chosen, "chosen", torch.int32, 2); _need(weight, "weight", torch.float32, 2)
    for t, n in ((pair_row, "pair_row"), (row_token, "row_token"), (tile_group, "tile_group")):
        _need(t, n, torch.int32)
    T, R = logits.shape
    top, tiles = chosen.shape[1], tile_group.numel() - 1
    if chosen.shape[0] != T or weight.shape != chosen.shape or pair_row.shape != chosen.shape or not (0 < top <= R) or T * top > MOE_SMALL_PAIRS \
            or row_token.numel() < tiles * tile or tiles < moe_tiles(T, top, experts, tile):
        raise KernelError("moe_route_place: shapes do not fit, or a buffer is too small")
    _f32(correction, "correction", R); _f32(bias, "bias", R)
    _check(_lib().hymt2_moe_route_place_small(_ptr(chosen), _ptr(weight), _ptr(pair_row), _ptr(row_token), _ptr(tile_group), _ptr(logits),
                                              _ptr(correction), _ptr(bias), c_int(1 if renormalise else 0), c_int(T), c_int(R), c_int(top),
                                              c_int(experts), c_int(tile), c_int(tiles), _stream()), "moe_route_place")


MOE_COMBINE_NORM_MAX_WIDTH = 12000   # a row of the fused combine-and-norm kernel lies in shared memory


def moe_combine_norm(residual: torch.Tensor, rows: torch.Tensor | None, branch: torch.Tensor | None, y: torch.Tensor, x: torch.Tensor,
                     pair_row: torch.Tensor, weight: torch.Tensor, gain: torch.Tensor, eps: float) -> None:
    """v[t] = (branch[t] if given) + sum_k weight[t, k] * (y[pair_row[t, k]] if pair_row[t, k] >= 0 else x[t]); residual[t] (float32)
    += v[t] / sqrt(mean(v[t]^2) + eps) * gain; rows[t] (if given) = the new residual row in rows' type."""
    _need(residual, "residual", torch.float32, 2); _need(y, "y", torch.float32, 2); _need(x, "x", None, 2)
    _need(pair_row, "pair_row", torch.int32, 2); _need(weight, "weight", torch.float32, 2); _need(gain, "gain", None, 1)
    T, H = residual.shape
    if x.shape != residual.shape or y.shape[1] != H or pair_row.shape[0] != T or weight.shape != pair_row.shape or gain.shape[0] != H \
            or H > MOE_COMBINE_NORM_MAX_WIDTH:
        raise KernelError(f"moe_combine_norm: shapes residual {tuple(residual.shape)} y {tuple(y.shape)} x {tuple(x.shape)}")
    if branch is not None:
        _need(branch, "branch", torch.float32, 2)
        if branch.shape != residual.shape:
            raise KernelError("moe_combine_norm: branch and residual differ in shape")
    if rows is not None:
        _need(rows, "rows", None, 2)
        if rows.shape != residual.shape:
            raise KernelError("moe_combine_norm: rows and residual differ in shape")
    _check(_lib().hymt2_moe_combine_norm(_ptr(residual), _ptr(rows), c_int(dtype_code(rows.dtype) if rows is not None else F32), _ptr(branch),
                                         _ptr(y), _ptr(x), c_int(dtype_code(x.dtype)), _ptr(pair_row), _ptr(weight), _ptr(gain),
                                         c_int(dtype_code(gain.dtype)), c_int(T), c_int(H), c_int(pair_row.shape[1]), c_float(eps), _stream()),
           "moe_combine_norm")


# -- a residual kept as several streams --------------------------------------------------------------------------------------------
MAX_STREAMS, MAX_BRANCHES = 8, 4


def streams_fill(X: torch.Tensor) -> None:
    """X float32 [streams, T, width]: every stream becomes a copy of stream 0."""
    _need(X, "X", torch.float32, 3)
    _check(_lib().hymt2_streams_fill(_ptr(X), c_int(X.shape[0]), c_int(X.shape[1]), c_int(X.shape[2]), _stream()), "streams_fill",
           1 if X.shape[0] > 1 else 0)


def streams_step(X: torch.Tensor, write: tuple | None = None, read: tuple | None = None) -> torch.Tensor | None:
    """One pass over the streams X float32 [streams, T, width], a block per token.
    write = (mix [streams, streams] indexed [from, to], w_out [streams], branches [float32 [T, width], ...], scales [float, ...]):
        y = sum_b scales[b] * branches[b];  X'[r] = sum_s mix[s, r] X[s] + w_out[r] * y, every stream from the old ones.
    read = (w_in [streams], gain [width] or None, eps, out): u = sum_s w_in[s] X[s] of the streams as the write left them;
        out = u / sqrt(mean(u^2) + eps) * gain, or u itself (float32) without a gain.  Returns out."""
    _need(X, "X", torch.float32, 3)
    S, T, W = X.shape
    mix = w_out = w_in = gain = out = None
    eps, branches, scales = 0.0, [], []
    if write is not None:
        mix, w_out, branches, scales = write
        _f32(mix, "mix", S * S); _f32(w_out, "w_out", S)
        if not (0 < len(branches) <= MAX_BRANCHES) or len(scales) != len(branches):
            raise KernelError(f"streams_step: {len(branches)} branches (1 to {MAX_BRANCHES})")
        for b in branches:
            _need(b, "branch", torch.float32, 2)
            if b.shape != (T, W):
                raise KernelError(f"streams_step: a branch is {tuple(b.shape)}, the streams hold rows of {(T, W)}")
    if read is not None:
        w_in, gain, eps, out = read
        _f32(w_in, "w_in", S); _need(out, "out", None, 2)
        if out.shape != (T, W) or (gain is None and out.dtype != torch.float32):
            raise KernelError(f"streams_step: out is {tuple(out.shape)} {out.dtype}")
        if gain is not None:
            _need(gain, "gain", None, 1)
            if gain.shape[0] != W:
                raise KernelError("streams_step: the gain's width differs")
    if S > MAX_STREAMS or (write is None and read is None):
        raise KernelError(f"streams_step: {S} streams (at most {MAX_STREAMS}), and something to do")
    ptrs = (c_void_p * max(1, len(branches)))(*[b.data_ptr() for b in branches])
    sc = (c_float * max(1, len(scales)))(*[float(v) for v in scales])
    _check(_lib().hymt2_streams_step(_ptr(X), c_int(S), c_int(T), c_int(W), _ptr(mix), _ptr(w_out), ptrs, sc, c_int(len(branches)),
                                     _ptr(w_in), _ptr(gain), c_int(dtype_code(gain.dtype) if gain is not None else F32), c_float(eps),
                                     _ptr(out), c_int(dtype_code(out.dtype) if out is not None else F32), _stream()), "streams_step")
    return out


# -- mixers with a matrix of state per head ------------------------------------------------------------------------------------------
SCAN_FIXED_DECAY, SCAN_TOKEN_DECAY = 0, 1


def linear_scan_chunking() -> tuple[int, int]:
    """(tokens of a chunk, the longest portion's length from which a step runs in three passes over chunks)."""
    return int(_lib().hymt2_linear_scan_chunk()), int(_lib().hymt2_linear_scan_min_chunked())


def linear_scan(out: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mode: int, state: torch.Tensor, state_offset: int,
                cu_seqlens: torch.Tensor, slot_ids: torch.Tensor, kv_lens: torch.Tensor, batch: int, heads: int, dk: int, dv: int,
                decay: torch.Tensor | None = None, k_scale: float = 1.0, x: torch.Tensor | None = None, w0: torch.Tensor | None = None,
                u: torch.Tensor | None = None, chunks: tuple | None = None) -> None:
    """The recurrence over a matrix of state S [dk, dv] float32 per (sequence, head), which lies at byte `state_offset` of the
    sequence's state row as [heads, dk, dv] and is ignored by a sequence that starts at position 0.
    SCAN_FIXED_DECAY: S = decay[h] S + (k_scale k_t) v_t^T; out_t = S^T q_t.
    SCAN_TOKEN_DECAY: out_t = (S + diag(u[h]) k_t v_t^T)^T q_t; S = diag(w_t) S + k_t v_t^T with w_t = exp(-exp(x_t + w0)).
    q, k [T, heads * dk] and v [T, heads * dv] in the compute type (rows may be columns of wider matrices); x [T, heads * dk] float32;
    out [T, heads * dv] float32.  `chunks` = (count, chunk_seq, chunk_first, chunk_len, seq_chunk0) int32 on the device: the
    three-pass form over those chunks; None: one serial walk per sequence."""
    _need(out, "out", torch.float32, 2)
    T = out.shape[0]
    ldq, ldk, ldv = _rows_view(q, "q"), _rows_view(k, "k", q.dtype), _rows_view(v, "v", q.dtype)
    if q.shape != (T, heads * dk) or k.shape != q.shape or v.shape != (T, heads * dv) or out.shape[1] != heads * dv:
        raise KernelError(f"linear_scan: shapes q {tuple(q.shape)} k {tuple(k.shape)} v {tuple(v.shape)} out {tuple(out.shape)}")
    ldx = 0
    if mode == SCAN_FIXED_DECAY:
        _f32(decay, "decay", heads)
    else:
        ldx = _rows_view(x, "x", torch.float32)
        _f32(w0, "w0", heads * dk); _f32(u, "u", heads * dk)
        if x.shape != (T, heads * dk):
            raise KernelError(f"linear_scan: x is {tuple(x.shape)}")
    if state.dtype != torch.uint8 or state.dim() != 2 or state_offset % 4 or state_offset + 4 * heads * dk * dv > state.shape[1]:
        raise KernelError("linear_scan: the state rows are too short")
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    count, B, A, cs, cf, cl, sc0, launches_ = 0, None, None, None, None, None, None, 1
    if chunks is not None:
        count, cs, cf, cl, sc0 = chunks
        B = torch.empty(count * heads * dk * dv, dtype=torch.float32, device=out.device)
        A = torch.empty(count * heads * dk, dtype=torch.float32, device=out.device) if mode == SCAN_TOKEN_DECAY else None
        launches_ = 3
    _check(_lib().hymt2_linear_scan(_ptr(out), _ptr(q), _ptr(k), _ptr(v), c_int(dtype_code(q.dtype)), c_long(ldq), c_long(ldk), c_long(ldv),
                                    _ptr(x), c_long(ldx), _ptr(w0), _ptr(u), _ptr(decay), c_float(k_scale), c_int(mode), _ptr(state),
                                    c_long(state_offset), c_long(state.stride(0)), _ptr(cu_seqlens), _ptr(slot_ids), _ptr(kv_lens),
                                    c_int(batch), c_int(heads), c_int(dk), c_int(dv), c_int(count), _ptr(B), _ptr(A), _ptr(cs), _ptr(cf),
                                    _ptr(cl), _ptr(sc0), _stream()), "linear_scan", launches_)


def head_norm_gate(out: torch.Tensor, o: torch.Tensor, gate: torch.Tensor | None, weight: torch.Tensor | None, heads: int, dv: int,
                   eps: float, gate_act: str = "silu") -> None:
    """out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight[h, :] * act(gate[t, h, :]); act is SiLU or, with
    gate_act "sigmoid", the sigmoid; weight and gate are optional,
    o is float32, gate (rows may be columns of a wider matrix) and out have the compute type."""
    _need(out, "out", None, 2); _need(o, "o", torch.float32, 2)
    T = out.shape[0]
    ldg = 0
    if gate is not None:
        ldg = _rows_view(gate, "gate", out.dtype)
        if gate.shape != out.shape:
            raise KernelError("head_norm_gate: the gate's shape differs")
    _f32(weight, "weight", heads * dv)
    if out.shape != (T, heads * dv) or o.shape != out.shape:
        raise KernelError(f"head_norm_gate: shapes out {tuple(out.shape)} o {tuple(o.shape)}")
    _check(_lib().hymt2_head_norm_gate(_ptr(out), _ptr(o), _ptr(gate), c_long(ldg), c_int(dtype_code(out.dtype)), _ptr(weight), c_int(T),
                                       c_int(heads), c_int(dv), c_float(eps), c_int(1 if gate_act == "sigmoid" else 0), _stream()), "head_norm_gate")


def token_shift(mixes: torch.Tensor, h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, state_offset: int, token_seq: torch.Tensor,
                cu_seqlens: torch.Tensor, slot_ids: torch.Tensor, kv_lens: torch.Tensor) -> None:
    """mixes[t, s * W : (s + 1) * W] = h[t] + (h[t - 1] - h[t]) * mu[s] for every row s of mu [count, W] (float32).  The row before
    a sequence's first new token is the float32 [W] at byte `state_offset` of its state row (zeros at position 0), which
    receives the step's last row."""
    ldh = _rows_view(h, "h")
    _need(mixes, "mixes", h.dtype, 2); _need(mu, "mu", torch.float32, 2)
    T, W = h.shape
    count = mu.shape[0]
    if mixes.shape != (T, count * W) or mu.shape[1] != W:
        raise KernelError(f"token_shift: shapes mixes {tuple(mixes.shape)} h {tuple(h.shape)} mu {tuple(mu.shape)}")
    if state.dtype != torch.uint8 or state.dim() != 2 or state_offset % 4 or state_offset + 4 * W > state.shape[1]:
        raise KernelError("token_shift: the state rows are too short")
    for t, n in ((token_seq, "token_seq"), (cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    _check(_lib().hymt2_token_shift(_ptr(mixes), _ptr(h), c_long(ldh), c_int(dtype_code(h.dtype)), _ptr(mu), c_int(count), _ptr(state),
                                    c_long(state_offset), c_long(state.stride(0)), _ptr(token_seq), _ptr(cu_seqlens), _ptr(slot_ids),
                                    _ptr(kv_lens), c_int(T), c_int(W), _stream()), "token_shift")


GATED_SILU, GATED_GELU_TANH = 0, 1


def gated_act(out: torch.Tensor, gate_up: torch.Tensor, kind: int) -> None:
    """out[r, c] = act(gate_up[r, c]) * gate_up[r, width + c]; act: GATED_SILU or GATED_GELU_TANH."""
    _need(out, "out", None, 2); _need(gate_up, "gate_up", out.dtype, 2)
    rows, width = out.shape
    if gate_up.shape != (rows, 2 * width):
        raise KernelError(f"gated_act: shapes out {tuple(out.shape)} gate_up {tuple(gate_up.shape)}")
    _check(_lib().hymt2_gated_act(_ptr(out), _ptr(gate_up), c_int(dtype_code(out.dtype)), c_int(rows), c_int(width), c_int(kind),
                                  _stream()), "gated_act")


def tanh_(x: torch.Tensor) -> None:
    """In place on float32 values."""
    _need(x, "x", torch.float32)
    _check(_lib().hymt2_tanh(_ptr(x), c_long(x.numel()), _stream()), "tanh")


# -- layer norm, and branches that are normed before they are added ------------------------------------------------------------------
def layernorm(out: torch.Tensor, x: torch.Tensor, gain: torch.Tensor, eps: float, rows_index: torch.Tensor | None = None,
              scale: float = 1.0, add: bool = False) -> None:
    """out[r] = (x[r'] - mean) / sqrt(mean((x[r'] - mean)^2) + eps) * gain * scale, r' = rows_index[r] or r; `add`: added into out
    (float32) instead of stored."""
    _need(out, "out", None, 2); _need(x, "x", None, 2); _need(gain, "gain", None, 1)
    rows, dim = out.shape
    if x.shape[1] != dim or gain.shape[0] != dim or (rows_index is None and x.shape[0] != rows):
        raise KernelError(f"layernorm: shapes out {tuple(out.shape)} x {tuple(x.shape)} gain {tuple(gain.shape)}")
    if rows_index is not None:
        _need(rows_index, "rows_index", torch.int32, 1)
        if rows_index.shape[0] < rows:
            raise KernelError("layernorm: fewer row numbers than rows")
    _check(_lib().hymt2_layernorm(_ptr(out), c_int(dtype_code(out.dtype)), _ptr(x), c_int(dtype_code(x.dtype)), _ptr(gain),
                                  c_int(dtype_code(gain.dtype)), _ptr(rows_index), c_int(rows), c_int(dim), c_float(eps), c_float(scale),
                                  c_int(1 if add else 0), _stream()), "layernorm")


def layernorm_add_norm(residual: torch.Tensor, x: torch.Tensor, gain_a: torch.Tensor, eps_a: float, out: torch.Tensor,
                       gain_b: torch.Tensor | None, eps_b: float) -> None:
    """residual (float32) += layernorm_a(x); out = layernorm_b(residual) of the new rows, or (gain_b None) the new rows themselves
    in out's type."""
    _need(residual, "residual", torch.float32, 2); _need(x, "x", torch.float32, 2); _need(out, "out", None, 2); _need(gain_a, "gain_a", None, 1)
    rows, dim = residual.shape
    if x.shape != residual.shape or out.shape != residual.shape or gain_a.shape[0] != dim:
        raise KernelError(f"layernorm_add_norm: shapes residual {tuple(residual.shape)} x {tuple(x.shape)} out {tuple(out.shape)}")
    if gain_b is not None:
        _need(gain_b, "gain_b", gain_a.dtype, 1)
        if gain_b.shape[0] != dim:
            raise KernelError("layernorm_add_norm: the second gain's width differs")
    _check(_lib().hymt2_layernorm_add_norm(_ptr(residual), _ptr(x), _ptr(gain_a), _ptr(out), c_int(dtype_code(out.dtype)), _ptr(gain_b),
                                           c_int(dtype_code(gain_a.dtype)), c_int(rows), c_int(dim), c_float(eps_a), c_float(eps_b),
                                           _stream()), "layernorm_add_norm")


MAX_NORMED_BRANCHES = 4


def rmsnorm_sum(out: torch.Tensor, branches: list, gains: list, scales: list, eps: float) -> None:
    """out (float32) = sum_b scales[b] * branches[b] / sqrt(mean(branches[b]^2) + eps) * gains[b], row by row."""
    _need(out, "out", torch.float32, 2)
    n = len(branches)
    if not (1 <= n <= MAX_NORMED_BRANCHES) or len(gains) != n or len(scales) != n:
        raise KernelError(f"rmsnorm_sum: {n} branches (1 to {MAX_NORMED_BRANCHES}), a gain and a scale each")
    for x, g in zip(branches, gains):
        _need(x, "branch", torch.float32, 2); _need(g, "gain", gains[0].dtype, 1)
        if x.shape != out.shape or g.shape[0] != out.shape[1]:
            raise KernelError(f"rmsnorm_sum: a branch is {tuple(x.shape)} with a gain of {tuple(g.shape)}, out is {tuple(out.shape)}")
    xs = (c_void_p * n)(*[x.data_ptr() for x in branches])
    gs = (c_void_p * n)(*[g.data_ptr() for g in gains])
    sc = (c_float * n)(*[float(s) for s in scales])
    _check(_lib().hymt2_rmsnorm_sum(_ptr(out), xs, gs, sc, c_int(n), c_int(dtype_code(gains[0].dtype)), c_int(out.shape[0]),
                                    c_int(out.shape[1]), c_float(eps), _stream()), "rmsnorm_sum")


# -- clamped gated activation; rotary positions on heads side by side ------------------------------------------------------------------
def clamped_glu(out: torch.Tensor, gate_up: torch.Tensor, bias: torch.Tensor | None, limit: float, alpha: float) -> None:
    """g = min(gate + bias_g, limit); u = clamp(up + bias_u, -limit, limit); out = g * sigmoid(alpha * g) * (u + 1), for rows
    [gate half | up half] of gate_up [rows, 2 * width] and bias [2 * width] float32 (or None)."""
    _need(out, "out", None, 2); _need(gate_up, "gate_up", out.dtype, 2)
    rows, width = out.shape
    if gate_up.shape != (rows, 2 * width):
        raise KernelError(f"clamped_glu: shapes out {tuple(out.shape)} gate_up {tuple(gate_up.shape)}")
    _f32(bias, "bias", 2 * width)
    _check(_lib().hymt2_clamped_glu(_ptr(out), _ptr(gate_up), c_int(dtype_code(out.dtype)), _ptr(bias), c_int(rows), c_int(width),
                                    c_float(limit), c_float(alpha), _stream()), "clamped_glu")


def rotate_heads(out: torch.Tensor, x: torch.Tensor, token_pos: torch.Tensor, inv_freq: torch.Tensor | None, heads: int, d: int,
                 rot_dims: int, pairing: str) -> None:
    """out[t] = x[t] with the first rot_dims entries of each of the first `heads` heads (d entries each, side by side from column
    0) turned by position * inv_freq[i]; pairing "half": entries (i, i + rot_dims/2), "interleaved": (2i, 2i + 1).  The columns
    behind the heads are copied.  out may have another type than x (rows of both may be columns of wider matrices)."""
    ldx, ldy = _rows_view(x, "x"), _rows_view(out, "out")
    if out.shape != x.shape or x.shape[1] < heads * d or pairing not in ("half", "interleaved"):
        raise KernelError(f"rotate_heads: shapes out {tuple(out.shape)} x {tuple(x.shape)} for {heads} heads of {d}, pairing {pairing}")
    _need(token_pos, "token_pos", torch.int32, 1); _f32(inv_freq, "inv_freq", rot_dims // 2)
    _check(_lib().hymt2_rotate_heads(_ptr(out), c_int(dtype_code(out.dtype)), c_long(ldy), _ptr(x), c_int(dtype_code(x.dtype)), c_long(ldx),
                                     _ptr(token_pos), _ptr(inv_freq), c_int(x.shape[0]), c_int(heads), c_int(d), c_int(rot_dims),
                                     c_int(1 if pairing == "interleaved" else 0), c_int(x.shape[1]), _stream()), "rotate_heads")


# -- attention whose heads talk ------------------------------------------------------------------------------------------------
MASKS = {None: 0, "chunk": 1, "window": 2}


def talk_prep(x: torch.Tensor, q_out: torch.Tensor, k_plane: torch.Tensor | None, v_plane: torch.Tensor | None, block_table: torch.Tensor,
              block_tokens: int, token_seq: torch.Tensor, token_pos: torch.Tensor, slot_ids: torch.Tensor, inv_freq: torch.Tensor | None,
              rot_dims: int, heads: int, kv_heads: int, d: int) -> None:
    """x [T, heads * d | kv_heads * d] (q, then k; rows may be columns of a wider matrix): q rotated in (2i, 2i+1) pairs goes to
    q_out [T, heads * d]; k rotated goes to the key plane and k as it is to the value plane of the token's cache row."""
    ldx = _rows_view(x, "x")
    T = x.shape[0]
    _need(q_out, "q_out", x.dtype, 2)
    if x.shape[1] != (heads + kv_heads) * d or q_out.shape != (T, heads * d):
        raise KernelError(f"talk_prep: shapes x {tuple(x.shape)} q_out {tuple(q_out.shape)}")
    if k_plane is not None:
        _need(k_plane, "k_plane", x.dtype, 4); _need(v_plane, "v_plane", x.dtype, 4)
        if k_plane.shape[1:] != (kv_heads, block_tokens, d) or v_plane.shape != k_plane.shape:
            raise KernelError(f"talk_prep: cache planes {tuple(k_plane.shape)} {tuple(v_plane.shape)}")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((token_seq, "token_seq"), (token_pos, "token_pos"), (slot_ids, "slot_ids")):
        _need(t, n, torch.int32, 1)
    _f32(inv_freq, "inv_freq", rot_dims // 2)
    _check(_lib().hymt2_talk_prep(_ptr(x), c_long(ldx), c_int(dtype_code(x.dtype)), _ptr(q_out), _ptr(k_plane), _ptr(v_plane), _ptr(block_table),
                                  c_int(block_table.stride(0)), c_int(block_tokens), _ptr(token_seq), _ptr(token_pos), _ptr(slot_ids),
                                  _ptr(inv_freq), c_int(rot_dims), c_int(T), c_int(heads), c_int(kv_heads), c_int(d), _stream()), "talk_prep")


TALK_SPLIT_KEYS = 128     # decode steps: keys a block (four tiles); a constant
TALK_MMA_MIN_TOKENS = 8   # a sequence's new tokens from which a step's attention runs 16 queries a block on the tensor cores
_talk_mma_ok: dict = {}


def talking_attention_mma_supported(heads: int, kv_heads: int, d: int, block_tokens: int) -> bool:
    key = (heads, kv_heads, d, block_tokens)
    if key not in _talk_mma_ok:
        _talk_mma_ok[key] = bool(_lib().hymt2_talking_attention_mma_supported(c_int(heads), c_int(kv_heads), c_int(d), c_int(block_tokens)))
    return _talk_mma_ok[key]


def talking_attention(out: torch.Tensor, q: torch.Tensor, gate: torch.Tensor | None, k_plane: torch.Tensor, v_plane: torch.Tensor,
                      block_table: torch.Tensor, cu_seqlens: torch.Tensor, slot_ids: torch.Tensor, kv_lens: torch.Tensor, batch: int,
                      max_new_tokens: int, heads: int, kv_heads: int, d: int, scale: float, talk: torch.Tensor, temp: torch.Tensor,
                      sink: torch.Tensor | None, mask: str | None, mask_size: int, max_kv_len: int = 0) -> None:
    """Attention of the new tokens over the paged cache with the heads' scores mixed before the softmax:
    s_h = sum_g talk[h, g] * temp[g] * scale * (q_g . k_g); a sink per head in the denominator (or None); mask None (causal),
    "chunk" (only keys of the query's own chunk of mask_size positions) or "window" (the last mask_size); the output times
    sigmoid(gate) entry by entry where a gate [T, heads * d] is given.  float32 scores and softmax.  `max_kv_len` (an upper bound
    of the sequences' lengths; 0: unknown): a decode step whose queries may see more than TALK_SPLIT_KEYS keys cuts them into
    splits of that many (a constant, so that the cut depends on nothing else), a block each, and folds them in split order."""
    _need(out, "out", None, 2); _need(q, "q", out.dtype, 2); _need(k_plane, "k_plane", out.dtype, 4); _need(v_plane, "v_plane", out.dtype, 4)
    T = out.shape[0]
    if out.shape[1] != heads * d or q.shape != out.shape or k_plane.shape[1] != kv_heads or k_plane.shape[3] != d or v_plane.shape != k_plane.shape:
        raise KernelError(f"talking_attention: shapes out {tuple(out.shape)} q {tuple(q.shape)} keys {tuple(k_plane.shape)} values {tuple(v_plane.shape)}")
    ldg = 0
    if gate is not None:
        ldg = _rows_view(gate, "gate", out.dtype)
        if gate.shape != out.shape:
            raise KernelError("talking_attention: the gate's shape differs")
    _f32(talk, "talk", heads * heads); _f32(temp, "temp", heads); _f32(sink, "sink", heads)
    if mask not in MASKS:
        raise KernelError(f"talking_attention: mask '{mask}' (known: None, 'chunk', 'window')")
    _need(block_table, "block_table", torch.int32, 2)
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    if out.dtype == torch.bfloat16 and max_new_tokens >= TALK_MMA_MIN_TOKENS and talking_attention_mma_supported(heads, kv_heads, d, k_plane.shape[2]) \
            and (gate is None or (gate.data_ptr() % 2 == 0)):
        # prompts in bfloat16: the two products on the tensor cores
        _check(_lib().hymt2_talking_attention_mma(_ptr(out), _ptr(q), _ptr(gate), c_long(ldg), _ptr(k_plane), _ptr(v_plane), _ptr(block_table),
                                                  c_int(block_table.stride(0)), c_int(k_plane.shape[2]), _ptr(cu_seqlens), _ptr(slot_ids),
                                                  _ptr(kv_lens), c_int(batch), c_int(max_new_tokens), c_int(heads), c_int(kv_heads), c_int(d),
                                                  c_float(scale), _ptr(talk), _ptr(temp), _ptr(sink), c_int(MASKS[mask]), c_int(mask_size),
                                                  _stream()), "talking_attention_mma")
        return
    split, max_splits, part_o, part_ml = 0, 0, None, None
    span = min(max_kv_len, mask_size + 31) if mask is not None else max_kv_len       # (the first tile may start up to 31 keys early)
    if max_new_tokens == 1 and span > TALK_SPLIT_KEYS and k_plane.shape[2] % 32 == 0:
        split, max_splits = TALK_SPLIT_KEYS, -(-(span + 31) // TALK_SPLIT_KEYS)
        part_o = torch.empty(batch * max_splits * heads * d, dtype=torch.float32, device=out.device)
        part_ml = torch.empty(batch * max_splits * 2 * heads, dtype=torch.float32, device=out.device)
    _check(_lib().hymt2_talking_attention(_ptr(out), _ptr(q), _ptr(gate), c_long(ldg), _ptr(k_plane), _ptr(v_plane), c_int(dtype_code(out.dtype)),
                                          _ptr(block_table), c_int(block_table.stride(0)), c_int(k_plane.shape[2]), _ptr(cu_seqlens),
                                          _ptr(slot_ids), _ptr(kv_lens), c_int(batch), c_int(max_new_tokens), c_int(heads), c_int(kv_heads),
                                          c_int(d), c_float(scale), _ptr(talk), _ptr(temp), _ptr(sink), c_int(MASKS[mask]),
                                          c_int(mask_size), c_int(split), c_int(max_splits), _ptr(part_o), _ptr(part_ml), _stream()),
           "talking_attention", 2 if split else 1)


# -- the gated delta rule ----------------------------------------------------------------------------------------------------------
def delta_scan_max_dk() -> int:
    return int(_lib().hymt2_delta_scan_max_dk())


def delta_prep(qk: torch.Tensor, qn: torch.Tensor, kn: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor, dt_bias: torch.Tensor,
               a_log: torch.Tensor, heads: int, kv_heads: int, dk: int, q_scale: float, unit_eps: float) -> None:
    """What enters the delta rule, in float32: qn, kn [T, kv_heads * dk] = q, k (columns of qk, q first) as unit vectors
    x / sqrt(sum(x^2) + unit_eps), q times q_scale; decay [T, heads * dk] in place x -> exp(-exp(a_log[h]) * softplus(x + dt_bias));
    beta [T, heads] in place x -> sigmoid(x)."""
    ldqk = _rows_view(qk, "qk")
    T = qk.shape[0]
    _need(qn, "qn", torch.float32, 2); _need(kn, "kn", torch.float32, 2); _need(decay, "decay", torch.float32, 2)
    ldb = _rows_view(beta, "beta", torch.float32)
    if qk.shape[1] != 2 * kv_heads * dk or qn.shape != (T, kv_heads * dk) or kn.shape != qn.shape or decay.shape != (T, heads * dk) \
            or beta.shape != (T, heads):
        raise KernelError(f"delta_prep: shapes qk {tuple(qk.shape)} qn {tuple(qn.shape)} decay {tuple(decay.shape)} beta {tuple(beta.shape)}")
    _f32(dt_bias, "dt_bias", heads * dk); _f32(a_log, "a_log", heads)
    _check(_lib().hymt2_delta_prep(_ptr(qk), c_long(ldqk), c_int(dtype_code(qk.dtype)), _ptr(qn), _ptr(kn), _ptr(decay), _ptr(beta), c_long(ldb),
                                   _ptr(dt_bias), _ptr(a_log), c_int(T), c_int(heads), c_int(kv_heads), c_int(dk), c_float(q_scale),
                                   c_float(unit_eps), _stream()), "delta_prep")


def delta_scan(out: torch.Tensor, qn: torch.Tensor, kn: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor, v: torch.Tensor,
               state: torch.Tensor, state_offset: int, cu_seqlens: torch.Tensor, slot_ids: torch.Tensor, kv_lens: torch.Tensor, batch: int,
               heads: int, kv_heads: int, dk: int, dv: int, max_new_tokens: int = 0) -> None:
    """Per (sequence, head), S [dk, dv] float32 at byte `state_offset` of the state row as [heads, dk, dv] (ignored by a sequence that
    starts at position 0): S = diag(decay_t) S; u = beta_t (v_t - S^T k_t); S += k_t u^T; out_t = S^T q_t.  qn, kn, decay, beta as
    delta_prep leaves them; v [T, heads * dv] in the compute type (rows may be columns of a wider matrix); out float32.
    `max_new_tokens`: the longest sequence's new tokens (1 picks the instance made for decode steps; 0: unknown)."""
    _need(out, "out", torch.float32, 2); _need(qn, "qn", torch.float32, 2); _need(kn, "kn", torch.float32, 2); _need(decay, "decay", torch.float32, 2)
    T = out.shape[0]
    ldv, ldb = _rows_view(v, "v"), _rows_view(beta, "beta", torch.float32)
    if out.shape[1] != heads * dv or qn.shape != (T, kv_heads * dk) or kn.shape != qn.shape or decay.shape != (T, heads * dk) \
            or beta.shape != (T, heads) or v.shape != (T, heads * dv):
        raise KernelError(f"delta_scan: shapes out {tuple(out.shape)} qn {tuple(qn.shape)} decay {tuple(decay.shape)} v {tuple(v.shape)}")
    if state.dtype != torch.uint8 or state.dim() != 2 or state_offset % 4 or state_offset + 4 * heads * dk * dv > state.shape[1]:
        raise KernelError("delta_scan: the state rows are too short")
    for t, n in ((cu_seqlens, "cu_seqlens"), (slot_ids, "slot_ids"), (kv_lens, "kv_lens")):
        _need(t, n, torch.int32, 1)
    _check(_lib().hymt2_delta_scan(_ptr(out), _ptr(qn), _ptr(kn), _ptr(decay), _ptr(beta), c_long(ldb), _ptr(v), c_long(ldv),
                                   c_int(dtype_code(v.dtype)), _ptr(state), c_long(state_offset), c_long(state.stride(0)), _ptr(cu_seqlens),
                                   _ptr(slot_ids), _ptr(kv_lens), c_int(batch), c_int(max_new_tokens), c_int(heads), c_int(kv_heads), c_int(dk),
                                   c_int(dv), _stream()), "delta_scan")
