"""Python launchers of the hand-written CUDA kernels.

Each function checks shapes, types and contiguity, then calls the C entry point of the compiled
library with raw device pointers on torch's current stream.  There is no CPU path and no library
stand-in: a CPU tensor or a missing library raises.
"""
from __future__ import annotations

import collections
import ctypes

import torch

from .csrc.build import CHECK_BUILD, load_library

CORE_SOURCES = ["elementwise.cu", "rope_kv.cu", "attn_tokenwise.cu", "gemm_f32.cu", "sampling.cu", "recurrent.cu", "moe.cu",
                "delta.cu", "latent.cu", "rglru.cu", "streams.cu"]

_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float

_SIGNATURES = {
    "tl_embed": [_P, _P, _I, _P, _I, _I, _F, _P],
    "tl_add_rmsnorm": [_P, _P, _P, _I, _P, _I, _P, _I, _I, _F, _I, _P, _I, ctypes.c_longlong, _F, _I, _P],
    "tl_silu_mul": [_P, _P, _I, _I, _I, _I, _I, _F, _F, _P],
    "tl_add_rmsnorm_pair": [_P, _P, _P, _P, _P, _I, _P, _P, _I, _P, _I, _I, _F, _P],
    "tl_head_gate": [_P, _I, _P, _I, _I, _I, _P],
    "tl_post_norm_add_norm": [_P, _P, _P, _P, _P, _I, _P, _I, _P, _I, _I, _F, _I, _P],
    "tl_rope_kv_write": [_P, _I, _P, _I, _P, _P, _P, _I, _I, _P, _I, _I, _I, _I, _P, _P, _I, _I, _P, _I, ctypes.c_longlong,
                         _I, _P, _P, _F, _I, _I, _I, _P, _P],
    "tl_attn_tokenwise": [_P, _I, _P, _I, _P, _P, _P, _I, _I, _P, _P, _I, _I, _I, _I, _I, _F, _P, _I, _P, _I, _P, _I, _I, _P, _P],
    "tl_gemm_f32": [_P, _I, _P, _I, _I, _P, _P, _I, _I, _I, _I, _P],
    "tl_argmax": [_P, _I, _I, _I, _P, _P, _P],
    "tl_sample": [_P, _I, _I, _I, _P, _P, _P, _P, _P],
    "tl_linear_scan": [_P, _I, _I, _I, _I, _I, _P, _F, _P, _P, _I, _I, _P, _F, _F, _P, ctypes.c_longlong, _P, _P, _P, _I, _I,
                       _I, _I, _F, _I, _P],
    "tl_scan_state_floats": [_I, _I],
    "tl_scan_columns": [],
    "tl_head_norm_gate": [_P, _P, _I, _I, _P, _I, _P, _I, _I, _I, _I, _F, _I, _P],
    "tl_sum_normed": [_P, _P, _P, _P, _I, _P, _I, _I, _I, _F, _F, _P],
    "tl_small_proj": [_P, _I, _I, _P, _P, _I, _P, _I, _I, _I, _I, _P],
    "tl_topk_softmax": [_P, _I, _I, _I, _P, _P, _I, _I, _P],
    "tl_moe_up": [_P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P, _F, _F, _I, _P],
    "tl_route_groups": [_P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _P, _P, _I, _P],
    "tl_causal_conv": [_P, _I, _I, _P, _P, _P, _I, _P, ctypes.c_longlong, _P, _P, _P, _I, _I, _I, _P],
    "tl_rglru_scan": [_P, _P, _P, _P, _I, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P, _I, ctypes.c_longlong, ctypes.c_longlong, _P],
    "tl_split3": [_P, _P, _I, _I, _I, _P],
    "tl_rglru_chunk": [],
    "tl_moe_down": [_P, _I, _P, _I, _P, _P, _P, _I, _I, _I, _I, _P, _P, _I, _I, _P, _P],
    "tl_moe_sort": [_P, _I, _I, _P, _P, _P, _P],
    "tl_moe_gather": [_P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _P, _P],
    "tl_relu_square": [_P, _I, ctypes.c_longlong, _P],
    "tl_moe_combine": [_P, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _P, _P, _I, _P],
    "tl_conv_prep": [_P, _I, _I, _P, _I, _I, _P, ctypes.c_longlong, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F, _P],
    "tl_delta_scan": [_P, _I, _I, _I, _I, _P, _I, _P, _P, _P, ctypes.c_longlong, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "tl_delta_state_floats": [_I, _I],
    "tl_delta_columns": [],
    "tl_latent_prep": [_P, _I, _I, _I, _I, _P, _P, _I, _F, _P, _I, _P, _P, _P, _I, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "tl_latent_qrot": [_P, _I, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "tl_embed_streams": [_P, _P, _I, _P, _I, _I, _F, _I, _P, _I, _I, _I, _P, _P, _P, _P],
    "tl_remember_last": [_P, _P, _P, _I, _P, _P],
    "tl_stream_step": [_P, _I, _I, _P, _F, _P, _F, _I, _P, _P, _P, _P, _I, _F, _P, _P, _P, _I, _I, _P],
    "tl_softcap": [_P, ctypes.c_longlong, _F, _P],
    "tl_sigmoid_gate": [_P, _P, _I, _P, _I, _I, _I, _P],
    "tl_head_matmul": [_P, _I, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _P],
}


class KernelError(RuntimeError):
    pass


_core = None


def core():
    global _core
    if _core is None:
        lib = load_library("tl_core", CORE_SOURCES)
        for name, sig in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = sig
            fn.restype = ctypes.c_int
        _core = lib
    return _core


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return 0
    if dt == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dt}")


def _ptr(t: torch.Tensor | None):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernel called with a CPU tensor: this engine has no CPU path")
    return t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


_launches = 0
kernel_counts: collections.Counter = collections.Counter()      # calls per kernel variant, by the name its launcher gives


def launch_count() -> int:
    """Kernels of this package launched so far in this process (a replayed CUDA graph counts the
    launches it holds)."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(status: int, what: str, launches: int = 1) -> None:
    global _launches
    if status != 0:
        raise KernelError(f"{what}: CUDA error {status} at launch")
    _launches += launches
    kernel_counts[what] += 1
    if _profile is not None:
        mark(what)


# ---------------------------------------------------------------------------------------------
# The device status word.  Kernels that wait on barriers (the tcgen05 products and attention, the TMA
# decode attention) bound every wait; a block whose wait runs out records a code here, stops and leaves
# output that is not valid.  The engine reads the word where the host waits for a step anyway (it
# travels with the sampled tokens) and fails the step's requests.

N_COUNTERS = 8192
_status: dict = {}
STATUS_ROLES = {1: "tcgen05 product: the copy thread waited for a free stage", 2: "tcgen05 product: the MMA thread waited for a stage's copies",
                3: "tcgen05 product: the epilogue waited for the accumulator",
                31: "two-block product: a copy thread waited for a free stage", 32: "two-block product: the MMA thread waited for a free accumulator",
                33: "two-block product: the MMA thread waited for a stage's copies", 34: "two-block product: the epilogue waited for the accumulator",
                20: "decode attention: a wait for a stage of keys and values"}


def device_status(device) -> torch.Tensor:
    """int32 [1 + N_COUNTERS + 4] on `device`: [0] is the status word (0 = no wait ran out), then the per-tile
    arrival counters of split products (zero between calls), then the four ints in which the checking build of the
    kernels records an index out of its bounds (code, kernel, value, limit)."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    t = _status.get(device)
    if t is None:
        with torch.inference_mode(False):                # an ordinary tensor: it is cleared in place from anywhere
            t = torch.zeros(1 + N_COUNTERS + 4, dtype=torch.int32, device=device)
        _status[device] = t
    return t


def raise_device_status(device, code: int) -> None:
    """Clear the word and raise: a wait ran out inside a kernel."""
    device_status(device)[:1].zero_()
    what = STATUS_ROLES.get(int(code), "an attention kernel's pipeline wait" if int(code) >= 10 else "a pipeline wait")
    raise KernelError(f"a kernel on {device} gave up on a wait that did not complete in time (code {int(code)}: {what}); "
                      "the step's output is not valid")


KERNEL_NAMES = {1: "rotary + page write", 2: "exact-order attention", 3: "mma.sync prompt attention", 4: "decode attention",
                5: "TMA decode attention", 6: "tcgen05 prompt attention", 7: "two-tile tcgen05 prompt attention"}


def fault_words(device):
    """Device address of the four ints of the checking build, or None when the kernels are the ordinary build."""
    if not CHECK_BUILD:
        return None
    return device_status(device).data_ptr() + 4 * (1 + N_COUNTERS)


def check_device_status(device=None) -> None:
    """Raise if any kernel launched so far gave up on a wait or, in the checking build, met an index out of
    its bounds (synchronises; reads a few words per device that has them)."""
    for dev, t in list(_status.items()):
        if CHECK_BUILD:
            code, kernel, value, limit = t[1 + N_COUNTERS:].tolist()
            if code:
                t[1 + N_COUNTERS:].zero_()
                raise KernelError(f"bounds check on {dev}: the {KERNEL_NAMES.get(kernel, kernel)} kernel met index {value}, "
                                  f"which is outside [0, {limit}); the access went to the sink instead")
        code = int(t[0].item())
        if code:
            raise_device_status(dev, code)


def num_sms(device=None) -> int:
    """Streaming multiprocessors of the device (asked once per device)."""
    dev = None if device is None else torch.device(device).index
    if dev is None:
        dev = torch.cuda.current_device()
    n = _sm_counts.get(dev)
    if n is None:
        n = _sm_counts[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return n


_sm_counts: dict = {}


# ---------------------------------------------------------------------------------------------
# Profile: an event after every launch; the time between two events goes to the later one's name.

_profile = None


def start_profile() -> None:
    global _profile
    torch.cuda.synchronize()
    first = torch.cuda.Event(enable_timing=True)
    first.record()
    _profile = [("start", first)]


def mark(name: str) -> None:
    """Inside a profile: everything launched since the last mark belongs to `name` (the launchers of this package
    call it themselves; callers of library kernels call it after them)."""
    if _profile is not None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        _profile.append((name, ev))


def stop_profile() -> dict:
    """name -> (calls, milliseconds) since `start_profile`."""
    global _profile
    marks, _profile = _profile, None
    torch.cuda.synchronize()
    out: dict = {}
    for (_, before), (name, ev) in zip(marks, marks[1:]):
        name = name.split("<")[0].split("+")[0] if name.startswith(("gemm_tc", "attn_")) else name
        calls, ms = out.get(name, (0, 0.0))
        out[name] = (calls + 1, ms + before.elapsed_time(ev))
    return out


def _contig(t: torch.Tensor, name: str) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _ints(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.int32:
        raise KernelError(f"{name} must be int32, got {t.dtype}")
    _contig(t, name)


# ---------------------------------------------------------------------------------------------

def embed(x: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, scale: float = 1.0) -> None:
    """x[t, :] = table[ids[t], :] * scale, x float32 [T, H]."""
    T, H = x.shape
    if x.dtype != torch.float32 or table.shape[1] != H or ids.numel() != T:
        raise KernelError("embed: x must be float32 [T, H] matching the table and ids")
    _contig(x, "x"); _contig(table, "table"); _ints(ids, "ids")
    _check(core().tl_embed(_ptr(x), _ptr(table), dtype_code(table.dtype), _ptr(ids), T, H, float(scale), _stream()), "embed")


def embed_streams(x: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, scale: float = 1.0, copies: int = 1,
                  pairs: torch.Tensor | None = None, mul_prev: int = 0, mul_cur: int = 0, pos: torch.Tensor | None = None,
                  req_slot: torch.Tensor | None = None, last_token: torch.Tensor | None = None) -> None:
    """x[t] = `copies` times side by side: table[ids[t]] * scale (+ pairs[row]), x float32 [T, copies * H].  `pairs`
    [buckets + 1, H] of the table's type: row = (previous token * mul_prev + ids[t] * mul_cur) mod buckets, and row `buckets`
    at position 0; the previous token is ids[t - 1] if that row belongs to the same request slot, else last_token[slot]
    (int32, one number a request slot: what `remember_last` left there in the step before)."""
    T, H = ids.numel(), table.shape[1]
    if x.dtype != torch.float32 or x.shape != (T, copies * H) or copies < 1:
        raise KernelError("embed_streams: x must be float32 [T, copies * H] matching the table and ids")
    _contig(x, "x"); _contig(table, "table"); _ints(ids, "ids")
    buckets = 0
    if pairs is not None:
        buckets = pairs.shape[0] - 1
        if pairs.dim() != 2 or pairs.shape[1] != H or pairs.dtype != table.dtype or buckets < 1:
            raise KernelError("embed_streams: pairs must be [buckets + 1, H] of the table's type")
        if pos is None or req_slot is None or last_token is None:
            raise KernelError("embed_streams: a table of pairs needs positions, request slots and the slots' last tokens")
        _contig(pairs, "pairs"); _ints(pos, "pos"); _ints(req_slot, "req_slot"); _ints(last_token, "last_token")
    _check(core().tl_embed_streams(_ptr(x), _ptr(table), dtype_code(table.dtype), _ptr(ids), T, H, float(scale), int(copies),
                                   _ptr(pairs), buckets, int(mul_prev), int(mul_cur), _ptr(pos), _ptr(req_slot), _ptr(last_token),
                                   _stream()), "embed_streams")


def remember_last(ids: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, last_token: torch.Tensor, B: int) -> None:
    """last_token[slots[b]] = the last of request b's ids in this step (its rows are q_start[b] .. q_start[b + 1] - 1)."""
    _ints(ids, "ids"); _ints(q_start, "q_start"); _ints(slots, "slots"); _ints(last_token, "last_token")
    if q_start.numel() < B + 1 or slots.numel() < B:
        raise KernelError("remember_last: q_start [B + 1], slots [B]")
    _check(core().tl_remember_last(_ptr(ids), _ptr(q_start), _ptr(slots), int(B), _ptr(last_token), _stream()), "remember_last")


def stream_step(x: torch.Tensor, S: int, a: torch.Tensor | None = None, alpha: float = 1.0, b: torch.Tensor | None = None,
                beta: float = 1.0, mix: torch.Tensor | None = None, out: torch.Tensor | None = None,
                read: torch.Tensor | None = None, w: torch.Tensor | None = None, eps: float = 0.0, h: torch.Tensor | None = None,
                u: torch.Tensor | None = None, rows: torch.Tensor | None = None) -> None:
    """One boundary between sublayers of a residual stream kept as S copies, x float32 [T, S * W], in one kernel:
    with `mix` (float32 [S, S], indexed [from, to]) and `out` (float32 [S]) every stream is rebuilt from the old ones,
    x_r <- sum_s mix[s, r] x_s + out[r] (alpha a + beta b)  (a, b [T, W] of the activation type, either may be None); then
    u = sum_r read[r] x_r (`read` float32 [S]; None: the plain sum) goes to `u` (float32 [R, W]) if given, and its RMS norm
    times `w` to `h` ([R, W] of the activation type) if given.  `rows` (int32 [R]) picks rows; x is then left alone."""
    T = x.shape[0]
    if x.dtype != torch.float32 or x.dim() != 2 or x.shape[1] % S or not x.is_contiguous():
        raise KernelError("stream_step: x must be float32 [T, S * W], contiguous")
    W = x.shape[1] // S
    R = T if rows is None else rows.numel()
    act = h.dtype if h is not None else (a.dtype if a is not None else (b.dtype if b is not None else torch.float32))
    for name, t in (("a", a), ("b", b)):
        if t is not None and (t.shape != (T, W) or t.dtype != act or not t.is_contiguous()):
            raise KernelError(f"stream_step: {name} must be [T, W] of the activation type, contiguous")
    if (mix is None) != (out is None) or (mix is None and (a is not None or b is not None)):
        raise KernelError("stream_step: mix and out come together, and the addends with them")
    for name, t, n in (("mix", mix, S * S), ("out", out, S), ("read", read, S)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
            raise KernelError(f"stream_step: {name} must be float32 with {n} numbers")
    if h is not None and (h.shape != (R, W) or w is None or w.numel() != W or not h.is_contiguous() or not w.is_contiguous()):
        raise KernelError("stream_step: h [R, W] comes with a weight [W]")
    if u is not None and (u.shape != (R, W) or u.dtype != torch.float32 or not u.is_contiguous()):
        raise KernelError("stream_step: u must be float32 [R, W]")
    if rows is not None:
        _ints(rows, "rows")
    _check(core().tl_stream_step(_ptr(x), S, W, _ptr(a), float(alpha), _ptr(b), float(beta), dtype_code(act), _ptr(mix), _ptr(out),
                                 _ptr(read), _ptr(w), dtype_code(w.dtype) if w is not None else 0, float(eps), _ptr(h), _ptr(u),
                                 _ptr(rows), R, int(rows is None), _stream()), "stream_step")


def softcap(z: torch.Tensor, cap: float) -> None:
    """z <- cap * tanh(z / cap) in place, z float32."""
    if z.dtype != torch.float32 or not z.is_contiguous():
        raise KernelError("softcap: z must be float32, contiguous")
    _check(core().tl_softcap(_ptr(z), z.numel(), float(cap), _stream()), "softcap")


def sigmoid_gate(o: torch.Tensor, gate: torch.Tensor, y: torch.Tensor) -> None:
    """y[t, c] = o[t, c] * sigmoid(gate[t, c]); o, y [T, N] of one type, gate float32 [T, N] (a column range of a wider
    tensor may be passed)."""
    T, N = o.shape
    if y.shape != o.shape or y.dtype != o.dtype or gate.dtype != torch.float32 or gate.shape != o.shape or gate.stride(1) != 1:
        raise KernelError("sigmoid_gate: o, y [T, N] of one type, gate float32 [T, N]")
    _contig(o, "o"); _contig(y, "y")
    _check(core().tl_sigmoid_gate(_ptr(o), _ptr(gate), gate.stride(0), _ptr(y), T, N, dtype_code(o.dtype), _stream()), "sigmoid_gate")


def add_rmsnorm(x: torch.Tensor, r: torch.Tensor | None, w: torch.Tensor, out: torch.Tensor, eps: float,
                rows: torch.Tensor | None = None, write_x: bool = True, pieces: torch.Tensor | None = None,
                alpha: float = 1.0, cast_first: bool = True) -> None:
    """x += alpha * r (if r), out = cast(x * rstd) * w.  x float32 [*, H]; r, out of the activation
    type; `rows` picks the rows (x is then left alone).  `cast_first` False: the norm stays float up to
    the weight and only the result is rounded.  `pieces` [S, rows of x, H] float32 instead
    of r: the addend as a split-K product left it; summed in split order and rounded to the
    activation type inside the kernel (needs H % 4 == 0 and H <= 32768)."""
    H = x.shape[-1]
    R = out.shape[0]
    if x.dtype != torch.float32 or out.shape[-1] != H or w.numel() != H:
        raise KernelError("add_rmsnorm: x must be float32 and out, w must match its width")
    if r is not None and (r.dtype != out.dtype or r.shape != x.shape):
        raise KernelError("add_rmsnorm: r must have x's shape and out's type")
    _contig(x, "x"); _contig(out, "out"); _contig(w, "w")
    if r is not None:
        _contig(r, "r")
    splits = plane = 0
    if pieces is not None:
        if r is not None or pieces.dtype != torch.float32 or pieces.dim() != 3 or pieces.shape[1:] != x.shape:
            raise KernelError("add_rmsnorm: pieces must be float32 [S, rows of x, H] and stand instead of r")
        if H % 4 or H > 32768:
            raise KernelError("add_rmsnorm: pieces need a width that is a multiple of 4 and at most 32768")
        _contig(pieces, "pieces")
        splits, plane = pieces.shape[0], x.numel()
    if rows is not None:
        _ints(rows, "rows")
        if rows.numel() != R:
            raise KernelError("add_rmsnorm: one output row per entry of rows")
        write_x = False
    elif x.shape[0] != R:
        raise KernelError("add_rmsnorm: out must have x's rows")
    _check(core().tl_add_rmsnorm(_ptr(x), _ptr(r), _ptr(w), dtype_code(w.dtype), _ptr(out), dtype_code(out.dtype),
                                 _ptr(rows), R, H, float(eps), int(write_x), _ptr(pieces), splits, plane, float(alpha),
                                 int(cast_first), _stream()),
           "add_rmsnorm")


GATE_ACTS = {"silu": 0, "gelu_tanh": 1, "relu_squared": 2, "swish_clamped": 3}


def gate_act(act) -> tuple:
    """(code, limit, alpha) of an activation given by name, or as ("swish_clamped", limit, alpha): with g' = min(g, limit) and
    u' = clamp(u, -limit, limit) the gated unit is g' sigmoid(alpha g') (u' + 1)."""
    if isinstance(act, tuple):
        name, limit, alpha = act
        if name != "swish_clamped" or not limit > 0:
            raise KernelError(f"an activation with constants is ('swish_clamped', limit > 0, alpha), not {act!r}")
        return GATE_ACTS[name], float(limit), float(alpha)
    if act not in GATE_ACTS or act == "swish_clamped":
        raise KernelError(f"activation {act!r} is not one of {sorted(GATE_ACTS)} ('swish_clamped' comes with its constants)")
    return GATE_ACTS[act], 0.0, 0.0


def silu_mul(gu: torch.Tensor, out: torch.Tensor, block: int | None = None, act="silu") -> None:
    """out = act(gate) * up from gu [T, 2I], act "silu", "gelu_tanh" (the tanh form of gelu) or ("swish_clamped", limit, alpha)
    (see `gate_act`).  block None: gate = gu[:, :I], up = gu[:, I:]; else gate
    and up columns alternate in blocks of `block` columns (gate first), as a product against weight rows
    interleaved that way leaves them."""
    T, I = out.shape
    if gu.shape != (T, 2 * I) or gu.dtype != out.dtype:
        raise KernelError("silu_mul: gu must be [T, 2I] of out's type")
    blk = I if block is None else int(block)
    if blk <= 0 or I % blk:
        raise KernelError(f"silu_mul: the block of {blk} columns must divide I = {I}")
    _contig(gu, "gu"); _contig(out, "out")
    code, limit, alpha = gate_act(act)
    if code == GATE_ACTS["relu_squared"]:
        raise KernelError("silu_mul: 'relu_squared' is not a gate of this kernel")
    _check(core().tl_silu_mul(_ptr(gu), _ptr(out), dtype_code(out.dtype), T, I, blk, code, limit, alpha, _stream()), "silu_mul")


def add_rmsnorm_pair(x: torch.Tensor, a: torch.Tensor | None, b: torch.Tensor | None, w1: torch.Tensor, w2: torch.Tensor | None,
                     h1: torch.Tensor, h2: torch.Tensor | None, eps: float, rows: torch.Tensor | None = None) -> None:
    """x += a + b (either may be None; b only with a), then h1 = x / rms(x) * w1 and h2 = x / rms(x) * w2 from one set of
    statistics, float32 up to the rounding of h1 and h2.  x float32 [*, H]; a, b, h1, h2 of the activation type; `rows`
    picks the rows that are produced (x is then left alone).  h2 and w2 None: one norm."""
    H = x.shape[-1]
    R = x.shape[0] if rows is None else rows.numel()
    if x.dtype != torch.float32 or not x.is_contiguous() or h1.shape != (R, H) or not h1.is_contiguous():
        raise KernelError("add_rmsnorm_pair: x must be contiguous float32 [*, H] and h1 [rows, H]")
    if (h2 is None) != (w2 is None) or (b is not None and a is None):
        raise KernelError("add_rmsnorm_pair: the second norm comes with its weight, the second addend with the first")
    for name, t in (("a", a), ("b", b)):
        if t is not None and (t.shape != x.shape or t.dtype != h1.dtype or not t.is_contiguous()):
            raise KernelError(f"add_rmsnorm_pair: {name} must have x's shape and h1's type")
    if h2 is not None and (h2.shape != h1.shape or h2.dtype != h1.dtype or not h2.is_contiguous()):
        raise KernelError("add_rmsnorm_pair: h2 must be like h1")
    for w in (w1, w2):
        if w is not None and (w.numel() != H or w.dtype != w1.dtype or not w.is_contiguous()):
            raise KernelError("add_rmsnorm_pair: weights must be [H] of one type")
    if rows is not None:
        _ints(rows, "rows")
    _check(core().tl_add_rmsnorm_pair(_ptr(x), _ptr(a), _ptr(b), _ptr(w1), _ptr(w2), dtype_code(w1.dtype), _ptr(h1), _ptr(h2),
                                      dtype_code(h1.dtype), _ptr(rows), R, H, float(eps), _stream()), "add_rmsnorm_pair")


def head_gate(o: torch.Tensor, gate: torch.Tensor, nq: int, d: int) -> None:
    """o[t, h, :] *= sigmoid(gate[t, h]) in place; o [T, nq * d] of the activation type, gate float32 [T, nq]."""
    T = o.shape[0]
    if o.shape != (T, nq * d) or gate.shape != (T, nq) or gate.dtype != torch.float32:
        raise KernelError("head_gate: o [T, nq d], gate float32 [T, nq]")
    _contig(o, "o"); _contig(gate, "gate")
    _check(core().tl_head_gate(_ptr(o), dtype_code(o.dtype), _ptr(gate), T, nq, d, _stream()), "head_gate")


def post_norm_add_norm(x: torch.Tensor, a: torch.Tensor | None, w_post: torch.Tensor | None, w_pre: torch.Tensor | None,
                       out: torch.Tensor | None, eps: float, extra: torch.Tensor | None = None,
                       rows: torch.Tensor | None = None) -> None:
    """x += a / rms(a) * w_post (+ extra, float32 [H], once a row); out = x / rms(x) * w_pre; float to the end.
    x float32 [*, H]; a (or None: no addend) and out (or None: the sum only) of the activation type; the two weights of
    one type.  `rows` picks the rows that are produced (x is then left alone)."""
    H = x.shape[-1]
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("post_norm_add_norm: x must be contiguous float32")
    if (a is None) != (w_post is None) or (out is None) != (w_pre is None):
        raise KernelError("post_norm_add_norm: an addend comes with its weight, an output with its weight")
    ws = [w for w in (w_post, w_pre) if w is not None]
    if any(w.numel() != H or not w.is_contiguous() or w.dtype != ws[0].dtype for w in ws):
        raise KernelError("post_norm_add_norm: weights must be [H] of one type")
    if a is not None and (a.shape != x.shape or not a.is_contiguous()):
        raise KernelError("post_norm_add_norm: a must have x's shape")
    if a is not None and out is not None and a.dtype != out.dtype:
        raise KernelError("post_norm_add_norm: a and out must have one type")
    if extra is not None and (extra.dtype != torch.float32 or extra.numel() != H or not extra.is_contiguous()):
        raise KernelError("post_norm_add_norm: extra must be float32 [H]")
    R = x.shape[0] if rows is None else rows.numel()
    if rows is not None:
        _ints(rows, "rows")
    if out is not None and (out.shape != (R, H) or not out.is_contiguous()):
        raise KernelError("post_norm_add_norm: out must be [rows, H]")
    act = out.dtype if out is not None else a.dtype if a is not None else torch.float32
    _check(core().tl_post_norm_add_norm(_ptr(x), _ptr(a), _ptr(w_post), _ptr(extra), _ptr(w_pre), dtype_code(ws[0].dtype) if ws else 0,
                                        _ptr(out), dtype_code(act), _ptr(rows), R, H, float(eps), int(rows is None), _stream()),
           "post_norm_add_norm")


def rope_kv_write(qkv: torch.Tensor, bias: torch.Tensor | None, pos: torch.Tensor, req_slot: torch.Tensor,
                  table: torch.Tensor, page_size: int, inv_freq: torch.Tensor, rot: int, nq: int, nkv: int,
                  d: int, k_pages: torch.Tensor | None, v_pages: torch.Tensor | None, write_kv: bool = True,
                  pieces: torch.Tensor | None = None, pairing: str = "half", q_norm: torch.Tensor | None = None,
                  k_norm: torch.Tensor | None = None, norm_eps: float = 0.0, norm_dim: int = 0) -> None:
    """Bias, rotary encoding of q and k in place, and the write of k, v into their pages.
    `pairing`: "half" rotates dimensions (i, i + rot/2), "interleaved" (2i, 2i + 1).  `q_norm`, `k_norm`
    (float32 [d], both or neither): every q and k head is RMS-normalised over its d dimensions (after the
    bias, before the rotation; statistics in float32) and multiplied by the weight.  `norm_dim` (0: d): the mean of squares
    is taken over this many dimensions (a head that is padded with zeros to d).
    `pieces` [S, T, width] float32: the projection as a split-K product left it; the kernel sums them
    (bfloat16, full rotary, d % 16 == 0 only) and qkv is output only (its q columns are written)."""
    T = qkv.shape[0]
    splits = plane = 0
    if pairing not in ("half", "interleaved"):
        raise KernelError(f"rope_kv_write: pairing {pairing!r} is neither 'half' nor 'interleaved'")
    if (q_norm is None) != (k_norm is None):
        raise KernelError("rope_kv_write: q_norm and k_norm come together")
    for name, w in (("q_norm", q_norm), ("k_norm", k_norm)):
        if w is not None and (w.dtype != torch.float32 or w.numel() != d or not w.is_contiguous()):
            raise KernelError(f"rope_kv_write: {name} must be float32 [d]")
    if pieces is not None and (pairing != "half" or q_norm is not None):
        raise KernelError("rope_kv_write: pieces go with rotate-half pairing and no q/k norm")
    if pieces is not None:
        if (pieces.dtype != torch.float32 or pieces.dim() != 3 or pieces.shape[1:] != qkv.shape
                or qkv.dtype != torch.bfloat16 or rot != d or d % 16):
            raise KernelError("rope_kv_write: pieces must be float32 [S, T, width] for bfloat16 qkv, full rotary, d % 16 == 0")
        _contig(pieces, "pieces")
        splits, plane = pieces.shape[0], qkv.numel()
    if qkv.shape[1] != (nq + 2 * nkv) * d:
        raise KernelError("rope_kv_write: qkv must be [T, (nq + 2 nkv) d]")
    _contig(qkv, "qkv"); _ints(pos, "pos"); _ints(req_slot, "req_slot"); _ints(table, "table")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != rot // 2:
        raise KernelError("rope_kv_write: inv_freq must be float32 [rot/2]")
    if write_kv:
        for name, pages in (("k_pages", k_pages), ("v_pages", v_pages)):
            if pages is None or pages.dtype != qkv.dtype or tuple(pages.shape[1:]) != (nkv, page_size, d):
                raise KernelError(f"rope_kv_write: {name} must be [pages, nkv, page, d] of qkv's type")
            _contig(pages, name)
    _check(core().tl_rope_kv_write(
        _ptr(qkv), dtype_code(qkv.dtype), _ptr(bias), dtype_code(bias.dtype) if bias is not None else 0,
        _ptr(pos), _ptr(req_slot), _ptr(table), table.shape[1], page_size, _ptr(inv_freq), rot, nq, nkv, d,
        _ptr(k_pages) if write_kv else None, _ptr(v_pages) if write_kv else None, int(write_kv), T,
        _ptr(pieces), splits, plane, int(pairing == "interleaved"), _ptr(q_norm), _ptr(k_norm), float(norm_eps),
        int(norm_dim), table.shape[0], k_pages.shape[0] if write_kv else 0, fault_words(qkv.device), _stream()), "rope_kv_write")


def attn_tokenwise(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                   table: torch.Tensor, page_size: int, pos: torch.Tensor, req_slot: torch.Tensor,
                   nq: int, nkv: int, d: int, window: int | None, scale: float, sink: torch.Tensor | None = None,
                   keep_first: int = 0, gate: torch.Tensor | None = None, chunk: int | None = None,
                   slopes: torch.Tensor | None = None) -> None:
    """Exact-order paged attention; q rows `q_stride` elements apart, out [T, nq*d].  `sink` (float32 [nq]): one more
    term exp(sink[h]) in every softmax denominator of head h.  `keep_first` (with a window): the keys at positions below
    it stay visible beside the window.  `gate` (float32 [T, nq]): the row of (t, h) is multiplied by sigmoid(gate[t, h]).
    `chunk` (instead of a window): a query reads the keys of its own chunk of that many positions, counted from position 0.
    `slopes` (float32 [nq]): the score of key j seen from position p loses slopes[h] * (p - j)."""
    T = out.shape[0]
    if out.shape[1] != nq * d or out.dtype != q.dtype or k_pages.dtype != q.dtype:
        raise KernelError("attn_tokenwise: out must be [T, nq*d] and all tensors of one type")
    if d > 512:
        raise KernelError(f"attn_tokenwise: head_dim {d} > 512 is not supported")
    _contig(out, "out"); _contig(k_pages, "k_pages"); _contig(v_pages, "v_pages")
    _ints(pos, "pos"); _ints(req_slot, "req_slot"); _ints(table, "table")
    _sink(sink, nq, "attn_tokenwise")
    if gate is not None and (gate.dtype != torch.float32 or gate.shape != (T, nq) or not gate.is_contiguous()):
        raise KernelError("attn_tokenwise: gate must be float32 [T, query heads]")
    if keep_first < 0:
        raise KernelError("attn_tokenwise: keep_first must not be negative")
    if chunk and window:
        raise KernelError("attn_tokenwise: a window or chunks, not both")
    _sink(slopes, nq, "attn_tokenwise (slopes)")
    _check(core().tl_attn_tokenwise(_ptr(q), q_stride, _ptr(out), dtype_code(q.dtype), _ptr(k_pages), _ptr(v_pages),
                                    _ptr(table), table.shape[1], page_size, _ptr(pos), _ptr(req_slot), T, nq, nkv, d,
                                    int(window or 0), float(scale), _ptr(sink), int(keep_first), _ptr(gate), int(chunk or 0),
                                    _ptr(slopes), table.shape[0], k_pages.shape[0], fault_words(out.device), _stream()),
           "attn_tokenwise")


def _sink(sink, nq: int, who: str) -> None:
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != nq or not sink.is_contiguous()):
        raise KernelError(f"{who}: sink must be float32 [query heads]")


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None) -> None:
    """out[M, N] = a[M, K] w[N, K]^T (+ bias), float32 FFMA; w float32 or bfloat16 (widened)."""
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.float32 or out.dtype != torch.float32 or w.shape[1] != K or out.shape != (M, N):
        raise KernelError("gemm_f32: a [M,K] and out [M,N] must be float32, w [N,K]")
    if a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_f32: a and out must have unit inner stride")
    _contig(w, "w")
    if bias is not None and bias.dtype != w.dtype:
        raise KernelError("gemm_f32: bias must have w's type")
    _check(core().tl_gemm_f32(_ptr(a), a.stride(0), _ptr(w), K, dtype_code(w.dtype), _ptr(bias), _ptr(out),
                              out.stride(0), M, N, K, _stream()), "gemm_f32")


ARGMAX_SLICES = 32


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the largest logit of row r, the lowest index on a tie."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("argmax: logits must be float32 with unit inner stride")
    _ints(out, "out")
    wide = V >= 8192                                     # wide rows are cut into slices, merged by a second kernel
    partial = torch.empty(R * 2 * ARGMAX_SLICES, dtype=torch.int32, device=logits.device) if wide else None
    _check(core().tl_argmax(_ptr(logits), logits.stride(0), R, V, _ptr(out), _ptr(partial), _stream()), "argmax",
           launches=2 if wide else 1)


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, uniform: torch.Tensor,
           out: torch.Tensor) -> None:
    """Per row: temperature <= 0 gives the argmax, else a draw from softmax(logits / T) cut to
    the top-p nucleus, picked by inverse CDF at `uniform`."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with unit inner stride")
    for name, t in (("temperature", temperature), ("top_p", top_p), ("uniform", uniform)):
        if t.dtype != torch.float32 or t.numel() != R:
            raise KernelError(f"sample: {name} must be float32 [R]")
    _ints(out, "out")
    _check(core().tl_sample(_ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(top_p), _ptr(uniform),
                            _ptr(out), _stream()), "sample")


# ---------------------------------------------------------------------------------------------
# Linear recurrences with a matrix state per head (csrc/recurrent.cu)

def scan_state_floats(d: int, gated: bool) -> int:
    """Floats of state that `linear_scan` keeps per (head, slice of `scan_columns()` value columns) for heads of d rows."""
    n = core().tl_scan_state_floats(int(d), int(gated))
    if n <= 0:
        raise KernelError(f"linear_scan: heads of {d} rows are not supported (at most 256)")
    return n


def scan_columns() -> int:
    return core().tl_scan_columns()


def linear_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, H: int, d: int, dv: int, state: torch.Tensor,
                q_start: torch.Tensor, slots: torch.Tensor, pos: torch.Tensor, out: torch.Tensor, *, B: int,
                decay: torch.Tensor | None = None, gates: torch.Tensor | None = None, cap: float = 1.0,
                inv_freq: torch.Tensor | None = None, rot: int = 0, pairing: str = "half", q_scale: float = 1.0,
                k_scale: float = 1.0, den_eps: float = 0.0, single_tokens: bool = False) -> None:
    """S_t = a_t S_(t-1) + b_t k_t v_t^T and o_t = S_t^T q_t per (request, head), tokens of a request in order, the state
    read from and left in `state[slot]` (float32, one row a slot, in the kernel's own layout: `scan_state_floats`).
    q, k [H, d] and v [H, dv] of token t are at `proj[t, q_off:]`, `proj[t, k_off:]`, `proj[t, v_off:]`.
    `decay` (float32 [H]): a_t = decay[h], b_t = 1.  `gates` (float32 [T, 2H], input then forget pre-activations): the
    capped log gates with a running maximum, a normaliser, and o_t divided by max(|n_t . q_t|, exp(-m_t)) + den_eps.
    q and k are rotated by `pos` over their first `rot` dimensions (`inv_freq` float32 [rot/2]) and scaled; a request's
    tokens of the step stand at consecutive positions (the kernel reads the first one's).  out float32 [T, H * dv].
    `single_tokens`: every request brings exactly one token (T == B): the step kernel, which gives the scan kernel's bits."""
    T = proj.shape[0]
    if (decay is None) == (gates is None):
        raise KernelError("linear_scan: either a fixed decay per head or gate pre-activations")
    if single_tokens and T != B:
        raise KernelError("linear_scan: a step of single tokens has as many rows as requests")
    _contig(proj, "proj"); _ints(q_start, "q_start"); _ints(slots, "slots"); _ints(pos, "pos"); _contig(state, "state"); _contig(out, "out")
    if out.dtype != torch.float32 or out.shape != (T, H * dv) or state.dtype != torch.float32:
        raise KernelError("linear_scan: out must be float32 [T, H * dv] and the state float32")
    nz = -(-dv // scan_columns())
    per_slot = H * nz * scan_state_floats(d, gates is not None)
    if state[0].numel() != per_slot:
        raise KernelError(f"linear_scan: a slot holds {state[0].numel()} floats, these sizes need {per_slot}")
    for name, off, width in (("q", q_off, H * d), ("k", k_off, H * d), ("v", v_off, H * dv)):
        if off < 0 or off + width > proj.shape[1]:
            raise KernelError(f"linear_scan: {name} does not lie inside a projection row")
    if decay is not None and (decay.dtype != torch.float32 or decay.numel() != H):
        raise KernelError("linear_scan: decay must be float32 [H]")
    if gates is not None and (gates.dtype != torch.float32 or gates.shape != (T, 2 * H) or not gates.is_contiguous()):
        raise KernelError("linear_scan: gates must be float32 [T, 2H]")
    if rot and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() != rot // 2):
        raise KernelError("linear_scan: inv_freq must be float32 [rot/2]")
    if pairing not in ("half", "interleaved"):
        raise KernelError(f"linear_scan: pairing {pairing!r} is neither 'half' nor 'interleaved'")
    _check(core().tl_linear_scan(_ptr(proj), dtype_code(proj.dtype), proj.shape[1], q_off, k_off, v_off, _ptr(gates), float(cap),
                                 _ptr(decay), _ptr(inv_freq) if rot else None, int(rot), int(pairing == "interleaved"), _ptr(pos),
                                 float(q_scale), float(k_scale), _ptr(state), per_slot, _ptr(q_start), _ptr(slots), _ptr(out),
                                 int(B), H, d, dv, float(den_eps), int(single_tokens), _stream()),
           "linear_step" if single_tokens else "linear_scan")


_ACTS = {None: 0, "sigmoid": 1, "silu": 2}


def head_norm_gate(o: torch.Tensor, out: torch.Tensor, H: int, dv: int, eps: float, weight: torch.Tensor | None = None,
                   gate: torch.Tensor | None = None, gate_off: int = 0, act: str | None = None) -> None:
    """out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * weight[h, :] * act(gate[t, gate_off + h dv + :]); o float32
    [T, H dv], out of the activation type, the gate rows float32 or bfloat16; weight (any float type, [H dv]) and the gate
    are optional."""
    T = o.shape[0]
    if o.dtype != torch.float32 or o.shape != (T, H * dv) or out.shape != o.shape:
        raise KernelError("head_norm_gate: o must be float32 [T, H dv] and out of its shape")
    if act not in _ACTS or (act is not None) != (gate is not None):
        raise KernelError("head_norm_gate: a gate comes with 'sigmoid' or 'silu'")
    _contig(o, "o"); _contig(out, "out")
    g_ptr, g_stride, g_code = None, 0, 0
    if gate is not None:
        if gate.stride(1) != 1 or gate_off + H * dv > gate.shape[1]:
            raise KernelError("head_norm_gate: the gate rows must hold H dv columns from gate_off")
        g_ptr, g_stride, g_code = _ptr(gate) + gate_off * gate.element_size(), gate.stride(0), dtype_code(gate.dtype)
    if weight is not None and (weight.numel() != H * dv or not weight.is_contiguous()):
        raise KernelError("head_norm_gate: weight must be [H dv]")
    _check(core().tl_head_norm_gate(_ptr(o), g_ptr, g_code, g_stride, _ptr(weight), dtype_code(weight.dtype) if weight is not None else 0,
                                    _ptr(out), dtype_code(out.dtype), T, H, dv, float(eps), _ACTS[act], _stream()), "head_norm_gate")


def sum_normed(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, out: torch.Tensor, eps: float,
               scale: float) -> None:
    """out = scale * (a / rms(a) * wa + b / rms(b) * wb), rows of the model width; statistics in float32."""
    T, W = a.shape
    if b.shape != a.shape or out.shape != a.shape or b.dtype != a.dtype or out.dtype != a.dtype or wa.dtype != wb.dtype \
            or wa.numel() != W or wb.numel() != W:
        raise KernelError("sum_normed: a, b, out [T, W] of one type, weights [W] of one type")
    _contig(a, "a"); _contig(b, "b"); _contig(out, "out"); _contig(wa, "wa"); _contig(wb, "wb")
    _check(core().tl_sum_normed(_ptr(a), _ptr(b), _ptr(wa), _ptr(wb), dtype_code(wa.dtype), _ptr(out), dtype_code(out.dtype),
                                T, W, float(eps), float(scale), _stream()), "sum_normed")


# ---------------------------------------------------------------------------------------------
# Routed feed-forward (csrc/moe.cu)

def small_proj(h: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor) -> None:
    """out[t, n] = bias[n] + h[t, :] . w[n, :] in float32 whatever h's type (router logits, gate pre-activations);
    out may be a column range of a wider float32 tensor."""
    T, K = h.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (T, N) or out.dtype != torch.float32 or out.stride(1) != 1 or h.stride(1) != 1:
        raise KernelError("small_proj: h [T, K], w [N, K], out float32 [T, N]")
    if bias is not None and (bias.dtype != w.dtype or bias.numel() != N):
        raise KernelError("small_proj: bias must be [N] of w's type")
    _contig(w, "w")
    _check(core().tl_small_proj(_ptr(h), dtype_code(h.dtype), h.stride(0), _ptr(w), _ptr(bias), dtype_code(w.dtype), _ptr(out),
                                out.stride(0), T, N, K, _stream()), "small_proj")


def topk_softmax(z: torch.Tensor, top: int, idx: torch.Tensor, wts: torch.Tensor, scoring: str = "softmax_chosen") -> None:
    """Per row of z (float32 [T, E], rows may be a column range of a wider tensor): the `top` largest entries (lowest index
    first on a tie) in idx int32 [T, top]; wts float32 [T, top]: the softmax over those entries alone ("softmax_chosen"),
    or the sigmoid of each ("sigmoid")."""
    T, E = z.shape
    if z.dtype != torch.float32 or wts.dtype != torch.float32 or idx.shape != (T, top) or wts.shape != (T, top) or z.stride(1) != 1:
        raise KernelError("topk_softmax: z float32 [T, E], idx int32 [T, top], wts float32 [T, top]")
    if scoring not in ("softmax_chosen", "sigmoid"):
        raise KernelError(f"topk_softmax: scoring {scoring!r} is neither 'softmax_chosen' nor 'sigmoid'")
    _ints(idx, "idx"); _contig(wts, "wts")
    _check(core().tl_topk_softmax(_ptr(z), z.stride(0), E, int(top), _ptr(idx), _ptr(wts), T, int(scoring == "sigmoid"), _stream()),
           "topk_softmax")


def route_groups(z: torch.Tensor, correction: torch.Tensor | None, top: int, groups: int, keep: int, group_top: int, scale: float,
                 idx: torch.Tensor, wts: torch.Tensor, softmax: bool = False) -> None:
    """Per row of z (float32 [T, E]): s = sigmoid(z) (`softmax`: the softmax of z over all E entries); the choice scores are s + correction (float32 [E] or None).  The experts
    form `groups` equal groups of neighbours; a group's score is the sum of its `group_top` largest choice scores; only the
    experts of the `keep` best groups can be chosen.  idx int32 [T, top]: the `top` largest choice scores among them (lowest
    index first on a tie); wts float32 [T, top]: the chosen experts' s divided by their sum (+ 1e-20), times `scale`."""
    T, E = z.shape
    if z.dtype != torch.float32 or wts.dtype != torch.float32 or idx.shape != (T, top) or wts.shape != (T, top) or z.stride(1) != 1:
        raise KernelError("route_groups: z float32 [T, E], idx int32 [T, top], wts float32 [T, top]")
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != E or not correction.is_contiguous()):
        raise KernelError("route_groups: correction must be float32 [E]")
    if groups < 1 or E % groups or not 1 <= keep <= groups or group_top < 1 or top > keep * (E // groups):
        raise KernelError(f"route_groups: {E} experts in {groups} groups, {keep} kept, top {top}")
    _ints(idx, "idx"); _contig(wts, "wts")
    _check(core().tl_route_groups(_ptr(z), z.stride(0), _ptr(correction), E, int(top), int(groups), int(keep), int(group_top),
                                  int(bool(softmax)), float(scale), _ptr(idx), _ptr(wts), T, _stream()), "route_groups")


def moe_up(h: torch.Tensor, w_up: torch.Tensor, idx: torch.Tensor, a: torch.Tensor, act="relu_squared",
           gated: bool = False, in_scale: torch.Tensor | None = None) -> None:
    """a[t * top + j, :] = act(s w_up[idx[t, j]] h[t]); w_up [E, F, K], a [T * top, F] of h's type; s = in_scale[t, j]
    (float32 [T, top]: the weight on the expert's input) or 1.  `gated`: w_up is [E, 2F, K], an expert's gate rows then its up
    rows, and a = act(s gate) * (s up).  An entry idx >= E has no matrices (an identity entry): its rows of a are left alone."""
    T, K = h.shape
    top = idx.shape[1]
    F = a.shape[1]
    if w_up.dim() != 3 or w_up.shape[1:] != ((2 * F if gated else F), K) or a.shape != (T * top, F) or a.dtype != h.dtype:
        raise KernelError("moe_up: w_up [E, F, K] ([E, 2F, K] gated), a [T top, F] of h's type")
    code, limit, alpha = gate_act(act)
    if in_scale is not None and (in_scale.dtype != torch.float32 or in_scale.shape != idx.shape or not in_scale.is_contiguous()):
        raise KernelError("moe_up: in_scale must be float32 [T, top]")
    _contig(h, "h"); _contig(w_up, "w_up"); _ints(idx, "idx"); _contig(a, "a")
    _check(core().tl_moe_up(_ptr(h), dtype_code(h.dtype), _ptr(w_up), dtype_code(w_up.dtype), _ptr(idx), _ptr(a), T * top, K, F,
                            top, int(gated), code, _ptr(in_scale), limit, alpha, w_up.shape[0], _stream()), "moe_up")


def _extra(extra, gate, y, who):
    """(pointer of the gate's first element, its row stride) of an addend `sigmoid(gate[t]) * extra[t]`."""
    if extra is None:
        if gate is not None:
            raise KernelError(f"{who}: a gate comes with an addend")
        return None, 0
    if extra.shape != y.shape or extra.dtype != y.dtype or not extra.is_contiguous():
        raise KernelError(f"{who}: the addend must have y's shape and type")
    if gate is None:
        return None, 0
    if gate.dtype != torch.float32 or gate.dim() != 1 or gate.numel() != y.shape[0]:
        raise KernelError(f"{who}: the gate must be float32, one number a token (a column of a wider tensor may be passed)")
    return _ptr(gate), gate.stride(0)


def moe_down(a: torch.Tensor, w_down: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor | None, y: torch.Tensor,
             extra: torch.Tensor | None = None, extra_gate: torch.Tensor | None = None, same: torch.Tensor | None = None) -> None:
    """y[t] = sum_j wts[t, j] * w_down[idx[t, j]] a[t * top + j] (+ sigmoid(extra_gate[t]) * extra[t]); w_down [E, N, F];
    wts None: an unweighted sum.  `same` ([T, N] of y's type): an entry idx >= E is an identity entry whose product is same[t]."""
    T, top = idx.shape
    E, N, F = w_down.shape
    if same is not None and (same.shape != y.shape or same.dtype != y.dtype or not same.is_contiguous()):
        raise KernelError("moe_down: the identity entries' rows must have y's shape and type")
    if a.shape != (T * top, F) or y.shape != (T, N) or y.dtype != a.dtype or \
            (wts is not None and (wts.dtype != torch.float32 or wts.shape != idx.shape or not wts.is_contiguous())):
        raise KernelError("moe_down: a [T top, F], w_down [E, N, F], y [T, N], wts float32 [T, top]")
    _contig(a, "a"); _contig(w_down, "w_down"); _ints(idx, "idx"); _contig(y, "y")
    g_ptr, ldg = _extra(extra, extra_gate, y, "moe_down")
    _check(core().tl_moe_down(_ptr(a), dtype_code(a.dtype), _ptr(w_down), dtype_code(w_down.dtype), _ptr(idx), _ptr(wts), _ptr(y),
                              T, F, N, top, _ptr(extra), g_ptr, ldg, E if same is not None else (1 << 30), _ptr(same), _stream()),
           "moe_down")


def moe_sort(idx: torch.Tensor, E: int):
    """Pairs (token, chosen expert) sorted by expert: (offsets int32 [E + 1], place_of int32 [P], pair_at int32 [P])."""
    P = idx.numel()
    _ints(idx, "idx")
    offsets = torch.empty(E + 1, dtype=torch.int32, device=idx.device)
    place_of = torch.empty(P, dtype=torch.int32, device=idx.device)
    pair_at = torch.empty(P, dtype=torch.int32, device=idx.device)
    _check(core().tl_moe_sort(_ptr(idx), P, E, _ptr(offsets), _ptr(place_of), _ptr(pair_at), _stream()), "moe_sort")
    return offsets, place_of, pair_at


def moe_gather(h: torch.Tensor, pair_at: torch.Tensor, idx: torch.Tensor, offsets: torch.Tensor, top: int, rows: torch.Tensor,
               cap: int = 0, scale: torch.Tensor | None = None) -> None:
    """rows[row of place] = h[pair_at[place] // top].  cap 0: row = place (rows [P, K], the experts' runs one behind the
    other); cap > 0: every expert has cap rows of its own (rows [E * cap, K], row = expert * cap + place - offsets[expert];
    the rows behind a run are set to zero)."""
    P, K = pair_at.numel(), rows.shape[1]
    E = offsets.numel() - 1
    if h.shape[1] != K or rows.dtype != h.dtype or rows.shape[0] != (E * cap if cap else P) or idx.numel() != P:
        raise KernelError("moe_gather: rows [P, K] (or [E cap, K]) of h's type")
    _contig(h, "h"); _contig(rows, "rows"); _ints(pair_at, "pair_at"); _ints(idx, "idx"); _ints(offsets, "offsets")
    if scale is not None and (scale.dtype != torch.float32 or scale.numel() != P or not scale.is_contiguous()):
        raise KernelError("moe_gather: scale must be float32, one number a pair (rows = scale * h)")
    _check(core().tl_moe_gather(_ptr(h), dtype_code(h.dtype), _ptr(pair_at), _ptr(idx), _ptr(offsets), int(cap), _ptr(rows), P, E, K,
                                int(top), _ptr(scale), _stream()), "moe_gather")


def relu_square(u: torch.Tensor) -> None:
    """u = relu(u)^2 in place."""
    _contig(u, "u")
    _check(core().tl_relu_square(_ptr(u), dtype_code(u.dtype), u.numel(), _stream()), "relu_square")


def moe_combine(rows: torch.Tensor, place_of: torch.Tensor, idx: torch.Tensor, offsets: torch.Tensor, wts: torch.Tensor | None,
                y: torch.Tensor, cap: int = 0, extra: torch.Tensor | None = None, extra_gate: torch.Tensor | None = None) -> None:
    """y[t] = sum_j wts[t, j] * rows[row of place_of[t * top + j]] (+ sigmoid(extra_gate[t]) * extra[t]); rows laid out as
    `moe_gather` lays them out; wts None: an unweighted sum."""
    T, top = idx.shape
    N = y.shape[1]
    E = offsets.numel() - 1
    if rows.shape != ((E * cap if cap else T * top), N) or rows.dtype != y.dtype or y.shape[0] != T or \
            (wts is not None and (wts.dtype != torch.float32 or wts.shape != idx.shape or not wts.is_contiguous())):
        raise KernelError("moe_combine: rows [T top, N] (or [E cap, N]) of y's type, wts float32 [T, top]")
    _contig(rows, "rows"); _ints(place_of, "place_of"); _ints(idx, "idx"); _ints(offsets, "offsets"); _contig(y, "y")
    g_ptr, ldg = _extra(extra, extra_gate, y, "moe_combine")
    _check(core().tl_moe_combine(_ptr(rows), dtype_code(rows.dtype), _ptr(place_of), _ptr(idx), _ptr(offsets), int(cap), _ptr(wts),
                                 _ptr(y), T, N, top, _ptr(extra), g_ptr, ldg, _stream()), "moe_combine")


# ---------------------------------------------------------------------------------------------
# The gated delta rule (csrc/delta.cu)

def delta_state_floats(d: int, compensated: bool = False) -> int:
    """Floats of state that `delta_scan` keeps per (head, slice of `delta_columns()` value columns) for heads of d rows; twice
    as many when every element is a pair of floats (`compensated`)."""
    n = core().tl_delta_state_floats(int(d), int(compensated))
    if n <= 0:
        raise KernelError(f"delta_scan: heads of {d} rows are not supported (at most 256)")
    return n


def delta_columns() -> int:
    return core().tl_delta_columns()


def conv_prep(proj: torch.Tensor, taps_w: torch.Tensor, conv_state: torch.Tensor | None, q_start: torch.Tensor,
              slots: torch.Tensor, out: torch.Tensor, *, B: int, max_q_len: int, nqk: int, d: int, nv: int, dv: int,
              unit_eps: float, q_scale: float) -> None:
    """The first C = 2 nqk d + nv dv columns of `proj` (q heads, k heads, v heads) through a causal convolution over time
    per channel (taps_w [C, taps], the last tap on the current token; the taps - 1 inputs before the step come from
    `conv_state[slot]`, float32 [taps - 1, C], which is then brought up to date) and silu; every q and k head scaled to
    unit length, x / sqrt(sum x^2 + unit_eps), q also by q_scale.  out float32 [T, C]."""
    T = proj.shape[0]
    C = 2 * nqk * d + nv * dv
    taps = taps_w.shape[1]
    if taps_w.shape != (C, taps) or proj.shape[1] < C or proj.stride(1) != 1 or out.shape != (T, C) or out.dtype != torch.float32:
        raise KernelError("conv_prep: proj [T, >= C], taps_w [C, taps], out float32 [T, C]")
    _contig(taps_w, "taps_w"); _contig(out, "out"); _ints(q_start, "q_start"); _ints(slots, "slots")
    slot_stride = 0
    if taps > 1:
        if conv_state is None or conv_state.dtype != torch.float32 or not conv_state.is_contiguous() or \
                conv_state[0].numel() != (taps - 1) * C:
            raise KernelError("conv_prep: conv_state must be float32 [slots, (taps - 1) * C]")
        slot_stride = conv_state[0].numel()
    _check(core().tl_conv_prep(_ptr(proj), dtype_code(proj.dtype), proj.stride(0), _ptr(taps_w), dtype_code(taps_w.dtype), taps,
                               _ptr(conv_state) if taps > 1 else None, slot_stride, _ptr(q_start), _ptr(slots), _ptr(out), int(B),
                               int(max_q_len), nqk, d, nv, dv, float(unit_eps), float(q_scale), _stream()), "conv_prep",
           launches=2 if taps > 1 else 1)


def delta_scan(qkv: torch.Tensor, gates: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor,
               q_start: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, *, B: int, H: int, nqk: int, d: int, dv: int,
               max_q_len: int | None = None, compensated: bool = False) -> None:
    """Per (request, head), tokens in order: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q, with
    beta = sigmoid(gates[t, h]) and g = exp(-exp(A_log[h]) softplus(gates[t, H + h] + dt_bias[h])).  qkv float32 [T, C] as
    `conv_prep` leaves it (q [nqk, d], k [nqk, d], v [H, dv]; head h reads q/k head h // (H / nqk)); the state is read from
    and left in `state[slot]` (float32, `delta_state_floats` per head and column slice); out float32 [T, H dv].  `max_q_len`: the most tokens a request brings
    (None: as many as the step has); it only picks between two forms of the kernel that give the same bits.  `compensated`:
    every state element is a pair of floats whose second gathers what the roundings of the first lose (the decay and the write as
    error-free steps): the state then stays at the accuracy of the sums that feed it however many tokens it has seen."""
    T = qkv.shape[0]
    C = 2 * nqk * d + H * dv
    if qkv.dtype != torch.float32 or qkv.shape != (T, C) or out.dtype != torch.float32 or out.shape != (T, H * dv):
        raise KernelError("delta_scan: qkv float32 [T, 2 nqk d + H dv], out float32 [T, H dv]")
    if gates.dtype != torch.float32 or gates.shape[0] != T or gates.shape[1] < 2 * H or gates.stride(1) != 1:
        raise KernelError("delta_scan: gates must be float32 [T, >= 2H]")
    for name, t in (("A_log", A_log), ("dt_bias", dt_bias)):
        if t.dtype != torch.float32 or t.numel() != H or not t.is_contiguous():
            raise KernelError(f"delta_scan: {name} must be float32 [H]")
    _contig(qkv, "qkv"); _contig(out, "out"); _contig(state, "state"); _ints(q_start, "q_start"); _ints(slots, "slots")
    per_slot = H * -(-dv // delta_columns()) * delta_state_floats(d, compensated)
    if state.dtype != torch.float32 or state[0].numel() != per_slot:
        raise KernelError(f"delta_scan: a slot holds {state[0].numel()} floats, these sizes need {per_slot}")
    _check(core().tl_delta_scan(_ptr(qkv), C, 0, nqk * d, 2 * nqk * d, _ptr(gates), gates.stride(0), _ptr(A_log), _ptr(dt_bias),
                                _ptr(state), per_slot, _ptr(q_start), _ptr(slots), _ptr(out), int(B), H, nqk, d, dv,
                                int(T if max_q_len is None else max_q_len), int(compensated), _stream()),
           "delta_scan")


# ---------------------------------------------------------------------------------------------
# Attention through a latent (csrc/latent.cu)

def latent_prep(down: torch.Tensor, qr: int, rank: int, dr: int, wq: torch.Tensor, wkv: torch.Tensor, eps: float,
                inv_freq: torch.Tensor, rot: int, pos: torch.Tensor, req_slot: torch.Tensor, table: torch.Tensor, page_size: int,
                cq: torch.Tensor | None, k_pages: torch.Tensor, write_kv: bool = True, pairing: str = "half") -> None:
    """Per token, from down float32 [T, qr + rank + dr (+ more)]: cq = the first qr columns RMS-normalised times wq; into the
    token's place in k_pages [pages, 1, page, d]: the next `rank` columns RMS-normalised times wkv, then the next dr columns
    with their first `rot` rotated by position (pairs (i, i + rot/2), or (2i, 2i + 1) with `pairing` "interleaved"), then zeros
    up to d.  qr 0 (cq and wq None): there is no query latent; columns behind the first qr + rank + dr are not read."""
    T = down.shape[0]
    d = k_pages.shape[-1]
    if down.dtype != torch.float32 or down.dim() != 2 or down.shape[1] < qr + rank + dr or down.stride(1) != 1:
        raise KernelError("latent_prep: down float32 [T, qr + rank + dr or more]")
    if qr == 0:
        if cq is not None or wq is not None:
            raise KernelError("latent_prep: without a query latent there is neither cq nor wq")
    elif cq.shape != (T, qr) or cq.dtype != k_pages.dtype or wq.numel() != qr or wq.dtype != wkv.dtype:
        raise KernelError("latent_prep: cq [T, qr] of the pages' type, wq [qr] of wkv's type")
    if tuple(k_pages.shape[1:3]) != (1, page_size) or rank + dr > d:
        raise KernelError("latent_prep: k_pages must be [pages, 1, page, d >= rank + dr]")
    if wkv.numel() != rank:
        raise KernelError("latent_prep: the latent's norm weight must be [rank]")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != rot // 2:
        raise KernelError("latent_prep: inv_freq must be float32 [rot/2]")
    _contig(k_pages, "k_pages"); _contig(wkv, "wkv")
    if qr:
        _contig(cq, "cq"); _contig(wq, "wq")
    _ints(pos, "pos"); _ints(req_slot, "req_slot"); _ints(table, "table")
    _check(core().tl_latent_prep(_ptr(down), down.stride(0), qr, rank, dr, _ptr(wq), _ptr(wkv), dtype_code(wkv.dtype), float(eps),
                                 _ptr(inv_freq), int(rot), _ptr(pos), _ptr(req_slot), _ptr(table), table.shape[1], page_size,
                                 _ptr(cq), _ptr(k_pages), dtype_code(k_pages.dtype), d, int(write_kv), T,
                                 int(_pairing(pairing, "latent_prep")), table.shape[0], k_pages.shape[0],
                                 fault_words(down.device), _stream()), "latent_prep")


def _pairing(pairing: str, who: str) -> bool:
    if pairing not in ("half", "interleaved"):
        raise KernelError(f"{who}: pairing {pairing!r} is neither 'half' nor 'interleaved'")
    return pairing == "interleaved"


def latent_qrot(q: torch.Tensor, dk: int, dr: int, inv_freq: torch.Tensor, rot: int, pos: torch.Tensor, qa: torch.Tensor,
                rank: int, H: int, pairing: str = "half") -> None:
    """qa[t, h, rank : rank + dr] = q[t, h, dk : dk + dr] with its first `rot` dimensions rotated by position; the columns of
    qa behind them are set to zero.  q [T, H (dk + dr)], qa [T, H d]."""
    T = q.shape[0]
    d = qa.shape[1] // H
    if q.shape != (T, H * (dk + dr)) or qa.shape != (T, H * d) or qa.dtype != q.dtype or rank + dr > d:
        raise KernelError("latent_qrot: q [T, H (dk + dr)], qa [T, H d] of one type, d >= rank + dr")
    _contig(q, "q"); _contig(qa, "qa"); _ints(pos, "pos")
    _check(core().tl_latent_qrot(_ptr(q), dk, dr, _ptr(inv_freq), int(rot), _ptr(pos), _ptr(qa), rank, d, H, T, dtype_code(q.dtype),
                                 int(_pairing(pairing, "latent_qrot")), _stream()), "latent_qrot")


def head_matmul(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, H: int, K: int, N: int, x_head_stride: int,
                y_head_stride: int) -> None:
    """y[t, h, :N] = x[t, h, :K] w[h]; w [H, K, N]; head h of row t starts at x[t, h * x_head_stride] (y alike); float sums."""
    T = x.shape[0]
    if w.shape != (H, K, N) or x.dtype != y.dtype or y.shape[0] != T or x.stride(1) != 1 or y.stride(1) != 1:
        raise KernelError("head_matmul: w [H, K, N], x and y of one type with unit inner stride")
    if (H - 1) * x_head_stride + K > x.shape[1] or (H - 1) * y_head_stride + N > y.shape[1]:
        raise KernelError("head_matmul: the heads do not lie inside the rows")
    _contig(w, "w")
    _check(core().tl_head_matmul(_ptr(x), x.stride(0), x_head_stride, _ptr(w), dtype_code(w.dtype), _ptr(y), y.stride(0),
                                 y_head_stride, T, H, K, N, dtype_code(x.dtype), _stream()), "head_matmul")


# ---------------------------------------------------------------------------------------------
# The real-gated linear recurrent unit and its short convolution (csrc/rglru.cu)

def causal_conv(proj: torch.Tensor, off: int, in_bias: torch.Tensor | None, W: int, taps_w: torch.Tensor, out_bias: torch.Tensor | None,
                conv_state: torch.Tensor | None, q_start: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, *, B: int,
                max_q_len: int) -> None:
    """out[t, c] = out_bias[c] + sum_k taps_w[c, k] x[t - (taps - 1) + k, c] with x = proj[:, off + c] + in_bias[off + c], a causal
    convolution over a request's tokens per channel (the last tap on the current token).  The taps - 1 inputs before the
    step come from `conv_state[slot]` (float32 [taps - 1, W], zero for a new request), which is then brought up to date.
    proj float32 [T, >= off + W], taps_w float32 [W, taps], out float32 [T, W]."""
    T = proj.shape[0]
    taps = taps_w.shape[1]
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or proj.shape[1] < off + W or out.shape != (T, W) or out.dtype != torch.float32:
        raise KernelError("causal_conv: proj float32 [T, >= off + W], out float32 [T, W]")
    if taps_w.shape != (W, taps) or taps_w.dtype != torch.float32:
        raise KernelError("causal_conv: taps_w must be float32 [W, taps]")
    for name, t, n in (("in_bias", in_bias, off + W), ("out_bias", out_bias, W)):
        if t is not None and (t.dtype != torch.float32 or t.numel() < n or not t.is_contiguous()):
            raise KernelError(f"causal_conv: {name} must be float32 with {n} entries")
    _contig(taps_w, "taps_w"); _contig(out, "out"); _ints(q_start, "q_start"); _ints(slots, "slots")
    slot_stride = 0
    if taps > 1:
        if conv_state is None or conv_state.dtype != torch.float32 or not conv_state.is_contiguous() or \
                conv_state[0].numel() != (taps - 1) * W:
            raise KernelError("causal_conv: conv_state must be float32 [slots, (taps - 1) * W]")
        slot_stride = conv_state[0].numel()
    _check(core().tl_causal_conv(_ptr(proj), proj.stride(0), int(off), _ptr(in_bias), _ptr(taps_w), _ptr(out_bias), taps,
                                 _ptr(conv_state) if taps > 1 else None, slot_stride, _ptr(q_start), _ptr(slots), _ptr(out), int(B),
                                 int(max_q_len), int(W), _stream()), "causal_conv", launches=2 if taps > 1 else 1)


def rglru_scan(gates: torch.Tensor, gate_bias: torch.Tensor, u: torch.Tensor, proj: torch.Tensor, in_bias: torch.Tensor | None,
               lam: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, *, B: int,
               blocks: int, sharpness: float, max_q_len: int, y_off: int = 0, in_order: bool = False, by_block: bool = False) -> None:
    """Per (request, channel c), tokens in order, from the state in `state[slot]` (float32 [W], left up to date):
    r = sigmoid(zr + br), i = sigmoid(zi + bi), log a = -sharpness r softplus(lam[c]), S <- exp(log a) S + sqrt(1 - a^2) i u[t, c],
    out[t, c] = S gelu_tanh(proj[t, y_off + c] + in_bias[y_off + c]).  gates float32 [T, 2W]: for each of the `blocks` equal
    parts of the channels its r pre-activations, then its i pre-activations (with `by_block`: [blocks, T, 2W / blocks], what a
    batched product leaves); gate_bias float32 [2W] laid out as a row of the former.
    A step with a request of two chunks of tokens or more (`rglru_chunk()`) runs its chunks side by side: per chunk the
    product of its decays and the state it reaches from zero, the chunks' starting states from these in order, then every
    chunk's tokens from its starting state.  A chunk's starting state is summed in another order than token by token, so it
    differs by roundings of float; `in_order` keeps every step in the one order (the float32 engine, whose results do not
    depend on how a prompt was cut, asks for it)."""
    T, W = u.shape
    if gates.numel() != 2 * T * W or gates.dtype != torch.float32 or u.dtype != torch.float32 or out.shape != (T, W) or W % blocks or \
            gates.shape != ((blocks, T, 2 * W // blocks) if by_block else (T, 2 * W)):
        raise KernelError("rglru_scan: gates float32 [T, 2W] or [blocks, T, 2W / blocks], u float32 [T, W], out [T, W]")
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or proj.shape[1] < y_off + W or proj.shape[0] != T:
        raise KernelError("rglru_scan: proj float32 [T, >= y_off + W]")
    if W % blocks or gate_bias.numel() != 2 * W or gate_bias.dtype != torch.float32 or lam.numel() != W or lam.dtype != torch.float32:
        raise KernelError("rglru_scan: gate_bias float32 [2W], lam float32 [W], W a multiple of blocks")
    if in_bias is not None and (in_bias.dtype != torch.float32 or in_bias.numel() < y_off + W):
        raise KernelError("rglru_scan: in_bias must be float32 with y_off + W entries")
    if state.dtype != torch.float32 or state[0].numel() != W:
        raise KernelError("rglru_scan: a slot holds W floats")
    _contig(gates, "gates"); _contig(gate_bias, "gate_bias"); _contig(u, "u"); _contig(lam, "lam"); _contig(state, "state")
    _contig(out, "out"); _ints(q_start, "q_start"); _ints(slots, "slots")
    summary, chunks, bw = None, 0, W // blocks
    if not in_order and max_q_len >= 2 * rglru_chunk():
        chunks = -(-int(max_q_len) // rglru_chunk())
        summary = torch.empty((int(B), chunks, 2, W), dtype=torch.float32, device=u.device)
    _check(core().tl_rglru_scan(_ptr(gates), _ptr(gate_bias), _ptr(u), _ptr(proj), proj.stride(0), int(y_off), _ptr(in_bias), _ptr(lam),
                                _ptr(state), _ptr(q_start), _ptr(slots), _ptr(out), dtype_code(out.dtype), int(B), W, int(blocks),
                                float(sharpness), int(max_q_len), _ptr(summary), chunks, T * 2 * bw if by_block else 2 * bw,
                                2 * bw if by_block else 2 * W, _stream()), "rglru_scan")


def split3(x: torch.Tensor, blocks: int) -> torch.Tensor:
    """A float32 [T, W] as bfloat16 [blocks, T, 3 * (W / blocks)]: per block of channels the leading, the middle and the last
    part of every float, three bfloat16 numbers that sum to it to within one part in 2^24.  Its batched product with
    bfloat16 weights stacked three times, summed in float32 on the tensor cores, is as exact as a float32 product."""
    T, W = x.shape
    if x.dtype != torch.float32 or W % blocks:
        raise KernelError("split3: float32 [T, W], W a multiple of blocks")
    _contig(x, "x")
    parts = torch.empty((blocks, T, 3 * (W // blocks)), dtype=torch.bfloat16, device=x.device)
    _check(core().tl_split3(_ptr(x), _ptr(parts), T, W, int(blocks), _stream()), "split3")
    return parts


_RGLRU_CHUNK = None


def rglru_chunk() -> int:
    """Tokens of one chunk of a long step of `rglru_scan`."""
    global _RGLRU_CHUNK
    if _RGLRU_CHUNK is None:
        _RGLRU_CHUNK = int(core().tl_rglru_chunk())
    return _RGLRU_CHUNK
