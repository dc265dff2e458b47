"""The engine's device operations.

Every function here launches hand-written sm_100a kernels from ``csrc/``
through the C entry points of ``libst_b200.so`` (loaded with ctypes; built on
first use by ``ops.build``), on torch's current CUDA stream, on tensors the
caller owns.  The only library calls are the bfloat16 matrix products, which
go to cuBLAS through ``torch`` (the reference uses cuBLAS for the same five
products, src/csrc/util/cublas_wrapper.cc:29-53).

There is no CPU path: a tensor that is not on a CUDA device is an error, and
so is a missing or unbuildable library.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import build as _build

_LIB = None

ACT_CODES = {"none": 0, "relu": 1, "gelu": 2, "gelu_tanh": 3, "silu": 4}
NORM_CODES = {"layernorm": 0, "rmsnorm": 1, "none": 2}

_ERRORS = {-1: "unsupported dtype", -2: "unsupported size", -3: "size beyond the kernel's limit",
           -4: "invalid argument"}


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """The loaded kernel library (built on first use)."""
    global _LIB
    if _LIB is None:
        path = _build.ensure_built()
        try:
            _LIB = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load {path}: {e}") from None
        _LIB.st_attention_decode_scratch_floats.restype = ctypes.c_longlong
        _LIB.st_latent_attention_mma_scratch.restype = ctypes.c_longlong
        _LIB.st_uniform_host.restype = ctypes.c_float
        _LIB.st_uniform_host.argtypes = [ctypes.c_longlong, ctypes.c_longlong]
    return _LIB


def library_path() -> str:
    return _build.ensure_built()


_LAUNCHES = 0


def launch_count() -> int:
    """How many kernel launchers of this library have been called so far (recorded launches count once)."""
    return _LAUNCHES


def _check(rc: int, what: str) -> None:
    global _LAUNCHES
    _LAUNCHES += 1
    if rc == 0:
        return
    if rc < 0:
        raise KernelError(f"{what}: refused ({_ERRORS.get(rc, rc)})")
    raise KernelError(f"{what}: CUDA error {rc} at launch")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"unsupported tensor type {t.dtype} (float32 or bfloat16)")


def _p(t: Optional[torch.Tensor]):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("this engine runs on a CUDA device only; got a CPU tensor")
    return ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream of the current device as a handle for the library.  torch.cuda.current_stream()
    costs ~15 us of host time per call (a fifth of the host's time for a step of eager launches); the raw
    query behind it is used where this torch has it."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _f(x: float):
    return ctypes.c_float(x)


_SM_COUNT = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of a CUDA device (the current one by default); asked once per device."""
    index = device.index if isinstance(device, torch.device) and device.index is not None \
        else torch.cuda.current_device()
    if index not in _SM_COUNT:
        _SM_COUNT[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return _SM_COUNT[index]


# ------------------------------------------------------------------ embedding
def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, positions: Optional[torch.Tensor] = None,
          pos_table: Optional[torch.Tensor] = None, pos_offset: int = 0, scale: float = 1.0) -> torch.Tensor:
    """out[t] = scale * table[ids[t]] (+ pos_table[positions[t] + pos_offset]); out is float32 or table's type."""
    n, width = ids.numel(), table.shape[1]
    assert out.shape == (n, width) and out.is_contiguous() and table.is_contiguous()
    if pos_table is not None:
        assert pos_table.shape[1] == width and pos_table.dtype == table.dtype
    _check(lib().st_embed(_p(ids), _p(table), n, width, _p(positions) if pos_table is not None else None,
                          _p(pos_table), pos_offset, _p(out), _dt(table), int(out.dtype == torch.float32),
                          _f(scale), _stream()), "embed")
    return out


def add_positions(x: torch.Tensor, positions: torch.Tensor, pos_table: torch.Tensor, pos_offset: int,
                  out: torch.Tensor) -> torch.Tensor:
    """out[t] = x[t] + pos_table[positions[t] + pos_offset]."""
    n, width = x.shape
    assert pos_table.shape[1] == width and x.dtype == pos_table.dtype and out.shape == x.shape
    _check(lib().st_add_positions(_p(x), n, width, _p(positions), _p(pos_table), pos_offset, _p(out),
                                  _dt(x), int(out.dtype == torch.float32), _stream()), "add_positions")
    return out


# ------------------------------------------------------------ residual + norm
def add_norm(x: torch.Tensor, *, delta: Optional[torch.Tensor] = None, delta_bias: Optional[torch.Tensor] = None,
             resid_out: Optional[torch.Tensor] = None, gamma: Optional[torch.Tensor] = None,
             beta: Optional[torch.Tensor] = None, eps: float = 1e-5, kind: str = "layernorm",
             rows: Optional[torch.Tensor] = None, out_act: Optional[torch.Tensor] = None,
             out_f32: Optional[torch.Tensor] = None, act_dtype: Optional[torch.dtype] = None,
             parts: Optional[torch.Tensor] = None) -> None:
    """s = x[i] + (delta[i] + parts[0][i] + parts[1][i] + ...) + delta_bias; resid_out[i] = s; y = norm(s);
    out_act[r] = y; out_f32[r] = y.

    ``x`` is the float32 residual stream; ``i = rows[r]`` when ``rows`` is given, else ``r``.  ``parts``: float32
    [n, rows of x, width], further addends (the slices of k of a product, see ``linear_parts``).
    """
    assert x.dtype == torch.float32 and x.is_contiguous()
    if parts is not None:
        assert parts.dtype == torch.float32 and parts.dim() == 3 and parts.shape[1:] == x.shape
        assert parts.stride(2) == 1 and parts.stride(1) == x.shape[1]
    width = x.shape[1]
    n = rows.numel() if rows is not None else x.shape[0]
    if out_act is not None:
        code = _dt(out_act)
    elif delta is not None:
        code = _dt(delta)
    else:
        code = 0 if act_dtype in (None, torch.float32) else 1
    if delta is not None and out_act is not None:
        assert delta.dtype == out_act.dtype
    _check(lib().st_add_norm(_p(x), _p(rows), _p(delta), _p(delta_bias), _p(parts),
                             parts.shape[0] if parts is not None else 0,
                             ctypes.c_longlong(parts.stride(0) if parts is not None else 0), _p(resid_out), _p(gamma), _p(beta),
                             _f(eps), NORM_CODES[kind], n, width, _p(out_act), _p(out_f32), code, _stream()),
           "add_norm")


def bias_act(y: torch.Tensor, bias: Optional[torch.Tensor], act: str) -> torch.Tensor:
    """y = act(y + bias) in place."""
    if bias is None and act == "none":
        return y
    assert y.is_contiguous()
    _check(lib().st_bias_act(_p(y), _p(bias), ACT_CODES[act], y.shape[0], y.shape[1], _dt(y), _stream()), "bias_act")
    return y


def scatter_i32(dst: torch.Tensor, idx: torch.Tensor, val: torch.Tensor, count: torch.Tensor, max_count: int) -> None:
    """dst.flatten()[idx[i]] = val[i] for i < count[0] (count lives on the device)."""
    _check(lib().st_scatter_i32(_p(dst), _p(idx), _p(val), _p(count), max_count, _stream()), "scatter_i32")


def gather_where_i32(dst: torch.Tensor, src_index: torch.Tensor, src: torch.Tensor) -> None:
    """dst[i] = src[src_index[i]] wherever src_index[i] >= 0 (int32 tensors on the device)."""
    assert dst.dtype == src.dtype == src_index.dtype == torch.int32 and dst.numel() == src_index.numel()
    _check(lib().st_gather_where_i32(_p(dst), _p(src_index), _p(src), dst.numel(), src.numel(), _stream()),
           "gather_where_i32")


# ------------------------------------------------------------ matrix products
_tc_status = {}


def _tc_status_word(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key not in _tc_status:
        _tc_status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_status[key]


def lossless_bf16(v: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """A bfloat16 copy of a float vector if every element survives the rounding unchanged, else None."""
    if v is None or v.dtype != torch.float32:
        return None
    low = v.to(torch.bfloat16)
    return low if bool(torch.equal(low.float(), v)) else None


_addmm_activation = getattr(torch, "_addmm_activation", None)    # the library product with bias and ReLU in its epilogue


def linear(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
           out_dtype: Optional[torch.dtype] = None, bias_bf16: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(a @ w.T + bias); w is [out, in].  float32: the plain fused-multiply-add kernel (true 32-bit).
    bfloat16, few rows: the weight-streaming kernel.  bfloat16, more rows: the library product with float
    accumulation; bias and ReLU ride in its epilogue when ``bias_bf16`` (a lossless bfloat16 copy of
    ``bias``, see lossless_bf16) is given, else the bias/activation kernel follows."""
    assert a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1] and a.dtype == w.dtype
    out_dtype = out_dtype or a.dtype
    n, m = a.shape[0], w.shape[0]
    if a.dtype == torch.float32:
        return gemm_plain(a, w, bias, act, out_dtype)
    if not a.is_cuda:
        raise KernelError("this engine runs on a CUDA device only; got a CPU tensor")
    if n == 0:
        return torch.empty((0, m), dtype=out_dtype, device=a.device)
    if n <= SKINNY_MAX_ROWS and a.shape[1] % 8 == 0:
        return gemm_skinny(a, w, bias, act, out_dtype)
    if stream_tc_applies(n, w):
        return gemm_stream_tc(a, w, bias, act, out_dtype)
    if out_dtype == torch.float32:
        y = torch.mm(a, w.t(), out_dtype=torch.float32)
    elif bias_bf16 is not None and (act == "none" or (act == "relu" and _addmm_activation is not None)):
        if act == "relu":
            return _addmm_activation(bias_bf16, a, w.t(), use_gelu=False)
        return torch.addmm(bias_bf16, a, w.t())
    else:
        y = torch.mm(a, w.t())
    return bias_act(y, bias, act)


# Up to this many tokens the weight-streaming kernel serves bfloat16 products.  The kernel itself takes up
# to 32 rows; from 9 rows on the library product is ahead (at 16 rows: on four of the model's five products).
SKINNY_MAX_ROWS = 8
SKINNY_KERNEL_MAX_ROWS = 32


# Up to this many tokens (and above SKINNY_MAX_ROWS) the tcgen05 weight-streaming kernel serves the bfloat16
# products that it runs in one wave of blocks; 0: off, the library product takes over from SKINNY_MAX_ROWS + 1 on.
# Off: the library is ahead at every row count (OPT-1.3B decode step at batch 16 / 64: 1.42 / 2.33 ms against 1.77 /
# 2.93 with this kernel; per layer 34 against 44 microseconds at 16 tokens, 35 against 54 at 64).
STREAM_TC_MAX_ROWS = 0


def stream_tc_applies(n_rows: int, w: torch.Tensor) -> bool:
    """Whether ``linear`` / ``linear_parts`` give a product of n_rows tokens with w [out, in] to the tcgen05
    weight-streaming kernel: bfloat16 on the device, more tokens than the mma.sync kernel serves, an inner dimension
    that is a multiple of 64, and few enough features for one block per SM (the output head is not)."""
    return (w.is_cuda and w.dtype == torch.bfloat16 and SKINNY_MAX_ROWS < n_rows <= min(STREAM_TC_MAX_ROWS, 128)
            and w.shape[1] % 64 == 0 and bool(lib().st_gemm_stream_tc_one_wave(w.shape[0])))


def gemm_stream_tc(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
                   out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """act(a @ w.T + bias) for at most 128 rows of bfloat16 ``a`` on tcgen05 fed by TMA; w is [out, in] with
    in % 64 == 0.  A wait that expires inside the kernel shows in ``kernel_status``."""
    out_dtype = out_dtype or a.dtype
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_stream_tc is a bfloat16 kernel")
    a = a.contiguous()
    assert w.is_contiguous()
    n, k = a.shape
    m = w.shape[0]
    out = torch.empty((n, m), dtype=out_dtype, device=a.device)
    _check(lib().st_gemm_stream_tc(_p(a), _p(w), _p(bias), _p(out), n, m, k, ACT_CODES[act],
                                   int(out_dtype == torch.float32), _p(_tc_status_word(a.device)), _stream()),
           "gemm_stream_tc")
    return out


def kernel_status(device: torch.device) -> int:
    """The status word of kernels that have no step context to report to (0: fine; 5: the tcgen05 product
    gave up waiting); reading it synchronises and clears it."""
    word = _tc_status_word(torch.device(device))
    code = int(word.item())
    if code:
        word.zero_()
    return code


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """act(a @ w.T + bias) for at most SKINNY_KERNEL_MAX_ROWS rows of bfloat16 ``a``; w is [out, in] with in % 8 == 0."""
    out_dtype = out_dtype or a.dtype
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_skinny is a bfloat16 kernel")
    a = a.contiguous()
    assert w.is_contiguous()
    n, k = a.shape
    m = w.shape[0]
    out = torch.empty((n, m), dtype=out_dtype, device=a.device)
    _check(lib().st_gemm_skinny(_p(a), _p(w), _p(bias), _p(out), n, m, k, ACT_CODES[act],
                                int(out_dtype == torch.float32), _stream()), "gemm_skinny")
    return out


# ---- the same products with their neighbours fused (steps of a few tokens) ----
# The residual sum behind a product (out[m, n] += ..., in float, in the product's epilogue) is used: a decode
# step gains 4 %.  The norm in front of a product (five kernels per pre-norm layer instead of seven) is built
# and tested but off: measured in the recorded step it loses, at batch 8 by 10 %, because the small norm
# kernel between two products is what lets the second product start all at once on an idle GPU with its
# first loads already under way.  With a switch off, the operation runs as
# the separate kernels it replaces.
FUSED_MAX_ROWS = 8
FUSE_NORM = False
FUSE_RESIDUAL = True
LINEAR_PARTS = True       # a product cut over k leaves its slices' sums for the next norm kernel (decode steps)
UNCUT_MAX_INNER = 2048    # up to this inner dimension ``linear_add`` runs uncut with its weights on chip: no parts


def fused_norm_applies(n_rows: int, k: int, w: torch.Tensor) -> bool:
    """Whether ``norm_linear`` / ``norm_qkv_linear_to_cache`` / ``linear_add`` take a step of n_rows tokens
    with inner dimension k and weights w."""
    return (w.is_cuda and w.dtype == torch.bfloat16 and 1 <= n_rows <= min(FUSED_MAX_ROWS, SKINNY_MAX_ROWS)
            and bool(lib().st_gemm_skinny_norm_applies(n_rows, k)))


def norm_linear(x: torch.Tensor, kind: str, gamma: Optional[torch.Tensor], beta: Optional[torch.Tensor], eps: float,
                w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
                out_dtype: Optional[torch.dtype] = None, delta: Optional[torch.Tensor] = None,
                delta_bias: Optional[torch.Tensor] = None, parts: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(norm(x) @ w.T + bias) for at most FUSED_MAX_ROWS float32 rows x (the residual stream) and bfloat16
    w [out, in]: the norm of ``add_norm`` (statistics in float, two passes; its result rounded to bfloat16 as
    ``add_norm`` stores it) in front of the weight-streaming product, in one kernel.  ``delta`` / ``delta_bias`` /
    ``parts``: what is still to be added to x (``add_norm`` adds it, x is updated); only with FUSE_NORM off."""
    assert x.dtype == torch.float32 and x.is_contiguous() and w.is_contiguous() and x.shape[1] == w.shape[1]
    n, k = x.shape
    m = w.shape[0]
    out_dtype = out_dtype or w.dtype
    pending = delta is not None or delta_bias is not None or parts is not None
    assert not (FUSE_NORM and pending)
    if not FUSE_NORM:
        h = torch.empty((n, k), dtype=w.dtype, device=x.device)
        add_norm(x, delta=delta, delta_bias=delta_bias, parts=parts, resid_out=x if pending else None, gamma=gamma,
                 beta=beta, eps=eps, kind=kind, out_act=h)
        return gemm_skinny(h, w, bias, act, out_dtype)
    out = torch.empty((n, m), dtype=out_dtype, device=x.device)
    _check(lib().st_gemm_skinny_norm(_p(x), _p(gamma), _p(beta), _f(eps), NORM_CODES[kind], _p(w), _p(bias), _p(out),
                                     n, m, k, ACT_CODES[act], int(out_dtype == torch.float32), _stream()),
           "norm_linear")
    return out


def linear_add(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], x: torch.Tensor) -> None:
    """x += a @ w.T + bias in place, for at most FUSED_MAX_ROWS bfloat16 rows a and float32 x (the residual
    stream): the residual sum behind the weight-streaming product, in float, in one kernel."""
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dtype == torch.float32
    assert a.is_contiguous() and w.is_contiguous() and x.is_contiguous()
    assert a.shape[1] == w.shape[1] and x.shape == (a.shape[0], w.shape[0])
    if not FUSE_RESIDUAL:
        add_norm(x, delta=gemm_skinny(a, w), delta_bias=bias, resid_out=x, kind="none", act_dtype=a.dtype)
        return
    _check(lib().st_gemm_skinny_add(_p(a), _p(w), _p(bias), _p(x), a.shape[0], w.shape[0], a.shape[1], _stream()),
           "linear_add")


_parts_scratch = {}


def linear_parts_slices(n_rows: int, w: torch.Tensor) -> int:
    """Into how many slices of k ``linear_parts`` cuts a product with w [out, in] for n_rows tokens (1: it does not
    apply: more than FUSED_MAX_ROWS tokens, weights that are not bfloat16 on the device, an inner dimension that is
    no multiple of 32, or a product that is not cut)."""
    if not (LINEAR_PARTS and w.is_cuda and w.dtype == torch.bfloat16 and n_rows >= 1):
        return 1
    if n_rows <= FUSED_MAX_ROWS:
        return int(lib().st_gemm_skinny_parts_slices(w.shape[0], w.shape[1]))
    if stream_tc_applies(n_rows, w):
        return int(lib().st_gemm_stream_tc_slices(w.shape[0], w.shape[1]))
    return 1


def linear_parts(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """The slices' sums of a @ w.T for bfloat16 rows (as many as ``linear_parts_slices`` answers for with more than
    one slice): float32 [slices, rows, out], to be added in slice order (``add_norm(parts=...)`` does, in the kernel
    that reads the residual rows anyway).  Up to FUSED_MAX_ROWS rows the mma.sync kernel, beyond it the tcgen05
    kernel.  The result lives in a buffer that the next call for the same sizes overwrites."""
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.is_contiguous() and w.is_contiguous()
    assert a.shape[1] == w.shape[1]
    n, m = a.shape[0], w.shape[0]
    slices = linear_parts_slices(n, w)
    cap = FUSED_MAX_ROWS if n <= FUSED_MAX_ROWS else 128
    key = (a.device.index, slices, m, cap)
    if key not in _parts_scratch:
        _parts_scratch[key] = torch.zeros(slices * cap * m, dtype=torch.float32, device=a.device)
    parts = _parts_scratch[key][:slices * n * m].view(slices, n, m)
    if n <= FUSED_MAX_ROWS:
        _check(lib().st_gemm_skinny_parts(_p(a), _p(w), _p(parts), n, m, a.shape[1], _stream()), "linear_parts")
    else:
        _check(lib().st_gemm_stream_tc_parts(_p(a), _p(w), _p(parts), n, m, a.shape[1],
                                             _p(_tc_status_word(a.device)), _stream()), "linear_parts")
    return parts


def norm_qkv_linear_to_cache(x: torch.Tensor, kind: str, gamma: Optional[torch.Tensor], beta: Optional[torch.Tensor],
                             eps: float, w: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                             pool: torch.Tensor, layer: int, positions: torch.Tensor, seq_of_token: torch.Tensor,
                             slots: torch.Tensor, block_table: torch.Tensor, nh: int, nkv: int, d: int,
                             status: torch.Tensor, write_kv: bool = True, delta: Optional[torch.Tensor] = None,
                             delta_bias: Optional[torch.Tensor] = None, parts: Optional[torch.Tensor] = None) -> None:
    """``qkv_linear_to_cache`` of norm(x) for float32 rows x: norm, product, bias and cache write in one kernel.
    ``delta`` / ``delta_bias`` / ``parts``: as in ``norm_linear``."""
    assert x.dtype == torch.float32 and x.is_contiguous() and w.is_contiguous() and pool.dtype == torch.bfloat16
    num_pages, n_layers, _, pnkv, page_size, pd = pool.shape
    assert pnkv == nkv and pd == d and w.shape[0] == (nh + 2 * nkv) * d
    pending = delta is not None or delta_bias is not None or parts is not None
    assert not (FUSE_NORM and pending)
    if not FUSE_NORM:
        h = torch.empty(x.shape, dtype=w.dtype, device=x.device)
        add_norm(x, delta=delta, delta_bias=delta_bias, parts=parts, resid_out=x if pending else None, gamma=gamma,
                 beta=beta, eps=eps, kind=kind, out_act=h)
        return qkv_linear_to_cache(h, w, bias, q_out, pool, layer, positions, seq_of_token, slots, block_table, nh, nkv,
                                   d, status, write_kv)
    _check(lib().st_gemm_skinny_norm_qkv(_p(x), _p(gamma), _p(beta), _f(eps), NORM_CODES[kind], _p(w), _p(bias),
                                         _p(q_out), _p(pool), _p(positions), _p(seq_of_token), _p(slots),
                                         _p(block_table), block_table.shape[1], num_pages, n_layers, layer,
                                         x.shape[0], x.shape[1], nh, nkv, d, page_size, int(write_kv), _p(status),
                                         _stream()), "norm_qkv_linear_to_cache")


def qkv_linear_to_cache(h: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                        pool: torch.Tensor, layer: int, positions: torch.Tensor, seq_of_token: torch.Tensor,
                        slots: torch.Tensor, block_table: torch.Tensor, nh: int, nkv: int, d: int,
                        status: torch.Tensor, write_kv: bool = True) -> None:
    """The fused form of ``linear`` + ``qkv_to_cache`` for at most SKINNY_KERNEL_MAX_ROWS bfloat16 tokens:
    q_out = (h @ w.T + bias)[:, :nh*d]; the k and v parts go straight into the paged cache."""
    if h.dtype != torch.bfloat16 or pool.dtype != torch.bfloat16:
        raise KernelError("qkv_linear_to_cache is a bfloat16 kernel")
    num_pages, n_layers, _, pnkv, page_size, pd = pool.shape
    assert pnkv == nkv and pd == d and w.shape[0] == (nh + 2 * nkv) * d and h.is_contiguous() and w.is_contiguous()
    _check(lib().st_gemm_skinny_qkv(_p(h), _p(w), _p(bias), _p(q_out), _p(pool), _p(positions), _p(seq_of_token),
                                    _p(slots), _p(block_table), block_table.shape[1], num_pages, n_layers, layer,
                                    h.shape[0], h.shape[1], nh, nkv, d, page_size, int(write_kv), _p(status),
                                    _stream()), "qkv_linear_to_cache")


def gemm_plain(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
               out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """The plain kernel for either storage type (float arithmetic, fixed summation order)."""
    out_dtype = out_dtype or a.dtype
    a = a.contiguous()
    assert w.is_contiguous()
    n, k = a.shape
    m = w.shape[0]
    out = torch.empty((n, m), dtype=out_dtype, device=a.device)
    _check(lib().st_gemm_plain(_p(a), _p(w), _p(bias), _p(out), n, m, k, ACT_CODES[act], _dt(a),
                               int(out_dtype == torch.float32), _stream()), "gemm_plain")
    return out


# ------------------------------------------------------------------ attention
def qkv_to_cache(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_out: Optional[torch.Tensor], pool: torch.Tensor,
                 layer: int, positions: torch.Tensor, seq_of_token: torch.Tensor, slots: torch.Tensor,
                 block_table: torch.Tensor, nh: int, nkv: int, d: int, status: torch.Tensor,
                 write_kv: bool = True) -> None:
    """q_out = q + bias; pool[page, layer, 0/1, head, pos % page, :] = k/v + bias.  ``q_out`` None: the queries
    stay where they are (in ``qkv``), only keys and values move.

    pool: [pages, layers, 2, nkv, page_size, d]; block_table: [slots, max_pages] int32."""
    n = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * d and pool.dtype == qkv.dtype
    num_pages, n_layers, _, pnkv, page_size, pd = pool.shape
    assert pnkv == nkv and pd == d
    _check(lib().st_qkv_to_cache(_p(qkv), _p(bias), _p(q_out), _p(pool), _p(positions), _p(seq_of_token),
                                 _p(slots), _p(block_table), block_table.shape[1], num_pages, n_layers, layer,
                                 n, nh, nkv, d, page_size, int(write_kv), _p(status), _dt(qkv), _stream()),
           "qkv_to_cache")


def attention_plain(q: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor, positions: torch.Tensor,
                    seq_of_token: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, nh: int,
                    scale: float, window: int = 0, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Paged causal attention, one block per (token, head), float arithmetic, any sizes.  ``status`` (as for
    the other attention kernels) is set to 1 when a key a query needs has no page in the block table."""
    n = q.shape[0]
    _, n_layers, _, nkv, page_size, d = pool.shape
    _check(lib().st_attention_plain(_p(q), _p(pool), _p(out), _p(positions), _p(seq_of_token), _p(slots),
                                    _p(block_table), block_table.shape[1], n_layers, layer, n, nh, nkv, d,
                                    page_size, _f(scale), window, _dt(q), _p(status), _stream()), "attention_plain")
    return out


_DECODE_COUNTERS = 1 << 16
DECODE_MMA_MIN_BLOCKS = 2048     # (token, kv head) pairs from which the tensor-core decode attention serves head sizes above 64
_decode_counter_buffers = {}


def _decode_counters(device: torch.device) -> torch.Tensor:
    """Per-device arrival counters of the split decode attention (zero between launches)."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key not in _decode_counter_buffers:
        _decode_counter_buffers[key] = torch.zeros(_DECODE_COUNTERS, dtype=torch.int32, device=device)
    return _decode_counter_buffers[key]


def attention_decode_scratch(n_items: int, nh: int, d: int, n_splits: int) -> int:
    return int(lib().st_attention_decode_scratch_floats(n_items, nh, d, n_splits))


def attention_decode(q: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor,
                     items: Optional[torch.Tensor], n_items: int, positions: torch.Tensor,
                     seq_of_token: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, nh: int,
                     scale: float, window: int = 0, n_splits: int = 1,
                     partial: Optional[torch.Tensor] = None, fused_merge: bool = True,
                     kernel: str = "auto", warps: int = 4, status: Optional[torch.Tensor] = None,
                     start_pos: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bfloat16 paged attention for single query tokens; ``items`` lists the token indices it serves
    (None: tokens 0..n_items-1).  A token whose position is negative is skipped.

    kernel: "mma" = the tensor-core kernel (head sizes that are multiples of 16 up to 128; with several
    splits it needs the fused merge), "lanes" = the kernel with eight lanes per key (multiples of 8 up to
    256), "auto" = the first that applies.  warps: warps per block of the tensor-core kernel, 4 or 8 (8 pays
    for few and long blocks with head sizes up to 64, see decode_warps).  start_pos: per request of the step, the
    tokens it had in the cache before the step: the tensor-core kernel starts copying those keys before the
    kernel that writes this step's keys has finished (None: it waits first)."""
    _, n_layers, _, nkv, page_size, d = pool.shape
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_decode is a bfloat16 kernel")
    if n_splits > 1:
        need = attention_decode_scratch(n_items, nh, d, n_splits)
        if partial is None or partial.numel() < need or partial.dtype != torch.float32:
            raise KernelError(f"attention_decode: needs {need} floats of scratch for {n_splits} splits")
    counters = _decode_counters(q.device) if (n_splits > 1 and fused_merge
                                              and n_items * nh <= _DECODE_COUNTERS) else None
    mma_ok = bool(lib().st_attention_decode_mma_applies(d)) and (n_splits == 1 or counters is not None)
    if kernel == "auto":
        # Head sizes up to 64: the tensor-core kernel; beyond, it holds fewer blocks per SM than the lanes
        # kernel and pays only for many blocks; grouped queries always gain from it (the group shares one
        # read of the keys and values).
        # (OPT-6.7B decode step, tensor-core / lanes kernel, ms: batch 1 2.98 / 3.08, batch 8 3.68 / 3.70, batch 16
        # 3.88 / 3.76, batch 64 the tensor-core kernel either way: it also serves launches of up to two blocks per SM)
        busy = n_items * nkv >= DECODE_MMA_MIN_BLOCKS
        few = n_items * nkv * n_splits <= 2 * sm_count(q.device)
        kernel = "mma" if mma_ok and (d <= 64 or nh != nkv or busy or few) else "lanes"
    if kernel == "mma":
        if not mma_ok:
            raise KernelError("attention_decode: the tensor-core kernel takes head sizes that are multiples of "
                              "16 up to 128 and merges its splits itself")
        _check(lib().st_attention_decode_mma(_p(q), _p(pool), _p(out), _p(partial), _p(items), n_items,
                                             _p(positions), _p(seq_of_token), _p(slots), _p(start_pos),
                                             _p(block_table), block_table.shape[1], n_layers, layer, nh, nkv, d,
                                             page_size, _f(scale), window, n_splits, _p(counters),
                                             warps if d <= 64 else 4,
                                             _p(status), _stream()), "attention_decode_mma")
    elif kernel == "lanes":
        _check(lib().st_attention_decode(_p(q), _p(pool), _p(out), _p(partial), _p(items), n_items, _p(positions),
                                         _p(seq_of_token), _p(slots), _p(block_table), block_table.shape[1],
                                         n_layers, layer, nh, nkv, d, page_size, _f(scale), window, n_splits,
                                         _p(counters), _p(status), _stream()), "attention_decode")
    else:
        raise KernelError(f"attention_decode: no kernel named {kernel!r}")
    return out


# Decode steps of more tokens than the weight-streaming product serves: the attention kernel works from the library's
# q|k|v product and writes the cache itself (False: a cache-write kernel between the two, for measurements).
DECODE_FROM_PROJECTION = True


def attention_decode_qkv_applies(qkv: torch.Tensor, pool: torch.Tensor, n_items: int, nh: int, n_splits: int) -> bool:
    """Whether ``attention_decode_qkv`` takes this step: bfloat16 on the device, a head size the tensor-core kernel
    takes, and (with several splits) few enough (token, head) pairs for its arrival counters."""
    d = pool.shape[-1]
    return (qkv.is_cuda and qkv.dtype == torch.bfloat16 and pool.dtype == torch.bfloat16
            and bool(lib().st_attention_decode_mma_applies(d)) and (n_splits == 1 or n_items * nh <= _DECODE_COUNTERS))


def attention_decode_qkv(qkv: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor, items: Optional[torch.Tensor], n_items: int, positions: torch.Tensor,
                         seq_of_token: torch.Tensor, slots: torch.Tensor, start_pos: torch.Tensor,
                         block_table: torch.Tensor, nh: int, scale: float, window: int = 0, n_splits: int = 1,
                         partial: Optional[torch.Tensor] = None, warps: int = 4, write_kv: bool = True,
                         status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Single-token attention straight from the fused projection: ``qkv`` [tokens, (nh + 2 nkv) d] holds the q, k and
    v features of ALL the step's tokens as the product left them (bias included), every token of the step is an item,
    and ``start_pos`` says where each request's tokens of this step begin.  The kernel writes each token's key and
    value into its page (``write_kv``) and attends over the cache and the step's own rows: the step needs no
    cache-write kernel.  Only for steps in which no other kernel reads this step's keys from the cache (no prompt
    tiles)."""
    _, n_layers, _, nkv, page_size, d = pool.shape
    if not attention_decode_qkv_applies(qkv, pool, n_items, nh, n_splits):
        raise KernelError("attention_decode_qkv: bfloat16, head sizes that are multiples of 16 up to 128")
    assert qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * d and out.shape == (qkv.shape[0], nh * d)
    counters = None
    if n_splits > 1:
        need = attention_decode_scratch(n_items, nh, d, n_splits)
        if partial is None or partial.numel() < need or partial.dtype != torch.float32:
            raise KernelError(f"attention_decode_qkv: needs {need} floats of scratch for {n_splits} splits")
        counters = _decode_counters(qkv.device)
    _check(lib().st_attention_decode_mma_qkv(_p(qkv), _p(pool), _p(out), _p(partial), _p(items), n_items,
                                             _p(positions), _p(seq_of_token), _p(slots), _p(start_pos),
                                             _p(block_table), block_table.shape[1], pool.shape[0], n_layers, layer,
                                             nh, nkv, d, page_size, _f(scale), window, n_splits, _p(counters),
                                             warps if d <= 64 else 4, int(write_kv), _p(status), _stream()),
           "attention_decode_qkv")
    return out


def decode_warps(n_items: int, nkv: int, d: int, n_splits: int, max_kv: int) -> int:
    """Warps per block for the tensor-core decode attention.  Eight when the launch is at most two blocks per
    SM and the key ranges are long: a warp's chain of groups is then half as long; with many blocks four are
    better (OPT-1.3B decode steps, eight against four warps: batch 8 1.256 / 1.299 ms, batch 64 2.61 / 2.46)."""
    return 8 if (d <= 64 and n_items * nkv * n_splits <= 2 * sm_count() and max_kv >= 256) else 4


# "auto", or the name of one prompt-attention kernel for every call that says "auto" (measurements)
PREFILL_KERNEL = "auto"


def attention_prefill_tile_rows() -> int:
    return int(lib().st_attention_prefill_tile_rows())


def attention_prefill(q: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor, tiles: torch.Tensor,
                      n_tiles: int, q_start: torch.Tensor, start_pos: torch.Tensor, slots: torch.Tensor,
                      block_table: torch.Tensor, nh: int, scale: float, window: int = 0,
                      status: Optional[torch.Tensor] = None, kernel: str = "auto", q_stride: int = 0) -> torch.Tensor:
    """bfloat16 tensor-core paged attention over tiles of 128 query tokens; tiles: int32 [n_tiles, 2] =
    (request index in the step, offset of the tile among the request's new tokens).  ``q_stride``: elements
    between the query rows of consecutive tokens when ``q`` is part of a wider tensor (the q|k|v product), 0 for
    a dense [tokens, nh * d] tensor.

    kernel: "tmap" = the persistent tcgen05 kernel fed by TMA (head size 64, pages of 8 to 64 positions: one block
    per SM walks through the (tile, head) pairs), "tma" = the same with one block per pair (head sizes 64 and 128;
    "tma3" = the same with three softmax warpgroups per block instead of two, at head size 64 only),
    "tc" = the tcgen05 kernel fed by asynchronous copies (head sizes up to 128), "mma" = the mma.sync
    kernel (up to 256), "auto" = the first of these that applies.  ``status`` receives 3 if a tcgen05
    kernel gave up waiting, and 1 from any of them when a key a query needs has no page in the block table."""
    n_pages, n_layers, _, nkv, page_size, d = pool.shape
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill is a bfloat16 kernel")
    if kernel == "auto":
        kernel = PREFILL_KERNEL
    if kernel == "auto":
        if lib().st_attention_prefill_tmap_applies(d, page_size):
            kernel = "tmap"
        elif lib().st_attention_prefill_tma_applies(d, page_size):
            kernel = "tma"
        else:
            kernel = "tc" if d <= 128 else "mma"
    if kernel == "tmap":
        st = status if status is not None else _tc_status_word(q.device)
        _check(lib().st_attention_prefill_tmap(_p(q), _p(pool), ctypes.c_longlong(n_pages), _p(out), _p(tiles),
                                               n_tiles, _p(q_start), _p(start_pos), _p(slots), _p(block_table),
                                               block_table.shape[1], n_layers, layer, nh, nkv, d, page_size,
                                               _f(scale), window, q_stride, _p(st), _stream()), "attention_prefill_tmap")
        return out
    if kernel in ("tma", "tma3"):
        st = status if status is not None else _tc_status_word(q.device)
        lib().st_attention_prefill_tma_warpgroups(3 if kernel == "tma3" else 2)
        _check(lib().st_attention_prefill_tma(_p(q), _p(pool), ctypes.c_longlong(n_pages), _p(out), _p(tiles),
                                              n_tiles, _p(q_start), _p(start_pos), _p(slots), _p(block_table),
                                              block_table.shape[1], n_layers, layer, nh, nkv, d, page_size,
                                              _f(scale), window, q_stride, _p(st), _stream()), "attention_prefill_tma")
        return out
    if kernel == "tc":
        st = status if status is not None else _tc_status_word(q.device)
        _check(lib().st_attention_prefill_tc(_p(q), _p(pool), _p(out), _p(tiles), n_tiles, _p(q_start),
                                             _p(start_pos), _p(slots), _p(block_table), block_table.shape[1],
                                             n_layers, layer, nh, nkv, d, page_size, _f(scale), window, q_stride,
                                             _p(st), _stream()), "attention_prefill_tc")
        return out
    if kernel != "mma":
        raise KernelError(f"attention_prefill: no kernel named {kernel!r}")
    _check(lib().st_attention_prefill(_p(q), _p(pool), _p(out), _p(tiles), n_tiles, _p(q_start), _p(start_pos),
                                      _p(slots), _p(block_table), block_table.shape[1], n_layers, layer, nh, nkv,
                                      d, page_size, _f(scale), window, q_stride, _p(status), _stream()),
           "attention_prefill")
    return out


# ------------------------------------------------- short convolutions, gated units, output norms
def conv_residual(x: torch.Tensor, w: torch.Tensor, state: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
                  seq_of_token: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor,
                  residual: bool = True) -> torch.Tensor:
    """out[t] = (x[t] if residual) + sum_j w[:, j] * x[t - taps + 1 + j] along each request's tokens, one filter per
    channel.  x: [tokens, channels] float32 (the residual stream) or the type of ``out``; w: float32 [channels, taps];
    state: float32 [slots, taps - 1, channels], a request's last taps - 1 inputs, read and moved on by this call."""
    n, c = x.shape
    taps = w.shape[1]
    assert x.is_contiguous() and out.is_contiguous() and out.shape == x.shape and w.dtype == torch.float32
    assert w.shape[0] == c and w.is_contiguous() and state.dtype == torch.float32
    assert state.shape[1:] == (taps - 1, c) and state.is_contiguous()
    assert x.dtype == torch.float32 or x.dtype == out.dtype
    _check(lib().st_conv_residual(_p(x), int(x.dtype == torch.float32), _p(w), _p(state), _p(out), _p(positions),
                                  _p(seq_of_token), _p(q_start), _p(slots), n, c, taps, int(residual), _dt(out),
                                  _stream()), "conv_residual")
    return out


def conv_state_update(x: torch.Tensor, channels: int, state: torch.Tensor, positions: torch.Tensor,
                      q_start: torch.Tensor, slots: torch.Tensor, n_seqs: int) -> None:
    """state[slot] <- the last taps - 1 rows of (state[slot], the request's rows of x in this step), for every request
    of the step; x: [tokens, >= channels] whose first ``channels`` columns are a convolution's inputs."""
    assert x.is_contiguous() and state.dtype == torch.float32 and state.is_contiguous() and state.shape[2] == channels
    _check(lib().st_conv_state_update(_p(x), x.shape[1], _p(state), _p(positions), _p(q_start), _p(slots), n_seqs, channels,
                                      state.shape[1] + 1, _dt(x), _stream()), "conv_state_update")


def norm_add(x: torch.Tensor, y: torch.Tensor, gain: torch.Tensor, mult: float, eps: float,
             positions: Optional[torch.Tensor] = None, out_act: Optional[torch.Tensor] = None) -> None:
    """x[r] += mult * gain * y[r] / sqrt(mean(y[r]^2) + eps) in place on the float32 residual rows; ``gain`` is one
    float32 number on the device.  ``out_act``: also the new x in y's type.  Rows whose position is negative
    (padding) are left alone."""
    assert x.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and y.shape == x.shape
    assert gain.dtype == torch.float32 and gain.numel() == 1
    if out_act is not None:
        assert out_act.dtype == y.dtype and out_act.shape == x.shape and out_act.is_contiguous()
    _check(lib().st_norm_add(_p(x), _p(y), _p(gain), _f(mult), _f(eps), x.shape[0], x.shape[1], _p(positions),
                             _p(out_act), _dt(y), _stream()), "norm_add")


def gated_act(gu: torch.Tensor, act: str) -> torch.Tensor:
    """act(gu[:, :inner]) * gu[:, inner:] for the fused gate | up product gu [rows, 2 * inner]."""
    assert gu.is_contiguous() and gu.shape[1] % 2 == 0
    inner = gu.shape[1] // 2
    out = torch.empty((gu.shape[0], inner), dtype=gu.dtype, device=gu.device)
    _check(lib().st_gated_act(_p(gu), _p(out), gu.shape[0], inner, ACT_CODES[act], _dt(gu), _stream()), "gated_act")
    return out


# ------------------------------------------------------------ differential attention
def _flat_pool(pool: torch.Tensor, layer: int, nkv: int, dim: int, vd: int, page_size: int):
    """(page stride, offset of the entry) in elements, for a pool [pages, entries, nkv * page_size * (2 dim + vd)]."""
    assert pool.dim() == 3 and pool.is_contiguous() and pool.shape[2] == nkv * page_size * (2 * dim + vd)
    return ctypes.c_longlong(pool.stride(0)), ctypes.c_longlong(layer * pool.stride(1))


def diff_qkv_prepare(proj: torch.Tensor, conv_w: torch.Tensor, conv_state: torch.Tensor, q_norm: torch.Tensor,
                     k_norm: torch.Tensor, eps: float, inv_freq: torch.Tensor, rot_dims: int, q_out: torch.Tensor,
                     pool: torch.Tensor, layer: int, positions: torch.Tensor, seq_of_token: torch.Tensor,
                     q_start: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, nh: int, nkv: int,
                     dim: int, vd: int, page_size: int, status: torch.Tensor, write_kv: bool = True,
                     move_state: bool = False) -> None:
    """From the fused projection q | k | v of the step's tokens: the short convolution over time of every channel
    (reading, not moving, the requests' last inputs in ``conv_state``), RMS norm of each map of each query and key
    head with the shared weights, rotation of the first ``rot_dims`` dimensions in neighbouring pairs by
    position * inv_freq, queries to ``q_out`` [tokens, nh * 2 * dim], keys and values into their pages.
    ``move_state``: only for steps in which every request brings exactly one token: the kernel then moves
    ``conv_state`` on itself and ``conv_state_update`` is not needed."""
    taps = conv_w.shape[1]
    channels = (nh + nkv) * 2 * dim + nkv * vd
    assert proj.is_contiguous() and proj.shape[1] == channels and conv_w.shape == (channels, taps)
    assert conv_state.shape[1:] == (taps - 1, channels) and pool.dtype == proj.dtype == q_out.dtype
    stride, offset = _flat_pool(pool, layer, nkv, dim, vd, page_size)
    _check(lib().st_diff_qkv_prepare(_p(proj), proj.shape[1], _p(conv_w), _p(conv_state), int(move_state), taps, _p(q_norm), _p(k_norm),
                                     _f(eps), _p(inv_freq), rot_dims, _p(q_out), _p(pool), stride, offset,
                                     _p(positions), _p(seq_of_token), _p(q_start), _p(slots), _p(block_table),
                                     block_table.shape[1], proj.shape[0], nh, nkv, dim, vd, page_size, int(write_kv),
                                     _p(status), _dt(proj), _stream()), "diff_qkv_prepare")


def diff_attention_plain(q: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor, positions: torch.Tensor,
                         seq_of_token: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, nh: int,
                         nkv: int, dim: int, vd: int, page_size: int, scale: float, cap: float, block: int,
                         window: int, lam: float, eps: float, out_scale: float,
                         status: Optional[torch.Tensor] = None, items: Optional[torch.Tensor] = None,
                         n_items: int = 0) -> torch.Tensor:
    """Differential attention of the step's queries q [tokens, nh * 2 * dim] over the paged cache, one block per
    (token, head), float arithmetic for either type: out [tokens, nh * vd] =
    rms(softmax(cap(q1 k1)) V - lam * softmax(cap(q2 k2)) V) * out_scale.  ``items``: the token indices to serve
    (-1: none), ``n_items`` of them; None: every token."""
    stride, offset = _flat_pool(pool, layer, nkv, dim, vd, page_size)
    _check(lib().st_diff_attention_plain(_p(q), _p(pool), stride, offset, _p(out), _p(items), _p(positions), _p(seq_of_token),
                                         _p(slots), _p(block_table), block_table.shape[1],
                                         n_items if items is not None else q.shape[0], nh, nkv, dim,
                                         vd, page_size, _f(scale), _f(cap), block, window, _f(lam), _f(eps),
                                         _f(out_scale), _p(status), _dt(q), _stream()), "diff_attention_plain")
    return out


def diff_attention_single(q: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor, positions: torch.Tensor,
                          seq_of_token: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, nh: int,
                          nkv: int, dim: int, vd: int, page_size: int, scale: float, cap: float, block: int,
                          window: int, lam: float, eps: float, out_scale: float,
                          status: Optional[torch.Tensor] = None, items: Optional[torch.Tensor] = None,
                          n_items: int = 0) -> torch.Tensor:
    """``diff_attention_plain`` for bfloat16 with 16-byte accesses (dim a multiple of 8 up to 128, vd a multiple of 4 up to 256): the
    kernel for single tokens and short portions, bound by the way of the keys and values from memory.  Sizes it
    does not take go to the plain kernel."""
    if not (q.dtype == torch.bfloat16 and bool(lib().st_diff_attention_single_applies(dim, vd))):
        return diff_attention_plain(q, pool, layer, out, positions, seq_of_token, slots, block_table, nh, nkv, dim, vd,
                                    page_size, scale, cap, block, window, lam, eps, out_scale, status, items, n_items)
    stride, offset = _flat_pool(pool, layer, nkv, dim, vd, page_size)
    _check(lib().st_diff_attention_single(_p(q), _p(pool), stride, offset, _p(out), _p(items), _p(positions),
                                          _p(seq_of_token), _p(slots), _p(block_table), block_table.shape[1],
                                          n_items if items is not None else q.shape[0], nh, nkv, dim, vd, page_size,
                                          _f(scale), _f(cap), block, window, _f(lam), _f(eps), _f(out_scale),
                                          _p(status), _stream()), "diff_attention_single")
    return out


def diff_attention_tiles_applies(q: torch.Tensor, dim: int, vd: int) -> bool:
    """Whether the tensor-core kernel for prompt portions takes these sizes: bfloat16, dim and vd multiples of 8,
    dim <= 128, vd <= 256."""
    return q.is_cuda and q.dtype == torch.bfloat16 and bool(lib().st_diff_attention_tiles_applies(dim, vd))


def diff_attention_tiles(q: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor, tiles: torch.Tensor,
                         n_tiles: int, tile_rows: int, q_start: torch.Tensor, start_pos: torch.Tensor,
                         slots: torch.Tensor, block_table: torch.Tensor, nh: int, nkv: int, dim: int, vd: int,
                         page_size: int, scale: float, cap: float, block: int, window: int, lam: float, eps: float,
                         out_scale: float, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The same attention for tiles of ``tile_rows`` query rows (tiles: int32 [n_tiles, 2] = request of the step,
    offset of the tile among its new tokens) on the warp-level tensor cores, bfloat16 only."""
    if not diff_attention_tiles_applies(q, dim, vd):
        raise KernelError("diff_attention_tiles: bfloat16, dim and vd multiples of 8, dim <= 128, vd <= 256")
    stride, offset = _flat_pool(pool, layer, nkv, dim, vd, page_size)
    _check(lib().st_diff_attention_tiles(_p(q), _p(pool), stride, offset, _p(out), _p(tiles), n_tiles, tile_rows,
                                         _p(q_start), _p(start_pos), _p(slots), _p(block_table), block_table.shape[1],
                                         nh, nkv, dim, vd, page_size, _f(scale), _f(cap), block, window, _f(lam),
                                         _f(eps), _f(out_scale), _p(status), _stream()), "diff_attention_tiles")
    return out


# ------------------------------------------------------------ gated linear recurrence
HGRN2_GATES_MIN_TOKENS = 64      # steps of more tokens prepare the recurrence's gates in a kernel of their own

def hgrn2_scan(proj: torch.Tensor, q_off: int, f_off: int, v_off: int, f_bias: torch.Tensor, lower: torch.Tensor,
               norm_w: torch.Tensor, eps: float, state: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
               q_start: torch.Tensor, slots: torch.Tensor, n_seqs: int, nh: int, dim: int, vd: int,
               scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The HGRN2 recurrence over each request's tokens of the step, from the fused projection (queries, gates and
    values at column offsets q_off, f_off, v_off): S <- diag(f) S + (1 - f) v^T, o = S^T silu(q), f = lower +
    (1 - lower) sigmoid(gate + f_bias); out [tokens, nh * vd] = rms(o) * norm_w per head.  ``state``: float32
    [slots, nh, dim, vd], read and moved on.  ``scratch``: float32, at least tokens * nh * vd elements: with it (and
    dim <= 128) the state is carried in registers and a head's columns are spread over blocks; without it one block
    per (request, head) keeps the state in shared memory.  With room for tokens * nh * (vd + 2 * dim) elements and
    more than HGRN2_GATES_MIN_TOKENS tokens, the gates and queries are prepared by a kernel of their own instead of
    by every block of a head again."""
    assert proj.is_contiguous() and out.is_contiguous() and out.shape == (proj.shape[0], nh * vd)
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (nh, dim, vd)
    gates = None
    if scratch is not None:
        assert scratch.dtype == torch.float32 and scratch.numel() >= out.numel()
        n = proj.shape[0]
        if n > HGRN2_GATES_MIN_TOKENS and scratch.numel() >= n * nh * (vd + 2 * dim):
            gates = scratch[n * nh * vd:]
    _check(lib().st_hgrn2_scan(_p(proj), proj.shape[1], q_off, f_off, v_off, _p(f_bias), _p(lower), _p(norm_w),
                               _f(eps), _p(state), _p(out), _p(scratch), _p(gates), _p(positions), _p(q_start), _p(slots),
                               proj.shape[0], n_seqs, nh, dim, vd, _dt(proj), _stream()), "hgrn2_scan")
    return out


# ------------------------------------------------------------ latent attention
def _latent_pool(pool: torch.Tensor, layer: int, kr: int, rot: int, page_size: int):
    """(page stride, offset of the entry) in elements, for a pool [pages, entries, page_size * (kr + rot)]."""
    assert pool.dim() == 3 and pool.is_contiguous() and pool.shape[2] == page_size * (kr + rot)
    return ctypes.c_longlong(pool.stride(0)), ctypes.c_longlong(layer * pool.stride(1))


def latent_prepare(proj: torch.Tensor, q_rank: int, q_norm: torch.Tensor, kv_norm: torch.Tensor, eps: float,
                   inv_freq: torch.Tensor, rot_dims: int, cq: torch.Tensor, pool: torch.Tensor, layer: int,
                   positions: torch.Tensor, seq_of_token: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor,
                   kr: int, rot: int, page_size: int, status: torch.Tensor, write_kv: bool = True) -> None:
    """From the fused projection [query latent (q_rank) | key/value latent (kr) | shared key part (rot) | ...] of the
    step's tokens: cq = the query latent, RMS-normed with ``q_norm``; the key/value latent RMS-normed with ``kv_norm``
    and the shared key part, its first ``rot_dims`` dimensions rotated in halves by position * inv_freq, go to the
    token's row of its page.  Statistics and angles are float."""
    assert proj.is_contiguous() and proj.shape[1] >= q_rank + kr + rot and cq.shape == (proj.shape[0], q_rank)
    assert cq.is_contiguous() and pool.dtype == proj.dtype == cq.dtype
    stride, offset = _latent_pool(pool, layer, kr, rot, page_size)
    _check(lib().st_latent_prepare(_p(proj), proj.shape[1], q_rank, _p(q_norm), _p(kv_norm), _f(eps), _p(inv_freq),
                                   rot_dims, _p(cq), _p(pool), stride, offset, _p(positions), _p(seq_of_token),
                                   _p(slots), _p(block_table), block_table.shape[1], proj.shape[0], kr, rot, page_size,
                                   int(write_kv), _p(status), _dt(proj), _stream()), "latent_prepare")


def latent_q_rotate(q: torch.Tensor, q_lat: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
                    rot_dims: int, nh: int, dim: int, rot: int, kr: int) -> None:
    """q [tokens, nh * (dim + rot)] -> the last ``rot`` numbers of every head's row of q_lat [tokens, nh, kr + rot]:
    the head's rotated query part, turned by position."""
    assert q.is_contiguous() and q_lat.is_contiguous() and q.dtype == q_lat.dtype
    assert q.shape[1] == nh * (dim + rot) and q_lat.shape == (q.shape[0], nh * (kr + rot))
    _check(lib().st_latent_q_rotate(_p(q), _p(q_lat), _p(positions), _p(inv_freq), rot_dims, q.shape[0], nh, dim, rot,
                                    kr, _dt(q), _stream()), "latent_q_rotate")


def latent_attention_plain(q_lat: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor,
                           positions: torch.Tensor, seq_of_token: torch.Tensor, slots: torch.Tensor,
                           block_table: torch.Tensor, nh: int, kr: int, rot: int, page_size: int, scale: float,
                           sink: Optional[torch.Tensor] = None, gates: Optional[torch.Tensor] = None,
                           status: Optional[torch.Tensor] = None, items: Optional[torch.Tensor] = None,
                           n_items: int = 0) -> torch.Tensor:
    """Causal attention in the latent space, one block per (token, head), float arithmetic for either type:
    out [tokens, nh * kr] = gate * softmax-with-sink(scale * q_lat . [c | k_rot]) c.  ``gates``: a view
    [tokens, nh] (any row stride) of the heads' gate logits; ``sink`` float [nh]."""
    assert q_lat.is_contiguous() and out.is_contiguous() and out.shape == (q_lat.shape[0], nh * kr)
    stride, offset = _latent_pool(pool, layer, kr, rot, page_size)
    if gates is not None:
        assert gates.dtype == q_lat.dtype and gates.stride(1) == 1 and gates.shape == (q_lat.shape[0], nh)
    _check(lib().st_latent_attention_plain(_p(q_lat), _p(pool), stride, offset, _p(out), _p(items), _p(positions),
                                           _p(seq_of_token), _p(slots), _p(block_table), block_table.shape[1],
                                           n_items if items is not None else q_lat.shape[0], nh, kr, rot, page_size,
                                           _p(sink), _p(gates), gates.stride(0) if gates is not None else 0,
                                           _f(scale), _p(status), _dt(q_lat), _stream()), "latent_attention_plain")
    return out


def latent_attention_mma_applies(q_lat: torch.Tensor, kr: int, rot: int) -> bool:
    """Whether the tensor-core kernel takes these sizes: bfloat16, kr a multiple of 16 up to 512, kr + rot a multiple
    of 8, tiles that fit an SM's shared memory."""
    return q_lat.is_cuda and q_lat.dtype == torch.bfloat16 and bool(lib().st_latent_attention_mma_applies(kr, rot))


def latent_attention(q_lat: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor, positions: torch.Tensor,
                     seq_of_token: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, nh: int, kr: int,
                     rot: int, page_size: int, scale: float, sink: Optional[torch.Tensor] = None,
                     gates: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None, kernel: str = "auto",
                     q_start: Optional[torch.Tensor] = None, start_pos: Optional[torch.Tensor] = None, n_seqs: int = 0,
                     lens=None, start=None, scratch=None, n_splits: Optional[int] = None) -> torch.Tensor:
    """Latent attention of the step's queries (see ``latent_attention_plain`` for the arguments).  kernel: "mma" = the
    tensor-core kernel over tiles of 64 (token, head) rows (bfloat16; it needs the step's requests: ``q_start``
    [n_seqs + 1], ``start_pos`` [n_seqs] on the device, or ``lens`` / ``start`` as host arrays), "plain" = the float
    kernel with one block per (token, head), "auto" = the first that applies.  Steps whose tiles do not fill the device
    (single tokens, short portions) have their key ranges cut into ``n_splits`` parts (None: chosen from the step's
    shape) whose partial rows meet in a second small kernel; ``scratch``: a function n -> float32 tensor of at least n
    elements for them (None: allocated here)."""
    if kernel == "auto":
        kernel = "mma" if latent_attention_mma_applies(q_lat, kr, rot) else "plain"
    if kernel == "plain":
        return latent_attention_plain(q_lat, pool, layer, out, positions, seq_of_token, slots, block_table, nh, kr, rot,
                                      page_size, scale, sink, gates, status)
    if kernel != "mma":
        raise KernelError(f"latent_attention: no kernel named {kernel!r}")
    if not latent_attention_mma_applies(q_lat, kr, rot):
        raise KernelError("latent_attention: the tensor-core kernel takes bfloat16, kr % 16 == 0, kr <= 512, (kr + rot) % 8 == 0")
    if q_start is None:
        import numpy as np
        lens = np.asarray(lens, dtype=np.int64)
        n_seqs = len(lens)
        q_start = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=q_lat.device)
        start_pos = torch.tensor(np.asarray(start), dtype=torch.int32, device=q_lat.device)
    assert q_lat.is_contiguous() and out.is_contiguous() and out.shape == (q_lat.shape[0], nh * kr)
    stride, offset = _latent_pool(pool, layer, kr, rot, page_size)
    if gates is not None:
        assert gates.dtype == q_lat.dtype and gates.stride(1) == 1 and gates.shape == (q_lat.shape[0], nh)
    n = q_lat.shape[0]
    if n_splits is None:
        n_splits = int(lib().st_latent_attention_mma_splits(n, n_seqs, nh))
    partial = None
    if n_splits > 1:
        need = int(lib().st_latent_attention_mma_scratch(n, n_seqs, nh, kr, n_splits))
        partial = scratch(need) if scratch is not None else torch.empty(need, dtype=torch.float32, device=q_lat.device)
        assert partial.dtype == torch.float32 and partial.numel() >= need
    _check(lib().st_latent_attention_mma(_p(q_lat), _p(pool), stride, offset, _p(out), _p(positions), _p(q_start),
                                         _p(start_pos), _p(slots), _p(block_table), block_table.shape[1],
                                         n, n_seqs, nh, kr, rot, page_size, _p(sink), _p(gates),
                                         gates.stride(0) if gates is not None else 0, _f(scale), n_splits, _p(partial),
                                         _p(status), _stream()),
           "latent_attention_mma")
    return out


# ------------------------------------------------------------ grouped products, mixtures of experts
def gemm_heads(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, n_groups: int, k_dim: int, n_out: int,
               a_goff: int, c_goff: int) -> torch.Tensor:
    """out[:, g * c_goff + n] = sum_k a[:, g * a_goff + k] * w[g, n, k] for every group g: one product per head, each
    on its own columns of ``a`` [rows, lda] and of ``out`` [rows, ldc]; w [groups, n_out, k_dim]."""
    assert a.dim() == 2 and out.dim() == 2 and a.shape[0] == out.shape[0] and a.stride(1) == 1 and out.stride(1) == 1
    assert w.is_contiguous() and w.shape == (n_groups, n_out, k_dim) and a.dtype == w.dtype
    ll = ctypes.c_longlong
    args = (_p(a), _p(w), _p(out), n_groups, a.shape[0], n_out, k_dim, 0, 0, ll(a.stride(0)), ll(a_goff), ll(out.stride(0)),
            ll(c_goff), ll(n_out * k_dim), None, None, None, 0, None, 1)
    if _grouped_mma(a, k_dim, a.stride(0), a_goff, n_out * k_dim):
        _check(lib().st_gemm_grouped_mma(*args, int(out.dtype == torch.float32), _stream()), "gemm_heads")
    else:
        _check(lib().st_gemm_grouped_plain(*args, _dt(a), int(out.dtype == torch.float32), _stream()), "gemm_heads")
    return out


# False: the grouped products of bfloat16 models run on the plain kernel too (measurements, tests)
GROUPED_MMA = True


def _grouped_mma(a: torch.Tensor, k_dim: int, lda: int, a_goff: int, w_gstride: int) -> bool:
    return (GROUPED_MMA and a.dtype == torch.bfloat16
            and bool(lib().st_gemm_grouped_mma_applies(k_dim, ctypes.c_longlong(lda), ctypes.c_longlong(a_goff),
                                                       ctypes.c_longlong(w_gstride))))


def moe_route(h: torch.Tensor, w_router: torch.Tensor, top: int, positions: Optional[torch.Tensor] = None,
              w_gate: Optional[torch.Tensor] = None, renorm: bool = False):
    """-> (experts int32 [tokens, top], weights float [tokens, top], gate float [tokens] or None).  Router logits,
    softmax over all experts and the choice in float; ``w_router`` float [experts, width]; ``w_gate`` float [width]:
    also sigmoid(w_gate . h) per token.  Tokens at a negative position get expert -1."""
    n, width = h.shape
    assert h.is_contiguous() and w_router.dtype == torch.float32 and w_router.is_contiguous() and w_router.shape[1] == width
    experts = torch.empty((n, top), dtype=torch.int32, device=h.device)
    weights = torch.empty((n, top), dtype=torch.float32, device=h.device)
    gate = torch.empty((n,), dtype=torch.float32, device=h.device) if w_gate is not None else None
    if w_gate is not None:
        assert w_gate.dtype == torch.float32 and w_gate.numel() == width and w_gate.is_contiguous()
    _check(lib().st_moe_route(_p(h), n, width, _p(w_router), w_router.shape[0], top, int(renorm), _p(w_gate),
                              _p(positions), _p(experts), _p(weights), _p(gate), _dt(h), _stream()), "moe_route")
    return experts, weights, gate


def grouped_tile_rows() -> int:
    return int(lib().st_gemm_grouped_tile_rows())


class ExpertOrder:
    """The step's (token, choice) items grouped by expert (device arrays, see ``moe_sort``)."""

    def __init__(self, offsets, sorted_items, place, tile_group, tile_row0, n_items, top):
        self.offsets, self.sorted, self.place = offsets, sorted_items, place
        self.tile_group, self.tile_row0, self.n_items, self.top = tile_group, tile_row0, n_items, top


def moe_sort(experts: torch.Tensor, n_experts: int) -> ExpertOrder:
    """Group the (token, choice) items of ``experts`` [tokens, top] by expert; everything stays on the device."""
    n, top = experts.shape
    items, rows = n * top, grouped_tile_rows()
    cap = (items + rows - 1) // rows + n_experts
    buf = torch.empty(n_experts + 1 + 2 * items + 2 * cap, dtype=torch.int32, device=experts.device)
    offsets, rest = buf[:n_experts + 1], buf[n_experts + 1:]
    sorted_items, place, tile_group, tile_row0 = rest[:items], rest[items:2 * items], rest[2 * items:2 * items + cap], rest[2 * items + cap:]
    _check(lib().st_moe_sort(_p(experts), items, n_experts, rows, cap, _p(offsets), _p(sorted_items), _p(place),
                             _p(tile_group), _p(tile_row0), _stream()), "moe_sort")
    return ExpertOrder(offsets, sorted_items, place, tile_group, tile_row0, items, top)


def gemm_experts(a: torch.Tensor, w: torch.Tensor, order: ExpertOrder, gather: bool, gated: bool = False,
                 act: str = "none") -> torch.Tensor:
    """One product per expert over the rows the order gives it: out [items, n_out] in sorted order.
    ``gather``: the rows of ``a`` are the tokens (row of item i = i // top), else ``a`` is already in sorted order.
    w [experts, n_out (twice with ``gated``: gate rows, then up rows), k]; gated: out = act(gate) * up."""
    assert a.is_contiguous() and w.is_contiguous() and w.dim() == 3 and a.dtype == w.dtype and a.shape[1] == w.shape[2]
    n_out = w.shape[1] // 2 if gated else w.shape[1]
    out = torch.empty((order.n_items, n_out), dtype=a.dtype, device=a.device)
    ll = ctypes.c_longlong
    args = (_p(a), _p(w), _p(out), w.shape[0], order.n_items, n_out, w.shape[2], int(gated), ACT_CODES[act], ll(a.stride(0)),
            ll(0), ll(n_out), ll(0), ll(w.shape[1] * w.shape[2]), _p(order.offsets), _p(order.tile_group),
            _p(order.tile_row0), order.tile_group.numel(), _p(order.sorted) if gather else None, order.top if gather else 1)
    if _grouped_mma(a, w.shape[2], a.stride(0), 0, w.shape[1] * w.shape[2]):
        _check(lib().st_gemm_grouped_mma(*args, 0, _stream()), "gemm_experts")
    else:
        _check(lib().st_gemm_grouped_plain(*args, _dt(a), 0, _stream()), "gemm_experts")
    return out


def moe_combine(y: torch.Tensor, order: ExpertOrder, weights: torch.Tensor, shared: Optional[torch.Tensor] = None,
                gate: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """out[t] = sum_k weights[t, k] * y[place of (t, k)] (+ gate[t] * shared[t]); sums in float."""
    n, top = weights.shape
    width = y.shape[1]
    assert y.is_contiguous() and (shared is None or (shared.is_contiguous() and shared.dtype == y.dtype and gate is not None))
    out = torch.empty((n, width), dtype=out_dtype, device=y.device)
    _check(lib().st_moe_combine(_p(y), _p(order.place), _p(weights), top, _p(shared), _p(gate), n, width, _p(out),
                                _dt(y), int(out_dtype == torch.float32), _stream()), "moe_combine")
    return out


def concat_rows(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """[a | b] row by row in b's type; ``a`` may be float32 (the residual rows)."""
    assert a.is_contiguous() and b.is_contiguous() and a.shape[0] == b.shape[0]
    assert a.dtype == b.dtype or a.dtype == torch.float32
    out = torch.empty((a.shape[0], a.shape[1] + b.shape[1]), dtype=b.dtype, device=b.device)
    _check(lib().st_concat_rows(_p(a), int(a.dtype == torch.float32), a.shape[1], _p(b), b.shape[1], _p(out), a.shape[0],
                                _dt(b), _stream()), "concat_rows")
    return out


def scale_softcap(x: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> torch.Tensor:
    """x <- cap * tanh(x * scale / cap) in place on float32 values (cap <= 0: x <- x * scale)."""
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(lib().st_scale_softcap(_p(x), ctypes.c_longlong(x.numel()), _f(scale), _f(cap), _stream()), "scale_softcap")
    return x


# ------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Lowest index of the largest value of each row of float32 logits -> int32 [rows]."""
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    n, v = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _check(lib().st_argmax(_p(logits), n, v, _p(out), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperatures: torch.Tensor, top_k: torch.Tensor, seeds: torch.Tensor,
           counters: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row r: temperature <= 0 -> greedy; else draw from softmax(logits/temperature) restricted to the
    top_k[r] largest (<= 0: all) with the uniform number ``uniform(seeds[r], counters[r])``."""
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    assert temperatures.dtype == torch.float32 and top_k.dtype == torch.int32
    assert seeds.dtype == torch.int64 and counters.dtype == torch.int64
    n, v = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _check(lib().st_sample(_p(logits), n, v, _p(temperatures), _p(top_k), _p(seeds), _p(counters), _p(out),
                           _stream()), "sample")
    return out


def uniform(seed: int, counter: int) -> float:
    """The uniform number in [0,1) that `sample` uses for (seed, counter); computed on the host."""
    return float(lib().st_uniform_host(seed, counter))


# ------------------------------------------------------------ grouped attention (keys and values of own sizes)
def _gqa_pool(pool: torch.Tensor, layer: int, nkv: int, dim: int, vd: int, page_size: int):
    """(page stride, offset of the entry) in elements, for a pool [pages, entries, nkv * page_size * (dim + vd)]."""
    assert pool.dim() == 3 and pool.is_contiguous() and pool.shape[2] == nkv * page_size * (dim + vd)
    return ctypes.c_longlong(pool.stride(0)), ctypes.c_longlong(layer * pool.stride(1))


def gqa_prepare(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, bias: Optional[torch.Tensor],
                inv_freq: Optional[torch.Tensor], rot_dims: int, temp_coef: float, temp_every: int,
                q_out: torch.Tensor, pool: torch.Tensor, layer: int, positions: torch.Tensor,
                seq_of_token: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, nh: int, nkv: int,
                dim: int, vd: int, page_size: int, status: Optional[torch.Tensor], write_kv: bool = True,
                norm_eps: float = 0.0) -> None:
    """Queries, keys and values of a step from the fused projection ``proj`` [tokens, columns] (queries at column
    q_off, keys at k_off, values at v_off): plus ``bias`` (float32, one number per column of proj, or None); the
    first ``rot_dims`` dimensions of every query and key head rotated by position in the halves layout; queries
    times 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1); queries to ``q_out`` [tokens, nh * dim], keys and
    values into their pages (``write_kv`` False: queries only).  ``norm_eps`` > 0: after the rotation every query and
    key head is divided by its root mean square over ``dim`` (eps inside the root, no weight)."""
    assert proj.is_contiguous() and q_out.is_contiguous() and q_out.shape == (proj.shape[0], nh * dim)
    assert proj.dtype == q_out.dtype == pool.dtype
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == proj.shape[1]
    stride, off = _gqa_pool(pool, layer, nkv, dim, vd, page_size)
    _check(lib().st_gqa_prepare(_p(proj), proj.shape[1], q_off, k_off, v_off, _p(bias), _p(inv_freq), rot_dims,
                                _f(temp_coef), temp_every, _p(q_out), _p(pool), stride, off, _p(positions),
                                _p(seq_of_token), _p(slots), _p(block_table), block_table.shape[1], proj.shape[0], nh,
                                nkv, dim, vd, page_size, int(write_kv), _p(status), _dt(proj), _stream(),
                                _f(norm_eps)), "gqa_prepare")


def _sink_args(sink, nh: int):
    """(has_sink, the one logit, the logits per head): ``sink`` is None, a number, or a float32 tensor [heads]."""
    if sink is None:
        return 0, _f(0.0), None
    if isinstance(sink, torch.Tensor):
        assert sink.dtype == torch.float32 and sink.numel() == nh and sink.is_contiguous()
        return 1, _f(0.0), _p(sink)
    return 1, _f(float(sink)), None


def _gqa_tail(pool, layer, nkv, dim, vd, page_size, scale, window, keep_first, sink, gate, gate_off, out_scale):
    stride, off = _gqa_pool(pool, layer, nkv, dim, vd, page_size)
    gate_ptr = None
    if gate is not None:
        assert gate.is_contiguous() and gate.dtype == pool.dtype
        gate_ptr = ctypes.c_void_p(gate.data_ptr() + gate_off * gate.element_size())
    return stride, off, gate_ptr, ctypes.c_longlong(gate.shape[1] if gate is not None else 0)


def gqa_attention_plain(q: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor, positions: torch.Tensor,
                        seq_of_token: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, nh: int, nkv: int,
                        dim: int, vd: int, page_size: int, scale: float, window: int, keep_first: int,
                        sink: Optional[float], gate: Optional[torch.Tensor], gate_off: int, out_scale: float,
                        status: Optional[torch.Tensor] = None, items: Optional[torch.Tensor] = None,
                        n_items: Optional[int] = None) -> torch.Tensor:
    """Grouped attention of every token of the step (or of those ``items`` lists) over the paged cache, in float
    arithmetic for either storage type.  ``window`` 0: all keys up to the query; else the last ``window`` keys and
    the request's first ``keep_first``.  ``sink``: a logit that joins the softmax's denominator (None: none).
    ``gate`` [tokens, columns]: the head's result is multiplied by sigmoid of its columns from ``gate_off`` on.
    ``sink`` may also be a float32 tensor [heads]: a logit per head."""
    assert q.is_contiguous() and out.is_contiguous() and out.shape == (q.shape[0], nh * vd)
    stride, off, gate_ptr, gate_ld = _gqa_tail(pool, layer, nkv, dim, vd, page_size, scale, window, keep_first, sink,
                                               gate, gate_off, out_scale)
    n = q.shape[0] if items is None else (n_items if n_items is not None else items.numel())
    has_sink, sink_one, sinks = _sink_args(sink, nh)
    _check(lib().st_gqa_attention_plain(_p(q), _p(pool), stride, off, _p(out), _p(items), _p(positions),
                                        _p(seq_of_token), _p(slots), _p(block_table), block_table.shape[1], n, nh, nkv,
                                        dim, vd, page_size, _f(scale), window, keep_first, has_sink,
                                        sink_one, gate_ptr, gate_ld, _f(out_scale), _p(status), _dt(q),
                                        _stream(), sinks), "gqa_attention_plain")
    return out


# ------------------------------------------------------------ the gated delta rule
def delta_rule_scratch(n_tokens: int, H: int, G: int, dim: int, vd: int) -> int:
    lib().st_delta_rule_scratch_floats.restype = ctypes.c_longlong
    return int(lib().st_delta_rule_scratch_floats(n_tokens, H, G, dim, vd))


def delta_rule_set_lanes(lanes: int) -> None:
    """How many lanes share a column of the state in the recurrence: 8 or 16, or 0 for the launcher's own choice by
    the number of blocks a step gives (the default)."""
    _check(lib().st_delta_rule_set_lanes(int(lanes)), "delta_rule_set_lanes")


def delta_rule(proj: torch.Tensor, b_off: int, a_off: int, g_off: int, conv_w: torch.Tensor, conv_state: torch.Tensor,
               w_a2: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, w_g2: torch.Tensor, norm_w: torch.Tensor,
               eps: float, out_scale: float, state: torch.Tensor, write_state: bool, single_tokens: bool,
               scratch: torch.Tensor, out: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
               q_start: torch.Tensor, slots: torch.Tensor, n_seqs: int, H: int, G: int, dim: int, vd: int,
               gate_silu: bool = False) -> torch.Tensor:
    """The gated delta rule over each request's tokens of the step, from the float32 projection ``proj`` [tokens,
    columns] = q (G * dim) | k (G * dim) | v (H * vd) from column 0, write strengths at b_off (H), the low-rank
    inputs of the decays at a_off and of the output gates at g_off.  ``conv_w`` float32 [channels, taps], the
    filters of q | k | v; ``conv_state`` float32 [slots, taps - 1, channels] is read and, when every request brings
    one token, moved on (else ``conv_state_update`` follows); ``state`` float32 [slots, H, dim, vd] is read and
    moved on.  out [tokens, H * vd] in the type of ``w_a2`` / ``w_g2``.  ``w_a2`` None: the projection holds one
    decay logit per head at a_off and ``dt_bias`` is [H]; ``w_g2`` None: it holds the output gate's H * vd logits
    at g_off.  ``gate_silu``: the gate is z * sigmoid(z) instead of sigmoid(z)."""
    assert proj.dtype == torch.float32 and proj.is_contiguous() and out.is_contiguous()
    assert out.shape == (proj.shape[0], H * vd) and all(w is None or w.dtype == out.dtype for w in (w_a2, w_g2))
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (H, dim, vd)
    channels = 2 * G * dim + H * vd
    taps = conv_w.shape[1]
    assert conv_w.dtype == torch.float32 and conv_w.shape[0] == channels and conv_w.is_contiguous()
    assert conv_state.dtype == torch.float32 and conv_state.shape[1:] == (taps - 1, channels)
    assert w_a2 is None or (w_a2.is_contiguous() and w_a2.shape[0] == H * dim)
    assert w_g2 is None or (w_g2.is_contiguous() and w_g2.shape[0] == H * vd)
    assert dt_bias.numel() == (H * dim if w_a2 is not None else H)
    assert scratch.dtype == torch.float32 and scratch.numel() >= delta_rule_scratch(proj.shape[0], H, G, dim, vd)
    _check(lib().st_delta_rule(_p(proj), proj.shape[1], 0, b_off, a_off, g_off,
                               w_a2.shape[1] if w_a2 is not None else 0, w_g2.shape[1] if w_g2 is not None else 0,
                               _p(conv_w), taps, _p(conv_state), _p(w_a2), _p(a_log), _p(dt_bias), _p(w_g2),
                               _p(norm_w), _f(eps), _f(out_scale), _p(state), int(write_state), int(single_tokens),
                               _p(scratch), _p(out), _p(positions), _p(seq_of_token), _p(q_start), _p(slots),
                               proj.shape[0], n_seqs, H, G, dim, vd, _dt(out), _stream(), int(gate_silu)), "delta_rule")
    return out


def gated_clamped_act(gu: torch.Tensor, bias: Optional[torch.Tensor], limit: float, alpha: float,
                      shift: float) -> torch.Tensor:
    """g * sigmoid(alpha * g) * (u + shift) with g = min(gate + b, limit), u = clamp(up + b, -limit, limit) for the
    fused gate | up product gu [rows, 2 * inner] and its float32 bias [2 * inner] (None: none; limit <= 0: none)."""
    assert gu.is_contiguous() and gu.shape[1] % 2 == 0
    inner = gu.shape[1] // 2
    out = torch.empty((gu.shape[0], inner), dtype=gu.dtype, device=gu.device)
    _check(lib().st_gated_clamped_act(_p(gu), _p(bias), _p(out), gu.shape[0], inner, _f(limit), _f(alpha), _f(shift),
                                      _dt(gu), _stream()), "gated_clamped_act")
    return out


def gqa_attention_fast_applies(q: torch.Tensor, nh: int, nkv: int, dim: int, vd: int) -> bool:
    """Whether the bfloat16 kernels (query tiles on the tensor cores; single tokens a block per key/value head with
    8-byte accesses) take these sizes: dim and vd multiples of 8, dim <= 128, vd <= 256, at most eight query heads
    per key/value head."""
    return (q.is_cuda and q.dtype == torch.bfloat16 and bool(lib().st_gqa_attention_tiles_applies(dim, vd))
            and bool(lib().st_gqa_attention_single_applies(nh, nkv, dim, vd)))


def gqa_attention_tiles(q: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor, tiles: torch.Tensor,
                        n_tiles: int, tile_rows: int, q_start: torch.Tensor, start_pos: torch.Tensor,
                        slots: torch.Tensor, block_table: torch.Tensor, nh: int, nkv: int, dim: int, vd: int,
                        page_size: int, scale: float, window: int, keep_first: int, sink: Optional[float],
                        gate: Optional[torch.Tensor], gate_off: int, out_scale: float,
                        status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The same attention for tiles of ``tile_rows`` query rows (tiles: int32 [n_tiles, 2] = request of the step,
    offset of the tile among its new tokens) on the warp-level tensor cores, bfloat16 only."""
    if not (q.dtype == torch.bfloat16 and bool(lib().st_gqa_attention_tiles_applies(dim, vd))):
        raise KernelError("gqa_attention_tiles: bfloat16, dim and vd multiples of 8, dim <= 128, vd <= 256")
    assert q.is_contiguous() and out.is_contiguous() and out.shape == (q.shape[0], nh * vd)
    stride, off, gate_ptr, gate_ld = _gqa_tail(pool, layer, nkv, dim, vd, page_size, scale, window, keep_first, sink,
                                               gate, gate_off, out_scale)
    has_sink, sink_one, sinks = _sink_args(sink, nh)
    _check(lib().st_gqa_attention_tiles(_p(q), _p(pool), stride, off, _p(out), _p(tiles), n_tiles, tile_rows,
                                        _p(q_start), _p(start_pos), _p(slots), _p(block_table), block_table.shape[1],
                                        nh, nkv, dim, vd, page_size, _f(scale), window, keep_first,
                                        has_sink, sink_one, gate_ptr, gate_ld, _f(out_scale),
                                        _p(status), _stream(), sinks), "gqa_attention_tiles")
    return out


def gqa_attention_single(q: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor, positions: torch.Tensor,
                         seq_of_token: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, nh: int, nkv: int,
                         dim: int, vd: int, page_size: int, scale: float, window: int, keep_first: int,
                         sink: Optional[float], gate: Optional[torch.Tensor], gate_off: int, out_scale: float,
                         status: Optional[torch.Tensor] = None, items: Optional[torch.Tensor] = None,
                         n_items: Optional[int] = None) -> torch.Tensor:
    """The same attention token by token in bfloat16, one block per (token, key/value head) for all the query heads
    that read it; ``items`` as for the plain kernel."""
    if not (q.dtype == torch.bfloat16 and bool(lib().st_gqa_attention_single_applies(nh, nkv, dim, vd))):
        raise KernelError("gqa_attention_single: bfloat16, dim and vd multiples of 8, dim <= 128, vd <= 256, at most "
                          "eight query heads per key/value head")
    assert q.is_contiguous() and out.is_contiguous() and out.shape == (q.shape[0], nh * vd)
    stride, off, gate_ptr, gate_ld = _gqa_tail(pool, layer, nkv, dim, vd, page_size, scale, window, keep_first, sink,
                                               gate, gate_off, out_scale)
    n = q.shape[0] if items is None else (n_items if n_items is not None else items.numel())
    has_sink, sink_one, sinks = _sink_args(sink, nh)
    _check(lib().st_gqa_attention_single(_p(q), _p(pool), stride, off, _p(out), _p(items), _p(positions),
                                         _p(seq_of_token), _p(slots), _p(block_table), block_table.shape[1], n, nh, nkv,
                                         dim, vd, page_size, _f(scale), window, keep_first, has_sink,
                                         sink_one, gate_ptr, gate_ld, _f(out_scale), _p(status), _stream(), sinks),
           "gqa_attention_single")
    return out


# ------------------------------------------------------------ several residual streams, paired norms, xIELU
def hc_spread(x: torch.Tensor, n_streams: int) -> torch.Tensor:
    """n copies of the float32 rows x [tokens, width] -> lanes [n, tokens, width]."""
    assert x.dtype == torch.float32 and x.is_contiguous()
    lanes = torch.empty((n_streams,) + tuple(x.shape), dtype=torch.float32, device=x.device)
    _check(lib().st_hc_spread(_p(x), _p(lanes), ctypes.c_longlong(x.numel()), n_streams, _stream()), "hc_spread")
    return lanes


def hc_sum(lanes: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The sum of the streams, lanes [n, tokens, width] float32 -> [tokens, width]."""
    assert lanes.dtype == torch.float32 and lanes.is_contiguous() and lanes.dim() == 3
    if out is None:
        out = torch.empty(lanes.shape[1:], dtype=torch.float32, device=lanes.device)
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape == lanes.shape[1:]
    _check(lib().st_hc_sum(_p(lanes), _p(out), ctypes.c_longlong(out.numel()), lanes.shape[0], _stream()), "hc_sum")
    return out


def hc_read_norm(lanes: torch.Tensor, coef: torch.Tensor, gain: torch.Tensor, eps: float,
                 positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """u = sum_s coef[s] * lanes[s]; -> u / sqrt(mean(u^2) + eps) * gain, float32 [tokens, width]."""
    n, tokens, width = lanes.shape
    assert lanes.dtype == torch.float32 and lanes.is_contiguous()
    assert coef.dtype == torch.float32 and coef.numel() == n and gain.dtype == torch.float32 and gain.numel() == width
    out = torch.empty((tokens, width), dtype=torch.float32, device=lanes.device)
    _check(lib().st_hc_read_norm(_p(lanes), n, _p(coef), _p(gain), _f(eps), tokens, width, _p(out), _p(positions),
                                 _stream()), "hc_read_norm")
    return out


def hc_write(lanes: torch.Tensor, mix: torch.Tensor, out_coef: torch.Tensor, y: torch.Tensor) -> None:
    """lanes[t] <- sum_s mix[s, t] * lanes[s] + out_coef[t] * y, all t at once from the old lanes, in place."""
    n, tokens, width = lanes.shape
    assert lanes.dtype == torch.float32 and lanes.is_contiguous() and y.is_contiguous() and y.shape == (tokens, width)
    assert mix.dtype == torch.float32 and mix.shape == (n, n) and mix.is_contiguous()
    assert out_coef.dtype == torch.float32 and out_coef.numel() == n
    _check(lib().st_hc_write(_p(lanes), n, _p(mix), _p(out_coef), _p(y), _dt(y), tokens, width, _stream()), "hc_write")


def norm_pair_sum(a: torch.Tensor, wa: torch.Tensor, ca: float, b: torch.Tensor, wb: torch.Tensor, cb: float,
                  eps: float, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """ca * wa * a / rms(a) + cb * wb * b / rms(b) row by row (rms over the row, eps inside the root), float32."""
    assert a.is_contiguous() and b.is_contiguous() and a.shape == b.shape and a.dim() == 2
    assert wa.dtype == wb.dtype == torch.float32 and wa.numel() == wb.numel() == a.shape[1]
    out = torch.empty(a.shape, dtype=torch.float32, device=a.device)
    _check(lib().st_norm_pair_sum(_p(a), _dt(a), _p(wa), _f(ca), _p(b), _dt(b), _p(wb), _f(cb), _f(eps), a.shape[0],
                                  a.shape[1], _p(out), _p(positions), _stream()), "norm_pair_sum")
    return out


def xielu(z: torch.Tensor, alpha_pos: float, alpha_neg: float, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """z > 0: alpha_pos * z^2 + z / 2;  z <= 0: alpha_neg * (exp(z) - 1 - z) + z / 2.  z float32 or the storage type."""
    assert z.is_contiguous()
    out_dtype = out_dtype or z.dtype
    assert z.dtype in (torch.float32, out_dtype)
    out = torch.empty(z.shape, dtype=out_dtype, device=z.device)
    _check(lib().st_xielu(_p(z), int(z.dtype == torch.float32), _p(out), ctypes.c_longlong(z.numel()), _f(alpha_pos),
                          _f(alpha_neg), _dt(out), _stream()), "xielu")
    return out


# ------------------------------------------------------------ attention whose weights are mixed over heads
def talk_attention_plain(q: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor, positions: torch.Tensor,
                         seq_of_token: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, nh: int, nkv: int,
                         dim: int, vd: int, page_size: int, scale: float, window: int, keep_first: int,
                         talk: Optional[torch.Tensor], sinks: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                         gate_off: int, gate_heads: bool, out_scale: float, status: Optional[torch.Tensor] = None,
                         items: Optional[torch.Tensor] = None, n_items: Optional[int] = None) -> torch.Tensor:
    """Grouped attention over the paged cache whose normalised softmax weights are mixed over the heads before they
    meet the values: P'_a = sum_b talk[a, b] P_b, head a applying P'_a to the values of its own key/value head.
    ``talk`` float32 [heads, heads] (None: the identity); ``sinks`` float32 [heads]: a logit per head in the
    denominator (None: none); ``gate`` [tokens, columns]: sigmoid of its columns from ``gate_off`` on, one per head
    (``gate_heads``) or one per (head, value dimension).  Float arithmetic for either storage type."""
    assert q.is_contiguous() and out.is_contiguous() and out.shape == (q.shape[0], nh * vd)
    stride, off, gate_ptr, gate_ld = _gqa_tail(pool, layer, nkv, dim, vd, page_size, scale, window, keep_first, None,
                                               gate, gate_off, out_scale)
    if talk is not None:
        assert talk.dtype == torch.float32 and talk.shape == (nh, nh) and talk.is_contiguous()
    if sinks is not None:
        assert sinks.dtype == torch.float32 and sinks.numel() == nh and sinks.is_contiguous()
    n = q.shape[0] if items is None else (n_items if n_items is not None else items.numel())
    _check(lib().st_talk_attention_plain(_p(q), _p(pool), stride, off, _p(out), _p(items), _p(positions),
                                         _p(seq_of_token), _p(slots), _p(block_table), block_table.shape[1], n, nh, nkv,
                                         dim, vd, page_size, _f(scale), window, keep_first, _p(talk), _p(sinks),
                                         gate_ptr, gate_ld, int(gate_heads), _f(out_scale), _p(status), _dt(q),
                                         _stream()), "talk_attention_plain")
    return out


def talk_attention_tiles_applies(q: torch.Tensor, nh: int, nkv: int, dim: int, vd: int) -> bool:
    """Whether the tensor-core kernel for query tiles takes these sizes (bfloat16 only)."""
    return q.is_cuda and q.dtype == torch.bfloat16 and bool(lib().st_talk_attention_tiles_applies(nh, nkv, dim, vd))


def talk_attention_tiles(q: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor, tiles: torch.Tensor,
                         n_tiles: int, tile_rows: int, q_start: torch.Tensor, start_pos: torch.Tensor,
                         slots: torch.Tensor, block_table: torch.Tensor, nh: int, nkv: int, dim: int, vd: int,
                         page_size: int, scale: float, window: int, keep_first: int, talk: Optional[torch.Tensor],
                         sinks: Optional[torch.Tensor], gate: Optional[torch.Tensor], gate_off: int, gate_heads: bool,
                         out_scale: float, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The same attention as ``talk_attention_plain`` for tiles of ``tile_rows`` query rows (tiles: int32 [n_tiles, 2]
    = request of the step, offset of the tile among its new tokens) on the warp-level tensor cores, bfloat16 only."""
    if not talk_attention_tiles_applies(q, nh, nkv, dim, vd):
        raise KernelError("talk_attention_tiles: bfloat16, dim and vd multiples of 8 up to 128, heads within a block")
    assert q.is_contiguous() and out.is_contiguous() and out.shape == (q.shape[0], nh * vd)
    stride, off, gate_ptr, gate_ld = _gqa_tail(pool, layer, nkv, dim, vd, page_size, scale, window, keep_first, None,
                                               gate, gate_off, out_scale)
    if talk is not None:
        assert talk.dtype == torch.float32 and talk.shape == (nh, nh) and talk.is_contiguous()
    if sinks is not None:
        assert sinks.dtype == torch.float32 and sinks.numel() == nh and sinks.is_contiguous()
    _check(lib().st_talk_attention_tiles(_p(q), _p(pool), stride, off, _p(out), _p(tiles), n_tiles, tile_rows,
                                         _p(q_start), _p(start_pos), _p(slots), _p(block_table), block_table.shape[1],
                                         nh, nkv, dim, vd, page_size, _f(scale), window, keep_first, _p(talk), _p(sinks),
                                         gate_ptr, gate_ld, int(gate_heads), _f(out_scale), _p(status), _stream()),
           "talk_attention_tiles")
    return out


def talk_attention_single_applies(q: torch.Tensor, nh: int, nkv: int, dim: int, vd: int, n_cap: int) -> bool:
    """Whether the two-kernel form for single tokens takes these sizes (bfloat16; all heads' weights of a token,
    heads * n_cap floats, within shared memory)."""
    return (q.is_cuda and q.dtype == torch.bfloat16
            and bool(lib().st_talk_attention_single_applies(nh, nkv, dim, vd, int(n_cap))))


def talk_attention_single_scratch(n_tokens: int, nh: int, n_cap: int) -> int:
    return int(n_tokens) * int(nh) * int(n_cap)


def talk_attention_single(q: torch.Tensor, pool: torch.Tensor, layer: int, out: torch.Tensor, positions: torch.Tensor,
                          seq_of_token: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, nh: int, nkv: int,
                          dim: int, vd: int, page_size: int, scale: float, window: int, keep_first: int,
                          talk: Optional[torch.Tensor], sinks: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                          gate_off: int, gate_heads: bool, out_scale: float, scratch: torch.Tensor, n_cap: int,
                          status: Optional[torch.Tensor] = None, items: Optional[torch.Tensor] = None,
                          n_items: Optional[int] = None) -> torch.Tensor:
    """The same attention as ``talk_attention_plain`` token by token in bfloat16: raw scores of every (token, head,
    seen key) into ``scratch`` (float32, ``talk_attention_single_scratch`` elements), then softmax, mixing and values
    per (token, key/value head).  ``n_cap``: the most keys a token of the step sees."""
    if not talk_attention_single_applies(q, nh, nkv, dim, vd, n_cap):
        raise KernelError("talk_attention_single: bfloat16, dim and vd multiples of 8, vd <= 256, at most eight query "
                          "heads per key/value head, and all heads' weights of a token within shared memory")
    assert q.is_contiguous() and out.is_contiguous() and out.shape == (q.shape[0], nh * vd)
    stride, off, gate_ptr, gate_ld = _gqa_tail(pool, layer, nkv, dim, vd, page_size, scale, window, keep_first, None,
                                               gate, gate_off, out_scale)
    n = q.shape[0] if items is None else (n_items if n_items is not None else items.numel())
    assert scratch.dtype == torch.float32 and scratch.numel() >= talk_attention_single_scratch(n, nh, n_cap)
    if talk is not None:
        assert talk.dtype == torch.float32 and talk.shape == (nh, nh) and talk.is_contiguous()
    if sinks is not None:
        assert sinks.dtype == torch.float32 and sinks.numel() == nh and sinks.is_contiguous()
    _check(lib().st_talk_attention_single(_p(q), _p(pool), stride, off, _p(out), _p(items), _p(positions),
                                          _p(seq_of_token), _p(slots), _p(block_table), block_table.shape[1], n, nh, nkv,
                                          dim, vd, page_size, _f(scale), window, keep_first, _p(talk), _p(sinks),
                                          gate_ptr, gate_ld, int(gate_heads), _f(out_scale), _p(scratch), int(n_cap),
                                          _p(status), _stream()), "talk_attention_single")
    return out


def hc_write_read_norm(lanes: torch.Tensor, mix: torch.Tensor, out_coef: torch.Tensor, y: torch.Tensor,
                       coef: torch.Tensor, gain: torch.Tensor, eps: float,
                       positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``hc_write(lanes, mix, out_coef, y)`` followed by ``hc_read_norm(lanes, coef, gain, eps)`` in one pass over the
    streams: the update of the sub-layer that just ran and the read of the next one.  Rows of padding tokens
    (negative position) are neither updated nor read."""
    n, tokens, width = lanes.shape
    assert lanes.dtype == torch.float32 and lanes.is_contiguous() and y.is_contiguous() and y.shape == (tokens, width)
    assert mix.dtype == torch.float32 and mix.shape == (n, n) and mix.is_contiguous()
    assert out_coef.dtype == torch.float32 and out_coef.numel() == n
    assert coef.dtype == torch.float32 and coef.numel() == n and gain.dtype == torch.float32 and gain.numel() == width
    out = torch.empty((tokens, width), dtype=torch.float32, device=lanes.device)
    _check(lib().st_hc_write_read_norm(_p(lanes), n, _p(mix), _p(out_coef), _p(y), _dt(y), _p(coef), _p(gain), _f(eps),
                                       tokens, width, _p(out), _p(positions), _stream()), "hc_write_read_norm")
    return out


def hc_step_conv(lanes: torch.Tensor, pending: Optional[tuple], coef: torch.Tensor, gain: torch.Tensor, eps: float,
                 conv_w: torch.Tensor, conv_state: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
                 seq_of_token: torch.Tensor, slots: torch.Tensor, write_state: bool = True) -> torch.Tensor:
    """For steps in which every request brings one token: the pending update of the streams (``pending`` = (mix,
    out_coef, y) or None), the next sub-layer's read and norm, and its input convolution h + conv(h) over the request's
    last taps - 1 inputs (``conv_state`` float32 [slots, taps - 1, width], moved on by h), in one kernel.  ``out``
    [tokens, width] in the activation type receives the sub-layer's input."""
    n, tokens, width = lanes.shape
    taps = conv_w.shape[1]
    assert lanes.dtype == torch.float32 and lanes.is_contiguous() and out.is_contiguous() and out.shape == (tokens, width)
    assert conv_w.dtype == torch.float32 and conv_w.shape == (width, taps) and conv_w.is_contiguous()
    assert conv_state.dtype == torch.float32 and conv_state.is_contiguous() and conv_state.shape[1:] == (taps - 1, width)
    assert coef.dtype == torch.float32 and coef.numel() == n and gain.dtype == torch.float32 and gain.numel() == width
    mix = out_coef = y = None
    if pending is not None:
        mix, out_coef, y = pending
        assert y.is_contiguous() and y.shape == (tokens, width) and mix.shape == (n, n) and out_coef.numel() == n
    tmp = torch.empty((tokens, width), dtype=torch.float32, device=lanes.device)
    _check(lib().st_hc_step_conv(_p(lanes), n, _p(mix), _p(out_coef), _p(y), _dt(y) if y is not None else 0, _p(coef),
                                 _p(gain), _f(eps), tokens, width, _p(conv_w), taps, _p(conv_state), int(write_state),
                                 _p(tmp), _p(out), _dt(out), _p(positions), _p(seq_of_token), _p(slots), _stream()),
           "hc_step_conv")
    return out
