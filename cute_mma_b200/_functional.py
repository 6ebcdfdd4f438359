"""``forward`` / ``backward``: the functional Prism API, bound to the sm_100a C-ABI library.

Mirrors ``cute_prism.forward`` / ``cute_prism.backward`` of the reference
(src/cute_prism/__init__.py:77-269 and :272-505): same positional arguments, same return
tuples, same ``ValueError`` for invalid parameters (src/cute_prism/_validate.py:12-84).
There is exactly one backend, so ``backend`` / ``mode`` / ``comp_params`` / ``autotuning``
style keywords are accepted for call compatibility and otherwise ignored.
"""
from __future__ import annotations

import ctypes
import threading

import torch

from . import _lib
from ._tile_table import lookup as _tile_lookup

KIND_FWD, KIND_BWD_DADR, KIND_BWD_DB, KIND_DBIAS, KIND_BWD_DADR_IB = 0, 1, 2, 3, 4
DTYPE_F32, DTYPE_SAME = 2, -1
ACTIVATIONS = (None, "silu_gate", "sigmoid_gate")
_GATE_CODES = {None: 0, "silu_gate": 1, "sigmoid_gate": 2}   # the C ABI's gate argument
_DTYPES = {torch.float16: 0, torch.bfloat16: 1}


def validate_kernel_params(group_size: int, reconn_sz: int) -> None:
    """Same rules and messages as the reference's ``validate_kernel_params``."""
    if not isinstance(group_size, int) or group_size <= 0:
        raise ValueError(f"group_size must be a positive integer, got {group_size}")
    if not isinstance(reconn_sz, int) or reconn_sz <= 0:
        raise ValueError(f"reconn_sz must be a positive integer, got {reconn_sz}")
    if reconn_sz % 8 != 0:
        raise ValueError(f"reconn_sz must be a multiple of 8, got {reconn_sz}")
    if group_size % 8 != 0:
        raise ValueError(f"group_size must be a multiple of 8, got {group_size}")
    if group_size % 16 != 0:
        # narrower than the reference (multiples of 8): the tcgen05 tiles are 16 wide
        raise ValueError(f"group_size must be a multiple of 16 for the sm_100a kernels, got {group_size}")


def validate_tensor_params(A, B, R, group_size, reconn_sz) -> None:
    """Same rules as the reference's ``validate_tensor_params``."""
    for name, t in (("A", A), ("B", B), ("R", R)):
        if not t.is_cuda:
            raise ValueError(f"{name} must be a CUDA tensor, got device={t.device}")
        if t.dtype not in _DTYPES:
            raise ValueError(f"{name} must be float16 or bfloat16, got dtype={t.dtype}")
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous (row-major)")
        if t.dim() != 2:
            raise ValueError(f"{name} must be 2D, got {t.dim()}D")
    if not (A.dtype == B.dtype == R.dtype):
        raise ValueError(f"All tensors must have the same dtype, got A={A.dtype}, B={B.dtype}, R={R.dtype}")
    if not (A.device == B.device == R.device):
        raise ValueError("All tensors must be on the same CUDA device")
    M, K = A.shape
    N = B.shape[0]
    if B.shape[1] != K:
        raise ValueError(f"K dimension mismatch: A has K={K} but B has K={B.shape[1]}")
    if R.shape[1] != K:
        raise ValueError(f"K dimension mismatch: A has K={K} but R has K={R.shape[1]}")
    if N % group_size != 0:
        raise ValueError(f"N ({N}) must be divisible by group_size ({group_size})")
    if K % reconn_sz != 0:
        raise ValueError(f"K ({K}) must be divisible by reconn_sz ({reconn_sz})")
    rows = (N // group_size) * reconn_sz
    if R.shape[0] != rows:
        raise ValueError(f"R must have shape ({rows}, {K}), but got ({R.shape[0]}, {R.shape[1]})")


# --------------------------------------------------------------------------- workspace
class _WorkspacePool:
    """Scratch buffers for the C ABI, one per (device, CUDA stream); the first 256 bytes are the
    status header.

    Calls issued on one stream run in order on the GPU, and every kernel rewrites what it later
    reads from the workspace, so one buffer per stream is enough whatever host thread issues the
    call (autograd runs the backward on its own threads but on the forward's stream).  Calls on
    different streams may overlap on the GPU and therefore never share a buffer.  A buffer that has
    to grow is replaced; the old one stays referenced until its status word has been read
    (``check_device_status``), so a device-side error recorded in it is not lost, and the caching
    allocator hands its memory out again in stream order only.
    """

    _MAX_RETIRED = 4

    def __init__(self):
        self._lock = threading.Lock()
        self._bufs = {}      # (device, stream handle) -> uint8 tensor
        self._retired = []   # [(device, tensor)] replaced by a larger buffer, status not read yet

    def get(self, device: torch.device, nbytes: int) -> torch.Tensor:
        stream = torch.cuda.current_stream(device)
        key = (device, stream.cuda_stream)
        with self._lock:
            buf = self._bufs.get(key)
            if buf is None or buf.numel() < nbytes:
                if buf is not None:
                    self._retired.append((device, buf))
                buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
                self._bufs[key] = buf
                overflow = self._retired[:-self._MAX_RETIRED] if len(self._retired) > self._MAX_RETIRED else []
                if overflow:
                    del self._retired[:len(overflow)]
            else:
                overflow = []
        for dev, old in overflow:   # bound the memory held by retired buffers: read their status now
            _read_status(dev, old)
        return buf

    def buffers(self, device: torch.device):
        """Every live or retired buffer of ``device`` (whatever thread or stream created it)."""
        with self._lock:
            live = [b for (d, _), b in self._bufs.items() if d == device]
            retired = [b for d, b in self._retired if d == device]
            self._retired = [(d, b) for d, b in self._retired if d != device]
        return live + retired


_workspace = _WorkspacePool()


def _read_status(device, buf) -> None:
    with torch.cuda.device(device):
        torch.cuda.synchronize(device)
        _lib.check(_lib.lib().prism_status(ctypes.c_void_p(buf.data_ptr()), _stream_ptr(device)))


def _cfg_array(cfg):
    if not cfg:
        return None
    arr = (ctypes.c_int * 8)(*([int(x) for x in cfg] + [0] * (8 - len(cfg))))
    return arr


def _stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def check_device_status(device=None) -> None:
    """Synchronise the device and raise if any kernel recorded a device-side error (a bounded wait
    that ran out) in any workspace of the device, including those used by autograd threads."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    first = None
    for buf in _workspace.buffers(device):
        try:
            _read_status(device, buf)
        except _lib.PrismError as e:   # keep polling: every header is read and cleared
            first = first or e
    if first is not None:
        raise first


def _gate_code(activation):
    if activation not in ACTIVATIONS:
        raise ValueError(f"Unknown activation {activation!r}, must be one of {ACTIVATIONS}")
    return _GATE_CODES[activation]


def _check_internal_bias(internal_bias, A, N, K, group_size, gate):
    """Same contract as the reference (src/cute_prism/__init__.py:166-170): a (N/group_size, K) tensor of
    A's dtype and device, gated modes only."""
    if internal_bias is None:
        return None
    if not gate:
        raise ValueError("internal_bias requires a gated activation; pass activation='silu_gate'")
    if (internal_bias.shape != (N // group_size, K) or internal_bias.dtype != A.dtype
            or internal_bias.device != A.device):
        raise ValueError(f"internal_bias must be a ({N // group_size}, {K}) tensor of the same dtype and device as A")
    return internal_bias.contiguous()


def _check_dropout(dropout_p, reconn_sz):
    if not 0.0 <= dropout_p < 1.0:
        raise ValueError(f"dropout_p must be in [0, 1), got {dropout_p}")
    if reconn_sz not in (8, 16):
        raise ValueError("dropout is supported for reconn_sz 8 and 16")


def _check_seeds(seeds, A, n_groups):
    """Per-group dropout seeds as the kernels take them: an int64 tensor (n_groups,) on A's device.  Accepts
    what the reference's forward returns as well (a one-element list holding that tensor)."""
    if isinstance(seeds, (list, tuple)):
        if len(seeds) == 0:
            return None
        seeds = seeds[0] if isinstance(seeds[0], torch.Tensor) else torch.tensor(list(seeds), dtype=torch.int64)
    if seeds.numel() == 0:
        return None
    if seeds.dtype != torch.int64 or seeds.shape != (n_groups,):
        raise ValueError(f"dropout_seeds must be an int64 tensor of shape ({n_groups},)")
    return seeds.to(A.device).contiguous()


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _reject_unsupported(**kw):
    for name, val in kw.items():
        if isinstance(val, torch.Tensor) or (val is not None and val is not False and val != 0.0):
            raise ValueError(f"{name} is not supported by the sm_100a kernels")


_fold_cache: dict = {}


def _shuffle_fold(shuffle_masks, K, group_size, reconn_sz, device):
    """Index maps of a set of shuffle masks (see ``_shuffle``), kept for repeated calls with the same tensor."""
    from ._shuffle import ShuffleFold
    if not isinstance(shuffle_masks, torch.Tensor) or shuffle_masks.dim() != 3 or shuffle_masks.dtype != torch.int64:
        raise ValueError("shuffle_masks must be an int64 tensor of shape (n_groups, K / 64, rounds)")
    key = (shuffle_masks.data_ptr(), shuffle_masks._version, tuple(shuffle_masks.shape), K, group_size, str(device))
    fold = _fold_cache.get(key)
    if fold is None:
        if len(_fold_cache) >= 16:
            _fold_cache.clear()
        fold = _fold_cache[key] = ShuffleFold(shuffle_masks, K, group_size, reconn_sz, device)
    return fold


def forward(A, B, R, group_size: int = 256, reconn_sz: int = 8, backend=None, mode: str = "ar",
            comp_params=None, activation=None, autotuning: bool = False, autotuning_search_space=None,
            force_rebenchmark: bool = False, internal_bias=None, dropout_p: float = 0.0,
            training: bool = False, shuffle_masks=None, *, bias=None, tile_cfg=None, dropout_seeds=None):
    """C = per-group (A . blockdiag(R_g)^T) @ B_g^T, or a gated form (``activation="silu_gate"``:
    ``(A * silu(A . blockdiag(R_g)^T)) @ B_g^T``; ``"sigmoid_gate"``: ``(A * 2 sigmoid(...)) @ B_g^T``);
    returns ``(C, [])``.

    ``bias`` (keyword-only, [N], same dtype) is added in the kernel epilogue.  With ``training=True`` and
    ``dropout_p > 0`` (gated modes) the gated activation goes through hash dropout and the second return
    value is ``[seeds]`` (int64, one per group) for ``backward(dropout_seeds=..., dropout_p=...)``.
    ``shuffle_masks`` (reconn_sz 16, chunks of 64 features): every group sees its own butterfly permutation
    of the input features (reference: src/cute_prism/__init__.py:114-117); served by the 64-wide rotation of
    the same kernels on folded parameters (``_shuffle``), not combined with dropout (the hash mask is
    indexed by physical feature there, by permuted feature in the reference).
    """
    if mode not in ("ar", "rw"):
        raise ValueError(f"Unknown mode {mode!r}, must be 'ar' or 'rw'")
    gate = _gate_code(activation)
    validate_kernel_params(group_size, reconn_sz)
    if mode == "rw":
        # inference with the rotation folded into the weight: C = A @ (B . blockdiag(R))^T
        if gate:
            raise ValueError("mode='rw' has no gated form (the gate needs A . blockdiag(R)^T itself)")
        _reject_unsupported(internal_bias=internal_bias, shuffle_masks=shuffle_masks)
        validate_tensor_params(A, B, R, group_size, reconn_sz)
        C = torch.matmul(A, fold_weight(B, R, group_size, reconn_sz).t())
        return (C if bias is None else C + bias), []
    validate_tensor_params(A, B, R, group_size, reconn_sz)
    M, K = A.shape
    N = B.shape[0]
    if shuffle_masks is not None:
        if training and dropout_p > 0.0:
            raise ValueError("input shuffle together with dropout is not supported by the sm_100a kernels")
        internal_bias = _check_internal_bias(internal_bias, A, N, K, group_size, gate)
        fold = _shuffle_fold(shuffle_masks, K, group_size, reconn_sz, A.device)
        return forward(A, fold.fold_cols(B, group_size), fold.fold_R(R), group_size, 64, activation=activation,
                       internal_bias=None if internal_bias is None else fold.fold_cols(internal_bias, 1),
                       bias=bias, tile_cfg=tile_cfg)
    internal_bias = _check_internal_bias(internal_bias, A, N, K, group_size, gate)
    # hash dropout of the gated activation, training only (reference: src/cute_prism/__init__.py:242-261): one
    # int64 seed per group, drawn here (or given as `dropout_seeds`) and returned for the backward
    seeds = None
    if gate and training and dropout_p > 0.0:
        _check_dropout(dropout_p, reconn_sz)
        seeds = dropout_seeds if dropout_seeds is not None else torch.randint(
            1, 1 << 62, (N // group_size,), dtype=torch.int64, device=A.device)
        seeds = _check_seeds(seeds, A, N // group_size)
    if bias is not None:
        if bias.dtype != A.dtype or bias.shape != (N,) or not bias.is_contiguous() or bias.device != A.device:
            raise ValueError("bias must be a contiguous (N,) tensor of the same dtype and device as A")
    C = torch.empty(M, N, dtype=A.dtype, device=A.device)
    if M == 0:
        return C, ([seeds] if seeds is not None else [])
    L = _lib.lib()
    cfg = tile_cfg if tile_cfg is not None else _tile_lookup("fwd", A.dtype, gate, M, N, K, group_size, reconn_sz)
    cfg_arr = _cfg_array(cfg)
    dt = _DTYPES[A.dtype]
    with torch.cuda.device(A.device):
        need = L.prism_workspace_bytes(KIND_FWD, M, N, K, group_size, reconn_sz, dt, cfg_arr)
        ws = _workspace.get(A.device, need)
        _lib.check(L.prism_fwd_dropout(
            ctypes.c_void_p(A.data_ptr()), ctypes.c_void_p(B.data_ptr()), ctypes.c_void_p(R.data_ptr()),
            _ptr(bias), _ptr(internal_bias), ctypes.c_void_p(C.data_ptr()),
            M, N, K, group_size, reconn_sz, dt, gate, A.stride(0), B.stride(0), R.stride(0), C.stride(0),
            _ptr(seeds), ctypes.c_float(dropout_p if seeds is not None else 0.0),
            cfg_arr, ctypes.c_void_p(ws.data_ptr()), ws.numel(), _stream_ptr(A.device)))
    return C, ([seeds] if seeds is not None else [])


def _grad_dtype(out_dtype, in_dtype, name):
    """(torch dtype, C-ABI code) of a parameter gradient: the inputs' 16-bit type or float32."""
    if out_dtype is None or out_dtype == in_dtype:
        return in_dtype, DTYPE_SAME
    if out_dtype == torch.float32:
        return torch.float32, DTYPE_F32
    raise ValueError(f"{name} must be None, the input dtype or torch.float32, got {out_dtype}")


def fold_weight(B, R, group_size: int, reconn_sz: int):
    """``Bp = B . blockdiag(R)`` per group through ``prism_fold_weight``: the weight of the "rw"
    mode, for which ``A @ Bp^T`` equals the plain-mode forward (reference:
    src/cute_prism/_pytorch_backend.py:115-124).  Fold once, then serve with an ordinary GEMM."""
    validate_kernel_params(group_size, reconn_sz)
    N, K = B.shape
    Bp = torch.empty_like(B)
    with torch.cuda.device(B.device):
        _lib.check(_lib.lib().prism_fold_weight(
            ctypes.c_void_p(B.data_ptr()), ctypes.c_void_p(R.data_ptr()), ctypes.c_void_p(Bp.data_ptr()),
            N, K, group_size, reconn_sz, _DTYPES[B.dtype], B.stride(0), R.stride(0), Bp.stride(0), _stream_ptr(B.device)))
    return Bp


_CAYLEY_DTYPES = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def cayley_supported(M, reconn_sz: int) -> bool:
    return M.is_cuda and M.dtype in _CAYLEY_DTYPES and reconn_sz in (8, 16) and M.dim() == 2


def cayley(M, reconn_sz: int):
    """R blocks of the plain mode from the stored parameter ``M`` ([G*rs, K]): per block
    ``S = M - M^T``, ``R = (I - S)^-1 (I + S)`` through ``prism_cayley`` (fp32 inside)."""
    M = M.contiguous()
    R = torch.empty_like(M)
    with torch.cuda.device(M.device):
        _lib.check(_lib.lib().prism_cayley(ctypes.c_void_p(M.data_ptr()), ctypes.c_void_p(R.data_ptr()),
                                           M.shape[0] // reconn_sz, M.shape[1], reconn_sz, _CAYLEY_DTYPES[M.dtype],
                                           M.stride(0), R.stride(0), _stream_ptr(M.device)))
    return R


def cayley_backward(M, dR, reconn_sz: int):
    """Gradient of ``cayley`` with respect to ``M`` through ``prism_cayley_bwd``."""
    M, dR = M.contiguous(), dR.contiguous().to(M.dtype)
    dM = torch.empty_like(M)
    with torch.cuda.device(M.device):
        _lib.check(_lib.lib().prism_cayley_bwd(ctypes.c_void_p(M.data_ptr()), ctypes.c_void_p(dR.data_ptr()),
                                               ctypes.c_void_p(dM.data_ptr()), M.shape[0] // reconn_sz, M.shape[1], reconn_sz,
                                               _CAYLEY_DTYPES[M.dtype], M.stride(0), dR.stride(0), dM.stride(0),
                                               _stream_ptr(M.device)))
    return dM


def _out_buffer(out, shape, dtype, device, name):
    """``out`` if given (a contiguous tensor of that shape and dtype, e.g. a view of a gradient staging
    buffer that other GPUs read), else a new tensor."""
    if out is None:
        return torch.empty(shape, dtype=dtype, device=device)
    if tuple(out.shape) != tuple(shape) or out.dtype != dtype or out.device != device or not out.is_contiguous():
        raise ValueError(f"{name} must be a contiguous {tuple(shape)} tensor of {dtype} on {device}")
    return out


def _backward_db(dC, A, R, group_size, reconn_sz, gate, dc_scale=1.0, tile_cfg=None, out_dtype=None,
                 internal_bias=None, dropout_seeds=None, dropout_p=0.0, dB_out=None):
    """dB = dc_scale * dC^T . H  through ``prism_bwd_db`` (H recomputed on chip); with
    ``out_dtype=torch.float32`` the kernel's fp32 sums are returned unrounded.  ``dB_out``: write there."""
    M, K = A.shape
    N = dC.shape[1]
    out_dtype, out_code = _grad_dtype(out_dtype, A.dtype, "dB_dtype")
    dB = _out_buffer(dB_out, (N, K), out_dtype, A.device, "dB_out")
    L = _lib.lib()
    cfg = tile_cfg if tile_cfg is not None else _tile_lookup("bwd_db", A.dtype, gate, M, N, K, group_size, reconn_sz)
    cfg_arr = _cfg_array(cfg)
    dt = _DTYPES[A.dtype]
    with torch.cuda.device(A.device):
        need = L.prism_workspace_bytes(KIND_BWD_DB, M, N, K, group_size, reconn_sz, dt, cfg_arr)
        ws = _workspace.get(A.device, need)
        _lib.check(L.prism_bwd_db(
            ctypes.c_void_p(dC.data_ptr()), ctypes.c_void_p(A.data_ptr()), ctypes.c_void_p(R.data_ptr()),
            _ptr(internal_bias), ctypes.c_void_p(dB.data_ptr()), M, N, K, group_size, reconn_sz, dt, gate, out_code,
            ctypes.c_float(dc_scale), dC.stride(0), A.stride(0), R.stride(0), dB.stride(0),
            _ptr(dropout_seeds), ctypes.c_float(dropout_p if dropout_seeds is not None else 0.0), cfg_arr, ctypes.c_void_p(ws.data_ptr()), ws.numel(), _stream_ptr(A.device)))
    return dB


def _backward_dadr(dC, A, B, R, group_size, reconn_sz, gate, dc_scale=1.0, tile_cfg=None, dR_dtype=None,
                   internal_bias=None, dropout_seeds=None, dropout_p=0.0, dR_out=None):
    """(dA, dR), both scaled by ``dc_scale``, through ``prism_bwd_dadr``; with
    ``dR_dtype=torch.float32`` the fp32 sums of the dR reduction are returned unrounded.  With an
    ``internal_bias`` the result is ``(dA, dR, d_internal_bias)``."""
    M, K = A.shape
    N = B.shape[0]
    dR_dtype, dr_code = _grad_dtype(dR_dtype, A.dtype, "dR_dtype")
    dA = torch.empty(M, K, dtype=A.dtype, device=A.device)
    dR = _out_buffer(dR_out, R.shape, dR_dtype, A.device, "dR_out")
    d_ib = torch.empty_like(internal_bias) if internal_bias is not None else None
    L = _lib.lib()
    cfg = tile_cfg if tile_cfg is not None else _tile_lookup("bwd_dadr", A.dtype, gate, M, N, K, group_size, reconn_sz)
    cfg_arr = _cfg_array(cfg)
    dt = _DTYPES[A.dtype]
    with torch.cuda.device(A.device):
        kind = KIND_BWD_DADR_IB if internal_bias is not None else KIND_BWD_DADR
        need = L.prism_workspace_bytes(kind, M, N, K, group_size, reconn_sz, dt, cfg_arr)
        ws = _workspace.get(A.device, need)
        _lib.check(L.prism_bwd_dadr(
            ctypes.c_void_p(dC.data_ptr()), ctypes.c_void_p(A.data_ptr()), ctypes.c_void_p(B.data_ptr()),
            ctypes.c_void_p(R.data_ptr()), _ptr(internal_bias), ctypes.c_void_p(dA.data_ptr()),
            ctypes.c_void_p(dR.data_ptr()), _ptr(d_ib),
            M, N, K, group_size, reconn_sz, dt, gate, dr_code, ctypes.c_float(dc_scale),
            dC.stride(0), A.stride(0), B.stride(0), R.stride(0), dA.stride(0), dR.stride(0),
            _ptr(dropout_seeds), ctypes.c_float(dropout_p if dropout_seeds is not None else 0.0), cfg_arr, ctypes.c_void_p(ws.data_ptr()), ws.numel(), _stream_ptr(A.device)))
    if internal_bias is not None:
        return dA, dR, d_ib
    return dA, dR


def backward(dC, A, B, R, group_size: int = 256, reconn_sz: int = 8, backend=None, activation=None,
             comp_params=None, autotuning: bool = False, autotuning_search_space_dadr=None,
             autotuning_search_space_db=None, bwd_dadr_params=None, bwd_db_params=None,
             force_rebenchmark: bool = False, dR_dtype=None, dB_dtype=None, internal_bias=None,
             dropout_seeds=None, dropout_p: float = 0.0, shuffle_masks=None, *, dc_scale: float = 1.0,
             tile_cfg_dadr=None, tile_cfg_db=None):
    """Gradients ``(dA, dR, dB, d_internal_bias)``; ``dB`` is None in plain mode and
    ``d_internal_bias`` is None when no ``internal_bias`` is given.
    ``dR_dtype`` / ``dB_dtype`` = ``torch.float32`` return the kernels' fp32 sums unrounded
    (reference: src/cute_prism/__init__.py:288-289, 368, 375).

    ``dc_scale`` (keyword-only) multiplies dC on the fly, i.e. scales every returned gradient.
    """
    gate = _gate_code(activation)
    validate_kernel_params(group_size, reconn_sz)
    validate_tensor_params(A, B, R, group_size, reconn_sz)
    M, K = A.shape
    N = B.shape[0]
    if shuffle_masks is not None:
        # the same kernels on the folded parameters (64-wide rotation); the parameter gradients come back through
        # the fold's index maps, dA needs none
        if dropout_seeds is not None and dropout_p > 0.0:
            raise ValueError("input shuffle together with dropout is not supported by the sm_100a kernels")
        internal_bias = _check_internal_bias(internal_bias, A, N, K, group_size, gate)
        fold = _shuffle_fold(shuffle_masks, K, group_size, reconn_sz, A.device)
        dA, dR64, dB2, d_ib2 = backward(
            dC, A, fold.fold_cols(B, group_size), fold.fold_R(R), group_size, 64, activation=activation,
            dR_dtype=dR_dtype, dB_dtype=dB_dtype,
            internal_bias=None if internal_bias is None else fold.fold_cols(internal_bias, 1),
            dc_scale=dc_scale, tile_cfg_dadr=tile_cfg_dadr, tile_cfg_db=tile_cfg_db)
        return (dA, fold.unfold_dR(dR64), None if dB2 is None else fold.unfold_cols(dB2, group_size),
                None if d_ib2 is None else fold.unfold_cols(d_ib2, 1))
    if dC.shape != (M, N) or dC.dtype != A.dtype or dC.device != A.device or not dC.is_contiguous():
        raise ValueError(f"dC must be a contiguous ({M}, {N}) tensor of the same dtype and device as A")
    internal_bias = _check_internal_bias(internal_bias, A, N, K, group_size, gate)
    seeds = None
    if gate and dropout_seeds is not None and dropout_p > 0.0:
        _check_dropout(dropout_p, reconn_sz)
        seeds = _check_seeds(dropout_seeds, A, N // group_size)
    out = _backward_dadr(dC, A, B, R, group_size, reconn_sz, gate, dc_scale, tile_cfg_dadr, dR_dtype, internal_bias,
                         seeds, dropout_p)
    dB = (_backward_db(dC, A, R, group_size, reconn_sz, gate, dc_scale, tile_cfg_db, dB_dtype, internal_bias,
                       seeds, dropout_p) if gate else None)
    return out[0], out[1], dB, (out[2] if internal_bias is not None else None)


def bias_grad(dC, out_dtype=None):
    """dbias [N] = sum of dC [M, N] over the token rows through ``prism_dbias`` (fixed summation
    order, bit-stable); ``out_dtype``: None (dC's dtype) or torch.float32."""
    if not dC.is_cuda or dC.dtype not in _DTYPES or dC.dim() != 2 or not dC.is_contiguous():
        raise ValueError("dC must be a contiguous 2-D float16 / bfloat16 CUDA tensor")
    M, N = dC.shape
    out_dtype, out_code = _grad_dtype(out_dtype, dC.dtype, "out_dtype")
    out = torch.empty(N, dtype=out_dtype, device=dC.device)
    L = _lib.lib()
    dt = _DTYPES[dC.dtype]
    with torch.cuda.device(dC.device):
        need = L.prism_workspace_bytes(KIND_DBIAS, M, N, 0, 0, 0, dt, None)
        ws = _workspace.get(dC.device, need)
        _lib.check(L.prism_dbias(ctypes.c_void_p(dC.data_ptr()), ctypes.c_void_p(out.data_ptr()), M, N, dt, out_code,
                                 dC.stride(0), ctypes.c_void_p(ws.data_ptr()), ws.numel(), _stream_ptr(dC.device)))
    return out
